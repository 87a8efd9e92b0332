"""ctypes binding of libsmore_b200.so (the C ABI declared in include/smore_b200.h).

There is no fallback: if the library has not been built, or a call fails, an exception is
raised.  Build with `python smore_b200/csrc/build.py`.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libsmore_b200.so")

DIST_IDS = {"box_out": 0, "box_in": 1, "rotate": 2, "l1": 3, "l2": 4, "complex": 5, "distmult": 6}
BOX_BOTH_ID = 7     # smore_union_* entry points only
GEOMETRY_IDS = {"add": 0, "rotate": 1, "complex": 2, "distmult": 3}   # smore_path_embed_*
OPT_IDS = {"sgd": 0, "adam": 1, "adagrad": 2}
ROW_PARTS = {"box_out": 1, "box_in": 1, "rotate": 2, "l1": 1, "l2": 1, "complex": 2, "distmult": 1}
QUERY_PARTS = {"box_out": 2, "box_in": 2, "rotate": 2, "l1": 1, "l2": 1, "complex": 2, "distmult": 1}

_p = ctypes.c_void_p
_sz = ctypes.c_size_t
_int = ctypes.c_int
_dbl = ctypes.c_double

# name -> (restype, argtypes); must list every function include/smore_b200.h declares
SIGNATURES = {
    "smore_last_error": (ctypes.c_char_p, []),
    "smore_version": (ctypes.c_char_p, []),
    "smore_kernel_launch_count": (ctypes.c_ulonglong, []),
    "smore_alu_probe": (_int, [_p, _sz, ctypes.POINTER(ctypes.c_double), _p]),
    "smore_dist_forward": (_int, [_int, _p, _p, _p, _p] + [_sz] * 7 + [_p]),
    "smore_dist_backward": (_int, [_int] + [_p] * 7 + [_sz] * 7 + [_p]),
    "smore_dist_forward_f64": (_int, [_int, _p, _p, _p, _p] + [_sz] * 7 + [_p]),
    "smore_dist_backward_f64": (_int, [_int] + [_p] * 7 + [_sz] * 7 + [_p]),
    "smore_dist_forward_rows": (_int, [_int, _p, _p, _sz, _p, _p, _p] + [_sz] * 7 + [_p]),
    "smore_dist_backward_rows": (_int, [_int, _p, _p, _p, _sz] + [_p] * 7 + [_sz] * 7 + [_p]),
    "smore_box_forward": (_int, [_p, _p, _sz] + [_p] * 4 + [_sz] * 7 + [_p]),
    "smore_box_backward": (_int, [_p] * 4 + [_sz] + [_p] * 8 + [_sz] * 7 + [_p]),
    "smore_async_status": (_int, [ctypes.POINTER(ctypes.c_int)]),
    "smore_async_status_clear": (_int, []),
    "smore_union_forward_rows": (_int, [_int, _p, _p, _sz] + [_p] * 4 + [_sz] * 4 + [_p]),
    "smore_union_backward_rows": (_int, [_int] + [_p] * 4 + [_sz] + [_p] * 7 + [_sz] * 4 + [_p]),
    "smore_gather_rows": (_int, [_p, _p, _sz, _p, _sz, _sz, _p]),
    "smore_unique_rows_workspace_bytes": (_sz, [_sz]),
    "smore_unique_rows": (_int, [_p, _sz, _sz, _p, _p, _p, _p, _p, _sz, _p]),
    "smore_unique_rows_static": (_int, [_p, _sz, _sz, _p, _p, _p, _p, _p]),
    "smore_zero_shared_rows": (_int, [_p, _p, _p, _sz, _sz, _p]),
    "smore_scatter_add_rows": (_int, [_p, _p, _p, _p, _sz, _sz, _p]),
    "smore_sparse_update_rows": (_int, [_int, _p, _p, _p, _p, _p, _p, _sz, _sz, _dbl, _dbl, _dbl, _dbl,
                                        ctypes.c_int64, _int, _p]),
    "smore_rows_backward_fused_adam": (_int, [_int, _p, _p, _p, _p, _sz] + [_p] * 7 + [_sz] * 4 + [_p, _p, _p, _dbl, _dbl,
                                              _dbl, _dbl, ctypes.c_int64, _p, _p]),
    "smore_adam_step_scalars": (_int, [_p, _dbl, _dbl, _dbl, _p, _p]),
    "smore_sparse_update_rows_dev": (_int, [_int, _p, _p, _p, _p, _p, _p, _sz, _sz, _dbl, _dbl, _dbl, _dbl, _p, _int,
                                            _p]),
    "smore_path_project_forward": (_int, [_p, _p, _p, _p, _sz, _p, _sz, _sz, _sz, _sz, _int, _p, _p, _p]),
    "smore_path_project_backward": (_int, [_p, _p, _p, _sz, _p, _sz, _sz, _sz, _sz, _int, _p, _p, _p]),
    "smore_path_embed_forward": (_int, [_int, _p, _p, _sz, _p, _p, _p, _sz, _p, _sz, _sz, _sz, _sz, _int, _dbl, _p, _p, _p]),
    "smore_path_embed_backward": (_int, [_int, _p, _p, _p, _p, _sz, _p, _p, _sz, _p, _sz, _sz, _sz, _sz, _int, _dbl,
                                         _p, _p, _p, _p, _p, _p, _p]),
    "smore_filtered_ranks_workspace_bytes": (_sz, [_sz]),
    "smore_filtered_ranks": (_int, [_p, _sz, _sz, _p, _p, _sz, _sz, _p, _p, _sz, _p]),
    "smore_score_filtered_ranks_workspace_bytes": (_sz, [_sz, _sz]),
    "smore_score_filtered_ranks": (_int, [_int, _p, _sz, _p, _p, _sz, _sz, _dbl, _dbl, _p, _p, _sz, _sz, _p, _p, _sz, _p]),
    "smore_alias_build": (_int, [_p, _sz, _p, _p, _p]),
    "smore_sample_negatives": (_int, [ctypes.c_uint64, ctypes.c_uint64, _sz, _p, _p, _p, _p, _p, _sz, _sz, _p, _p]),
    "smore_negative_mask": (_int, [_p, _sz, _p, _p, _sz, _p, _p]),
    "smore_dot_available": (_int, []),
    "smore_dot_two_sm": (_int, []),
    "smore_dot_workspace_bytes": (_sz, [_sz, _sz, _sz, _int]),
    "smore_dot_forward_shared": (_int, [_p, _p, _p, _sz, _sz, _sz, _int, _p, _sz, _p]),
    "smore_dot_backward_shared": (_int, [_p, _p, _p, _p, _p, _sz, _sz, _sz, _int, _p, _sz, _p]),
    "smore_fetch_rows": (_int, [_p, _sz, _p, _p, _sz, _sz, _p, _p]),
    "smore_fetch_rows_background": (_int, [_p, _sz, _p, _p, _sz, _sz, _p, _sz, _p]),
    "smore_refresh_rows": (_int, [_p, _p, _sz, _sz, _p, _p, _sz, _sz, _p, _p, _p]),
    "smore_shard_mark_dirty": (_int, [_p, _p, _sz, _sz, _p, _p]),
    "smore_shard_owner_plan_workspace_bytes": (_sz, [_sz]),
    "smore_shard_owner_plan": (_int, [_p, _p, _sz, _sz, ctypes.POINTER(ctypes.c_int32), ctypes.c_int64, _sz, _sz] +
                               [_p] * 9 + [_sz, _p]),
    "smore_shard_reduce_update_rows": (_int, [_p] * 7 + [_sz, _p, _p, _p, _sz, _sz, _dbl, _dbl, _dbl, _dbl,
                                              ctypes.c_int64, _int, _p]),
    "smore_shard_reduce_update_rows_dev": (_int, [_p] * 7 + [_sz, _p, _p, _p, _sz, _sz, _dbl, _dbl, _dbl, _dbl, _p, _int,
                                                  _p]),
    "smore_owner_select_pairs": (_int, [_p, _p, _sz, _sz, _sz, _sz, _sz, _sz, ctypes.c_int64, _sz, _sz, _p, _p, _p, _p,
                                        _p]),
    "smore_owner_gather_queries": (_int, [_p, _p, _p, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _p, _p, _p]),
    "smore_rows_forward_ragged": (_int, [_int, _p, _p, _sz, _p, _p, _p, _sz, _sz, _p, _p, _p, _sz, _p, _p, _sz, _sz, _p]),
    "smore_rows_backward_fused_adam_ragged": (_int, [_int, _p, _p, _p, _p, _sz, _p, _p, _p, _sz] + [_p] * 5 +
                                              [_sz, _p, _p, _p, _dbl, _dbl, _dbl, _dbl, ctypes.c_int64, _p, _p, _sz,
                                               _p, _p, _sz, _sz, _p]),
    "smore_owner_plan": (_int, [_p, _p, _sz, _sz, ctypes.POINTER(ctypes.c_int32), ctypes.c_int64, _sz, _sz] +
                         [_p] * 8 + [_sz, _p, _sz, _p]),
    "smore_owner_add_list_rows": (_int, [_p, _p, _sz, _p, _p, _p, _sz, _sz, _p]),
    "smore_owner_sum_query_grads": (_int, [_p, _sz, _sz, _sz, _sz, _sz, _p, _p]),
}

_lib = None


class SmoreError(RuntimeError):
    pass


def lib():
    """The loaded library; raises if it is missing (no CPU or torch fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SmoreError("%s not found: build it with `python smore_b200/csrc/build.py`" % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc, what):
    if rc != 0:
        msg = lib().smore_last_error()
        raise SmoreError("%s failed (%d): %s" % (what, rc, msg.decode() if msg else ""))


def async_status():
    """Status word of the current device's bulk-copy kernels (synchronises); 0 means no wait gave up."""
    v = ctypes.c_int(0)
    check(lib().smore_async_status(ctypes.byref(v)), "smore_async_status")
    return v.value


def async_status_clear():
    check(lib().smore_async_status_clear(), "smore_async_status_clear")


STATUS_COPY_WAIT, STATUS_PEER_WAIT, STATUS_BAD_ROW_ID, STATUS_CAPACITY = 1, 2, 4, 8


# ---- optional per-kernel timing (benchmarks only) ----------------------------------------------

class KernelTimer(object):
    """Brackets library calls with CUDA events on the stream they are enqueued on.  Install with
    `set_timer(KernelTimer())`; read `elapsed_ms()` after synchronising."""

    def __init__(self):
        self.records = {}
        self.notes = {}

    def range(self, name):
        return _TimedRange(self, name)

    def elapsed_ms(self):
        return {k: [a.elapsed_time(b) for a, b in v] for k, v in self.records.items()}


class _TimedRange(object):
    def __init__(self, timer, name):
        self.timer, self.name = timer, name

    def __enter__(self):
        import torch
        self.start = torch.cuda.Event(enable_timing=True)
        self.end = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def __exit__(self, *exc):
        self.end.record()
        self.timer.records.setdefault(self.name, []).append((self.start, self.end))
        return False


class _NoRange(object):
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_RANGE = _NoRange()
_timer = None


def set_timer(timer):
    global _timer
    _timer = timer


def timed(name):
    return _NO_RANGE if _timer is None else _timer.range(name)


def note(name, device_scalar):
    """Keep a copy of a device-side scalar (e.g. the number of distinct rows of a step) for the
    installed timer; no host synchronisation happens here."""
    if _timer is not None:
        _timer.notes.setdefault(name, []).append(device_scalar.clone())
