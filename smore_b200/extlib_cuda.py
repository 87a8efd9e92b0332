"""Drop-in for the reference's `extlib_cuda` extension module.

Exposes the function and class names the reference registers with pybind
(smore/common/torchext/extlib_cuda.cpp:307-342) so that `import extlib_cuda as extlib` in
smore/common/torchext/dist_func/*.py and smore/common/embedding/embed_rw.py can resolve to
this module (put it in sys.modules under that name).  Every distance function forwards to the
C ABI of libsmore_b200.so with raw device pointers and the current CUDA stream of the
tensors' device.  Argument order and meaning are the reference's; what differs is the error
behaviour: a bad argument raises (the reference prints and exits the process, or does
nothing for an unknown distance name).
"""
import torch

from . import _lib

__all__ = [
    "box_dist_forward", "box_dist_backward", "rotate_dist_forward", "rotate_dist_backward",
    "l1_dist_forward", "l1_dist_backward", "l2_dist_forward", "l2_dist_backward",
    "complex_dist_forward", "complex_dist_backward", "distmult_dist_forward", "distmult_dist_backward",
    "beta_dist_forward", "beta_dist_backward", "ThreadPool", "CudaEvent", "AsyncGPUJob", "async_read",
    "async_write",
]


def _stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def _check_operands(name, entity, first, second, inputs, outputs):
    """Inputs may arrive with any strides (autograd hands the backward of a `torch.stack` over
    union branches, box_dist.py:60-68, a strided grad_out); the kernels write the output buffers
    in place, so those must be contiguous as given."""
    if not entity.is_cuda:
        raise _lib.SmoreError("%s: operands must be CUDA tensors (there is no CPU path)" % name)
    if entity.dtype not in (torch.float32, torch.float64):
        raise TypeError("%s: float32 or float64 expected, got %s" % (name, entity.dtype))
    for t in (entity, first, second) + tuple(inputs) + tuple(outputs):
        if t is None:
            continue
        if t.device != entity.device or t.dtype != entity.dtype:
            raise TypeError("%s: all operands must share device and dtype" % name)
    for t in outputs:
        if t is not None and not t.is_contiguous():
            raise ValueError("%s: output buffers must be contiguous" % name)
    if entity.dim() != 3 or first.dim() != 3:
        raise ValueError("%s: entity and query operands must be 3-D" % name)
    if second is not None and second.shape != first.shape:
        raise ValueError("%s: the two query operands must have the same shape" % name)
    if entity.shape[2] != _lib.ROW_PARTS[name] * first.shape[2]:
        raise ValueError("%s: entity rows must be %d x the query dim" % (name, _lib.ROW_PARTS[name]))


def _sizes(entity, first, out):
    be, ne = entity.shape[0], entity.shape[1]
    bc, nc, dim = first.shape
    if out.dim() != 2 or out.shape[0] != max(be, bc) or out.shape[1] != max(ne, nc):
        raise ValueError("output must be [max(be, bc), max(ne, nc)] = [%d, %d], got %s"
                         % (max(be, bc), max(ne, nc), tuple(out.shape)))
    return out.shape[0], out.shape[1], be, ne, bc, nc, dim


def _ptr(t):
    return None if t is None else t.data_ptr()


def dist_forward(name, entity, first, second, dst):
    """dst[i, j] = distance(entity[i % be, j % ne], query[i % bc, j % nc]); see
    extlib_cuda.cpp:172-196 for the reference binding this replaces."""
    if _lib.QUERY_PARTS[name] == 1:
        second = None
    _check_operands(name, entity, first, second, (), (dst,))
    sizes = _sizes(entity, first, dst)
    entity, first = entity.contiguous(), first.contiguous()
    second = None if second is None else second.contiguous()
    L = _lib.lib()
    fn = L.smore_dist_forward if entity.dtype == torch.float32 else L.smore_dist_forward_f64
    with torch.cuda.device(entity.device):
        rc = fn(_lib.DIST_IDS[name], _ptr(entity), _ptr(first), _ptr(second), _ptr(dst), *sizes,
                _stream_ptr(entity.device))
    _lib.check(rc, name + "_dist_forward")


def dist_backward(name, grad_out, entity, first, second, g_entity, g_first, g_second):
    """Fills g_entity, g_first (and g_second) completely; see extlib_cuda.cpp:233-262."""
    if _lib.QUERY_PARTS[name] == 1:
        second = g_second = None
    _check_operands(name, entity, first, second, (grad_out,), (g_entity, g_first, g_second))
    if g_entity.shape != entity.shape or g_first.shape != first.shape:
        raise ValueError("gradient buffers must have the shapes of their operands")
    sizes = _sizes(entity, first, grad_out)
    grad_out, entity, first = grad_out.contiguous(), entity.contiguous(), first.contiguous()
    second = None if second is None else second.contiguous()
    L = _lib.lib()
    fn = L.smore_dist_backward if entity.dtype == torch.float32 else L.smore_dist_backward_f64
    with torch.cuda.device(entity.device):
        rc = fn(_lib.DIST_IDS[name], _ptr(grad_out), _ptr(entity), _ptr(first), _ptr(second), _ptr(g_entity),
                _ptr(g_first), _ptr(g_second), *sizes, _stream_ptr(entity.device))
    _lib.check(rc, name + "_dist_backward")


def _box_name(dist_type):
    if dist_type not in ("in", "out"):
        raise ValueError("box dist_type must be 'in' or 'out', got %r" % (dist_type,))
    return "box_" + dist_type


# ---- the reference's pybind names (extlib_cuda.cpp:322-341) --------------------------------

def box_dist_forward(entity_embed, center_embed, offset_embed, dst, dist_type):
    dist_forward(_box_name(dist_type), entity_embed, center_embed, offset_embed, dst)


def box_dist_backward(grad_out, entity_embed, center_embed, offset_embed, grad_entity, grad_center, grad_offset,
                      dist_type):
    dist_backward(_box_name(dist_type), grad_out, entity_embed, center_embed, offset_embed, grad_entity,
                  grad_center, grad_offset)


def rotate_dist_forward(entity_embed, re_embed, im_embed, dst):
    dist_forward("rotate", entity_embed, re_embed, im_embed, dst)


def rotate_dist_backward(grad_out, entity_embed, re_embed, im_embed, grad_entity, grad_re, grad_im):
    dist_backward("rotate", grad_out, entity_embed, re_embed, im_embed, grad_entity, grad_re, grad_im)


def complex_dist_forward(entity_embed, re_embed, im_embed, dst):
    dist_forward("complex", entity_embed, re_embed, im_embed, dst)


def complex_dist_backward(grad_out, entity_embed, re_embed, im_embed, grad_entity, grad_re, grad_im):
    dist_backward("complex", grad_out, entity_embed, re_embed, im_embed, grad_entity, grad_re, grad_im)


def l1_dist_forward(entity_embed, center_embed, dst):
    dist_forward("l1", entity_embed, center_embed, None, dst)


def l1_dist_backward(grad_out, entity_embed, center_embed, grad_entity, grad_center):
    dist_backward("l1", grad_out, entity_embed, center_embed, None, grad_entity, grad_center, None)


def l2_dist_forward(entity_embed, center_embed, dst):
    dist_forward("l2", entity_embed, center_embed, None, dst)


def l2_dist_backward(grad_out, entity_embed, center_embed, grad_entity, grad_center):
    dist_backward("l2", grad_out, entity_embed, center_embed, None, grad_entity, grad_center, None)


def distmult_dist_forward(entity_embed, center_embed, dst):
    dist_forward("distmult", entity_embed, center_embed, None, dst)


def distmult_dist_backward(grad_out, entity_embed, center_embed, grad_entity, grad_center):
    dist_backward("distmult", grad_out, entity_embed, center_embed, None, grad_entity, grad_center, None)


def beta_dist_forward(*args, **kwargs):
    raise NotImplementedError("the beta-distribution distances (BetaE) are not part of this library")


def beta_dist_backward(*args, **kwargs):
    raise NotImplementedError("the beta-distribution distances (BetaE) are not part of this library")


# ---- host-side objects embed_rw.py constructs unconditionally (embed_rw.py:45) ----------------

class ThreadPool(object):
    """Placeholder for the worker pool of the CPU-resident table path (extlib_cuda.cpp:308-309).
    A table kept in GPU memory needs no staging threads; the object only has to exist."""

    def __init__(self, num_threads):
        self.num_threads = int(num_threads)


class CudaEvent(object):
    """extlib_cuda.cpp:160-169: an event recorded on the current stream of `device`."""

    def __init__(self, device):
        self.device = int(device)
        self.event = None

    def record(self):
        if self.event is None:
            self.event = torch.cuda.Event(enable_timing=False)
        self.event.record(torch.cuda.current_stream(self.device))


class AsyncGPUJob(object):
    """extlib_cuda.h:26-52: a handle whose sync() waits for a staged copy.  Nothing is staged
    for a GPU-resident table, so sync() returns immediately."""

    def __init__(self, device):
        self.device = int(device)

    def sync(self):
        return None


def async_read(*args, **kwargs):
    raise NotImplementedError(
        "async_read stages rows of a CPU-resident table through pinned memory (extlib_cuda.cpp:82-112); "
        "this library keeps the table (or its shard) in GPU memory instead")


def async_write(*args, **kwargs):
    raise NotImplementedError(
        "async_write copies row updates back to a CPU-resident table (extlib_cuda.cpp:115-144); "
        "this library keeps the table (or its shard) in GPU memory instead")
