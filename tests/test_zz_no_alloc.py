"""smore_unique_rows_static: de-duplication with the scratch inside the library (needs a B200).

This entry point serves hosts that cannot give the library a scratch buffer because they cannot
allocate at call time (all device memory already claimed by their own memory manager, or a
steady-state loop in which cudaMalloc's device-wide synchronisation is not acceptable).  The
check: called through the C ABI, twice in a row on different inputs (the built-in scratch still
holds the first call's bitmap when the second call starts), it must return exactly what
smore_unique_rows returns with a caller-provided workspace; and it must refuse tables beyond
its stated limit with an error code.

Kept in a file that sorts last so that a run stopping at the first failure has already run every
other test; it does not depend on any of them (it passes alone in a fresh process too).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(n):
    return (torch.full((n,), -3, dtype=torch.int64, device="cuda"),
            torch.full((n,), -3, dtype=torch.int32, device="cuda"),
            torch.full((n,), -3, dtype=torch.int32, device="cuda"),
            torch.full((2,), -3, dtype=torch.int32, device="cuda"))


def _with_workspace(L, _lib, idx, n_rows):
    n = idx.numel()
    uniq, inverse, counts, n_unique = _buffers(n)
    ws = torch.empty(L.smore_unique_rows_workspace_bytes(n_rows), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.smore_unique_rows(idx.data_ptr(), n, n_rows, uniq.data_ptr(), inverse.data_ptr(), counts.data_ptr(),
                                   n_unique.data_ptr(), ws.data_ptr(), ws.numel(), st), "smore_unique_rows")
    return uniq, inverse, counts, n_unique


def _static(L, _lib, idx, n_rows):
    n = idx.numel()
    uniq, inverse, counts, n_unique = _buffers(n)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.smore_unique_rows_static(idx.data_ptr(), n, n_rows, uniq.data_ptr(), inverse.data_ptr(),
                                          counts.data_ptr(), n_unique.data_ptr(), st), "smore_unique_rows_static")
    return uniq, inverse, counts, n_unique


def test_static_scratch_variant_matches_workspace_variant_twice_in_a_row():
    from smore_b200 import _lib
    L = _lib.lib()
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(11)
    # two different calls back to back: a large id space first, then a small one whose bitmap
    # lies inside the region the first call dirtied
    cases = [(300000, 10000019), (70000, 40001)]
    for n, n_rows in cases:
        idx = torch.randint(0, n_rows, (n,), device="cuda", generator=g)
        idx[:100] = idx[100:200]                      # guaranteed repeats
        want = _with_workspace(L, _lib, idx, n_rows)
        got = _static(L, _lib, idx, n_rows)
        torch.cuda.synchronize()
        nu = int(want[3][0])
        assert got[3].tolist() == want[3].tolist() and nu > 0
        assert torch.equal(got[0][:nu], want[0][:nu])          # sorted distinct ids
        assert torch.equal(got[1], want[1])                    # inverse map
        assert torch.equal(got[2][:nu], want[2][:nu])          # multiplicities
        # and both equal the torch call the reference makes
        t_u, t_i = torch.unique(idx, return_inverse=True)
        assert torch.equal(got[0][:nu], t_u) and torch.equal(got[1].long(), t_i)


def test_static_scratch_variant_leaves_device_memory_in_use_unchanged():
    """"Allocates nothing", measured: the driver's count of free device memory is the same before and
    after a series of calls (the first call on the device, which may load the library's code and
    looks up the scratch array's address, is made beforehand)."""
    from smore_b200 import _lib
    L = _lib.lib()
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(12)
    idx = torch.randint(0, 5000011, (200000,), device="cuda", generator=g)
    outs = _buffers(idx.numel())
    st = torch.cuda.current_stream().cuda_stream

    def call(n_rows):
        _lib.check(L.smore_unique_rows_static(idx.data_ptr(), idx.numel(), n_rows, outs[0].data_ptr(),
                                              outs[1].data_ptr(), outs[2].data_ptr(), outs[3].data_ptr(), st),
                   "smore_unique_rows_static")

    call(5000011)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for n_rows in (5000011, 1 << 24, 6000000):
        call(n_rows)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before


def test_static_scratch_variant_rejects_tables_beyond_its_limit():
    from smore_b200 import _lib
    L = _lib.lib()
    idx = torch.zeros(4, dtype=torch.int64, device="cuda")
    uniq, inverse, counts, n_unique = _buffers(4)
    limit = 1 << 24
    rc = L.smore_unique_rows_static(idx.data_ptr(), 4, limit + 1, uniq.data_ptr(), inverse.data_ptr(),
                                    counts.data_ptr(), n_unique.data_ptr(), None)
    assert rc == -6 and b"at most" in L.smore_last_error()
    # exactly at the limit is accepted
    rc = L.smore_unique_rows_static(idx.data_ptr(), 4, limit, uniq.data_ptr(), inverse.data_ptr(),
                                    counts.data_ptr(), n_unique.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert n_unique.tolist() == [1, 0] and uniq[0].item() == 0 and counts[0].item() == 4
