"""Row ids outside the table (needs a B200).

Ids are the caller's data.  An id that is negative or >= n_table_rows must never turn into an
address: the kernels read row 0 in its place, the forward result of that pair is NaN, the backward
pass neither takes a gradient from the pair nor writes one for it, a gathered row is NaN, and the
device status word gets bit 2.  Nothing faults; every other pair is computed as usual.  (The
reference indexes with torch, which raises a device-side assertion, embed_rw.py:74-77.)
"""
import numpy as np
import pytest
import torch

from tests.util import RTOL, RTOL_ATOMIC, close, forward_scale, make_operands

pytestmark = pytest.mark.gpu


def _st():
    return torch.cuda.current_stream().cuda_stream


@pytest.fixture()
def status_word():
    """The checks below set the status bit on purpose: start clean, verify, and leave it clean."""
    from smore_b200 import _lib
    _lib.async_status_clear()
    yield _lib
    _lib.async_status_clear()


# (op, be, ne, bc, nc, dim): register-staged rows, bulk-copied rows, bulk backward (wide rows),
# shared candidates (tile kernels), odd dim (cell kernels), positives (one row per query)
CASES = [("l1", 4, 64, 4, 1, 64), ("box_out", 3, 40, 3, 1, 400), ("box_in", 3, 40, 3, 1, 400),
         ("rotate", 2, 40, 2, 1, 500), ("box_out", 1, 24, 16, 1, 64), ("l2", 3, 10, 3, 1, 37),
         ("distmult", 9, 1, 9, 1, 64)]


@pytest.mark.parametrize("op,be,ne,bc,nc,dim", CASES)
def test_out_of_range_ids_are_skipped_not_dereferenced(status_word, oracle, op, be, ne, bc, nc, dim):
    _lib = status_word
    L = _lib.lib()
    N = 50
    mul = 2 if op in ("rotate", "complex") else 1
    tab, q0, q1 = make_operands(op, N, 1, bc, nc, dim, seed=be * 131 + dim)
    table = tab.reshape(N, dim * mul)
    rng = np.random.default_rng(dim + ne)
    idx = rng.integers(0, N, be * ne)
    bad_pos = sorted(set(int(x) for x in rng.integers(0, be * ne, 5)))
    idx_bad = idx.copy()
    for n, p in enumerate(bad_pos):
        idx_bad[p] = (-1, N, -(2 ** 40), N + 7, 2 ** 40)[n % 5]
    bad = np.zeros(be * ne, bool)
    bad[bad_pos] = True
    bsize, num = max(be, bc), max(ne, nc)
    # which output cells pair with a bad entity position
    cell_bad = np.zeros((bsize, num), bool)
    for i in range(bsize):
        for j in range(num):
            cell_bad[i, j] = bad[(i % be) * ne + (j % ne)]

    ent = table[idx].reshape(be, ne, dim * mul)          # valid stand-ins at the bad positions
    want = oracle.dist_forward(op, ent, q0, q1)
    gout = rng.standard_normal(want.shape).astype(np.float32)
    gout_eff = np.where(cell_bad, 0.0, gout).astype(np.float32)
    w_ent, w_q0, w_q1 = oracle.dist_backward(op, gout_eff, ent, q0, q1)

    t = torch.from_numpy(table).cuda()
    i64 = torch.from_numpy(idx_bad.astype(np.int64)).cuda()
    d_q0 = torch.from_numpy(q0).cuda()
    d_q1 = None if q1 is None else torch.from_numpy(q1).cuda()
    dst = torch.empty(bsize, num, device="cuda")
    sizes = (bsize, num, be, ne, bc, nc, dim)
    _lib.check(L.smore_dist_forward_rows(_lib.DIST_IDS[op], t.data_ptr(), i64.data_ptr(), N, d_q0.data_ptr(),
                                         None if q1 is None else d_q1.data_ptr(), dst.data_ptr(), *sizes, _st()), "fwd")
    got = dst.cpu().numpy()
    assert np.isnan(got[cell_bad]).all() and not np.isnan(got[~cell_bad]).any()
    scale = forward_scale(oracle, op, ent, q0, q1)
    close(got[~cell_bad], want[~cell_bad], RTOL, scale, what=op + " forward")
    assert _lib.async_status() & _lib.STATUS_BAD_ROW_ID

    # backward: the step's de-duplication gives bad positions the slot -1
    n = be * ne
    uniq = torch.empty(n, dtype=torch.int64, device="cuda")
    inverse = torch.empty(n, dtype=torch.int32, device="cuda")
    counts = torch.empty(n, dtype=torch.int32, device="cuda")
    n_unique = torch.empty(2, dtype=torch.int32, device="cuda")
    ws = torch.empty(L.smore_unique_rows_workspace_bytes(N), dtype=torch.uint8, device="cuda")
    _lib.check(L.smore_unique_rows(i64.data_ptr(), n, N, uniq.data_ptr(), inverse.data_ptr(), counts.data_ptr(),
                                   n_unique.data_ptr(), ws.data_ptr(), ws.numel(), _st()), "unique")
    assert n_unique.tolist()[1] == len(bad_pos)
    assert (inverse.cpu().numpy()[bad] == -1).all()
    nu = int(n_unique[0])
    g_rows = torch.zeros(n, dim * mul, device="cuda")
    g_q0 = torch.full_like(d_q0, float("nan"))
    g_q1 = None if q1 is None else torch.full_like(d_q1, float("nan"))
    _lib.check(L.smore_dist_backward_rows(_lib.DIST_IDS[op], torch.from_numpy(gout).cuda().data_ptr(), t.data_ptr(),
                                          i64.data_ptr(), N, d_q0.data_ptr(), None if q1 is None else d_q1.data_ptr(),
                                          inverse.data_ptr(), None, g_rows.data_ptr(), g_q0.data_ptr(),
                                          None if q1 is None else g_q1.data_ptr(), *sizes, _st()), "bwd")
    w_uniq, w_inv, _ = oracle.unique_rows(idx[~bad])
    assert np.array_equal(uniq[:nu].cpu().numpy(), w_uniq)
    w_rows = oracle.scatter_sum_rows(w_ent.reshape(n, -1)[~bad], w_inv, len(w_uniq))
    close(g_rows[:nu].cpu().numpy(), w_rows, RTOL_ATOMIC, what=op + " g_rows")
    assert not g_rows[nu:].any()
    close(g_q0.cpu().numpy(), w_q0, RTOL_ATOMIC, what=op + " g_first")
    if q1 is not None:
        close(g_q1.cpu().numpy(), w_q1, RTOL_ATOMIC, what=op + " g_second")


def test_union_and_box_both_with_bad_ids(status_word, oracle):
    _lib = status_word
    L = _lib.lib()
    B, U, K, dim, N = 3, 2, 33, 64, 40
    tab, q0, q1 = make_operands("box_out", N, 1, B * U, 1, dim, seed=4)
    table = tab.reshape(N, dim)
    rng = np.random.default_rng(2)
    idx = rng.integers(0, N, (B, K))
    idx_bad = idx.copy()
    idx_bad[0, 3], idx_bad[2, 32], idx_bad[1, 0] = -5, N, 10 ** 12
    cell_bad = idx_bad != idx
    t, i64 = torch.from_numpy(table).cuda(), torch.from_numpy(idx_bad).cuda()
    d_q0, d_q1 = torch.from_numpy(q0.reshape(B, U, dim)).cuda(), torch.from_numpy(q1.reshape(B, U, dim)).cuda()
    d_out = torch.empty(B, U, K, device="cuda")
    d_in = torch.empty(B, U, K, device="cuda")
    _lib.check(L.smore_union_forward_rows(_lib.BOX_BOTH_ID, t.data_ptr(), i64.data_ptr(), N, d_q0.data_ptr(),
                                          d_q1.data_ptr(), d_out.data_ptr(), d_in.data_ptr(), U, B, K, dim, _st()), "fwd")
    ent = table[idx].reshape(B, K, dim)
    for u in range(U):
        f = np.ascontiguousarray(q0.reshape(B, U, 1, dim)[:, u])
        s = np.ascontiguousarray(q1.reshape(B, U, 1, dim)[:, u])
        for got, name in ((d_out, "box_out"), (d_in, "box_in")):
            g = got[:, u].cpu().numpy()
            want = oracle.dist_forward(name, ent, f, s)
            assert np.isnan(g[cell_bad]).all()
            close(g[~cell_bad], want[~cell_bad], RTOL, forward_scale(oracle, name, ent, f, s), what=name)
    assert _lib.async_status() & _lib.STATUS_BAD_ROW_ID


def test_gather_rows_with_bad_ids(status_word):
    _lib = status_word
    L = _lib.lib()
    N, W = 20, 12
    table = torch.arange(N * W, dtype=torch.float32, device="cuda").view(N, W)
    idx = torch.tensor([3, -1, 19, 20, 0], dtype=torch.int64, device="cuda")
    out = torch.zeros(5, W, device="cuda")
    _lib.check(L.smore_gather_rows(table.data_ptr(), idx.data_ptr(), N, out.data_ptr(), 5, W, _st()), "gather")
    assert torch.equal(out[[0, 2, 4]], table[[3, 19, 0]])
    assert torch.isnan(out[[1, 3]]).all()
    assert _lib.async_status() == _lib.STATUS_BAD_ROW_ID
    _lib.async_status_clear()
    assert _lib.async_status() == 0


def test_optimizer_check_status_raises_once_after_a_bad_lookup(status_word):
    """EmbeddingOptimizer.check_status turns the device status word into an exception and clears it."""
    from smore_b200 import embedding, ext_ops

    class _Args(object):
        optim_mode = ("aggr", "adam", "gpu", True, 0)
        share_optim_stats = False

    dev = torch.device("cuda", 0)
    emb = embedding.SparseEmbedding(0, 64)
    emb.num_rows = 100
    emb.embedding = torch.nn.Parameter(torch.rand(100, 64, device=dev), requires_grad=False)
    opt = embedding.AdamEmbedOptimizer(_Args(), emb, 0, lazy_names=("negative_entity",))
    emb.train()
    opt.zero_grad()
    opt.check_status()                                   # clean: no exception
    ids = torch.tensor([[3, 100, 7, 9]], device=dev)     # 100 is one past the table
    rows = emb(ids.view(-1), "negative_entity")
    query = torch.rand(1, 1, 64, device=dev, requires_grad=True)
    dist = ext_ops.l1_dist(rows.view(1, 4, -1), query)
    assert torch.isnan(dist[0, 1]) and not torch.isnan(dist[0, [0, 2, 3]]).any()
    with pytest.raises(RuntimeError, match="row id outside the table"):
        opt.check_status()
    opt.check_status()                                   # cleared by the first call
