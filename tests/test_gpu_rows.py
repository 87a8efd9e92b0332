"""Table-resident lookups, per-step de-duplication and the fused row-wise optimizers on the GPU,
checked against the CPU oracle and the reference-generated golden vectors (needs a B200)."""
import numpy as np
import pytest
import torch

from tests.util import RTOL, RTOL_ATOMIC, TWO_QUERY, close, forward_scale, make_operands

pytestmark = pytest.mark.gpu


def _st():
    return torch.cuda.current_stream().cuda_stream


def _unique(idx_np, n_table_rows):
    from smore_b200 import _lib
    L = _lib.lib()
    idx = torch.from_numpy(np.ascontiguousarray(idx_np, dtype=np.int64)).cuda()
    n = idx.numel()
    uniq = torch.full((max(n, 1),), -7, dtype=torch.int64, device="cuda")
    inverse = torch.full((max(n, 1),), -7, dtype=torch.int32, device="cuda")
    counts = torch.full((max(n, 1),), -7, dtype=torch.int32, device="cuda")
    n_unique = torch.full((2,), -7, dtype=torch.int32, device="cuda")
    ws = torch.empty(L.smore_unique_rows_workspace_bytes(n_table_rows), dtype=torch.uint8, device="cuda")
    ws.fill_(0xAB)  # the workspace may hold anything on entry
    _lib.check(L.smore_unique_rows(idx.data_ptr(), n, n_table_rows, uniq.data_ptr(), inverse.data_ptr(),
                                   counts.data_ptr(), n_unique.data_ptr(), ws.data_ptr(), ws.numel(), _st()),
               "unique")
    torch.cuda.synchronize()
    return uniq, inverse, counts, n_unique


@pytest.mark.parametrize("n,n_rows,dist", [
    (1, 1, "uniform"), (5, 40, "uniform"), (1000, 97, "uniform"), (50000, 14505, "uniform"),
    (200000, 2500604, "zipf"), (1050624, 10756769, "uniform"), (4096, 33, "uniform"), (70000, 32768 * 3 + 5, "zipf"),
    # few ids over a large id space: the one-CTA sort route (a step's anchor lookups on a sharded table)
    (1024, 86054151, "uniform"), (1024, 86054151, "zipf"), (4096, 10756769, "zipf"), (1, 1 << 20, "uniform"),
    (37, 300000, "zipf"), (4097, 10756769, "uniform"), (33, 1 << 18, "uniform"),
])
def test_unique_rows_bit_exact(n, n_rows, dist):
    rng = np.random.default_rng(n)
    if dist == "uniform":
        idx = rng.integers(0, n_rows, n)
    else:
        idx = np.minimum(rng.zipf(1.2, n) - 1, n_rows - 1)
    uniq, inverse, counts, n_unique = _unique(idx, n_rows)
    w_uniq, w_inv, w_cnt = np.unique(idx, return_inverse=True, return_counts=True)
    nu = int(n_unique[0])
    assert nu == len(w_uniq) and int(n_unique[1]) == 0
    assert np.array_equal(uniq[:nu].cpu().numpy(), w_uniq)
    assert np.array_equal(inverse[:n].cpu().numpy().astype(np.int64), w_inv.reshape(-1))
    assert np.array_equal(counts[:nu].cpu().numpy().astype(np.int64), w_cnt)
    # same answer as the torch call the reference makes (embed_optimizer.py:41)
    t_u, t_i = torch.unique(torch.from_numpy(idx).cuda(), return_inverse=True)
    assert torch.equal(t_u, uniq[:nu]) and torch.equal(t_i.int(), inverse[:n])


def test_unique_rows_edge_cases():
    # empty input
    _, _, _, n_unique = _unique(np.zeros(0, np.int64), 100)
    assert n_unique.tolist() == [0, 0]
    # ids outside the table are counted, get slot -1 and do not disturb the others
    idx = np.array([5, -1, 99, 100, 5, 7, 1 << 40], np.int64)
    uniq, inverse, counts, n_unique = _unique(idx, 100)
    assert n_unique.tolist() == [3, 3]
    assert uniq[:3].tolist() == [5, 7, 99]
    assert inverse[:7].tolist() == [0, -1, 2, -1, 0, 1, -1]
    assert counts[:3].tolist() == [2, 1, 1]
    # the same through the short-list route (large id space)
    big = 5000000
    idx = np.array([5, -1, big - 1, big, 5, 7, 1 << 40, 7, 7], np.int64)
    uniq, inverse, counts, n_unique = _unique(idx, big)
    assert n_unique.tolist() == [3, 3]
    assert uniq[:3].tolist() == [5, 7, big - 1]
    assert inverse[:9].tolist() == [0, -1, 2, -1, 0, 1, -1, 1, 1]
    assert counts[:3].tolist() == [2, 3, 1]
    uniq, inverse, counts, n_unique = _unique(np.full(3000, big - 1), big)
    assert n_unique.tolist() == [1, 0] and uniq[0].item() == big - 1 and counts[0].item() == 3000
    assert inverse[:3000].unique().tolist() == [0]
    uniq, inverse, counts, n_unique = _unique(np.array([-3, big + 1], np.int64), big)
    assert n_unique.tolist() == [0, 2] and inverse[:2].tolist() == [-1, -1]
    # every id identical; last id of the table; table size not a multiple of 32
    uniq, inverse, counts, n_unique = _unique(np.full(1000, 32), 33)
    assert n_unique.tolist() == [1, 0] and uniq[0].item() == 32 and counts[0].item() == 1000


def test_gather_rows(oracle):
    from smore_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(0)
    for N, W, n in [(100, 7, 33), (5000, 400, 1000), (77, 1000, 5), (10, 4, 1)]:
        table = rng.standard_normal((N, W)).astype(np.float32)
        idx = rng.integers(0, N, n)
        t, i = torch.from_numpy(table).cuda(), torch.from_numpy(idx).cuda()
        out = torch.empty(n, W, device="cuda")
        _lib.check(L.smore_gather_rows(t.data_ptr(), i.data_ptr(), N, out.data_ptr(), n, W, _st()), "gather")
        assert np.array_equal(out.cpu().numpy(), oracle.gather_rows(table, idx))


@pytest.mark.parametrize("W", [24, 400, 37])
def test_scatter_add_rows(oracle, W):
    from smore_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(W)
    N, n = 300, 2000
    idx = rng.integers(0, N, n)
    grad = rng.standard_normal((n, W)).astype(np.float32)
    uniq, inverse, counts, n_unique = _unique(idx, N)
    g_rows = torch.full((n, W), float("nan"), device="cuda")
    _lib.check(L.smore_zero_shared_rows(g_rows.data_ptr(), counts.data_ptr(), n_unique.data_ptr(), n, W, _st()), "zero")
    g = torch.from_numpy(grad).cuda()
    _lib.check(L.smore_scatter_add_rows(g.data_ptr(), inverse.data_ptr(), counts.data_ptr(), g_rows.data_ptr(), n, W,
                                        _st()), "scatter")
    w_uniq, w_inv, _ = oracle.unique_rows(idx)
    want = oracle.scatter_sum_rows(grad, w_inv, len(w_uniq))
    close(g_rows[:len(w_uniq)].cpu().numpy(), want, RTOL_ATOMIC)


@pytest.mark.parametrize("opt,squeeze", [("adam", False), ("adam", True), ("adagrad", False), ("adagrad", True),
                                         ("sgd", False)])
def test_row_optimizers_vs_reference_golden(golden, opt, squeeze):
    """Three consecutive steps against tables produced by the reference's own update_step code."""
    from smore_b200 import embedding
    z = golden["optimizer"]
    tag = "opt/%s_%s/" % (opt, "rowwise" if squeeze else "full")
    emb = embedding.SparseEmbedding(*z["opt/table0"].shape)
    emb.embedding.data.copy_(torch.from_numpy(z["opt/table0"]))
    emb = emb.cuda()

    class Args(object):
        optim_mode = "(aggr,%s,gpu,%s,0)" % (opt, squeeze)
        share_optim_stats = False

    o = embedding.get_optim_class(Args())(Args(), emb, 0)
    lr = float(z["opt/lr"])
    for step in range(3):
        o.step += 1
        o.update_step(torch.from_numpy(z["opt/step%d/uniq" % step]), None,
                      torch.from_numpy(z["opt/step%d/merged_grad" % step]), lr)
        close(emb.embedding.data.cpu().numpy(), z[tag + "table_after%d" % step], RTOL, what="table")
        if opt == "adam":
            close(o.state("state_sum_fo").cpu().numpy(), z[tag + "m_after%d" % step], RTOL, what="m")
            close(o.state("state_sum_sq").cpu().numpy(), z[tag + "v_after%d" % step], RTOL, what="v")
        elif opt == "adagrad":
            close(o.state("state_sum").cpu().numpy(), z[tag + "v_after%d" % step], RTOL, what="state")


@pytest.mark.parametrize("squeeze", [False, True])
def test_device_side_step_counter_matches_host_side(golden, squeeze):
    """Adam with its step counter kept on the device (what a replayed CUDA graph needs) follows
    the reference-generated tables exactly like the host-side counter does."""
    from smore_b200 import embedding
    z = golden["optimizer"]
    tag = "opt/adam_%s/" % ("rowwise" if squeeze else "full")
    emb = embedding.SparseEmbedding(*z["opt/table0"].shape)
    emb.embedding.data.copy_(torch.from_numpy(z["opt/table0"]))
    emb = emb.cuda()

    class Args(object):
        optim_mode = ("aggr", "adam", "gpu", squeeze, 0)
        share_optim_stats = False

    o = embedding.AdamEmbedOptimizer(Args(), emb, 0)
    o.use_device_step()
    lr = float(z["opt/lr"])
    for step in range(3):
        o.update_step(torch.from_numpy(z["opt/step%d/uniq" % step]), None,
                      torch.from_numpy(z["opt/step%d/merged_grad" % step]), lr)
        close(emb.embedding.data.cpu().numpy(), z[tag + "table_after%d" % step], RTOL, what="table")
        close(o.state("state_sum_fo").cpu().numpy(), z[tag + "m_after%d" % step], RTOL, what="m")
    assert int(o._step_dev.item()) == 3


@pytest.mark.parametrize("opt,squeeze", [("adam", False), ("adam", True), ("adagrad", True)])
def test_lookup_merge_update_through_optimizer_api(golden, oracle, opt, squeeze):
    """zero_grad -> three lookups -> backward -> apply_grad, as train_step_mp drives it
    (train_process.py:174-220), with the gradients of the golden step lists."""
    from smore_b200 import embedding
    z = golden["optimizer"]
    tag = "opt/%s_%s/" % (opt, "rowwise" if squeeze else "full")
    emb = embedding.SparseEmbedding(*z["opt/table0"].shape)
    emb.embedding.data.copy_(torch.from_numpy(z["opt/table0"]))
    emb = emb.cuda()
    emb.train()

    class Args(object):
        optim_mode = ("aggr", opt, "gpu", squeeze, 0)
        share_optim_stats = False

    o = embedding.get_optim_class(Args())(Args(), emb, 0)
    lr = float(z["opt/lr"])
    for step in range(3):
        idx = torch.from_numpy(z["opt/step%d/idx" % step])
        grad = torch.from_numpy(z["opt/step%d/grad" % step]).cuda()
        o.zero_grad()
        parts, at = [], 0
        for n in (5, 40, 5):                      # the three lookups of the golden step
            rows = emb(idx[at:at + n], "lookup%d" % n)
            assert np.array_equal(rows.detach().cpu().numpy(),
                                  emb.embedding.data.cpu().numpy()[idx[at:at + n].numpy()])
            parts.append((rows * grad[at:at + n]).sum())
            at += n
        sum(parts).backward()
        o.apply_grad(lr)
        close(emb.embedding.data.cpu().numpy(), z[tag + "table_after%d" % step], RTOL_ATOMIC, what="table")
    assert o.step == 3


@pytest.mark.parametrize("op", ["l1", "l2", "box_out", "box_in", "rotate", "complex", "distmult"])
@pytest.mark.parametrize("shape", [(6, 50, 6, 1, 64), (4, 9, 4, 1, 30), (1, 40, 5, 1, 36), (5, 1, 5, 1, 400),
                                   (1, 70, 16, 1, 48)],
                         ids=lambda s: "x".join(map(str, s)))
def test_table_resident_rows_equal_gathered_rows(oracle, op, shape):
    """forward_rows(table, idx) == forward(table[idx]); backward_rows accumulates what
    merge_grad_list would build from the dense entity gradient."""
    from smore_b200 import _lib
    L = _lib.lib()
    be, ne, bc, nc, dim = shape
    N = 64                                       # small table: many duplicate rows
    mul = 2 if op in ("rotate", "complex") else 1
    tab, q0, q1 = make_operands(op, N, 1, bc, nc, dim, seed=sum(shape))
    table = tab.reshape(N, dim * mul)
    rng = np.random.default_rng(1)
    idx = rng.integers(0, N, be * ne)
    ent = table[idx].reshape(be, ne, dim * mul)
    bsize, num = max(be, bc), max(ne, nc)
    want = oracle.dist_forward(op, ent, q0, q1)
    gout = rng.standard_normal(want.shape).astype(np.float32)
    w_ent, w_q0, w_q1 = oracle.dist_backward(op, gout, ent, q0, q1)
    w_uniq, w_inv, _ = oracle.unique_rows(idx)
    w_rows = oracle.scatter_sum_rows(w_ent.reshape(be * ne, -1), w_inv, len(w_uniq))

    t, i = torch.from_numpy(table).cuda(), torch.from_numpy(idx).cuda()
    d_q0 = torch.from_numpy(q0).cuda()
    d_q1 = None if q1 is None else torch.from_numpy(q1).cuda()
    dst = torch.empty(bsize, num, device="cuda")
    sizes = (bsize, num, be, ne, bc, nc, dim)
    _lib.check(L.smore_dist_forward_rows(_lib.DIST_IDS[op], t.data_ptr(), i.data_ptr(), N, d_q0.data_ptr(),
                                         None if q1 is None else d_q1.data_ptr(), dst.data_ptr(), *sizes, _st()), "fwd")
    close(dst.cpu().numpy(), want, RTOL, forward_scale(oracle, op, ent, q0, q1))

    uniq, inverse, counts, n_unique = _unique(idx, N)
    g_rows = torch.full((be * ne, dim * mul), float("nan"), device="cuda")
    _lib.check(L.smore_zero_shared_rows(g_rows.data_ptr(), counts.data_ptr(), n_unique.data_ptr(), be * ne,
                                        dim * mul, _st()), "zero")
    g_q0 = torch.full_like(d_q0, float("nan"))
    g_q1 = None if q1 is None else torch.full_like(d_q1, float("nan"))
    _lib.check(L.smore_dist_backward_rows(_lib.DIST_IDS[op], torch.from_numpy(gout).cuda().data_ptr(), t.data_ptr(),
                                          i.data_ptr(), N, d_q0.data_ptr(), None if q1 is None else d_q1.data_ptr(),
                                          inverse.data_ptr(), counts.data_ptr(), g_rows.data_ptr(), g_q0.data_ptr(),
                                          None if q1 is None else g_q1.data_ptr(), *sizes, _st()), "bwd")
    close(g_rows[:len(w_uniq)].cpu().numpy(), w_rows, RTOL_ATOMIC, what="g_rows")
    close(g_q0.cpu().numpy(), w_q0, 2 * RTOL, what="g_first")
    if q1 is not None:
        close(g_q1.cpu().numpy(), w_q1, 2 * RTOL, what="g_second")


@pytest.mark.parametrize("op", ["l1", "l2", "box_out", "box_in", "box_both", "rotate", "complex", "distmult"])
@pytest.mark.parametrize("shape", [(6, 50, 64), (3, 9, 36), (5, 700, 400), (2, 33, 1000)],
                         ids=lambda s: "x".join(map(str, s)))
def test_union_branches_in_one_pass(oracle, op, shape):
    """smore_union_*_rows == the per-branch oracle calls stacked on the branch axis, with the row
    gradients of both branches summed into the step's compact gradient rows."""
    from smore_b200 import _lib
    L = _lib.lib()
    B, K, dim = shape
    U, N = 2, 97
    base = "box_out" if op == "box_both" else op
    mul = 2 if op in ("rotate", "complex") else 1
    tab, q0, q1 = make_operands(base, N, 1, B * U, 1, dim, seed=sum(shape))
    table = tab.reshape(N, dim * mul)
    q0 = q0.reshape(B, U, dim)
    q1 = None if q1 is None else q1.reshape(B, U, dim)
    rng = np.random.default_rng(2)
    idx = rng.integers(0, N, B * K)
    ent = table[idx].reshape(B, K, dim * mul)
    names = ["box_out", "box_in"] if op == "box_both" else [op]
    gouts = [rng.standard_normal((B, U, K)).astype(np.float32) for _ in names]
    want = [np.zeros((B, U, K), np.float32) for _ in names]
    w_ent = np.zeros_like(ent)
    w_q0, w_q1 = np.zeros_like(q0), None if q1 is None else np.zeros_like(q1)
    for u in range(U):
        f = np.ascontiguousarray(q0[:, u:u + 1])
        s = None if q1 is None else np.ascontiguousarray(q1[:, u:u + 1])
        for k, nm in enumerate(names):
            want[k][:, u] = oracle.dist_forward(nm, ent, f, s)
            ge, g0, g1 = oracle.dist_backward(nm, np.ascontiguousarray(gouts[k][:, u]), ent, f, s)
            w_ent += ge
            w_q0[:, u:u + 1] += g0
            if q1 is not None:
                w_q1[:, u:u + 1] += g1
    w_uniq, w_inv, _ = oracle.unique_rows(idx)
    w_rows = oracle.scatter_sum_rows(w_ent.reshape(B * K, -1), w_inv, len(w_uniq))

    dev = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ptr = lambda t_: None if t_ is None else t_.data_ptr()
    t, i, d_q0, d_q1 = dev(table), dev(idx), dev(q0), dev(q1)
    dist_id = _lib.BOX_BOTH_ID if op == "box_both" else _lib.DIST_IDS[op]
    dst = [torch.full((B, U, K), float("nan"), device="cuda") for _ in names]
    _lib.check(L.smore_union_forward_rows(dist_id, t.data_ptr(), i.data_ptr(), N, ptr(d_q0), ptr(d_q1), dst[0].data_ptr(),
                                          dst[1].data_ptr() if len(dst) > 1 else None, U, B, K, dim, _st()), "fwd")
    for k, nm in enumerate(names):
        scale = forward_scale(oracle, nm, ent, np.ascontiguousarray(q0[:, :1]),
                              None if q1 is None else np.ascontiguousarray(q1[:, :1]))
        close(dst[k].cpu().numpy(), want[k], RTOL, scale, what=nm)

    uniq, inverse, counts, n_unique = _unique(idx, N)
    g_rows = torch.full((B * K, dim * mul), float("nan"), device="cuda")
    _lib.check(L.smore_zero_shared_rows(g_rows.data_ptr(), counts.data_ptr(), n_unique.data_ptr(), B * K, dim * mul,
                                        _st()), "zero")
    g_q0 = torch.full_like(d_q0, float("nan"))
    g_q1 = None if q1 is None else torch.full_like(d_q1, float("nan"))
    d_g = [dev(g) for g in gouts]
    _lib.check(L.smore_union_backward_rows(dist_id, d_g[0].data_ptr(), d_g[1].data_ptr() if len(d_g) > 1 else None,
                                           t.data_ptr(), i.data_ptr(), N, ptr(d_q0), ptr(d_q1), inverse.data_ptr(),
                                           counts.data_ptr(), g_rows.data_ptr(), g_q0.data_ptr(), ptr(g_q1), U, B, K,
                                           dim, _st()), "bwd")
    close(g_rows[:len(w_uniq)].cpu().numpy(), w_rows, RTOL_ATOMIC, what="g_rows")
    close(g_q0.cpu().numpy(), w_q0, 4 * RTOL, what="g_first")
    if q1 is not None:
        close(g_q1.cpu().numpy(), w_q1, 4 * RTOL, what="g_second")
    # other branch counts are the caller's loop
    assert L.smore_union_forward_rows(dist_id, t.data_ptr(), i.data_ptr(), N, ptr(d_q0), ptr(d_q1), dst[0].data_ptr(),
                                      dst[-1].data_ptr(), 3, B, K, dim, _st()) == -2


@pytest.mark.parametrize("op", ["l1", "box", "rotate"])
def test_union_front_end_equals_branch_loop(op, monkeypatch):
    """ext_ops with a [B, 2, 1, dim] query on table rows: the one-pass route and the per-branch loop
    of the reference front-end give the same scores, query gradients and table update."""
    from smore_b200 import embedding, ext_ops
    B, K, dim, N = 8, 64, 64, 300
    mul = 2 if op == "rotate" else 1
    torch.manual_seed(3)
    init = (torch.rand(N, dim * mul) - 0.5) * 0.3
    idx = torch.randint(0, N, (B, K)).cuda()
    q = [((torch.rand(B, 2, 1, dim) - 0.5) * 0.3).cuda() for _ in range(2)]
    q[1] = q[1].abs()

    class Args(object):
        optim_mode = ("aggr", "adam", "gpu", True, 0)
        share_optim_stats = False

    results = []
    for fused in (True, False):
        if not fused:
            monkeypatch.setattr(ext_ops, "_union_in_one_pass", lambda *a: False)
        emb = embedding.SparseEmbedding(N, dim * mul)
        emb.embedding.data.copy_(init)
        emb = emb.cuda()
        emb.train()
        opt = embedding.AdamEmbedOptimizer(Args(), emb, 0, lazy_names=("negative_entity",))
        opt.zero_grad()
        rows = emb(idx.view(-1), "negative_entity").view(B, K, -1)
        a, b = q[0].clone().requires_grad_(), q[1].clone().requires_grad_()
        if op == "l1":
            score = ext_ops.l1_dist(rows, a)
        elif op == "rotate":
            score = ext_ops.rotate_dist(rows, a, b)
        else:
            score = ext_ops.box_dist_out(rows, a, b) + 0.02 * ext_ops.box_dist_in(rows, a, b)
        assert score.shape == (B, 2, K)
        (torch.max(score, dim=1)[0] ** 2).sum().backward()
        opt.apply_grad(1e-2)
        torch.cuda.synchronize()
        results.append((score.detach().cpu(), a.grad.cpu(), None if b.grad is None else b.grad.cpu(),
                        emb.embedding.data.cpu()))
    (s1, a1, b1, t1), (s0, a0, b0, t0) = results
    assert torch.equal(s1, s0)
    close(a1.numpy(), a0.numpy(), RTOL, what="g_first")
    if b0 is not None:
        close(b1.numpy(), b0.numpy(), RTOL, what="g_second")
    close(t1.numpy(), t0.numpy(), RTOL_ATOMIC, what="table")
