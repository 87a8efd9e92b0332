"""Parity of the CUDA distance ops with the CPU oracle and the golden vectors (needs a B200).

Every case goes through the C ABI: either via the `extlib_cuda`-compatible module (the entry
the reference's autograd functions call) or via smore_b200.ext_ops (the op API the models call).
"""
import numpy as np
import pytest
import torch

from tests.util import OPS, RTOL, RTOL_ATOMIC, TWO_QUERY, close, forward_scale, make_operands

pytestmark = pytest.mark.gpu

# (be, ne, bc, nc, dim) — all broadcast combinations the op contract allows, dims that are not
# multiples of 4 / 32 / 128, ragged candidate counts, and the row-streaming fast path
SHAPES = [
    (30, 1, 1, 20, 40),      # the reference self-check orientation
    (1, 7, 5, 1, 33),        # shared candidates, odd dim
    (6, 1, 6, 1, 100),       # positives
    (4, 6, 2, 3, 17),        # mixed broadcast both ways
    (2, 3, 4, 6, 9),
    (1, 1, 1, 1, 1),         # smallest possible
    (3, 37, 3, 1, 64),       # per-query candidates, ragged K, 1 chunk of 16 bytes per lane
    (5, 96, 5, 1, 400),      # the Query2box row shape
    (2, 300, 2, 1, 500),     # the RotatE row shape (two-part rows of 1000 floats)
    (3, 40, 3, 1, 1000),     # widest rows the streaming kernels take
    (2, 19, 2, 1, 1028),     # wider than that: falls back to the cell kernels
    (3, 12, 3, 1, 30),       # dim not a multiple of 4: cell kernels
    (1, 5000, 1, 1, 128),    # one query against many rows (evaluation orientation), several CTAs per query
    (1, 100, 40, 1, 64),     # shared candidates: the tiled kernels, ragged tiles
    (1, 512, 70, 1, 400),    # shared candidates at the Query2box row shape
    (1, 33, 9, 1, 500),      # shared candidates, two-part rows of 1000 floats, dim not a multiple of 16
    (1, 64, 64, 1, 16),      # exactly one tile
]


def _dev(a):
    return None if a is None else torch.from_numpy(a).cuda()


@pytest.fixture(scope="module")
def ext():
    from smore_b200 import extlib_cuda
    return extlib_cuda


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("op", OPS)
def test_forward_backward_vs_oracle(oracle, ext, op, shape):
    be, ne, bc, nc, dim = shape
    ent, q0, q1 = make_operands(op, be, ne, bc, nc, dim, seed=sum(map(ord, op)) + sum(shape))
    want = oracle.dist_forward(op, ent, q0, q1)
    d_ent, d_q0, d_q1 = _dev(ent), _dev(q0), _dev(q1)
    dst = torch.full(want.shape, float("nan"), device="cuda")
    ext.dist_forward(op, d_ent, d_q0, d_q1, dst)
    close(dst.cpu().numpy(), want, RTOL, forward_scale(oracle, op, ent, q0, q1), "forward")

    rng = np.random.default_rng(7)
    gout = rng.standard_normal(want.shape).astype(np.float32)
    w_ent, w_q0, w_q1 = oracle.dist_backward(op, gout, ent, q0, q1)
    g_ent = torch.full_like(d_ent, float("nan"))
    g_q0 = torch.full_like(d_q0, float("nan"))
    g_q1 = None if q1 is None else torch.full_like(d_q1, float("nan"))
    ext.dist_backward(op, _dev(gout), d_ent, d_q0, d_q1, g_ent, g_q0, g_q1)
    # several CTAs may share one query row (atomics) when a query has many candidate rows
    q_rtol = RTOL_ATOMIC if (nc == 1 and ne >= 256) else 2 * RTOL
    close(g_ent.cpu().numpy(), w_ent, 2 * RTOL, what="g_entity")
    close(g_q0.cpu().numpy(), w_q0, q_rtol, what="g_first")
    if q1 is not None:
        close(g_q1.cpu().numpy(), w_q1, q_rtol, what="g_second")


@pytest.mark.parametrize("op", OPS)
def test_fp64_path(oracle, ext, op):
    be, ne, bc, nc, dim = 3, 8, 3, 1, 37
    ent, q0, q1 = make_operands(op, be, ne, bc, nc, dim, seed=11)
    want = oracle.dist_forward_f64acc(op, ent, q0, q1)
    d = [None if a is None else torch.from_numpy(a.astype(np.float64)).cuda() for a in (ent, q0, q1)]
    dst = torch.empty(want.shape, dtype=torch.float64, device="cuda")
    ext.dist_forward(op, d[0], d[1], d[2], dst)
    np.testing.assert_allclose(dst.cpu().numpy(), want, rtol=1e-6, atol=1e-7)
    gout = torch.ones_like(dst)
    g = [torch.empty_like(d[0]), torch.empty_like(d[1]), None if d[2] is None else torch.empty_like(d[2])]
    ext.dist_backward(op, gout, d[0], d[1], d[2], g[0], g[1], g[2])
    w = oracle.dist_backward(op, np.ones(want.shape, np.float32), ent, q0, q1)
    for got, ref in zip(g, w):
        if got is not None:
            np.testing.assert_allclose(got.cpu().numpy(), ref, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("shape_name", ["selfcheck", "per_query_neg", "shared_neg", "positives"])
@pytest.mark.parametrize("op", OPS)
def test_op_api_vs_reference_golden(golden, op, shape_name):
    """The ops as the models call them (autograd included) against vectors produced by the
    reference's pure-torch twins with its self-check loss sum(out ** 2) * 3.14."""
    from smore_b200 import ext_ops
    fn = {"l1": ext_ops.l1_dist, "l2": ext_ops.l2_dist, "box_out": ext_ops.box_dist_out,
          "box_in": ext_ops.box_dist_in, "rotate": ext_ops.rotate_dist, "complex": ext_ops.complex_sim,
          "distmult": ext_ops.distmult_sim}[op]
    z = golden["ops"]
    k = "%s/%s/" % (shape_name, op)
    entity = torch.from_numpy(z[k + "entity"]).cuda().requires_grad_()
    qs = [torch.from_numpy(z[k + "q%d" % i]).cuda().requires_grad_() for i in range(2 if op in TWO_QUERY else 1)]
    out = fn(entity, *qs)
    want = z[k + "out"]
    scale = float(np.abs(want).max()) * (8.0 if op in ("complex", "distmult") else 1.0)
    close(out.detach().cpu().numpy(), want, RTOL, scale, "forward")
    (torch.sum(out ** 2) * 3.14).backward()
    close(entity.grad.cpu().numpy(), z[k + "g_entity"], 3 * RTOL, what="g_entity")
    for i, q in enumerate(qs):
        close(q.grad.cpu().numpy(), z[k + "g_q%d" % i], 3 * RTOL, what="g_q%d" % i)


def test_model_logits_with_union_branches(golden):
    """4-D query operands [B, U, 1, D]: per-branch op calls stacked to [B, U, K], then the
    models' gamma - dist and max over branches (box.py:157-164, vec.py:85-90, rotate.py:137-142)."""
    from smore_b200 import ext_ops
    z = golden["logits"]
    ent, c, o = (torch.from_numpy(z["logit/box/" + n]).cuda() for n in ("entity", "center", "offset"))
    d1, d2 = ext_ops.box_dist_out(ent, c, o), ext_ops.box_dist_in(ent, c, o)
    assert d1.shape == (ent.shape[0], c.shape[1], ent.shape[1])
    box = torch.max(12.0 - d1 - 0.02 * d2, dim=1)[0]
    close(box.cpu().numpy(), z["logit/box/out"], RTOL, 12.0)
    both = ext_ops.box_dist_both(ent, c, o)
    assert torch.equal(both[0], d1) and torch.equal(both[1], d2)
    vec = torch.max(12.0 - ext_ops.l1_dist(ent, c), dim=1)[0]
    close(vec.cpu().numpy(), z["logit/vec/out"], RTOL, 12.0)
    ent2, re, im = (torch.from_numpy(z["logit/rotate/" + n]).cuda() for n in ("entity", "re", "im"))
    rot = torch.max(12.0 - ext_ops.rotate_dist(ent2, re, im), dim=1)[0]
    close(rot.cpu().numpy(), z["logit/rotate/out"], RTOL, 12.0)


def test_tie_rules_follow_the_reference(oracle, ext):
    """Exact ties (e == c, |e-c| == o, zero distance) take the reference functors' branches."""
    rng = np.random.default_rng(3)
    for op in OPS:
        mul = 2 if op in ("rotate", "complex") else 1
        for (be, ne, bc, nc, dim) in [(3, 40, 3, 1, 64), (2, 5, 4, 1, 12)]:
            ent = rng.integers(-2, 3, (be, ne, dim * mul)).astype(np.float32) * 0.5
            q0 = rng.integers(-2, 3, (bc, nc, dim)).astype(np.float32) * 0.5
            q1 = (rng.integers(0, 3, (bc, nc, dim)).astype(np.float32) * 0.5) if op in TWO_QUERY else None
            gout = rng.integers(-2, 3, (max(be, bc), max(ne, nc))).astype(np.float32)
            want = oracle.dist_backward(op, gout, ent, q0, q1)
            d = [_dev(ent), _dev(q0), _dev(q1)]
            g = [torch.empty_like(d[0]), torch.empty_like(d[1]), None if q1 is None else torch.empty_like(d[2])]
            ext.dist_backward(op, _dev(gout), d[0], d[1], d[2], g[0], g[1], g[2])
            for got, ref in zip(g, want):
                if got is not None:
                    close(got.cpu().numpy(), ref, 2 * RTOL, what=op)


def test_shim_rejects_bad_arguments(ext):
    from smore_b200._lib import SmoreError
    e = torch.zeros(2, 3, 8, device="cuda")
    c = torch.zeros(2, 1, 8, device="cuda")
    with pytest.raises(ValueError):
        ext.l1_dist_forward(e, c, torch.zeros(3, 3, device="cuda"))          # wrong output shape
    with pytest.raises(ValueError):
        ext.l1_dist_forward(e, c, torch.zeros(3, 2, device="cuda").t())      # output buffer not contiguous
    with pytest.raises(ValueError):
        ext.rotate_dist_forward(e, c, c, torch.zeros(2, 3, device="cuda"))   # rows must be 2 x dim
    with pytest.raises(ValueError):
        ext.box_dist_forward(e, c, c, torch.zeros(2, 3, device="cuda"), "sideways")
    with pytest.raises(TypeError):
        ext.l1_dist_forward(e, c.double(), torch.zeros(2, 3, device="cuda"))
    with pytest.raises(SmoreError):
        ext.l1_dist_forward(torch.zeros(2, 3, 8, device="cuda"), torch.zeros(3, 1, 8, device="cuda"),
                            torch.zeros(3, 3, device="cuda"))                # 2 vs 3 do not broadcast
    with pytest.raises(NotImplementedError):
        ext.beta_dist_forward()
    assert ext.ThreadPool(1).num_threads == 1
    ext.AsyncGPUJob(0).sync()
    ext.CudaEvent(0).record()


def test_shim_accepts_strided_inputs(oracle, ext):
    """Inputs with any strides are accepted (autograd hands the backward of the reference front-ends'
    torch.stack over union branches, box_dist.py:60-68, a strided grad_out)."""
    ent, q0, q1 = make_operands("box_out", 5, 7, 5, 1, 24, seed=2)
    gout = np.random.default_rng(3).standard_normal((5, 7)).astype(np.float32)
    want = oracle.dist_backward("box_out", gout, ent, q0, q1)
    d = [_dev(ent), _dev(q0), _dev(q1)]
    stacked = torch.stack([_dev(gout), _dev(gout) * 2], dim=1)     # [5, 2, 7]
    strided_gout = stacked[:, 0]                                     # strides (14, 1): not contiguous
    assert not strided_gout.is_contiguous()
    strided_ent = torch.stack([d[0], d[0]], dim=2)[:, :, 0]          # [5, 7, 24] view with gaps
    assert not strided_ent.is_contiguous()
    g = [torch.empty_like(d[0]), torch.empty_like(d[1]), torch.empty_like(d[2])]
    ext.box_dist_backward(strided_gout, strided_ent, d[1], d[2], g[0], g[1], g[2], "out")
    for got, ref in zip(g, want):
        close(got.cpu().numpy(), ref, 2 * RTOL)
    dst = torch.empty(5, 7, device="cuda")
    ext.box_dist_forward(strided_ent, d[1], d[2], dst, "out")
    close(dst.cpu().numpy(), oracle.dist_forward("box_out", ent, q0, q1), RTOL)


def test_reference_cuda_kernels_agree(oracle):
    """Cross-check against the reference's own kernels recompiled for sm_100a, at a size the CPU
    oracle would take minutes for (skipped where that library was not built)."""
    import ctypes
    from oracle.oracle import reference_cuda_path
    from smore_b200 import extlib_cuda as ext
    path = reference_cuda_path()
    if path is None:
        pytest.skip("reference CUDA library not built")
    ref = ctypes.CDLL(path)
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    ref.ref_cuda_dist_forward.argtypes = [ctypes.c_int, vp, vp, vp, vp] + [sz] * 7 + [vp]
    ref.ref_cuda_dist_backward.argtypes = [ctypes.c_int] + [vp] * 7 + [sz] * 7 + [vp]
    from oracle.oracle import DIST_IDS
    B, K, dim = 64, 512, 400
    st = torch.cuda.current_stream().cuda_stream
    for op in OPS:
        ent, q0, q1 = make_operands(op, B, K, B, 1, dim, seed=5)
        d = [_dev(ent), _dev(q0), _dev(q1)]
        mine = torch.empty(B, K, device="cuda")
        theirs = torch.empty(B, K, device="cuda")
        ext.dist_forward(op, d[0], d[1], d[2], mine)
        assert ref.ref_cuda_dist_forward(DIST_IDS[op], d[0].data_ptr(), d[1].data_ptr(),
                                         None if q1 is None else d[2].data_ptr(), theirs.data_ptr(), B, K, B, K, B,
                                         1, dim, st) == 0
        torch.cuda.synchronize()
        close(mine.cpu().numpy(), theirs.cpu().numpy(), RTOL, forward_scale(oracle, op, ent[:2], q0[:2],
                                                                            None if q1 is None else q1[:2]))
        gout = torch.randn(B, K, device="cuda")
        g = [torch.empty_like(d[0]), torch.empty_like(d[1]), None if q1 is None else torch.empty_like(d[2])]
        r = [torch.zeros_like(d[0]), torch.zeros_like(d[1]), None if q1 is None else torch.zeros_like(d[2])]
        ext.dist_backward(op, gout, d[0], d[1], d[2], g[0], g[1], g[2])
        assert ref.ref_cuda_dist_backward(DIST_IDS[op], gout.data_ptr(), d[0].data_ptr(), d[1].data_ptr(),
                                          None if q1 is None else d[2].data_ptr(), r[0].data_ptr(), r[1].data_ptr(),
                                          None if q1 is None else r[2].data_ptr(), B, K, B, K, B, 1, dim, st) == 0
        torch.cuda.synchronize()
        close(g[0].cpu().numpy(), r[0].cpu().numpy(), 2 * RTOL, what=op + " g_entity")
        close(g[1].cpu().numpy(), r[1].cpu().numpy(), RTOL_ATOMIC, what=op + " g_first")
        if q1 is not None:
            close(g[2].cpu().numpy(), r[2].cpu().numpy(), RTOL_ATOMIC, what=op + " g_second")


@pytest.mark.parametrize("op,shared", [("box_out", False), ("box_in", False), ("rotate", False), ("l1", False),
                                       ("box_out", True), ("distmult", True)])
def test_speed_against_reference_kernels(op, shared, capsys):
    """The reference's kernels recompiled for sm_100a are the kernels to beat: same operands
    (materialised candidate rows, B = K = 1024), CUDA-event times of forward and backward, results
    compared; prints one line per case (run with -s to see it)."""
    import ctypes
    from oracle.oracle import DIST_IDS, reference_cuda_path
    from smore_b200 import extlib_cuda as ext
    path = reference_cuda_path()
    if path is None:
        pytest.skip("reference CUDA library not built")
    ref = ctypes.CDLL(path)
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    ref.ref_cuda_dist_forward.argtypes = [ctypes.c_int, vp, vp, vp, vp] + [sz] * 7 + [vp]
    ref.ref_cuda_dist_backward.argtypes = [ctypes.c_int] + [vp] * 7 + [sz] * 7 + [vp]
    B, K = 1024, 1024
    dim = 500 if op == "rotate" else 400
    mul = 2 if op == "rotate" else 1
    two = op in ("box_out", "box_in", "rotate")
    be = 1 if shared else B
    g = torch.Generator(device="cuda").manual_seed(11)
    ent = (torch.rand(be, K, mul * dim, device="cuda", generator=g) - 0.5) * 0.1
    q0 = (torch.rand(B, 1, dim, device="cuda", generator=g) - 0.5) * 0.1
    q1 = torch.rand(B, 1, dim, device="cuda", generator=g) * 0.05 if two else None
    gout = torch.randn(B, K, device="cuda", generator=g)
    st = torch.cuda.current_stream().cuda_stream
    p = lambda t: None if t is None else t.data_ptr()
    mine, theirs = torch.empty(B, K, device="cuda"), torch.empty(B, K, device="cuda")
    gm = [torch.empty_like(ent), torch.empty_like(q0), None if q1 is None else torch.empty_like(q1)]
    gr = [torch.zeros_like(ent), torch.zeros_like(q0), None if q1 is None else torch.zeros_like(q1)]

    def ours_fwd():
        ext.dist_forward(op, ent, q0, q1, mine)

    def ours_bwd():
        ext.dist_backward(op, gout, ent, q0, q1, gm[0], gm[1], gm[2])

    def ref_fwd():
        assert ref.ref_cuda_dist_forward(DIST_IDS[op], p(ent), p(q0), p(q1), p(theirs), B, K, be, K, B, 1, dim, st) == 0

    def ref_bwd():
        assert ref.ref_cuda_dist_backward(DIST_IDS[op], p(gout), p(ent), p(q0), p(q1), p(gr[0]), p(gr[1]), p(gr[2]),
                                          B, K, be, K, B, 1, dim, st) == 0

    def time_ms(fn, reps):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    t = {"ours_fwd": time_ms(ours_fwd, 5), "ref_fwd": time_ms(ref_fwd, 3),
         "ours_bwd": time_ms(ours_bwd, 5), "ref_bwd": time_ms(ref_bwd, 2)}
    # forward and entity gradient: sums re-associated only; query gradient: the reference's order over
    # the K candidates differs and its kernel for shared candidates accumulates with atomics
    fscale = float((ent.abs().reshape(-1, mul * dim)[:64] @ q0.abs().reshape(-1, dim)[:64].t()).max()) \
        if op == "distmult" else None
    close(mine.cpu().numpy(), theirs.cpu().numpy(), RTOL, fscale, what=op + " forward")
    tol = RTOL if not shared else RTOL_ATOMIC      # compared on the device: up to 4 GB per operand
    bound = tol * float(gr[0].abs().max()) + tol * gr[0].abs()
    assert bool(((gm[0] - gr[0]).abs() <= bound).all()), op + " g_entity"
    del bound
    close(gm[1].cpu().numpy(), gr[1].cpu().numpy(), RTOL_ATOMIC, what=op + " g_first")
    if q1 is not None:
        close(gm[2].cpu().numpy(), gr[2].cpu().numpy(), RTOL_ATOMIC, what=op + " g_second")
    with capsys.disabled():
        print("\nreference-kernel comparison %s %s B=K=1024 dim=%d: forward %.3f ms vs %.3f ms (x%.1f), "
              "backward %.3f ms vs %.3f ms (x%.1f)" % (op, "shared" if shared else "per-query", dim, t["ours_fwd"],
                                                       t["ref_fwd"], t["ref_fwd"] / t["ours_fwd"], t["ours_bwd"],
                                                       t["ref_bwd"], t["ref_bwd"] / t["ours_bwd"]))
    assert t["ours_fwd"] < t["ref_fwd"] * 1.1 and t["ours_bwd"] < t["ref_bwd"]
