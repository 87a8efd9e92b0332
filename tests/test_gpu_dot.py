"""DistMult / ComplEx scoring against shared candidates on the tensor cores (needs a B200).

Tolerances (relative to the sum of |terms| of a score, which bounds the rounding error of any
summation order): "fp32" mode (three bf16 terms per operand, nine MMAs per product) 2e-5;
"tf32" mode 2e-3.  The SIMT kernels (mode "off") are the exact-fp32 comparison."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops(monkeypatch, mode):
    monkeypatch.setenv("SMORE_B200_DOT", mode)
    from smore_b200 import ext_ops
    return ext_ops


@pytest.mark.parametrize("mode,tol", [("fp32", 2e-5), ("tf32", 2e-3)])
@pytest.mark.parametrize("op", ["distmult", "complex"])
def test_shared_candidate_scores_and_gradients(monkeypatch, mode, tol, op):
    from smore_b200 import _lib
    if not _lib.lib().smore_dot_available():
        pytest.skip("library built without the tensor-core GEMM path")
    ops = _ops(monkeypatch, mode)
    B, K, D = 256, 384, 200
    g = torch.Generator(device="cuda").manual_seed(3)
    W = D * (2 if op == "complex" else 1)
    ent = (torch.randn(1, K, W, device="cuda", generator=g) * 0.05).requires_grad_()
    qs = [(torch.randn(B, 1, D, device="cuda", generator=g) * 0.05).requires_grad_()
          for _ in range(2 if op == "complex" else 1)]
    w = torch.randn(B, K, device="cuda", generator=g)
    fn = ops.complex_sim if op == "complex" else ops.distmult_sim
    out = fn(ent, *qs)
    (out * w).sum().backward()
    # float64 reference
    e64 = ent.detach().double().requires_grad_()
    q64 = [q.detach().double().requires_grad_() for q in qs]
    qcat = torch.cat(q64, dim=-1)
    ref = (qcat[:, 0, :] @ e64[0].t())
    (ref * w.double()).sum().backward()
    scale = (qcat[:, 0, :].abs() @ e64[0].abs().t()).max().item()
    assert (out.double() - ref).abs().max().item() <= tol * scale
    g_scale_e = (w.abs().double().t() @ qcat[:, 0, :].abs()).max().item()
    assert (ent.grad.double() - e64.grad).abs().max().item() <= tol * g_scale_e
    g_scale_q = (w.abs().double() @ e64[0].abs()).max().item()
    for q, r in zip(qs, q64):
        assert (q.grad.double() - r.grad).abs().max().item() <= tol * g_scale_q


@pytest.mark.parametrize("mode,tol", [("fp32", 2e-5), ("tf32", 2e-3)])
def test_full_depth_block_against_fp64(monkeypatch, mode, tol):
    """A block of the wikikg-size DistMult workload with the full inner dimension (512 queries x 1024
    shared candidates x 1000), scores and both gradients against float64."""
    from smore_b200 import _lib
    if not _lib.lib().smore_dot_available():
        pytest.skip("library built without the tensor-core GEMM path")
    ops = _ops(monkeypatch, mode)
    B, K, W = 512, 1024, 1000
    g = torch.Generator(device="cuda").manual_seed(17)
    ent = (torch.randn(1, K, W, device="cuda", generator=g) * 0.05).requires_grad_()
    q = (torch.randn(B, 1, W, device="cuda", generator=g) * 0.05).requires_grad_()
    w = torch.randn(B, K, device="cuda", generator=g)
    out = ops.distmult_sim(ent, q)
    (out * w).sum().backward()
    e64, q64, w64 = ent.detach().double()[0], q.detach().double()[:, 0], w.double()
    assert (out.double() - q64 @ e64.t()).abs().max().item() <= tol * (q64.abs() @ e64.abs().t()).max().item()
    assert (ent.grad.double()[0] - w64.t() @ q64).abs().max().item() <= tol * (w64.abs().t() @ q64.abs()).max().item()
    assert (q.grad.double()[:, 0] - w64 @ e64).abs().max().item() <= tol * (w64.abs() @ e64.abs()).max().item()


def test_full_size_gemm_route_against_simt_route_and_fp64(monkeypatch):
    """The whole wikikg-size problem (4096 queries x 8192 shared candidates x 1000): the GEMM route in
    its default precision against the exact-fp32 SIMT kernels on 65,536 sampled cells, and scores and
    gradients of sampled rows against float64."""
    from smore_b200 import _lib
    if not _lib.lib().smore_dot_available():
        pytest.skip("library built without the tensor-core GEMM path")
    B, K, W = 4096, 8192, 1000
    g = torch.Generator(device="cuda").manual_seed(23)
    ent = torch.randn(1, K, W, device="cuda", generator=g) * 0.05
    q = torch.randn(B, 1, W, device="cuda", generator=g) * 0.05
    w = torch.randn(B, K, device="cuda", generator=g)
    res = {}
    for mode in ("off", "fp32"):
        ops = _ops(monkeypatch, mode)
        e, qq = ent.clone().requires_grad_(), q.clone().requires_grad_()
        out = ops.distmult_sim(e, qq)
        (out * w).sum().backward()
        res[mode] = (out.detach(), e.grad[0], qq.grad[:, 0])
    torch.cuda.synchronize()
    bi = torch.randint(0, B, (65536,), device="cuda", generator=g)
    ki = torch.randint(0, K, (65536,), device="cuda", generator=g)
    e64, q64, w64 = ent.double()[0], q.double()[:, 0], w.double()
    cells64 = (q64[bi] * e64[ki]).sum(-1)
    scale = (q64[bi].abs() * e64[ki].abs()).sum(-1).max().item()
    tol = 2e-5
    assert (res["fp32"][0][bi, ki].double() - res["off"][0][bi, ki].double()).abs().max().item() <= tol * scale
    assert (res["fp32"][0][bi, ki].double() - cells64).abs().max().item() <= tol * scale
    rows_k = torch.randint(0, K, (64,), device="cuda", generator=g)
    rows_b = torch.randint(0, B, (64,), device="cuda", generator=g)
    ge64 = w64[:, rows_k].t() @ q64
    gq64 = w64[rows_b] @ e64
    ge_scale = (w64[:, rows_k].abs().t() @ q64.abs()).max().item()
    gq_scale = (w64[rows_b].abs() @ e64.abs()).max().item()
    for mode in ("off", "fp32"):
        assert (res[mode][1][rows_k].double() - ge64).abs().max().item() <= tol * ge_scale, mode
        assert (res[mode][2][rows_b].double() - gq64).abs().max().item() <= tol * gq_scale, mode


def test_gemm_route_agrees_with_simt_route_and_handles_table_rows(monkeypatch):
    """Same op through the SIMT kernels (exact fp32) and through the GEMM route, with the candidates
    given as table rows (a LazyRows handle) the second time."""
    from smore_b200 import _lib, embedding
    if not _lib.lib().smore_dot_available():
        pytest.skip("library built without the tensor-core GEMM path")
    B, K, D, N = 128, 256, 64, 5000
    g = torch.Generator(device="cuda").manual_seed(5)
    emb = embedding.SparseEmbedding(N, D)
    emb = emb.cuda()
    emb.embedding.data.normal_(0, 0.05, generator=g)
    emb.train()

    class Args(object):
        optim_mode = ("aggr", "sgd", "gpu", False, 0)
        share_optim_stats = False

    opt = embedding.SGDEmbedOptimizer(Args(), emb, 0, lazy_names=("negative_entity",))
    idx = torch.randint(0, N, (K,), device="cuda", generator=g)
    q = torch.randn(B, 1, D, device="cuda", generator=g) * 0.05
    outs, tables = [], []
    for mode in ("off", "fp32"):
        ops = _ops(monkeypatch, mode)
        table0 = emb.embedding.data.clone()
        opt.zero_grad()
        rows = emb(idx, "negative_entity").view(1, K, -1)
        qq = q.clone().requires_grad_()
        out = ops.distmult_sim(rows, qq)
        (out ** 2).sum().backward()
        opt.apply_grad(0.1)
        outs.append(out.detach())
        tables.append(emb.embedding.data - table0)
        emb.embedding.data.copy_(table0)
    torch.cuda.synchronize()
    np.testing.assert_allclose(outs[1].cpu().numpy(), outs[0].cpu().numpy(), rtol=0, atol=2e-5 * 64 * 0.05 * 0.05 * 9)
    np.testing.assert_allclose(tables[1].cpu().numpy(), tables[0].cpu().numpy(), rtol=1e-4,
                               atol=1e-4 * tables[0].abs().max().item())


def test_tile_variant_is_reported():
    """The two-SM tiles live in an optional companion library; the main library says whether it found
    it, and the products above were checked on whichever variant is active."""
    from smore_b200 import _lib
    assert _lib.lib().smore_dot_two_sm() in (0, 1)
    print("tensor-core tiles:", "two SMs per tile" if _lib.lib().smore_dot_two_sm() else "one SM per tile")
