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
