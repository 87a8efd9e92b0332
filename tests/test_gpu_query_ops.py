"""Fused relation projection of path queries against the per-hop torch ops of the reference models
(vec.py:58-60, box.py:126-129) - needs a B200."""
import numpy as np
import pytest
import torch

from tests.util import close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,H,D,R", [(7, 1, 64, 11), (33, 3, 400, 50), (5, 2, 30, 4)])
@pytest.mark.parametrize("box,relu,with_start_offset", [(False, False, False), (True, False, False),
                                                        (True, True, True), (True, False, True)])
def test_project_path_equals_per_hop_ops(B, H, D, R, box, relu, with_start_offset):
    from smore_b200 import query_ops
    g = torch.Generator().manual_seed(B * 1000 + H)
    queries = torch.randint(0, R, (B, H + 3), generator=g).cuda()       # relation ids are a column block
    rel_ids = queries[:, 2:2 + H]
    start = torch.randn(B, D, generator=g).cuda()
    start_off = torch.rand(B, D, generator=g).cuda() if with_start_offset else None
    rel = torch.randn(R, D, generator=g).cuda()
    off = (torch.randn(R, D, generator=g) * 0.5).cuda() if box else None
    w_c, w_o = torch.randn(B, D, generator=g).cuda(), torch.randn(B, D, generator=g).cuda()

    def run(fused):
        leaves = [t.clone().requires_grad_() if t is not None else None for t in (start, start_off, rel, off)]
        s, so, r, o = leaves
        if fused:
            out = query_ops.project_path(s, r, rel_ids, start_offset=so, off_table=o, relu_offset=relu)
            c, of = out if box else (out, None)
        else:
            c = s
            of = (so if so is not None else torch.zeros_like(s)) if box else None
            for h in range(H):
                c = c + r[rel_ids[:, h]]
                if box:
                    x = o[rel_ids[:, h]]
                    of = of + (torch.relu(x) if relu else x)
        loss = (c * w_c).sum() + ((of * w_o).sum() if box else 0.0)
        loss.backward()
        return [c.detach(), None if of is None else of.detach()] + [None if t is None else t.grad for t in leaves]

    got, want = run(True), run(False)
    assert torch.equal(got[0], want[0])                       # same additions in the same order
    if box:
        assert torch.equal(got[1], want[1])
    for a, b, name in zip(got[2:], want[2:], ("g_start", "g_start_offset", "g_rel", "g_off")):
        assert (a is None) == (b is None), name
        if a is not None:
            close(a.cpu().numpy(), b.cpu().numpy(), 1e-5, what=name)


@pytest.mark.parametrize("geo_workload", ["q2b_fb15k", "gqe_fb15k237", "rotate_wikikg", "complex_wikikg", "distmult_wikikg"])
@pytest.mark.parametrize("structure", ["1p", "2p", "3p", "2i", "ip", "pi", "2u", "up"])
def test_query_model_with_fused_paths_matches_per_hop_model(geo_workload, structure):
    """The step with every path embedded by one kernel, anchors read from the table in place, against
    the same step with gathered anchors and per-hop torch ops."""
    import bench
    from smore_b200 import embedding, ext_ops
    cfg = dict(bench.WORKLOADS[geo_workload])
    cfg.update(B=16, K=32, structures=[structure], dim=min(cfg["dim"], 200))
    n_rows, dev = 500, torch.device("cuda", 0)
    torch.manual_seed(4)
    a = bench.QueryModel(cfg, n_rows, dev, ext_ops, embedding, fused_paths=True)
    torch.manual_seed(4)
    b = bench.QueryModel(cfg, n_rows, dev, ext_ops, embedding, fused_paths=False)
    b.load_state_dict(a.state_dict())
    a.train(), b.train()
    pos, neg, q = [t.to(dev) for t in bench.make_batch(cfg, n_rows, structure, seed=9)]
    la = bench.train_step(a, pos, neg, q, structure)
    lb = bench.train_step(b, pos, neg, q, structure)
    torch.cuda.synchronize()
    close(la.item(), lb.item(), 1e-6 if cfg["geo"] in ("box", "vec") else 1e-5, what="loss")
    close(a.relation_embedding.detach().cpu().numpy(), b.relation_embedding.detach().cpu().numpy(), 1e-5, what="relations")
    close(a.entity_embedding.embedding.detach().cpu().numpy(), b.entity_embedding.embedding.detach().cpu().numpy(), 1e-4,
          what="entity table")


def _per_hop(geometry, state, rel, rel_ids, phase_scale):
    """The reference models' relation_projection, hop by hop (rotate.py:101-109, complex.py:108-117 and
    distmult.py:106-111 with the identity normaliser, vec.py:58-60)."""
    H = rel_ids.shape[1]
    if geometry in ("rotate", "complex"):
        D = state.shape[1] // 2
        re, im = state[:, :D], state[:, D:]
        for h in range(H):
            r = rel[rel_ids[:, h]]
            if geometry == "rotate":
                ph = r * phase_scale
                c, s = torch.cos(ph), torch.sin(ph)
            else:
                c, s = r[:, :D], r[:, D:]
            re, im = re * c - im * s, re * s + im * c
        return re, im
    out = state
    for h in range(H):
        r = rel[rel_ids[:, h]]
        out = out * r if geometry == "distmult" else out + r
    return (out,)


@pytest.mark.parametrize("geometry", ["rotate", "complex", "distmult", "add"])
@pytest.mark.parametrize("B,H,D,R", [(9, 1, 64, 7), (33, 3, 100, 20), (4, 2, 30, 3)])
def test_embed_path_equals_per_hop_ops(geometry, B, H, D, R):
    from smore_b200 import query_ops
    g = torch.Generator().manual_seed(B + 10 * H + len(geometry))
    two = geometry in ("rotate", "complex")
    W = 2 * D if two else D
    rel_ids = torch.randint(0, R, (B, H + 2), generator=g).cuda()[:, 1:1 + H]
    start = (torch.randn(B, W, generator=g) * 0.5).cuda()
    rel = (torch.randn(R, 2 * D if geometry == "complex" else D, generator=g) * (1.5 if geometry == "rotate" else 0.8)).cuda()
    scale = 2.7 if geometry == "rotate" else 1.0
    weights = [torch.randn(B, D, generator=g).cuda() for _ in range(2)]

    def run(fused):
        s, r = start.clone().requires_grad_(), rel.clone().requires_grad_()
        out = query_ops.embed_path(geometry, s, r, rel_ids, phase_scale=scale) if fused else \
            _per_hop(geometry, s, r, rel_ids, scale)
        out = out if isinstance(out, tuple) else (out,)
        sum((o * w).sum() for o, w in zip(out, weights)).backward()
        return [o.detach() for o in out], s.grad, r.grad

    (o1, gs1, gr1), (o2, gs2, gr2) = run(True), run(False)
    for a, b in zip(o1, o2):
        close(a.cpu().numpy(), b.cpu().numpy(), 1e-5, what=geometry + " out")
    close(gs1.cpu().numpy(), gs2.cpu().numpy(), 1e-5, what=geometry + " g_start")
    close(gr1.cpu().numpy(), gr2.cpu().numpy(), 1e-4, what=geometry + " g_rel")


@pytest.mark.parametrize("geometry", ["rotate", "add", "distmult"])
def test_embed_path_from_table_rows_equals_gathered_anchors(geometry):
    """Anchors given as a table-resident lookup: same outputs, same relation gradients and - after the
    optimizer step - the same table as the gathered lookup followed by the per-hop ops."""
    from smore_b200 import embedding, query_ops
    N, D, B, H, R = 500, 48, 40, 2, 9
    two = geometry == "rotate"
    W = 2 * D if two else D
    g = torch.Generator().manual_seed(len(geometry))
    init = (torch.rand(N, W, generator=g) - 0.5) * 0.6
    ids = torch.randint(0, N, (B,), generator=g)
    ids[:6] = ids[6:12]                                      # anchors shared between queries
    ids = ids.cuda()
    rel_ids = torch.randint(0, R, (B, H), generator=g).cuda()
    rel0 = (torch.randn(R, D, generator=g) * 0.7).cuda()
    weights = [torch.randn(B, D, generator=g).cuda() for _ in range(2)]

    class Args(object):
        optim_mode = ("aggr", "adam", "gpu", True, 0)
        share_optim_stats = False

    results = []
    for lazy in (True, False):
        emb = embedding.SparseEmbedding(N, W)
        emb.embedding.data.copy_(init)
        emb = emb.cuda()
        emb.train()
        opt = embedding.AdamEmbedOptimizer(Args(), emb, 0, lazy_names=("anchor_entity",) if lazy else ())
        opt.zero_grad()
        rel = rel0.clone().requires_grad_()
        rows = emb(ids, "anchor_entity")
        if lazy:
            assert isinstance(rows, embedding.LazyRows)
            out = query_ops.embed_path(geometry, rows, rel, rel_ids, phase_scale=1.3)
        else:
            out = _per_hop(geometry, rows, rel, rel_ids, 1.3)
        out = out if isinstance(out, tuple) else (out,)
        sum((o * w).sum() for o, w in zip(out, weights)).backward()
        opt.apply_grad(1e-2)
        torch.cuda.synchronize()
        results.append(([o.detach().cpu().numpy() for o in out], rel.grad.cpu().numpy(), emb.embedding.data.cpu().numpy()))
    (o1, gr1, t1), (o2, gr2, t2) = results
    for a, b in zip(o1, o2):
        close(a, b, 1e-5, what="outputs")
    close(gr1, gr2, 1e-4, what="g_rel")
    close(t1, t2, 1e-4, what="table after the step")
    untouched = np.ones(N, bool)
    untouched[ids.cpu().numpy()] = False
    assert np.array_equal(t1[untouched], init.numpy()[untouched])
