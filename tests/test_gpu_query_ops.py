"""Fused relation projection of path queries against the per-hop torch ops of the reference models
(vec.py:58-60, box.py:126-129) - needs a B200."""
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


@pytest.mark.parametrize("geo_workload", ["q2b_fb15k", "gqe_fb15k237"])
@pytest.mark.parametrize("structure", ["1p", "2p", "3p", "ip", "pi", "2u", "up"])
def test_query_model_with_fused_paths_matches_per_hop_model(geo_workload, structure):
    import bench
    from smore_b200 import embedding, ext_ops
    cfg = dict(bench.WORKLOADS[geo_workload])
    cfg.update(B=16, K=32, structures=[structure])
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
    close(la.item(), lb.item(), 1e-6, what="loss")
    close(a.relation_embedding.detach().cpu().numpy(), b.relation_embedding.detach().cpu().numpy(), 1e-5, what="relations")
    close(a.entity_embedding.embedding.detach().cpu().numpy(), b.entity_embedding.embedding.detach().cpu().numpy(), 1e-4,
          what="entity table")
