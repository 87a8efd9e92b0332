"""Host-side logic that needs no GPU: option parsing, the lazy row handle, the benchmark's
synthetic batches, and the torch-native baseline against the reference-generated vectors."""
import numpy as np
import pytest
import torch

import bench
from smore_b200 import embedding


def test_eval_tuple_matches_reference_parsing():
    assert embedding.eval_tuple("(aggr,adam,gpu,True,5)") == ("aggr", "adam", "gpu", True, 5)
    assert embedding.eval_tuple("(fast,adagrad,gpu,False,0)") == ("fast", "adagrad", "gpu", False, 0)
    assert embedding.eval_tuple(("aggr", "sgd", "gpu", False, 1)) == ("aggr", "sgd", "gpu", False, 1)
    assert embedding.eval_tuple("[aggr, adam, gpu, True, 5]") == ("aggr", "adam", "gpu", True, 5)


def test_get_optim_class():
    class A(object):
        optim_mode = "(aggr,adam,gpu,True,5)"
    assert embedding.get_optim_class(A) is embedding.AdamEmbedOptimizer
    A.optim_mode = "(aggr,adagrad,gpu,True,5)"
    assert embedding.get_optim_class(A) is embedding.AdaGradEmbedOptimizer
    A.optim_mode = "(aggr,sgd,gpu,True,5)"
    assert embedding.get_optim_class(A) is embedding.SGDEmbedOptimizer
    A.optim_mode = "(aggr,rmsprop,gpu,True,5)"
    with pytest.raises(NotImplementedError):
        embedding.get_optim_class(A)


def test_optimizer_refuses_cpu_table():
    from smore_b200._lib import SmoreError
    emb = embedding.SparseEmbedding(10, 4)

    class A(object):
        optim_mode = "(aggr,adam,gpu,True,5)"
    with pytest.raises(SmoreError):
        embedding.AdamEmbedOptimizer(A(), emb, 0)


class _Owner(object):
    table = torch.zeros(50, 8)


class _Lk(object):
    n = 24


def test_lazy_rows_shape_algebra():
    rows = embedding.LazyRows(_Owner(), _Lk(), (24, 8))
    assert rows.dim() == 2 and tuple(rows.shape) == (24, 8)
    v = rows.view(4, 6, -1)
    assert tuple(v.shape) == (4, 6, 8) and v.as_3d() == (4, 6, 8) and v.lookup is rows.lookup
    assert tuple(rows.view(-1, 6, 8).shape) == (4, 6, 8)
    assert tuple(rows.unsqueeze(1).shape) == (24, 1, 8) and rows.unsqueeze(1).as_3d() == (24, 1, 8)
    assert rows.as_3d() == (24, 1, 8)
    rows.job_handle.sync()
    with pytest.raises(ValueError):
        rows.view(4, 6, 4)          # rows cannot be split
    with pytest.raises(ValueError):
        rows.view(5, 5, 8)
    with pytest.raises(ValueError):
        rows.unsqueeze(2)


def test_remote_rows_stay_remote_through_views():
    """Rows of a sharded table that their owners score: views keep the handle's kind (so that the
    distance ops route them to the owners), and they cannot be turned into a local tensor."""
    from smore_b200 import _lib, sharded
    rows = sharded.RemoteRows(_Owner(), _Lk(), (24, 8))
    v = rows.view(4, 6, -1)
    assert isinstance(v, sharded.RemoteRows) and v.remote and v.as_3d() == (4, 6, 8)
    assert isinstance(v.unsqueeze(0), sharded.RemoteRows)
    assert not getattr(embedding.LazyRows(_Owner(), _Lk(), (24, 8)), "remote", False)
    with pytest.raises(_lib.SmoreError):
        rows.materialize()
    with pytest.raises(ValueError):
        sharded.RemoteSpec(pairs=0, queries=4, dim=8)


def test_structure_columns_and_batches():
    want = {"1p": "er", "2p": "err", "3p": "errr", "2i": "erer", "3i": "ererer", "ip": "ererr", "pi": "errer",
            "2u": "ereru", "up": "ererur"}
    for name, cols in want.items():
        assert "".join(bench.structure_columns(bench.STRUCTURES[name])) == cols
    cfg = bench.WORKLOADS["freebase_q2b"]
    pos, neg, q = bench.make_batch(cfg, 1000003, "up", seed=1)
    assert pos.shape == (1024,) and neg.shape == (1024, 1024) and q.shape == (1024, 6)
    assert int(neg.min()) >= 0 and int(neg.max()) < 1000003
    assert (q[:, 4] == -1).all() and int(q[:, 0].max()) < 1000003 and int(q[:, 1].max()) < cfg["relations"]
    pos2, neg2, q2 = bench.make_batch(cfg, 1000003, "up", seed=1)
    assert torch.equal(neg, neg2) and torch.equal(q, q2)          # seeded
    # anchors are skewed (power law), negatives are not
    assert torch.unique(q[:, 0]).numel() < 1024 * 0.9
    shared = bench.make_batch(bench.WORKLOADS["q2b_fb15k"], 14951, "2i", seed=0)[1]
    assert shared.shape == (1, 512)


def test_native_torch_baseline_vs_reference_golden(golden):
    from oracle import native_torch as nt
    z = golden["logits"]
    t = lambda k: torch.from_numpy(z[k])
    box = nt.box_logit(t("logit/box/entity"), (t("logit/box/center"), t("logit/box/offset")), 12.0, 0.02)
    assert torch.equal(box, t("logit/box/out"))
    vec = nt.vec_logit(t("logit/box/entity"), (t("logit/box/center"),), 12.0)
    assert torch.equal(vec, t("logit/vec/out"))
    rot = nt.rotate_logit(t("logit/rotate/entity"), (t("logit/rotate/re"), t("logit/rotate/im")), 12.0)
    assert torch.equal(rot, t("logit/rotate/out"))
    zo = golden["optimizer"]
    for squeeze in (False, True):
        tag = "opt/adam_%s/" % ("rowwise" if squeeze else "full")
        table = torch.from_numpy(zo["opt/table0"].copy())
        m = torch.zeros_like(table)
        v = torch.zeros(table.shape[0], 1) if squeeze else torch.zeros_like(table)
        for step in range(3):
            idx = torch.from_numpy(zo["opt/step%d/idx" % step])
            grad = torch.from_numpy(zo["opt/step%d/grad" % step])
            u, inv, merged = nt.merge_grads([idx], [grad])
            assert np.array_equal(u.numpy(), zo["opt/step%d/uniq" % step])
            nt.adam_rows(table, m, v, u, merged, float(zo["opt/lr"]), step + 1, squeeze)
            np.testing.assert_allclose(table.numpy(), zo[tag + "table_after%d" % step], rtol=1e-6, atol=1e-7)


def test_reference_ranking_block_matches_the_counting_definition():
    """The restated argsort/scatter block (the checker of the GPU ranks) against the definition it is
    replaced by: rank = 1 + candidates ahead - answers ahead, ahead = higher logit or equal logit
    and lower id."""
    import numpy as np
    import torch
    from oracle.native_torch import reference_filtered_ranks
    rng = np.random.default_rng(0)
    for n, levels in [(1, 0), (50, 0), (400, 5)]:
        x = rng.standard_normal(n).astype(np.float32)
        if levels:
            x = np.round(x * levels) / levels
        ids = rng.choice(n, size=min(n, 30), replace=False)
        easy, hard = [int(i) for i in ids[:len(ids) // 3]], [int(i) for i in ids[len(ids) // 3:]]
        answers = set(easy) | set(hard)
        want = []
        for a in hard:
            ahead = [e for e in range(n) if x[e] > x[a] or (x[e] == x[a] and e < a)]
            want.append(1 + len(ahead) - len([e for e in ahead if e in answers]))
        got = reference_filtered_ranks(torch.from_numpy(x), easy, hard)
        assert sorted(want) == [int(v) for v in got.tolist()]
