"""Filtered ranks by counting (smore_filtered_ranks) against the reference's argsort/scatter
block restated on the CPU (needs a B200)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _answers(rng, n, n_easy, n_hard):
    ids = rng.choice(n, size=min(n, n_easy + n_hard), replace=False)
    return list(map(int, ids[:min(n_easy, len(ids))])), list(map(int, ids[min(n_easy, len(ids)):]))


@pytest.mark.parametrize("n,levels", [(1, 0), (17, 0), (5000, 0), (5000, 7), (300000, 0), (300000, 50)])
def test_filtered_ranks_equal_reference_block(n, levels):
    """Exact equality, ties included (levels > 0 quantises the logits so that many are equal)."""
    from oracle.native_torch import reference_filtered_ranks
    from smore_b200 import ranking
    rng = np.random.default_rng(n + levels)
    sizes = [(0, 1), (3, 1), (0, 40), (25, 60), (700, 900), (0, 0)]
    Q = len(sizes)
    logits = torch.from_numpy(rng.standard_normal((Q, n)).astype(np.float32))
    if levels:
        logits = torch.round(logits * levels) / levels
    easy, hard = [], []
    for ne, nh in sizes:
        e, h = _answers(rng, n, ne, nh)
        easy.append(e)
        hard.append(h)
    got = ranking.filtered_ranks(logits.cuda(), easy, hard)
    for q in range(Q):
        want = reference_filtered_ranks(logits[q], easy[q], hard[q]) if hard[q] else torch.empty(0)
        assert got[q].dtype == torch.int64 and got[q].numel() == len(hard[q])
        assert torch.equal(got[q].cpu().float(), want), "query %d" % q


def test_metrics_and_full_table_scoring_path():
    """The evaluation path end to end: box logits of 5 queries against every entity through the
    distance ops (one shared candidate set, be = 1, ne = N), filtered ranks, metrics."""
    from oracle.native_torch import reference_filtered_ranks, reference_ranking_metrics
    from smore_b200 import ext_ops, ranking
    torch.manual_seed(0)
    N, D, Q = 20000, 64, 5
    table = ((torch.rand(N, D) - 0.5) * 0.4).cuda()
    center = ((torch.rand(Q, 1, D) - 0.5) * 0.4).cuda()
    offset = (torch.rand(Q, 1, D) * 0.1).cuda()
    all_entities = table.unsqueeze(0)                      # [1, N, D]: every query scores all entities
    logits = 12.0 - ext_ops.box_dist_out(all_entities, center, offset) \
        - 0.02 * ext_ops.box_dist_in(all_entities, center, offset)
    assert logits.shape == (Q, N)
    rng = np.random.default_rng(5)
    easy, hard = zip(*[_answers(rng, N, 10 * q, 1 + 30 * q) for q in range(Q)])
    # make the answers score well, as a trained model would: some of them rank first
    for q in range(Q):
        logits[q, hard[q][0]] = logits[q].max() + 1.0
    ranks = ranking.filtered_ranks(logits, easy, hard)
    for q in range(Q):
        want = reference_filtered_ranks(logits[q].cpu(), easy[q], hard[q])
        assert torch.equal(ranks[q].cpu().float(), want)
        got_m, want_m = ranking.ranking_metrics(ranks[q]), reference_ranking_metrics(want)
        for k in want_m:
            assert abs(got_m[k] - want_m[k]) < 1e-6, k
        assert got_m["HITS1max"] == 1.0


def test_filtered_ranks_rejects_bad_input():
    from smore_b200 import _lib, ranking
    logits = torch.zeros(1, 10, device="cuda")
    with pytest.raises(ValueError):
        ranking.filtered_ranks(logits, [[]], [[10]])
    with pytest.raises(TypeError):
        ranking.filtered_ranks(logits.double(), [[]], [[1]])
    with pytest.raises(_lib.SmoreError):
        ranking.filtered_ranks(torch.zeros(1, 9000, device="cuda"), [[]], [list(range(8193))])


def test_filtered_ranks_special_values_follow_torch_sort_order():
    """NaN ranks first (torch.sort treats it as the largest value), then +inf; -0 ties with +0."""
    from oracle.native_torch import reference_filtered_ranks
    from smore_b200 import ranking
    x = torch.tensor([[0.5, float("nan"), -0.0, 0.0, float("inf"), -float("inf"), 0.5, float("nan"), 1.0, -2.0]])
    easy, hard = [[2]], [[0, 1, 3, 5, 6, 8]]
    got = ranking.filtered_ranks(x.cuda(), easy, hard)[0]
    want = reference_filtered_ranks(x[0], easy[0], hard[0])
    assert torch.equal(got.cpu().float(), want)


def test_evaluation_pair_of_box_calls_is_one_pass_and_exact():
    """Under no_grad, box_dist_out then box_dist_in on the same tensors return what the separate ops
    return; changed operands are not served from the parked result."""
    from smore_b200 import _lib, ext_ops
    torch.manual_seed(1)
    ent = torch.rand(1, 3000, 64, device="cuda") - 0.5
    c = torch.rand(5, 1, 64, device="cuda") - 0.5
    o = torch.rand(5, 1, 64, device="cuda") * 0.2
    ref_out = ext_ops._dist("box_out", ent, c, o)
    ref_in = ext_ops._dist("box_in", ent, c, o)
    L = _lib.lib()
    with torch.no_grad():
        n0 = L.smore_kernel_launch_count()
        d_out = ext_ops.box_dist_out(ent, c, o)
        d_in = ext_ops.box_dist_in(ent, c, o)
        assert L.smore_kernel_launch_count() - n0 == 1          # one pass served both
        assert torch.equal(d_out, ref_out) and torch.equal(d_in, ref_in)
        d_out2 = ext_ops.box_dist_out(ent, c, o)
        c.add_(0.1)                                             # operand changed in place: no reuse
        d_in2 = ext_ops.box_dist_in(ent, c, o)
        assert torch.equal(d_out2, ref_out)
        assert torch.equal(d_in2, ext_ops._dist("box_in", ent, c, o))
        assert not torch.equal(d_in2, ref_in)


def test_ranks_reproduce_the_reference_test_step_metrics(golden):
    """MRR / HITS of the library's filtered ranks against the values the reference's own test_step_mp
    (train_process.py:94-169) logged for the same logits and answer sets (tests/golden/make_golden.py)."""
    from smore_b200 import ranking
    r = golden["ranking"]
    n = int(r["rank/n_cases"])
    cases = [(str(r["rank/%d/tag" % i]), r["rank/%d/logits" % i], r["rank/%d/easy" % i].tolist(),
              r["rank/%d/hard" % i].tolist(), r["rank/%d/metrics" % i]) for i in range(n)]
    logits = torch.from_numpy(np.stack([c[1] for c in cases])).cuda()
    ranks = ranking.filtered_ranks(logits, [c[2] for c in cases], [c[3] for c in cases])
    checked = 0
    for (tag, lg, easy, hard, want), rk in zip(cases, ranks):
        got = ranking.ranking_metrics(rk)
        if tag == "tie_on_answer":
            continue          # the reference leaves the order of tied logits to the sort implementation
        for k, w in zip(("MRR", "HITS1", "HITS3", "HITS10", "HITS1max"), want.tolist()):
            assert abs(got[k] - w) <= 1e-6, (tag, k, got[k], w)
        checked += 1
    assert checked >= 5


@pytest.mark.parametrize("geo,N,D,Q", [("box", 20000, 64, 9), ("vec", 5000, 36, 16), ("rotate", 3000, 40, 8),
                                         ("distmult", 7001, 48, 33), ("l2", 1000, 16, 8), ("box", 300000, 400, 12)])
def test_score_and_rank_equals_ranks_of_materialised_logits(geo, N, D, Q):
    """smore_score_filtered_ranks (scores ranked straight from the scoring tiles) against the two-step
    path: distance ops on all entities -> the model's logit arithmetic in torch -> filtered_ranks.
    Bit-identical ranks: both paths run the same tile code and the same roundings."""
    from smore_b200 import ext_ops, ranking
    g = torch.Generator().manual_seed(N + D)
    two_part = geo in ("rotate", "complex")
    W = 2 * D if two_part else D
    table = ((torch.rand(N, W, generator=g) - 0.5) * 0.4).cuda()
    table[N // 2] = table[N // 3]                       # two identical rows: an exact tie
    n_parts = 1 if geo in ("vec", "distmult", "l2") else 2
    query = [((torch.rand(Q, 1, D, generator=g) - 0.5) * 0.4).cuda() for _ in range(n_parts)]
    if geo == "box":
        query[1] = query[1].abs() * 0.3
    gamma, cen = 12.0, 0.02
    every = table.unsqueeze(0)
    with torch.no_grad():
        if geo == "box":
            logits = gamma - ext_ops.box_dist_out(every, *query) - cen * ext_ops.box_dist_in(every, *query)
        elif geo == "vec":
            logits = gamma - ext_ops.l1_dist(every, query[0])
        elif geo == "l2":
            logits = gamma - ext_ops.l2_dist(every, query[0])
        elif geo == "rotate":
            logits = gamma - ext_ops.rotate_dist(every, *query)
        else:
            import os
            os.environ["SMORE_B200_DOT"] = "off"         # the exact-fp32 kernels, as the fused path uses
            try:
                logits = ext_ops.distmult_sim(every, query[0])
            finally:
                del os.environ["SMORE_B200_DOT"]
    rng = np.random.default_rng(Q)
    easy, hard = zip(*[_answers(rng, N, 3 * (q % 4), 1 + 5 * (q % 5)) for q in range(Q)])
    hard = [list(h) for h in hard]
    hard[0] = sorted(set(hard[0]) | {N // 2, N // 3} - set(easy[0]))     # the tied rows are answers of query 0
    want = ranking.filtered_ranks(logits, easy, hard)
    got = ranking.score_and_rank(geo, table, query, easy, hard, gamma=gamma, cen=cen)
    for q in range(Q):
        assert torch.equal(got[q], want[q]), "query %d" % q
