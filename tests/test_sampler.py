"""Negative sampling: the alias tables against the reference's own AliasMethod (compiled where it
lies into oracle/_ref/libsmore_ref_kg.so; CPU), and the GPU draws' properties (marked gpu)."""
import ctypes
import os

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libsmore_ref_kg.so")


@pytest.mark.parametrize("n,kind", [(1, "flat"), (7, "flat"), (1000, "power"), (50000, "power"), (64, "one_hot"),
                                    (333, "zeros")])
def test_alias_tables_equal_the_reference_tables(n, kind):
    from smore_b200 import sampler
    if not os.path.exists(REF):
        pytest.skip("reference library not built")
    lib = ctypes.CDLL(REF)
    lib.ref_alias_build.argtypes = [ctypes.c_void_p, ctypes.c_size_t] + [ctypes.c_void_p] * 3
    rng = np.random.default_rng(n)
    if kind == "flat":
        w = np.ones(n)
    elif kind == "power":
        w = 1.0 / (1.0 + rng.permutation(n)) ** 1.2
    elif kind == "one_hot":
        w = np.zeros(n)
        w[n // 3] = 2.5
    else:
        w = rng.random(n)
        w[rng.integers(0, n, n // 2)] = 0.0          # entities nobody points to
    prob, small, large = sampler.build_alias_table(w)
    r_prob, r_small, r_large = np.empty(n), np.empty(n, np.int64), np.empty(n, np.int64)
    w64 = np.ascontiguousarray(w, np.float64)
    assert lib.ref_alias_build(w64.ctypes.data, n, r_prob.ctypes.data, r_small.ctypes.data, r_large.ctypes.data) == 0
    assert np.array_equal(prob, r_prob) and np.array_equal(small, r_small) and np.array_equal(large, r_large)
    # and the tables encode the weights: P(i) = sum over slots of the share that lands on i
    p = np.zeros(n)
    np.add.at(p, small, prob / n)
    np.add.at(p, large, (1.0 - prob) / n)
    np.testing.assert_allclose(p, w / w.sum(), atol=1e-12)


@pytest.mark.gpu
def test_uniform_draws_are_reproducible_in_range_and_never_answers():
    from smore_b200 import sampler
    N, Q, K = 1000, 64, 512
    rng = np.random.default_rng(0)
    answers = [rng.choice(N, size=rng.integers(1, 400), replace=False) for _ in range(Q)]
    csr = sampler.answers_csr(answers, "cuda")
    a = sampler.NegativeSampler(N, "cuda", seed=7)
    b = sampler.NegativeSampler(N, "cuda", seed=7)
    x, y = a.sample(Q, K, csr), b.sample(Q, K, csr)
    assert torch.equal(x, y) and x.shape == (Q, K)
    assert not torch.equal(x, a.sample(Q, K, csr))          # the stream moves on
    assert x.min().item() >= 0 and x.max().item() < N
    xs = x.cpu().numpy()
    for q in range(Q):
        assert not np.isin(xs[q], answers[q]).any()
    assert not torch.equal(sampler.NegativeSampler(N, "cuda", seed=8).sample(Q, K, csr), x)
    # uniform over the non-answers: chi-square of the counts of one query with few answers
    big = sampler.NegativeSampler(200, "cuda", seed=1).sample(1, 400000, sampler.answers_csr([[5, 6, 7]], "cuda"))
    counts = np.bincount(big.cpu().numpy().ravel(), minlength=200)
    assert counts[5:8].sum() == 0
    expect = 400000 / 197.0
    chi2 = ((np.delete(counts, [5, 6, 7]) - expect) ** 2 / expect).sum()
    assert chi2 < 197 + 6 * np.sqrt(2 * 197)


@pytest.mark.gpu
def test_weighted_draws_follow_the_weights_and_shared_mask_marks_answers():
    from smore_b200 import sampler
    N = 300
    rng = np.random.default_rng(3)
    w = 1.0 / (1.0 + rng.permutation(N)) ** 1.1
    w[:10] = 0.0
    s = sampler.NegativeSampler(N, "cuda", weights=w, seed=11)
    draws = s.sample(4, 250000).cpu().numpy().ravel()
    counts = np.bincount(draws, minlength=N)
    assert counts[:10].sum() == 0
    p = w / w.sum()
    keep = p > 0
    expect = p[keep] * draws.size
    chi2 = ((counts[keep] - expect) ** 2 / expect).sum()
    dof = keep.sum() - 1
    assert chi2 < dof + 6 * np.sqrt(2 * dof)
    answers = [rng.choice(N, size=40, replace=False) for _ in range(9)]
    neg, mask = s.sample_shared(128, sampler.answers_csr(answers, "cuda"))
    assert neg.shape == (1, 128) and mask.shape == (9, 128)
    nn, mm = neg.cpu().numpy()[0], mask.cpu().numpy()
    for q in range(9):
        assert np.array_equal(mm[q] == 0.0, np.isin(nn, answers[q]))
