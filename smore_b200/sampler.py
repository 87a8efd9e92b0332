"""Negative sampling on the GPU (smore_sample_negatives / smore_negative_mask / smore_alias_build).

The step before the row lookups: per query `k` entity ids that are not answers of the query, drawn
uniformly or with per-entity weights through an alias table, or one list shared by the batch with the
mask of entries that are answers - what the reference's NaiveSampler does on host threads
(smore/cpp_sampler/src/lib/naive_sampler.cpp:28-50, sampler.cpp:90-99, alias_method.cpp:33-99).
Draws are a function of (seed, position in the stream): reproducible, unlike the reference's
clock-seeded generators.
"""
import numpy as np
import torch

from . import _lib


def build_alias_table(weights):
    """(prob_small float64 [n], choice_small int64 [n], choice_large int64 [n]) for non-negative
    weights, by the reference's procedure (alias_method.cpp:55-99); numpy arrays on the host."""
    w = np.ascontiguousarray(weights, dtype=np.float64)
    n = w.size
    prob = np.empty(n, np.float64)
    small = np.empty(n, np.int64)
    large = np.empty(n, np.int64)
    _lib.check(_lib.lib().smore_alias_build(w.ctypes.data, n, prob.ctypes.data, small.ctypes.data, large.ctypes.data),
               "smore_alias_build")
    return prob, small, large


def answers_csr(answer_lists, device):
    """Per-query answer ids (any order) -> (ptr int64 [Q + 1], ids int64, ascending per query) on `device`."""
    ptr, ids = [0], []
    for a in answer_lists:
        ids.extend(sorted(int(x) for x in a))
        ptr.append(len(ids))
    return (torch.tensor(ptr, dtype=torch.int64, device=device),
            torch.tensor(ids if ids else [0], dtype=torch.int64, device=device))


class NegativeSampler(object):
    """n_entities ids, uniform or weighted (e.g. by in-degree, as --online_weighted_negative_sampling);
    every call continues one reproducible stream of draws."""

    def __init__(self, n_entities, device, weights=None, seed=0):
        self.n_entities, self.device, self.seed, self.offset = int(n_entities), torch.device(device), int(seed), 0
        self.tables = None
        if weights is not None:
            if len(weights) != self.n_entities:
                raise ValueError("one weight per entity")
            prob, small, large = build_alias_table(weights)
            self.tables = (torch.from_numpy(prob).to(self.device), torch.from_numpy(small).to(self.device),
                           torch.from_numpy(large).to(self.device))

    def _draw(self, n_queries, k, csr):
        out = torch.empty(n_queries, k, dtype=torch.int64, device=self.device)
        t = self.tables
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().smore_sample_negatives(
                self.seed, self.offset, self.n_entities, None if t is None else t[0].data_ptr(),
                None if t is None else t[1].data_ptr(), None if t is None else t[2].data_ptr(),
                None if csr is None else csr[0].data_ptr(), None if csr is None else csr[1].data_ptr(), n_queries, k,
                out.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream), "smore_sample_negatives")
        self.offset += n_queries * k
        return out

    def sample(self, n_queries, k, answers=None):
        """negatives [n_queries, k]; `answers`: (ptr, ids) from answers_csr, whose ids are never drawn."""
        return self._draw(n_queries, k, answers)

    def sample_shared(self, k, answers):
        """One list for the whole batch: (negatives [1, k], is_negative float32 [Q, k])."""
        neg = self._draw(1, k, None)
        n_queries = answers[0].numel() - 1
        mask = torch.empty(n_queries, k, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().smore_negative_mask(neg.data_ptr(), k, answers[0].data_ptr(), answers[1].data_ptr(),
                                                      n_queries, mask.data_ptr(),
                                                      torch.cuda.current_stream(self.device).cuda_stream),
                       "smore_negative_mask")
        return neg, mask
