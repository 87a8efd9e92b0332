"""Evaluation of ranked answers: the part of the reference's test step that follows the scoring of
a query against every entity (smore/training/train_process.py:113-153).

    logits = gamma - dist(all_entities, query)          # the distance ops with be = 1, ne = N
    ranks = filtered_ranks(logits, easy_answers, hard_answers)
    logs  = ranking_metrics(ranks)                      # MRR, HITS1/3/10, HITS1max per query

`filtered_ranks` replaces argsort + scatter over the N logits by a count per answer
(smore_filtered_ranks in libsmore_b200.so); there is no CPU path.
"""
import torch

from . import _lib


def filtered_ranks(logits, easy_answers, hard_answers):
    """Ranks of the hard answers in the filtered setting.

    logits        float32 CUDA tensor [Q, N] (one row of scores over all candidates per query)
    easy_answers  Q iterables of candidate ids that are filtered out but not scored
    hard_answers  Q iterables of candidate ids to rank
    Returns a list of Q int64 CUDA tensors: the ranks of each query's hard answers in ascending
    order, the quantity `cur_ranking[masks]` of train_process.py:140-141.
    """
    if logits.dim() != 2 or logits.dtype != torch.float32 or not logits.is_cuda:
        raise TypeError("logits must be a 2-D float32 CUDA tensor")
    logits = logits.contiguous()
    Q, N = logits.shape
    if len(easy_answers) != Q or len(hard_answers) != Q:
        raise ValueError("one easy and one hard answer list per query")
    ptr, ids, hard_mask = [0], [], []
    for easy, hard in zip(easy_answers, hard_answers):
        easy, hard = list(easy), list(hard)
        ids.extend(easy)
        ids.extend(hard)
        hard_mask.extend([False] * len(easy) + [True] * len(hard))
        ptr.append(len(ids))
    n_answers = len(ids)
    if n_answers == 0:
        return [torch.empty(0, dtype=torch.int64, device=logits.device) for _ in range(Q)]
    if any((i < 0 or i >= N) for i in ids):
        raise ValueError("answer ids must lie in [0, %d)" % N)
    max_answers = max(b - a for a, b in zip(ptr[:-1], ptr[1:]))
    dev = logits.device
    d_ptr = torch.tensor(ptr, dtype=torch.int64, device=dev)
    d_ids = torch.tensor(ids, dtype=torch.int64, device=dev)
    ranks = torch.empty(n_answers, dtype=torch.int64, device=dev)
    L = _lib.lib()
    ws = torch.empty(L.smore_filtered_ranks_workspace_bytes(n_answers), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev), _lib.timed("filtered_ranks"):
        _lib.check(L.smore_filtered_ranks(logits.data_ptr(), Q, N, d_ptr.data_ptr(), d_ids.data_ptr(), n_answers,
                                          max_answers, ranks.data_ptr(), ws.data_ptr(), ws.numel(),
                                          torch.cuda.current_stream(dev).cuda_stream), "smore_filtered_ranks")
    mask = torch.tensor(hard_mask, dtype=torch.bool, device=dev)
    out = []
    for q in range(Q):
        r = ranks[ptr[q]:ptr[q + 1]][mask[ptr[q]:ptr[q + 1]]]
        out.append(torch.sort(r)[0])
    return out


def _answer_lists(easy_answers, hard_answers, n_candidates):
    ptr, ids, hard_mask = [0], [], []
    for easy, hard in zip(easy_answers, hard_answers):
        easy, hard = list(easy), list(hard)
        ids.extend(easy)
        ids.extend(hard)
        hard_mask.extend([False] * len(easy) + [True] * len(hard))
        ptr.append(len(ids))
    if any((i < 0 or i >= n_candidates) for i in ids):
        raise ValueError("answer ids must lie in [0, %d)" % n_candidates)
    return ptr, ids, hard_mask


_SCORE_IDS = {"box": _lib.BOX_BOTH_ID, "vec": _lib.DIST_IDS["l1"], "l1": _lib.DIST_IDS["l1"], "l2": _lib.DIST_IDS["l2"],
              "rotate": _lib.DIST_IDS["rotate"], "complex": _lib.DIST_IDS["complex"],
              "distmult": _lib.DIST_IDS["distmult"]}


def score_and_rank(geo, table, query, easy_answers, hard_answers, gamma=0.0, cen=0.0):
    """The evaluation step in one call: score Q queries against every row of `table` with the model's
    logit and return the filtered ranks of their hard answers, without materialising the [Q, N]
    logits (smore_score_filtered_ranks).

    geo      "box" (gamma - d_out - cen * d_in), "vec" / "l1" / "rotate" (gamma - d), "l2" (gamma - sqrt(d)),
             "complex" / "distmult" (the similarity)
    table    float32 CUDA [N, W] - the whole entity table (W = dim, or 2 * dim for rotate / complex rows)
    query    one or two float32 CUDA tensors [Q, dim] (or [Q, 1, dim]): center (and offset), re and im, ...
    Returns what filtered_ranks returns for the logits the distance ops would have produced."""
    if geo not in _SCORE_IDS:
        raise ValueError("geo must be one of %s" % sorted(_SCORE_IDS))
    parts = [q.reshape(q.shape[0], -1).contiguous() for q in query]
    Q, dim = parts[0].shape
    N = table.shape[0]
    if table.dtype != torch.float32 or not table.is_cuda or not table.is_contiguous():
        raise TypeError("table must be a contiguous float32 CUDA tensor")
    ptr, ids, hard_mask = _answer_lists(easy_answers, hard_answers, N)
    if len(ptr) != Q + 1:
        raise ValueError("one easy and one hard answer list per query")
    n_answers = len(ids)
    dev = table.device
    if n_answers == 0:
        return [torch.empty(0, dtype=torch.int64, device=dev) for _ in range(Q)]
    max_answers = max(b - a for a, b in zip(ptr[:-1], ptr[1:]))
    d_ptr = torch.tensor(ptr, dtype=torch.int64, device=dev)
    d_ids = torch.tensor(ids, dtype=torch.int64, device=dev)
    ranks = torch.empty(n_answers, dtype=torch.int64, device=dev)
    L = _lib.lib()
    ws = torch.empty(L.smore_score_filtered_ranks_workspace_bytes(Q, n_answers), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev), _lib.timed("score_filtered_ranks"):
        _lib.check(L.smore_score_filtered_ranks(
            _SCORE_IDS[geo], table.data_ptr(), N, parts[0].data_ptr(), parts[1].data_ptr() if len(parts) > 1 else None,
            Q, dim, float(gamma), float(cen), d_ptr.data_ptr(), d_ids.data_ptr(), n_answers, max_answers,
            ranks.data_ptr(), ws.data_ptr(), ws.numel(), torch.cuda.current_stream(dev).cuda_stream),
            "smore_score_filtered_ranks")
    mask = torch.tensor(hard_mask, dtype=torch.bool, device=dev)
    return [torch.sort(ranks[ptr[q]:ptr[q + 1]][mask[ptr[q]:ptr[q + 1]]])[0] for q in range(Q)]


def ranking_metrics(hard_ranks):
    """Per-query metrics of train_process.py:142-146 from the sorted filtered ranks of a query's hard
    answers: MRR, HITS1, HITS3, HITS10 (means over the answers) and HITS1max (best answer ranked 1)."""
    r = hard_ranks.to(torch.float32)
    if r.numel() == 0:
        return {"MRR": 0.0, "HITS1": 0.0, "HITS3": 0.0, "HITS10": 0.0, "HITS1max": 0.0}
    return {"MRR": torch.mean(1.0 / r).item(),
            "HITS1": torch.mean((r <= 1).float()).item(),
            "HITS3": torch.mean((r <= 3).float()).item(),
            "HITS10": torch.mean((r <= 10).float()).item(),
            "HITS1max": float(r[0].item() == 1)}
