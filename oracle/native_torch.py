"""Pure-torch restatement of the reference's CPU-capable path (TEST / BASELINE INFRASTRUCTURE ONLY).

Without its CUDA extension the reference scores candidates with the models' `native_cal_logit`
methods and merges / applies sparse gradients with torch index ops.  This module restates those
few expressions so that (a) they can be timed on host cores as the CPU baseline where the
reference tree is not mounted, and (b) end-to-end training steps of the CUDA path can be checked
against an independent implementation.  It is pinned by tests/test_oracle_golden.py against
vectors produced by the reference's own code.

Restated (paths relative to the reference project root):
    smore/models/vec.py:78-83          native_cal_logit (GQE, L1)
    smore/models/box.py:147-155        native_cal_logit (Query2box)
    smore/models/rotate.py:125-135     native_cal_logit (RotatE)
    smore/models/complex.py:169-187    native_cal_logit (ComplEx)
    smore/models/distmult.py:126-133   native_cal_logit (DistMult)
    smore/training/train_process.py:195-213   negative-sampling loss
    smore/common/embedding/embed_optimizer.py:39-48,155-163   merge of a step's row gradients
    smore/common/embedding/embed_optimizer.py:166-185,208-252,328-349   SGD / Adam / Adagrad rows
"""
import math

import torch
import torch.nn.functional as F

EPS = 1e-8  # smore/common/consts.py:20


def vec_logit(entity, query, gamma):
    """entity [B, K, D]; query (center [B, U, 1, D],)"""
    distance = entity.unsqueeze(1) - query[0]
    logit = gamma - torch.norm(distance, p=1, dim=-1)
    return torch.max(logit, dim=1)[0]


def box_logit(entity, query, gamma, cen):
    center, offset = query
    delta = (entity.unsqueeze(1) - center).abs()
    distance_out = F.relu(delta - offset)
    distance_in = torch.min(delta, offset)
    logit = gamma - torch.norm(distance_out, p=1, dim=-1) - cen * torch.norm(distance_in, p=1, dim=-1)
    return torch.max(logit, dim=1)[0]


def rotate_logit(entity, query, gamma):
    re, im = query
    e_re, e_im = torch.chunk(entity.unsqueeze(1), 2, dim=-1)
    distance = torch.stack([e_re - re, e_im - im], dim=0).norm(dim=0)
    logit = gamma - distance.sum(dim=-1)
    return torch.max(logit, dim=1)[0]


def complex_logit(entity, query):
    re, im = query
    e_re, e_im = torch.chunk(entity.unsqueeze(1), 2, dim=-1)
    logit = (e_re * re + e_im * im).sum(dim=-1)
    return torch.max(logit, dim=1)[0]


def distmult_logit(entity, query):
    logit = (entity.unsqueeze(1) * query[0]).sum(dim=-1)
    return torch.max(logit, dim=1)[0]


def sampling_loss(positive_logit, negative_logit, adversarial_temperature=None, subsampling_weight=None,
                  is_negative_mat=None, world_size=1):
    """train_process.py:195-213 (reg_coeff = 0)."""
    if is_negative_mat is not None:
        negative_logit = negative_logit * is_negative_mat
    if adversarial_temperature is not None:
        negative_score = (F.softmax(negative_logit * adversarial_temperature, dim=1).detach()
                          * F.logsigmoid(-negative_logit)).sum(dim=1)
    else:
        negative_score = F.logsigmoid(-negative_logit).mean(dim=1)
    positive_score = F.logsigmoid(positive_logit).squeeze(dim=1)
    if subsampling_weight is not None:
        pos = -(subsampling_weight * positive_score).sum() / subsampling_weight.sum()
        neg = -(subsampling_weight * negative_score).sum() / subsampling_weight.sum()
    else:
        pos = -torch.mean(positive_score)
        neg = -torch.mean(negative_score)
    return (pos + neg) / 2 / world_size


def merge_grads(idx_list, grad_list):
    """(sorted distinct ids, inverse map, summed gradients) of a step's lookups."""
    cat_idx = torch.cat(idx_list, dim=0)
    merged_indices, inverse = torch.unique(cat_idx, return_inverse=True)
    cat_grad = torch.cat(grad_list, dim=0)
    merged = torch.zeros(merged_indices.numel(), cat_grad.shape[1], dtype=cat_grad.dtype, device=cat_grad.device)
    merged.index_add_(0, inverse, cat_grad)
    return merged_indices, inverse, merged


def adam_rows(table, m, v, indices, grad, lr, step, squeeze, beta1=0.9, beta2=0.999):
    bias_correction1 = 1 - beta1 ** step
    bias_correction2 = 1 - beta2 ** step
    if squeeze:
        grad_sum_sq = torch.mean(grad * grad, dim=1, keepdim=True)
    avg_fo = m[indices]
    avg_sq = v[indices]
    bak_fo, bak_sq = avg_fo.clone(), avg_sq.clone()
    if squeeze:
        avg_sq.mul_(beta2).add_(grad_sum_sq * (1 - beta2))
    else:
        avg_sq.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
    avg_fo.mul_(beta1).add_(grad, alpha=1 - beta1)
    denom = (avg_sq.sqrt() / math.sqrt(bias_correction2)).add_(EPS)
    tmp = -lr / bias_correction1 * avg_fo / denom
    table.index_add_(0, indices, tmp)
    m.index_add_(0, indices, avg_fo - bak_fo)
    v.index_add_(0, indices, avg_sq - bak_sq)


def adagrad_rows(table, state, indices, grad, lr, squeeze):
    grad_sum = torch.mean(grad * grad, dim=1, keepdim=True) if squeeze else grad * grad
    square_avg = state[indices] + grad_sum
    avg = square_avg.sqrt().add_(EPS)
    table.index_add_(0, indices, -lr * grad / avg)
    state.index_add_(0, indices, grad_sum)


def sgd_rows(table, indices, grad, lr):
    table.index_add_(0, indices, -lr * grad)


def reference_filtered_ranks(negative_logit, easy_answer, hard_answer):
    """The ranking block of the reference's test step for one query, as torch ops on the CPU
    (smore/training/train_process.py:113-141): argsort of the [1, N] logits (descending), ranks by
    scatter, the answers' ranks sorted, minus their position in that list, plus one; only the hard
    answers' entries are kept.  `stable=True` fixes the order of tied logits (lower id first), which
    the reference leaves to the sort implementation.  Returns the float tensor `cur_ranking`."""
    negative_logit = negative_logit.reshape(1, -1).float().cpu()
    easy_answer, hard_answer = list(easy_answer), list(hard_answer)
    argsort = torch.argsort(negative_logit, dim=1, descending=True, stable=True)
    ranking = argsort.clone().to(torch.float)
    ranking = ranking.scatter_(1, argsort, torch.arange(negative_logit.shape[1]).to(torch.float).repeat(argsort.shape[0], 1))
    num_easy, num_hard = len(easy_answer), len(hard_answer)
    cur_ranking = ranking[0, easy_answer + hard_answer]
    cur_ranking, indices = torch.sort(cur_ranking)
    masks = indices >= num_easy
    answer_list = torch.arange(num_hard + num_easy).to(torch.float)
    cur_ranking = cur_ranking - answer_list + 1
    return cur_ranking[masks]


def reference_ranking_metrics(cur_ranking):
    """train_process.py:142-146."""
    return {"MRR": torch.mean(1. / cur_ranking).item(),
            "HITS1": torch.mean((cur_ranking <= 1).to(torch.float)).item(),
            "HITS3": torch.mean((cur_ranking <= 3).to(torch.float)).item(),
            "HITS10": torch.mean((cur_ranking <= 10).to(torch.float)).item(),
            "HITS1max": ((cur_ranking[0] == 1).to(torch.float)).item()}
