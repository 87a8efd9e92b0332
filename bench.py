"""Benchmark of the distance-op + sparse-row-update hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one training step of a multi-hop query-embedding model on one synthetic batch:
row lookups -> query embedding (torch, the unchanged caller side) -> candidate scoring with the
library's distance ops -> negative-sampling loss -> backward (query gradients + entity-row
gradients) -> per-step de-duplication of touched rows -> fused row-wise Adam; plus the dense
optimizer step of the small relation / intersection parameters.  The metric is queries per
second (B queries per GPU per step).

The default workload is the Freebase-scale Query2box configuration (B=1024 queries per GPU,
K=1024 negatives per query, dim 400, row-wise second moment, nine query structures in
rotation) with the entity table sized at 1/8 of 86,054,151 rows per GPU, so that per-GPU work
is the same at every N ("weak" scaling; at N=8 the table is the full 86M rows).  Inputs are
synthetic with the shapes and value distributions of that configuration; no dataset is read.

Prints one JSON line.  Its contract keys: metric, value (whole-job queries/s with the index tensors
resident on the device: the median of `--repeats` timed regions of exactly `--steps` steps), unit,
n_gpus, steps, warmup, ms_per_step, higher_is_better, scaling, vs_baseline, dtype, data, config,
e2e (the same metric with every step's index tensors copied from pinned host memory and the loss
read back), gpu_launches (this library's kernels per timed region), clocks, roofline (the kernel
with the largest share: algorithmic bytes / CUDA-event time against the measured copy bandwidth),
kernels (every library call of an eager pass over the same steps), cpu_baseline.  At one GPU the
other configurations (RotatE, shared-negative Query2box, GQE, DistMult on the tensor cores in both
precisions) run afterwards in the same process and are reported under `workloads`; at several GPUs
a parity check of the prefetching graph mode against the plain mode runs first (`parity_check`).
`--impl reference` instead times the reference's own CPU implementation of the path (its Python,
imported by oracle/ref_harness.py, else the torch restatement in oracle/native_torch.py) on the host
cores, on a bounded sample of the same workload.
"""
import argparse
import json
import math
import os
import sys
import threading
import time

if "reference" in sys.argv and os.environ.get("OMP_NUM_THREADS") == "1":
    # the launcher of multi-process runs pins every rank to one OpenMP thread; the reference arm is
    # one process (rank 0) that is meant to use all host cores
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

import torch
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FREEBASE_ENTITIES = 86054151
FREEBASE_RELATIONS = 14824

# query structures (smore/common/config.py:21-43), in the reference's nested-tuple notation
E1 = ("e", ("r",))
STRUCTURES = {
    "1p": E1,
    "2p": ("e", ("r", "r")),
    "3p": ("e", ("r", "r", "r")),
    "2i": (E1, E1),
    "3i": (E1, E1, E1),
    "ip": ((E1, E1), ("r",)),
    "pi": (("e", ("r", "r")), E1),
    "2u": (E1, E1, ("u",)),
    "up": ((E1, E1, ("u",)), ("r",)),
}


def structure_columns(qs):
    """Column kinds ('e', 'r', 'u') of the flattened query matrix, in embed order."""
    if all(isinstance(x, str) for x in qs[-1]) and all(x in ("r", "n") for x in qs[-1]):
        head = ["e"] if qs[0] == "e" else structure_columns(qs[0])
        return head + list(qs[-1])
    cols = []
    is_union = qs[-1][0] == "u"
    for branch in (qs[:-1] if is_union else qs):
        cols += structure_columns(branch)
    return cols + (["u"] if is_union else [])


WORKLOADS = {
    # name: geo, rows per GPU (None = FREEBASE/8), relations, dim, B, K, shared negatives, gamma, structures,
    #       adversarial temperature, lr, row-wise second moment
    "freebase_q2b": dict(geo="box", rows=None, relations=FREEBASE_RELATIONS, dim=400, B=1024, K=1024, shared=False,
                         gamma=2.0, cen=0.02, structures=["1p", "2p", "3p", "2i", "3i", "ip", "pi", "2u", "up"],
                         adv=0.5, lr=5e-5, squeeze=True),
    "rotate_wikikg": dict(geo="rotate", rows=2500604, relations=535, dim=500, B=1024, K=1024, shared=False,
                          gamma=24.0, cen=0.0, structures=["1p"], adv=1.0, lr=1e-4, squeeze=False, zipf_anchor=1.1),
    "q2b_fb15k": dict(geo="box", rows=14951, relations=1345, dim=400, B=1024, K=512, shared=True, gamma=12.0,
                      cen=0.02, structures=["1p", "2p", "3p", "2i"], adv=None, lr=1e-4, squeeze=False),
    # dot-product scoring against shared negatives: the op and its gradients are GEMMs (tensor cores)
    "distmult_wikikg": dict(geo="distmult", rows=2500604, relations=535, dim=1000, B=4096, K=8192, shared=True,
                            gamma=0.0, cen=0.0, structures=["1p"], adv=None, lr=1e-4, squeeze=False, init_std=0.05),
    "complex_wikikg": dict(geo="complex", rows=2500604, relations=535, dim=500, B=4096, K=8192, shared=True,
                           gamma=0.0, cen=0.0, structures=["1p"], adv=None, lr=1e-4, squeeze=False, init_std=0.05),
    "gqe_fb15k237": dict(geo="vec", rows=14505, relations=237, dim=64, B=512, K=128, shared=False, gamma=12.0,
                         cen=0.0, structures=["1p"], adv=None, lr=1e-4, squeeze=False),
}


# ------------------------------------------------------------------------------------------------
# synthetic index batches (what the online sampler hands to the training step)
# ------------------------------------------------------------------------------------------------

def _power_law_ids(gen, n, size, s, mult):
    """Ids in [0, n) whose popularity rank follows ~ rank^-s; rank -> id through a fixed bijection."""
    u = torch.rand(size, generator=gen, dtype=torch.float64)
    if abs(s - 1.0) < 1e-9:
        x = torch.exp(u * math.log(n))
    else:
        x = (1.0 + u * (float(n) ** (1.0 - s) - 1.0)) ** (1.0 / (1.0 - s))
    rank = x.floor().long().clamp_(1, n) - 1
    return (rank * mult + 12345) % n


def _coprime_multiplier(n):
    m = 2654435761 % n
    while m < 2 or math.gcd(m, n) != 1:
        m += 1
    return m


def make_batch(cfg, n_rows, structure, seed):
    """(positive [B], negative [B, K] or [1, K], queries [B, n_cols]) as int64 CPU tensors."""
    gen = torch.Generator().manual_seed(seed)
    B, K = cfg["B"], cfg["K"]
    cols = structure_columns(STRUCTURES[structure])
    mult_e, mult_r = _coprime_multiplier(n_rows), _coprime_multiplier(cfg["relations"])
    q = torch.empty(B, len(cols), dtype=torch.int64)
    for c, kind in enumerate(cols):
        if kind == "e":
            q[:, c] = _power_law_ids(gen, n_rows, (B,), cfg.get("zipf_anchor", 1.2), mult_e)
        elif kind == "r":
            q[:, c] = _power_law_ids(gen, cfg["relations"], (B,), 1.0, mult_r)
        else:
            q[:, c] = -1
    pos = torch.randint(0, n_rows, (B,), generator=gen)
    neg = torch.randint(0, n_rows, (1 if cfg["shared"] else B, K), generator=gen)
    return pos, neg, q


# ------------------------------------------------------------------------------------------------
# the caller side: query embedding in plain torch (smore/models/{box,vec,rotate}.py), scoring through
# the library's ops
# ------------------------------------------------------------------------------------------------

class Intersection(nn.Module):
    """CenterIntersection (box.py:55-70): attention over the branches."""

    def __init__(self, dim):
        super().__init__()
        self.dim = dim
        self.layers = nn.Parameter(torch.zeros(dim * 2 + 2, dim))
        nn.init.xavier_uniform_(self.layers[:dim * 2, :])

    def forward(self, embeddings):
        w1, w2, b1, b2 = torch.split(self.layers, [self.dim, self.dim, 1, 1], dim=0)
        act = F.relu(F.linear(embeddings, w1, b1.view(-1)))
        attention = F.softmax(F.linear(act, w2, b2.view(-1)), dim=0)
        return torch.sum(attention * embeddings, dim=0)


class OffsetIntersection(nn.Module):
    """BoxOffsetIntersection (box.py:38-53)."""

    def __init__(self, dim):
        super().__init__()
        self.dim = dim
        self.layers = nn.Parameter(torch.zeros(dim * 2 + 2, dim))
        nn.init.xavier_uniform_(self.layers[:dim * 2, :])

    def forward(self, embeddings):
        w1, w2, b1, b2 = torch.split(self.layers, [self.dim, self.dim, 1, 1], dim=0)
        act = F.relu(F.linear(embeddings, w1, b1.view(-1)))
        gate = torch.sigmoid(F.linear(torch.mean(act, dim=0), w2, b2.view(-1)))
        offset, _ = torch.min(embeddings, dim=0)
        return offset * gate


class QueryModel(nn.Module):
    """Entity table (sparse, updated by the library's optimizer) + dense relation parameters and
    intersection nets; embeds one batch of same-structure queries and scores candidates."""

    def __init__(self, cfg, n_rows, device, ops, embedding_mod, lazy=True, shard=None, barrier=None, world=1,
                 capturable=False, fused_paths=False):
        super().__init__()
        # relation projections of a path as one library op instead of per-hop torch ops; an anchor lookup
        # that starts a path is read from the table inside that op (never gathered)
        self.fused_paths = bool(fused_paths)
        self.cfg, self.geo, self.dim = cfg, cfg["geo"], cfg["dim"]
        self.gamma, self.cen = cfg["gamma"], cfg.get("cen", 0.0)
        self.ops = ops
        self.world = world
        two_part = self.geo in ("rotate", "complex")      # rows laid out [part0 | part1]
        width = self.dim * (2 if two_part else 1)
        self.embedding_range = (self.gamma + 2.0) / self.dim
        r = self.embedding_range
        self.entity_embedding = embedding_mod.SparseEmbedding(0, width)
        self.entity_embedding.num_rows = n_rows
        lazy_names = ("negative_entity", "positive_entity") if lazy else ()
        if lazy and self.fused_paths:
            lazy_names += ("anchor_entity",)
        if shard is None:
            table = torch.empty(n_rows, width, device=device)
            if cfg.get("init_std"):
                table.normal_(0.0, cfg["init_std"])
            else:
                table.uniform_(-r, r)
            self.entity_embedding.embedding = nn.Parameter(table, requires_grad=False)
        R = cfg["relations"]
        rel_width = self.dim * (2 if self.geo == "complex" else 1)
        rel = torch.empty(R, rel_width, device=device)
        rel = rel.normal_(0.0, cfg["init_std"]) if cfg.get("init_std") else rel.uniform_(-r, r)
        self.relation_embedding = nn.Parameter(rel)
        if self.geo == "box":
            self.offset_embedding = nn.Parameter(torch.empty(R, self.dim, device=device).uniform_(0, r))
            self.offset_net = OffsetIntersection(self.dim).to(device)
        self.center_net = Intersection(width).to(device)

        class _Args(object):
            optim_mode = ("aggr", "adam", "gpu", bool(cfg["squeeze"]), 0)
            share_optim_stats = False

        if shard is None:
            self.embed_opt = embedding_mod.AdamEmbedOptimizer(_Args(), self.entity_embedding, device.index,
                                                              lazy_names=lazy_names)
        else:
            # the table is a row shard per GPU: lookups and the update go through the sharded optimizer
            from smore_b200 import sharded
            # (every lookup of the step is made before the candidates are scored: the owners may plan early)
            self.embed_opt = sharded.ShardedAdamOptimizer(shard, lazy_names=lazy_names, barrier=barrier,
                                                          early_owner_plan=shard.remote is not None)
            self.entity_embedding.fwd_delegate = self.embed_opt.forward
        dense = [p for n, p in self.named_parameters() if p.requires_grad and "dummy" not in n]
        self.dense_opt = torch.optim.Adam(dense, lr=cfg["lr"], fused=True, capturable=capturable)

    # -- query embedding (kg_reasoning.py:217-250 with the per-model hooks) -----------------------
    def _retrieve(self, ids):
        e = self.entity_embedding(ids)
        if self.geo in ("rotate", "complex"):
            re, im = torch.chunk(e, 2, dim=1)
            return [re.unsqueeze(1), im.unsqueeze(1)]
        if self.geo == "box":
            # a fresh anchor is a box of zero size (box.py:138-139)
            return [e.unsqueeze(1), torch.zeros_like(e).unsqueeze(1)]
        return [e.unsqueeze(1)]

    def _embed_path(self, start, rel_ids):
        """All hops of a path at once (smore_b200.query_ops.embed_path).  `start` is the list of
        [B, 1, dim] parts of the state the path starts from, or the anchor ids' table-resident rows."""
        from smore_b200 import query_ops
        fresh = not isinstance(start, list)
        if self.geo == "box":
            c, o = query_ops.embed_path("add", start if fresh else start[0].squeeze(1), self.relation_embedding, rel_ids,
                                        start_offset=None if fresh else start[1].squeeze(1),
                                        off_table=self.offset_embedding)
            return [c.unsqueeze(1), o.unsqueeze(1)]
        if self.geo in ("rotate", "complex"):
            state = start if fresh else torch.cat([start[0], start[1]], dim=-1).squeeze(1)
            scale = math.pi / self.embedding_range if self.geo == "rotate" else 1.0
            re, im = query_ops.embed_path(self.geo, state, self.relation_embedding, rel_ids, phase_scale=scale)
            return [re.unsqueeze(1), im.unsqueeze(1)]
        geometry = "distmult" if self.geo == "distmult" else "add"
        out = query_ops.embed_path(geometry, start if fresh else start[0].squeeze(1), self.relation_embedding, rel_ids)
        return [out.unsqueeze(1)]

    def _project(self, emb, rel_ids):
        rel = self.relation_embedding[rel_ids].unsqueeze(1)
        if self.geo == "rotate":
            phase = rel / (self.embedding_range / math.pi)
            re_r, im_r = torch.cos(phase), torch.sin(phase)
            re, im = emb
            return [re * re_r - im * im_r, re * im_r + im * re_r]
        if self.geo == "box":
            return [emb[0] + rel, emb[1] + self.offset_embedding[rel_ids].unsqueeze(1)]
        if self.geo == "complex":      # complex.py:108-117: multiply by the relation as a complex number
            re_r, im_r = torch.chunk(rel, 2, dim=-1)
            re, im = emb
            return [re * re_r - im * im_r, re * im_r + im * re_r]
        if self.geo == "distmult":     # distmult.py:106-111
            return [emb[0] * rel]
        return [emb[0] + rel]

    def _intersect(self, branches):
        if self.geo == "box":
            centers = torch.stack([b[0] for b in branches])
            offsets = torch.stack([b[1] for b in branches])
            return [self.center_net(centers), self.offset_net(offsets)]
        if self.geo in ("rotate", "complex"):
            stacked = torch.stack([torch.cat(b, dim=-1) for b in branches])
            return list(torch.chunk(self.center_net(stacked), 2, dim=-1))
        return [self.center_net(torch.stack([b[0] for b in branches]))]

    def embed_query(self, queries, qs, col):
        if all(isinstance(x, str) for x in qs[-1]) and all(x in ("r", "n") for x in qs[-1]):
            fused = self.fused_paths and all(x == "r" for x in qs[-1])
            n_hops = len(qs[-1])
            if qs[0] == "e":
                if fused:
                    rows = self.entity_embedding(queries[:, col], "anchor_entity")   # table-resident when lazy
                    return self._embed_path(rows, queries[:, col + 1:col + 1 + n_hops]), col + 1 + n_hops
                emb = self._retrieve(queries[:, col])
                col += 1
            else:
                emb, col = self.embed_query(queries, qs[0], col)
            if fused and emb[0].shape[1] == 1:   # not after a union
                return self._embed_path(emb, queries[:, col:col + n_hops]), col + n_hops
            for _ in qs[-1]:
                emb = self._project(emb, queries[:, col])
                col += 1
            return emb, col
        is_union = qs[-1][0] == "u"
        branches = []
        for b in (qs[:-1] if is_union else qs):
            emb, col = self.embed_query(queries, b, col)
            branches.append(emb)
        if is_union:
            n = len(branches[0])
            return [torch.cat([b[i] for b in branches], dim=1) for i in range(n)], col + 1
        return self._intersect(branches), col

    def cal_logit(self, entity, query):
        ops = self.ops
        if self.geo == "box":
            d1 = ops.box_dist_out(entity, query[0], query[1])
            d2 = ops.box_dist_in(entity, query[0], query[1])
            logit = self.gamma - d1 - self.cen * d2
        elif self.geo == "rotate":
            logit = self.gamma - ops.rotate_dist(entity, query[0], query[1])
        elif self.geo == "complex":
            logit = ops.complex_sim(entity, query[0], query[1])
        elif self.geo == "distmult":
            logit = ops.distmult_sim(entity, query[0])
        else:
            logit = self.gamma - ops.l1_dist(entity, query[0])
        return torch.max(logit, dim=1)[0]

    def forward(self, pos, neg, queries, structure):
        """kg_reasoning.py:270-364 for one structure: (positive_logit [B,1], negative_logit [B,K])."""
        B = queries.shape[0]
        pos_rows = self.entity_embedding(pos, "positive_entity")
        neg_rows = self.entity_embedding(neg.view(-1), "negative_entity")
        emb, col = self.embed_query(queries, STRUCTURES[structure], 0)
        assert col == queries.shape[1]
        query = [e.unsqueeze(-2) for e in emb]
        pos_logit = self.cal_logit(pos_rows.unsqueeze(1), query)
        neg_logit = self.cal_logit(neg_rows.view(neg.shape[0], neg.shape[1], -1), query)
        return pos_logit, neg_logit


def sampling_loss(pos_logit, neg_logit, adv, world_size=1):
    """train_process.py:195-213 with uniform query weights and no regulariser."""
    if adv is not None:
        neg_score = (F.softmax(neg_logit * adv, dim=1).detach() * F.logsigmoid(-neg_logit)).sum(dim=1)
    else:
        neg_score = F.logsigmoid(-neg_logit).mean(dim=1)
    pos_score = F.logsigmoid(pos_logit).squeeze(dim=1)
    return (-pos_score.mean() - neg_score.mean()) / 2 / world_size


def first_lookup_group(pos, neg, queries, remote=False):
    """The id tensors a step looks up before it first needs rows: positives, negatives, first anchors
    (without the negatives when their owners score them: those rows are never fetched)."""
    return [pos, queries[:, 0]] if remote else [pos, neg.view(-1), queries[:, 0]]


def train_step(model, pos, neg, queries, structure, reduce_dense=None, upcoming=None):
    """train_process.py:172-227 on device-resident index tensors.  `reduce_dense(list of gradients)` sums the
    dense parameter's gradient over the ranks (train_process.py:221-225) when there are several.
    `upcoming` = (pos, neg, queries, event or None) of the NEXT step, whose rows a sharded table
    starts pulling now (the role of the reference's asynchronous embedding read, embedding.py:98-121)."""
    model.dense_opt.zero_grad(set_to_none=True)
    model.embed_opt.zero_grad()
    if getattr(model, "fused_update", False):
        # rows touched by a single position of the step are updated inside the backward kernel
        model.embed_opt.announce_lr(model.cfg["lr"])
    if upcoming is not None:
        model.embed_opt.prefetch(first_lookup_group(*upcoming[:3], remote=getattr(model, "remote_scoring", False)),
                                 after=upcoming[3])
    pos_logit, neg_logit = model(pos, neg, queries, structure)
    loss = sampling_loss(pos_logit, neg_logit, model.cfg["adv"], model.world)
    loss.backward()
    if reduce_dense is not None:
        # the all-reduce of the dense gradients also orders the ranks after their backward passes:
        # the sharded update needs no barrier of its own before it reads the ranks' gradient rows
        reduce_dense([p.grad for p in model.parameters() if p.requires_grad and p.grad is not None])
        model.embed_opt.apply_grad(model.cfg["lr"], ranks_ordered=True)
    else:
        model.embed_opt.apply_grad(model.cfg["lr"])
    model.dense_opt.step()
    return loss


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------

class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU every 100 ms through NVML (read-only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.stop_flag = index, threading.Event()
        self.sm, self.reasons, self.sm_max, self.ok = [], set(), None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        while self.ok and not self.stop_flag.is_set():
            try:
                self.sm.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self.stop_flag.wait(0.1)

    def summary(self):
        self.stop_flag.set()
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons)}
        s = sorted(self.sm)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------------------
# The reference arm: the reference's own CPU implementation of the path on the host cores
# ------------------------------------------------------------------------------------------------

def cpu_reference_steps(cfg, steps, warmup, sample_queries=64, table_rows=1000000):
    """Times whole training steps of `sample_queries` queries (full K and dim, the workload's query
    structures in rotation) on the host cores.  Returns a dict with value (queries/s), ms_per_step,
    cores, kind and a description of the sample.

    kind "reference": the reference's own Python - its model class with native_cal_logit, its
    train_step_mp and its AdamEmbedOptimizer - imported from a reference checkout or from the copy
    the oracle build places beside its compiled sources (oracle/ref_harness.py), for the geometries
    whose model that harness builds.  kind "port": the torch restatement of the same expressions
    (oracle/native_torch.py) where the reference package is not available or for DistMult / ComplEx
    (whose torch-native scoring needs a [B, 1, K, dim] temporary per step: 134 GB at this size)."""
    torch.set_num_threads(os.cpu_count() or 1)
    from oracle import ref_harness as rh
    geo = cfg["geo"]
    if rh.locate() is not None and geo in ("box", "rotate", "vec"):
        return _cpu_reference_python(rh, cfg, steps, warmup, sample_queries, table_rows)
    return _cpu_reference_port(cfg, steps, warmup, sample_queries, table_rows)


def _cpu_reference_python(rh, cfg, steps, warmup, sample_queries, table_rows):
    rh.install()
    rh.ensure_group()
    from smore.training.train_process import train_step_mp
    geo, D, K = cfg["geo"], cfg["dim"], cfg["K"]
    n_rows = min(table_rows, cfg["rows"] or table_rows)
    Bs = min(sample_queries, cfg["B"])
    small = dict(cfg, B=Bs)
    rargs = rh.train_args(adv=cfg["adv"], optim_mode="(aggr,adam,gpu,%s,0)" % bool(cfg["squeeze"]))
    model = rh.build_model(geo, n_rows, cfg["relations"], D, cfg["gamma"], Bs, "native", cen=cfg.get("cen", 0.02))
    opts = rh.reference_embedding_optimizers(model, rargs, -1)
    dense = rh.dense_optimizer(model, cfg["lr"])
    structures = cfg["structures"]
    batches = []
    for i in range(warmup + steps):
        s = structures[i % len(structures)]
        pos, neg, q = make_batch(small, n_rows, s, seed=77 + i)
        batches.append((s, pos, neg, q))
    it = rh.batch_iterator(batches)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        train_step_mp(model, [dense], opts, it, rargs, i, cfg["lr"], "cpu", 1)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    sample = ("the reference's train_step_mp (native_cal_logit, its AdamEmbedOptimizer, dense Adam) on %d of %d "
              "queries per step, K=%d, dim=%d, structures %s, host table %d rows, %d timed steps"
              % (Bs, cfg["B"], K, D, "/".join(structures), n_rows, len(times)))
    return {"value": Bs / (ms / 1e3), "ms_per_step": ms, "cores": torch.get_num_threads(), "kind": "reference",
            "sample": sample}


def _cpu_reference_port(cfg, steps, warmup, sample_queries, table_rows):
    """fwd + bwd + touched-row merge + row-wise Adam through the torch restatement, random query operands."""
    from oracle import native_torch as nt
    geo, D, K = cfg["geo"], cfg["dim"], cfg["K"]
    width = D * (2 if geo in ("rotate", "complex") else 1)
    n_rows = min(table_rows, cfg["rows"] or table_rows)
    g = torch.Generator().manual_seed(0)
    r = (cfg["gamma"] + 2.0) / D
    table = (torch.rand(n_rows, width, generator=g) * 2 - 1) * r
    m = torch.zeros_like(table)
    v = torch.zeros(n_rows, 1) if cfg["squeeze"] else torch.zeros_like(table)
    Bs = min(sample_queries, cfg["B"])
    times = []
    for it in range(warmup + steps):
        pos = torch.randint(0, n_rows, (Bs,), generator=g)
        neg = torch.randint(0, n_rows, (1 if cfg["shared"] else Bs, K), generator=g)
        qparts = [((torch.rand(Bs, 1, 1, D, generator=g) * 2 - 1) * r).requires_grad_() for _ in range(2)]
        t0 = time.perf_counter()
        pos_rows = table[pos].requires_grad_()
        neg_rows = table[neg.view(-1)].requires_grad_()
        ent_pos, ent_neg = pos_rows.unsqueeze(1), neg_rows.view(neg.shape[0], K, width)
        if geo == "box":
            q = (qparts[0], qparts[1].abs())
            pl, nl = nt.box_logit(ent_pos, q, cfg["gamma"], cfg["cen"]), nt.box_logit(ent_neg, q, cfg["gamma"], cfg["cen"])
        elif geo == "rotate":
            q = (qparts[0], qparts[1])
            pl, nl = nt.rotate_logit(ent_pos, q, cfg["gamma"]), nt.rotate_logit(ent_neg, q, cfg["gamma"])
        elif geo == "complex":
            # shared candidates: the reference's torch.mm branch (complex.py:176-186)
            q = (qparts[0], qparts[1])
            pl = nt.complex_logit(ent_pos, q)
            e_re, e_im = torch.chunk(ent_neg[0], 2, dim=-1)
            nl = torch.mm(q[0].view(Bs, D), e_re.t()) + torch.mm(q[1].view(Bs, D), e_im.t())
        elif geo == "distmult":
            q = (qparts[0],)
            pl = nt.distmult_logit(ent_pos, q)
            nl = torch.mm(q[0].view(Bs, D), ent_neg[0].t())
        else:
            q = (qparts[0],)
            pl, nl = nt.vec_logit(ent_pos, q, cfg["gamma"]), nt.vec_logit(ent_neg, q, cfg["gamma"])
        loss = nt.sampling_loss(pl, nl, cfg["adv"])
        loss.backward()
        idx, inv, merged = nt.merge_grads([pos, neg.view(-1)], [pos_rows.grad, neg_rows.grad])
        nt.adam_rows(table, m, v, idx, merged, cfg["lr"], it + 1, cfg["squeeze"])
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    sample = ("torch restatement of the reference's native path (scoring, loss, merge, Adam rows; random query "
              "operands) on %d of %d queries per step, K=%d, dim=%d, host table %d rows, %d timed steps"
              % (Bs, cfg["B"], K, D, n_rows, len(times)))
    return {"value": Bs / (ms / 1e3), "ms_per_step": ms, "cores": torch.get_num_threads(), "kind": "port",
            "sample": sample}


# ------------------------------------------------------------------------------------------------
# the GPU arm
# ------------------------------------------------------------------------------------------------

# DRAM bytes per launch measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum, a one-pass
# capture) on the Query2box workload.  Forward, and backward with the update folded in: captured at
# the full benchmark size (10.76M-row table, 1p structure; the kernels process B*K rows per launch).
# Backward without the folded-in update: a 2M-row capture scaled by the rows processed.  The update
# kernel moves 8070 bytes per distinct row it updates.  Other workloads: None.
NCU_TRAFFIC_BYTES = {"rows_forward": 1.758e9, "rows_backward": 4.094e9, "rows_backward_fused": 6.934e9}
NCU_UPDATE_BYTES_PER_ROW = 8070.0

# fp32 ALU instructions per (pair, dim) term evaluation in the inner loop of the shared-candidate
# kernels, counted in their source (csrc/dist_terms.cuh): box both = |e-c|, -o, max, +acc, min, |.|+acc
ALU_OPS_PER_TERM = {"box": {"fwd": 6, "bwd": 14}, "vec": {"fwd": 2, "bwd": 5}}


def ncu_traffic(workload, kernel, n_unique_mean, fused=False):
    if workload != "freebase_q2b":
        return None
    if kernel in ("sparse_update_rows", "shard_reduce_update"):
        return None if fused else round(NCU_UPDATE_BYTES_PER_ROW * n_unique_mean)
    if kernel in ("owner_forward", "owner_backward"):
        # the same two kernels in their ragged form, over about as many pairs: the single-GPU captures
        return NCU_TRAFFIC_BYTES["rows_forward" if kernel == "owner_forward" else "rows_backward_fused"]
    return NCU_TRAFFIC_BYTES.get(kernel + "_fused" if fused and kernel == "rows_backward" else kernel)


def algorithmic_bytes(cfg, n_unique_mean, n_single_mean=0.0):
    """Bytes each kernel has to move per launch (per union branch for the two distance kernels).
    n_single_mean: rows of a step that the backward kernel updates itself (one contributing position:
    it reads the row and its first moment and writes both back, 16 W bytes, instead of reading the row
    and writing the gradient, 8 W); the update kernel then handles the remaining distinct rows only."""
    B, K, D = cfg["B"], cfg["K"], cfg["dim"]
    W = D * (2 if cfg["geo"] in ("rotate", "complex") else 1)
    nq = 1 if cfg["geo"] == "vec" else 2
    nout = 2 if cfg["geo"] == "box" else 1
    pairs = B * K
    fwd = pairs * (4 * W + 8 + 4 * nout) + B * D * 4 * nq
    bwd = pairs * (8 * W + 8 + 4 + 4 + 4 * nout) + 2 * B * D * 4 * nq + n_single_mean * (8 * W + 8)
    v_bytes = 8 if cfg["squeeze"] else 8 * W
    upd = (n_unique_mean - n_single_mean) * (4 * W + 8 * W + 8 * W + v_bytes + 8) + n_single_mean * 8
    # sharded run: the owner-side kernel moves the same bytes as the update (the gradient read is a
    # peer read); the fetch copies every distinct row once (read + write)
    out = {"sparse_update_rows": upd, "shard_reduce_update": upd, "fetch_rows": n_unique_mean * 8 * W}
    if not cfg["shared"]:
        # with shared candidates the distance kernels are bound by fp32 ALU throughput, not by HBM
        out.update({"rows_forward": fwd, "rows_backward": bwd})
        # owner-side scoring of a sharded table: with uniform candidates every owner receives about as
        # many pairs as a rank sends, and runs the same two kernels over them
        out.update({"owner_forward": fwd, "owner_backward": bwd})
    return out


def algorithmic_flops(cfg):
    """Useful floating-point operations per launch of the shared-candidate GEMM kernels."""
    B, K, D = cfg["B"], cfg["K"], cfg["dim"]
    W = D * (2 if cfg["geo"] in ("rotate", "complex") else 1)
    return {"dot_forward": 2.0 * B * K * W, "dot_backward": 4.0 * B * K * W}


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measure_fma_rate(device):
    """fp32 fused multiply-adds per second of this GPU, measured with the library's probe kernel
    (every thread runs eight independent chains of dependent FMAs; grid of 8 blocks per SM), best of
    three launches timed with CUDA events."""
    import ctypes
    from smore_b200 import _lib
    L = _lib.lib()
    out = torch.zeros(1, device=device)
    count = ctypes.c_double(0.0)
    st = torch.cuda.current_stream(device).cuda_stream
    best = None
    for _ in range(4):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _lib.check(L.smore_alu_probe(out.data_ptr(), 20000, ctypes.byref(count), st), "smore_alu_probe")
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        best = ms if best is None else min(best, ms)
    return count.value / (best * 1e-3)


class StepRunner(object):
    """One workload on this rank's GPU: model, optimizer, pre-generated batches, and the ways of
    running steps (eager, replayed CUDA graphs, with host batches)."""

    def __init__(self, cfg, rows_per_gpu, device, world=1, rank=0, graphs=True, prefetch=True, lazy=True,
                 fused_paths=True, pool=18, resettable=False, fused_update=True, remote=True):
        from smore_b200 import _lib, embedding, ext_ops
        import torch.distributed as dist
        self.cfg, self.device, self.world, self.rank = cfg, device, world, rank
        self.rows_per_gpu = rows_per_gpu
        self.n_rows = n_rows = rows_per_gpu * world     # weak scaling: the table grows with the number of GPUs
        self.L = _lib.lib()
        torch.manual_seed(1234)           # dense parameters start identical on every rank
        self.reduce_dense = None
        self.shard = None
        self.remote = False
        self.prefetching = world > 1 and prefetch
        self.use_graphs = world == 1 and graphs
        self.chained_graphs = world > 1 and self.prefetching and graphs
        capturable = self.use_graphs or self.chained_graphs
        if world > 1:
            # table + Adam state row-sharded over the ranks; rows and row gradients move over NVLink
            from smore_b200 import sharded
            B, K = cfg["B"], cfg["K"]
            width = cfg["dim"] * (2 if cfg["geo"] in ("rotate", "complex") else 1)
            # owner-side scoring: the negatives' rows stay with their owners (one candidate list per
            # query, Adam with the row-wise second moment, rows the ragged kernels take)
            self.remote = bool(remote) and not cfg["shared"] and cfg["squeeze"] and cfg["dim"] > 256 and width * 4 <= 4096
            spec = None
            if self.remote:
                # union structures score every branch as a query of its own: twice the pairs
                spec = sharded.RemoteSpec(pairs=2 * B * K, queries=2 * B, dim=cfg["dim"])
                caps = (2 * B, B, B)
            else:
                caps = ((K if cfg["shared"] else B * K) + 2 * B, B, B)
            self.shard = sharded.ShardGroup.from_process_group(n_rows, width, caps, squeeze=cfg["squeeze"], device=device,
                                                               remote=spec)
            self._init_range = (cfg["gamma"] + 2.0) / cfg["dim"]
            self.shard.init_uniform(-self._init_range, self._init_range, seed=1234)
            self.model = QueryModel(cfg, n_rows, device, ext_ops, embedding, lazy=True, shard=self.shard, world=world,
                                    capturable=capturable, fused_paths=fused_paths)

            def reduce_dense(grads):
                # one all-reduce over all dense gradients instead of one per parameter
                flat = torch.cat([g.reshape(-1) for g in grads])
                dist.all_reduce(flat)
                torch._foreach_copy_(grads, [f.view_as(g) for f, g in zip(flat.split([g.numel() for g in grads]), grads)])
            self.reduce_dense = reduce_dense
        else:
            self.model = QueryModel(cfg, n_rows, device, ext_ops, embedding, lazy=lazy, capturable=capturable,
                                    fused_paths=fused_paths)
        model = self.model
        model.remote_scoring = world > 1 and self.remote
        # (the owners of remotely scored rows update them inside the backward pass: the rate must be announced)
        model.fused_update = (bool(fused_update) and world == 1 and lazy) or model.remote_scoring
        # (a copy of the initial state, table included at one GPU: only for runs that start over)
        self._initial = {k: v.detach().clone() for k, v in model.state_dict().items()} if resettable else None
        if capturable:
            model.embed_opt.use_device_step()      # the Adam step counter must advance inside replayed graphs
        model.train()
        self.structures = structures = cfg["structures"]
        self.pool = pool = max(len(structures), pool)
        self.host_batches = []
        for i in range(pool):
            s = structures[i % len(structures)]
            pos, neg, q = make_batch(cfg, n_rows, s, seed=1000 * rank + i)
            self.host_batches.append((s, pos.pin_memory(), neg.pin_memory(), q.pin_memory()))
        self.dev_batches = [(s, p.to(device), n.to(device), q.to(device)) for s, p, n, q in self.host_batches]
        self.h2d_bytes = sum(p.numel() + n.numel() + q.numel() for _, p, n, q in self.host_batches) * 8 / pool
        # untimed set-up: one eager step of every query structure (allocator blocks, optimizer state)
        for i in range(len(structures)):
            self.eager_step(*self.dev_batches[i])
        self.sync_all()
        self.graphs, self.launches_per_step = {}, {}
        self.static, self.chain = [], {}
        if self.use_graphs:
            self._capture_single()
        if self.chained_graphs:
            self._capture_chained()
        self.copy_stream = torch.cuda.Stream(device)
        from smore_b200.feed import BatchFeeder
        self.feeder = BatchFeeder(device, depth=2)

    # ---- plumbing -----------------------------------------------------------------------------------
    def sync_all(self):
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()

    def eager_step(self, s, p, n, q, upcoming=None):
        return train_step(self.model, p, n, q, s, self.reduce_dense, upcoming if self.prefetching else None)

    def _capture_single(self):
        """One CUDA graph per query structure: the whole step (lookups, query embedding, scoring, loss,
        backward, de-duplication, row-wise Adam, dense Adam) is captured once and replayed on new index
        tensors copied into its static input buffers.  Python and launch latency leave the step."""
        L = self.L
        for s in self.structures:
            ex = next(b for b in self.dev_batches if b[0] == s)
            static = [t.clone() for t in ex[1:]]
            before = L.smore_kernel_launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                loss = train_step(self.model, static[0], static[1], static[2], s)
            self.launches_per_step[s] = L.smore_kernel_launch_count() - before
            self.graphs[s] = (g, static, loss)
        self.sync_all()

    def _load_static(self, par, batch):
        pos, neg, q = self.static[par]
        pos.copy_(batch[1], non_blocking=True)
        neg.copy_(batch[2], non_blocking=True)
        q[:, :batch[3].shape[1]].copy_(batch[3], non_blocking=True)

    def start_chain(self, i, first_batch):
        """Make step i replayable: its index tensors in static buffer i % 2, their rows pulled by the
        prefetch branch of one eager step (on batch i - 1) on the other arena."""
        par = i % 2
        self._load_static(par, first_batch)
        self.model.embed_opt.reset_prefetch(next_parity=par ^ 1)
        prev = self.dev_batches[(i - 1) % self.pool]
        train_step(self.model, prev[1], prev[2], prev[3], prev[0], self.reduce_dense, self.static[par] + (None,))

    def _capture_chained(self):
        """Several GPUs: a step's graph also holds the side-stream branch that pulls the NEXT step's rows
        (forked at the start of the step, joined at its end), and steps alternate between two arenas of
        peer-visible id lists / gradient rows.  So there is one graph per (structure, arena); the index
        tensors of step i live in static buffer i % 2 and those of step i + 1 are copied into the other
        buffer before the graph of step i is launched."""
        L, device = self.L, self.device
        max_cols = max(b[3].shape[1] for b in self.host_batches)
        for par in range(2):
            _, p0, n0, q0 = self.dev_batches[0]
            self.static.append((torch.zeros_like(p0), torch.zeros_like(n0),
                                torch.zeros(q0.shape[0], max_cols, dtype=q0.dtype, device=device)))
        n_cols = {b[0]: b[3].shape[1] for b in self.host_batches}
        self.start_chain(0, self.dev_batches[0])
        pool_handle = torch.cuda.graph_pool_handle()
        for s in self.structures:
            for par in range(2):            # captures alternate between the arenas like the steps do
                pos, neg, q = self.static[par]
                before = L.smore_kernel_launch_count()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=pool_handle):
                    loss = train_step(self.model, pos, neg, q[:, :n_cols[s]], s, self.reduce_dense,
                                      self.static[par ^ 1] + (None,))
                self.launches_per_step[s] = L.smore_kernel_launch_count() - before
                self.graphs[(s, par)] = (g, loss)
        self.sync_all()
        self.chain["next"] = 0                   # static buffer 0 holds batch 0 and its rows are staged

    def step(self, s, p, n, q, upcoming=None):
        if not self.use_graphs:
            return self.eager_step(s, p, n, q, upcoming)
        g, static_in, loss = self.graphs[s]
        static_in[0].copy_(p, non_blocking=True)
        static_in[1].copy_(n, non_blocking=True)
        static_in[2].copy_(q, non_blocking=True)
        g.replay()
        return loss

    def _replay_chained(self, i, this_structure, next_batch):
        par = i % 2
        self._load_static(par ^ 1, next_batch)
        g, loss = self.graphs[(this_structure, par)]
        g.replay()
        self.chain["next"] = i + 1
        return loss

    # ---- ways of running steps ------------------------------------------------------------------------
    def run_resident(self, k0, k):
        """Steps k0 .. k0+k-1 on the device-resident batches (batch i % pool)."""
        pool, dev_batches = self.pool, self.dev_batches
        if self.chained_graphs:
            if self.chain.get("next") != k0:
                self.start_chain(k0, dev_batches[k0 % pool])
            for i in range(k0, k0 + k):
                self._replay_chained(i, dev_batches[i % pool][0], dev_batches[(i + 1) % pool])
            return
        for i in range(k0, k0 + k):
            self.step(*dev_batches[i % pool], upcoming=dev_batches[(i + 1) % pool][1:] + (None,))

    def launches_in(self, k0, k, counted_eagerly):
        if self.use_graphs or self.chained_graphs:
            return sum(self.launches_per_step[self.dev_batches[i % self.pool][0]] for i in range(k0, k0 + k))
        return counted_eagerly

    def _upload(self, i):
        """Start the host -> device copy of batch i's index tensors (pinned memory) on the copy stream;
        the previous step's compute overlaps it, as the sampler's prefetch thread would."""
        s, p, n, q = self.host_batches[i % self.pool]
        with torch.cuda.stream(self.copy_stream):
            dev = [t.to(self.device, non_blocking=True) for t in (p, n, q)]
            done = torch.cuda.Event()
            done.record(self.copy_stream)
        return s, dev, done

    def prepare_e2e(self, k0):
        """Untimed: with chained graphs, stage step k0 (its indices come from the host like all others)."""
        if self.chained_graphs:
            s, dev, done = self._upload(k0)
            torch.cuda.current_stream(self.device).wait_event(done)
            self.start_chain(k0, (s,) + tuple(dev))

    def run_e2e(self, k0, k):
        """The same steps fed from pinned host memory, the loss read back by the host every step."""
        last = 0.0
        pool, host_batches = self.pool, self.host_batches
        main = torch.cuda.current_stream(self.device)
        if self.chained_graphs:
            # the indices of step i + 1 are uploaded while step i - 1 runs and copied into the free
            # static buffer just before step i is launched
            ahead = [self._upload(k0 + 1), self._upload(k0 + 2)]
            for i in range(k0, k0 + k):
                s_next, dev, done = ahead.pop(0)
                ahead.append(self._upload(i + 3))
                main.wait_event(done)
                for t in dev:
                    t.record_stream(main)
                last = self._replay_chained(i, host_batches[i % pool][0], (s_next,) + tuple(dev)).item()
            return last
        # host batches go through the library's BatchFeeder (pinned staging, copy stream): batch i + 1 is
        # on its way when step i is launched, batch i + 2 is staged while step i runs on the GPU - the
        # role of the sampler's prefetch thread
        feeder = self.feeder
        for j in range(k0, min(k0 + 2, k0 + k)):
            feeder.submit(host_batches[j % pool][0], *host_batches[j % pool][1:])
        for i in range(k0, k0 + k):
            batch = feeder.get()
            upcoming = None
            if self.prefetching and len(feeder):
                nxt = feeder.peek()
                upcoming = tuple(nxt.tensors) + (nxt.event,)
            loss = self.step(batch.tag, *batch.tensors, upcoming=upcoming)
            if i + 2 < k0 + k:
                feeder.submit(host_batches[(i + 2) % pool][0], *host_batches[(i + 2) % pool][1:])
            last = loss.item()        # the step's loss is read back by the host every step
        return last

    def eager_timed_pass(self, k0, k):
        """The same k steps once more, eagerly, with CUDA events around each library call (kernels inside
        a replayed graph cannot be bracketed by events; the kernels are the same).  Returns (ms for the
        k steps, {kernel: [ms]}, notes)."""
        from smore_b200 import _lib
        if self.chained_graphs:
            self.model.embed_opt.reset_prefetch()
        if self.use_graphs or self.chained_graphs:
            # graph capture emptied the allocator's cache: give eager mode its blocks back first
            for i in range(len(self.structures)):
                self.eager_step(*self.dev_batches[i])
            self.sync_all()
        timer = _lib.KernelTimer()
        _lib.set_timer(timer)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(k0, k0 + k):
            self.eager_step(*self.dev_batches[i % self.pool], upcoming=self.dev_batches[(i + 1) % self.pool][1:] + (None,))
        b.record()
        self.sync_all()
        _lib.set_timer(None)
        self.chain["next"] = None
        return a.elapsed_time(b), timer.elapsed_ms(), timer.notes

    # ---- state (parity checks) ---------------------------------------------------------------------------
    def reset_state(self):
        """Back to the state right after construction: table, optimizer state, dense parameters, step
        counters; nothing prepared for coming steps."""
        model = self.model
        if self._initial is None:
            raise RuntimeError("StepRunner(resettable=True) is needed to start over")
        with torch.no_grad():
            model.load_state_dict(self._initial)
            if self.shard is not None:
                self.shard.init_uniform(-self._init_range, self._init_range, seed=1234)
                self.shard.m.zero_()
                self.shard.v.zero_()
                self.shard.dirty.zero_()
            else:
                for name in model.embed_opt.state_names:
                    model.embed_opt.state(name).zero_()
            for st in model.dense_opt.state.values():
                for t in st.values():
                    if torch.is_tensor(t):
                        t.zero_()
        opt = model.embed_opt
        opt.step = 0
        if getattr(opt, "_step_dev", None) is not None:
            opt._step_dev.zero_()
        if hasattr(opt, "reset_prefetch"):
            opt.reset_prefetch()
        self.chain["next"] = None
        self.sync_all()

    def state_tensors(self):
        model = self.model
        out = {}
        if self.shard is not None:
            n = self.shard.local_rows
            out.update(table=self.shard.table[:n], m=self.shard.m[:n], v=self.shard.v[:n])
        else:
            out["table"] = model.entity_embedding.embedding.data
            for name in model.embed_opt.state_names:
                out[name] = model.embed_opt.state(name)
        for name, p in model.named_parameters():
            if p.requires_grad and "dummy" not in name:
                out["dense/" + name] = p.data
        return out

    def close(self):
        """Drop graphs, model and table so that the next workload finds the memory free."""
        import gc
        torch.cuda.synchronize()
        self.graphs, self.static = {}, []
        self.model = self.shard = self.feeder = None
        self.dev_batches = self.host_batches = []
        self._initial = None
        gc.collect()
        torch.cuda.empty_cache()


def timed_steps(runner, k0, k, e2e=False):
    """ms for steps k0..k0+k-1, bracketed by barrier + synchronize on both sides, CUDA events on the
    launching stream; with e2e the steps are fed from host memory and the loss is read back."""
    if e2e:
        runner.prepare_e2e(k0)
    runner.sync_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    t0 = time.perf_counter()
    last = runner.run_e2e(k0, k) if e2e else runner.run_resident(k0, k)
    host = time.perf_counter() - t0
    b.record()
    runner.sync_all()
    return a.elapsed_time(b), host, last


def kernel_table(cfg, workload, kernel_ms, notes, peak, peak_kind, fma_rate=None):
    """Per-kernel averages of the eager pass with the roofline of the kernel that took longest."""
    nus = [int(t.item()) for t in notes.get("n_unique", []) + notes.get("n_unique_owner", [])]
    n_unique_mean = sum(nus) / len(nus) if nus else cfg["B"] * cfg["K"]
    singles = [int(t.item()) for t in notes.get("n_single", [])]
    n_single_mean = sum(singles) / max(1, len(nus)) if singles else 0.0
    alg = algorithmic_bytes(cfg, n_unique_mean=n_unique_mean, n_single_mean=n_single_mean)
    flops = algorithmic_flops(cfg)
    if "owner_backward" in kernel_ms:
        # owner-side scoring: the fetch and the last update only see the few rows of the ordinary lookups
        for k in ("fetch_rows", "sparse_update_rows", "shard_reduce_update"):
            alg.pop(k, None)
    kernels = {}
    for name, ms_list in kernel_ms.items():
        if not ms_list:
            continue
        # the median launch: the first eager launch of a kernel after the graph captures can take many
        # times longer than the others (observed: 21.8 ms against 1.39 ms) and would skew a mean
        avg = sorted(ms_list)[len(ms_list) // 2]
        entry = {"launches": len(ms_list), "avg_ms": round(avg, 4), "total_ms": round(avg * len(ms_list), 3)}
        if name in alg:
            gbs = alg[name] / (avg * 1e-3) / 1e9
            entry.update({"algorithmic_bytes": int(alg[name]), "achieved_gbs": round(gbs, 1),
                          "frac_of_%s_peak" % peak_kind: round(gbs / peak, 4)})
        if name in flops:
            entry.update({"algorithmic_flops": flops[name], "achieved_tflops": round(flops[name] / (avg * 1e-3) / 1e12, 1)})
        kernels[name] = entry
    timing_note = "CUDA events around each launch, eager pass over the same K steps"
    roofline = None
    if cfg["shared"] and cfg["geo"] in ALU_OPS_PER_TERM and fma_rate:
        # shared candidates: every pair re-uses rows that other pairs use, so these kernels are bound by
        # fp32 ALU throughput.  Work unit = one (pair, dim) term evaluation; the bound is the measured
        # fp32 instruction rate divided by the instructions one term costs in the kernel's inner loop.
        terms = float(cfg["B"]) * cfg["K"] * cfg["dim"]
        ops = ALU_OPS_PER_TERM[cfg["geo"]]
        for name, key in (("rows_forward", "fwd"), ("rows_backward", "bwd")):
            if name in kernels:
                rate = terms / (kernels[name]["avg_ms"] * 1e-3)
                kernels[name].update({"term_evals_per_s": rate, "alu_ops_per_term": ops[key],
                                      "frac_of_fp32_alu": round(rate * ops[key] / fma_rate, 4)})
        cands = [k for k in ("rows_forward", "rows_backward") if k in kernels]
        if cands:
            dom = max(cands, key=lambda k: kernels[k]["total_ms"])
            key = "fwd" if dom == "rows_forward" else "bwd"
            roofline = {"kernel": dom, "bound": "fp32_alu", "achieved": round(kernels[dom]["term_evals_per_s"] / 1e12, 3),
                        "peak": round(fma_rate / ops[key] / 1e12, 3), "unit": "T term-evaluations/s",
                        "peak_source": "fp32 FMA rate of the library's probe kernel, measured in this run "
                                       "(%.1f T instr/s) / %d ALU instructions per term" % (fma_rate / 1e12, ops[key]),
                        "frac": kernels[dom]["frac_of_fp32_alu"], "traffic": None, "timing": timing_note}
        return kernels, roofline, n_unique_mean
    dom = max((k for k in kernels if k in alg or k in flops), key=lambda k: kernels[k]["total_ms"], default=None)
    if dom in flops:
        # tensor-core GEMM: useful flops against the measured dense bf16 rate scaled to the mode in use
        # (TF32 issues at half the bf16 rate; the fp32 mode spends nine bf16 MMAs per product)
        from smore_b200 import ext_ops as _ops
        mode = _ops.dot_precision()
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                bf16, src = float(json.load(f)["bf16_tflops"]), "measured bf16 burst"
        except Exception:
            bf16, src = 1590.0, "fallback bf16"
        tpeak = bf16 / (9.0 if mode == "fp32" else 2.0)
        roofline = {"kernel": dom, "bound": "tensor", "achieved": kernels[dom]["achieved_tflops"], "peak": round(tpeak, 1),
                    "peak_source": "%s / %s" % (src, "9 (bf16x9 fp32 emulation)" if mode == "fp32" else "2 (tf32)"),
                    "unit": "TFLOP/s", "frac": round(kernels[dom]["achieved_tflops"] / tpeak, 4), "traffic": None,
                    "timing": timing_note}
    elif dom:
        roofline = {"kernel": dom, "bound": "hbm", "achieved": kernels[dom]["achieved_gbs"], "peak": peak,
                    "peak_source": peak_kind, "unit": "GB/s", "frac": round(kernels[dom]["achieved_gbs"] / peak, 4),
                    "traffic": ncu_traffic(workload, dom, n_unique_mean, fused=n_single_mean > 0), "timing": timing_note}
    if n_single_mean:
        roofline = dict(roofline or {}, rows_updated_in_backward=round(n_single_mean, 1))
    return kernels, roofline, n_unique_mean


def cublas_comparison(cfg, device):
    """torch.mm (cuBLAS) on the operands of the shared-candidate inner products - the reference's own
    call for this shape (complex.py:186) - in TF32 and in fp32: ms for the forward product and for the
    two gradient products."""
    B, K = cfg["B"], cfg["K"]
    W = cfg["dim"] * (2 if cfg["geo"] == "complex" else 1)
    q = torch.randn(B, W, device=device) * 0.05
    e = torch.randn(K, W, device=device) * 0.05
    g = torch.randn(B, K, device=device)
    out = {}
    prev = torch.backends.cuda.matmul.allow_tf32
    for name, tf32 in (("tf32", True), ("fp32", False)):
        torch.backends.cuda.matmul.allow_tf32 = tf32
        for what, fn in (("forward", lambda: torch.mm(q, e.t())),
                         ("backward", lambda: (torch.mm(g, e), torch.mm(g.t(), q)))):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                fn()
            b.record()
            torch.cuda.synchronize()
            out["%s_%s_ms" % (name, what)] = round(a.elapsed_time(b) / 10, 4)
    torch.backends.cuda.matmul.allow_tf32 = prev
    return out


def parity_check(args, device, world, rank):
    """Several GPUs, before anything is timed: the production mode of the sharded step (candidate rows
    scored and updated by their owners, replayed CUDA graphs, the next step's remaining rows prefetched
    by bulk copies from peer memory, stale rows repaired from the owners' bitmaps) and the plain mode
    (every row pulled to the rank that looked it up after the previous update, row gradients pulled
    back by the owners, eager launches) run the same five steps (2i, up structures) from identical state on a small
    table; every rank compares its shard of the table and of the Adam state and all dense parameters.
    The two modes run the same kernels on the same values; the only freedom is the order of atomic
    additions into gradient rows that several positions of a rank share, so the comparison allows
    the atomic-accumulation tolerance and also reports whether the results were bit-identical."""
    import torch.distributed as dist
    cfg = dict(WORKLOADS["freebase_q2b"], B=128, K=256, structures=["2i", "up"])
    rows = 200000
    results = []
    for graphs, prefetch, remote in ((True, True, not args.no_remote), (False, False, False)):
        r = StepRunner(cfg, rows, device, world, rank, graphs=graphs, prefetch=prefetch, pool=4, resettable=True,
                       remote=remote)
        r.reset_state()
        if r.chained_graphs:
            r.run_resident(0, 4)           # start_chain runs batch -1 eagerly, then four replays
        else:
            r.run_resident(-1, 5)
        r.sync_all()
        results.append({k: v.detach().clone() for k, v in r.state_tensors().items()})
        r.close()
    # Two correct implementations that add the same numbers in different orders do not stay within
    # rounding of each other for five Adam steps: an L1-type term whose operands nearly tie can take
    # the other sign, and Adam turns a gradient element of rounding-noise size into a full-size step.
    # Such elements are isolated (a few per million); a defect in the exchange (contributions lost or
    # applied twice for the rows several positions share, a rank's gradients missing) moves percents of
    # the rows.  So, relative to each tensor's largest magnitude: at most `frac_allowed` of a tensor's
    # elements may differ by more than `tol`, none by more than `cap`, and everything must be finite.
    tol, cap, frac_allowed = 1e-4, 0.1, 1e-4
    worst, worst_frac, identical = 0.0, 0.0, 1.0
    for k in results[0]:
        a, b = results[0][k].float(), results[1][k].float()
        if a.numel() == 0:
            continue
        scale = float(b.abs().max().clamp_min(1e-30))
        diff = (a - b).abs() / scale
        diff = torch.where(torch.isfinite(diff), diff, torch.full_like(diff, float("inf")))
        worst = max(worst, min(float(diff.max()), 1e30))
        worst_frac = max(worst_frac, float((diff > tol).sum()) / diff.numel())
        identical = min(identical, float(torch.equal(a, b)))
    t = torch.tensor([worst, worst_frac, -identical], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    worst, worst_frac, identical = float(t[0]), float(t[1]), bool(-float(t[2]) > 0.5)
    ok = worst <= cap and worst_frac <= frac_allowed
    verdict = {"prefetch_vs_sync": ("bit-identical" if identical else "within tolerance" if worst <= tol else
                                    "within tolerance (isolated elements beyond it)" if ok else "MISMATCH"),
               "modes": ("owner-side scoring, replayed graphs, prefetch" if not args.no_remote else
                         "pulled rows, replayed graphs, prefetch") + " vs pulled rows, eager launches, no prefetch",
               "steps": 5, "max_rel_diff": worst, "tolerance": tol, "fraction_beyond_tolerance": worst_frac,
               "fraction_allowed": frac_allowed, "largest_allowed": cap, "rows_per_gpu": rows,
               "structures": cfg["structures"], "compared": "per-rank table shard, Adam state, dense parameters"}
    if not ok:
        if rank == 0:
            print(json.dumps({"parity_check": verdict}), flush=True)
        raise SystemExit("parity check failed: prefetch/graph mode and plain mode differ by %g" % worst)
    return verdict


def run_workload(name, cfg, args, device, world, rank, steps, warmup, repeats, peak, peak_kind, fma_rate, clocks=None):
    """Build one workload, time it (device-resident inputs, then end to end), take the per-kernel
    times, free it.  Returns the dict that describes it."""
    import torch.distributed as dist
    from smore_b200 import _lib
    rows_per_gpu = args.rows or cfg["rows"] or (FREEBASE_ENTITIES + 7) // 8
    runner = StepRunner(cfg, rows_per_gpu, device, world, rank, graphs=not args.no_graphs, prefetch=not args.no_prefetch,
                        lazy=not args.no_lazy, fused_paths=not args.no_fused_paths, pool=args.pool,
                        fused_update=not args.no_fused_update, remote=not args.no_remote)
    import gc
    gc.collect()
    gc.freeze()        # keep the cycle collector from scanning the long-lived model objects inside a timed region
    runner.run_resident(0, warmup)
    runner.sync_all()
    if clocks is not None:
        clocks.start()
    L = runner.L
    # ---- resident-input timing ("value"): `repeats` timed regions of exactly `steps` steps each -------
    samples = []
    k0 = warmup
    for _ in range(repeats):
        launches0 = L.smore_kernel_launch_count()
        ms, host, _ = timed_steps(runner, k0, steps)
        launches = runner.launches_in(k0, steps, L.smore_kernel_launch_count() - launches0)
        samples.append((ms, host, launches))
        k0 += steps
    # ---- end-to-end timing: pinned host index tensors in, loss out, every step --------------------------
    runner.prepare_e2e(0)
    runner.run_e2e(0, min(3, warmup))
    runner.sync_all()
    e2e_samples, last_loss = [], 0.0
    for rep in range(repeats):
        ms, _, last_loss = timed_steps(runner, warmup + rep * steps, steps, e2e=True)
        e2e_samples.append(ms)
    if _lib.async_status() != 0:
        raise RuntimeError("device status word %d (a bulk-copy wait gave up, or a row id lay outside the table): "
                           "the timed results are invalid" % _lib.async_status())
    ms_eager, kernel_ms, notes = runner.eager_timed_pass(warmup, steps)
    gc.unfreeze()
    launch_counts = [s[2] for s in samples]
    host_issue = sorted(s[1] for s in samples)[len(samples) // 2]   # host time to enqueue a region's steps
    samples = torch.tensor([[s[0] for s in samples], e2e_samples], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(samples, op=dist.ReduceOp.MAX)      # per timed region: the slowest rank
    res_ms = sorted(samples[0].tolist())
    e2e_ms = sorted(samples[1].tolist())
    med, med_e2e = res_ms[len(res_ms) // 2], e2e_ms[len(e2e_ms) // 2]
    structures = runner.structures
    out = None
    if rank == 0:
        kernels, roofline, n_unique_mean = kernel_table(cfg, name, kernel_ms, notes, peak, peak_kind, fma_rate)
        total_queries = cfg["B"] * world * steps
        out = {
            "value": round(total_queries / (med * 1e-3), 1), "unit": "queries/s",
            "ms_per_step": round(med / steps, 4),
            "repeats": {"n": repeats, "steps_each": steps, "statistic": "median",
                        "ms_per_step_min": round(res_ms[0] / steps, 4), "ms_per_step_max": round(res_ms[-1] / steps, 4)},
            "execution": ("one captured CUDA graph per query structure, replayed" if runner.use_graphs else
                          "one captured CUDA graph per (query structure, arena), replayed; next step's rows prefetched "
                          "inside the graph" if runner.chained_graphs else "eager launches"),
            "eager_ms_per_step": round(ms_eager / steps, 4),
            "config": {"workload": name, "geo": cfg["geo"], "queries_per_gpu": cfg["B"], "negatives": cfg["K"],
                       "shared_negatives": cfg["shared"], "dim": cfg["dim"], "table_rows_per_gpu": rows_per_gpu,
                       "table_rows_total": runner.n_rows, "structures": structures,
                       "parallelism": "1 GPU, table resident" if world == 1 else
                                      ("table and Adam state row-sharded over %d GPUs; candidate rows scored and updated by "
                                       "their owners (queries, scores and their gradients over NVLink)" % world
                                       if runner.remote else
                                       "table and Adam state row-sharded over %d GPUs, rows and row gradients over NVLink"
                                       % world),
                       "optimizer": "adam, row-wise v" if cfg["squeeze"] else "adam, full v",
                       "lazy_rows": not args.no_lazy,
                       "l2_policy": ("inputs larger than L2: every step touches ~%.1f GB of table rows" %
                                     (cfg["B"] * cfg["K"] * cfg["dim"] * 4 / 1e9)) if not cfg["shared"] else
                                    "working set smaller than L2 by construction (shared candidates): the kernels "
                                    "are bound by arithmetic, not by memory"},
            "e2e": {"value": round(total_queries / (med_e2e * 1e-3), 1), "unit": "queries/s",
                    "ms_per_step": round(med_e2e / steps, 4),
                    "h2d_bytes_per_step": int(runner.h2d_bytes), "d2h_bytes_per_step": 4},
            "gpu_launches": int(launch_counts[0]),
            "distinct_rows_per_step": round(n_unique_mean, 1),
            "roofline": roofline,
            "kernels": kernels,
            "host_issue_ms_per_step": round(1e3 * host_issue / steps, 4),
            "last_loss": last_loss,
        }
        if args.dump_kernel_times:
            out["kernel_ms_raw"] = {k: [round(x, 3) for x in v] for k, v in kernel_ms.items()}
    runner.close()
    return out


def run_gpu(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path for the product arm)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peak, peak_kind = load_peaks()
    fma_rate = measure_fma_rate(device)
    parity = parity_check(args, device, world, rank) if world > 1 and not args.no_parity_check else None

    cfg = dict(WORKLOADS[args.workload])
    if args.structures:
        cfg["structures"] = args.structures.split(",")
    clocks = ClockSampler(local_rank)
    head = run_workload(args.workload, cfg, args, device, world, rank, args.steps, args.warmup, args.repeats, peak,
                        peak_kind, fma_rate, clocks)
    clock_summary = clocks.summary()

    # the other configurations, one after the other in the same process (1 GPU, default workload only)
    others = {}
    if world == 1 and args.workload == "freebase_q2b" and not args.headline_only and not args.structures:
        extra = [("rotate_wikikg", None), ("q2b_fb15k", None), ("gqe_fb15k237", None),
                 ("distmult_wikikg", "fp32"), ("distmult_wikikg", "tf32")]
        for name, dot_mode in extra:
            wcfg = dict(WORKLOADS[name])
            prev = os.environ.get("SMORE_B200_DOT")
            if dot_mode:
                os.environ["SMORE_B200_DOT"] = dot_mode
            try:
                res = run_workload(name, wcfg, args, device, 1, 0, args.steps, max(3, args.warmup), 3, peak, peak_kind,
                                   fma_rate)
                if dot_mode:
                    res["dot_precision"] = dot_mode
                    from smore_b200 import _lib as _l
                    res["gemm_tiles"] = ("256x128 / 256x256 tiles on SM pairs (companion library loaded)"
                                         if _l.lib().smore_dot_two_sm() else "128x128 tiles, one SM each")
                    cb = cublas_comparison(wcfg, device)
                    res["cublas"] = cb
                    for kname, what in (("dot_forward", "forward"), ("dot_backward", "backward")):
                        if kname in res["kernels"]:
                            res["kernels"][kname]["vs_cublas"] = round(
                                cb["%s_%s_ms" % (dot_mode, what)] / res["kernels"][kname]["avg_ms"], 3)
                slim = {k: res[k] for k in ("value", "unit", "ms_per_step", "repeats", "eager_ms_per_step", "e2e", "roofline",
                                            "kernels", "gpu_launches", "distinct_rows_per_step", "gemm_tiles") if k in res}
                slim["config"] = {k: res["config"][k] for k in ("geo", "queries_per_gpu", "negatives", "shared_negatives",
                                                                "dim", "table_rows_per_gpu", "structures", "optimizer")}
                for k in ("dot_precision", "cublas"):
                    if k in res:
                        slim[k] = res[k]
                others[name if not dot_mode else "%s[%s]" % (name, dot_mode)] = slim
            except Exception as exc:      # a side workload must not take the headline line down with it
                others[name if not dot_mode else "%s[%s]" % (name, dot_mode)] = {"failed": repr(exc)}
            finally:
                if dot_mode:
                    if prev is None:
                        os.environ.pop("SMORE_B200_DOT", None)
                    else:
                        os.environ["SMORE_B200_DOT"] = prev

    def shutdown():
        torch.cuda.synchronize()
        if world > 1:
            # every graph that captured a collective is gone (StepRunner.close); should the communicator
            # still be busy, do not let the process hang on it after the line has been printed
            sys.stdout.flush()
            sys.stderr.flush()
            watchdog = threading.Timer(20.0, lambda: os._exit(0))
            watchdog.daemon = True
            watchdog.start()
            dist.destroy_process_group()
            watchdog.cancel()

    if rank != 0:
        shutdown()
        return

    cpu = None
    if not args.no_cpu_baseline and world == 1:      # reported at N=1 only
        try:
            r = cpu_reference_steps(cfg, steps=args.cpu_steps, warmup=2)
            cpu = {"value": round(r["value"], 1), "unit": "queries/s", "cores": r["cores"], "kind": r["kind"],
                   "ms_per_step": round(r["ms_per_step"], 2), "sample": r["sample"]}
        except Exception as exc:  # the baseline is a report, not a dependency of the product arm
            cpu = {"value": None, "unit": "queries/s", "cores": None, "kind": "port", "sample": "failed: %r" % (exc,)}

    out = {
        "metric": "queries/sec (fwd+bwd+sparse update)",
        "value": head["value"], "unit": "queries/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
    }
    for k in ("repeats", "execution", "eager_ms_per_step", "config", "e2e", "gpu_launches", "distinct_rows_per_step",
              "roofline", "kernels", "last_loss"):
        out[k] = head[k]
    if "kernel_ms_raw" in head:
        out["kernel_ms_raw"] = head["kernel_ms_raw"]
    out["cpu_baseline"] = cpu
    out["clocks"] = clock_summary
    out["fp32_fma_per_s"] = fma_rate
    if parity is not None:
        out["parity_check"] = parity
    if others:
        out["workloads"] = others
    print(json.dumps(out), flush=True)
    shutdown()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(WORKLOADS[args.workload])
    r = cpu_reference_steps(cfg, steps=args.steps, warmup=args.warmup)
    qps, ms = r["value"], r["ms_per_step"]
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    out = {
        "impl": "reference",
        "metric": "queries/sec (fwd+bwd+sparse update)", "value": round(qps, 1), "unit": "queries/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "geo": cfg["geo"], "queries_per_gpu": cfg["B"],
                   "negatives": cfg["K"], "dim": cfg["dim"], "structures": cfg["structures"]},
        "cpu_baseline": {"value": round(qps, 1), "unit": "queries/s", "cores": r["cores"], "kind": r["kind"],
                         "sample": r["sample"]},
        "e2e": {"value": round(qps, 1), "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out), flush=True)


def run_eval(args):
    """Side benchmark (not the contract line): the evaluation step that follows the hot path in the
    reference (train_process.py:104-153) - score a batch of queries against EVERY entity with the
    distance ops (one shared candidate set), then the filtered ranks of their answers - and the same
    work through the reference's argsort/scatter block on the host cores."""
    from smore_b200 import _lib, ext_ops, ranking
    from oracle.native_torch import box_logit, vec_logit, reference_filtered_ranks
    cfg = dict(WORKLOADS[args.workload])
    if cfg["geo"] not in ("box", "vec"):
        raise SystemExit("--eval covers the box and vec workloads")
    device = torch.device("cuda", 0)
    N = args.rows or cfg["rows"] or (FREEBASE_ENTITIES + 7) // 8
    D, Q = cfg["dim"], args.eval_queries
    r = (cfg["gamma"] + 2.0) / D
    g = torch.Generator(device=device).manual_seed(7)
    table = torch.empty(N, D, device=device).uniform_(-r, r, generator=g)
    center = torch.empty(Q, 1, D, device=device).uniform_(-r, r, generator=g)
    offset = torch.empty(Q, 1, D, device=device).uniform_(0, r, generator=g)
    rng = torch.Generator().manual_seed(8)
    easy = [torch.randint(0, N, (10,), generator=rng).unique().tolist() for _ in range(Q)]
    hard = [[i for i in torch.randint(0, N, (20,), generator=rng).unique().tolist() if i not in set(e)]
            for e in easy]
    everything = table.unsqueeze(0)

    def score():
        if cfg["geo"] == "box":
            d_out, d_in = ext_ops.box_dist_both(everything, center, offset)     # one pass over the table
            return cfg["gamma"] - d_out - cfg["cen"] * d_in
        return cfg["gamma"] - ext_ops.l1_dist(everything, center)

    geo = "box" if cfg["geo"] == "box" else "vec"
    query = (center, offset) if geo == "box" else (center,)

    def step():
        # scoring and counting in one kernel: the [Q, N] logits are never written
        with torch.no_grad():
            return ranking.score_and_rank(geo, table, query, easy, hard, cfg["gamma"], cfg["cen"])

    def two_steps():
        with torch.no_grad():
            return ranking.filtered_ranks(score(), easy, hard)

    def time_ms(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps, out

    ms, ranks = time_ms(step)
    ms_two, ranks_two = time_ms(two_steps)
    if not all(torch.equal(a, b) for a, b in zip(ranks, ranks_two)):
        raise RuntimeError("fused scoring + ranking and ranking from materialised logits disagree")
    # host cores: the reference's scoring (torch twins) and ranking block, a few queries of the same batch
    torch.set_num_threads(os.cpu_count() or 1)
    n_cpu = min(Q, args.cpu_steps)
    tab_c, cen_c, off_c = table.cpu(), center.cpu(), offset.cpu()
    t0 = time.perf_counter()
    for q in range(n_cpu):
        pieces = []
        for lo in range(0, N, 200000):          # the torch twins materialise [N, D] temporaries
            blk = tab_c[lo:lo + 200000].unsqueeze(0)
            if cfg["geo"] == "box":
                pieces.append(box_logit(blk, [cen_c[q:q + 1], off_c[q:q + 1]], cfg["gamma"], cfg["cen"]))
            else:
                pieces.append(vec_logit(blk, [cen_c[q:q + 1]], cfg["gamma"]))
        lg = torch.cat(pieces, dim=1)
        want = reference_filtered_ranks(lg, easy[q], hard[q])
        got = ranks[q].cpu().float()
        if not torch.equal(got, want):      # the host scoring rounds differently: ranks may move by near-ties
            close = (got - want).abs().max().item() <= max(2.0, 1e-5 * N)
            if not close:
                raise RuntimeError("evaluation ranks differ from the reference block: %s vs %s" % (got, want))
    cpu_s = (time.perf_counter() - t0) / n_cpu
    out = {
        "metric": "evaluation queries/sec (score every entity + filtered ranks)", "value": round(Q / (ms * 1e-3), 1),
        "unit": "queries/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "eval:" + args.workload, "queries_per_step": Q, "candidates": N, "dim": D,
                   "answers_per_query": "~10 easy + ~20 hard"},
        "path": "smore_score_filtered_ranks (scores never written); ranks equal to the two-step route",
        "two_step_ms_per_step": round(ms_two, 3), "two_step_logits_bytes": Q * N * 4,
        "cpu_baseline": {"value": round(1.0 / cpu_s, 2), "unit": "queries/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": "%d queries of the same batch" % n_cpu},
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=18)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--headline-only", action="store_true", help="1 GPU: skip the other configurations")
    ap.add_argument("--no-parity-check", action="store_true",
                    help="several GPUs: skip the comparison of the graph + prefetch mode with the plain mode")
    ap.add_argument("--workload", default="freebase_q2b", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="smore_b200", choices=["smore_b200", "reference"])
    ap.add_argument("--rows", type=int, default=0, help="override entity-table rows per GPU")
    ap.add_argument("--structures", default="", help="comma-separated subset of query structures (profiling runs)")
    ap.add_argument("--pool", type=int, default=18, help="distinct pre-generated batches to cycle through")
    ap.add_argument("--no-lazy", action="store_true", help="gather candidate rows instead of reading the table in place")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graphs", action="store_true", help="launch every step eagerly instead of replaying CUDA graphs")
    ap.add_argument("--no-prefetch", action="store_true",
                    help="several GPUs: pull every step's rows after the previous update instead of during it")
    ap.add_argument("--no-fused-paths", action="store_true",
                    help="embed path queries hop by hop with torch ops, as the reference models do")
    ap.add_argument("--no-fused-update", action="store_true",
                    help="1 GPU: write every row gradient out and update all touched rows in the update kernel")
    ap.add_argument("--no-remote", action="store_true",
                    help="several GPUs: pull candidate rows to the rank that scores them (and their gradients back) "
                         "instead of scoring them on their owners")
    ap.add_argument("--cpu-steps", type=int, default=6)
    ap.add_argument("--dump-kernel-times", action="store_true", help="add every timed launch's duration to the JSON")
    ap.add_argument("--eval", action="store_true",
                    help="side benchmark: score queries against every entity and rank their answers (1 GPU)")
    ap.add_argument("--eval-queries", type=int, default=32)
    args = ap.parse_args()
    if args.eval:
        run_eval(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
