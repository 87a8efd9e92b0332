"""Entity table and Adam state row-sharded over the GPUs of one NVLink / NVSwitch box.

One process per GPU.  Rank g owns global rows [g*S, (g+1)*S), S = ceil(N / G), of the table and of
its optimizer state.  Every rank trains on its own batches (as the reference's per-GPU processes
do, smore/training/train_process.py:306-310); what the reference does through a table in CPU
shared memory with pinned PCIe staging and hogwild additive writes
(smore/common/embedding/embed_rw.py:53-134, smore/common/embedding/embed_optimizer.py:248-252)
happens here over NVLink with plain peer loads, synchronously per step:

  forward   the ids a rank looks up are de-duplicated; each distinct row is pulled once from its
            owner into a local staging block (smore_fetch_rows); lookups and the distance kernels
            then address the staging block by slot.
  backward  row gradients accumulate in the rank's compact buffer, which lives in peer-visible
            memory together with the sorted id list.
  update    after a stream-ordered barrier every owner collects the ids of its range from all
            ranks' lists (one contiguous run per sorted list), de-duplicates them
            (smore_shard_owner_plan), and one kernel pulls the matching gradient rows with bulk
            copies kept in flight ahead of the row being updated, sums them in a fixed order and
            applies Adam to the shard (smore_shard_reduce_update_rows); a second barrier ends the
            step.
  prefetch  (optional) the rows of the NEXT step's first lookup group are pulled on a side stream
            while the current step computes; after the step's last barrier only the rows their
            owners updated meanwhile (published as a bitmap) are pulled again, so the result is
            the same as fetching everything after the barrier.

  remote    (optional, `remote=RemoteSpec(...)`) the candidate-scoring op of the step - B*K rows per
            rank - does not move rows at all: the rank publishes the candidate ids, its queries and
            later the upstream gradients of its scores; every owner scores and differentiates the
            pairs that fall into its range against its own shard (smore_owner_* and the ragged
            row-stream kernels), applies the row gradients in place (Adam folded into the backward
            kernel) and hands back scores and partial query gradients: a few bytes per pair over
            NVLink instead of a row each way.

A step therefore equals one optimizer step of a single process on the union of all ranks'
batches (all gradients of a row are summed before its one Adam update).

`ShardGroup.emulated(...)` builds the same objects for G ranks inside one process on one GPU (all
"peer" pointers local, barriers replaced by call order) for tests.
"""
import ctypes
import os

import torch

from . import _lib
from .embedding import (EmbeddingOptimizer, LazyRows, _DUMMY_JOB, _EmbedLookupFunc, _Lookup, _stream_ptr,
                        eps)

MAX_PLANS = 4


def rows_of_rank(full, rank, world):
    """The rows of a full [N, ...] tensor that rank `rank` of `world` owns."""
    S = shard_rows(full.shape[0], world)
    return full[rank * S:min(full.shape[0], (rank + 1) * S)]


def merge_shard_states(states, prefix="entity_embedding."):
    """Rebuild the reference's checkpoint entries of a sparse embedding from the ranks' shard states
    (ShardedTable.shard_state()), in any order: `<prefix>embedding`, `<prefix>state_sum_fo`,
    `<prefix>state_sum_sq` - the keys `model.state_dict()` holds for a SparseEmbedding whose optimizer
    registered its state on it (sparse_embed.py:50-53, embed_optimizer.py:192-197), as saved by
    train_process.py:250-260."""
    states = sorted(states, key=lambda st: st["rank"])
    world = states[0]["world"]
    if [st["rank"] for st in states] != list(range(world)):
        raise ValueError("need the state of every rank 0..%d exactly once" % (world - 1))
    for st in states:
        for k in ("world", "n_rows_total", "width", "squeeze"):
            if st[k] != states[0][k]:
                raise ValueError("shard states disagree on %s" % k)
    out = {}
    for key in ("embedding", "state_sum_fo", "state_sum_sq"):
        out[prefix + key] = torch.cat([st[key] for st in states], dim=0)
        if out[prefix + key].shape[0] != states[0]["n_rows_total"]:
            raise ValueError("shard states do not add up to %d rows" % states[0]["n_rows_total"])
    return out


class _DeviceBlock(object):
    """A byte block of device memory (a uint8 tensor) that typed views are cut from.

    Peer-visible blocks come from torch's symmetric-memory allocator, which maps every rank's
    block into every process with large pages.  (Mapping a peer's cudaMalloc block through a CUDA
    IPC handle also works, but random 1.6 KB row reads through such a mapping ran at ~80 GB/s on
    B200 against ~700 GB/s through a symmetric-memory mapping, so that route is not offered.)"""

    def __init__(self, tensor):
        self.tensor = tensor
        self.ptr, self.nbytes = tensor.data_ptr(), tensor.numel()

    def view(self, device, offset, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.tensor[offset:offset + nbytes].view(dtype).view(shape)


def _round(x, a=256):
    return (x + a - 1) // a * a


class ArenaLayout(object):
    """Byte layout of a rank's peer-visible per-step arena (identical on every rank):
    [n_unique int32[MAX_PLANS][2] | ids int64[sum caps] | gradient rows float32[sum caps, width]]."""

    def __init__(self, plan_caps, width):
        if not 1 <= len(plan_caps) <= MAX_PLANS:
            raise ValueError("1..%d plan capacities expected" % MAX_PLANS)
        self.plan_caps = tuple(int(c) for c in plan_caps)
        self.width = int(width)
        self.prefix = [0]
        for c in self.plan_caps:
            self.prefix.append(self.prefix[-1] + c)
        self.span = self.prefix[-1]
        self.off_nuniq = 0
        self.off_ids = _round(MAX_PLANS * 2 * 4)
        self.off_grads = self.off_ids + _round(self.span * 8)
        self.nbytes = self.off_grads + _round(self.span * self.width * 4)

    def nuniq_offset(self, p):
        return self.off_nuniq + p * 8

    def ids_offset(self, p):
        return self.off_ids + self.prefix[p] * 8

    def grads_offset(self, p):
        return self.off_grads + self.prefix[p] * self.width * 4


class RemoteSpec(object):
    """Sizes of owner-side scoring: at most `queries` queries of `dim` floats per operand and `pairs`
    (query, candidate) pairs per rank and step (a union step counts every branch as a query);
    `owner_pairs` bounds the pairs one owner may receive from all ranks in a step (default: twice a
    rank's own, at least all of them on one GPU)."""

    def __init__(self, pairs, queries, dim, owner_pairs=None):
        self.pairs, self.queries, self.dim = int(pairs), int(queries), int(dim)
        self.owner_pairs = None if owner_pairs is None else int(owner_pairs)
        if self.dim % 4 or self.pairs <= 0 or self.queries <= 0:
            raise ValueError("RemoteSpec: dim must be a multiple of 4, pairs and queries positive")


class RemoteLayout(object):
    """Byte layout of a rank's peer-visible block for owner-side scoring:
    [descriptor int32[8] | candidate ids int64[pairs] | queries float32[2][queries*dim] |
     results float32[2][pairs] | upstream gradients float32[2][pairs] |
     partial query gradients float32[2][world*queries*dim] (written by this rank as an owner)]."""

    def __init__(self, spec, world):
        P, QD = spec.pairs, spec.queries * spec.dim
        self.off_desc = 0
        self.off_ids = 256
        self.off_queries = self.off_ids + _round(P * 8)
        self.off_results = self.off_queries + 2 * _round(QD * 4)
        self.off_upstream = self.off_results + 2 * _round(P * 4)
        self.off_partial = self.off_upstream + 2 * _round(P * 4)
        self.nbytes = self.off_partial + 2 * _round(world * QD * 4)
        self.stride_queries = _round(QD * 4)
        self.stride_pairs = _round(P * 4)
        self.stride_partial = _round(world * QD * 4)


def shard_rows(n_rows_total, world):
    return (n_rows_total + world - 1) // world


def owner_of(ids, n_rows_total, world):
    """Owning rank of each global row id (contiguous ranges of ceil(N / G) rows)."""
    return ids // shard_rows(n_rows_total, world)


def pointer_tables(layout, arena_ptrs):
    """Addresses of every (rank, plan) list inside the ranks' arenas, in list order
    l = rank * n_plans + plan — the order the owner-side kernels index them by."""
    P = len(layout.plan_caps)
    pairs = [(g, p) for g in range(len(arena_ptrs)) for p in range(P)]
    return {"ids": [arena_ptrs[g] + layout.ids_offset(p) for g, p in pairs],
            "nuniq": [arena_ptrs[g] + layout.nuniq_offset(p) for g, p in pairs],
            "grads": [arena_ptrs[g] + layout.grads_offset(p) for g, p in pairs]}


def exchange_handles(my_handles, group=None):
    """All ranks' handle lists, indexed by rank (object all-gather over the process group); for
    transports that pass their own handles between processes."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = [None] * world
    dist.all_gather_object(out, my_handles, group=group)
    return out


BACKGROUND_CTAS = 148     # thread blocks of a prefetch copy: one per SM


class ShardedTable(object):
    """The local shard (table + Adam state), two peer-visible per-step arenas (steps alternate
    between them, so the next step's id list can be prepared while owners still read the current
    one), the bitmap of rows updated in the last step, and the pointer tables."""

    def __init__(self, n_rows_total, width, rank, world, device, plan_caps, squeeze=True, symmetric=False, remote=None):
        self.n_rows_total, self.width, self.rank, self.world = int(n_rows_total), int(width), rank, world
        self.remote = remote
        self.device = torch.device(device)
        self.squeeze = bool(squeeze)
        self.S = shard_rows(n_rows_total, world)
        self.base = rank * self.S
        self.local_rows = max(0, min(self.S, n_rows_total - self.base))
        self.layout = ArenaLayout(plan_caps, width)
        self.symmetric = symmetric
        self._table_block = self._alloc(max(self.S, 1) * width * 4)
        self._arena_blocks = [self._alloc(self.layout.nbytes) for _ in range(2)]
        self._dirty_block = self._alloc(((max(self.S, 1) + 31) // 32) * 4)
        self.table = self._table_block.view(self.device, 0, (self.S, width), torch.float32)
        self.dirty = self._dirty_block.view(self.device, 0, ((max(self.S, 1) + 31) // 32,), torch.int32)
        self.dirty.zero_()
        self.bitmap_scratch = torch.empty(world * self.dirty.numel(), dtype=torch.int32, device=self.device)
        self.m = torch.zeros(self.S, width, device=self.device)
        self.v = torch.zeros(self.S, 1, device=self.device) if squeeze else torch.zeros(self.S, width, device=self.device)
        lay = self.layout
        P = len(lay.plan_caps)
        self.nuniq = [[blk.view(self.device, lay.nuniq_offset(p), (2,), torch.int32) for p in range(P)]
                      for blk in self._arena_blocks]
        self.nuniq_all = [blk.view(self.device, 0, (MAX_PLANS * 2,), torch.int32) for blk in self._arena_blocks]
        for t in self.nuniq_all:
            t.zero_()
        self.ids = [[blk.view(self.device, lay.ids_offset(p), (lay.plan_caps[p],), torch.int64) for p in range(P)]
                    for blk in self._arena_blocks]
        self.grads = [[blk.view(self.device, lay.grads_offset(p), (lay.plan_caps[p], width), torch.float32)
                       for p in range(P)] for blk in self._arena_blocks]
        self.peer_table_ptrs = None   # filled by connect()
        self._handles = []
        self._remote_block = None
        if remote is not None:
            if not squeeze:
                raise _lib.SmoreError("owner-side scoring updates rows with the row-wise second moment (squeeze=True)")
            rl = self.remote_layout = RemoteLayout(remote, world)
            blk = self._remote_block = self._alloc(rl.nbytes)
            blk.tensor.zero_()
            dev, P, QD = self.device, remote.pairs, remote.queries * remote.dim
            self.r_desc = blk.view(dev, rl.off_desc, (8,), torch.int32)
            self.r_ids = blk.view(dev, rl.off_ids, (P,), torch.int64)
            self.r_queries = [blk.view(dev, rl.off_queries + i * rl.stride_queries, (QD,), torch.float32) for i in range(2)]
            self.r_results = [blk.view(dev, rl.off_results + i * rl.stride_pairs, (P,), torch.float32) for i in range(2)]
            self.r_upstream = [blk.view(dev, rl.off_upstream + i * rl.stride_pairs, (P,), torch.float32) for i in range(2)]
            self.r_partial = [blk.view(dev, rl.off_partial + i * rl.stride_partial, (world * QD,), torch.float32)
                              for i in range(2)]

    def _alloc(self, nbytes):
        nbytes = _round(nbytes, 16)
        if self.symmetric:
            # this library reads peers with plain loads only; keep the blocks off NVLink multicast
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem
            with torch.cuda.device(self.device):
                t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        else:
            t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return _DeviceBlock(t)

    def connect(self, table_ptrs, arena_ptrs, dirty_ptrs, remote_ptrs=None):
        """Install the base pointers of every rank's shard, arenas (`arena_ptrs[parity][rank]`),
        updated-rows bitmap and, with owner-side scoring, remote block (this rank's own included)."""
        self.peer_table_ptrs = list(table_ptrs)
        dev = self.device
        if self.remote is not None:
            if remote_ptrs is None:
                raise _lib.SmoreError("connect: the ranks' remote blocks are missing")
            rl = self.remote_layout
            tab = lambda off: torch.tensor([p + off for p in remote_ptrs], dtype=torch.int64, device=dev)
            self.d_r_desc, self.d_r_ids = tab(rl.off_desc), tab(rl.off_ids)
            self.d_r_queries = [tab(rl.off_queries + i * rl.stride_queries) for i in range(2)]
            self.d_r_results = [tab(rl.off_results + i * rl.stride_pairs) for i in range(2)]
            self.d_r_upstream = [tab(rl.off_upstream + i * rl.stride_pairs) for i in range(2)]
            self.d_r_partial = [tab(rl.off_partial + i * rl.stride_partial) for i in range(2)]
        self.d_shard_ptrs = torch.tensor(self.peer_table_ptrs, dtype=torch.int64, device=dev)
        self.d_dirty_ptrs = torch.tensor(list(dirty_ptrs), dtype=torch.int64, device=dev)
        self.d_uniq_ptrs, self.d_nuniq_ptrs, self.d_grad_ptrs = [], [], []
        for parity in range(2):
            tabs = pointer_tables(self.layout, list(arena_ptrs[parity]))
            self.d_uniq_ptrs.append(torch.tensor(tabs["ids"], dtype=torch.int64, device=dev))
            self.d_nuniq_ptrs.append(torch.tensor(tabs["nuniq"], dtype=torch.int64, device=dev))
            self.d_grad_ptrs.append(torch.tensor(tabs["grads"], dtype=torch.int64, device=dev))

    def connect_processes(self, group=None):
        """Map the other ranks' blocks (symmetric-memory rendezvous over `group`)."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if not self.symmetric:
            raise _lib.SmoreError("connect_processes needs blocks from the symmetric-memory allocator")
        group = group if group is not None else dist.group.WORLD
        blocks = [self._table_block] + self._arena_blocks + [self._dirty_block]
        if self._remote_block is not None:
            blocks.append(self._remote_block)
        ptrs = []
        with torch.cuda.device(self.device):
            for blk in blocks:
                h = symm_mem.rendezvous(blk.tensor, group)
                self._handles.append(h)
                p = [int(x) for x in h.buffer_ptrs]
                if p[self.rank] != blk.ptr:
                    raise _lib.SmoreError("symmetric-memory rendezvous returned a different address for a local block")
                ptrs.append(p)
        self.connect(ptrs[0], [ptrs[1], ptrs[2]], ptrs[3], ptrs[4] if len(ptrs) > 4 else None)

    def close(self):
        self._handles = []

    def shard_state(self):
        """This rank's rows of the table and of the Adam state as CPU tensors (one file per rank when
        saved); merge_shard_states() turns all ranks' states into the reference's checkpoint keys."""
        n = self.local_rows
        return {"rank": self.rank, "world": self.world, "n_rows_total": self.n_rows_total, "width": self.width,
                "squeeze": self.squeeze, "embedding": self.table[:n].detach().cpu(),
                "state_sum_fo": self.m[:n].detach().cpu(), "state_sum_sq": self.v[:n].detach().cpu()}

    def load_shard_state(self, state):
        for k in ("rank", "world", "n_rows_total", "width", "squeeze"):
            if state[k] != getattr(self, k):
                raise _lib.SmoreError("shard state was saved with %s = %r, this shard has %r" % (k, state[k], getattr(self, k)))
        n = self.local_rows
        self.table[:n].copy_(state["embedding"])
        self.m[:n].copy_(state["state_sum_fo"])
        self.v[:n].copy_(state["state_sum_sq"])

    def load_full(self, embedding, state_sum_fo=None, state_sum_sq=None):
        """Take this rank's rows from full [N, ...] tensors, e.g. the entries of a reference checkpoint
        (`checkpoint['model_state_dict']['entity_embedding.embedding']`, main_train.py:191-194).
        Optimizer state that is not given starts at zero, as a fresh optimizer's would."""
        if embedding.shape != (self.n_rows_total, self.width):
            raise _lib.SmoreError("embedding must be [%d, %d]" % (self.n_rows_total, self.width))
        n = self.local_rows
        self.table[:n].copy_(rows_of_rank(embedding, self.rank, self.world))
        for dst, src, shape in ((self.m, state_sum_fo, (self.n_rows_total, self.width)),
                                (self.v, state_sum_sq, (self.n_rows_total, 1 if self.squeeze else self.width))):
            if src is None:
                dst.zero_()
            else:
                if tuple(src.shape) != shape:
                    raise _lib.SmoreError("optimizer state must be %s, got %s" % (shape, tuple(src.shape)))
                dst[:n].copy_(rows_of_rank(src, self.rank, self.world))

    def init_uniform(self, lo, hi, seed):
        """Fill the shard as rows [base, base+S) of a table drawn uniform(lo, hi); the values depend
        on (seed, rank) only."""
        g = torch.Generator(device=self.device).manual_seed(seed * 1000003 + self.rank)
        self.table.uniform_(lo, hi, generator=g)


class _PlanBuffers(object):
    """Persistent storage of one prefetched plan (ids, slots, counts, staged rows) at full capacity."""

    def __init__(self, capacity, width, device):
        self.idx = torch.empty(capacity, dtype=torch.int64, device=device)
        self.slot = torch.empty(capacity, dtype=torch.int32, device=device)
        self.counts = torch.empty(capacity, dtype=torch.int32, device=device)
        self.slot64 = torch.empty(capacity, dtype=torch.int64, device=device)
        self.staging = torch.empty(capacity, width, dtype=torch.float32, device=device)


def _id_key(t):
    """Identity of an id tensor as the caller holds it: address, element count, innermost stride."""
    return (t.device, t.data_ptr(), t.numel(), t.stride()[-1] if t.dim() else 1, t.dtype)


class _ShardedPlan(object):
    """One de-duplicated group of lookups of a rank: ids and gradients in the arena, rows staged."""

    def __init__(self, opt, id_tensors, index, parity, workspace, buffers=None):
        """Runs on the current stream: unique over the ids, pull of the distinct rows.  `buffers`
        (a _PlanBuffers) replaces the per-step allocations by persistent storage."""
        shard = opt.shard
        dev = shard.device
        self.index, self.parity = index, parity
        self.lookups = []
        self.n = sum(t.numel() for t in id_tensors)
        cap = shard.layout.plan_caps[index]
        if self.n > cap:
            raise _lib.SmoreError("plan %d holds %d looked-up ids, its capacity is %d (plan_caps)" % (index, self.n, cap))
        self.uniq = shard.ids[parity][index]
        self.n_unique = shard.nuniq[parity][index]
        self.g_rows = shard.grads[parity][index]
        if buffers is None:
            self.idx_all = id_tensors[0] if len(id_tensors) == 1 else torch.cat(list(id_tensors))
            self.slot = torch.empty(self.n, dtype=torch.int32, device=dev)
            self.counts = torch.empty(self.n, dtype=torch.int32, device=dev)
            self.staging = torch.empty(self.n, shard.width, dtype=torch.float32, device=dev)
            self.slot64 = None
        else:
            self.idx_all = buffers.idx[:self.n]
            off = 0
            for t in id_tensors:
                self.idx_all[off:off + t.numel()].copy_(t.reshape(-1))
                off += t.numel()
            self.slot, self.counts = buffers.slot[:self.n], buffers.counts[:self.n]
            self.staging, self.slot64 = buffers.staging[:self.n], buffers.slot64[:self.n]
        L = _lib.lib()
        st = _stream_ptr(dev)
        with torch.cuda.device(dev):
            with _lib.timed("unique_rows"):
                _lib.check(L.smore_unique_rows(self.idx_all.data_ptr(), self.n, shard.n_rows_total,
                                               self.uniq.data_ptr(), self.slot.data_ptr(), self.counts.data_ptr(),
                                               self.n_unique.data_ptr(), workspace.data_ptr(), workspace.numel(), st),
                           "smore_unique_rows")
            if opt.exchange == "nccl":
                self._fetch_by_all_to_all(opt)
            with _lib.timed("fetch_rows"):
                if opt.exchange == "nccl":
                    pass
                elif buffers is None:
                    _lib.check(L.smore_fetch_rows(shard.d_shard_ptrs.data_ptr(), shard.S, self.uniq.data_ptr(),
                                                  self.n_unique.data_ptr(), self.n, shard.width,
                                                  self.staging.data_ptr(), st), "smore_fetch_rows")
                else:
                    # a prefetch shares the GPU with the step in progress: one thread block per SM
                    _lib.check(L.smore_fetch_rows_background(shard.d_shard_ptrs.data_ptr(), shard.S,
                                                             self.uniq.data_ptr(), self.n_unique.data_ptr(), self.n,
                                                             shard.width, self.staging.data_ptr(), BACKGROUND_CTAS,
                                                             st), "smore_fetch_rows_background")
            _lib.check(L.smore_zero_shared_rows(self.g_rows.data_ptr(), self.counts.data_ptr(),
                                                self.n_unique.data_ptr(), self.n, shard.width, st),
                       "smore_zero_shared_rows")
        if self.slot64 is None:
            self.slot64 = self.slot.long()
        else:
            self.slot64.copy_(self.slot)

    def _fetch_by_all_to_all(self, opt):
        """The row pull without peer-mapped memory: the distinct ids go to their owners, the owners'
        rows come back, both with torch.distributed.all_to_all_single.  The sorted id list is already
        grouped by owner (owners hold contiguous id ranges), so the send buffers are slices of it.
        Split sizes have to be known on the host: this route synchronises once per lookup group."""
        import torch.distributed as dist
        shard = opt.shard
        dev, G, W = shard.device, shard.world, shard.width
        nu = int(self.n_unique[0].item())
        edges = torch.arange(G + 1, device=dev, dtype=torch.int64) * shard.S
        cut = torch.searchsorted(self.uniq[:nu].contiguous(), edges)
        send_counts = (cut[1:] - cut[:-1])
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=opt._group)
        self.send_counts, self.recv_counts = send_counts.tolist(), recv_counts.tolist()
        n_recv = sum(self.recv_counts)
        self.recv_ids = torch.empty(n_recv, dtype=torch.int64, device=dev)
        dist.all_to_all_single(self.recv_ids, self.uniq[:nu].contiguous(), self.recv_counts, self.send_counts,
                               group=opt._group)
        rows = torch.empty(n_recv, W, dtype=torch.float32, device=dev)
        if n_recv:
            local = (self.recv_ids - shard.base).contiguous()
            _lib.check(_lib.lib().smore_gather_rows(shard.table.data_ptr(), local.data_ptr(), shard.S, rows.data_ptr(),
                                                    n_recv, W, _stream_ptr(dev)), "smore_gather_rows")
        dist.all_to_all_single(self.staging[:nu], rows, self.send_counts, self.recv_counts, group=opt._group)
        self.n_sent = nu

    def adopt(self, lookups):
        off = 0
        for lk in lookups:
            lk.offset, lk.plan = off, self
            off += lk.n
        self.lookups = list(lookups)

    def refresh(self, opt):
        """Pull again the rows whose owners updated them after (or while) they were fetched."""
        shard = opt.shard
        with torch.cuda.device(shard.device), _lib.timed("refresh_rows"):
            _lib.check(_lib.lib().smore_refresh_rows(shard.d_shard_ptrs.data_ptr(), shard.d_dirty_ptrs.data_ptr(),
                                                     shard.world, shard.S, self.uniq.data_ptr(),
                                                     self.n_unique.data_ptr(), self.n, shard.width,
                                                     self.staging.data_ptr(), shard.bitmap_scratch.data_ptr(),
                                                     _stream_ptr(shard.device)), "smore_refresh_rows")

    def slot_of(self, lookup):
        return self.slot[lookup.offset:lookup.offset + lookup.n]

    def slot64_of(self, lookup):
        return self.slot64[lookup.offset:lookup.offset + lookup.n]


class RemoteRows(LazyRows):
    """Candidate rows of a sharded table that never come to this rank: a distance op on them is
    computed by the rows' owners (ShardedAdamOptimizer.remote_dist)."""

    remote = True

    def _reshaped(self, shape):
        return RemoteRows(self.owner, self.lookup, shape)

    def materialize(self):
        raise _lib.SmoreError("remotely scored rows are not brought to this rank; look them up under another name "
                              "to use them as a tensor")


class _RemoteDistFunc(torch.autograd.Function):
    """A distance between this rank's queries and candidate rows that stay with their owners.  Both
    passes are collective over the ranks of the shard group: publish, barrier, every owner's share
    of the work, barrier, collect."""

    @staticmethod
    def forward(ctx, opt, name, dummy, first, second, n_queries, per_query, out_shape):
        opt.remote_publish(name, first, second, n_queries, per_query)
        opt.barrier()
        opt.remote_owner_forward()
        opt.barrier()
        outs = opt.remote_collect_forward(out_shape)
        ctx.opt, ctx.two = opt, second is not None
        return outs if len(outs) > 1 else outs[0]

    @staticmethod
    def backward(ctx, *gouts):
        opt = ctx.opt
        opt.remote_publish_upstream(gouts)
        opt.barrier()
        opt.remote_owner_backward()
        opt.barrier()
        g_first, g_second = opt.remote_collect_backward()
        return None, None, None, g_first, g_second if ctx.two else None, None, None, None


class ShardedAdamOptimizer(EmbeddingOptimizer):
    """EmbeddingOptimizer over a ShardedTable.  `barrier` is a callable that orders the ranks on the
    current stream (default: a one-element NCCL all-reduce); in the single-process emulation it is a
    no-op and the caller runs each phase for all ranks before the next."""

    opt_name = "adam"
    state_names = ()

    @classmethod
    def prepare_embed(cls, args, optim_mode, embed, fn_register):
        pass

    def __init__(self, shard, lazy_names=("negative_entity", "positive_entity"), barrier=None, group=None,
                 exchange="p2p", remote_names=("negative_entity",), early_owner_plan=False):
        """exchange: "p2p" - rows and row gradients are read straight from the peers' memory by this
        library's kernels (the shard must be connected: ShardGroup.from_process_group / emulated);
        "nccl" - the fallback for boxes without peer-mapped memory: the same two exchanges as
        torch.distributed.all_to_all_single calls on owner-bucketed id / row buffers, followed by the
        same owner-side de-duplication and update kernels reading the received blocks.  The fallback
        synchronises with the host for its split sizes, does not prefetch, and needs every rank to make
        the same number of lookup groups per step (each group is a collective)."""
        if exchange not in ("p2p", "nccl"):
            raise ValueError("exchange must be 'p2p' or 'nccl'")
        self.exchange = exchange
        self.shard = shard
        self.table = shard.table          # local shard: device / dtype / width of the rows
        self.squeeze = shard.squeeze
        self.lazy_names = tuple(lazy_names)
        self.training = True
        self.dummy_tensor = torch.nn.Parameter(torch.zeros(1, 1, device=shard.device))
        self.step = 0
        self.parity = 0                   # arena of the step in progress
        self._ws = None
        self._prefetch_ws = None
        self._owner_ws = None
        self._prefetched = None           # (plan, done_event, id tensors) being prepared for the next step
        self._ready = None                # the same, prepared during the previous step for this one
        self._prefetch_stream = None
        self._prefetch_buffers = [None, None]   # per arena; a buffer is reused two steps later
        self._group = group
        self._plans = []
        if barrier is None:
            import torch.distributed as dist
            flag = torch.zeros(1, device=shard.device)

            def barrier():
                dist.all_reduce(flag, group=group)
        self.barrier = barrier
        lay = shard.layout
        self._caps = (ctypes.c_int32 * len(lay.plan_caps))(*lay.plan_caps)
        n_in = shard.world * lay.span
        dev = shard.device
        self._in_ids = torch.empty(n_in, dtype=torch.int64, device=dev)
        self._runs = torch.zeros(80, dtype=torch.int32, device=dev)     # SMORE_SHARD_RUNS_INTS
        self._o_uniq = torch.empty(n_in, dtype=torch.int64, device=dev)
        self._o_slot = torch.empty(n_in, dtype=torch.int32, device=dev)
        self._o_counts = torch.empty(n_in, dtype=torch.int32, device=dev)
        self._o_src = torch.empty(n_in, dtype=torch.int32, device=dev)
        self._o_nuniq = torch.zeros(2, dtype=torch.int32, device=dev)
        self._started = False
        self.remote_names = tuple(remote_names) if shard.remote is not None else ()
        # early_owner_plan: a promise that no rank looks up rows after the forward pass of the remotely
        # scored op in a step (the reference's model makes all its lookups before it scores,
        # kg_reasoning.py:270-310).  The owners then de-duplicate the step's rows on a side stream while
        # the scores are computed, instead of at the start of the backward pass.
        self.early_owner_plan = bool(early_owner_plan)
        self._plan_stream = None
        self._r_op = None
        if shard.remote is not None:
            if exchange != "p2p":
                raise ValueError("owner-side scoring reads the peers' memory: exchange must be 'p2p'")
            self._init_remote()
        self.zero_grad()

    def _init_remote(self):
        """Owner-side buffers of the remote scoring: compact arrays over the pairs this shard may
        receive, followed by the lists' runs (ids, slots, counts), and the gradient rows of the
        shard's touched rows."""
        sh, spec = self.shard, self.shard.remote
        dev, G, W = sh.device, sh.world, sh.width
        cap = spec.owner_pairs or (spec.pairs if G == 1 else min(G * spec.pairs, 2 * spec.pairs))
        n_tot = cap + G * sh.layout.span
        QD = G * spec.queries * spec.dim
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
        f32 = lambda *shape: torch.empty(*shape, dtype=torch.float32, device=dev)
        self._r_cap, self._r_total = cap, n_tot
        self._r_rows = torch.zeros(n_tot, dtype=torch.int64, device=dev)
        self._r_pos, self._r_seg, self._r_nsel = i32(cap), i32(G * spec.queries * 2), i32(2)
        self._r_queries = [f32(QD), f32(QD)]
        self._r_uniq = torch.zeros(n_tot, dtype=torch.int64, device=dev)
        self._r_slot, self._r_counts, self._r_nuniq = i32(n_tot), i32(n_tot), i32(2)
        self._r_g = f32(n_tot, W)

    # ---- lookups ----------------------------------------------------------------------------------
    def _workspace(self, which):
        if getattr(self, which) is None:
            nbytes = _lib.lib().smore_unique_rows_workspace_bytes(self.shard.n_rows_total)
            setattr(self, which, torch.empty(nbytes, dtype=torch.uint8, device=self.shard.device))
        return getattr(self, which)

    def zero_grad(self):
        """Begins a step: the step uses the other arena than the previous one."""
        self.n_fwd = 0
        self._pending = []
        self._drop_plans()
        self.grad_list = []
        self.has_grad_list = []
        self._fused_lr = None
        self._step_advanced = False
        self._r_op = None
        if self._started:
            self.parity ^= 1
        self._started = True
        nu = self.shard.nuniq_all[self.parity]
        self._ready, self._prefetched = self._prefetched, None
        if self._ready is not None and self._ready[0].parity == self.parity:
            # list 0 of this arena was already filled by the prefetch (apply_grad waited for it);
            # the others start unused
            nu[2:].zero_()
        else:
            # no list of this rank is in use until a plan of this step fills it (owners read these
            # counters only after the step's first barrier)
            self._ready = None
            nu.zero_()

    def reset_prefetch(self, next_parity=None):
        """Forget anything prepared for coming steps.  `next_parity` (0 or 1) chooses the arena the
        next step will use, for hosts that replay per-arena CUDA graphs and must line them up."""
        self._prefetched = self._ready = None
        if next_parity is not None:
            self.parity = int(next_parity) ^ 1     # zero_grad flips it

    def prefetch(self, id_tensors, after=None):
        """Prepare the NEXT step's first lookup group now, on a side stream: `id_tensors` are the
        device id tensors that step will look up, in order, up to and including the first lookup
        whose rows are needed (e.g. positives, negatives, first anchors).  Call it after this step's
        zero_grad() and pass the same tensors, unchanged, to the lookups of the next step; a step
        that looks up anything else simply ignores what was prepared.  `after` is an event that
        marks the id tensors as written, if another stream than the current one produces them."""
        dev = self.shard.device
        if self.exchange == "nccl":
            return          # the fallback pulls every step's rows when they are first needed
        if any(t.device != dev or t.dtype != torch.int64 for t in id_tensors):
            raise _lib.SmoreError("prefetch takes int64 id tensors that already live on the shard's device")
        if self._prefetch_stream is None:
            self._prefetch_stream = torch.cuda.Stream(dev)
        main = torch.cuda.current_stream(dev)
        ready = torch.cuda.Event()
        ready.record(main)                       # everything before this step (the last update) is done
        side = self._prefetch_stream
        side.wait_event(ready)
        if after is not None:
            side.wait_event(after)
        target = self.parity ^ 1
        if self._prefetch_buffers[target] is None:
            self._prefetch_buffers[target] = _PlanBuffers(self.shard.layout.plan_caps[0], self.shard.width, dev)
        with torch.cuda.stream(side):
            plan = _ShardedPlan(self, id_tensors, 0, target, self._workspace("_prefetch_ws"),
                                self._prefetch_buffers[target])
            done = torch.cuda.Event()
            done.record(side)
        # the raw tensors stay referenced so that their addresses cannot be reused before the match
        self._prefetched = (plan, done, [_id_key(t) for t in id_tensors], list(id_tensors))

    def forward(self, indices, name=None):
        if indices is None:
            raise _lib.SmoreError("a sharded table cannot be returned whole; rank it shard by shard")
        idx = self._device_indices(indices)
        lookup = _Lookup(idx, name, self.n_fwd)
        lookup.key = _id_key(indices)
        self.n_fwd += 1
        if name is not None and name in self.remote_names and self.training and torch.is_grad_enabled():
            # scored where the rows live: nothing is fetched, the ids are published for the owners
            if self._r_op is not None:
                raise _lib.SmoreError("one remotely scored lookup per step")
            if lookup.n > self.shard.remote.pairs:
                raise _lib.SmoreError("%d candidate ids, the remote block holds %d (RemoteSpec.pairs)"
                                      % (lookup.n, self.shard.remote.pairs))
            self.shard.r_ids[:lookup.n].copy_(idx)
            self._r_op = {"lookup": lookup, "stage": "ids"}
            return RemoteRows(self, lookup, (lookup.n, self.shard.width))
        self._pending.append(lookup)
        if name is not None and name in self.lazy_names:
            return LazyRows(self, lookup, (lookup.n, self.shard.width))
        if self.training and torch.is_grad_enabled():
            out = _EmbedLookupFunc.apply(self, self.dummy_tensor, lookup)
        else:
            out = self._gather_lookup(lookup)
        out.job_handle = _DUMMY_JOB
        return out

    def _device_indices(self, indices):
        idx = indices.reshape(-1)
        if idx.dtype != torch.int64:
            idx = idx.long()
        if idx.device != self.shard.device:
            idx = idx.to(self.shard.device, non_blocking=True)
        return idx.contiguous()

    def _matches_prefetch(self, lookups):
        if self._ready is None:
            return False
        keys = self._ready[2]
        return len(keys) == len(lookups) and all(k == lk.key for k, lk in zip(keys, lookups))

    def plan_for(self, lookup):
        if lookup.plan is None:
            index = len(self._plans)
            if index >= len(self.shard.layout.plan_caps):
                raise _lib.SmoreError("more than %d lookup groups in one step" % len(self.shard.layout.plan_caps))
            if index == 0 and self._matches_prefetch(self._pending):
                plan = self._ready[0]
                plan.refresh(self)          # rows their owners updated since the prefetch began
            else:
                # (a step that does not look up what was prefetched rebuilds list 0 here)
                plan = _ShardedPlan(self, [lk.idx for lk in self._pending], index, self.parity,
                                    self._workspace("_ws"))
            if index == 0:
                self._ready = None
            plan.adopt(self._pending)
            self._plans.append(plan)
            self._pending = []
        return lookup.plan

    def rows_operands(self, lookup):
        plan = self.plan_for(lookup)
        return plan.staging, plan.slot64_of(lookup)

    def _gather_lookup(self, lookup):
        plan = self.plan_for(lookup)
        out = torch.empty(lookup.n, self.shard.width, dtype=torch.float32, device=self.shard.device)
        with torch.cuda.device(self.shard.device):
            _lib.check(_lib.lib().smore_gather_rows(plan.staging.data_ptr(), plan.slot64_of(lookup).data_ptr(),
                                                    plan.staging.shape[0], out.data_ptr(), lookup.n,
                                                    self.shard.width,
                                                    _stream_ptr(self.shard.device)), "smore_gather_rows")
        return out

    def _materialize(self, lookup):
        return _EmbedLookupFunc.apply(self, self.dummy_tensor, lookup)

    # ---- owner-side scoring -----------------------------------------------------------------------
    def announce_lr(self, lr):
        """The learning rate apply_grad(lr) will get; needed before the backward pass of a remotely
        scored lookup, whose owners apply the row updates inside that pass."""
        self._fused_lr = float(lr)
        if getattr(self, "_step_dev", None) is not None and not self._step_advanced:
            self._advance_device_step(lr)
            self._step_advanced = True

    def fused_update_args(self, lookup, plan):
        return None         # staged rows are copies: nothing to update in place on the requester

    def remote_dist(self, name, rows, first, second):
        """name: a distance of ext_ops ("box_both" included) between `rows` (a RemoteRows handle viewed
        as [B, K, width]) and query operands [B, 1, dim] or, for union queries, [B, 2, 1, dim].  Every
        rank of the shard group must make this call in the same steps, with the same distance, the
        same number of queries, the same K and the same number of branches."""
        B, K, width = rows.as_3d()
        if self._r_op is None or self._r_op["lookup"] is not rows.lookup or self._r_op["stage"] != "ids":
            raise _lib.SmoreError("a remotely scored lookup takes exactly one distance op per step")
        if first.dim() == 4:
            if first.shape[0] != B or first.shape[2] != 1 or first.shape[1] not in (1, 2):
                raise ValueError("%s: union operands must be [B, U, 1, dim] with U = 1 or 2" % name)
            branches = first.shape[1]          # every branch is scored against the query's candidates
            out_shape = (B, branches, K)
        elif first.dim() == 3 and first.shape[0] == B and first.shape[1] == 1:
            branches, out_shape = 1, (B, K)
        else:
            raise ValueError("%s: remotely scored rows take one candidate list per query" % name)
        n_queries = B
        if n_queries * branches * K > self.shard.remote.pairs:
            raise _lib.SmoreError("%d scores, the remote block holds %d (RemoteSpec.pairs)"
                                  % (n_queries * branches * K, self.shard.remote.pairs))
        dim = first.shape[-1]
        if dim != self.shard.remote.dim or n_queries * branches > self.shard.remote.queries:
            raise _lib.SmoreError("queries [%d, %d] do not fit the remote block (RemoteSpec queries=%d, dim=%d)"
                                  % (n_queries * branches, dim, self.shard.remote.queries, self.shard.remote.dim))
        if self.early_owner_plan and self._pending:
            self.plan_for(self._pending[0])      # every id list of this rank is published before the op's first barrier
        flat = lambda t: None if t is None else t.reshape(n_queries * branches, dim).contiguous()
        return _RemoteDistFunc.apply(self, name, self.dummy_tensor, flat(first), flat(second), n_queries, K, out_shape)

    def remote_publish(self, name, first, second, n_queries, per_query):
        """first / second: [n_queries * branches, dim] (the branches of a query next to each other)."""
        sh, op = self.shard, self._r_op
        branches = first.shape[0] // n_queries
        op.update(name=name, dist_id=_lib.BOX_BOTH_ID if name == "box_both" else _lib.DIST_IDS[name],
                  n_out=2 if name == "box_both" else 1, two=second is not None, nq=n_queries, K=per_query,
                  branches=branches, dim=first.shape[1], stage="published")
        sh.r_desc[0].fill_(n_queries)
        sh.r_desc[1].fill_(per_query)
        sh.r_desc[2].fill_(branches)
        n = n_queries * branches * op["dim"]
        sh.r_queries[0][:n].copy_(first.reshape(-1))
        if second is not None:
            sh.r_queries[1][:n].copy_(second.reshape(-1))
        for i in range(op["n_out"]):        # a pair no owner claims (an id outside the table) reads NaN
            sh.r_results[i][:n_queries * branches * per_query].fill_(float("nan"))

    def remote_owner_forward(self):
        sh, spec, op = self.shard, self.shard.remote, self._r_op
        L, dev = _lib.lib(), self.shard.device
        st = _stream_ptr(dev)
        G, Q, P = sh.world, spec.queries, spec.pairs
        ptr = lambda t: None if t is None else t.data_ptr()
        second_all = self._r_queries[1] if op["two"] else None
        with torch.cuda.device(dev):
            with _lib.timed("owner_select"):
                _lib.check(L.smore_owner_select_pairs(sh.d_r_ids.data_ptr(), sh.d_r_desc.data_ptr(), G, Q, P, op["nq"],
                                                      op["K"], op["branches"], sh.base, max(sh.S, 1), self._r_cap,
                                                      self._r_rows.data_ptr(),
                                                      self._r_pos.data_ptr(), self._r_seg.data_ptr(),
                                                      self._r_nsel.data_ptr(), st), "smore_owner_select_pairs")
                _lib.check(L.smore_owner_gather_queries(sh.d_r_queries[0].data_ptr(),
                                                        sh.d_r_queries[1].data_ptr() if op["two"] else None,
                                                        sh.d_r_desc.data_ptr(), G, Q, P, op["nq"], op["K"],
                                                        op["branches"], op["dim"], sh.rank,
                                                        self._r_queries[0].data_ptr(), ptr(second_all), st),
                           "smore_owner_gather_queries")
            with _lib.timed("owner_forward"):
                # every result goes straight to its position in the requesting rank's result arrays
                _lib.check(L.smore_rows_forward_ragged(op["dist_id"], sh.table.data_ptr(), self._r_rows.data_ptr(),
                                                       max(sh.S, 1), self._r_queries[0].data_ptr(), ptr(second_all),
                                                       self._r_seg.data_ptr(), G * Q, op["dim"], None, None,
                                                       self._r_pos.data_ptr(), Q, sh.d_r_results[0].data_ptr(),
                                                       sh.d_r_results[1].data_ptr() if op["n_out"] == 2 else None,
                                                       op["branches"], op["K"], st),
                           "smore_rows_forward_ragged")
        op["stage"] = "scored"
        if self.early_owner_plan:
            # (forked behind the selection; the backward pass joins it)
            if self._plan_stream is None:
                self._plan_stream = torch.cuda.Stream(dev)
            main, side = torch.cuda.current_stream(dev), self._plan_stream
            selected = torch.cuda.Event()
            selected.record(main)
            side.wait_event(selected)
            with torch.cuda.stream(side):
                self._owner_plan()
                op["plan_done"] = torch.cuda.Event()
                op["plan_done"].record(side)
            op["plans_seen"] = len(self._plans)

    def remote_collect_forward(self, out_shape):
        op = self._r_op
        n = op["nq"] * op["branches"] * op["K"]
        return tuple(self.shard.r_results[i][:n].view(out_shape).clone() for i in range(op["n_out"]))

    def remote_publish_upstream(self, gouts):
        op = self._r_op
        if op is None or op["stage"] != "scored":
            raise _lib.SmoreError("backward of a remotely scored lookup without its forward in this step")
        if self._fused_lr is None:
            raise _lib.SmoreError("call announce_lr(lr) before the backward pass: the owners of remotely scored rows "
                                  "update them inside it")
        n = op["nq"] * op["branches"] * op["K"]
        for i in range(op["n_out"]):
            self.shard.r_upstream[i][:n].copy_(gouts[i].reshape(-1))

    def _owner_plan(self):
        """The selected pairs' rows and the runs of the ranks' id lists (positives, anchors),
        de-duplicated together: one slot per distinct row of this shard touched in the step; the rows
        several contributions share are zeroed in the local gradient buffer.  On the current stream."""
        sh, lay = self.shard, self.shard.layout
        L, dev = _lib.lib(), self.shard.device
        st = _stream_ptr(dev)
        if self._owner_ws is None:
            nbytes = L.smore_shard_owner_plan_workspace_bytes(max(sh.S, 1))
            self._owner_ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        par = self.parity
        with torch.cuda.device(dev), _lib.timed("shard_collect"):
            _lib.check(L.smore_owner_plan(sh.d_uniq_ptrs[par].data_ptr(), sh.d_nuniq_ptrs[par].data_ptr(), sh.world,
                                          len(lay.plan_caps), self._caps, sh.base, max(sh.S, 1), self._r_total,
                                          self._r_rows.data_ptr(), self._runs.data_ptr(), self._r_uniq.data_ptr(),
                                          self._r_slot.data_ptr(), self._r_counts.data_ptr(), self._r_nuniq.data_ptr(),
                                          sh.dirty.data_ptr(), self._owner_ws.data_ptr(), self._owner_ws.numel(),
                                          self._r_nsel.data_ptr(), self._r_cap, st), "smore_owner_plan")
            _lib.check(L.smore_zero_shared_rows(self._r_g.data_ptr(), self._r_counts.data_ptr(),
                                                self._r_nuniq.data_ptr(), self._r_total, sh.width, st),
                       "smore_zero_shared_rows")

    def remote_owner_backward(self):
        sh, spec, op = self.shard, self.shard.remote, self._r_op
        L, dev, lay = _lib.lib(), self.shard.device, self.shard.layout
        st = _stream_ptr(dev)
        G, Q, W, par = sh.world, spec.queries, sh.width, self.parity
        ptr = lambda t: None if t is None else t.data_ptr()
        second_all = self._r_queries[1] if op["two"] else None
        dev_step = getattr(self, "_step_dev", None) is not None
        if self.early_owner_plan:
            if len(self._plans) != op.get("plans_seen") or self._pending:
                raise _lib.SmoreError("early_owner_plan: this rank looked up rows after the forward pass of the remotely "
                                      "scored op; construct the optimizer without early_owner_plan")
            torch.cuda.current_stream(dev).wait_event(op["plan_done"])
        else:
            self._owner_plan()
        with torch.cuda.device(dev):
            _lib.note("n_unique_owner", self._r_nuniq[0])
            if _lib._timer is not None:     # (timing passes only: rows with one contribution in the step)
                live = torch.arange(self._r_total, device=dev) < self._r_nuniq[0]
                _lib.note("n_single", ((self._r_counts == 1) & live).sum())
            with _lib.timed("owner_backward"):
                # (each pair's upstream gradient is read from its position in the requesting rank's arrays)
                _lib.check(L.smore_rows_backward_fused_adam_ragged(
                    op["dist_id"], None, None, sh.table.data_ptr(), self._r_rows.data_ptr(),
                    max(sh.S, 1), self._r_queries[0].data_ptr(), ptr(second_all), self._r_seg.data_ptr(), G * Q,
                    self._r_slot.data_ptr(), self._r_counts.data_ptr(), self._r_g.data_ptr(), sh.r_partial[0].data_ptr(),
                    sh.r_partial[1].data_ptr() if op["two"] else None, op["dim"], sh.m.data_ptr(), sh.v.data_ptr(),
                    self._r_uniq.data_ptr(), self._fused_lr, 0.9, 0.999, eps, 1 if dev_step else int(self.step) + 1,
                    self._step_scalars.data_ptr() if dev_step else None, self._r_pos.data_ptr(), Q,
                    sh.d_r_upstream[0].data_ptr(), sh.d_r_upstream[1].data_ptr() if op["n_out"] == 2 else None,
                    op["branches"], op["K"], st), "smore_rows_backward_fused_adam_ragged")
        op["stage"] = "differentiated"

    def remote_collect_backward(self):
        sh, spec, op = self.shard, self.shard.remote, self._r_op
        L, dev = _lib.lib(), self.shard.device
        outs = []
        with torch.cuda.device(dev), _lib.timed("owner_sum_query_grads"):
            for i in range(2 if op["two"] else 1):
                g = torch.empty(op["nq"] * op["branches"], op["dim"], dtype=torch.float32, device=dev)
                _lib.check(L.smore_owner_sum_query_grads(sh.d_r_partial[i].data_ptr(), sh.world, sh.rank, spec.queries,
                                                         op["nq"] * op["branches"], op["dim"], g.data_ptr(),
                                                         _stream_ptr(dev)),
                           "smore_owner_sum_query_grads")
                outs.append(g)
        return outs[0], outs[1] if op["two"] else None

    def _apply_grad_remote(self, lr, ranks_ordered=False):
        """The end of a step whose candidate rows were scored by their owners: the rows those pairs
        alone touch are already updated; add the gradient rows that came back through the ranks'
        lists (positives, anchors) and update what is left."""
        sh, lay = self.shard, self.shard.layout
        L, dev = _lib.lib(), self.shard.device
        if float(lr) != self._fused_lr:
            raise _lib.SmoreError("apply_grad(lr=%r) after announce_lr(%r)" % (lr, self._fused_lr))
        if self.early_owner_plan and len(self._plans) != self._r_op.get("plans_seen"):
            raise _lib.SmoreError("early_owner_plan: this rank looked up rows after the forward pass of the remotely "
                                  "scored op; construct the optimizer without early_owner_plan")
        if not ranks_ordered:
            self.barrier()          # every rank's gradient rows are complete
        with torch.cuda.device(dev):
            with _lib.timed("owner_add_list_rows"):
                _lib.check(L.smore_owner_add_list_rows(sh.d_grad_ptrs[self.parity].data_ptr(), self._runs.data_ptr(),
                                                       sh.world * len(lay.plan_caps), self._r_slot.data_ptr(),
                                                       self._r_counts.data_ptr(), self._r_g.data_ptr(), sh.width,
                                                       lay.span, _stream_ptr(dev)), "smore_owner_add_list_rows")
        self._run_update("adam", sh.m, sh.v, self._r_uniq, self._r_g, self._r_nuniq, self._r_total, lr)
        self.barrier()              # every shard is updated; this step's arena may be overwritten
        if self._prefetched is not None:
            torch.cuda.current_stream(dev).wait_event(self._prefetched[1])
        self._drop_plans()

    # ---- the update ---------------------------------------------------------------------------------
    def _neutralise_unused_lookups(self):
        """A lookup that never received a gradient must not leave uninitialised rows in the arena:
        give it a zero gradient (its rows then see an Adam step with g = 0)."""
        for plan in self._plans:
            for lk in plan.lookups:
                if not lk.received:
                    zeros = torch.zeros(lk.n, self.shard.width, device=self.shard.device)
                    self.accumulate_grad(lk, zeros)
        if self._pending:           # looked up but never used: no plan, nothing published
            self._pending = []

    def _apply_grad_all_to_all(self, lr):
        """Gradient return of the fallback: every plan's gradient rows go to their owners (the split of
        the forward exchange, reversed); the received (ids, gradient rows) blocks then serve as the
        lists the owner-side kernels read - one per (rank, plan), here in local memory."""
        import torch.distributed as dist
        sh = self.shard
        dev, G, W = sh.device, sh.world, sh.width
        P = len(sh.layout.plan_caps)
        n_plans = torch.tensor([len(self._plans)], device=dev)
        hi = n_plans.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self._group)
        if int(hi.item()) != len(self._plans):
            raise _lib.SmoreError("the all-to-all exchange needs the same number of lookup groups on every rank "
                                  "in a step (%d here, %d elsewhere)" % (len(self._plans), int(hi.item())))
        ids_ptr, cnt, grad_ptr, keep = [0] * (G * P), [0] * (G * P), [0] * (G * P), []
        for plan in self._plans:
            recv = torch.empty(sum(plan.recv_counts), W, dtype=torch.float32, device=dev)
            dist.all_to_all_single(recv, plan.g_rows[:plan.n_sent].contiguous(), plan.recv_counts, plan.send_counts,
                                   group=self._group)
            keep += [recv, plan.recv_ids]
            off = 0
            for g in range(G):
                l = g * P + plan.index
                ids_ptr[l] = plan.recv_ids.data_ptr() + off * 8
                grad_ptr[l] = recv.data_ptr() + off * W * 4
                cnt[l] = plan.recv_counts[g]
                off += plan.recv_counts[g]
        counts = torch.tensor(cnt, dtype=torch.int32, device=dev)
        tables = {"ids": torch.tensor(ids_ptr, dtype=torch.int64, device=dev),
                  "nuniq": torch.tensor([counts.data_ptr() + 4 * l for l in range(G * P)], dtype=torch.int64, device=dev),
                  "grads": torch.tensor(grad_ptr, dtype=torch.int64, device=dev)}
        self.owner_update(lr, tables)
        del keep, counts
        self._drop_plans()

    def apply_grad(self, lr, ranks_ordered=False):
        """ranks_ordered: the caller has already run a collective over the shard group on this stream
        after the backward pass (e.g. the all-reduce of the dense gradients), so every rank's gradient
        rows are known to be complete and the first barrier of the update is left out.  (Not possible in
        a step with a lookup that received no gradient: its rows are only zeroed here.)"""
        if ranks_ordered and any(not lk.received for plan in self._plans for lk in plan.lookups):
            raise _lib.SmoreError("apply_grad(ranks_ordered=True): a lookup of this step received no gradient before "
                                  "the collective that ordered the ranks; call apply_grad(lr) instead")
        self.step += 1
        self._neutralise_unused_lookups()
        if self._r_op is not None:
            if self._r_op["stage"] != "differentiated":
                raise _lib.SmoreError("a remotely scored lookup must be used by one distance op and differentiated "
                                      "before apply_grad (stage: %s)" % self._r_op["stage"])
            return self._apply_grad_remote(lr, ranks_ordered)
        if self.exchange == "nccl":
            return self._apply_grad_all_to_all(lr)
        if not ranks_ordered:
            self.barrier()          # every rank's id lists and gradient rows are complete
        self.owner_update(lr)
        self.barrier()              # every shard is updated; this step's arena may be overwritten
        if self._prefetched is not None:
            # the copy prepared for the next step joins the step's stream here (inside a CUDA graph
            # capture a forked stream has to re-join before the capture ends)
            torch.cuda.current_stream(self.shard.device).wait_event(self._prefetched[1])
        self._drop_plans()

    def owner_update(self, lr, tables=None):
        """`tables`: device arrays of the lists' id / length / gradient addresses; default: the peers'
        arenas of the step in progress."""
        sh = self.shard
        lay = sh.layout
        L = _lib.lib()
        dev = sh.device
        st = _stream_ptr(dev)
        G, P = sh.world, len(lay.plan_caps)
        n_in = G * lay.span
        par = self.parity
        if tables is None:
            tables = {"ids": sh.d_uniq_ptrs[par], "nuniq": sh.d_nuniq_ptrs[par], "grads": sh.d_grad_ptrs[par]}
        if self._owner_ws is None:
            nbytes = L.smore_shard_owner_plan_workspace_bytes(max(sh.S, 1))
            self._owner_ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            with _lib.timed("shard_collect"):
                # every list's run of ids in this shard's range -> compact local ids -> distinct rows,
                # one source position per row, the updated-rows bitmap for the next step's refresh
                _lib.check(L.smore_shard_owner_plan(
                    tables["ids"].data_ptr(), tables["nuniq"].data_ptr(), G, P, self._caps, sh.base,
                    max(sh.S, 1), n_in, self._in_ids.data_ptr(), self._runs.data_ptr(), self._o_uniq.data_ptr(),
                    self._o_slot.data_ptr(), self._o_counts.data_ptr(), self._o_src.data_ptr(),
                    self._o_nuniq.data_ptr(), sh.dirty.data_ptr(), self._owner_ws.data_ptr(),
                    self._owner_ws.numel(), st), "smore_shard_owner_plan")
            _lib.note("n_unique_owner", self._o_nuniq[0])
            dev_step = getattr(self, "_step_dev", None) is not None
            if dev_step:
                self._advance_device_step(lr)
            with _lib.timed("shard_reduce_update"):
                if dev_step:
                    _lib.check(L.smore_shard_reduce_update_rows_dev(
                        sh.table.data_ptr(), sh.m.data_ptr(), sh.v.data_ptr(), self._o_uniq.data_ptr(),
                        self._o_counts.data_ptr(), self._o_src.data_ptr(), self._o_nuniq.data_ptr(), n_in,
                        tables["grads"].data_ptr(), self._in_ids.data_ptr(), self._runs.data_ptr(), G * P,
                        sh.width, float(lr), 0.9, 0.999, eps, self._step_scalars.data_ptr(),
                        int(self.squeeze), st), "smore_shard_reduce_update_rows_dev")
                    return
                _lib.check(L.smore_shard_reduce_update_rows(
                    sh.table.data_ptr(), sh.m.data_ptr(), sh.v.data_ptr(), self._o_uniq.data_ptr(),
                    self._o_counts.data_ptr(), self._o_src.data_ptr(), self._o_nuniq.data_ptr(), n_in,
                    tables["grads"].data_ptr(), self._in_ids.data_ptr(), self._runs.data_ptr(), G * P,
                    sh.width, float(lr), 0.9, 0.999, eps, int(self.step), int(self.squeeze), st),
                    "smore_shard_reduce_update_rows")

    def update_step(self, indices, inverse_indices, grad, lr):
        raise _lib.SmoreError("update_step with caller-merged gradients is not defined for a sharded table")


class ShardGroup(object):
    """Convenience constructors."""

    @staticmethod
    def from_process_group(n_rows_total, width, plan_caps, squeeze=True, group=None, device=None, exchange="p2p",
                           remote=None):
        """exchange="p2p": blocks from the symmetric-memory allocator, mapped into every rank;
        exchange="nccl": plain local blocks (use ShardedAdamOptimizer(shard, exchange="nccl")).
        remote: a RemoteSpec to set up owner-side scoring (p2p only)."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        if remote is not None and exchange != "p2p":
            raise ValueError("owner-side scoring reads the peers' memory: exchange must be 'p2p'")
        shard = ShardedTable(n_rows_total, width, rank, world, device, plan_caps, squeeze, symmetric=exchange == "p2p",
                             remote=remote)
        if exchange == "p2p":
            shard.connect_processes(group)
        return shard

    @staticmethod
    def emulated(world, n_rows_total, width, plan_caps, squeeze=True, device="cuda:0", remote=None):
        """`world` shards in this process on one GPU, wired to each other by raw pointers."""
        shards = [ShardedTable(n_rows_total, width, r, world, device, plan_caps, squeeze, remote=remote)
                  for r in range(world)]
        tables = [s._table_block.ptr for s in shards]
        arenas = [[s._arena_blocks[par].ptr for s in shards] for par in range(2)]
        dirty = [s._dirty_block.ptr for s in shards]
        remotes = [s._remote_block.ptr for s in shards] if remote is not None else None
        for s in shards:
            s.connect(tables, arenas, dirty, remotes)
        return shards
