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
            ranks' lists, de-duplicates them, and one kernel pulls the matching gradient rows,
            sums them in a fixed order and applies Adam to the shard
            (smore_shard_reduce_update_rows); a second barrier ends the step.

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


class ShardedTable(object):
    """The local shard (table + Adam state), the peer-visible arena, and the pointer tables."""

    def __init__(self, n_rows_total, width, rank, world, device, plan_caps, squeeze=True, symmetric=False):
        self.n_rows_total, self.width, self.rank, self.world = int(n_rows_total), int(width), rank, world
        self.device = torch.device(device)
        self.squeeze = bool(squeeze)
        self.S = shard_rows(n_rows_total, world)
        self.base = rank * self.S
        self.local_rows = max(0, min(self.S, n_rows_total - self.base))
        self.layout = ArenaLayout(plan_caps, width)
        self.symmetric = symmetric
        self._table_block = self._alloc(max(self.S, 1) * width * 4)
        self._arena_block = self._alloc(self.layout.nbytes)
        self.table = self._table_block.view(self.device, 0, (self.S, width), torch.float32)
        self.m = torch.zeros(self.S, width, device=self.device)
        self.v = torch.zeros(self.S, 1, device=self.device) if squeeze else torch.zeros(self.S, width, device=self.device)
        lay = self.layout
        self.nuniq = [self._arena_block.view(self.device, lay.nuniq_offset(p), (2,), torch.int32)
                      for p in range(len(lay.plan_caps))]
        self.nuniq_all = self._arena_block.view(self.device, 0, (MAX_PLANS * 2,), torch.int32)
        self.nuniq_all.zero_()
        self.ids = [self._arena_block.view(self.device, lay.ids_offset(p), (lay.plan_caps[p],), torch.int64)
                    for p in range(len(lay.plan_caps))]
        self.grads = [self._arena_block.view(self.device, lay.grads_offset(p), (lay.plan_caps[p], width), torch.float32)
                      for p in range(len(lay.plan_caps))]
        self.peer_table_ptrs = None   # filled by connect()
        self.peer_arena_ptrs = None
        self._handles = []

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

    def connect(self, table_ptrs, arena_ptrs):
        """Install the base pointers of every rank's shard and arena (this rank's own included)."""
        self.peer_table_ptrs, self.peer_arena_ptrs = list(table_ptrs), list(arena_ptrs)
        tabs = pointer_tables(self.layout, self.peer_arena_ptrs)
        dev = self.device
        self.d_shard_ptrs = torch.tensor(self.peer_table_ptrs, dtype=torch.int64, device=dev)
        self.d_uniq_ptrs = torch.tensor(tabs["ids"], dtype=torch.int64, device=dev)
        self.d_nuniq_ptrs = torch.tensor(tabs["nuniq"], dtype=torch.int64, device=dev)
        self.d_grad_ptrs = torch.tensor(tabs["grads"], dtype=torch.int64, device=dev)

    def connect_processes(self, group=None):
        """Map the other ranks' shard and arena blocks (symmetric-memory rendezvous over `group`)."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if not self.symmetric:
            raise _lib.SmoreError("connect_processes needs blocks from the symmetric-memory allocator")
        group = group if group is not None else dist.group.WORLD
        with torch.cuda.device(self.device):
            ht = symm_mem.rendezvous(self._table_block.tensor, group)
            ha = symm_mem.rendezvous(self._arena_block.tensor, group)
        self._handles = [ht, ha]
        table_ptrs, arena_ptrs = [int(p) for p in ht.buffer_ptrs], [int(p) for p in ha.buffer_ptrs]
        if table_ptrs[self.rank] != self._table_block.ptr or arena_ptrs[self.rank] != self._arena_block.ptr:
            raise _lib.SmoreError("symmetric-memory rendezvous returned a different address for the local block")
        self.connect(table_ptrs, arena_ptrs)

    def close(self):
        self._handles = []

    def init_uniform(self, lo, hi, seed):
        """Fill the shard as rows [base, base+S) of a table drawn uniform(lo, hi); the values depend
        on (seed, rank) only."""
        g = torch.Generator(device=self.device).manual_seed(seed * 1000003 + self.rank)
        self.table.uniform_(lo, hi, generator=g)


class _ShardedPlan(object):
    """One de-duplicated group of lookups of a rank: ids and gradients in the arena, rows staged."""

    def __init__(self, opt, lookups, index):
        shard = opt.shard
        dev = shard.device
        self.lookups, self.index = lookups, index
        off = 0
        for lk in lookups:
            lk.offset, lk.plan = off, self
            off += lk.n
        self.n = off
        cap = shard.layout.plan_caps[index]
        if self.n > cap:
            raise _lib.SmoreError("plan %d holds %d looked-up ids, its capacity is %d (plan_caps)" % (index, self.n, cap))
        self.idx_all = lookups[0].idx if len(lookups) == 1 else torch.cat([lk.idx for lk in lookups])
        self.uniq = shard.ids[index]
        self.n_unique = shard.nuniq[index]
        self.g_rows = shard.grads[index]
        self.slot = torch.empty(self.n, dtype=torch.int32, device=dev)
        self.counts = torch.empty(self.n, dtype=torch.int32, device=dev)
        self.staging = torch.empty(self.n, shard.width, dtype=torch.float32, device=dev)
        L = _lib.lib()
        ws = opt._unique_workspace()
        st = _stream_ptr(dev)
        with torch.cuda.device(dev):
            with _lib.timed("unique_rows"):
                _lib.check(L.smore_unique_rows(self.idx_all.data_ptr(), self.n, shard.n_rows_total,
                                               self.uniq.data_ptr(), self.slot.data_ptr(), self.counts.data_ptr(),
                                               self.n_unique.data_ptr(), ws.data_ptr(), ws.numel(), st),
                           "smore_unique_rows")
            with _lib.timed("fetch_rows"):
                _lib.check(L.smore_fetch_rows(shard.d_shard_ptrs.data_ptr(), shard.S, self.uniq.data_ptr(),
                                              self.n_unique.data_ptr(), self.n, shard.width, self.staging.data_ptr(),
                                              st), "smore_fetch_rows")
            _lib.check(L.smore_zero_shared_rows(self.g_rows.data_ptr(), self.counts.data_ptr(),
                                                self.n_unique.data_ptr(), self.n, shard.width, st),
                       "smore_zero_shared_rows")
        self.slot64 = self.slot.long()

    def slot_of(self, lookup):
        return self.slot[lookup.offset:lookup.offset + lookup.n]

    def slot64_of(self, lookup):
        return self.slot64[lookup.offset:lookup.offset + lookup.n]


class ShardedAdamOptimizer(EmbeddingOptimizer):
    """EmbeddingOptimizer over a ShardedTable.  `barrier` is a callable that orders the ranks on the
    current stream (default: a one-element NCCL all-reduce); in the single-process emulation it is a
    no-op and the caller runs each phase for all ranks before the next."""

    opt_name = "adam"
    state_names = ()

    @classmethod
    def prepare_embed(cls, args, optim_mode, embed, fn_register):
        pass

    def __init__(self, shard, lazy_names=("negative_entity", "positive_entity"), barrier=None, group=None):
        self.shard = shard
        self.table = shard.table          # local shard: device / dtype / width of the rows
        self.squeeze = shard.squeeze
        self.lazy_names = tuple(lazy_names)
        self.training = True
        self.dummy_tensor = torch.nn.Parameter(torch.zeros(1, 1, device=shard.device))
        self.step = 0
        self._ws = None
        self._owner_ws = None
        self._group = group
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
        self._in_bounds = torch.empty(shard.world * len(lay.plan_caps) * 2, dtype=torch.int32, device=dev)
        self._o_uniq = torch.empty(n_in, dtype=torch.int64, device=dev)
        self._o_slot = torch.empty(n_in, dtype=torch.int32, device=dev)
        self._o_counts = torch.empty(n_in, dtype=torch.int32, device=dev)
        self._o_src = torch.empty(n_in, dtype=torch.int32, device=dev)
        self._o_nuniq = torch.zeros(2, dtype=torch.int32, device=dev)
        self.zero_grad()

    # ---- lookups ----------------------------------------------------------------------------------
    def _unique_workspace(self):
        if self._ws is None:
            nbytes = _lib.lib().smore_unique_rows_workspace_bytes(self.shard.n_rows_total)
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=self.shard.device)
        return self._ws

    def zero_grad(self):
        self.n_fwd = 0
        self._pending = []
        self._drop_plans()
        self.grad_list = []
        self.has_grad_list = []
        # no list of this rank is in use until a plan of this step fills it (owners read these
        # counters only after the step's first barrier)
        self.shard.nuniq_all.zero_()

    def forward(self, indices, name=None):
        if indices is None:
            raise _lib.SmoreError("a sharded table cannot be returned whole; rank it shard by shard")
        idx = self._device_indices(indices)
        lookup = _Lookup(idx, name, self.n_fwd)
        self.n_fwd += 1
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

    def plan_for(self, lookup):
        if lookup.plan is None:
            index = len(self._plans)
            if index >= len(self.shard.layout.plan_caps):
                raise _lib.SmoreError("more than %d lookup groups in one step" % len(self.shard.layout.plan_caps))
            self._plans.append(_ShardedPlan(self, self._pending, index))
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
                                                    out.data_ptr(), lookup.n, self.shard.width,
                                                    _stream_ptr(self.shard.device)), "smore_gather_rows")
        return out

    def _materialize(self, lookup):
        return _EmbedLookupFunc.apply(self, self.dummy_tensor, lookup)

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

    def apply_grad(self, lr):
        self.step += 1
        self._neutralise_unused_lookups()
        self.barrier()              # every rank's id lists and gradient rows are complete
        self.owner_update(lr)
        self.barrier()              # every shard is updated; arenas may be overwritten
        self._drop_plans()

    def owner_update(self, lr):
        sh = self.shard
        lay = sh.layout
        L = _lib.lib()
        dev = sh.device
        st = _stream_ptr(dev)
        G, P = sh.world, len(lay.plan_caps)
        n_in = G * lay.span
        if self._owner_ws is None:
            nbytes = L.smore_unique_rows_workspace_bytes(max(sh.S, 1))
            self._owner_ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            with _lib.timed("shard_collect"):
                _lib.check(L.smore_shard_collect_ids(sh.d_uniq_ptrs.data_ptr(), sh.d_nuniq_ptrs.data_ptr(), G, P,
                                                     self._caps, sh.base, sh.S, self._in_ids.data_ptr(),
                                                     self._in_bounds.data_ptr(), st), "smore_shard_collect_ids")
                _lib.check(L.smore_unique_rows(self._in_ids.data_ptr(), n_in, max(sh.S, 1), self._o_uniq.data_ptr(),
                                               self._o_slot.data_ptr(), self._o_counts.data_ptr(),
                                               self._o_nuniq.data_ptr(), self._owner_ws.data_ptr(),
                                               self._owner_ws.numel(), st), "smore_unique_rows(owner)")
                _lib.check(L.smore_shard_record_sources(self._o_slot.data_ptr(), n_in, self._o_src.data_ptr(), st),
                           "smore_shard_record_sources")
            _lib.note("n_unique_owner", self._o_nuniq[0])
            with _lib.timed("shard_reduce_update"):
                _lib.check(L.smore_shard_reduce_update_rows(
                    sh.table.data_ptr(), sh.m.data_ptr(), sh.v.data_ptr(), self._o_uniq.data_ptr(),
                    self._o_counts.data_ptr(), self._o_src.data_ptr(), self._o_nuniq.data_ptr(), n_in,
                    sh.d_grad_ptrs.data_ptr(), self._in_ids.data_ptr(), self._in_bounds.data_ptr(), G, P, self._caps,
                    sh.width, float(lr), 0.9, 0.999, eps, int(self.step), int(self.squeeze), st),
                    "smore_shard_reduce_update_rows")

    def update_step(self, indices, inverse_indices, grad, lr):
        raise _lib.SmoreError("update_step with caller-merged gradients is not defined for a sharded table")


class ShardGroup(object):
    """Convenience constructors."""

    @staticmethod
    def from_process_group(n_rows_total, width, plan_caps, squeeze=True, group=None, device=None):
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        shard = ShardedTable(n_rows_total, width, rank, world, device, plan_caps, squeeze, symmetric=True)
        shard.connect_processes(group)
        return shard

    @staticmethod
    def emulated(world, n_rows_total, width, plan_caps, squeeze=True, device="cuda:0"):
        """`world` shards in this process on one GPU, wired to each other by raw pointers."""
        shards = [ShardedTable(n_rows_total, width, r, world, device, plan_caps, squeeze) for r in range(world)]
        tables = [s._table_block.ptr for s in shards]
        arenas = [s._arena_block.ptr for s in shards]
        for s in shards:
            s.connect(tables, arenas)
        return shards
