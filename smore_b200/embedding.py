"""Sparse embedding storage, per-step gradient merge and row-wise optimizers on the GPU.

Counterparts of the reference's embedding layer for a table that lives in GPU memory:

    SparseEmbedding        smore/common/embedding/sparse_embed.py:26-67  (same fields and hooks)
    EmbeddingOptimizer     smore/common/embedding/embed_optimizer.py:69-163
    SGD/Adam/AdaGradEmbedOptimizer, get_optim_class      embed_optimizer.py:166-252,312-364

The call surface is the reference's (`zero_grad`, `forward` installed as
`SparseEmbedding.fwd_delegate`, `accumulate_grad`, `apply_grad(lr)`, `update_step`,
`prepare_optimizers`, `share_memory`, state buffers named `state_sum_fo` / `state_sum_sq` /
`state_sum`).  What changes is where the work happens:

  * lookups listed in `lazy_names` return a LazyRows handle instead of a gathered copy; the
    distance ops of smore_b200.ext_ops read those rows straight from the table;
  * the first backward of a step de-duplicates all row ids looked up in that step (sorted
    unique + inverse map, identical to torch.unique(..., return_inverse=True)) and every
    gradient producer adds straight into one compact [n_ids, width] buffer;
  * `apply_grad` runs one fused kernel per step that reads gradient, row and optimizer state
    once and writes row and state once.

Nothing here synchronises with the host; sizes that are only known on the device (the number
of distinct rows) stay there.
"""
import os

import torch
import torch.nn as nn

from . import _lib

eps = 1e-8  # smore/common/consts.py:20


def eval_tuple(arg):
    """'(aggr,adam,gpu,True,5)' -> ('aggr', 'adam', 'gpu', True, 5)  (smore/common/util.py:94-112)."""
    if isinstance(arg, (tuple, list)):
        return tuple(arg)
    s = arg.strip()
    if s[0] in "([":
        s = s[1:-1]
    out = []
    for item in s.split(","):
        item = item.strip()
        if item == "":
            continue
        if item in ("True", "False"):
            out.append(item == "True")
            continue
        try:
            out.append(int(item))
        except ValueError:
            try:
                out.append(float(item))
            except ValueError:
                out.append(item.strip("'\""))
    return tuple(out)


def _stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


class DummyJob(object):
    """embed_rw.py:25-27: the handle a synchronous read returns."""

    def sync(self):
        pass


_DUMMY_JOB = DummyJob()


class SparseEmbedding(nn.Module):
    """A [num_rows, num_cols] table whose lookups can be taken over by an optimizer
    (sparse_embed.py:26-67)."""

    def __init__(self, num_rows, num_cols):
        super(SparseEmbedding, self).__init__()
        self.num_rows = num_rows
        self.embedding = nn.Parameter(torch.zeros(num_rows, num_cols))
        self.fwd_delegate = None
        self.dummy_job = _DUMMY_JOB

    @property
    def device(self):
        return self.embedding.device

    @property
    def shape(self):
        return self.embedding.shape

    def init_params(self, lb, ub):
        nn.init.uniform_(tensor=self.embedding, a=lb, b=ub)

    def register_tensor(self, name, tensor_obj):
        self.register_buffer(name, tensor_obj)
        if self.embedding.is_shared():
            tensor_obj.share_memory_()

    def forward(self, indices, name=None):
        if self.num_rows == 0:
            return None
        if self.fwd_delegate is not None:
            return self.fwd_delegate(indices, name)
        mat = self.embedding if indices is None else self.embedding[indices]
        mat.job_handle = self.dummy_job
        return mat


class LazyRows(object):
    """Rows `table[idx]` viewed as [d0, d1, width] without being gathered.

    Supports what the model code does to a looked-up block between the lookup and the
    distance op (kg_reasoning.py:299-355): `.job_handle.sync()`, `.view(B, K, -1)`,
    `.unsqueeze(1)`, `.shape`, `.dim()`.  `materialize()` gives the ordinary gathered tensor
    (with gradient tracking) for any other use.
    """

    def __init__(self, owner, lookup, shape):
        self.owner = owner
        self.lookup = lookup
        self._shape = tuple(shape)
        self.job_handle = _DUMMY_JOB
        self._box_cache = None

    @property
    def shape(self):
        return torch.Size(self._shape)

    @property
    def device(self):
        return self.owner.table.device

    @property
    def dtype(self):
        return self.owner.table.dtype

    @property
    def is_cuda(self):
        return True

    def dim(self):
        return len(self._shape)

    def size(self, d=None):
        return self.shape if d is None else self._shape[d]

    def is_contiguous(self):
        return True

    def contiguous(self):
        return self

    def _reshaped(self, shape):
        out = LazyRows(self.owner, self.lookup, shape)
        return out

    def view(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        width = self._shape[-1]
        n = self.lookup.n
        shape = list(shape)
        if shape[-1] == -1:
            shape[-1] = width
        if shape[-1] != width:
            raise ValueError("LazyRows.view keeps whole rows: last dim must stay %d" % width)
        lead = shape[:-1]
        if lead.count(-1) > 1:
            raise ValueError("only one dimension can be inferred")
        known = 1
        for v in lead:
            if v != -1:
                known *= v
        if -1 in lead:
            lead[lead.index(-1)] = n // max(known, 1)
            known = 1
            for v in lead:
                known *= v
        if known != n:
            raise ValueError("shape %s is invalid for %d rows" % (shape, n))
        return self._reshaped(tuple(lead) + (width,))

    reshape = view

    def unsqueeze(self, d):
        nd = len(self._shape)
        if d < 0:
            d += nd + 1
        if d >= nd:
            raise ValueError("LazyRows.unsqueeze: cannot add a dimension after the row dimension")
        return self._reshaped(self._shape[:d] + (1,) + self._shape[d:])

    def as_3d(self):
        """(be, ne, width) for the distance ops."""
        s = self._shape
        if len(s) == 3:
            return s
        if len(s) == 2:
            return (s[0], 1, s[1])
        raise ValueError("LazyRows with shape %s cannot be used as a 3-D entity operand" % (s,))

    def materialize(self):
        return self.owner._materialize(self.lookup).view(self._shape)


class _Lookup(object):
    __slots__ = ("idx", "n", "name", "order", "offset", "plan", "received", "key", "n_consumers")

    def __init__(self, idx, name, order):
        self.idx = idx          # int64 [n] on the table's device
        self.n = idx.numel()
        self.name = name
        self.order = order
        self.offset = None      # position of this lookup in its plan's concatenated id list
        self.plan = None
        self.received = False   # a gradient producer has run for this lookup
        self.key = None         # identity of the caller's id tensor (sharded tables with prefetch)
        self.n_consumers = 0    # distance ops that took this lookup's rows in the forward pass


class _StepPlan(object):
    """De-duplicated view of the rows a group of lookups touched, plus their gradient buffer."""

    def __init__(self, opt, lookups):
        table = opt.table
        dev = table.device
        self.lookups = lookups
        off = 0
        for lk in lookups:
            lk.offset = off
            lk.plan = self
            off += lk.n
        self.n = off
        self.idx_all = lookups[0].idx if len(lookups) == 1 else torch.cat([lk.idx for lk in lookups])
        self.uniq = torch.empty(self.n, dtype=torch.int64, device=dev)
        self.slot = torch.empty(self.n, dtype=torch.int32, device=dev)
        self.counts = torch.empty(self.n, dtype=torch.int32, device=dev)
        self.n_unique = torch.empty(2, dtype=torch.int32, device=dev)
        self.g_rows = torch.empty(self.n, table.shape[1], dtype=table.dtype, device=dev)
        L = _lib.lib()
        ws = opt._unique_workspace()
        st = _stream_ptr(dev)
        with torch.cuda.device(dev), _lib.timed("unique_rows"):
            _lib.check(L.smore_unique_rows(self.idx_all.data_ptr(), self.n, table.shape[0], self.uniq.data_ptr(),
                                           self.slot.data_ptr(), self.counts.data_ptr(), self.n_unique.data_ptr(),
                                           ws.data_ptr(), ws.numel(), st), "smore_unique_rows")
            _lib.check(L.smore_zero_shared_rows(self.g_rows.data_ptr(), self.counts.data_ptr(),
                                                self.n_unique.data_ptr(), self.n, table.shape[1], st),
                       "smore_zero_shared_rows")

    def slot_of(self, lookup):
        return self.slot[lookup.offset:lookup.offset + lookup.n]


class _EmbedLookupFunc(torch.autograd.Function):
    """Gathered copy of table rows with the gradient routed to the optimizer
    (embed_optimizer.py:51-66)."""

    @staticmethod
    def forward(ctx, opt, dummy, lookup):
        ctx.opt = opt
        ctx.lookup = lookup
        return opt._gather_lookup(lookup)

    @staticmethod
    def backward(ctx, grad_output):
        ctx.opt.accumulate_grad(ctx.lookup, grad_output.contiguous(), ctx.lookup.order)
        return None, None, None


class EmbeddingOptimizer(object):
    """Owns the lookups of one SparseEmbedding during a training step and applies the row-wise
    update (embed_optimizer.py:69-163).  `args` needs `optim_mode` (the reference's tuple string
    '(aggr,adam,gpu,<row-wise v>,<queue>)') and may carry `share_optim_stats`.
    """

    opt_name = None
    state_names = ()

    # ---- the reference's class-level hooks -------------------------------------------------
    @classmethod
    def prepare_embed(cls, args, optim_mode, embed, fn_register):
        raise NotImplementedError

    @classmethod
    def prepare_optimizers(cls, args, list_sparse_embeds):
        if not getattr(args, "share_optim_stats", False):
            return
        optim_mode = eval_tuple(args.optim_mode)
        for e in list_sparse_embeds:
            cls.prepare_embed(args, optim_mode, e, e.register_tensor)

    def share_memory(self):
        # state lives in GPU memory next to the table; there is nothing to move to shared host memory
        pass

    def prepare_forward(self, indices, name):
        # optimizer state is read inside the fused update kernel, not prefetched per lookup
        pass

    # ---- construction --------------------------------------------------------------------------
    def __init__(self, args, sp_embed, gpu_id, lazy_names=None):
        self.args = args
        self.sparse_embed = sp_embed
        self.gpu_id = gpu_id
        if not sp_embed.embedding.is_cuda:
            raise _lib.SmoreError("the embedding table must be in GPU memory (move the module to cuda:%s first)"
                                  % gpu_id)
        self.table = sp_embed.embedding.data
        if self.table.dtype != torch.float32 or not self.table.is_contiguous():
            raise TypeError("the embedding table must be contiguous float32")
        sp_embed.fwd_delegate = self.forward
        self.dummy_tensor = nn.Parameter(torch.zeros(1, 1, device=self.table.device))
        optim_mode = eval_tuple(args.optim_mode)
        self.optim_mode = optim_mode
        if optim_mode[0] not in ("fast", "aggr"):
            raise ValueError("optim_mode[0] must be 'fast' or 'aggr'")
        self.optimizer_name = optim_mode[1]
        self.optimizer_device = optim_mode[2]
        if self.optimizer_device != "gpu":
            raise _lib.SmoreError("optimizer state is kept in GPU memory: use optim_mode (..., 'gpu', ...)")
        self.squeeze = bool(optim_mode[3])
        self.queue_size = optim_mode[4] if len(optim_mode) > 4 else 0
        self.share_optim_stats = getattr(args, "share_optim_stats", False)
        if lazy_names is None:
            env = os.environ.get("SMORE_B200_LAZY_ROWS", "")
            lazy_names = tuple(x for x in env.split(",") if x)
        self.lazy_names = tuple(lazy_names)
        self.step = 0
        self._ws = None
        self._local_state = {}
        if self.share_optim_stats:
            for name in self.state_names:
                if not hasattr(sp_embed, name):
                    raise _lib.SmoreError("share_optim_stats is set but %s was not registered "
                                          "(call prepare_optimizers first)" % name)
        else:
            self.prepare_embed(args, optim_mode, sp_embed, self._register_local)
        self.zero_grad()

    def _register_local(self, name, tensor):
        self._local_state[name] = tensor.to(self.table.device)

    def state(self, name):
        if self.share_optim_stats:
            return getattr(self.sparse_embed, name)
        return self._local_state[name]

    def _unique_workspace(self):
        if self._ws is None:
            nbytes = _lib.lib().smore_unique_rows_workspace_bytes(self.table.shape[0])
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=self.table.device)
        return self._ws

    # ---- per-step bookkeeping ----------------------------------------------------------------------
    def _drop_plans(self):
        """Forget the step's plans.  A plan and its lookups refer to each other; cutting the links
        here lets the step's large buffers be released at once instead of at the next cycle
        collection."""
        for plan in getattr(self, "_plans", []):
            for lk in plan.lookups:
                lk.plan = None
            plan.lookups = []
        self._plans = []       # plans built in this step (normally one)

    def zero_grad(self):
        self.n_fwd = 0
        self._pending = []     # lookups registered since the last plan was built
        self._drop_plans()
        self.grad_list = []    # kept for interface parity; gradients never queue up here
        self.has_grad_list = []
        self._fused_lr = None          # set by announce_lr(): rows may be updated inside the backward pass
        self._step_advanced = False    # the device-side step counter was already advanced for this step

    def announce_lr(self, lr):
        """Optional, after zero_grad() and before the step's backward pass: tells the optimizer the
        learning rate apply_grad(lr) will be called with.  Table-resident lookups consumed by exactly
        one distance op may then have the rows that only ONE position of the step touches updated
        inside that op's backward kernel (smore_rows_backward_fused_adam) instead of writing their
        gradient out for apply_grad to read back; the result is the same update.  Only the Adam
        optimizer with a row-wise second moment does this; others ignore the call.  A step that
        announced a learning rate must end with apply_grad of the same value (some rows have
        already moved)."""
        if self.opt_name != "adam" or not self.squeeze:
            return
        self._fused_lr = float(lr)
        if getattr(self, "_step_dev", None) is not None and not self._step_advanced:
            self._advance_device_step(lr)
            self._step_advanced = True

    def fused_update_args(self, lookup, plan):
        """Arguments of the in-backward update for `lookup`, or None when it does not apply."""
        if getattr(self, "_fused_lr", None) is None or lookup.n_consumers != 1 or lookup.received:
            return None
        if len(self._plans) != 1 or plan is not self._plans[0] or self.share_optim_stats:
            return None
        dev_step = getattr(self, "_step_dev", None) is not None
        return {"m": self.state("state_sum_fo"), "v": self.state("state_sum_sq"), "uniq": plan.uniq,
                "lr": self._fused_lr, "step": 1 if dev_step else int(self.step) + 1,
                "step_scalars": self._step_scalars if dev_step else None}

    def _device_indices(self, indices):
        idx = indices.reshape(-1)
        if idx.dtype != torch.int64:
            idx = idx.long()
        if idx.device != self.table.device:
            idx = idx.to(self.table.device, non_blocking=True)
        return idx.contiguous()

    def _gather(self, idx):
        out = torch.empty(idx.numel(), self.table.shape[1], dtype=self.table.dtype, device=self.table.device)
        with torch.cuda.device(self.table.device):
            _lib.check(_lib.lib().smore_gather_rows(self.table.data_ptr(), idx.data_ptr(), self.table.shape[0],
                                                    out.data_ptr(), idx.numel(), self.table.shape[1],
                                                    _stream_ptr(self.table.device)), "smore_gather_rows")
        return out

    def forward(self, indices, name=None):
        """What SparseEmbedding.forward delegates to (embed_optimizer.py:150-153)."""
        if indices is None:
            mat = self.table
            mat.job_handle = _DUMMY_JOB
            return mat
        idx = self._device_indices(indices)
        track = self.sparse_embed.training and torch.is_grad_enabled()
        if not track:
            out = self._gather(idx)
            out.job_handle = _DUMMY_JOB
            return out
        lookup = _Lookup(idx, name, self.n_fwd)
        self.n_fwd += 1
        self._pending.append(lookup)
        if name is not None and name in self.lazy_names:
            return LazyRows(self, lookup, (lookup.n, self.table.shape[1]))
        out = _EmbedLookupFunc.apply(self, self.dummy_tensor, lookup)
        out.job_handle = _DUMMY_JOB
        return out

    def _materialize(self, lookup):
        return _EmbedLookupFunc.apply(self, self.dummy_tensor, lookup)

    def _gather_lookup(self, lookup):
        return self._gather(lookup.idx)

    def rows_operands(self, lookup):
        """(rows tensor, int64 row ids into it) that the distance kernels read for `lookup`."""
        return self.table, lookup.idx

    def plan_for(self, lookup):
        """The step plan that covers `lookup`, built on first use from every lookup made so far."""
        if lookup.plan is None:
            self._plans.append(_StepPlan(self, self._pending))
            self._pending = []
        return lookup.plan

    def accumulate_grad(self, lookup, grad_submat, fwd_idx=None):
        """Add a dense [n, width] gradient block of one lookup (embed_optimizer.py:146-148)."""
        plan = self.plan_for(lookup)
        # a second producer for the same positions must add to what the first one stored
        counts_ptr = None if lookup.received else plan.counts.data_ptr()
        lookup.received = True
        self.has_grad_list.append(lookup.order)
        with torch.cuda.device(self.table.device):
            _lib.check(_lib.lib().smore_scatter_add_rows(grad_submat.data_ptr(), plan.slot_of(lookup).data_ptr(),
                                                         counts_ptr, plan.g_rows.data_ptr(), lookup.n,
                                                         self.table.shape[1], _stream_ptr(self.table.device)),
                       "smore_scatter_add_rows")

    # ---- the update ------------------------------------------------------------------------------
    def _launch_update(self, uniq, g_rows, n_unique, capacity, lr):
        raise NotImplementedError

    def check_status(self):
        """Raise if a kernel of this process reported trouble since the last check: a bounded wait on
        an asynchronous copy that ran out (results of that launch are invalid) or a row id outside the
        table (that position got NaN and no gradient).  Synchronises the device, so call it between
        steps or every few hundred steps, not inside one; the status word is cleared."""
        torch.cuda.synchronize(self.table.device)
        with torch.cuda.device(self.table.device):
            status = _lib.async_status()
            if status:
                _lib.async_status_clear()
        if status:
            what = [name for bit, name in ((_lib.STATUS_COPY_WAIT, "a local bulk-copy wait gave up"),
                                           (_lib.STATUS_PEER_WAIT, "a wait on a copy from a peer gave up"),
                                           (_lib.STATUS_BAD_ROW_ID, "a row id outside the table was looked up"),
                                           (_lib.STATUS_CAPACITY, "an owner of a sharded table received more pairs than "
                                                                  "its buffers hold, or a rank's scoring op did not match "
                                                                  "the others' (K, branches): that work was dropped"))
                    if status & bit]
            raise RuntimeError("smore_b200 kernels reported status %d: %s" % (status, "; ".join(what) or "unknown"))

    def use_device_step(self):
        """Keep the optimizer's step counter on the device from now on (it starts from the current
        host-side value).  Needed when training steps are captured in a CUDA graph and replayed:
        Python does not run during a replay, so the bias corrections must come from device memory."""
        dev = self.table.device
        self._step_dev = torch.tensor([int(self.step)], dtype=torch.int64, device=dev)
        self._step_scalars = torch.zeros(2, dtype=torch.float32, device=dev)

    def _advance_device_step(self, lr):
        dev = self.table.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().smore_adam_step_scalars(self._step_dev.data_ptr(), float(lr), 0.9, 0.999,
                                                          self._step_scalars.data_ptr(), _stream_ptr(dev)),
                       "smore_adam_step_scalars")

    def _run_update(self, opt_name, m, v, uniq, g_rows, n_unique, capacity, lr):
        dev = self.table.device
        if getattr(self, "_step_dev", None) is not None:
            if not getattr(self, "_step_advanced", False):
                self._advance_device_step(lr)
            with torch.cuda.device(dev), _lib.timed("sparse_update_rows"):
                _lib.check(_lib.lib().smore_sparse_update_rows_dev(
                    _lib.OPT_IDS[opt_name], self.table.data_ptr(), None if m is None else m.data_ptr(),
                    None if v is None else v.data_ptr(), uniq.data_ptr(), g_rows.data_ptr(), n_unique.data_ptr(),
                    capacity, self.table.shape[1], float(lr), 0.9, 0.999, eps, self._step_scalars.data_ptr(),
                    int(self.squeeze), _stream_ptr(dev)), "smore_sparse_update_rows_dev")
            return
        with torch.cuda.device(dev), _lib.timed("sparse_update_rows"):
            _lib.check(_lib.lib().smore_sparse_update_rows(
                _lib.OPT_IDS[opt_name], self.table.data_ptr(), None if m is None else m.data_ptr(),
                None if v is None else v.data_ptr(), uniq.data_ptr(), g_rows.data_ptr(), n_unique.data_ptr(),
                capacity, self.table.shape[1], float(lr), 0.9, 0.999, eps, int(self.step),
                int(self.squeeze), _stream_ptr(dev)), "smore_sparse_update_rows")

    def _merge_plans(self):
        """More than one plan in a step (lookups made after a backward had already run): fold
        them into one by treating each plan's (rows, gradients) as a dense block."""
        plans = self._plans
        dev = self.table.device
        lookups, blocks = [], []
        for p in plans:
            ids = p.uniq.clone()
            nu = p.n_unique[0]
            ids[torch.arange(p.n, device=dev) >= nu] = -1      # tail beyond the distinct rows: ignored
            untouched = self._untouched_mask(p)
            if untouched is not None:
                ids[untouched] = -1
            lk = _Lookup(ids, None, -1)
            lookups.append(lk)
            blocks.append(p.g_rows)
        merged = _StepPlan(self, lookups)
        for lk, g in zip(lookups, blocks):
            lk.received = True
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().smore_scatter_add_rows(g.data_ptr(), merged.slot_of(lk).data_ptr(),
                                                             merged.counts.data_ptr(), merged.g_rows.data_ptr(),
                                                             lk.n, self.table.shape[1], _stream_ptr(dev)),
                           "smore_scatter_add_rows")
        return merged

    def _untouched_mask(self, plan):
        """Rows of a plan that no gradient producer wrote (their lookups never got a backward
        call): the reference leaves such rows out of the update (embed_optimizer.py:146-163)."""
        missing = [lk for lk in plan.lookups if not lk.received]
        if not missing:
            return None
        live = torch.zeros(plan.n, dtype=torch.int32, device=self.table.device)
        for lk in plan.lookups:
            if lk.received:
                s = plan.slot_of(lk).long()
                live.index_put_((s[s >= 0],), torch.ones((), dtype=torch.int32, device=live.device))
        return live == 0

    def apply_grad(self, lr):
        """embed_optimizer.py:155-163: the step counter advances even when nothing was looked up."""
        self.step += 1
        if getattr(self, "_fused_lr", None) is not None and float(lr) != self._fused_lr:
            raise _lib.SmoreError("apply_grad(%r) after announce_lr(%r): rows updated inside the backward pass "
                                  "used the announced value" % (lr, self._fused_lr))
        if not self._plans:
            self._pending = []
            if getattr(self, "_step_dev", None) is not None and not getattr(self, "_step_advanced", False):
                self._advance_device_step(lr)
            return
        plan = self._plans[0] if len(self._plans) == 1 else self._merge_plans()
        uniq = plan.uniq
        untouched = self._untouched_mask(plan) if len(self._plans) == 1 else None
        if untouched is not None:
            # point untouched rows' update at nothing: give them a zero gradient and skip them by
            # marking the row id negative is not possible for the kernel, so they are compacted out
            keep = ~untouched & (torch.arange(plan.n, device=uniq.device) < plan.n_unique[0])
            sel = keep.nonzero().view(-1)
            uniq = plan.uniq[sel].contiguous()
            g_rows = plan.g_rows[sel].contiguous()
            n_unique = torch.tensor([sel.numel(), 0], dtype=torch.int32, device=uniq.device)
            self._launch_update(uniq, g_rows, n_unique, sel.numel(), lr)
        else:
            _lib.note("n_unique", plan.n_unique[0])
            self._launch_update(uniq, plan.g_rows, plan.n_unique, plan.n, lr)
        self._drop_plans()
        self._pending = []

    def update_step(self, indices, inverse_indices, grad, lr):
        """Reference-shaped entry (embed_optimizer.py:84-86): distinct row ids + their merged gradient."""
        dev = self.table.device
        indices = indices.to(dev).contiguous()
        grad = grad.to(dev).contiguous()
        n_unique = torch.tensor([indices.numel(), 0], dtype=torch.int32, device=dev)
        self._launch_update(indices, grad, n_unique, indices.numel(), lr)


class SGDEmbedOptimizer(EmbeddingOptimizer):
    opt_name = "sgd"
    state_names = ()

    @classmethod
    def prepare_embed(cls, args, optim_mode, embed, fn_register):
        pass

    def _launch_update(self, uniq, g_rows, n_unique, capacity, lr):
        self._run_update("sgd", None, None, uniq, g_rows, n_unique, capacity, lr)


class AdamEmbedOptimizer(EmbeddingOptimizer):
    opt_name = "adam"
    state_names = ("state_sum_fo", "state_sum_sq")

    @classmethod
    def prepare_embed(cls, args, optim_mode, embed, fn_register):
        dev = embed.embedding.device
        fn_register("state_sum_fo", torch.zeros(embed.embedding.size(), device=dev))
        if optim_mode[3]:
            fn_register("state_sum_sq", torch.zeros(embed.embedding.size(0), 1, device=dev))
        else:
            fn_register("state_sum_sq", torch.zeros(embed.embedding.size(), device=dev))

    def _launch_update(self, uniq, g_rows, n_unique, capacity, lr):
        self._run_update("adam", self.state("state_sum_fo"), self.state("state_sum_sq"), uniq, g_rows, n_unique,
                         capacity, lr)


class AdaGradEmbedOptimizer(EmbeddingOptimizer):
    opt_name = "adagrad"
    state_names = ("state_sum",)

    @classmethod
    def prepare_embed(cls, args, optim_mode, embed, fn_register):
        dev = embed.embedding.device
        if optim_mode[3]:
            fn_register("state_sum", torch.zeros(embed.embedding.size(0), 1, device=dev))
        else:
            fn_register("state_sum", torch.zeros(embed.embedding.size(), device=dev))

    def _launch_update(self, uniq, g_rows, n_unique, capacity, lr):
        self._run_update("adagrad", None, self.state("state_sum"), uniq, g_rows, n_unique, capacity, lr)


def get_optim_class(args):
    """embed_optimizer.py:352-364.  'rmsprop' is rejected: the reference class of that name cannot
    be called by its own apply_grad (update_step signature mismatch, embed_optimizer.py:271 vs :163)."""
    name = eval_tuple(args.optim_mode)[1]
    if name == "adam":
        return AdamEmbedOptimizer
    if name == "adagrad":
        return AdaGradEmbedOptimizer
    if name == "sgd":
        return SGDEmbedOptimizer
    raise NotImplementedError("embedding optimizer %r" % (name,))
