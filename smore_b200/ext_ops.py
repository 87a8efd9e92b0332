"""The custom distance ops, with the names, tensor contracts and autograd behaviour of
smore/common/torchext/ext_ops.py:15-22 and the dist_func/*.py modules behind it.

    l1_dist, l2_dist, box_dist_in, box_dist_out, rotate_dist, complex_sim, distmult_sim
    (+ box_dist_both, which returns the two box distances from a single pass)

Operand rule (e.g. box_dist.py:50-70): the entity operand is 3-D [be, ne, rows]; the query
operands are 3-D [bc, nc, dim], or 4-D [B, U, 1, dim] with U union branches, in which case the
op runs once per branch and the results are stacked to [B, U, num].  l2_dist takes the root
outside the kernel, as l2_dist.py:59,62 does.

The entity operand may also be a smore_b200.embedding.LazyRows handle (rows of the table named
by index).  Then nothing is gathered: the kernels read the table rows in place and the
backward pass adds the row gradients into the owning optimizer's per-step buffer.
"""
import torch

from . import _lib
from . import extlib_cuda as extlib
from .embedding import LazyRows

__all__ = ["l1_dist", "l2_dist", "box_dist_in", "box_dist_out", "box_dist_both", "rotate_dist", "complex_sim",
           "distmult_sim"]


def _out_shape(entity_shape, query_shape):
    return max(entity_shape[0], query_shape[0]), max(entity_shape[1], query_shape[1])


def _check_broadcast(entity_shape, query_shape):
    for a, b in ((entity_shape[0], query_shape[0]), (entity_shape[1], query_shape[1])):
        if a % b != 0 and b % a != 0:
            raise ValueError("entity %s and query %s do not broadcast" % (tuple(entity_shape), tuple(query_shape)))


class _DistFunc(torch.autograd.Function):
    """One distance on materialised operands (the pattern of l1_dist.py:21-46 / box_dist.py:21-47)."""

    @staticmethod
    def forward(ctx, name, entity, first, second):
        _check_broadcast(entity.shape, first.shape)
        entity, first = entity.contiguous(), first.contiguous()
        second = None if second is None else second.contiguous()
        dst = torch.empty(_out_shape(entity.shape, first.shape), dtype=entity.dtype, device=entity.device)
        extlib.dist_forward(name, entity, first, second, dst)
        ctx.name = name
        ctx.two = second is not None
        if ctx.two:
            ctx.save_for_backward(entity, first, second)
        else:
            ctx.save_for_backward(entity, first)
        return dst

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.two:
            entity, first, second = ctx.saved_tensors
        else:
            entity, first = ctx.saved_tensors
            second = None
        grad_out = grad_out.contiguous()
        # the kernels write every element, so the buffers need not be cleared first
        g_entity = torch.empty_like(entity)
        g_first = torch.empty_like(first)
        g_second = torch.empty_like(second) if ctx.two else None
        extlib.dist_backward(ctx.name, grad_out, entity, first, second, g_entity, g_first, g_second)
        return None, g_entity, g_first, g_second


class _BoxBothFunc(torch.autograd.Function):
    """Both box distances of materialised operands in one pass over the entity rows."""

    @staticmethod
    def forward(ctx, entity, center, offset):
        _check_broadcast(entity.shape, center.shape)
        entity, center, offset = entity.contiguous(), center.contiguous(), offset.contiguous()
        bsize, num = _out_shape(entity.shape, center.shape)
        d_out = torch.empty(bsize, num, dtype=entity.dtype, device=entity.device)
        d_in = torch.empty_like(d_out)
        L = _lib.lib()
        with torch.cuda.device(entity.device):
            _lib.check(L.smore_box_forward(entity.data_ptr(), None, 0, center.data_ptr(), offset.data_ptr(),
                                           d_out.data_ptr(), d_in.data_ptr(), bsize, num, entity.shape[0],
                                           entity.shape[1], center.shape[0], center.shape[1], center.shape[2],
                                           torch.cuda.current_stream(entity.device).cuda_stream),
                       "smore_box_forward")
        ctx.save_for_backward(entity, center, offset)
        return d_out, d_in

    @staticmethod
    def backward(ctx, g_out, g_in):
        entity, center, offset = ctx.saved_tensors
        g_out, g_in = g_out.contiguous(), g_in.contiguous()
        g_entity, g_center, g_offset = torch.empty_like(entity), torch.empty_like(center), torch.empty_like(offset)
        bsize, num = g_out.shape
        L = _lib.lib()
        with torch.cuda.device(entity.device):
            _lib.check(L.smore_box_backward(g_out.data_ptr(), g_in.data_ptr(), entity.data_ptr(), None, 0,
                                            center.data_ptr(), offset.data_ptr(), g_entity.data_ptr(), None, None,
                                            None, g_center.data_ptr(), g_offset.data_ptr(), bsize, num,
                                            entity.shape[0], entity.shape[1], center.shape[0], center.shape[1],
                                            center.shape[2],
                                            torch.cuda.current_stream(entity.device).cuda_stream),
                       "smore_box_backward")
        return g_entity, g_center, g_offset


def _check_rows_operands(name, rows, first, second):
    table = rows.owner.table
    if first.dim() != 3:
        raise ValueError("%s: query operands must be 3-D" % name)
    if not first.is_cuda or first.device != table.device or first.dtype != torch.float32:
        raise TypeError("%s: query operands must be float32 on the table's device" % name)
    if second is not None and second.shape != first.shape:
        raise ValueError("%s: the two query operands must have the same shape" % name)
    be, ne, width = rows.as_3d()
    parts = 1 if name == "box_both" else _lib.ROW_PARTS[name]
    if width != parts * first.shape[2]:
        raise ValueError("%s: table rows must be %d x the query dim" % (name, parts))
    _check_broadcast((be, ne), first.shape)
    return be, ne


def _fused_backward(name_or_id, owner, lookup, plan, table, row_ids, first, second, gouts, g_first, g_second, branches,
                    bsize, num, dim):
    """Backward with the Adam step of single-contributor rows folded in, when the owning optimizer
    announced its learning rate for this step and the shape is covered.  True when it ran."""
    fn = getattr(owner, "fused_update_args", None)
    fu = fn(lookup, plan) if fn is not None else None
    if fu is None:
        return False
    L = _lib.lib()
    dist_id = name_or_id if isinstance(name_or_id, int) else (
        _lib.BOX_BOTH_ID if name_or_id == "box_both" else _lib.DIST_IDS[name_or_id])
    if _lib._timer is not None:
        _lib.note("n_single", (plan.counts == 1).sum())
    rc = L.smore_rows_backward_fused_adam(
        dist_id, gouts[0].data_ptr(), gouts[1].data_ptr() if len(gouts) > 1 else None, table.data_ptr(),
        row_ids.data_ptr(), table.shape[0], first.data_ptr(), None if second is None else second.data_ptr(),
        plan.slot_of(lookup).data_ptr(), plan.counts.data_ptr(), plan.g_rows.data_ptr(), g_first.data_ptr(),
        None if g_second is None else g_second.data_ptr(), branches, bsize, num, dim, fu["m"].data_ptr(),
        fu["v"].data_ptr(), fu["uniq"].data_ptr(), fu["lr"], 0.9, 0.999, 1e-8, fu["step"],
        None if fu["step_scalars"] is None else fu["step_scalars"].data_ptr(),
        torch.cuda.current_stream(table.device).cuda_stream)
    if rc == -2:          # SMORE_ERR_BAD_SHAPE: not covered, nothing was enqueued
        return False
    _lib.check(rc, "smore_rows_backward_fused_adam")
    return True


class _RowsDistFunc(torch.autograd.Function):
    """A distance whose entity operand is table rows named by index.  `dummy` is the owning
    optimizer's one-element parameter: it makes autograd call backward even when no query
    operand needs a gradient (the same device the reference uses, embed_optimizer.py:128,153)."""

    @staticmethod
    def forward(ctx, name, rows, dummy, first, second):
        first = first.contiguous()
        second = None if second is None else second.contiguous()
        be, ne = _check_rows_operands(name, rows, first, second)
        owner, lookup = rows.owner, rows.lookup
        lookup.n_consumers += 1
        table, row_ids = owner.rows_operands(lookup)
        bc, nc, dim = first.shape
        bsize, num = max(be, bc), max(ne, nc)
        L = _lib.lib()
        st = torch.cuda.current_stream(table.device).cuda_stream
        sizes = (bsize, num, be, ne, bc, nc, dim)
        with torch.cuda.device(table.device), _lib.timed("rows_forward" if num >= 16 else "rows_forward_few"):
            if name == "box_both":
                d0 = torch.empty(bsize, num, dtype=table.dtype, device=table.device)
                d1 = torch.empty_like(d0)
                _lib.check(L.smore_box_forward(table.data_ptr(), row_ids.data_ptr(), table.shape[0],
                                               first.data_ptr(), second.data_ptr(), d0.data_ptr(), d1.data_ptr(), *sizes, st),
                           "smore_box_forward")
                outs = (d0, d1)
            else:
                d0 = torch.empty(bsize, num, dtype=table.dtype, device=table.device)
                _lib.check(L.smore_dist_forward_rows(_lib.DIST_IDS[name], table.data_ptr(), row_ids.data_ptr(),
                                                     table.shape[0], first.data_ptr(), None if second is None else second.data_ptr(),
                                                     d0.data_ptr(), *sizes, st), "smore_dist_forward_rows")
                outs = (d0,)
        ctx.name, ctx.rows, ctx.sizes = name, rows, sizes
        ctx.two = second is not None
        if ctx.two:
            ctx.save_for_backward(first, second)
        else:
            ctx.save_for_backward(first)
        return outs if name == "box_both" else outs[0]

    @staticmethod
    def backward(ctx, *gouts):
        if ctx.two:
            first, second = ctx.saved_tensors
        else:
            (first,) = ctx.saved_tensors
            second = None
        owner, lookup = ctx.rows.owner, ctx.rows.lookup
        table, row_ids = owner.rows_operands(lookup)
        plan = owner.plan_for(lookup)
        # the first gradient producer of a lookup may store rows that nothing else touches; any
        # later one over the same positions (another union branch) has to add to what is there
        g_first = torch.empty_like(first)
        g_second = torch.empty_like(second) if ctx.two else None
        gouts = [g.contiguous() for g in gouts]
        L = _lib.lib()
        st = torch.cuda.current_stream(table.device).cuda_stream
        bsize, num, be, ne, bc, nc, dim = ctx.sizes
        if be == bsize and ne == num and bc == bsize and nc == 1 and num >= 16:
            with torch.cuda.device(table.device), _lib.timed("rows_backward"):
                if _fused_backward(ctx.name, owner, lookup, plan, table, row_ids, first, second, gouts, g_first,
                                   g_second, 1, bsize, num, dim):
                    lookup.received = True
                    return None, None, None, g_first, g_second
        counts_ptr = None if lookup.received else plan.counts.data_ptr()
        lookup.received = True
        slot = plan.slot_of(lookup)
        with torch.cuda.device(table.device), _lib.timed("rows_backward" if ctx.sizes[1] >= 16 else "rows_backward_few"):
            if ctx.name == "box_both":
                _lib.check(L.smore_box_backward(gouts[0].data_ptr(), gouts[1].data_ptr(), table.data_ptr(),
                                                row_ids.data_ptr(), table.shape[0], first.data_ptr(), second.data_ptr(), None,
                                                slot.data_ptr(), counts_ptr, plan.g_rows.data_ptr(),
                                                g_first.data_ptr(), g_second.data_ptr(), *ctx.sizes, st),
                           "smore_box_backward")
            else:
                _lib.check(L.smore_dist_backward_rows(_lib.DIST_IDS[ctx.name], gouts[0].data_ptr(), table.data_ptr(),
                                                      row_ids.data_ptr(), table.shape[0], first.data_ptr(),
                                                      None if second is None else second.data_ptr(),
                                                      slot.data_ptr(), counts_ptr, plan.g_rows.data_ptr(),
                                                      g_first.data_ptr(),
                                                      None if g_second is None else g_second.data_ptr(),
                                                      *ctx.sizes, st), "smore_dist_backward_rows")
        return None, None, None, g_first, g_second


class _RowsUnionFunc(torch.autograd.Function):
    """All branches of a union query ([B, U, 1, dim] operands) against table rows in one pass:
    results [B, U, num], the same values as the per-branch loop of the reference front-ends
    (box_dist.py:60-68); backward adds the sum of the branches' row gradients once."""

    @staticmethod
    def forward(ctx, name, rows, dummy, first, second):
        first = first.contiguous()
        second = None if second is None else second.contiguous()
        owner, lookup = rows.owner, rows.lookup
        lookup.n_consumers += 1
        table, row_ids = owner.rows_operands(lookup)
        B, U, _, dim = first.shape
        num = rows.as_3d()[1]
        both = name == "box_both"
        dist_id = _lib.BOX_BOTH_ID if both else _lib.DIST_IDS[name]
        d0 = torch.empty(B, U, num, dtype=table.dtype, device=table.device)
        d1 = torch.empty_like(d0) if both else None
        with torch.cuda.device(table.device), _lib.timed("rows_forward_union"):
            _lib.check(_lib.lib().smore_union_forward_rows(
                dist_id, table.data_ptr(), row_ids.data_ptr(), table.shape[0], first.data_ptr(),
                None if second is None else second.data_ptr(), d0.data_ptr(), None if d1 is None else d1.data_ptr(),
                U, B, num, dim, torch.cuda.current_stream(table.device).cuda_stream), "smore_union_forward_rows")
        ctx.name, ctx.rows, ctx.sizes, ctx.dist_id = name, rows, (U, B, num, dim), dist_id
        ctx.two = second is not None
        if ctx.two:
            ctx.save_for_backward(first, second)
        else:
            ctx.save_for_backward(first)
        return (d0, d1) if both else d0

    @staticmethod
    def backward(ctx, *gouts):
        if ctx.two:
            first, second = ctx.saved_tensors
        else:
            (first,) = ctx.saved_tensors
            second = None
        owner, lookup = ctx.rows.owner, ctx.rows.lookup
        table, row_ids = owner.rows_operands(lookup)
        plan = owner.plan_for(lookup)
        g_first = torch.empty_like(first)
        g_second = torch.empty_like(second) if ctx.two else None
        gouts = [g.contiguous() for g in gouts]
        U, B, num, dim = ctx.sizes
        with torch.cuda.device(table.device), _lib.timed("rows_backward_union"):
            if _fused_backward(ctx.dist_id, owner, lookup, plan, table, row_ids, first, second, gouts, g_first,
                               g_second, U, B, num, dim):
                lookup.received = True
                return None, None, None, g_first, g_second
        counts_ptr = None if lookup.received else plan.counts.data_ptr()
        lookup.received = True
        slot = plan.slot_of(lookup)
        with torch.cuda.device(table.device), _lib.timed("rows_backward_union"):
            _lib.check(_lib.lib().smore_union_backward_rows(
                ctx.dist_id, gouts[0].data_ptr(), gouts[1].data_ptr() if len(gouts) > 1 else None, table.data_ptr(),
                row_ids.data_ptr(), table.shape[0], first.data_ptr(), None if second is None else second.data_ptr(),
                slot.data_ptr(),
                counts_ptr, plan.g_rows.data_ptr(), g_first.data_ptr(),
                None if g_second is None else g_second.data_ptr(), *ctx.sizes,
                torch.cuda.current_stream(table.device).cuda_stream), "smore_union_backward_rows")
        return None, None, None, g_first, g_second


def _union_in_one_pass(name, entity, first, second):
    """Whether the fused union kernels cover this call: table rows, two branches, one candidate
    list per query, row width within the row-stream kernels' limits."""
    if not isinstance(entity, LazyRows) or first.shape[1] != 2 or first.shape[2] != 1:
        return False
    if not first.is_cuda or first.dtype != torch.float32 or (second is not None and second.shape != first.shape):
        return False
    be, ne, width = entity.as_3d()
    dim = first.shape[3]
    parts = 1 if name == "box_both" else _lib.ROW_PARTS[name]
    return be == first.shape[0] and ne >= 4 and width == parts * dim and dim % 4 == 0 and dim <= 1024


_DOT_PRECISIONS = {"tf32": 0, "fp32": 1}


def dot_precision():
    """How shared-candidate inner products are computed: 'fp32' (tensor cores, every fp32 operand
    split into three bf16 terms: fp32-level accuracy, the default), 'tf32' (tensor cores, 10-bit
    mantissa products) or 'off' (SIMT kernels in exact fp32).  Environment: SMORE_B200_DOT."""
    import os
    mode = os.environ.get("SMORE_B200_DOT", "fp32").lower()
    if mode not in ("fp32", "tf32", "off"):
        raise ValueError("SMORE_B200_DOT must be fp32, tf32 or off")
    return mode


_dot_workspaces = {}     # (device, stream) -> uint8 scratch tensor, grown on demand


def _dot_workspace(device, nbytes):
    """Scratch for the GEMM route, kept per (device, stream): calls on one stream are ordered, so
    they can share it, and nothing is allocated in the steady state."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _dot_workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _dot_workspaces[key] = ws
    return ws


class _DotSharedFunc(torch.autograd.Function):
    """score[B, K] = query[B, W] . cand[K, W]^T and its two gradients as tensor-core GEMMs."""

    @staticmethod
    def forward(ctx, cand, query, precision):
        cand, query = cand.contiguous(), query.contiguous()
        K, W = cand.shape[-2], cand.shape[-1]
        B = query.shape[0]
        L = _lib.lib()
        dst = torch.empty(B, K, dtype=torch.float32, device=cand.device)
        ws = _dot_workspace(cand.device, L.smore_dot_workspace_bytes(B, K, W, precision))
        with torch.cuda.device(cand.device), _lib.timed("dot_forward"):
            _lib.check(L.smore_dot_forward_shared(cand.data_ptr(), query.data_ptr(), dst.data_ptr(), B, K, W, precision,
                                                  ws.data_ptr(), ws.numel(),
                                                  torch.cuda.current_stream(cand.device).cuda_stream),
                       "smore_dot_forward_shared")
        ctx.save_for_backward(cand, query)
        ctx.precision = precision
        return dst

    @staticmethod
    def backward(ctx, gout):
        cand, query = ctx.saved_tensors
        gout = gout.contiguous()
        K, W = cand.shape[-2], cand.shape[-1]
        B = query.shape[0]
        L = _lib.lib()
        g_cand, g_query = torch.empty_like(cand), torch.empty_like(query)
        ws = _dot_workspace(cand.device, L.smore_dot_workspace_bytes(B, K, W, ctx.precision))
        with torch.cuda.device(cand.device), _lib.timed("dot_backward"):
            _lib.check(L.smore_dot_backward_shared(gout.data_ptr(), cand.data_ptr(), query.data_ptr(), g_cand.data_ptr(),
                                                   g_query.data_ptr(), B, K, W, ctx.precision, ws.data_ptr(), ws.numel(),
                                                   torch.cuda.current_stream(cand.device).cuda_stream),
                       "smore_dot_backward_shared")
        return g_cand, g_query, None


def _dot_shared(name, entity, first, second):
    """The GEMM route for DistMult / ComplEx against shared candidates, or None if it does not apply."""
    if name not in ("distmult", "complex") or first.dim() != 3:
        return None
    mode = dot_precision()
    if mode == "off" or not _lib.lib().smore_dot_available():
        return None
    eshape = entity.as_3d() if isinstance(entity, LazyRows) else tuple(entity.shape)
    B, nc, dim = first.shape
    K, W = eshape[1], eshape[2]
    if eshape[0] != 1 or nc != 1 or B < 128 or K < 128 or (B | K | W) & 3 or first.dtype != torch.float32:
        return None
    if W != _lib.ROW_PARTS[name] * dim or not first.is_cuda:
        return None
    if isinstance(entity, LazyRows):
        entity = entity.materialize()          # K rows only: the gathered copy is small here
    query = first if second is None else torch.cat([first, second], dim=-1)
    return _DotSharedFunc.apply(entity.reshape(K, W), query.reshape(B, W), _DOT_PRECISIONS[mode])


def _apply(name, entity, first, second):
    routed = _dot_shared(name, entity, first, second)
    if routed is not None:
        return routed
    if isinstance(entity, LazyRows):
        return _RowsDistFunc.apply(name, entity, entity.owner.dummy_tensor, first, second)
    if name == "box_both":
        return _BoxBothFunc.apply(entity, first, second)
    return _DistFunc.apply(name, entity, first, second)


def _dist(name, entity, first, second=None):
    """Front-end shared by all ops: 3-D operands, or a per-branch loop for 4-D query operands."""
    if getattr(entity, "remote", False):
        # rows of a sharded table that stay with their owners (smore_b200.sharded.RemoteRows)
        return entity.owner.remote_dist(name, entity, first, second)
    if entity.dim() != first.dim():
        if first.dim() != 4 or entity.dim() != 3:
            raise ValueError("expected a 3-D entity operand with 3-D or 4-D query operands")
        if _union_in_one_pass(name, entity, first, second):
            return _RowsUnionFunc.apply(name, entity, entity.owner.dummy_tensor, first, second)
        outs = []
        for i in range(first.shape[1]):
            f = first[:, i, :, :].contiguous()
            s = None if second is None else second[:, i, :, :].contiguous()
            outs.append(_apply(name, entity, f, s))
        if name == "box_both":
            return torch.stack([o[0] for o in outs], dim=1), torch.stack([o[1] for o in outs], dim=1)
        return torch.stack(outs, dim=1)
    if entity.dim() != 3:
        raise ValueError("operands must be 3-D")
    return _apply(name, entity, first, second)


def l1_dist(entity_embed, center_embed):
    return _dist("l1", entity_embed, center_embed)


def l2_dist(entity_embed, center_embed):
    return torch.sqrt(_dist("l2", entity_embed, center_embed))


def rotate_dist(entity_embed, re_embed, im_embed):
    return _dist("rotate", entity_embed, re_embed, im_embed)


def complex_sim(entity_embed, re_embed, im_embed):
    return _dist("complex", entity_embed, re_embed, im_embed)


def distmult_sim(entity_embed, center_embed):
    return _dist("distmult", entity_embed, center_embed)


def box_dist_both(entity_embed, center_embed, offset_embed):
    """(dist_out, dist_in) of the same operands from one pass over the entity rows."""
    return _dist("box_both", entity_embed, center_embed, offset_embed)


_eval_box_cache = None      # (entity, center, offset, versions, which, other result) of the last no-grad call


def _box_one_eval(which, entity_embed, center_embed, offset_embed):
    """Without autograd (evaluation: every entity scored against a batch of queries) the pair of
    calls box_dist_out / box_dist_in on the same tensors (box.py:160-161) is served by one pass:
    the first computes both distances and parks the other one until the second call asks for it."""
    global _eval_box_cache
    versions = (entity_embed._version, center_embed._version, offset_embed._version)
    c = _eval_box_cache
    _eval_box_cache = None
    if (c is not None and c[0] is entity_embed and c[1] is center_embed and c[2] is offset_embed and
            c[3] == versions and c[4] != which):
        return c[5]
    d_out, d_in = _dist("box_both", entity_embed, center_embed, offset_embed)
    if which == "out":
        _eval_box_cache = (entity_embed, center_embed, offset_embed, versions, "out", d_in)
        return d_out
    _eval_box_cache = (entity_embed, center_embed, offset_embed, versions, "in", d_out)
    return d_in


def _box_one(which, entity_embed, center_embed, offset_embed):
    if not isinstance(entity_embed, LazyRows):
        if (not torch.is_grad_enabled() and entity_embed.dim() == 3 and center_embed.dim() == 3
                and entity_embed.is_cuda):
            return _box_one_eval(which, entity_embed, center_embed, offset_embed)
        return _dist("box_" + which, entity_embed, center_embed, offset_embed)
    # Query2box asks for "out" and then "in" of the same operands (box.py:160-161).  For table rows
    # the first request computes both in one pass and parks the other result on the handle.
    cache = entity_embed._box_cache
    if cache is not None and cache[0] is center_embed and cache[1] is offset_embed and cache[2] != which:
        entity_embed._box_cache = None
        return cache[3]
    d_out, d_in = _dist("box_both", entity_embed, center_embed, offset_embed)
    if which == "out":
        entity_embed._box_cache = (center_embed, offset_embed, "out", d_in)
        return d_out
    entity_embed._box_cache = (center_embed, offset_embed, "in", d_out)
    return d_in


def box_dist_out(entity_embed, center_embed, offset_embed):
    return _box_one("out", entity_embed, center_embed, offset_embed)


def box_dist_in(entity_embed, center_embed, offset_embed):
    return _box_one("in", entity_embed, center_embed, offset_embed)
