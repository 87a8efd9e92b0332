"""Query-embedding front half: the relation projections of a batch of path queries as one op
(smore_path_project_* / smore_path_embed_* in libsmore_b200.so), in place of the per-hop loop of the
reference (kg_reasoning.py:229-236 calling vec.py:58-60, box.py:126-129, rotate.py:101-109,
complex.py:108-117, distmult.py:106-111), optionally starting from table rows named by index so that
the anchor rows are never gathered (kg_reasoning.py:217-250)."""
import torch

from . import _lib
from .embedding import LazyRows


class _PathProjectFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, start_center, start_offset, rel_table, off_table, rel_ids, relu_offset):
        start_center = start_center.contiguous()
        start_offset = None if start_offset is None else start_offset.contiguous()
        B, D = start_center.shape
        H = rel_ids.shape[1]
        dev = start_center.device
        center = torch.empty_like(start_center)
        offset = torch.empty_like(start_center) if off_table is not None else None
        ptr = lambda t: None if t is None else t.data_ptr()
        with torch.cuda.device(dev), _lib.timed("path_project"):
            _lib.check(_lib.lib().smore_path_project_forward(
                start_center.data_ptr(), ptr(start_offset), rel_table.data_ptr(), ptr(off_table), rel_table.shape[0],
                rel_ids.data_ptr(), rel_ids.stride(0), B, H, D, int(relu_offset), center.data_ptr(), ptr(offset),
                torch.cuda.current_stream(dev).cuda_stream), "smore_path_project_forward")
        ctx.save_for_backward(rel_ids, rel_table, off_table if off_table is not None else rel_table)
        ctx.has_off, ctx.relu_offset, ctx.had_start_offset = off_table is not None, bool(relu_offset), start_offset is not None
        ctx.sizes = (B, H, D)
        if offset is None:
            return center
        return center, offset

    @staticmethod
    def backward(ctx, g_center, g_offset=None):
        rel_ids, rel_table, off_table = ctx.saved_tensors
        B, H, D = ctx.sizes
        dev = rel_table.device
        g_center = g_center.contiguous()
        g_offset = g_offset.contiguous() if (ctx.has_off and g_offset is not None) else None
        g_rel = torch.empty_like(rel_table)
        g_off = torch.empty_like(off_table) if g_offset is not None else None
        ptr = lambda t: None if t is None else t.data_ptr()
        with torch.cuda.device(dev), _lib.timed("path_project_backward"):
            _lib.check(_lib.lib().smore_path_project_backward(
                g_center.data_ptr(), ptr(g_offset), off_table.data_ptr() if ctx.has_off else None, rel_table.shape[0],
                rel_ids.data_ptr(), rel_ids.stride(0), B, H, D, int(ctx.relu_offset), g_rel.data_ptr(), ptr(g_off),
                torch.cuda.current_stream(dev).cuda_stream), "smore_path_project_backward")
        return (g_center, g_offset if ctx.had_start_offset else None, g_rel, g_off, None, None)


def project_path(start_center, rel_table, rel_ids, start_offset=None, off_table=None, relu_offset=False):
    """All relation projections of a batch of path queries.

    start_center [B, D]   embedding the path starts from (anchor rows, or an intersection's output)
    rel_table    [R, D]   relation embedding table (dense parameter)
    rel_ids      [B, H]   int64 relation ids of the H hops; may be a column block of the query matrix
    start_offset / off_table  the box-offset part of Query2box (start_offset None = zeros)
    Returns center [B, D], or (center, offset) when off_table is given.
    """
    if rel_ids.dim() != 2 or rel_ids.dtype != torch.int64 or rel_ids.stride(1) != 1:
        raise ValueError("rel_ids must be an int64 [B, H] tensor with unit stride along the hops")
    for t in (start_center, rel_table, off_table, start_offset):
        if t is not None and (not t.is_cuda or t.dtype != torch.float32):
            raise TypeError("project_path takes float32 CUDA tensors")
    if start_center.dim() != 2 or rel_table.dim() != 2 or start_center.shape[1] != rel_table.shape[1]:
        raise ValueError("start_center [B, D] and rel_table [R, D] must share D")
    if rel_ids.shape[0] != start_center.shape[0]:
        raise ValueError("one row of relation ids per query")
    if off_table is not None and off_table.shape != rel_table.shape:
        raise ValueError("off_table must have the shape of rel_table")
    if not rel_table.is_contiguous() or (off_table is not None and not off_table.is_contiguous()):
        raise ValueError("relation tables must be contiguous")
    return _PathProjectFunc.apply(start_center, start_offset, rel_table, off_table, rel_ids, relu_offset)


class _PathEmbedFunc(torch.autograd.Function):
    """project_path for the multiplicative geometries and / or a start given as table rows."""

    @staticmethod
    def forward(ctx, geometry, start, dummy, start_offset, rel_table, off_table, rel_ids, relu_offset, phase_scale):
        lazy = isinstance(start, LazyRows)
        if lazy:
            owner, lookup = start.owner, start.lookup
            rows, row_ids = owner.rows_operands(lookup)
            B, W = lookup.n, rows.shape[1]
            n_start = rows.shape[0]
        else:
            rows, row_ids = start.contiguous(), None
            B, W = rows.shape
            n_start = 0
        two = geometry in ("rotate", "complex")
        D = W // 2 if two else W
        H = rel_ids.shape[1]
        dev = rows.device
        out0 = torch.empty(B, D, dtype=torch.float32, device=dev)
        need1 = two or (geometry == "add" and off_table is not None)
        out1 = torch.empty_like(out0) if need1 else None
        start_offset = None if start_offset is None else start_offset.contiguous()
        ptr = lambda t: None if t is None else t.data_ptr()
        with torch.cuda.device(dev), _lib.timed("path_project"):
            _lib.check(_lib.lib().smore_path_embed_forward(
                _lib.GEOMETRY_IDS[geometry], rows.data_ptr(), ptr(row_ids), n_start, ptr(start_offset),
                rel_table.data_ptr(), ptr(off_table), rel_table.shape[0], rel_ids.data_ptr(), rel_ids.stride(0), B, H, D,
                int(relu_offset), float(phase_scale), out0.data_ptr(), ptr(out1),
                torch.cuda.current_stream(dev).cuda_stream), "smore_path_embed_forward")
        ctx.geometry, ctx.lazy, ctx.start = geometry, lazy, start if lazy else None
        ctx.sizes, ctx.relu_offset, ctx.phase_scale = (B, H, D, W), bool(relu_offset), float(phase_scale)
        ctx.has_off, ctx.had_start_offset = off_table is not None, start_offset is not None
        keep = [rel_ids, rel_table, off_table if off_table is not None else rel_table]
        if not lazy:
            keep.append(rows)
        ctx.save_for_backward(*keep)
        return out0 if out1 is None else (out0, out1)

    @staticmethod
    def backward(ctx, g0, g1=None):
        saved = ctx.saved_tensors
        rel_ids, rel_table, off_table = saved[:3]
        B, H, D, W = ctx.sizes
        dev = rel_table.device
        g0 = g0.contiguous()
        g1 = None if g1 is None else g1.contiguous()
        g_rel = torch.empty_like(rel_table)
        g_off = torch.empty_like(off_table) if (ctx.has_off and g1 is not None and ctx.geometry == "add") else None
        ptr = lambda t: None if t is None else t.data_ptr()
        if ctx.lazy:
            owner, lookup = ctx.start.owner, ctx.start.lookup
            rows, row_ids = owner.rows_operands(lookup)
            plan = owner.plan_for(lookup)
            counts_ptr = None if lookup.received else plan.counts.data_ptr()
            lookup.received = True
            slot, g_rows, g_start, n_start = plan.slot_of(lookup), plan.g_rows, None, rows.shape[0]
        else:
            rows, row_ids, slot, g_rows, counts_ptr, n_start = saved[3], None, None, None, None, 0
            g_start = torch.empty(B, W, dtype=torch.float32, device=dev) if ctx.geometry != "add" else None
        with torch.cuda.device(dev), _lib.timed("path_project_backward"):
            _lib.check(_lib.lib().smore_path_embed_backward(
                _lib.GEOMETRY_IDS[ctx.geometry], g0.data_ptr(), ptr(g1), rows.data_ptr(), ptr(row_ids), n_start,
                rel_table.data_ptr(), off_table.data_ptr() if ctx.has_off else None, rel_table.shape[0],
                rel_ids.data_ptr(), rel_ids.stride(0), B, H, D, int(ctx.relu_offset), ctx.phase_scale, g_rel.data_ptr(),
                ptr(g_off), ptr(g_start), ptr(slot), counts_ptr, ptr(g_rows),
                torch.cuda.current_stream(dev).cuda_stream), "smore_path_embed_backward")
        if not ctx.lazy and ctx.geometry == "add":
            g_start = g0
        g_start_offset = g1 if (ctx.had_start_offset and ctx.geometry == "add") else None
        return (None, None if ctx.lazy else g_start, None, g_start_offset, g_rel, g_off, None, None, None)


def embed_path(geometry, start, rel_table, rel_ids, start_offset=None, off_table=None, relu_offset=False,
               phase_scale=1.0):
    """All relation projections of a batch of path queries, any geometry.

    geometry     "add" (GQE, Query2box), "rotate" (RotatE), "complex" (ComplEx), "distmult" (DistMult)
    start        the state the paths start from: a float32 CUDA tensor [B, W], or a LazyRows handle (an
                 anchor lookup listed in the optimizer's lazy_names): the rows are then read from the
                 table in place and their gradient goes into the step's compact buffer.  W = D for
                 "add" / "distmult", 2 D ([re | im]) for "rotate" / "complex"
    rel_table    [R, D] ("complex": [R, 2 D] rows [re | im]; "rotate": phases, multiplied by phase_scale)
    rel_ids      [B, H] int64 relation ids of the H hops (a column block of the query matrix)
    start_offset / off_table / relu_offset   the box-offset part of Query2box ("add" only)
    Returns: "add": center, or (center, offset) with off_table; "rotate" / "complex": (re, im); "distmult": one tensor.
    """
    if geometry not in _lib.GEOMETRY_IDS:
        raise ValueError("geometry must be one of %s" % sorted(_lib.GEOMETRY_IDS))
    if rel_ids.dim() != 2 or rel_ids.dtype != torch.int64 or rel_ids.stride(1) != 1:
        raise ValueError("rel_ids must be an int64 [B, H] tensor with unit stride along the hops")
    lazy = isinstance(start, LazyRows)
    tensors = [rel_table, off_table, start_offset] + ([] if lazy else [start])
    for t in tensors:
        if t is not None and (not t.is_cuda or t.dtype != torch.float32):
            raise TypeError("embed_path takes float32 CUDA tensors")
    width = start.shape[-1]
    two = geometry in ("rotate", "complex")
    D = width // 2 if two else width
    if (two and width % 2) or rel_table.dim() != 2 or rel_table.shape[1] != (2 * D if geometry == "complex" else D):
        raise ValueError("start rows of width %d do not match a relation table %s for geometry %r"
                         % (width, tuple(rel_table.shape), geometry))
    n = start.lookup.n if lazy else start.shape[0]
    if (not lazy and start.dim() != 2) or rel_ids.shape[0] != n:
        raise ValueError("one start row and one row of relation ids per query")
    if geometry != "add" and (off_table is not None or start_offset is not None):
        raise ValueError("offsets belong to the additive geometry")
    if off_table is not None and off_table.shape != rel_table.shape:
        raise ValueError("off_table must have the shape of rel_table")
    if not rel_table.is_contiguous() or (off_table is not None and not off_table.is_contiguous()):
        raise ValueError("relation tables must be contiguous")
    dummy = start.owner.dummy_tensor if lazy else None
    return _PathEmbedFunc.apply(geometry, start, dummy, start_offset, rel_table, off_table, rel_ids, relu_offset,
                                phase_scale)
