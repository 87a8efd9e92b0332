"""Query-embedding front half for the additive geometries: the relation projections of a batch of
path queries as one op (smore_path_project_* in libsmore_b200.so), in place of the per-hop loop of
the reference (kg_reasoning.py:229-236 calling vec.py:58-60 / box.py:126-129)."""
import torch

from . import _lib


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
