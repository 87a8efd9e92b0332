"""smore_b200: B200 (sm_100a) distance ops and sparse row updates behind SMORE's op API.

    smore_b200.extlib_cuda   drop-in for the reference's `extlib_cuda` extension module
    smore_b200.ext_ops       the op set of smore/common/torchext/ext_ops.py (autograd functions)
    smore_b200.embedding     SparseEmbedding / EmbeddingOptimizer counterparts with table-resident
                             gathers, per-step de-duplication and fused row-wise optimizers
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
