"""Helpers shared by the tests: input generators, tolerance rule, C-ABI header parsing."""
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

OPS = ["l1", "l2", "box_out", "box_in", "rotate", "complex", "distmult"]
TWO_PART_ROWS = {"rotate", "complex"}
TWO_QUERY = {"box_out", "box_in", "rotate", "complex"}

# fp32 contract: 1e-5 relative where a sum is only re-associated, 1e-4 where atomic
# accumulation reorders it.  `scale` is the magnitude the absolute part is relative to.
RTOL = 1e-5
RTOL_ATOMIC = 1e-4


def close(got, want, rtol=RTOL, scale=None, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    if scale is None:
        scale = float(np.abs(want).max()) if want.size else 0.0
    np.testing.assert_allclose(got, want, rtol=rtol, atol=rtol * max(scale, 1e-30), err_msg=what)


def make_operands(op, be, ne, bc, nc, dim, seed, value_range=0.3):
    rng = np.random.default_rng(seed)
    mul = 2 if op in TWO_PART_ROWS else 1
    ent = rng.uniform(-value_range, value_range, (be, ne, dim * mul)).astype(np.float32)
    q0 = rng.uniform(-value_range, value_range, (bc, nc, dim)).astype(np.float32)
    q1 = None
    if op in TWO_QUERY:
        if op.startswith("box"):
            q1 = rng.uniform(0, value_range, (bc, nc, dim)).astype(np.float32)
        else:
            q1 = rng.uniform(-value_range, value_range, (bc, nc, dim)).astype(np.float32)
    return ent, q0, q1


def forward_scale(oracle, op, ent, q0, q1):
    """Magnitude of the summed |terms| (bounds the rounding error of any summation order)."""
    if op in ("complex", "distmult"):
        return float(oracle.dist_forward(op, np.abs(ent), np.abs(q0), None if q1 is None else np.abs(q1)).max())
    return float(np.abs(oracle.dist_forward(op, ent, q0, q1)).max())


def header_functions():
    """Names of all functions include/smore_b200.h declares."""
    text = open(os.path.join(ROOT, "include", "smore_b200.h")).read()
    return sorted(set(re.findall(r"SMORE_API\s+[\w\s\*]+?\b(smore_\w+)\s*\(", text)))
