"""The C-ABI library: it loads, exports every function the header declares, and rejects bad
arguments with error codes before touching the GPU (so these run without one)."""
import ctypes
import subprocess

import pytest

from tests.util import header_functions


@pytest.fixture(scope="module")
def lib():
    from smore_b200.csrc import build
    build.build()
    from smore_b200 import _lib
    return _lib


def test_header_and_binding_agree(lib):
    declared = header_functions()
    assert len(declared) >= 15
    assert sorted(lib.SIGNATURES) == declared


def test_library_exports_every_declared_symbol(lib):
    out = subprocess.run(["nm", "-D", "--defined-only", lib.LIB_PATH], capture_output=True, text=True, check=True)
    exported = {line.split()[-1] for line in out.stdout.splitlines() if " T " in line}
    missing = [f for f in header_functions() if f not in exported]
    assert not missing, missing
    handle = lib.lib()
    for f in header_functions():
        assert getattr(handle, f) is not None
    assert handle.smore_version().startswith(b"smore_b200")


def test_argument_errors_are_codes_not_exits(lib):
    L = lib.lib()
    # unknown distance id
    rc = L.smore_dist_forward(99, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 4, None)
    assert rc == -1 and b"unknown distance" in L.smore_last_error()
    # NULL operand
    rc = L.smore_dist_forward(3, None, None, None, None, 1, 1, 1, 1, 1, 1, 4, None)
    assert rc == -3
    # output not [max(be,bc), max(ne,nc)]
    rc = L.smore_dist_forward(3, 16, 16, None, 16, 2, 2, 4, 2, 1, 1, 4, None)
    assert rc == -2
    # operand sizes that do not divide the output
    rc = L.smore_dist_forward(3, 16, 16, None, 16, 6, 2, 6, 2, 4, 1, 4, None)
    assert rc == -2
    # box needs both query operands
    rc = L.smore_dist_forward(0, 16, 16, None, 16, 1, 1, 1, 1, 1, 1, 4, None)
    assert rc == -3
    # workspace checks of the unique-rows entry point
    need = L.smore_unique_rows_workspace_bytes(1000)
    assert need >= 2 * ((1000 + 31) // 32) * 4
    rc = L.smore_unique_rows(256, 4, 1000, 256, 256, 256, 256, None, 0, None)
    assert rc == -5
    rc = L.smore_unique_rows(256, 4, 1000, 256, 256, 256, 256, 512, 16, None)
    assert rc == -5 and b"workspace" in L.smore_last_error()
    rc = L.smore_sparse_update_rows(7, 256, 256, 256, 256, 256, 256, 4, 4, 0.1, 0.9, 0.999, 1e-8, 1, 0, None)
    assert rc == -1
    rc = L.smore_sparse_update_rows(1, 256, None, None, 256, 256, 256, 4, 4, 0.1, 0.9, 0.999, 1e-8, 1, 0, None)
    assert rc == -3


def test_missing_library_fails_loudly(lib, monkeypatch, tmp_path):
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(lib.SmoreError):
        lib.lib()


def test_cpu_tensors_are_rejected(lib):
    import torch
    from smore_b200 import ext_ops
    with pytest.raises(lib.SmoreError):
        ext_ops.l1_dist(torch.zeros(2, 3, 8), torch.zeros(2, 1, 8))
