"""CPU checks of the drop-in boundary: the library builds, loads, and exports every symbol that
include/flagtree_b200.h declares.  No compute call is made here."""
import ctypes
import os

import pytest

from flagtree_b200 import _lib, build


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_header_declares_entry_points():
    names = _lib.declared_symbols()
    assert "ftb_sparse_mla_fwd" in names and "ftb_abi_version" in names


def test_library_exports_every_declared_symbol(lib):
    for name in _lib.declared_symbols():
        assert hasattr(lib, name), name


def test_struct_mirror_matches(lib):
    assert lib.ftb_sizeof_sparse_mla_args() == ctypes.sizeof(_lib.SparseMlaArgs)


def test_argument_validation_without_gpu(lib):
    # NULL args and bad sizes are rejected on the host before any CUDA call.
    assert lib.ftb_sparse_mla_fwd(None, None) == _lib.FTB_ERR_INVALID
    a = _lib.SparseMlaArgs()
    a.s_q, a.h, a.s_kv, a.topk = 4, 0, 16, 8
    assert lib.ftb_sparse_mla_fwd(ctypes.byref(a), None) == _lib.FTB_ERR_INVALID
    assert "bad sizes" in _lib.last_error()
    a.h = 200
    assert lib.ftb_sparse_mla_fwd(ctypes.byref(a), None) == _lib.FTB_ERR_UNSUPPORTED
    a.h = 16
    assert lib.ftb_sparse_mla_fwd(ctypes.byref(a), None) == _lib.FTB_ERR_INVALID   # null tensors
    a.s_q = 0
    assert lib.ftb_sparse_mla_fwd(ctypes.byref(a), None) == _lib.FTB_OK             # empty input


def test_host_wrapper_rejects_cpu_tensors_and_bad_dtypes():
    import torch
    from flagtree_b200 import sparse_mla_fwd
    q = torch.zeros(2, 4, 576, dtype=torch.bfloat16)
    kv = torch.zeros(8, 576, dtype=torch.bfloat16)
    idx = torch.zeros(2, 4, dtype=torch.int32)
    with pytest.raises(ValueError):
        sparse_mla_fwd(q, kv, idx)


def test_no_product_import_of_oracle():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dirpath, _, files in os.walk(os.path.join(root, "flagtree_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
