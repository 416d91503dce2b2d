"""ctypes binding of libflagtree_b200.so.  Loading fails loudly: there is no CPU fallback."""
from __future__ import annotations

import ctypes as C
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libflagtree_b200.so")

FTB_OK, FTB_ERR_INVALID, FTB_ERR_CUDA, FTB_ERR_TIMEOUT, FTB_ERR_BAD_INDEX, FTB_ERR_UNSUPPORTED = range(6)
STATUS_NAMES = {0: "OK", 1: "INVALID", 2: "CUDA", 3: "TIMEOUT", 4: "BAD_INDEX", 5: "UNSUPPORTED"}


class SparseMlaArgs(C.Structure):
    """Mirror of `ftb_sparse_mla_args` (include/flagtree_b200.h)."""
    _fields_ = [
        ("q", C.c_void_p), ("kv", C.c_void_p), ("indices", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("s_q", C.c_int32), ("h", C.c_int32), ("s_kv", C.c_int32), ("topk", C.c_int32),
        ("q_stride_token", C.c_int64), ("q_stride_head", C.c_int64),
        ("kv_stride_row", C.c_int64),
        ("idx_stride_token", C.c_int64),
        ("out_stride_token", C.c_int64), ("out_stride_head", C.c_int64),
        ("lse_stride_token", C.c_int64),
        ("sm_scale", C.c_float), ("lse_base2", C.c_int32), ("algo_id", C.c_int32),
        ("status", C.c_void_p),
        ("kv_is_fp8", C.c_int32),
        ("kv_scale", C.c_void_p), ("block_table", C.c_void_p), ("context_lens", C.c_void_p),
        ("page_size", C.c_int32), ("q_per_seq", C.c_int32),
        ("block_table_stride", C.c_int64),
        ("dbg_scores", C.c_void_p),
        ("n_splits", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
    ]


class GemmArgs(C.Structure):
    """Mirror of `ftb_gemm_args`."""
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p),
                ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
                ("status", C.c_void_p)]


class GemmFp8Args(C.Structure):
    """Mirror of `ftb_gemm_fp8_args`."""
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p), ("a_scale", C.c_void_p), ("b_scale", C.c_void_p),
                ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("a_scale_ld", C.c_int64), ("b_scale_ld", C.c_int64),
                ("status", C.c_void_p), ("b_kmajor", C.c_int32)]


class SparseMlaMergeArgs(C.Structure):
    """Mirror of `ftb_sparse_mla_merge_args`."""
    _fields_ = [("part_out", C.c_void_p), ("part_lse", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
                ("s_q", C.c_int32), ("h", C.c_int32), ("n_parts", C.c_int32),
                ("part_is_fp32", C.c_int32), ("lse_base2", C.c_int32),
                ("part_stride_part", C.c_int64), ("part_stride_token", C.c_int64), ("part_stride_head", C.c_int64),
                ("lse_stride_part", C.c_int64), ("lse_stride_part_token", C.c_int64),
                ("out_stride_token", C.c_int64), ("out_stride_head", C.c_int64), ("lse_stride_token", C.c_int64)]


class KvCacheWriteArgs(C.Structure):
    """Mirror of `ftb_kv_cache_write_args`."""
    _fields_ = [("rows", C.c_void_p), ("slot_mapping", C.c_void_p), ("kv_cache", C.c_void_p), ("kv_scale", C.c_void_p),
                ("n_rows", C.c_int32), ("num_pages", C.c_int32), ("page_size", C.c_int32),
                ("row_stride", C.c_int64), ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
                ("status", C.c_void_p)]


class TopkArgs(C.Structure):
    """Mirror of `ftb_topk_args`."""
    _fields_ = [("scores", C.c_void_p), ("lengths", C.c_void_p), ("out", C.c_void_p),
                ("s_q", C.c_int32), ("s_kv", C.c_int32), ("topk", C.c_int32),
                ("scores_stride_token", C.c_int64), ("out_stride_token", C.c_int64)]


_lib = None
_lock = threading.Lock()


def load() -> C.CDLL:
    """Load the shared library once.  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m flagtree_b200.build` "
                    "(nvcc, sm_100a). flagtree_b200 has no CPU or PyTorch fallback.")
            lib = C.CDLL(LIB_PATH)
            lib.ftb_abi_version.restype = C.c_int
            lib.ftb_last_error_string.restype = C.c_char_p
            for name in declared_symbols():
                if not hasattr(lib, name):
                    raise RuntimeError(f"{LIB_PATH} does not export {name}; rebuild the library")
            lib.ftb_sparse_mla_fwd.argtypes = [C.POINTER(SparseMlaArgs), C.c_void_p]
            lib.ftb_sparse_mla_fwd.restype = C.c_int
            lib.ftb_sparse_mla_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32]
            lib.ftb_sparse_mla_workspace_bytes.restype = C.c_int64
            lib.ftb_sparse_mla_dequant_workspace_bytes.argtypes = [C.c_int32, C.c_int32]
            lib.ftb_sparse_mla_dequant_workspace_bytes.restype = C.c_int64
            lib.ftb_sparse_mla_fwd_static_scratch.argtypes = [C.POINTER(SparseMlaArgs), C.c_void_p]
            lib.ftb_sparse_mla_fwd_static_scratch.restype = C.c_int
            lib.ftb_sparse_mla_static_scratch_bytes.restype = C.c_int64
            if lib.ftb_sizeof_sparse_mla_args() != C.sizeof(SparseMlaArgs):
                raise RuntimeError("ftb_sparse_mla_args layout differs between the header and the Python mirror")
            if lib.ftb_sizeof_gemm_args() != C.sizeof(GemmArgs):
                raise RuntimeError("ftb_gemm_args layout differs between the header and the Python mirror")
            if lib.ftb_sizeof_sparse_mla_merge_args() != C.sizeof(SparseMlaMergeArgs):
                raise RuntimeError("ftb_sparse_mla_merge_args layout differs between the header and the Python mirror")
            lib.ftb_sparse_mla_merge.argtypes = [C.POINTER(SparseMlaMergeArgs), C.c_void_p]
            if lib.ftb_sizeof_kv_cache_write_args() != C.sizeof(KvCacheWriteArgs):
                raise RuntimeError("ftb_kv_cache_write_args layout differs between the header and the Python mirror")
            lib.ftb_kv_cache_write_fp8.argtypes = [C.POINTER(KvCacheWriteArgs), C.c_void_p]
            lib.ftb_kv_cache_write_workspace_bytes.argtypes = [C.c_int32]
            lib.ftb_kv_cache_write_workspace_bytes.restype = C.c_int64
            if lib.ftb_sizeof_topk_args() != C.sizeof(TopkArgs):
                raise RuntimeError("ftb_topk_args layout differs between the header and the Python mirror")
            lib.ftb_topk_indices.argtypes = [C.POINTER(TopkArgs), C.c_void_p]
            lib.ftb_gemm_bf16.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
            if lib.ftb_sizeof_gemm_fp8_args() != C.sizeof(GemmFp8Args):
                raise RuntimeError("ftb_gemm_fp8_args layout differs between the header and the Python mirror")
            lib.ftb_gemm_fp8_blockscaled.argtypes = [C.POINTER(GemmFp8Args), C.c_void_p]
            lib.ftb_gemm_rs_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
            lib.ftb_gemm_rs_ctx_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_int,
                                                   C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
            lib.ftb_gemm_rs_ctx_destroy.argtypes = [C.c_void_p]
            lib.ftb_gemm_rs_ctx_set_multicast.argtypes = [C.c_void_p, C.c_void_p]
            lib.ftb_gemm_rs_ctx_set_staged.argtypes = [C.c_void_p, C.c_int]
            lib.ftb_gemm_rs_ctx_set_wait_limit.argtypes = [C.c_void_p, C.c_int64]
            lib.ftb_gemm_rs_ctx_set_copy_engine.argtypes = [C.c_void_p, C.c_int]
            lib.ftb_gemm_rs.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64,
                                        C.c_int64, C.c_void_p, C.c_void_p]
            lib.ftb_gemm_rs_fp8.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                            C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
            lib.ftb_gemm_rs_fp8.restype = C.c_int
            lib.ftb_ag_gemm_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
            lib.ftb_ag_gemm_ctx_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_int,
                                                   C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
            lib.ftb_ag_gemm_ctx_set_wait_limit.argtypes = [C.c_void_p, C.c_int64]
            lib.ftb_ag_gemm_ctx_destroy.argtypes = [C.c_void_p]
            lib.ftb_ag_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64,
                                        C.c_int64, C.c_void_p, C.c_void_p]
            lib.ftb_ipc_alloc.argtypes = [C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_uint8)]
            lib.ftb_ipc_open.argtypes = [C.POINTER(C.c_uint8), C.POINTER(C.c_void_p)]
            lib.ftb_ipc_close.argtypes = [C.c_void_p]
            lib.ftb_ipc_free.argtypes = [C.c_void_p]
            _lib = lib
    return _lib


def declared_symbols():
    """Names of every function `include/flagtree_b200.h` declares (parsed from the header)."""
    import re
    hdr = os.path.join(_PKG, "..", "include", "flagtree_b200.h")
    with open(hdr) as f:
        text = f.read()
    return sorted(set(re.findall(r"FTB_API\s+[\w\s\*]+?\b(ftb_\w+)\s*\(", text)))


def last_error() -> str:
    s = load().ftb_last_error_string()
    return s.decode() if s else ""


def check(rc: int, what: str) -> None:
    """Map a C-ABI status to the exception types the reference's wrappers raise."""
    if rc == FTB_OK:
        return
    msg = f"{what}: {STATUS_NAMES.get(rc, rc)}: {last_error()}"
    if rc in (FTB_ERR_INVALID, FTB_ERR_UNSUPPORTED):
        raise ValueError(msg)
    raise RuntimeError(msg)
