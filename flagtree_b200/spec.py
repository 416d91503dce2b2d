"""Adapter for FlagTree's backend-specialisation hooks (`spec` / `spec_func`,
python/triton/runtime/driver.py:63-80).  A backend driver that sets `self.spec = flagtree_b200.spec`
routes the reference's `triton.ops.matmul` through the sm_100a GEMM: the hook at
python/triton/ops/matmul.py:218 calls `matmul_kernel(...)` and skips the Triton kernel when the return
value is truthy.  `ops_modify_all` (python/triton/ops/__init__.py:9-12) appends this package's ops.
"""
from __future__ import annotations

import torch

from . import ops

__all__ = ["matmul_kernel", "ops_modify_all"]


def matmul_kernel(grid, a, b, c, M, N, K, acc_dtype, input_precision, fp8_fast_accum, ab_dtype):
    """Writes A @ B into the caller-allocated `c`; returns True when it handled the call, None otherwise
    (None lets the reference's own kernel run, the convention of the hook)."""
    if not (a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and c.dtype == torch.bfloat16):
        return None
    if a.stride(1) != 1 or b.stride(1) != 1 or c.stride(1) != 1 or (N % 8) or (K % 8):
        return None
    ops._gemm_into(a, b, c)
    return True


def ops_modify_all(all_array):
    all_array += ["sparse_mla_fwd", "sparse_mla_fwd_paged", "sparse_mla_merge", "kv_cache_write_fp8", "gemm_rs", "gemm_rs_fp8", "ag_gemm", "topk_indices"]
    return all_array
