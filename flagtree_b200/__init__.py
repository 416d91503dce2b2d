"""B200-native (sm_100a) kernels for FlagTree's sparse-MLA forward and GEMM + reduce-scatter.

The product is the C-ABI library `libflagtree_b200.so` (include/flagtree_b200.h); this package
is the thin Python mirror of the reference's operator wrappers on top of it.
"""
from .ops import (AgGemmContext, GemmRsContext, ag_gemm, decode_attention_fwd, gemm_rs, gemm_rs_close_all, gemm_rs_fp8,  # noqa: F401
                  kv_cache_write_fp8, matmul, matmul_fp8_blockscaled, shard_indices, sparse_mla_fwd,
                  sparse_mla_fwd_host, sparse_mla_fwd_paged, sparse_mla_merge, topk_indices)

__all__ = ["sparse_mla_fwd", "sparse_mla_fwd_host", "sparse_mla_fwd_paged", "sparse_mla_merge", "shard_indices", "topk_indices",
           "decode_attention_fwd", "kv_cache_write_fp8", "matmul", "matmul_fp8_blockscaled", "gemm_rs", "gemm_rs_fp8",
           "gemm_rs_close_all", "GemmRsContext", "ag_gemm", "AgGemmContext"]
