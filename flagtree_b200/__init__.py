"""B200-native (sm_100a) kernels for FlagTree's sparse-MLA forward and GEMM + reduce-scatter.

The product is the C-ABI library `libflagtree_b200.so` (include/flagtree_b200.h); this package
is the thin Python mirror of the reference's operator wrappers on top of it.
"""
from .ops import (GemmRsContext, decode_attention_fwd, gemm_rs, matmul, matmul_fp8_blockscaled,  # noqa: F401
                  sparse_mla_fwd, sparse_mla_fwd_host, sparse_mla_fwd_paged)

__all__ = ["sparse_mla_fwd", "sparse_mla_fwd_host", "sparse_mla_fwd_paged", "decode_attention_fwd", "matmul", "matmul_fp8_blockscaled", "gemm_rs", "GemmRsContext"]
