"""CPU oracle for the row-parallel GEMM fused with reduce-scatter (TEST INFRASTRUCTURE).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.

The reference ships no collective at all, so the cross-rank part is defined mathematically:
C = sum_r A_r @ B_r with fp32 accumulation, rank r keeps rows [r*M/tp, (r+1)*M/tp).  The
per-rank product follows the reference's dense matmul conventions:

* python/triton/ops/matmul.py:184-190 -- bf16/fp16 inputs accumulate in fp32;
* python/test/unit/operators/test_matmul.py:187-199 -- golden = torch.matmul on the same
  inputs;
* python/test/unit/language/test_core.py:5130-5136 -- fp8 e4m3 inputs are promoted to fp32
  before the golden product.

Block scales for the FP8 variant (1x128 along K for A, 128x128 for B) do not exist in the
reference op; this oracle is their definition ("parity unpinned").
"""
from __future__ import annotations

from typing import List, Sequence

import torch


def _f32(x: torch.Tensor) -> torch.Tensor:
    return x.detach().to("cpu").to(torch.float32)


def gemm_rs_ref(a_ranks: Sequence[torch.Tensor], b_ranks: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    """a_ranks[r] [M, K/tp], b_ranks[r] [K/tp, N] -> list of tp fp32 shards [M/tp, N].

    The cross-rank sum is taken in rank order 0..tp-1 in fp32.
    """
    tp = len(a_ranks)
    total = None
    for a, b in zip(a_ranks, b_ranks):
        part = torch.matmul(_f32(a), _f32(b))
        total = part if total is None else total + part
    m = total.shape[0]
    assert m % tp == 0
    return list(total.chunk(tp, dim=0))


def gemm_rs_rows_ref(a_ranks: Sequence[torch.Tensor], b_ranks: Sequence[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
    """Rows `rows` (global row numbers) of C = sum_r A_r @ B_r in fp32, rank order: the same definition as
    `gemm_rs_ref`, for spot checks at sizes where the whole product is too much CPU work."""
    total = None
    for a, b in zip(a_ranks, b_ranks):
        part = torch.matmul(_f32(a[rows]), _f32(b))
        total = part if total is None else total + part
    return total


def ag_gemm_ref(a_shards: Sequence[torch.Tensor], b_rank: torch.Tensor) -> torch.Tensor:
    """All-gather + GEMM: a_shards[r] [M/tp, K] stacked in rank order, times this rank's B [K, N_local], fp32.
    The dense product follows python/test/unit/operators/test_matmul.py:187-199 (golden = torch.matmul); the
    reference has no collective, so the gather is defined here: rows of rank r are rows [r*M/tp, (r+1)*M/tp)."""
    return torch.matmul(torch.cat([_f32(a) for a in a_shards], dim=0), _f32(b_rank))


def dequant_block_scaled(x_u8: torch.Tensor, scale: torch.Tensor, block_r: int, block_c: int) -> torch.Tensor:
    """e4m3 bytes [R, C] with one fp32 scale per (block_r x block_c) block -> fp32 [R, C]."""
    if x_u8.dtype != torch.uint8:
        x_u8 = x_u8.view(torch.uint8)
    x = x_u8.detach().to("cpu").view(torch.float8_e4m3fn).to(torch.float32)
    s = _f32(scale)
    s = s.repeat_interleave(block_r, dim=0)[: x.shape[0]]
    s = s.repeat_interleave(block_c, dim=1)[:, : x.shape[1]]
    return x * s


def gemm_rs_fp8_ref(a_ranks, a_scales, b_ranks, b_scales) -> List[torch.Tensor]:
    """FP8 e4m3 A [M,K/tp] with a_scale [M,(K/tp)/128]; B [K/tp,N] with b_scale [(K/tp)/128,N/128].

    C = sum_r sum_kb (A_r[:,kb] @ B_r[kb,:]) * a_scale[:,kb] (x) b_scale[kb,:/128], which equals
    the product of the dequantised operands.
    """
    a_deq = [dequant_block_scaled(a, s, 1, 128) for a, s in zip(a_ranks, a_scales)]
    b_deq = [dequant_block_scaled(b, s, 128, 128) for b, s in zip(b_ranks, b_scales)]
    return gemm_rs_ref(a_deq, b_deq)


def gemm_rs_flops_per_rank(m: int, n: int, k_local: int) -> int:
    return 2 * m * n * k_local
