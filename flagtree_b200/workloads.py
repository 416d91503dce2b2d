"""Seeded synthetic inputs for the five benchmark configurations.

Every generator takes a `device` and a `scale` knob so that tests can build a small case with
the same value distributions and index structure as the full-size benchmark.  Seeds follow
`1000 * cfg + rank`.  No dataset is involved: all tensors are drawn from torch generators.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional

import torch

D_QK = 576
D_V = 512
SM_SCALE_CFG = 192 ** -0.5
E4M3_MAX = 448.0


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


@dataclasses.dataclass
class SparseMlaCase:
    q: torch.Tensor          # [S_q, h, 576] bf16
    kv: torch.Tensor         # [S_kv, 576] bf16
    indices: torch.Tensor    # [S_q, topk] int32, -1 padded
    sm_scale: float
    name: str

    @property
    def n_valid(self) -> int:
        return int((self.indices >= 0).sum())

    @property
    def flops(self) -> int:
        return 2 * (D_QK + D_V) * self.q.shape[1] * self.n_valid


def _distinct_topk(n_rows: int, pool: int, topk: int, g: torch.Generator, device) -> torch.Tensor:
    """Per row: `topk` distinct positions drawn uniformly from [0, pool)."""
    keys = torch.rand(n_rows, pool, generator=g, device=device)
    return keys.argsort(dim=1)[:, :topk].to(torch.int32)


def mla_cfg1(device="cpu", s_q: int = 128, h: int = 16, s_kv: int = 4096, topk: int = 256,
             rank: int = 0) -> SparseMlaCase:
    """CPU-runnable case: uniform distinct indices, no padding."""
    g = _gen(1000 * 1 + rank, device)
    q = torch.randn(s_q, h, D_QK, generator=g, device=device).to(torch.bfloat16)
    kv = torch.randn(s_kv, D_QK, generator=g, device=device).to(torch.bfloat16)
    idx = _distinct_topk(s_q, s_kv, topk, g, device)
    return SparseMlaCase(q, kv, idx, SM_SCALE_CFG, f"mla_cfg1_sq{s_q}_h{h}_topk{topk}_skv{s_kv}")


def causal_topk_indices(s_q: int, topk: int, g: torch.Generator, device, t0: int = 0) -> torch.Tensor:
    """Token t picks min(t+1, topk) distinct positions from [0, t], then -1 padding.

    `t0` offsets the token ids (used when a rank generates only its own token shard).
    """
    out = torch.full((s_q, topk), -1, dtype=torch.int32, device=device)
    step = 512
    for a in range(0, s_q, step):
        b = min(s_q, a + step)
        t = torch.arange(t0 + a, t0 + b, device=device)
        pool = int(t[-1]) + 1
        keys = torch.rand(b - a, pool, generator=g, device=device)
        keys = keys.masked_fill(torch.arange(pool, device=device)[None, :] > t[:, None], 2.0)
        order = keys.argsort(dim=1)[:, :topk]
        width = order.shape[1]
        n_t = torch.clamp(t + 1, max=topk)
        keep = torch.arange(width, device=device)[None, :] < n_t[:, None]
        out[a:b, :width] = torch.where(keep, order, torch.full_like(order, -1)).to(torch.int32)
    return out


def mla_cfg2(device="cpu", s_q: int = 4096, s_kv: int = 4096, h: int = 128, topk: int = 2048,
             rank: int = 0) -> SparseMlaCase:
    """Prefill, DeepSeek-V3.2 shape: causal top-k with -1 padding.

    The latent KV is the same on every rank (it is replicated in a token-sharded run); `rank`
    only changes the seed of the query tokens and of their index lists, so each rank gets an
    independent batch of the same shape.
    """
    g = _gen(1000 * 2, device)
    kv = torch.randn(s_kv, D_QK, generator=g, device=device).to(torch.bfloat16)
    gq = _gen(1000 * 2 + 1 + rank, device)
    q = torch.randn(s_q, h, D_QK, generator=gq, device=device).to(torch.bfloat16)
    idx = causal_topk_indices(s_q, topk, gq, device)
    idx = torch.where(idx >= s_kv, torch.full_like(idx, -1), idx)
    return SparseMlaCase(q, kv, idx, SM_SCALE_CFG,
                         f"mla_cfg2_prefill_sq{s_q}_skv{s_kv}_h{h}_topk{topk}")


@dataclasses.dataclass
class PagedMlaCase:
    q: torch.Tensor             # [B, n_q, h, 576] bf16
    kv_cache: torch.Tensor      # [num_pages, page, 576] uint8 (e4m3 bytes)
    kv_scale: torch.Tensor      # [num_pages] fp32
    block_table: torch.Tensor   # [B, max_pages] int32
    context_lens: torch.Tensor  # [B] int32
    indices: torch.Tensor       # [B, n_q, topk] int32 logical positions
    sm_scale: float
    page_size: int
    name: str

    @property
    def flops(self) -> int:
        return 2 * (D_QK + D_V) * self.q.shape[2] * int((self.indices >= 0).sum())


def quantize_pages_e4m3(kv_pages_f32: torch.Tensor):
    """[num_pages, page, d] fp32 -> (e4m3 bytes uint8, per-page scale = amax/448 fp32)."""
    amax = kv_pages_f32.abs().amax(dim=(1, 2)).clamp(min=1e-12)
    scale = (amax / E4M3_MAX).to(torch.float32)
    qv = (kv_pages_f32 / scale[:, None, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return qv.view(torch.uint8), scale


def mla_cfg3(device="cpu", batch: int = 64, n_q: int = 2, h: int = 128, topk: int = 2048,
             len_lo: int = 8192, len_hi: int = 65536, page_size: int = 64, rank: int = 0) -> PagedMlaCase:
    """Decode over a paged FP8 latent cache with per-page scales."""
    g = _gen(1000 * 3 + rank, device)
    lens = torch.randint(len_lo, len_hi + 1, (batch,), generator=g, device=device)
    pages_per = (lens + page_size - 1) // page_size
    n_pages = int(pages_per.sum())
    max_pages = int(pages_per.max())
    perm = torch.randperm(n_pages, generator=g, device=device).to(torch.int32)
    block_table = torch.zeros(batch, max_pages, dtype=torch.int32, device=device)
    off = 0
    for b in range(batch):
        n = int(pages_per[b])
        block_table[b, :n] = perm[off:off + n]
        off += n
    cache = torch.empty(n_pages, page_size, D_QK, dtype=torch.uint8, device=device)
    scale = torch.empty(n_pages, dtype=torch.float32, device=device)
    step = 2048
    for a in range(0, n_pages, step):
        e = min(n_pages, a + step)
        blk = torch.randn(e - a, page_size, D_QK, generator=g, device=device)
        cache[a:e], scale[a:e] = quantize_pages_e4m3(blk)
    q = torch.randn(batch, n_q, h, D_QK, generator=g, device=device).to(torch.bfloat16)
    idx = torch.empty(batch, n_q, topk, dtype=torch.int32, device=device)
    for b in range(batch):
        L = int(lens[b])
        k = min(topk, L)
        sel = _distinct_topk(n_q, L, k, g, device)
        idx[b].fill_(-1)
        idx[b, :, :k] = sel
    return PagedMlaCase(q, cache, scale, block_table, lens.to(torch.int32), idx, SM_SCALE_CFG, page_size,
                        f"mla_cfg3_decode_b{batch}x{n_q}_h{h}_topk{topk}_fp8_page{page_size}")


@dataclasses.dataclass
class GemmRsCase:
    a: torch.Tensor   # [M, K/tp] this rank
    b: torch.Tensor   # [K/tp, N] this rank
    tp: int
    rank: int
    name: str
    a_scale: Optional[torch.Tensor] = None
    b_scale: Optional[torch.Tensor] = None

    @property
    def flops(self) -> int:
        return 2 * self.a.shape[0] * self.b.shape[1] * self.a.shape[1]


def gemm_cfg4(device="cpu", tp: int = 8, rank: int = 0, m: int = 8192, n: int = 7168,
              k_total: int = 18432) -> GemmRsCase:
    """bf16 row-parallel GEMM + reduce-scatter: entries ~ N(0,1)/sqrt(K)."""
    assert k_total % tp == 0
    k_loc = k_total // tp
    g = _gen(1000 * 4 + rank, device)
    s = k_total ** -0.5
    a = (torch.randn(m, k_loc, generator=g, device=device) * s).to(torch.bfloat16)
    b = (torch.randn(k_loc, n, generator=g, device=device) * s).to(torch.bfloat16)
    return GemmRsCase(a, b, tp, rank, f"gemm_rs_cfg4_tp{tp}_m{m}_n{n}_k{k_total}")


def quantize_block_e4m3(x: torch.Tensor, block_r: int, block_c: int):
    """fp32 [R, C] -> (e4m3 bytes, fp32 scales [R/block_r, C/block_c]); scale = amax/448."""
    r, c = x.shape
    assert r % block_r == 0 and c % block_c == 0
    xb = x.reshape(r // block_r, block_r, c // block_c, block_c)
    amax = xb.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale = (amax / E4M3_MAX).to(torch.float32)
    qv = (xb / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return qv.reshape(r, c).view(torch.uint8), scale


def gemm_cfg5(device="cpu", tp: int = 8, rank: int = 0, m: int = 4096, n: int = 8192,
              k_total: int = 28672) -> GemmRsCase:
    """FP8 e4m3 GEMM + reduce-scatter with 1x128 (A) and 128x128 (B) fp32 block scales."""
    assert k_total % tp == 0
    k_loc = k_total // tp
    assert k_loc % 128 == 0 and n % 128 == 0
    g = _gen(1000 * 5 + rank, device)
    a = torch.randn(m, k_loc, generator=g, device=device)
    b = torch.randn(k_loc, n, generator=g, device=device)
    a8, a_s = quantize_block_e4m3(a, 1, 128)
    b8, b_s = quantize_block_e4m3(b, 128, 128)
    return GemmRsCase(a8, b8, tp, rank, f"gemm_rs_fp8_cfg5_tp{tp}_m{m}_n{n}_k{k_total}", a_s, b_s)


def shard_bounds(n: int, world: int, rank: int):
    """Contiguous shard [lo, hi) of n units for `rank` of `world` (n need not divide)."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)
