"""CPU oracle for the top-k sparse MLA forward (TEST INFRASTRUCTURE, not product code).

This module is the checker: only tests, the smoke check and the benchmark's CPU-baseline
leg may import it.  The product path (flagtree_b200.ops) never does.

It restates, in fp32 torch on the CPU, the arithmetic of the reference's gather-by-index
MLA decode attention:

* third_party/mthreads/python/test/wmma/test_accuracy_musa_vllm_mla.py:206-337
  (_fwd_grouped_kernel_stage1): token-table gather, q.k over 512 latent + 64 rope dims,
  scale, -inf mask past the valid length, natural-exp online softmax, p.v over the first
  512 dims of the same latent row, stores acc/e_sum and e_max+log(e_sum).
* same file :426-477 (_fwd_kernel_stage2): merge of the per-split partial results.

Parity status: the reference holds no stored golden answers for this path (its tests compare
two code paths of the same kernel).  The restatement is pinned against the reference's own
kernel source executed by a CPU interpreter on small fp16 cases; the outputs of that run are
committed under tests/golden/ together with the script that made them.  Three compositions
have no reference kernel at all and are defined by this oracle alone ("parity unpinned" for
them): top-k indices resolved *through* a page table, FP8 e4m3 KV with per-page scales, and
-1 padding entries (the reference takes a valid length instead).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

D_QK = 576
D_V = 512


def _as_f32(x: torch.Tensor) -> torch.Tensor:
    return x.detach().to("cpu").to(torch.float32)


def sparse_mla_fwd_ref(
    q: torch.Tensor,            # [S_q, h, 576]
    kv: torch.Tensor,           # [S_kv, 576]
    indices: torch.Tensor,      # [S_q, topk] int32, -1 = padding
    sm_scale: Optional[float] = None,
    d_v: int = D_V,
    *,
    round_p_to: Optional[torch.dtype] = None,
    chunk: int = 64,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 gather -> QK^T*scale -> mask -> logsumexp/softmax -> P.V[:, :d_v].

    Follows test_accuracy_musa_vllm_mla.py:276-337: scores are q.k over all 576 dims times
    sm_scale (:284-299), masked entries are -inf (:304), LSE is natural-log e_max+log(e_sum)
    (:331-337), output is acc/e_sum (:322-329).  `round_p_to=torch.bfloat16` reproduces the
    kernel's cast of p to the V dtype before the second dot (:317) and is a diagnostic mode;
    the parity gate uses exact fp32 p.
    Returns (out [S_q,h,d_v] fp32, lse [S_q,h] fp32).  A token with no valid index gives
    out = 0 and lse = -inf.
    """
    qf, kvf = _as_f32(q), _as_f32(kv)
    idx = indices.detach().to("cpu").to(torch.int64)
    s_q, h, d = qf.shape
    assert d == kvf.shape[-1]
    if sm_scale is None:
        sm_scale = d ** -0.5
    out = torch.zeros(s_q, h, d_v, dtype=torch.float32)
    lse = torch.full((s_q, h), -math.inf, dtype=torch.float32)
    for t0 in range(0, s_q, chunk):
        t1 = min(s_q, t0 + chunk)
        ii = idx[t0:t1]                                   # [c, topk]
        valid = (ii >= 0) & (ii < kvf.shape[0])
        rows = kvf[ii.clamp(min=0, max=kvf.shape[0] - 1)]  # [c, topk, 576]
        s = torch.einsum("chd,ckd->chk", qf[t0:t1], rows) * sm_scale
        s = s.masked_fill(~valid[:, None, :], -math.inf)
        l = torch.logsumexp(s, dim=-1)                    # [c, h]
        m = s.amax(dim=-1, keepdim=True)
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p = torch.exp(s - m)
        den = p.sum(dim=-1, keepdim=True)
        if round_p_to is not None:
            p = p.to(round_p_to).to(torch.float32)
        o = torch.einsum("chk,ckv->chv", p, rows[..., :d_v])
        o = torch.where(den > 0, o / den.clamp(min=1e-38), torch.zeros_like(o))
        out[t0:t1] = o
        lse[t0:t1] = l
    return out, lse


def e4m3_decode(raw_u8: torch.Tensor) -> torch.Tensor:
    """Decode e4m3fn bytes (uint8) to fp32 (OCP FP8 e4m3: bias 7, no inf, 0x7f/0xff NaN)."""
    return raw_u8.detach().to("cpu").view(torch.float8_e4m3fn).to(torch.float32)


def physical_rows(block_table: torch.Tensor, positions: torch.Tensor, page_size: int) -> torch.Tensor:
    """Logical position -> physical cache row: table[p // PAGE] * PAGE + p % PAGE.

    Same rule as test_accuracy_musa_vllm_mla.py:278-283 (kv_loc).  block_table [max_pages],
    positions [...] int64; negative positions stay negative (padding).
    """
    pos = positions.to(torch.int64)
    safe = pos.clamp(min=0)
    phys = block_table.to(torch.int64)[safe // page_size] * page_size + safe % page_size
    return torch.where(pos >= 0, phys, pos)


def sparse_mla_fwd_paged_ref(
    q: torch.Tensor,              # [B, n_q, h, 576] bf16
    kv_cache_u8: torch.Tensor,    # [num_pages, page, 576] e4m3 bytes (uint8 or float8_e4m3fn)
    kv_scale: torch.Tensor,       # [num_pages] fp32, value = fp8 * scale
    block_table: torch.Tensor,    # [B, max_pages] int32
    context_lens: torch.Tensor,   # [B] int32
    indices: torch.Tensor,        # [B, n_q, topk] int32 logical positions, -1 = padding
    sm_scale: Optional[float] = None,
    d_v: int = D_V,
    page_size: int = 64,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Paged FP8 variant: dequantise the gathered rows, then the same math as above.

    A logical index >= context_len is treated as padding.  Returns
    (out [B,n_q,h,d_v] fp32, lse [B,n_q,h] fp32).
    """
    if kv_cache_u8.dtype != torch.uint8:
        kv_cache_u8 = kv_cache_u8.view(torch.uint8)
    n_pages, page, d = kv_cache_u8.shape
    assert page == page_size
    deq = e4m3_decode(kv_cache_u8).reshape(n_pages, page, d) * _as_f32(kv_scale)[:, None, None]
    flat = deq.reshape(n_pages * page, d)
    b, n_q, h, _ = q.shape
    outs, lses = [], []
    for i in range(b):
        ii = indices[i].to("cpu").to(torch.int64)
        ii = torch.where(ii < int(context_lens[i]), ii, torch.full_like(ii, -1))
        phys = physical_rows(block_table[i].to("cpu"), ii, page_size)
        o, l = sparse_mla_fwd_ref(q[i], flat, phys.to(torch.int32), sm_scale, d_v)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


def merge_splits_ref(part_out: torch.Tensor, part_lse: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge per-split normalised partial outputs by their LSE.

    part_out [..., splits, d_v] fp32, part_lse [..., splits] fp32 (-inf = empty split).
    Follows _fwd_kernel_stage2 (test_accuracy_musa_vllm_mla.py:455-477): running max,
    acc = acc*exp(m-m') + exp(lse_k-m')*out_k, out = acc/sum.  The merged LSE (which the
    reference does not store) is logaddexp over the splits.
    """
    po, pl = _as_f32(part_out), _as_f32(part_lse)
    lse = torch.logsumexp(pl, dim=-1)
    m = pl.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(pl - m)
    den = w.sum(dim=-1, keepdim=True)
    out = (w[..., None] * po).sum(dim=-2)
    out = torch.where(den > 0, out / den.clamp(min=1e-38), torch.zeros_like(out))
    return out, lse


def sparse_mla_flops(indices: torch.Tensor, h: int, s_kv: Optional[int] = None) -> int:
    """Algorithmic work: 2*(576+512)*h*sum_t n_valid(t); padding is not counted."""
    valid = indices >= 0
    if s_kv is not None:
        valid = valid & (indices < s_kv)
    return 2 * (D_QK + D_V) * h * int(valid.sum())


E4M3_MAX = 448.0


def quantize_pages_e4m3_ref(kv_pages_f32: torch.Tensor):
    """[num_pages, page, d] fp32 -> (e4m3 bytes uint8, per-page scale = amax / 448 fp32, at least 1e-12 / 448):
    the definition of the paged FP8 cache format (value = e4m3 * scale[page]).  No reference kernel produces
    this format; the nearest is the int4 writer with per-group scale and zero point,
    third_party/hcu/python/test/unit/sglang/decode_attention_int4kv.py:934."""
    x = _as_f32(kv_pages_f32)
    amax = x.abs().amax(dim=(1, 2)).clamp(min=1e-12)
    scale = (amax / E4M3_MAX).to(torch.float32)
    qv = (x / scale[:, None, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return qv.view(torch.uint8), scale


def kv_cache_write_fp8_ref(rows: torch.Tensor, slot_mapping: torch.Tensor, kv_cache_u8: torch.Tensor,
                           kv_scale: torch.Tensor, page_size: int = 64):
    """CPU restatement of the cache write path; returns new (kv_cache_u8, kv_scale), inputs untouched.

    rows [n, d] (bf16 or fp32), slot_mapping [n] int (slot = page * page_size + position, -1 = skip, distinct),
    kv_cache_u8 [num_pages, page, d] e4m3 bytes, kv_scale [num_pages] fp32 with 0 = empty page.
    Per touched page: new = max(old, max|new rows of the page| / 448) with the maximum floored at 1e-12; if
    new > old and old > 0 every byte of the page is requantised as e4m3(decode(byte) * old / new); then the new
    rows are stored as e4m3(clamp(x / new, +-448)).  All arithmetic in fp32, divisions IEEE, conversion to e4m3
    round-to-nearest-even."""
    x = _as_f32(rows)
    slots = slot_mapping.detach().to("cpu").to(torch.int64)
    cache = kv_cache_u8.detach().to("cpu").clone()
    if cache.dtype != torch.uint8:
        cache = cache.view(torch.uint8)
    scale = _as_f32(kv_scale).clone()
    n_pages, page, d = cache.shape
    assert page == page_size
    keep = slots >= 0
    pages = slots[keep] // page_size
    row_amax = x[keep].abs().amax(dim=1).clamp(min=1e-12)
    cand = torch.zeros(n_pages, dtype=torch.float32)
    cand.scatter_reduce_(0, pages, (row_amax / E4M3_MAX).to(torch.float32), reduce="amax", include_self=True)
    for pg in torch.unique(pages).tolist():
        old, new = scale[pg].item(), cand[pg].item()
        if not new > old:
            continue
        if old > 0:
            dec = cache[pg].view(torch.float8_e4m3fn).to(torch.float32)
            re = ((dec * torch.tensor(old, dtype=torch.float32)) / torch.tensor(new, dtype=torch.float32))
            cache[pg] = re.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
        scale[pg] = new
    flat = cache.view(n_pages * page, d)
    qv = (x[keep] / scale[pages][:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
    flat[slots[keep]] = qv
    return cache, scale


def topk_indices_ref(scores: torch.Tensor, topk: int, lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
    """CPU restatement of the index producer: per token the positions of the `topk` largest scores among the first
    lengths[t] positions, ascending, padded with -1.  Floats are ordered through the usual order-preserving map to
    unsigned 32-bit keys (sign bit flipped for non-negative values, all bits for negative ones), so -0 < +0 and NaN
    patterns sort by their bits; ties go to the lower position (stable sort)."""
    import numpy as np
    sc = scores.detach().to("cpu").to(torch.float32).contiguous().numpy()
    s_q, s_kv = sc.shape
    u = sc.view(np.uint32)
    keys = np.where(u & np.uint32(0x80000000), ~u, u | np.uint32(0x80000000))
    out = np.full((s_q, topk), -1, dtype=np.int32)
    for t in range(s_q):
        n = s_kv if lengths is None else max(0, min(int(lengths[t]), s_kv))
        k = min(topk, n)
        if k == 0:
            continue
        # stable descending order: negate the key order by sorting (max - key) ascending with a stable sort
        order = np.argsort(np.uint32(0xFFFFFFFF) - keys[t, :n], kind="stable")[:k]
        out[t, :k] = np.sort(order).astype(np.int32)
    return torch.from_numpy(out)
