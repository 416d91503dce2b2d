"""CPU checks of the cache-write restatement (the checker of the GPU write path): filling whole pages in one call
reproduces the page quantiser that defines the format, and the format round-trips through the paged attention
oracle's dequantiser."""
import torch

from oracle.sparse_mla_ref import e4m3_decode, kv_cache_write_fp8_ref, quantize_pages_e4m3_ref


def test_one_call_fill_equals_page_quantiser():
    g = torch.Generator().manual_seed(0)
    n_pages, page, d = 5, 64, 576
    x = torch.randn(n_pages, page, d, generator=g).bfloat16()
    ref_bytes, ref_scale = quantize_pages_e4m3_ref(x.float())
    perm = torch.randperm(n_pages * page, generator=g)                    # rows arrive in any order
    cache0 = torch.zeros(n_pages, page, d, dtype=torch.uint8)
    scale0 = torch.zeros(n_pages)
    cache, scale = kv_cache_write_fp8_ref(x.view(-1, d)[perm], perm.int(), cache0, scale0, page)
    assert torch.equal(scale, ref_scale)
    assert torch.equal(cache, ref_bytes)
    assert (cache0 == 0).all() and (scale0 == 0).all()                    # inputs untouched


def test_incremental_fill_keeps_values_within_two_roundings():
    g = torch.Generator().manual_seed(1)
    page, d = 64, 576
    x = (torch.randn(page, d, generator=g) * torch.linspace(0.2, 3.0, page)[:, None]).bfloat16()   # growing rows
    cache = torch.zeros(1, page, d, dtype=torch.uint8)
    scale = torch.zeros(1)
    for lo in range(0, page, 16):                                         # four calls, the scale rises each time
        cache, scale = kv_cache_write_fp8_ref(x[lo:lo + 16], torch.arange(lo, lo + 16).int(), cache, scale, page)
    assert scale[0] == x.float().abs().max() / 448
    deq = e4m3_decode(cache[0]) * scale[0]
    # e4m3 keeps 3 mantissa bits: one rounding is within 2^-4 relative (or half a subnormal step), two within 2^-3
    err = (deq - x.float()).abs()
    bound = x.float().abs() * 2 ** -3 + scale[0] * 2 ** -9
    assert (err <= bound).all()


def test_skipped_rows_and_untouched_pages():
    g = torch.Generator().manual_seed(2)
    page, d = 64, 576
    x = torch.randn(3, d, generator=g).bfloat16()
    cache0 = torch.full((2, page, d), 7, dtype=torch.uint8)
    scale0 = torch.tensor([0.5, 0.25])
    cache, scale = kv_cache_write_fp8_ref(x, torch.tensor([-1, 70, -1]).int(), cache0, scale0, page)
    assert torch.equal(cache[0], cache0[0]) and scale[0] == 0.5           # page 0 untouched
    assert scale[1] == 0.25                                               # N(0,1) rows fit under 0.25 * 448
    changed = (cache[1] != cache0[1]).any(dim=1).nonzero().flatten().tolist()
    assert changed == [70 - 64]
