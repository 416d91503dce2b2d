"""GPU parity of the FP8 cache write path (through the C ABI) against its CPU restatement: bytes and scales must
agree bit for bit, for pages filled in one call, pages filled in several calls (the scale rises and the page is
requantised), skipped rows and untouched pages; and the cache it produces must feed the paged forward."""
import pytest
import torch

from conftest import LSE_RTOL, OUT_ATOL

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from flagtree_b200 import kv_cache_write_fp8, sparse_mla_fwd_paged
from oracle.sparse_mla_ref import kv_cache_write_fp8_ref, quantize_pages_e4m3_ref, sparse_mla_fwd_paged_ref

DEV = "cuda:0"


def _write_both(rows, slots, cache, scale, page):
    """One call on the GPU (in place on device copies) and one of the restatement; returns both results."""
    d_cache, d_scale = cache.to(DEV), scale.to(DEV)
    kv_cache_write_fp8(rows.to(DEV), slots.to(DEV), d_cache, d_scale, page, check=True)
    torch.cuda.synchronize()
    r_cache, r_scale = kv_cache_write_fp8_ref(rows, slots, cache, scale, page)
    return d_cache.cpu(), d_scale.cpu(), r_cache, r_scale


def test_whole_pages_in_one_call_bit_exact():
    g = torch.Generator().manual_seed(0)
    n_pages, page, d = 37, 64, 576
    x = (torch.randn(n_pages, page, d, generator=g) * torch.rand(n_pages, 1, 1, generator=g) * 4).bfloat16()
    perm = torch.randperm(n_pages * page, generator=g)
    cache0 = torch.zeros(n_pages, page, d, dtype=torch.uint8)
    scale0 = torch.zeros(n_pages)
    g_cache, g_scale, r_cache, r_scale = _write_both(x.view(-1, d)[perm], perm.int(), cache0, scale0, page)
    assert torch.equal(g_scale, r_scale)
    assert torch.equal(g_cache, r_cache)
    q_bytes, q_scale = quantize_pages_e4m3_ref(x.float())                 # the format's own definition
    assert torch.equal(g_scale, q_scale) and torch.equal(g_cache, q_bytes)


def test_incremental_fill_requantises_bit_exact():
    g = torch.Generator().manual_seed(1)
    n_pages, page, d = 6, 64, 576
    amp = torch.linspace(0.1, 5.0, page)[None, :, None]                   # later rows are larger: the scale rises
    x = (torch.randn(n_pages, page, d, generator=g) * amp).bfloat16().view(-1, d)
    cache, scale = torch.zeros(n_pages, page, d, dtype=torch.uint8), torch.zeros(n_pages)
    for step in range(8):                                                 # 8 rows of every page per call
        slots = torch.cat([torch.arange(pg * page + step * 8, pg * page + step * 8 + 8) for pg in range(n_pages)]).int()
        slots[3] = -1                                                     # a skipped row
        g_cache, g_scale, r_cache, r_scale = _write_both(x[slots.clamp(min=0).long()], slots, cache, scale, page)
        assert torch.equal(g_scale, r_scale), step
        assert torch.equal(g_cache, r_cache), step
        cache, scale = r_cache, r_scale
    assert (scale > 0).all()


def test_bad_slot_is_reported_and_zero_rows_is_a_no_op():
    cache = torch.zeros(2, 64, 576, dtype=torch.uint8, device=DEV)
    scale = torch.zeros(2, device=DEV)
    rows = torch.ones(1, 576, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="BAD_INDEX"):
        kv_cache_write_fp8(rows, torch.tensor([2 * 64 + 1], dtype=torch.int32, device=DEV), cache, scale, 64, check=True)
    assert (cache == 0).all() and (scale == 0).all()
    kv_cache_write_fp8(rows[:0], torch.zeros(0, dtype=torch.int32, device=DEV), cache, scale, 64, check=True)


def test_written_cache_feeds_the_paged_forward():
    """End of the decode chain: rows written by the GPU write path, read by the paged sparse-MLA forward."""
    g = torch.Generator().manual_seed(3)
    page, n_seq, h, topk = 64, 3, 128, 256
    lens = torch.tensor([300, 700, 1000])
    pages_per = (lens + page - 1) // page
    n_pages = int(pages_per.sum())
    perm = torch.randperm(n_pages, generator=g).int()
    block_table = torch.zeros(n_seq, int(pages_per.max()), dtype=torch.int32)
    rows, slots, off = [], [], 0
    for b in range(n_seq):
        n = int(pages_per[b])
        block_table[b, :n] = perm[off:off + n]
        off += n
        pos = torch.arange(int(lens[b]))
        rows.append(torch.randn(int(lens[b]), 576, generator=g).bfloat16())
        slots.append((block_table[b, pos // page].long() * page + pos % page).int())
    rows, slots = torch.cat(rows), torch.cat(slots)
    cache = torch.zeros(n_pages, page, 576, dtype=torch.uint8, device=DEV)
    scale = torch.zeros(n_pages, device=DEV)
    half = rows.shape[0] // 2                                             # two calls: prefill in two chunks
    kv_cache_write_fp8(rows[:half].to(DEV), slots[:half].to(DEV), cache, scale, page, check=True)
    kv_cache_write_fp8(rows[half:].to(DEV), slots[half:].to(DEV), cache, scale, page, check=True)
    q = torch.randn(n_seq, 2, h, 576, generator=g).bfloat16()
    idx = torch.stack([torch.stack([torch.randperm(int(lens[b]), generator=g)[:topk] for _ in range(2)]) for b in range(n_seq)]).int()
    out, lse = sparse_mla_fwd_paged(q.to(DEV), cache, scale, block_table.to(DEV), lens.int().to(DEV), idx.to(DEV), 0.07,
                                    page_size=page, check=True, num_splits=1)
    ref_out, ref_lse = sparse_mla_fwd_paged_ref(q, cache.cpu(), scale.cpu(), block_table, lens.int(), idx, 0.07, page_size=page)
    assert (out.float().cpu() - ref_out).abs().max().item() <= OUT_ATOL
    assert ((lse.cpu() - ref_lse).abs() / ref_lse.abs().clamp(min=1)).max().item() <= LSE_RTOL
    # and the values it holds are the rows, within e4m3 precision (two roundings at most)
    from oracle.sparse_mla_ref import e4m3_decode
    deq = (e4m3_decode(cache.cpu()) * scale.cpu()[:, None, None]).view(-1, 576)[slots.long()]
    assert ((deq - rows.float()).abs() <= rows.float().abs() * 2 ** -3 + scale.cpu().max() * 2 ** -9).all()
