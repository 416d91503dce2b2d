"""GPU parity tests of the sparse MLA forward: the CUDA path (through the C ABI) against the CPU
oracle on identical seeded inputs.  Tolerances are the benchmark contract's: bf16 output max-abs
error <= 2e-2, LSE relative error <= 1e-3 (relative to max(|lse|, 1))."""
import glob
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR, LSE_RTOL, OUT_ATOL

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from flagtree_b200 import decode_attention_fwd, sparse_mla_fwd, sparse_mla_fwd_paged
    from flagtree_b200 import workloads as W
from oracle.sparse_mla_ref import sparse_mla_fwd_paged_ref, sparse_mla_fwd_ref

DEV = "cuda:0"


def _errors(out, lse, ref_out, ref_lse):
    out = out.float().cpu()
    lse = lse.float().cpu()
    e_out = (out - ref_out).abs().max().item() if out.numel() else 0.0
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin), "finite/-inf pattern of LSE differs"
    if (~fin).any():
        assert (lse[~fin] == ref_lse[~fin]).all()
    e_lse = ((lse[fin] - ref_lse[fin]).abs() / ref_lse[fin].abs().clamp(min=1.0)).max().item() if fin.any() else 0.0
    return e_out, e_lse


# every bf16 kernel behind algo_id: 5 is what algo_id 0 selects
ALGOS = [1, 2, 3, 4, 5, 7]
ALGO_IDS = ["single_cta", "cta_pair", "cta_duo", "cta_duo_qtmem", "persistent", "persistent_64row"]


def _check(q, kv, idx, sm_scale, name="", algo=0):
    out, lse = sparse_mla_fwd(q.to(DEV), kv.to(DEV), idx.to(DEV), sm_scale, check=True, algo=algo)
    torch.cuda.synchronize()
    ref_out, ref_lse = sparse_mla_fwd_ref(q, kv, idx, sm_scale)
    e_out, e_lse = _errors(out, lse, ref_out, ref_lse)
    print(f"[{name}] out max-abs err {e_out:.3e}  lse rel err {e_lse:.3e}")
    assert torch.isfinite(out.float()).all()
    assert e_out <= OUT_ATOL, (name, e_out)
    assert e_lse <= LSE_RTOL, (name, e_lse)
    return out, lse


def test_scores_tap_matches_qk():
    """Raw Q.K^T scores of the first tiles (debug tap) against a direct fp32 product."""
    g = torch.Generator().manual_seed(1)
    s_q, h, s_kv, topk = 2, 128, 300, 128
    q = torch.randn(s_q, h, 576, generator=g).bfloat16()
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).int()
    dbg = torch.zeros(s_q, 128, topk, dtype=torch.float32, device=DEV)
    sparse_mla_fwd(q.to(DEV), kv.to(DEV), idx.to(DEV), 0.05, check=True, _dbg_scores=dbg)
    torch.cuda.synchronize()
    ref = torch.einsum("thd,tkd->thk", q.float(), kv.float()[idx.long()])
    err = (dbg.cpu() - ref).abs().max().item()
    print("scores tap max-abs err", err)
    assert err < 1e-2 * ref.abs().max().item()


GOLDEN = sorted(glob.glob(os.path.join(GOLDEN_DIR, "mla_topk_*.npz")))


@pytest.mark.parametrize("algo", ALGOS, ids=ALGO_IDS)
@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_golden_vectors_from_reference_kernel(path, algo):
    d = np.load(path)
    q = torch.from_numpy(d["q"]).to(torch.bfloat16)       # exact: fixtures hold bf16-representable values
    kv = torch.from_numpy(d["kv"]).to(torch.bfloat16)
    assert torch.equal(q.float(), torch.from_numpy(d["q"]).float())
    idx = torch.from_numpy(d["indices"])
    out, lse = sparse_mla_fwd(q.to(DEV), kv.to(DEV), idx.to(DEV), float(d["sm_scale"]), check=True, algo=algo)
    e_out, e_lse = _errors(out, lse, torch.from_numpy(d["out"]).float(), torch.from_numpy(d["lse"]).float())
    print(f"[golden {os.path.basename(path)}] out {e_out:.3e} lse {e_lse:.3e}")
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL


@pytest.mark.parametrize("algo", ALGOS, ids=ALGO_IDS)
def test_cfg1_cpu_runnable_case_full(algo):
    c = W.mla_cfg1()
    _check(c.q, c.kv, c.indices, c.sm_scale, c.name, algo)


@pytest.mark.parametrize("algo", ALGOS, ids=ALGO_IDS)
@pytest.mark.parametrize("h", [1, 16, 64, 65, 128])
@pytest.mark.parametrize("topk", [1, 37, 64, 200])
def test_head_counts_and_ragged_topk(h, topk, algo):
    g = torch.Generator().manual_seed(100 + h + topk)
    s_q, s_kv = 5, 333
    q = torch.randn(s_q, h, 576, generator=g).bfloat16()
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).int()
    _check(q, kv, idx, 576 ** -0.5, f"h{h}_topk{topk}_algo{algo}", algo)


@pytest.mark.parametrize("algo", ALGOS, ids=ALGO_IDS)
def test_padding_patterns(algo):
    """Trailing -1 padding, a token with no valid entry, one valid entry, and -1 in the middle."""
    g = torch.Generator().manual_seed(7)
    s_q, h, s_kv, topk = 6, 128, 500, 192
    q = torch.randn(s_q, h, 576, generator=g).bfloat16()
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).int()
    idx[0, 100:] = -1
    idx[1, :] = -1
    idx[2, 1:] = -1
    idx[3, 10:70] = -1            # a hole spanning a tile boundary
    idx[4, 0:64] = -1             # a fully masked first tile
    out, lse = _check(q, kv, idx, 0.07, "padding", algo)
    assert (out[1] == 0).all() and torch.isinf(lse[1]).all()
    # single selected row: the output is that row's first 512 values exactly (weight 1.0)
    assert torch.equal(out[2].cpu(), kv[idx[2, 0].item(), :512].expand(h, 512))


@pytest.mark.parametrize("algo", ALGOS, ids=ALGO_IDS)
def test_causal_prefill_shape_scaled_down(algo):
    c = W.mla_cfg2(s_q=192, s_kv=192, h=128, topk=128)
    _check(c.q, c.kv, c.indices, c.sm_scale, c.name, algo)
    c = W.mla_cfg2(s_q=300, s_kv=300, h=128, topk=512)      # more tiles than ring stages
    _check(c.q, c.kv, c.indices, c.sm_scale, c.name, algo)


def test_large_scores_are_stable():
    g = torch.Generator().manual_seed(3)
    # scores with a standard deviation near 100: the softmax is close to one-hot and the running
    # maximum moves by large steps between tiles (kv stays N(0,1) so that the absolute output
    # tolerance keeps its meaning)
    q = (torch.randn(3, 128, 576, generator=g) * 8).bfloat16()
    kv = torch.randn(256, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(256, generator=g)[:128] for _ in range(3)]).int()
    _check(q, kv, idx, 0.5, "large_scores_pair", 2)
    _check(q, kv, idx, 0.5, "large_scores_duo", 3)
    _check(q, kv, idx, 0.5, "large_scores_duo_qtmem", 4)
    _check(q, kv, idx, 0.5, "large_scores_single", 1)


def test_order_invariance_determinism_and_token_sharding():
    c = W.mla_cfg2(device=DEV, s_q=512, s_kv=512, h=128, topk=256)
    out, lse = sparse_mla_fwd(c.q, c.kv, c.indices, c.sm_scale, check=True)
    out2, lse2 = sparse_mla_fwd(c.q, c.kv, c.indices, c.sm_scale, check=True)
    assert torch.equal(out, out2) and torch.equal(lse, lse2), "two runs differ"
    # sharding query tokens across ranks must give bit-identical rows
    for lo, hi in ((0, 128), (128, 512)):
        o_s, l_s = sparse_mla_fwd(c.q[lo:hi], c.kv, c.indices[lo:hi], c.sm_scale, check=True)
        assert torch.equal(o_s, out[lo:hi]) and torch.equal(l_s, lse[lo:hi])
    # sharding heads: bit-identical columns
    o_h, l_h = sparse_mla_fwd(c.q[:, 16:32].contiguous(), c.kv, c.indices, c.sm_scale, check=True)
    assert torch.equal(o_h, out[:, 16:32]) and torch.equal(l_h, lse[:, 16:32])
    # permuting a token's index list changes only the summation order
    perm = torch.randperm(256, device=DEV)
    o_p, l_p = sparse_mla_fwd(c.q, c.kv, c.indices[:, perm].contiguous(), c.sm_scale, check=True)
    assert (o_p.float() - out.float()).abs().max().item() <= OUT_ATOL
    assert ((l_p - lse).abs() / lse.abs().clamp(min=1)).max().item() <= LSE_RTOL


def test_full_size_prefill_sampled_tokens():
    """cfg2 at full size (S_q = S_kv = 4096, h = 128, topk = 2048): every output is produced on the
    GPU; a seeded sample of tokens is compared with the CPU oracle, LSE of all tokens is checked
    for finiteness, and the all-tokens checksum is compared between two runs."""
    c = W.mla_cfg2(device=DEV)
    out, lse = sparse_mla_fwd(c.q, c.kv, c.indices, c.sm_scale, check=True)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    g = torch.Generator().manual_seed(5)
    sample = torch.cat([torch.tensor([0, 1, 63, 64, 2047, 2048, 4095]), torch.randint(0, 4096, (9,), generator=g)])
    ref_out, ref_lse = sparse_mla_fwd_ref(c.q[sample].cpu(), c.kv.cpu(), c.indices[sample].cpu(), c.sm_scale, chunk=4)
    e_out, e_lse = _errors(out[sample], lse[sample], ref_out, ref_lse)
    print(f"[cfg2 full, {len(sample)} sampled tokens] out {e_out:.3e} lse {e_lse:.3e}")
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL
    out2, _ = sparse_mla_fwd(c.q, c.kv, c.indices, c.sm_scale)
    assert torch.equal(out, out2)


def test_full_size_decode_fp8_sampled_sequences():
    """cfg3 at full size (64 sequences x 2 query tokens, h = 128, topk = 2048, paged FP8 cache with contexts of
    8192..65536 tokens): every output is produced on the GPU by the default path (selected rows dequantised
    once, then the persistent kernel); three sequences are cut out with their own pages and compared with
    the CPU oracle; the one-pass kernel must agree on all of them."""
    c = W.mla_cfg3(device=DEV)
    args = (c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens, c.indices, c.sm_scale)
    out, lse = sparse_mla_fwd_paged(*args, page_size=c.page_size, check=True)                 # two passes
    out1, lse1 = sparse_mla_fwd_paged(*args, page_size=c.page_size, check=True, num_splits=1, two_pass=False)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert (out.float() - out1.float()).abs().max().item() <= OUT_ATOL
    assert ((lse - lse1).abs() / lse1.abs().clamp(min=1)).max().item() <= LSE_RTOL
    for b in (0, 17, 63):
        n_pages = (int(c.context_lens[b]) + c.page_size - 1) // c.page_size
        pages = c.block_table[b, :n_pages].long()
        ref_out, ref_lse = sparse_mla_fwd_paged_ref(
            c.q[b:b + 1].cpu(), c.kv_cache[pages].cpu(), c.kv_scale[pages].cpu(),
            torch.arange(n_pages, dtype=torch.int32).view(1, -1), c.context_lens[b:b + 1].cpu(),
            c.indices[b:b + 1].cpu(), c.sm_scale, page_size=c.page_size)
        e_out, e_lse = _errors(out[b:b + 1], lse[b:b + 1], ref_out, ref_lse)
        print(f"[cfg3 full, sequence {b}] out {e_out:.3e} lse {e_lse:.3e}")
        assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL


def test_host_buffer_form_matches_device_form():
    """sparse_mla_fwd_host (pinned host tensors in and out, chunks of query tokens pipelined over three streams)
    gives the same bits as the device form, for a chunk size that does not divide the token count and for
    two calls in a row on the same staging buffers."""
    from flagtree_b200 import sparse_mla_fwd_host
    c = W.mla_cfg2(device="cpu", s_q=700, s_kv=1024, h=128, topk=512)
    out_d, lse_d = sparse_mla_fwd(c.q.to(DEV), c.kv.to(DEV), c.indices.to(DEV), c.sm_scale, check=True)
    hq, hkv, hidx = c.q.pin_memory(), c.kv.pin_memory(), c.indices.pin_memory()
    for _ in range(2):
        out_h, lse_h = sparse_mla_fwd_host(hq, hkv, hidx, c.sm_scale, device=torch.device(DEV), chunk_tokens=192)
        torch.cuda.synchronize()
        assert torch.equal(out_h, out_d.cpu()) and torch.equal(lse_h, lse_d.cpu())


def test_more_than_128_heads_and_strided_views():
    g = torch.Generator().manual_seed(11)
    q_big = torch.randn(3, 160, 640, generator=g).bfloat16()
    kv_big = torch.randn(100, 1, 640, generator=g).bfloat16()
    q, kv = q_big[:, :, :576], kv_big[:, :, :576]           # non-contiguous rows
    idx = torch.stack([torch.randperm(100, generator=g)[:70] for _ in range(3)]).int()
    out, lse = sparse_mla_fwd(q.to(DEV)[:, :, :], kv.to(DEV), idx.to(DEV), 0.05, check=True)
    ref_out, ref_lse = sparse_mla_fwd_ref(q, kv[:, 0], idx, 0.05)
    e_out, e_lse = _errors(out, lse, ref_out, ref_lse)
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL


def test_bad_index_is_reported_not_read():
    g = torch.Generator().manual_seed(2)
    q = torch.randn(1, 16, 576, generator=g).bfloat16().to(DEV)
    kv = torch.randn(32, 576, generator=g).bfloat16().to(DEV)
    idx = torch.tensor([[0, 1, 999999, 3]], dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="BAD_INDEX"):
        sparse_mla_fwd(q, kv, idx, 0.1, check=True)


def test_decode_attention_fwd_shim_matches_reference_signature():
    d = np.load(os.path.join(GOLDEN_DIR, "mla_topk_ragged_sq6_h16_topk96.npz"))
    q = torch.from_numpy(d["q"]).to(torch.bfloat16).to(DEV)
    kv = torch.from_numpy(d["kv"]).to(torch.bfloat16).to(DEV)
    idx = torch.from_numpy(d["indices"]).to(DEV)
    n_valid = (idx >= 0).sum(dim=1).int()
    o = torch.zeros(q.shape[0], q.shape[1], 512, dtype=torch.bfloat16, device=DEV)
    attn_logits = torch.empty(q.shape[0], q.shape[1], 4, 513, device=DEV)
    decode_attention_fwd(q, kv.view(-1, 1, 576), kv.view(-1, 1, 576)[..., :512], o, idx.clamp(min=0), n_valid,
                         attn_logits, 4, float(d["sm_scale"]))
    assert (o.float().cpu() - torch.from_numpy(d["out"]).float()).abs().max().item() <= OUT_ATOL


@pytest.mark.parametrize("two_pass", [False, True], ids=["one_pass", "dequant_then_persistent"])
def test_paged_fp8_decode_scaled_down(two_pass):
    c = W.mla_cfg3(batch=4, n_q=2, h=128, topk=256, len_lo=300, len_hi=1500)
    out, lse = sparse_mla_fwd_paged(c.q.to(DEV), c.kv_cache.to(DEV), c.kv_scale.to(DEV), c.block_table.to(DEV),
                                    c.context_lens.to(DEV), c.indices.to(DEV), c.sm_scale, page_size=c.page_size,
                                    check=True, num_splits=1, two_pass=two_pass)
    ref_out, ref_lse = sparse_mla_fwd_paged_ref(c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens,
                                                c.indices, c.sm_scale, page_size=c.page_size)
    e_out, e_lse = _errors(out, lse, ref_out, ref_lse)
    print(f"[paged fp8] out {e_out:.3e} lse {e_lse:.3e}")
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL


@pytest.mark.parametrize("two_pass", [False, True], ids=["one_pass", "dequant_then_persistent"])
def test_paged_fp8_short_context_and_padding(two_pass):
    c = W.mla_cfg3(batch=3, n_q=2, h=16, topk=128, len_lo=20, len_hi=100)   # topk > context: -1 padded
    out, lse = sparse_mla_fwd_paged(c.q.to(DEV), c.kv_cache.to(DEV), c.kv_scale.to(DEV), c.block_table.to(DEV),
                                    c.context_lens.to(DEV), c.indices.to(DEV), c.sm_scale, page_size=c.page_size,
                                    check=True, num_splits=1, two_pass=two_pass)
    ref_out, ref_lse = sparse_mla_fwd_paged_ref(c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens,
                                                c.indices, c.sm_scale, page_size=c.page_size)
    e_out, e_lse = _errors(out, lse, ref_out, ref_lse)
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL


@pytest.mark.parametrize("splits", [2, 3, 8])
def test_split_topk_and_merge_match_unsplit(splits):
    """Top-k axis split over several CTAs + merge kernel (the reference's stage 2) against the oracle and
    against the unsplit kernel; includes a token whose later splits are empty and one with no valid entry."""
    g = torch.Generator().manual_seed(40 + splits)
    s_q, h, s_kv, topk = 5, 128, 700, 448
    q = torch.randn(s_q, h, 576, generator=g).bfloat16()
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).int()
    idx[1, 70:] = -1
    idx[2, :] = -1
    out, lse = sparse_mla_fwd(q.to(DEV), kv.to(DEV), idx.to(DEV), 0.06, check=True, num_splits=splits)
    ref_out, ref_lse = sparse_mla_fwd_ref(q, kv, idx, 0.06)
    e_out, e_lse = _errors(out, lse, ref_out, ref_lse)
    print(f"[split {splits}] out {e_out:.3e} lse {e_lse:.3e}")
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL
    out1, lse1 = sparse_mla_fwd(q.to(DEV), kv.to(DEV), idx.to(DEV), 0.06, check=True, algo=1)
    assert (out.float() - out1.float()).abs().max().item() <= 1e-2


def test_paged_fp8_decode_with_splits():
    c = W.mla_cfg3(batch=3, n_q=2, h=128, topk=512, len_lo=600, len_hi=2500)
    args = (c.q.to(DEV), c.kv_cache.to(DEV), c.kv_scale.to(DEV), c.block_table.to(DEV), c.context_lens.to(DEV),
            c.indices.to(DEV), c.sm_scale)
    out, lse = sparse_mla_fwd_paged(*args, page_size=c.page_size, check=True)            # automatic split count
    out4, lse4 = sparse_mla_fwd_paged(*args, page_size=c.page_size, check=True, num_splits=4)
    ref_out, ref_lse = sparse_mla_fwd_paged_ref(c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens,
                                                c.indices, c.sm_scale, page_size=c.page_size)
    for o, l in ((out, lse), (out4, lse4)):
        e_out, e_lse = _errors(o, l, ref_out, ref_lse)
        assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL
