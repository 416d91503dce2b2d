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


# both bf16 kernels behind algo_id: 5 is what algo_id 0 selects
ALGOS = [1, 5]
ALGO_IDS = ["single_cta", "persistent"]


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


def _stepped_scores_case(order, n_tiles=5, h=128, s_q=3, seed=3):
    """Inputs whose scores climb (or fall) from one tile of 128 selected rows to the next by far more than the
    2^8 that the kernels let the running maximum lag: kv row j = c_j * u + noise with c_j growing along the index
    list, every q row a positive multiple a_h of u plus noise, so that score(h, j) ~ 12 * a_h * c_j (natural
    units, sm_scale = 1) and the per-tile maximum of every head with a_h >= 1 grows by >= 17 in the log2 domain
    per tile.  `order`: "up" = every tile after the first rescales the accumulator, "down" = none does,
    "mixed" = only the heads with a large a_h do (the others have a_h = 0.01 and stay within the lag).
    The values stay O(1) so that the absolute output tolerance keeps its meaning."""
    g = torch.Generator().manual_seed(seed)
    topk = 128 * n_tiles
    s_kv = topk + 64
    u = (torch.randint(0, 2, (576,), generator=g).float() * 2 - 1)
    c = torch.arange(s_kv, dtype=torch.float32) / 128.0                  # + 1 per tile of 128 rows
    kv = (0.5 * c[:, None] * u[None, :] + 0.1 * torch.randn(s_kv, 576, generator=g)).bfloat16()
    a = 1.0 + torch.rand(s_q, h, generator=g)
    if order == "mixed":
        a[:, ::2] = 0.01
    q = (a[:, :, None] * u[None, None, :] / 24.0 + 0.02 * torch.randn(s_q, h, 576, generator=g)).bfloat16()
    rows = torch.arange(topk, dtype=torch.int32)
    if order == "down":
        rows = rows.flip(0)
    idx = rows[None, :].repeat(s_q, 1).contiguous()
    idx[1, topk - 100:] = -1                                              # a ragged last tile
    return q, kv, idx


@pytest.mark.parametrize("algo", [0, 1], ids=["default", "single_cta"])
@pytest.mark.parametrize("order", ["up", "down", "mixed"])
def test_running_maximum_steps_across_tiles(order, algo):
    """The online softmax (test_accuracy_musa_vllm_mla.py:313-320) rescales its accumulator whenever the row
    maximum moves.  The persistent kernels move their reference maximum only when it grows by more than 2^8 and
    rescale the accumulator in tensor memory in a separate role; this drives that path on every tile after the
    first ("up"), on none ("down"), and on half of the heads of a warp only ("mixed")."""
    q, kv, idx = _stepped_scores_case(order)
    # make sure the construction does what it says: per-tile maxima of a rescaling head, log2 domain
    s = (q[0, 1].float() @ kv[idx[0].clamp(min=0).long()].float().T) * 1.4426950408889634
    tile_max = s.view(-1, 128).amax(dim=1)
    steps = tile_max[1:] - tile_max[:-1]
    assert (steps > 8).all() if order != "down" else (steps < -8).all(), steps
    _check(q, kv, idx, 1.0, f"stepped_{order}_algo{algo}", algo)


def test_large_random_scores_are_stable():
    g = torch.Generator().manual_seed(3)
    # scores with a standard deviation near 100: the softmax is close to one-hot and the running
    # maximum moves by large steps between tiles (kv stays N(0,1) so that the absolute output
    # tolerance keeps its meaning)
    q = (torch.randn(3, 128, 576, generator=g) * 8).bfloat16()
    kv = torch.randn(700, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(700, generator=g)[:640] for _ in range(3)]).int()
    for algo in (0, 1):
        _check(q, kv, idx, 0.5, f"large_scores_algo{algo}", algo)


@pytest.mark.parametrize("algo", [0, 1], ids=["default", "single_cta"])
def test_base2_lse_convention(algo):
    """lse_base2: the log-sum-exp in base-2 units of score * log2(e), the convention of the reference's dense
    attention (python/triton/ops/flash_attention.py:103) = natural-log LSE / ln 2; the output does not change."""
    c = W.mla_cfg2(s_q=70, s_kv=400, h=128, topk=300)
    c.indices[5, :] = -1
    out, lse2 = sparse_mla_fwd(c.q.to(DEV), c.kv.to(DEV), c.indices.to(DEV), c.sm_scale, check=True, algo=algo, lse_base2=True)
    ref_out, ref_lse = sparse_mla_fwd_ref(c.q, c.kv, c.indices, c.sm_scale)
    e_out, e_lse = _errors(out, lse2, ref_out, ref_lse / 0.6931471805599453)
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL, (e_out, e_lse)
    if algo == 1:
        _, lse_s = sparse_mla_fwd(c.q.to(DEV), c.kv.to(DEV), c.indices.to(DEV), c.sm_scale, check=True, num_splits=3, lse_base2=True)
        _, e_lse = _errors(out, lse_s, ref_out, ref_lse / 0.6931471805599453)
        assert e_lse <= LSE_RTOL


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


def test_negative_index_other_than_padding_is_reported():
    g = torch.Generator().manual_seed(2)
    q = torch.randn(2, 16, 576, generator=g).bfloat16().to(DEV)
    kv = torch.randn(32, 576, generator=g).bfloat16().to(DEV)
    idx = torch.tensor([[0, 1, -2, 3], [4, -1, 5, 6]], dtype=torch.int32, device=DEV)
    for algo in (0, 1):
        with pytest.raises(RuntimeError, match="BAD_INDEX"):
            sparse_mla_fwd(q, kv, idx, 0.1, check=True, algo=algo)


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


def test_paged_two_pass_with_masked_first_entry_over_poisoned_scratch():
    """The two-pass path gathers row 0 of its compact table for every masked entry (and multiplies it by zero).
    When the very first entry is itself masked nothing used to write that row: with NaN patterns left in the
    scratch the whole result turned NaN.  Here entry (token 0, slot 0) is padding, sequence 0 has context length
    0, and the scratch memory is filled with 0xFF bytes just before the call."""
    c = W.mla_cfg3(batch=3, n_q=2, h=128, topk=256, len_lo=300, len_hi=900)
    c.indices[0, 0, 0] = -1
    c.context_lens[0] = 0
    args = [t.to(DEV) for t in (c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens, c.indices)]
    from flagtree_b200 import _lib
    need = int(_lib.load().ftb_sparse_mla_dequant_workspace_bytes(6, 256))
    poison = torch.full((need,), 0xFF, dtype=torch.uint8, device=DEV)
    torch.cuda.synchronize()
    del poison                                   # the caching allocator hands the same block to the next request
    out, lse = sparse_mla_fwd_paged(*args, c.sm_scale, page_size=c.page_size, check=True, num_splits=1, two_pass=True)
    ref_out, ref_lse = sparse_mla_fwd_paged_ref(c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens,
                                                c.indices, c.sm_scale, page_size=c.page_size)
    assert torch.isfinite(out.float()).all()
    e_out, e_lse = _errors(out, lse, ref_out, ref_lse)
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL
    assert (out[0] == 0).all() and torch.isinf(lse[0]).all()


def test_paged_context_longer_than_block_table_is_reported():
    c = W.mla_cfg3(batch=2, n_q=1, h=16, topk=64, len_lo=100, len_hi=200)
    c.context_lens[1] = c.block_table.shape[1] * c.page_size + 500       # claims pages the table does not have
    c.indices[1, 0, 0] = c.block_table.shape[1] * c.page_size + 3
    args = [t.to(DEV) for t in (c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens, c.indices)]
    for two_pass in (False, True):
        with pytest.raises(RuntimeError, match="BAD_INDEX"):
            sparse_mla_fwd_paged(*args, c.sm_scale, page_size=c.page_size, check=True, num_splits=1, two_pass=two_pass)
