"""Pins the CPU oracle to the golden vectors produced from the reference's own kernel source
(tests/golden/make_golden.py).  The reference kernel ran in fp16 with P rounded to fp16 and a
32-wide online softmax, so agreement is to fp16 rounding, not bit-exact."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle.sparse_mla_ref import (merge_splits_ref, physical_rows, sparse_mla_fwd_paged_ref,
                                   sparse_mla_fwd_ref)

from conftest import GOLDEN_DIR

TOPK_CASES = sorted(glob.glob(os.path.join(GOLDEN_DIR, "mla_topk_*.npz")))


def test_golden_fixtures_present():
    assert len(TOPK_CASES) >= 3
    assert os.path.exists(os.path.join(GOLDEN_DIR, "mla_paged16_b3_h16_len73.npz"))


@pytest.mark.parametrize("path", TOPK_CASES, ids=[os.path.basename(p)[:-4] for p in TOPK_CASES])
def test_oracle_matches_reference_kernel_topk(path):
    d = np.load(path)
    q, kv = torch.from_numpy(d["q"]), torch.from_numpy(d["kv"])
    idx = torch.from_numpy(d["indices"])
    out, lse = sparse_mla_fwd_ref(q, kv, idx, float(d["sm_scale"]))
    ref_out = torch.from_numpy(d["out"]).float()
    ref_lse = torch.from_numpy(d["lse"]).float()
    assert (out - ref_out).abs().max().item() < 2e-3          # fp16 output rounding
    assert torch.allclose(lse, ref_lse, rtol=1e-5, atol=1e-5)


def test_oracle_merge_matches_reference_stage2():
    d = np.load(os.path.join(GOLDEN_DIR, "mla_topk_full_sq4_h16_topk64.npz"))
    att = torch.from_numpy(d["att"])                            # [S_q, h, splits, 513]
    out, lse = merge_splits_ref(att[..., :512], att[..., 512])
    assert (out - torch.from_numpy(d["out"]).float()).abs().max().item() < 1e-3
    assert torch.allclose(lse, torch.from_numpy(d["lse"]), rtol=1e-6, atol=1e-6)


def test_oracle_page_table_rule_matches_reference_kernel():
    d = np.load(os.path.join(GOLDEN_DIR, "mla_paged16_b3_h16_len73.npz"))
    q = torch.from_numpy(d["q"])
    cache = torch.from_numpy(d["kv_cache"])                     # [pages, 16, 576] fp16
    table = torch.from_numpy(d["block_table"])
    lens = torch.from_numpy(d["context_lens"])
    page = int(d["page_size"])
    flat = cache.reshape(-1, 576)
    for b in range(q.shape[0]):
        pos = torch.arange(int(lens[b]))
        phys = physical_rows(table[b], pos, page).to(torch.int32)[None, :]
        out, lse = sparse_mla_fwd_ref(q[b:b + 1], flat, phys, float(d["sm_scale"]))
        assert (out[0] - torch.from_numpy(d["out"][b]).float()).abs().max().item() < 2e-3
        assert torch.allclose(lse[0], torch.from_numpy(d["lse"][b]), rtol=1e-5, atol=1e-5)


def test_oracle_edge_cases():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(3, 4, 576, generator=g).bfloat16()
    kv = torch.randn(50, 576, generator=g).bfloat16()
    idx = torch.full((3, 8), -1, dtype=torch.int32)
    idx[0, :8] = torch.arange(8, dtype=torch.int32)
    idx[1, 0] = 7                                              # a single valid entry
    out, lse = sparse_mla_fwd_ref(q, kv, idx, 0.1)
    assert torch.isfinite(out).all()
    # single index: softmax weight 1 -> output is the selected row, lse is the score itself
    assert torch.allclose(out[1], kv[7, :512].float().expand(4, 512), atol=1e-6)
    s = (q[1].float() @ kv[7].float()) * 0.1
    assert torch.allclose(lse[1], s, rtol=1e-5, atol=1e-5)
    # no valid index: zero output, -inf lse
    assert (out[2] == 0).all() and torch.isinf(lse[2]).all() and (lse[2] < 0).all()
    # order of the indices does not matter
    perm = torch.randperm(8, generator=g)
    out_p, lse_p = sparse_mla_fwd_ref(q[:1], kv, idx[:1, perm], 0.1)
    assert torch.allclose(out_p, out[:1], atol=1e-5) and torch.allclose(lse_p, lse[:1], atol=1e-5)


def test_paged_fp8_oracle_equals_dense_on_dequantised_cache():
    from flagtree_b200.workloads import mla_cfg3
    c = mla_cfg3(batch=2, n_q=2, h=4, topk=32, len_lo=70, len_hi=200, page_size=64)
    out, lse = sparse_mla_fwd_paged_ref(c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens,
                                        c.indices, c.sm_scale, page_size=c.page_size)
    assert out.shape == (2, 2, 4, 512) and lse.shape == (2, 2, 4)
    deq = c.kv_cache.view(torch.float8_e4m3fn).float() * c.kv_scale[:, None, None]
    flat = deq.reshape(-1, 576)
    b = 1
    phys = physical_rows(c.block_table[b], c.indices[b].long(), 64).to(torch.int32)
    o2, l2 = sparse_mla_fwd_ref(c.q[b], flat, phys, c.sm_scale)
    assert torch.equal(o2, out[b]) and torch.equal(l2, lse[b])
