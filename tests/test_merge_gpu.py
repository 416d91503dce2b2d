"""GPU parity of the public split merge (ftb_sparse_mla_merge, the reference's second launch as an operation of
its own) against the CPU restatement of _fwd_kernel_stage2, and its use for a context whose latent rows are
sharded: every "rank" runs the forward on its own rows, the parts are merged, and the result must equal the
forward over the whole context within the contract's tolerances."""
import numpy as np
import os

import pytest
import torch

from conftest import GOLDEN_DIR, LSE_RTOL, OUT_ATOL

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from flagtree_b200 import shard_indices, sparse_mla_fwd, sparse_mla_merge
from oracle.sparse_mla_ref import merge_splits_ref, sparse_mla_fwd_ref

DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32_parts", "bf16_parts"])
@pytest.mark.parametrize("base2", [False, True], ids=["natural", "base2"])
def test_merge_matches_stage2_restatement(dtype, base2):
    g = torch.Generator().manual_seed(9)
    n_parts, s_q, h = 5, 7, 48
    po = torch.randn(n_parts, s_q, h, 512, generator=g).to(dtype)
    pl = torch.randn(n_parts, s_q, h, generator=g) * 6
    pl[2, 3] = -float("inf")                     # an empty part
    pl[:, 5, 7] = -float("inf")                  # a (token, head) without any valid row
    ref_out, ref_lse = merge_splits_ref(po.float().permute(1, 2, 0, 3), pl.permute(1, 2, 0))
    scale = 1.0 / 0.6931471805599453 if base2 else 1.0
    out, lse = sparse_mla_merge(po.to(DEV), (pl * scale).to(DEV), lse_base2=base2)
    torch.cuda.synchronize()
    assert (out.float().cpu() - ref_out).abs().max().item() <= OUT_ATOL
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    assert ((lse.cpu()[fin] - ref_lse[fin] * scale).abs() / (ref_lse[fin] * scale).abs().clamp(min=1)).max().item() <= LSE_RTOL
    assert (out[5, 7] == 0).all()


def test_merge_of_reference_stage1_partials():
    """The stage-1 partials of the reference's own kernel (fixture) merged on the GPU give the reference's output."""
    d = np.load(os.path.join(GOLDEN_DIR, "mla_topk_full_sq4_h16_topk64.npz"))    # full lists: every split holds rows
    att = torch.from_numpy(d["att"])                                     # [s_q, h, splits, 513]
    po = att[..., :512].permute(2, 0, 1, 3).contiguous()
    pl = att[..., 512].permute(2, 0, 1).contiguous()
    out, lse = sparse_mla_merge(po.to(DEV), pl.to(DEV))
    assert (out.float().cpu() - torch.from_numpy(d["out"]).float()).abs().max().item() <= OUT_ATOL
    ref_lse = torch.from_numpy(d["lse"]).float()
    assert ((lse.cpu() - ref_lse).abs() / ref_lse.abs().clamp(min=1)).max().item() <= LSE_RTOL


@pytest.mark.parametrize("n_ranks", [2, 4])
def test_sequence_sharded_context_merges_to_the_unsharded_result(n_ranks):
    g = torch.Generator().manual_seed(21 + n_ranks)
    s_q, h, s_kv, topk = 9, 128, 1024, 384
    q = torch.randn(s_q, h, 576, generator=g).bfloat16()
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).int()
    idx[1, 200:] = -1
    idx[2] = -1
    idx[2, :s_kv // n_ranks] = torch.randperm(s_kv // n_ranks, generator=g)[:topk].int()    # every selected row lives on rank 0
    ref_out, ref_lse = sparse_mla_fwd_ref(q, kv, idx, 0.06)
    parts_o, parts_l = [], []
    per = s_kv // n_ranks
    for r in range(n_ranks):
        lo, hi = r * per, (r + 1) * per
        o, l = sparse_mla_fwd(q.to(DEV), kv[lo:hi].to(DEV), shard_indices(idx, lo, hi).to(DEV), 0.06, check=True)
        parts_o.append(o)
        parts_l.append(l)
    out, lse = sparse_mla_merge(torch.stack(parts_o), torch.stack(parts_l))
    torch.cuda.synchronize()
    assert (out.float().cpu() - ref_out).abs().max().item() <= OUT_ATOL
    assert ((lse.cpu() - ref_lse).abs() / ref_lse.abs().clamp(min=1)).max().item() <= LSE_RTOL
