"""Query batches longer than one launch of the persistent sparse-MLA kernels walks through.

The persistent kernel gives every CTA pair at most 64 tokens per launch (74 pairs on a B200: 4736 tokens);
a longer batch becomes several launches over consecutive token ranges, each with its own offsets into q,
indices, out and lse.  Long prefill is the normal case for sparse attention, so the range arithmetic gets a
test of its own: 4936 tokens (two launches), compared token by token with the one-CTA-per-token kernel (a
different code path with no notion of token ranges) and, on a sample of tokens from both ranges, with the
CPU oracle.  Causal top-k with -1 padding, so the first tokens of the batch are short and the rest full.
"""
import pytest
import torch

from conftest import LSE_RTOL, OUT_ATOL

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from flagtree_b200 import sparse_mla_fwd
    from flagtree_b200 import workloads as W
from oracle.sparse_mla_ref import sparse_mla_fwd_ref

DEV = "cuda:0"
S_Q = 74 * 64 + 200


def test_more_tokens_than_one_launch_takes():
    algo = 0
    c = W.mla_cfg2(device=DEV, s_q=S_Q, s_kv=2048, h=64, topk=128)
    out, lse = sparse_mla_fwd(c.q, c.kv, c.indices, c.sm_scale, check=True, algo=algo)
    ref_out, ref_lse = sparse_mla_fwd(c.q, c.kv, c.indices, c.sm_scale, check=True, algo=1)
    torch.cuda.synchronize()
    # every token against the per-token kernel (both are within OUT_ATOL of the oracle, so 2 x between them)
    d_out = (out.float() - ref_out.float()).abs().amax(dim=(1, 2))
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin)
    d_lse = ((lse - ref_lse).abs() / ref_lse.abs().clamp(min=1.0)).masked_fill(~fin, 0.0).amax(dim=1)
    worst = int(d_out.argmax())
    assert d_out.max().item() <= 2 * OUT_ATOL, f"token {worst}: out differs by {d_out.max().item():.4f}"
    assert d_lse.max().item() <= 2 * LSE_RTOL, f"token {int(d_lse.argmax())}: lse differs by {d_lse.max().item():.2e}"
    # a sample from both token ranges against the oracle
    sample = torch.tensor([0, 1, 63, 64, 2047, 4735, 4736, 4737, 4800, S_Q - 1])
    o_ref, l_ref = sparse_mla_fwd_ref(c.q[sample].cpu(), c.kv.cpu(), c.indices[sample].cpu(), c.sm_scale)
    e_out = (out[sample].float().cpu() - o_ref).abs().max().item()
    e_lse = ((lse[sample].cpu() - l_ref).abs() / l_ref.abs().clamp(min=1.0)).max().item()
    assert e_out <= OUT_ATOL and e_lse <= LSE_RTOL, f"vs oracle: out {e_out:.4f}, lse {e_lse:.2e}"
