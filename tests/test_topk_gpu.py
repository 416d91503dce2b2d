"""GPU parity of the top-k index producer (through the C ABI) against its CPU restatement: index lists must be
identical, including ties (lower position wins), signed zeros, infinities, lengths shorter than topk, empty rows
and rows longer than one pass of the block; and its output must drive the sparse MLA forward."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from flagtree_b200 import sparse_mla_fwd, topk_indices
from oracle.sparse_mla_ref import sparse_mla_fwd_ref, topk_indices_ref

DEV = "cuda:0"


@pytest.mark.parametrize("s_kv,topk", [(1, 1), (37, 5), (512, 512), (513, 64), (1024, 1000), (4096, 2048), (32768, 2048),
                                       (70000, 2048)])
def test_random_scores_match_exactly(s_kv, topk):
    g = torch.Generator().manual_seed(s_kv + topk)
    sc = torch.randn(9, s_kv, generator=g)
    got = topk_indices(sc.to(DEV), topk).cpu()
    assert torch.equal(got, topk_indices_ref(sc, topk))


def test_ties_zeros_infinities_and_lengths():
    g = torch.Generator().manual_seed(3)
    s_q, s_kv, topk = 12, 1500, 300
    sc = torch.randint(-3, 4, (s_q, s_kv), generator=g).float()          # seven distinct values: ties everywhere
    sc[0, ::7] = -0.0
    sc[1, 5] = float("inf")
    sc[1, 9] = -float("inf")
    sc[2] = 1.0                                                            # a constant row: the first topk positions
    lengths = torch.tensor([1500, 1500, 1500, 0, 1, 299, 300, 301, 777, 1500, 1024, 513], dtype=torch.int32)
    got = topk_indices(sc.to(DEV), topk, lengths.to(DEV)).cpu()
    want = topk_indices_ref(sc, topk, lengths)
    assert torch.equal(got, want)
    assert torch.equal(got[2], torch.arange(topk, dtype=torch.int32))
    assert (got[3] == -1).all() and got[4, 0] == 0 and (got[4, 1:] == -1).all()
    assert (got[5, :299] == torch.arange(299)).all() and got[5, 299] == -1


def test_many_rows_with_causal_lengths_and_a_strided_view():
    """More rows than SMs (the persistent kernel takes several rows per CTA), ragged lengths, ties from rounding the
    scores to bf16, and a view whose rows are not contiguous."""
    g = torch.Generator().manual_seed(11)
    s_q, s_kv, topk = 700, 8192, 512
    wide = torch.randn(s_q, s_kv + 64, generator=g).bfloat16().float()
    sc = wide[:, :s_kv]
    lengths = torch.randint(0, s_kv + 1, (s_q,), generator=g).int()
    lengths[:4] = torch.tensor([0, 1, s_kv, 512])
    got = topk_indices(wide.to(DEV)[:, :s_kv], topk, lengths.to(DEV)).cpu()
    assert torch.equal(got, topk_indices_ref(sc, topk, lengths))


def test_long_rows_with_few_distinct_values_and_a_misleading_sample():
    """Rows long enough for the sampled bracket: few distinct values (crowded bins, ties across many threads), a
    constant row, a sorted row, and a row whose sampled positions hold values unlike the rest (the bracket is
    rejected and the whole key range is searched)."""
    g = torch.Generator().manual_seed(21)
    s_kv, topk = 32768, 2048
    rows = [torch.randint(-3, 4, (s_kv,), generator=g).float(),
            torch.full((s_kv,), 2.5),
            torch.arange(s_kv).float(),
            -torch.arange(s_kv).float(),
            torch.randn(s_kv, generator=g).mul(1e-30),                  # denormal-range keys
            torch.randn(s_kv, generator=g)]
    odd = torch.randn(s_kv, generator=g)
    sample_at = (torch.arange(256) * s_kv >> 8) + (torch.arange(256) & 15)
    odd[sample_at] = 1e6
    rows.append(odd)
    low = torch.randn(s_kv, generator=g)
    low[sample_at] = -1e6
    rows.append(low)
    sc = torch.stack(rows)
    lengths = torch.tensor([s_kv, s_kv, s_kv, s_kv, s_kv, 4096, s_kv, s_kv], dtype=torch.int32)
    for k in (topk, 1, 32767):
        got = topk_indices(sc.to(DEV), k, lengths.to(DEV)).cpu()
        assert torch.equal(got, topk_indices_ref(sc, k, lengths)), k


def test_causal_lengths_feed_the_forward():
    """The producer's output as the `indices` of the forward: causal lengths, scores = q.k of head 0."""
    g = torch.Generator().manual_seed(8)
    s_q, h, s_kv, topk = 64, 16, 640, 128
    q = torch.randn(s_q, h, 576, generator=g).bfloat16()
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    scores = q[:, 0].float() @ kv.float().T
    lengths = (torch.arange(s_q) * 10 + 1).int()
    idx = topk_indices(scores.to(DEV), topk, lengths.to(DEV))
    assert torch.equal(idx.cpu(), topk_indices_ref(scores, topk, lengths))
    out, lse = sparse_mla_fwd(q.to(DEV), kv.to(DEV), idx, 0.05, check=True)
    ref_out, ref_lse = sparse_mla_fwd_ref(q, kv, idx.cpu(), 0.05)
    assert (out.float().cpu() - ref_out).abs().max().item() <= 2e-2
    assert ((lse.cpu() - ref_lse).abs() / ref_lse.abs().clamp(min=1)).max().item() <= 1e-3
