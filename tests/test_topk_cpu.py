"""CPU check of the index producer's restatement against torch.topk on inputs without ties."""
import torch

from oracle.sparse_mla_ref import topk_indices_ref


def test_restatement_agrees_with_torch_topk_when_there_are_no_ties():
    g = torch.Generator().manual_seed(0)
    sc = torch.randn(7, 300, generator=g)
    got = topk_indices_ref(sc, 40)
    want = torch.topk(sc, 40, dim=1).indices.sort(dim=1).values.int()
    assert torch.equal(got, want)
    lengths = torch.tensor([300, 10, 0, 40, 41, 1, 299], dtype=torch.int32)
    got = topk_indices_ref(sc, 40, lengths)
    for t in range(7):
        n = int(lengths[t]); k = min(40, n)
        want_t = torch.topk(sc[t, :n], k).indices.sort().values.int() if k else torch.zeros(0, dtype=torch.int32)
        assert torch.equal(got[t, :k], want_t) and (got[t, k:] == -1).all()


def test_ties_go_to_the_lower_position_and_negative_zero_sorts_below_zero():
    sc = torch.tensor([[1.0, 2.0, 2.0, 2.0, 0.0, -0.0, 0.0]])
    assert topk_indices_ref(sc, 2).tolist() == [[1, 2]]
    assert topk_indices_ref(sc, 5).tolist() == [[0, 1, 2, 3, 4]]
    assert topk_indices_ref(sc, 6).tolist() == [[0, 1, 2, 3, 4, 6]]      # +0 at 6 before -0 at 5
