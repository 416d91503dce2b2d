"""GPU parity of the few-heads kernel (algo 2: one CTA per token, the gathered rows on the rows of the MMA, scores
transposed) against the CPU oracle, through the C ABI: every head count up to 32, ragged and padded index lists,
tokens that select nothing, a running maximum that moves on every tile, bad indices, and agreement with the
kernel for many heads on the same inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from flagtree_b200 import sparse_mla_fwd
    from flagtree_b200 import workloads as W
from oracle.sparse_mla_ref import sparse_mla_fwd_ref

DEV = "cuda:0"


def _check(q, kv, idx, sm_scale, name):
    out, lse = sparse_mla_fwd(q.to(DEV), kv.to(DEV), idx.to(DEV), sm_scale, check=True, algo=2)
    ref_out, ref_lse = sparse_mla_fwd_ref(q, kv, idx, sm_scale)
    err = (out.float().cpu() - ref_out).abs().max().item()
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse.cpu()), fin), name
    lerr = ((lse.cpu()[fin] - ref_lse[fin]).abs() / ref_lse[fin].abs().clamp(min=1)).max().item() if fin.any() else 0.0
    print(f"[{name}] out max-abs err {err:.3e}  lse rel err {lerr:.3e}")
    assert err <= 2e-2 and lerr <= 1e-3, (name, err, lerr)
    return out, lse


@pytest.mark.parametrize("h", [1, 8, 16, 17, 24, 32])
@pytest.mark.parametrize("topk", [1, 100, 128, 129, 640])
def test_head_counts_and_ragged_topk(h, topk):
    g = torch.Generator().manual_seed(100 * h + topk)
    s_q, s_kv = 7, 900
    q = torch.randn(s_q, h, 576, generator=g).bfloat16()
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).int()
    _check(q, kv, idx, 576 ** -0.5, f"h{h}_topk{topk}")


def test_padding_inside_the_list_and_tokens_that_select_nothing():
    g = torch.Generator().manual_seed(5)
    s_q, h, s_kv, topk = 9, 16, 500, 300
    q = torch.randn(s_q, h, 576, generator=g).bfloat16()
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).int()
    idx[0] = -1                                  # nothing selected: out 0, lse -inf
    idx[1, 1:] = -1                              # one row
    idx[2, ::2] = -1                             # holes
    idx[3, :200] = -1                            # a whole first tile masked
    idx[4, 128:256] = -1                         # a whole middle tile masked
    out, lse = _check(q, kv, idx, 0.07, "padding")
    assert (out[0] == 0).all() and torch.isinf(lse[0]).all()


def test_running_maximum_moves_on_every_tile():
    """Keys ordered so that every tile of 128 holds a larger score than all tiles before it: the accumulator is
    rescaled on every tile, for every head."""
    g = torch.Generator().manual_seed(9)
    h, s_kv = 16, 1024
    kv = torch.randn(s_kv, 576, generator=g).bfloat16()
    q = torch.randn(3, h, 576, generator=g).bfloat16()
    scores = q[0, 0].float() @ kv.float().T
    order = scores.argsort()                     # ascending for head 0 of token 0
    idx = order[None, :].repeat(3, 1).int()
    idx[1] = order.flip(0).int()                 # descending: the maximum never moves after the first tile
    _check(q, kv, idx, 0.3, "stepped")


def test_bad_indices_are_reported_and_never_read():
    g = torch.Generator().manual_seed(2)
    q = torch.randn(2, 16, 576, generator=g).bfloat16().to(DEV)
    kv = torch.randn(64, 576, generator=g).bfloat16().to(DEV)
    idx = torch.randint(0, 64, (2, 40), generator=g).int()
    idx[1, 3] = 64
    with pytest.raises(RuntimeError):
        sparse_mla_fwd(q, kv, idx.to(DEV), 0.1, check=True, algo=2)
    idx[1, 3] = -7
    with pytest.raises(RuntimeError):
        sparse_mla_fwd(q, kv, idx.to(DEV), 0.1, check=True, algo=2)


def test_agrees_with_the_default_kernel_on_the_cpu_runnable_case():
    c = W.mla_cfg1()                             # S_q 128, h 16, topk 256, S_kv 4096
    q, kv, idx = c.q.to(DEV), c.kv.to(DEV), c.indices.to(DEV)
    o_few, l_few = sparse_mla_fwd(q, kv, idx, c.sm_scale, check=True, algo=2)
    o_def, l_def = sparse_mla_fwd(q, kv, idx, c.sm_scale, check=True)
    assert (o_few.float() - o_def.float()).abs().max().item() <= 2e-2
    assert ((l_few - l_def).abs() / l_def.abs().clamp(min=1)).max().item() <= 1e-3
    _check(c.q, c.kv, c.indices, c.sm_scale, c.name)


def test_more_than_32_heads_are_refused():
    q = torch.zeros(1, 33, 576, dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros(8, 576, dtype=torch.bfloat16, device=DEV)
    idx = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    with pytest.raises((RuntimeError, ValueError)):
        sparse_mla_fwd(q, kv, idx, 0.1, algo=2)
