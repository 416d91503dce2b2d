"""Host-side multi-rank logic on CPU (gloo, world_size 2): handle exchange of the symmetric workspace,
token sharding of the sparse MLA batch, and the reduce-scatter sharding convention of the oracle."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flagtree_b200 import workloads as W


def _worker(rank, world, port, fn_name, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        globals()[fn_name](rank, world)
        q.put((rank, "ok"))
    except Exception as e:   # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def _spawn(fn_name, world=2, port=29611):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(r[1] == "ok" for r in res), res


def _case_symmetric_exchange(rank, world):
    from flagtree_b200.symm import SymmetricBuffer
    opened = []

    def alloc(nbytes):
        return 1000 * (rank + 1), f"handle-of-{rank}-{nbytes}".encode()

    def open_(handle):
        opened.append(handle)
        owner = int(handle.decode().split("-")[2])
        return 1000 * (owner + 1) + 7          # a "mapped" address, distinct from the owner's own

    buf = SymmetricBuffer(4096, None, None, _alloc=alloc, _open=open_)
    assert buf.world == world and buf.local_ptr == 1000 * (rank + 1)
    for r in range(world):
        assert buf.ptrs[r] == (1000 * (r + 1) if r == rank else 1000 * (r + 1) + 7)
    assert len(opened) == world - 1 and all(h.endswith(b"-4096") for h in opened)


def _case_mla_token_sharding(rank, world):
    from oracle.sparse_mla_ref import sparse_mla_fwd_ref
    c = W.mla_cfg2(s_q=48, s_kv=48, h=4, topk=16)
    lo, hi = W.shard_bounds(48, world, rank)
    out, lse = sparse_mla_fwd_ref(c.q[lo:hi], c.kv, c.indices[lo:hi], c.sm_scale)
    gathered = [None] * world
    dist.all_gather_object(gathered, (lo, hi, out, lse))
    full_out, full_lse = sparse_mla_fwd_ref(c.q, c.kv, c.indices, c.sm_scale)
    covered = 0
    for lo_r, hi_r, o_r, l_r in gathered:
        assert torch.equal(o_r, full_out[lo_r:hi_r]) and torch.equal(l_r, full_lse[lo_r:hi_r])
        covered += hi_r - lo_r
    assert covered == 48


def _case_reduce_scatter_convention(rank, world):
    from oracle.gemm_rs_ref import gemm_rs_ref
    cases = [W.gemm_cfg4(tp=world, rank=r, m=world * 8, n=16, k_total=world * 24) for r in range(world)]
    ref = gemm_rs_ref([c.a for c in cases], [c.b for c in cases])[rank]
    part = cases[rank].a.float() @ cases[rank].b.float()
    out = torch.empty(8, 16)
    dist.reduce_scatter_tensor(out, part)
    assert torch.allclose(out, ref, rtol=1e-6, atol=1e-8)


def _case_reduce_scatter_fp8_convention(rank, world):
    """Block-scaled FP8 form: the oracle's shard of rank r equals the reduce-scatter of the ranks' dequantised
    partial products (the convention the staged kernels follow: partial per rank, sum over ranks, row shard)."""
    from oracle.gemm_rs_ref import dequant_block_scaled, gemm_rs_fp8_ref
    cases = [W.gemm_cfg5(tp=world, rank=r, m=world * 8, n=128, k_total=world * 128) for r in range(world)]
    ref = gemm_rs_fp8_ref([c.a for c in cases], [c.a_scale for c in cases], [c.b for c in cases],
                          [c.b_scale for c in cases])[rank]
    me = cases[rank]
    part = dequant_block_scaled(me.a, me.a_scale, 1, 128).float() @ dequant_block_scaled(me.b, me.b_scale, 128, 128).float()
    out = torch.empty(8, 128)
    dist.reduce_scatter_tensor(out, part)
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)


def _case_all_gather_gemm_convention(rank, world):
    """All-gather + GEMM: the oracle's result of rank r equals gloo's all_gather of the row shards times the rank's
    weight columns; rows of rank s sit at [s * M / tp, (s + 1) * M / tp)."""
    from oracle.gemm_rs_ref import ag_gemm_ref
    g = torch.Generator().manual_seed(5)
    shards = [torch.randn(8, 24, generator=g).bfloat16() for _ in range(world)]
    bs = [torch.randn(24, 16, generator=g).bfloat16() for _ in range(world)]
    gathered = [torch.empty(8, 24, dtype=torch.bfloat16) for _ in range(world)]
    dist.all_gather(gathered, shards[rank])
    out = torch.cat(gathered).float() @ bs[rank].float()
    ref = ag_gemm_ref(shards, bs[rank])
    assert torch.equal(out, ref)
    assert torch.equal(ref[rank * 8:(rank + 1) * 8], shards[rank].float() @ bs[rank].float())


def _case_mla_sequence_sharded_kv(rank, world):
    """A context whose latent rows are sharded over the ranks: each rank runs the forward over its own rows with
    `shard_indices` (entries outside its range become padding), the (out, lse) parts are all-gathered, and the
    split merge of the reference's second launch gives the result of the unsharded forward."""
    from flagtree_b200.ops import shard_indices
    from oracle.sparse_mla_ref import merge_splits_ref, sparse_mla_fwd_ref
    c = W.mla_cfg1(s_q=6, h=4, s_kv=64 * world, topk=40)
    c.indices[1, 10:] = -1
    c.indices[2] = torch.arange(40, dtype=torch.int32)              # every row of this token lives on rank 0
    lo, hi = W.shard_bounds(c.kv.shape[0], world, rank)
    local = shard_indices(c.indices, lo, hi)
    assert ((local >= 0) == ((c.indices >= lo) & (c.indices < hi))).all() and int(local.max()) < hi - lo
    out, lse = sparse_mla_fwd_ref(c.q, c.kv[lo:hi], local, c.sm_scale)
    parts = [None] * world
    dist.all_gather_object(parts, (out, lse))
    po = torch.stack([p[0] for p in parts], dim=2)                  # [s_q, h, world, 512]
    pl = torch.stack([p[1] for p in parts], dim=2)
    m_out, m_lse = merge_splits_ref(po, pl)
    full_out, full_lse = sparse_mla_fwd_ref(c.q, c.kv, c.indices, c.sm_scale)
    assert torch.allclose(m_out, full_out, rtol=1e-5, atol=1e-5)
    assert torch.allclose(m_lse, full_lse, rtol=1e-5, atol=1e-5)
    if rank != 0:
        assert torch.isinf(lse[2]).all() and (out[2] == 0).all()    # an empty part: weight 0 in the merge


@pytest.mark.parametrize("fn,port", [("_case_symmetric_exchange", 29611), ("_case_mla_token_sharding", 29612),
                                     ("_case_reduce_scatter_convention", 29613),
                                     ("_case_reduce_scatter_fp8_convention", 29614),
                                     ("_case_mla_sequence_sharded_kv", 29615),
                                     ("_case_all_gather_gemm_convention", 29616)])
def test_two_ranks_gloo(fn, port):
    _spawn(fn, 2, port)


def test_shard_bounds_cover_everything():
    for n in (0, 1, 7, 64, 4096):
        for world in (1, 2, 3, 8):
            spans = [W.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
