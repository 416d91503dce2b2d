"""Worker of the multi-GPU GEMM + reduce-scatter test: one process per GPU (torchrun).  Every rank
builds all ranks' seeded inputs, so each can check its own shard against the CPU oracle."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from flagtree_b200 import GemmRsContext  # noqa: E402
from flagtree_b200 import workloads as W  # noqa: E402
from oracle.gemm_rs_ref import gemm_rs_ref  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    provider = os.environ.get("FTB_SYMM_PROVIDER", "auto")
    protocol = os.environ.get("FTB_RS_PROTOCOL", "auto")
    ok = True
    for (m, n, k_total) in [(world * 128, 256, world * 64), (world * 256, 1024, world * 320), (world * 1024, 7168, world * 2304 // 4)]:
        cases = [W.gemm_cfg4(tp=world, rank=r, m=m, n=n, k_total=k_total) for r in range(world)]
        ref = gemm_rs_ref([c.a for c in cases], [c.b for c in cases])[rank]
        ctx = GemmRsContext(m, n, None, dev, provider, protocol)
        a, b = cases[rank].a.to(dev), cases[rank].b.to(dev)
        outs = []
        for it in range(3):                      # repeated calls reuse the slots (epoch handling)
            outs.append(ctx(a, b).clone())
        torch.cuda.synchronize()
        ctx.check()
        nccl_in = (a.float() @ b.float())
        nccl_out = torch.empty(m // world, n, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(nccl_out, nccl_in)
        err = (outs[0].float().cpu() - ref).abs().max().item()
        scale = ref.abs().max().item()
        err_nccl = (outs[0].float() - nccl_out).abs().max().item()
        same = all(torch.equal(outs[0], o) for o in outs[1:])
        print(f"[rank {rank}] m={m} n={n} k={k_total} provider={ctx.recv.provider} protocol={ctx.protocol}: err {err:.3e} scale {scale:.3e} "
              f"vs-nccl {err_nccl:.3e} repeat-identical {same}", flush=True)
        # every partial is rounded to bf16 (2^-9 relative to a partial that may be as large as the sum)
        # and the fp32 sum is rounded once more
        tol = (world + 1) * 2 ** -8 * scale
        ok = ok and err <= tol and err_nccl <= tol and same
        ctx.close()
    # block-scaled FP8 form (cfg5 family, scaled down): GEMM, then this library's own reduce-scatter kernels
    from oracle.gemm_rs_ref import gemm_rs_fp8_ref
    for (m, n, k_total) in [(world * 128, 256, world * 128), (world * 256, 1024, world * 384)]:
        cases = [W.gemm_cfg5(tp=world, rank=r, m=m, n=n, k_total=k_total) for r in range(world)]
        ref = gemm_rs_fp8_ref([c.a for c in cases], [c.a_scale for c in cases], [c.b for c in cases],
                              [c.b_scale for c in cases])[rank]
        # a context of the copy-engine protocol serves bf16 calls only: the FP8 form gets its own
        ctx = GemmRsContext(m, n, None, dev, provider, "auto" if protocol == "copy" else protocol, fp8=True)
        me = cases[rank]
        a, b, a_s, b_s = me.a.to(dev), me.b.to(dev), me.a_scale.to(dev), me.b_scale.to(dev)
        outs = [ctx.fp8(a, a_s, b, b_s).clone() for _ in range(3)]
        torch.cuda.synchronize()
        ctx.check()
        err = (outs[0].float().cpu() - ref).abs().max().item()
        scale = ref.abs().max().item()
        same = all(torch.equal(outs[0], o) for o in outs[1:])
        print(f"[rank {rank}] fp8 m={m} n={n} k={k_total} protocol={ctx.protocol}: err {err:.3e} scale {scale:.3e} "
              f"repeat-identical {same}", flush=True)
        ok = ok and err <= (world + 1) * 2 ** -8 * scale and same
        ctx.close()
    # all-gather + GEMM: every rank's row shard of A against this rank's weight columns
    from flagtree_b200 import AgGemmContext
    from oracle.gemm_rs_ref import ag_gemm_ref
    for (m, k, n_local) in [(world * 128, 64, 256), (world * 256, 320, 1000), (world * 1024, 2304, 1792)]:
        g = torch.Generator().manual_seed(4242)
        shards = [(torch.randn(m // world, k, generator=g) * k ** -0.5).bfloat16() for _ in range(world)]
        bs = [(torch.randn(k, n_local, generator=g)).bfloat16() for _ in range(world)]
        ref = ag_gemm_ref(shards, bs[rank])
        ctx = AgGemmContext(m, k, None, dev, provider)
        a, b = shards[rank].to(dev), bs[rank].to(dev)
        outs = [ctx(a, b).clone() for _ in range(3)]
        torch.cuda.synchronize()
        ctx.check()
        err = (outs[0].float().cpu() - ref).abs().max().item()
        scale = ref.abs().max().item()
        same = all(torch.equal(outs[0], o) for o in outs[1:])
        print(f"[rank {rank}] ag_gemm m={m} k={k} n_local={n_local}: err {err:.3e} scale {scale:.3e} repeat-identical {same}", flush=True)
        ok = ok and err <= 2 ** -8 * scale and same
        ctx.close()
    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(t.item()) == 1 else 1)


if __name__ == "__main__":
    main()
