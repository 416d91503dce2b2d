#!/usr/bin/env python
"""Benchmark of the hot path: top-k sparse MLA forward on the DeepSeek-V3.2 prefill shape
(S_q = S_kv = 4096, h = 128, d_qk = 576, d_v = 512, topk = 2048 causal, -1 padded).

    python bench.py --gpus N --steps K --warmup W            # this repo's CUDA path
    python bench.py --impl reference ...                      # the CPU restatement, host cores

One "step" is one forward over one batch of synthetic, seed-generated input.  With N > 1 every
rank runs a full-size batch of its own query tokens against the replicated latent KV (tokens
are independent units, so there is no data-path collective: weak scaling) and the line reports
total FLOP/s over all ranks divided by the slowest rank's device time.  Prints ONE JSON line.
Further sections of the same line: the end-to-end form with host buffers, the strong-scaling form
(one batch split over the ranks), the paged FP8 decode (cfg3), the FP8 cache write path, and the
second hot path, GEMM + reduce-scatter in bf16 (cfg4) and block-scaled FP8 (cfg5), each with a
numeric check against an fp32 reduce-scatter and the CPU oracle.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "sparse_mla_fwd_tflops"
UNIT = "TFLOP/s"
KERNEL_OF_ALGO = {0: "sparse_mla_ring_kernel", 5: "sparse_mla_ring_kernel", 1: "sparse_mla_fwd_kernel"}
SM_SCALE = 192 ** -0.5
FLOPS_CFG2 = 2 * (576 + 512) * 128 * 6292480          # sum over tokens of min(t + 1, 2048) valid entries


def make_config(s_q: int):
    """The workload description both arms print: the driver compares it key by key."""
    return {"workload": "mla_cfg2_prefill_sq4096_skv4096_h128_topk2048_causal", "s_q_per_gpu": s_q,
            "sharding": "query tokens per rank, latent KV replicated, no collective",
            "l2": "inputs larger than L2 (q 604 MB per step)", "sm_scale": SM_SCALE,
            "flops_per_gpu_step": FLOPS_CFG2 if s_q == 4096 else None}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append((time.time(), ln.strip()))

    def stop(self, t_begin: float, t_end: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        rows = [ln for (ts, ln) in self.lines if t_begin - 0.05 <= ts <= t_end + 0.15] or [ln for _, ln in self.lines]
        for ln in rows:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline_mla(n_tokens: int, reps: int = 1):
    """Times the CPU oracle on a bounded, evenly spaced sample of the cfg2 query tokens (all of them at 4096)."""
    from flagtree_b200 import workloads as W
    from oracle.sparse_mla_ref import sparse_mla_fwd_ref
    c = W.mla_cfg2(device="cpu", s_q=4096, s_kv=4096, h=128, topk=2048)
    sel = torch.linspace(0, 4095, n_tokens).round().long()
    q, idx = c.q[sel].contiguous(), c.indices[sel].contiguous()
    flops = 2 * (576 + 512) * 128 * int((idx >= 0).sum())
    torch.set_num_threads(os.cpu_count() or 1)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        sparse_mla_fwd_ref(q, c.kv, idx, c.sm_scale, chunk=8)
        best = min(best, time.perf_counter() - t0)
    return {"value": flops / best / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_tokens} of 4096 query tokens of the cfg2 prefill batch, evenly spaced (h=128, topk<=2048), "
                      f"fp32 torch restatement, best of {reps}; {best:.2f} s",
            "seconds": best, "flops": flops}


def _time_events(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_mla_decode_fp8(args, dev, peaks):
    """Third workload (a parity-test case with a timing beside it, not the headline): sparse MLA decode over
    the paged FP8 latent cache of cfg3 (64 sequences x 2 query tokens, h = 128, topk = 2048, 64-token pages
    with one fp32 scale each, context 8192..65536).  The gathered FP8 rows (151 MB) exceed L2.  Near the
    ridge: reported both as TFLOP/s and as GB/s of the bytes that must move."""
    from flagtree_b200 import sparse_mla_fwd_paged
    from flagtree_b200 import workloads as W
    c = W.mla_cfg3(device=dev, batch=args.decode_batch)
    b, n_q, h, _ = c.q.shape
    n_valid = int((c.indices >= 0).sum())
    flops = 2 * (576 + 512) * h * n_valid
    nbytes = n_valid * 576 + c.q.numel() * 2 + b * n_q * h * 512 * 2 + c.indices.numel() * 4
    iters = max(5, min(args.steps, 20))
    ms = _time_events(lambda: sparse_mla_fwd_paged(c.q, c.kv_cache, c.kv_scale, c.block_table, c.context_lens, c.indices,
                                                   c.sm_scale, page_size=c.page_size), iters, max(3, args.warmup))
    return {"workload": c.name, "dtype": "fp8 e4m3 KV (bf16 math)", "ms": ms, "iters": iters, "flops": flops,
            "tflops": flops / (ms * 1e-3) / 1e12, "bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
            "frac_of_bf16_peak": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
            "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "l2": "gathered rows (151 MB) larger than L2", "kernel": "mla_dequant_rows_kernel + persistent sparse-MLA kernel"}


def bench_kv_cache_write(args, dev, peaks):
    """The producer of cfg3's cache format: 262144 new latent rows (4096 pages of 64 tokens) quantised to e4m3
    with per-page scales and scattered into a cache of 8192 pages.  Bound by device memory: per row 1152 bytes
    are read (twice: once for the page maximum, once to quantise) and 576 written; the algorithmic figure counts
    one read and one write.  The rows (302 MB) exceed L2."""
    from flagtree_b200 import kv_cache_write_fp8
    g = torch.Generator(device=dev)
    g.manual_seed(3100)
    page, n_pages, n_rows = 64, 8192, 4096 * 64
    rows = torch.randn(n_rows, 576, generator=g, device=dev).bfloat16()
    pages = torch.randperm(n_pages, generator=g, device=dev)[:n_rows // page]
    slots = (pages[:, None] * page + torch.arange(page, device=dev)[None, :]).reshape(-1).int()
    cache = torch.zeros(n_pages, page, 576, dtype=torch.uint8, device=dev)
    scale = torch.zeros(n_pages, device=dev)
    iters = max(5, min(args.steps, 20))

    def step():
        scale.zero_()                       # every timed call fills empty pages (no requantisation pass)
        kv_cache_write_fp8(rows, slots, cache, scale, page)

    ms = _time_events(step, iters)
    nbytes = n_rows * (1152 + 576) + n_rows * 4
    return {"workload": f"kv_cache_write_fp8_rows{n_rows}_pages{n_pages}x{page}", "ms": ms, "iters": iters,
            "bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "bound": "hbm", "kernels": "row_amax_kernel + page_settle_kernel + row_store_kernel",
            "l2": "new rows (302 MB) larger than L2"}


def bench_topk_indices(args, dev, peaks):
    """The index producer of the headline workload: 4096 tokens, 32768 scores each, the 2048 largest.  Bound by
    device memory: 4 * s_kv bytes of scores read and 4 * topk bytes of indices written per token; the scores
    (537 MB) exceed L2."""
    from flagtree_b200 import topk_indices
    g = torch.Generator(device=dev)
    g.manual_seed(3200)
    s_q, s_kv, topk = 4096, 32768, 2048
    scores = torch.randn(s_q, s_kv, generator=g, device=dev)
    out = torch.empty(s_q, topk, dtype=torch.int32, device=dev)
    iters = max(5, min(args.steps, 20))
    ms = _time_events(lambda: topk_indices(scores, topk, out=out), iters)
    nbytes = s_q * (4 * s_kv + 4 * topk)
    return {"workload": f"topk_indices_sq{s_q}_skv{s_kv}_topk{topk}", "ms": ms, "iters": iters, "bytes": nbytes,
            "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "bound": "hbm", "kernel": "topk_select_rows_kernel", "l2": "scores (537 MB) larger than L2"}


def bench_fp8_dense_peak(dev):
    """A plain library FP8 GEMM (cuBLASLt through torch._scaled_mm, e4m3 x e4m3 -> bf16, 8192^3) timed once as the
    dense FP8 figure to hold the block-scaled FP8 kernels against; None when this torch has no such op."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()       # column-major second operand
        one = torch.ones((), device=dev)
        ms = _time_events(lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16), 10)
        return {"tflops": 2 * n ** 3 / (ms * 1e-3) / 1e12, "ms": ms, "shape": f"{n}^3", "kind": "cuBLASLt e4m3 GEMM via torch._scaled_mm"}
    except Exception as e:                                                 # noqa: BLE001
        return {"tflops": None, "unavailable": repr(e)[:200]}


def _timed_collective(fn, iters, flush, dist, sync_word, dev):
    """Median over `iters` of per-iteration CUDA-event times, L2 flushed and the ranks' streams aligned before
    each start event; max over ranks."""
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.fill_(1)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if dist is not None:
            dist.all_reduce(sync_word)      # aligns the ranks' streams on the device before the start event
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def _parity_vs_fp32_reduce_scatter(out, partial_fp32, world, dist, dev, oracle_rows=None):
    """Numeric check of a fused GEMM + reduce-scatter result, outside every timed loop: against NCCL's
    reduce_scatter_tensor of the ranks' fp32 partial products (all rows) and, on rank 0, against the CPU oracle
    on a few rows.  The bound is the one of the parity tests: every partial is rounded to bf16 (2^-9 of a value
    that may be as large as the sum) and the fp32 sum once more."""
    ref = torch.empty(out.shape, dtype=torch.float32, device=dev)
    dist.reduce_scatter_tensor(ref, partial_fp32)
    err = (out.float() - ref).abs().max()
    scale = ref.abs().max()
    tol = (world + 1) * 2 ** -8 * float(scale)
    res = {"max_abs_err": float(err), "tol": tol, "max_abs_ref": float(scale)}
    if oracle_rows is not None:
        rows, want = oracle_rows
        e2 = float((out[rows].float().cpu() - want).abs().max())
        res["oracle_rows"] = len(rows)
        res["oracle_max_abs_err"] = e2
        err = torch.maximum(err, torch.tensor(e2, device=dev))
    ok = torch.tensor([1 if float(err) <= tol else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    worst = err.clone().double()
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    res["max_abs_err_all_ranks"] = float(worst)
    res["ok"] = bool(int(ok.item()) == 1)
    return res


def bench_gemm_rs(args, dev, rank, world, dist, peaks):
    """Second hot path: row-parallel bf16 GEMM fused with reduce-scatter at tp = number of GPUs, per-rank
    shape of cfg4 (A [8192 x 2304], B [2304 x 7168]; K grows with tp).  tp = 1 is the plain GEMM.  Each
    timed iteration is bracketed by its own CUDA events with an L2 flush (256 MB write) in between."""
    from flagtree_b200 import GemmRsContext, matmul
    from flagtree_b200 import workloads as W
    m, n, k_loc = 8192, 7168, 2304
    case = W.gemm_cfg4(device=dev, tp=world, rank=rank, m=m, n=n, k_total=k_loc * world)
    flops = case.flops
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    c_full = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    iters = max(5, min(args.steps, 20))
    sync_word = torch.zeros(1, device=dev)

    t_gemm = _timed_collective(lambda: matmul(case.a, case.b, out=c_full), iters, flush, dist, sync_word, dev)
    res = {"workload": f"gemm_rs_cfg4_per_rank_m{m}_n{n}_klocal{k_loc}_tp{world}", "tp": world, "dtype": "bf16",
           "flops_per_gpu": flops, "gemm_only_ms": t_gemm, "gemm_only_tflops_per_gpu": flops / t_gemm / 1e9,
           "l2": "256 MB flush write between timed iterations", "iters": iters, "timing": "median per rank, max over ranks"}
    if world > 1:
        ctx = GemmRsContext(m, n, None, dev, "auto", args.rs_protocol)
        out = torch.empty(m // world, n, dtype=torch.bfloat16, device=dev)
        t_fused = _timed_collective(lambda: ctx(case.a, case.b, out), iters, flush, dist, sync_word, dev)
        ctx.check()
        nccl_out = torch.empty(m // world, n, dtype=torch.bfloat16, device=dev)

        def nccl_path():
            matmul(case.a, case.b, out=c_full)
            dist.reduce_scatter_tensor(nccl_out, c_full)

        t_nccl = _timed_collective(nccl_path, iters, flush, dist, sync_word, dev)
        # numeric check of the fused result, not timed
        # the CPU oracle on a few rows of rank 0's shard (global rows [0, m / world)), from the very operands the ranks hold
        rows = torch.tensor([0, 1, 127, 128, 511, m // world - 1], device=dev)
        a_rows = [torch.empty(len(rows), k_loc, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        b_all = [torch.empty(k_loc, n, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        dist.all_gather(a_rows, case.a[rows].contiguous())
        dist.all_gather(b_all, case.b)
        oracle_rows = None
        if rank == 0:
            from oracle.gemm_rs_ref import gemm_rs_rows_ref
            want = gemm_rs_rows_ref([t.cpu() for t in a_rows], [t.cpu() for t in b_all], torch.arange(len(rows)))
            oracle_rows = (rows.cpu(), want)
        del a_rows, b_all
        ctx(case.a, case.b, out)
        torch.cuda.synchronize()
        parity = _parity_vs_fp32_reduce_scatter(out, case.a.float() @ case.b.float(), world, dist, dev, oracle_rows)
        pushed = (world - 1) / world * m * n * 2
        res.update({"fused_ms": t_fused, "tflops_per_gpu": flops / t_fused / 1e9,
                    "frac_of_peak": flops / t_fused / 1e9 / peaks["bf16_tflops"],
                    "exposed_comm": t_fused / t_gemm - 1.0, "gemm_plus_nccl_rs_ms": t_nccl,
                    "pushed_bytes_per_gpu": pushed, "nvlink_floor_ms": pushed / 770e9 * 1e3,
                    "symm_provider": ctx.recv.provider, "protocol": ctx.protocol, "parity": parity})
        ctx.close()
    else:
        res.update({"tflops_per_gpu": flops / t_gemm / 1e9, "frac_of_peak": flops / t_gemm / 1e9 / peaks["bf16_tflops"]})
    return res


def bench_ag_gemm(args, dev, rank, world, dist, peaks):
    """The column-parallel sibling of cfg4: all-gather of the row shards of A [8192, 7168] fused with the GEMM against
    this rank's weight columns [7168, 2304] (the same flops and the same bytes over NVLink per rank as cfg4).
    Timed against the plain GEMM on an A that is already complete; checked against an fp32 product of NCCL's
    all-gather of the shards."""
    from flagtree_b200 import AgGemmContext, matmul
    m, k, n_loc = 8192, 7168, 2304
    g = torch.Generator(device=dev)
    g.manual_seed(4100 + rank)
    a_shard = (torch.randn(m // world, k, generator=g, device=dev) * k ** -0.5).bfloat16()
    b = torch.randn(k, n_loc, generator=g, device=dev).bfloat16()
    a_all = [torch.empty_like(a_shard) for _ in range(world)]
    dist.all_gather(a_all, a_shard)
    a_full = torch.cat(a_all)
    flops = 2 * m * k * n_loc
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    sync_word = torch.zeros(1, device=dev)
    iters = max(5, min(args.steps, 20))
    c = torch.empty(m, n_loc, dtype=torch.bfloat16, device=dev)
    t_gemm = _timed_collective(lambda: matmul(a_full, b, out=c), iters, flush, dist, sync_word, dev)
    ctx = AgGemmContext(m, k, None, dev)
    out = torch.empty(m, n_loc, dtype=torch.bfloat16, device=dev)
    t_fused = _timed_collective(lambda: ctx(a_shard, b, out), iters, flush, dist, sync_word, dev)
    ctx.check()

    def nccl_path():
        dist.all_gather(a_all, a_shard)
        matmul(torch.cat(a_all), b, out=c)

    t_nccl = _timed_collective(nccl_path, iters, flush, dist, sync_word, dev)
    ctx(a_shard, b, out)
    torch.cuda.synchronize()
    ref = a_full.float() @ b.float()
    err, scale = float((out.float() - ref).abs().max()), float(ref.abs().max())
    okt = torch.tensor([1 if err <= 2 ** -8 * scale else 0], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    res = {"workload": f"ag_gemm_m{m}_k{k}_nlocal{n_loc}_tp{world}", "tp": world, "dtype": "bf16", "flops_per_gpu": flops,
           "gemm_only_ms": t_gemm, "fused_ms": t_fused, "tflops_per_gpu": flops / t_fused / 1e9,
           "frac_of_peak": flops / t_fused / 1e9 / peaks["bf16_tflops"], "exposed_comm": t_fused / t_gemm - 1.0,
           "nccl_all_gather_plus_gemm_ms": t_nccl, "gathered_bytes_per_gpu": (world - 1) / world * m * k * 2,
           "parity": {"max_abs_err": err, "tol": 2 ** -8 * scale, "ok": bool(int(okt.item()) == 1)}, "iters": iters}
    ctx.close()
    return res


def bench_gemm_rs_fp8(args, dev, rank, world, dist, peaks):
    """cfg5: block-scaled FP8 GEMM + reduce-scatter, tp = number of GPUs, M in {1024, 4096, 16384}, N = 8192,
    K = 28672 / tp per rank.  tp = 1 times the block-scaled GEMM alone."""
    from flagtree_b200 import GemmRsContext, matmul_fp8_blockscaled
    from flagtree_b200 import workloads as W
    n, k_total = 8192, 28672
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    sync_word = torch.zeros(1, device=dev)
    iters = max(5, min(args.steps, 10))
    sweep = []
    for m in (1024, 4096, 16384):
        case = W.gemm_cfg5(device=dev, tp=world, rank=rank, m=m, n=n, k_total=k_total)
        flops = case.flops
        c_full = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        t_gemm = _timed_collective(lambda: matmul_fp8_blockscaled(case.a, case.a_scale, case.b, case.b_scale, out=c_full),
                                   iters, flush, dist, sync_word, dev)
        row = {"m": m, "n": n, "k_local": k_total // world, "flops_per_gpu": flops, "gemm_only_ms": t_gemm,
               "gemm_only_tflops_per_gpu": flops / t_gemm / 1e9}
        # the same product with the weight kept as [N, K] (K contiguous) and passed as its transposed view
        bt = case.b.t().contiguous()
        t_km = _timed_collective(lambda: matmul_fp8_blockscaled(case.a, case.a_scale, bt.t(), case.b_scale, out=c_full), iters, flush, dist, sync_word, dev)
        row.update({"gemm_only_weight_nk_ms": t_km, "gemm_only_weight_nk_tflops_per_gpu": flops / t_km / 1e9})
        del bt
        if world > 1:
            ctx = GemmRsContext(m, n, None, dev, "auto", "auto", fp8=True)
            out = torch.empty(m // world, n, dtype=torch.bfloat16, device=dev)
            t_fused = _timed_collective(lambda: ctx.fp8(case.a, case.a_scale, case.b, case.b_scale, out), iters, flush, dist, sync_word, dev)
            ctx.check()
            ctx.fp8(case.a, case.a_scale, case.b, case.b_scale, out)
            torch.cuda.synchronize()
            # fp32 partial of this rank from the dequantised operands, on the device
            a_s = case.a_scale.repeat_interleave(128, dim=1)
            b_s = case.b_scale.repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)
            part = (case.a.view(torch.float8_e4m3fn).float() * a_s) @ (case.b.view(torch.float8_e4m3fn).float() * b_s)
            parity = _parity_vs_fp32_reduce_scatter(out, part, world, dist, dev)
            del part, a_s, b_s
            row.update({"fused_ms": t_fused, "tflops_per_gpu": flops / t_fused / 1e9, "exposed_comm": t_fused / t_gemm - 1.0,
                        "protocol": ctx.protocol, "parity": parity})
            ctx.close()
        sweep.append(row)
        del case, c_full
    res = {"workload": f"gemm_rs_fp8_cfg5_n{n}_k{k_total}_tp{world}", "tp": world, "dtype": "fp8 e4m3, fp32 block scales (1x128, 128x128)",
           "sweep": sweep, "iters": iters, "l2": "256 MB flush write between timed iterations"}
    return res


def run_reference(args, rank, world):
    """CPU arm: the restatement of the reference's torch idiom on the box's host cores, same workload."""
    if rank != 0:
        return
    n_tok = args.ref_tokens
    times = []
    res = None
    for i in range(args.warmup + args.steps):
        res = cpu_baseline_mla(n_tok, reps=1)
        if i >= args.warmup:
            times.append(res["seconds"])
    t = sum(times) / len(times)
    val = res["flops"] / t / 1e12
    cfg = make_config(args.s_q)
    if n_tok != 4096:
        cfg["sample_tokens"] = n_tok
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": res["cores"], "kind": "port", "sample": res["sample"]},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def _progress(msg):
    """A line on stderr per finished section when FTB_BENCH_PROGRESS is set (stdout carries the one JSON line)."""
    if os.environ.get("FTB_BENCH_PROGRESS"):
        torch.cuda.synchronize()
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--ref-tokens", type=int, default=4096, help="query tokens per step of the CPU arm (4096 = the whole batch)")
    ap.add_argument("--cpu-tokens", type=int, default=4096, help="query tokens of the cpu_baseline sample")
    ap.add_argument("--s-q", type=int, default=4096, help="query tokens per rank (default = full cfg2)")
    ap.add_argument("--algo", type=int, default=0, help="algo_id of the sparse-MLA kernel (0 = the library's default)")
    ap.add_argument("--rs-protocol", default="auto", choices=["auto", "push", "pull", "staged", "copy"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-gemm", action="store_true", help="skip the GEMM + reduce-scatter sections (cfg4, cfg5)")
    ap.add_argument("--no-fp8-sweep", action="store_true", help="skip the cfg5 sweep")
    ap.add_argument("--no-decode", action="store_true", help="skip the paged FP8 decode and cache-write sections (cfg3)")
    ap.add_argument("--decode-batch", type=int, default=64, help="sequences of the decode section (64 = cfg3; fewer for profiler captures)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return 0

    if args.warmup < 3:
        args.warmup = 3
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the native arm has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    from flagtree_b200 import sparse_mla_fwd
    from flagtree_b200 import workloads as W
    peaks = load_peaks()

    case = W.mla_cfg2(device=dev, s_q=args.s_q, s_kv=4096, h=128, topk=2048, rank=rank)
    flops_rank = case.flops
    out = torch.empty(case.q.shape[0], 128, 512, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(case.q.shape[0], 128, dtype=torch.float32, device=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        sparse_mla_fwd(case.q, case.kv, case.indices, case.sm_scale, out=out, lse=lse, algo=args.algo)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    t_begin = time.time()
    evs[0].record()
    for i in range(args.steps):
        step()
        evs[i + 1].record()
    barrier()
    t_end = time.time()
    total_ms = evs[0].elapsed_time(evs[-1])
    per_launch_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None

    t = torch.tensor([total_ms, float(flops_rank)], dtype=torch.float64, device=dev)
    if dist is not None:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        total_ms_max, flops_all = float(tmax[0]), float(tsum[1])
    else:
        total_ms_max, flops_all = total_ms, float(flops_rank)
    ms_per_step = total_ms_max / args.steps
    value = flops_all / (ms_per_step * 1e-3) / 1e12

    # ---- strong scaling: ONE cfg2 batch (rank 0's) split over the ranks, tokens dealt round-robin so that the
    # short early tokens of the causal batch are spread evenly; same kernel, max over ranks
    _progress("headline done")
    strong = None
    if world > 1 and args.s_q == 4096:
        c0 = W.mla_cfg2(device=dev, s_q=4096, s_kv=4096, h=128, topk=2048, rank=0)
        sq, sidx = c0.q[rank::world].contiguous(), c0.indices[rank::world].contiguous()
        so = torch.empty(sq.shape[0], 128, 512, dtype=torch.bfloat16, device=dev)
        sl = torch.empty(sq.shape[0], 128, dtype=torch.float32, device=dev)
        del c0
        barrier()
        ms_s = _time_events(lambda: sparse_mla_fwd(sq, case.kv, sidx, case.sm_scale, out=so, lse=sl, algo=args.algo),
                            max(5, min(args.steps, 20)))
        ts = torch.tensor([ms_s], dtype=torch.float64, device=dev)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        one_gpu_ms = total_ms_max / args.steps          # a full batch on one GPU takes what a weak-scaling step takes
        strong = {"s_q_per_gpu": 4096 // world, "ms_per_step": float(ts[0]), "value": FLOPS_CFG2 / (float(ts[0]) * 1e-3) / 1e12,
                  "unit": UNIT, "efficiency_vs_full_batch_on_one_gpu": one_gpu_ms / (world * float(ts[0])),
                  "sharding": "query tokens of one batch dealt round-robin over the ranks"}
        del sq, sidx, so, sl

    # ---- end-to-end through the public API with host buffers (pinned), copies inside the timed region
    _progress("strong scaling done")
    e2e = None
    if not args.no_e2e:
        hq = case.q.cpu().pin_memory()
        hkv = case.kv.cpu().pin_memory()
        hidx = case.indices.cpu().pin_memory()
        hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        hlse = torch.empty(lse.shape, dtype=lse.dtype).pin_memory()
        from flagtree_b200 import sparse_mla_fwd_host

        def e2e_step():
            # the host-buffer form of the operator: every input goes host -> device and every result device ->
            # host inside this call (chunks of query tokens on three streams)
            sparse_mla_fwd_host(hq, hkv, hidx, case.sm_scale, out=hout, lse=hlse, device=dev)

        n_e2e = max(3, min(args.steps, 8))
        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te[0]) / n_e2e
        h2d = hq.numel() * 2 + hkv.numel() * 2 + hidx.numel() * 4
        d2h = hout.numel() * 2 + hlse.numel() * 4
        # what the host link gives this step at best: the same bytes, one pinned copy each way at the same time
        # (all ranks at once), no kernel in between
        s_up, s_dn = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def link_only():
            cur = torch.cuda.current_stream(dev)
            s_up.wait_stream(cur); s_dn.wait_stream(cur)
            with torch.cuda.stream(s_up):
                case.q.copy_(hq, non_blocking=True)
                case.indices.copy_(hidx, non_blocking=True)
            with torch.cuda.stream(s_dn):
                hout.copy_(out, non_blocking=True)
                hlse.copy_(lse, non_blocking=True)
            cur.wait_stream(s_up); cur.wait_stream(s_dn)

        barrier()
        link_ms = _time_events(link_only, 3, 1)
        tl = torch.tensor([link_ms], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(tl, op=dist.ReduceOp.MAX)
        link_ms = float(tl[0])
        e2e = {"value": flops_all / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": n_e2e,
               "host_link_floor_ms": link_ms, "host_link_h2d_gbs": h2d / link_ms / 1e6, "host_link_d2h_gbs": d2h / link_ms / 1e6,
               "frac_of_host_link_floor": link_ms / e2e_ms,
               "note": "the step is bound by the host link: the floor is the same bytes copied both ways at once with no kernel"}
        del hq, hkv, hidx, hout, hlse

    _progress("e2e done")
    decode_fp8 = kv_write = topk_b = None
    if world == 1 and not args.no_decode:
        decode_fp8 = bench_mla_decode_fp8(args, dev, peaks)
        kv_write = bench_kv_cache_write(args, dev, peaks)
        topk_b = bench_topk_indices(args, dev, peaks)
    del case, out, lse
    torch.cuda.empty_cache()
    gemm_rs = gemm_rs_fp8 = fp8_peak = ag = None
    if not args.no_gemm:
        gemm_rs = bench_gemm_rs(args, dev, rank, world, dist, peaks)
        _progress("gemm_rs done")
        if world > 1:
            ag = bench_ag_gemm(args, dev, rank, world, dist, peaks)
            _progress("ag_gemm done")
        if not args.no_fp8_sweep:
            if world == 1:
                fp8_peak = bench_fp8_dense_peak(dev)
            gemm_rs_fp8 = bench_gemm_rs_fp8(args, dev, rank, world, dist, peaks)
            _progress("gemm_rs_fp8 done")
            if fp8_peak is not None:
                gemm_rs_fp8["fp8_dense_peak"] = fp8_peak

    if rank == 0:
        avg_launch_ms = sum(per_launch_ms) / len(per_launch_ms)
        achieved = flops_rank / (avg_launch_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        kernel = KERNEL_OF_ALGO.get(args.algo, "sparse_mla kernel")
        prof_traffic = None
        tpath = os.path.join(ROOT, "profiles", f"{kernel}_cfg2_traffic.txt")   # figures of the ncu capture, JSON text
        if os.path.exists(tpath):
            try:
                with open(tpath) as f:
                    prof_traffic = json.load(f).get("dram_bytes_per_launch_cfg2")
            except Exception:
                prof_traffic = None
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": prof_traffic, "peak_source": f"bf16_tflops (burst) of {peaks['source']} MEASURED_PEAKS.json",
                    "kernel": kernel, "flops_per_launch": flops_rank, "avg_launch_ms": avg_launch_ms}
        cpu_b = None
        if not args.no_cpu_baseline:
            cpu_b = cpu_baseline_mla(args.cpu_tokens, reps=3)
            cpu_b.pop("seconds"); cpu_b.pop("flops")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": make_config(args.s_q),
            "roofline": roofline, "cpu_baseline": cpu_b, "e2e": e2e, "gpu_launches": args.steps,
            "strong_scaling": strong,
            "gemm_rs": gemm_rs, "gemm_rs_fp8": gemm_rs_fp8, "ag_gemm": ag,
            "mla_decode_fp8": decode_fp8, "kv_cache_write": kv_write, "topk_indices": topk_b,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
