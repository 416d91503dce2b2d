"""Generate the golden fixtures that pin the sparse-MLA oracle to the reference's own kernel.

Run in a container that has the reference checkout and a Triton with a CPU interpreter:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/FlagTree

What it does: reads the reference's MLA decode test file, takes the text of its two Triton
kernels (`_fwd_grouped_kernel_stage1`, `_fwd_kernel_stage2`) plus the small `tanh` helper,
executes that text with the CPU interpreter on small seeded fp16 cases (bf16 mis-executes in
the interpreter, and the reference skips it there too), and stores inputs and outputs as
.npz files next to this script.  No reference text is written anywhere: only the numerical
inputs/outputs are saved.

Mapping used (page size 1 turns the reference's token table into a top-k index list):
  Req_to_tokens := indices (clamped), B_Seqlen := number of valid indices (front packed),
  K_Buffer := kv [S_kv, 1, 576], V_Buffer := kv[..., :512].
A second family runs the kernel in its native paged mode (page size 16, dense positions)
to pin the page-table addressing rule.
"""
from __future__ import annotations

import argparse
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

REL = "third_party/mthreads/python/test/wmma/test_accuracy_musa_vllm_mla.py"
HERE = os.path.dirname(os.path.abspath(__file__))


def _load_reference_kernels(ref_root: str):
    path = os.path.join(ref_root, REL)
    with open(path) as f:
        lines = f.read().split("\n")

    def block(start_marker: str) -> str:
        # take the @triton.jit-decorated function that starts at `def <marker>(`
        for i, ln in enumerate(lines):
            if ln.startswith(f"def {start_marker}("):
                j = i + 1
                while j < len(lines) and (lines[j].startswith((" ", ")")) or lines[j].strip() == ""):
                    j += 1
                return "@triton.jit\n" + "\n".join(lines[i:j])
        raise RuntimeError(f"{start_marker} not found in {path}")

    src = "import triton\nimport triton.language as tl\n\n"
    for name in ("tanh", "_fwd_grouped_kernel_stage1", "_fwd_kernel_stage2"):
        src += block(name) + "\n\n"
    import tempfile
    work = tempfile.mkdtemp(prefix="ref_kernels_")          # scratch outside the repository, removed below
    mod_path = os.path.join(work, "_ref_kernels_tmp.py")
    with open(mod_path, "w") as f:
        f.write(src)
    import importlib.util
    spec = importlib.util.spec_from_file_location("_ref_kernels_tmp", mod_path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod, mod_path


def run_reference(mod, q, k_buffer, v_buffer, req_to_tokens, b_seqlen, sm_scale, splits, page_size):
    """Two launches as in _decode_grouped_att_m_fwd / _decode_softmax_reducev_fwd of the reference."""
    s_q, h, lk = q.shape
    lv = v_buffer.shape[-1]
    att = torch.zeros(s_q, h, splits, lv + 1, dtype=torch.float32)
    o = torch.zeros(s_q, h, lv, dtype=q.dtype)
    block_h = 16
    grid1 = (s_q, (h + min(block_h, h) - 1) // min(block_h, h), splits)
    mod._fwd_grouped_kernel_stage1[grid1](
        q, k_buffer, v_buffer, sm_scale, req_to_tokens, b_seqlen, att,
        req_to_tokens.stride(0), q.stride(0), q.stride(1),
        k_buffer.stride(-3), k_buffer.stride(-2), v_buffer.stride(-3), v_buffer.stride(-2),
        att.stride(0), att.stride(1), att.stride(2),
        kv_group_num=h, q_head_num=h, BLOCK_DMODEL=512, BLOCK_DPE=64, BLOCK_DV=512,
        BLOCK_N=32, BLOCK_H=block_h, NUM_KV_SPLITS=splits, PAGE_SIZE=page_size,
        logit_cap=0.0, Lk=lk, Lv=lv,
    )
    mod._fwd_kernel_stage2[(s_q, h)](
        att, o, b_seqlen, att.stride(0), att.stride(1), att.stride(2), o.stride(0), o.stride(1),
        NUM_KV_SPLITS=splits, BLOCK_DV=512, Lv=lv,
    )
    # The reference does not emit the merged LSE; it is the logaddexp of the non-empty splits.
    per = (b_seqlen + splits - 1) // splits
    lse = torch.full((s_q, h), -float("inf"))
    for k in range(splits):
        nonempty = torch.minimum(per * (k + 1), b_seqlen) > per * k
        part = att[:, :, k, lv]
        part = torch.where(nonempty[:, None], part, torch.full_like(part, -float("inf")))
        lse = torch.logaddexp(lse, part)
    return o, lse, att


def _randn_bf16_exact_fp16(shape, g):
    """N(0,1) values that are exactly representable in BOTH bf16 and fp16, returned as fp16.

    The interpreter run needs fp16; the CUDA kernels take bf16.  Rounding to bf16 first and
    flushing magnitudes below the fp16 normal range makes the two casts exact, so GPU parity
    tests can feed the kernels the very same numbers.
    """
    x = torch.randn(*shape, generator=g).to(torch.bfloat16).to(torch.float32)
    x = torch.where(x.abs() < 2.0 ** -14, torch.zeros_like(x), x)
    y = x.to(torch.float16)
    assert torch.equal(y.to(torch.float32), x) and torch.equal(x.to(torch.bfloat16).to(torch.float32), x)
    return y


def case_topk(mod, seed, s_q, h, s_kv, topk, splits, ragged):
    g = torch.Generator().manual_seed(seed)
    q = _randn_bf16_exact_fp16((s_q, h, 576), g)
    kv = _randn_bf16_exact_fp16((s_kv, 576), g)
    idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).to(torch.int32)
    if ragged:
        n_valid = torch.randint(1, topk + 1, (s_q,), generator=g).to(torch.int32)
    else:
        n_valid = torch.full((s_q,), topk, dtype=torch.int32)
    idx = torch.where(torch.arange(topk)[None, :] < n_valid[:, None], idx, torch.full_like(idx, -1))
    sm_scale = 576 ** -0.5
    k_buf = kv.view(s_kv, 1, 576)
    o, lse, att = run_reference(mod, q, k_buf, k_buf[..., :512], idx.clamp(min=0).contiguous(),
                                n_valid, sm_scale, splits, 1)
    d = dict(q=q.numpy(), kv=kv.numpy(), indices=idx.numpy(), sm_scale=np.float32(sm_scale),
             out=o.numpy(), lse=lse.numpy(), splits=np.int32(splits))
    if not ragged:
        d["att"] = att.numpy()     # stage-1 partials [S_q, h, splits, 513]: pins the split merge
    return d


def case_paged(mod, seed, batch, h, n_pages, page, seq_len, splits):
    g = torch.Generator().manual_seed(seed)
    q = _randn_bf16_exact_fp16((batch, h, 576), g)
    cache = _randn_bf16_exact_fp16((n_pages, page, 1, 576), g)
    pages_per = (seq_len + page - 1) // page
    table = torch.stack([torch.randperm(n_pages, generator=g)[:pages_per] for _ in range(batch)]).to(torch.int32)
    lens = torch.full((batch,), seq_len, dtype=torch.int32)
    sm_scale = 576 ** -0.5
    o, lse, _ = run_reference(mod, q, cache, cache[..., :512], table, lens, sm_scale, splits, page)
    return dict(q=q.numpy(), kv_cache=cache.view(n_pages, page, 576).numpy(), block_table=table.numpy(),
                context_lens=lens.numpy(), sm_scale=np.float32(sm_scale), page_size=np.int32(page),
                out=o.numpy(), lse=lse.numpy())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the FlagTree checkout whose kernel source is executed")
    args = ap.parse_args()
    mod, tmp = _load_reference_kernels(args.reference)
    try:
        cases = {
            "mla_topk_full_sq4_h16_topk64": case_topk(mod, 996, 4, 16, 256, 64, 4, False),
            "mla_topk_ragged_sq6_h16_topk96": case_topk(mod, 42, 6, 16, 300, 96, 3, True),
            "mla_topk_h32_sq3_topk40": case_topk(mod, 20, 3, 32, 128, 40, 2, True),
        }
        for name, d in cases.items():
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
            print("wrote", name, {k: getattr(v, "shape", v) for k, v in d.items()})
        d = case_paged(mod, 7, 3, 16, 12, 16, 73, 2)
        np.savez_compressed(os.path.join(HERE, "mla_paged16_b3_h16_len73.npz"), **d)
        print("wrote paged", {k: getattr(v, "shape", v) for k, v in d.items()})
    finally:
        import shutil
        shutil.rmtree(os.path.dirname(tmp), ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
