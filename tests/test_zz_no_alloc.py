"""The entry point for hosts that must not allocate device memory (ftb_sparse_mla_fwd_static_scratch).

An inference engine that has given the whole GPU to its own memory pool, or a plugin that runs where the
CUDA allocator is hooked or forbidden, cannot hand this library a freshly allocated workspace.  For them the
split sparse-MLA forward keeps its per-split partials in a fixed 32 MiB array inside the library.  This
test drives that entry point through the C ABI twice in a row (the array keeps the first call's contents,
so the second call also proves that stale data does no harm) and compares each result with the regular
entry point, which gets its workspace from the caller, and with the CPU oracle, so that the entry point is
checked on its own and not only against its sibling.  The file name sorts last on purpose: a run that
stops at the first failure has already executed every other test.
"""
import ctypes as C

import pytest
import torch

from oracle.sparse_mla_ref import sparse_mla_fwd_ref   # the checker

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _args(lib_mod, q, kv, idx, out, lse, sm_scale, n_splits, ws):
    a = lib_mod.SparseMlaArgs()
    a.q, a.kv, a.indices, a.out, a.lse = q.data_ptr(), kv.data_ptr(), idx.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.s_q, a.h, a.s_kv, a.topk = q.shape[0], q.shape[1], kv.shape[0], idx.shape[1]
    a.q_stride_token, a.q_stride_head, a.kv_stride_row = q.stride(0), q.stride(1), kv.stride(0)
    a.idx_stride_token = idx.stride(0)
    a.out_stride_token, a.out_stride_head, a.lse_stride_token = out.stride(0), out.stride(1), lse.stride(0)
    a.sm_scale, a.lse_base2, a.algo_id = sm_scale, 0, 1
    a.n_splits = n_splits
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a


def test_static_scratch_entry_matches_regular_entry_twice():
    from flagtree_b200 import _lib
    lib = _lib.load()
    stream = C.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
    g = torch.Generator().manual_seed(77)
    for call, (s_q, topk, n_splits) in enumerate([(6, 512, 4), (3, 320, 5)]):     # two calls in a row, different shapes
        h, s_kv = 128, 900
        q = torch.randn(s_q, h, 576, generator=g).bfloat16().to(DEV)
        kv = torch.randn(s_kv, 576, generator=g).bfloat16().to(DEV)
        idx = torch.stack([torch.randperm(s_kv, generator=g)[:topk] for _ in range(s_q)]).int().to(DEV)
        idx[0, topk // 3:] = -1                      # later splits of this token are empty
        out_a = torch.empty(s_q, h, 512, dtype=torch.bfloat16, device=DEV)
        lse_a = torch.empty(s_q, h, dtype=torch.float32, device=DEV)
        out_b, lse_b = torch.empty_like(out_a), torch.empty_like(lse_a)
        ws = torch.empty(int(lib.ftb_sparse_mla_workspace_bytes(s_q, h, n_splits)), dtype=torch.uint8, device=DEV)
        a_ref = _args(_lib, q, kv, idx, out_a, lse_a, 0.05, n_splits, ws)
        a_new = _args(_lib, q, kv, idx, out_b, lse_b, 0.05, n_splits, None)
        with torch.cuda.device(DEV):
            assert lib.ftb_sparse_mla_fwd(C.byref(a_ref), stream) == 0, _lib.last_error()
            assert lib.ftb_sparse_mla_fwd_static_scratch(C.byref(a_new), stream) == 0, _lib.last_error()
        torch.cuda.synchronize()
        err = (out_a.float() - out_b.float()).abs().max().item()
        lerr = (lse_a - lse_b).abs().max().item()
        print(f"call {call}: out diff {err:.3e}, lse diff {lerr:.3e}")
        assert err <= 2e-2 and lerr <= 1e-3          # the tolerances of the other sparse-MLA tests
        assert torch.isfinite(out_b.float()).all()
        ref_out, ref_lse = sparse_mla_fwd_ref(q.cpu(), kv.cpu(), idx.cpu(), 0.05)
        o_err = (out_b.float().cpu() - ref_out).abs().max().item()
        l_err = ((lse_b.cpu() - ref_lse).abs() / ref_lse.abs().clamp(min=1.0)).max().item()
        print(f"call {call}: against the oracle: out {o_err:.3e}, lse {l_err:.3e}")
        assert o_err <= 2e-2 and l_err <= 1e-3


def test_static_scratch_rejects_oversized_problems():
    from flagtree_b200 import _lib
    lib = _lib.load()
    cap = int(lib.ftb_sparse_mla_static_scratch_bytes())
    assert cap == 32 << 20
    s_q, h, n_splits = 64, 128, 16                   # 64 * 16 * 128 * 513 * 4 bytes = 269 MB > 32 MiB
    assert lib.ftb_sparse_mla_workspace_bytes(s_q, h, n_splits) > cap
    q = torch.zeros(s_q, h, 576, dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros(64, 576, dtype=torch.bfloat16, device=DEV)
    idx = torch.zeros(s_q, 64, dtype=torch.int32, device=DEV)
    out = torch.empty(s_q, h, 512, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(s_q, h, dtype=torch.float32, device=DEV)
    a = _args(_lib, q, kv, idx, out, lse, 0.05, n_splits, None)
    rc = lib.ftb_sparse_mla_fwd_static_scratch(C.byref(a), None)
    assert rc == _lib.FTB_ERR_INVALID
    assert "built-in" in _lib.last_error()
