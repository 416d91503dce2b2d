"""A bounded device-side wait that runs out, on one GPU, without a fault or a hang: a tensor-parallel context of
two ranks whose buffers both live on this GPU, of which only rank 0 ever launches.  Rank 0's kernel pushes its
partial of rank 1's rows, then waits for rank 1's partial of its own rows, which never comes; with the wait limit
set to a few milliseconds the kernel gives up, returns, and the status word reads FTB_ERR_TIMEOUT.  The next call
on the same status word returns at once (the context is dead until it is rebuilt), and the Python layer turns the
status into a RuntimeError."""
import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def test_wait_for_a_rank_that_never_launches_times_out():
    from flagtree_b200 import _lib
    from flagtree_b200.ops import _check_status
    lib = _lib.load()
    m, n, k, tp = 512, 512, 128, 2
    rb, fb = C.c_int64(), C.c_int64()
    assert lib.ftb_gemm_rs_workspace_bytes(m, n, tp, C.byref(rb), C.byref(fb)) == 0
    recv = [torch.zeros(rb.value, dtype=torch.uint8, device=DEV) for _ in range(tp)]
    flags = [torch.zeros(fb.value, dtype=torch.uint8, device=DEV) for _ in range(tp)]
    recv_ptrs = (C.c_void_p * tp)(*[t.data_ptr() for t in recv])
    flag_ptrs = (C.c_void_p * tp)(*[t.data_ptr() for t in flags])
    ctx = C.c_void_p()
    with torch.cuda.device(DEV):
        assert lib.ftb_gemm_rs_ctx_create(C.byref(ctx), 0, tp, m, n, recv_ptrs, flag_ptrs) == 0, _lib.last_error()
        assert lib.ftb_gemm_rs_ctx_set_wait_limit(ctx, 0) == _lib.FTB_ERR_INVALID
        assert lib.ftb_gemm_rs_ctx_set_wait_limit(ctx, 20_000_000) == 0          # about 10 ms
    a = torch.randn(m, k, device=DEV).bfloat16()
    b = torch.randn(k, n, device=DEV).bfloat16()
    out = torch.zeros(m // tp, n, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)

    def call():
        with torch.cuda.device(DEV):
            rc = lib.ftb_gemm_rs(ctx, a.data_ptr(), b.data_ptr(), out.data_ptr(), k, a.stride(0), b.stride(0), out.stride(0),
                                 status.data_ptr(), stream)
        assert rc == 0, _lib.last_error()
        t0 = time.perf_counter()
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    t_first = call()
    assert int(status.item()) == _lib.FTB_ERR_TIMEOUT
    assert t_first < 1.0, f"the wait took {t_first:.3f} s with a limit of about 10 ms"
    # rank 0's partial of rank 1's rows did arrive in rank 1's receive slot before the wait began
    assert recv[1].view(torch.bfloat16).float().abs().sum().item() > 0
    t_second = call()                                                            # returns at once: status is set
    assert int(status.item()) == _lib.FTB_ERR_TIMEOUT and t_second < 0.05
    with pytest.raises(RuntimeError, match="TIMEOUT"):
        _check_status(status, "gemm_rs")
    lib.ftb_gemm_rs_ctx_destroy(ctx)
    # the device is healthy: an ordinary call still works
    from flagtree_b200 import matmul
    c = matmul(a, b)
    assert torch.isfinite(c.float()).all()
