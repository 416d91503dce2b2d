"""GPU parity of the block-scaled FP8 GEMM against the CPU oracle (dequantise, fp32 product).  Tolerance:
the reference's fp8 GEMM tests use rtol = atol = 1e-2 on fp16 outputs
(third_party/mthreads/python/test/sqmma/base_cases/test_batch_fp8.py:54-57); the inputs here are exact e4m3
values, so the only error is fp32 accumulation order and the bf16 rounding of the output."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from flagtree_b200 import matmul_fp8_blockscaled
    from flagtree_b200 import workloads as W
from oracle.gemm_rs_ref import gemm_rs_fp8_ref

DEV = "cuda:0"


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (128, 256, 512), (256, 384, 1024), (200, 128, 256), (1024, 8192, 3584)])
def test_fp8_blockscaled_matches_oracle(m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    a8, a_s = W.quantize_block_e4m3(torch.randn(m, k, generator=g), 1, 128)
    b8, b_s = W.quantize_block_e4m3(torch.randn(k, n, generator=g), 128, 128)
    c = matmul_fp8_blockscaled(a8.to(DEV), a_s.to(DEV), b8.to(DEV), b_s.to(DEV))
    torch.cuda.synchronize()
    ref = gemm_rs_fp8_ref([a8], [a_s], [b8], [b_s])[0]
    err = (c.float().cpu() - ref).abs().max().item()
    scale = ref.abs().max().item()
    print(f"[fp8 {m}x{n}x{k}] max-abs err {err:.3e} (max |C| {scale:.3e})")
    assert err <= 2 ** -8 * scale


def test_weight_kept_as_n_by_k_gives_the_same_bits():
    """B passed as the transposed view of an [N, K] weight (the K-major operand of the tensor cores) must give the
    result of the [K, N] row-major call bit for bit: the same products are summed in the same order."""
    c = W.gemm_cfg5(tp=1, rank=0, m=384, n=512, k_total=640)
    a, b, a_s, b_s = c.a.to(DEV), c.b.to(DEV), c.a_scale.to(DEV), c.b_scale.to(DEV)
    ref = matmul_fp8_blockscaled(a, a_s, b, b_s)
    w = b.t().contiguous()                      # [N, K]
    got = matmul_fp8_blockscaled(a, a_s, w.t(), b_s)
    assert torch.equal(ref, got)


def test_fp8_unit_scales_equal_plain_product():
    g = torch.Generator().manual_seed(3)
    a = torch.randint(-8, 9, (256, 256), generator=g).float()
    b = torch.randint(-8, 9, (256, 256), generator=g).float()
    a8, b8 = a.to(torch.float8_e4m3fn).view(torch.uint8), b.to(torch.float8_e4m3fn).view(torch.uint8)
    ones_a, ones_b = torch.ones(256, 2), torch.ones(2, 2)
    c = matmul_fp8_blockscaled(a8.to(DEV), ones_a.to(DEV), b8.to(DEV), ones_b.to(DEV)).float().cpu()
    assert torch.equal(c, (a @ b).bfloat16().float())      # small integers: every partial sum is exact
