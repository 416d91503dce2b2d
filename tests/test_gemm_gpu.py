"""GPU parity of the tcgen05 GEMM (through the C ABI) against the fp32 CPU product, following the
reference's matmul test idiom (python/test/unit/operators/test_matmul.py:187-199: golden = torch.matmul
of the same inputs).  bf16 output: relative error bound 2^-8 of the row-block magnitude."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from flagtree_b200 import matmul, spec
    from flagtree_b200 import workloads as W

DEV = "cuda:0"


def _check(a, b, name=""):
    c = matmul(a.to(DEV), b.to(DEV))
    torch.cuda.synchronize()
    ref = a.float() @ b.float()
    err = (c.float().cpu() - ref).abs().max().item()
    scale = ref.abs().max().item()
    print(f"[{name}] max-abs err {err:.3e} (max |C| {scale:.3e})")
    assert err <= 2 ** -8 * scale + 1e-30, (name, err, scale)
    return c


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 128), (384, 768, 320),
                                   (200, 264, 72), (1, 8, 8), (130, 1000, 1096), (1024, 256, 2304)])
def test_matmul_shapes(m, n, k):
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = torch.randn(k, n, generator=g).bfloat16()
    _check(a, b, f"{m}x{n}x{k}")


@pytest.mark.parametrize("m,n,k", [(4096, 4864, 256), (2048, 9992, 128), (3072, 2560, 192)])
def test_leftover_tiles_run_as_half_width_steps(m, n, k):
    """Shapes whose tile count leaves a few tiles after the whole waves of a 148-SM GPU: 304 = 4 x 74 + 8 pair
    tiles; 320 = 4 x 74 + 24 with a last column block of 8 columns; 120 = 74 + 46 (too many left to halve).  The
    leftover runs as 128-column halves where that helps, and every element must still be the product."""
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = torch.randn(k, n, generator=g).bfloat16()
    c = _check(a, b, f"{m}x{n}x{k}")
    assert torch.equal(c, matmul(a.to(DEV), b.to(DEV)))


def test_matmul_powers_of_two_exact():
    """Inputs 2^randint(-3,0) as in test_matmul.py:164-176; K=64 keeps every fp32 partial sum exact,
    so the result must equal the fp32 product rounded to bf16 bit for bit."""
    g = torch.Generator().manual_seed(0)
    a = (2.0 ** torch.randint(-3, 1, (256, 64), generator=g)).bfloat16()
    b = (2.0 ** torch.randint(-3, 1, (64, 512), generator=g)).bfloat16()
    c = matmul(a.to(DEV), b.to(DEV)).cpu()
    assert torch.equal(c, (a.float() @ b.float()).bfloat16())


def test_cfg4_per_rank_product():
    case = W.gemm_cfg4(tp=8, rank=3)
    _check(case.a, case.b, case.name)


def test_strided_and_transposed_inputs_are_copied_like_the_reference():
    g = torch.Generator().manual_seed(5)
    a = torch.randn(96, 300, generator=g).bfloat16().to(DEV)
    b = torch.randn(512, 96, generator=g).bfloat16().to(DEV)
    c = matmul(a.t()[:256], b.t())          # both operands column-major views
    ref = a.t()[:256].float().cpu() @ b.t().float().cpu()
    assert (c.float().cpu() - ref).abs().max().item() <= 2 ** -8 * ref.abs().max().item()


def test_spec_hook_writes_into_caller_buffer():
    g = torch.Generator().manual_seed(9)
    a = torch.randn(256, 128, generator=g).bfloat16().to(DEV)
    b = torch.randn(128, 512, generator=g).bfloat16().to(DEV)
    c = torch.zeros(256, 512, dtype=torch.bfloat16, device=DEV)
    handled = spec.matmul_kernel(None, a, b, c, 256, 512, 128, torch.float32, None, True, torch.bfloat16)
    assert handled is True
    assert torch.equal(c, matmul(a, b))
    # unsupported dtype -> None, the reference's own kernel would run
    assert spec.matmul_kernel(None, a.half(), b.half(), c, 256, 512, 128, None, None, True, torch.float16) is None


def test_determinism():
    g = torch.Generator().manual_seed(1)
    a = torch.randn(1024, 2304, generator=g).bfloat16().to(DEV)
    b = torch.randn(2304, 1792, generator=g).bfloat16().to(DEV)
    assert torch.equal(matmul(a, b), matmul(a, b))
