"""The tcgen05 GEMM entries (dsv32_gemm_bf16, dsv32_gemm_i8) against torch on the CPU.

int8 products are exact.  bf16 products are exact in fp32, so the only difference from a float64 reference is the
order of the fp32 additions: bounded here by 2e-6 x k x max|a| x max|b| absolute per element (and one bf16 rounding
for bf16 results)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("t,k,n", [(1, 64, 8), (37, 1024, 520), (300, 4096, 1024), (128, 128, 128), (5, 2560, 24)])
@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_bf16_matches_a_float64_product(t, k, n, layout, out_dtype):
    import pypto_b200
    from pypto_b200 import _runtime as rt
    g = torch.Generator().manual_seed(t * 7 + k + n)
    a = (torch.rand((t, k), generator=g) * 2 - 1).to(torch.bfloat16)
    b = (torch.rand((k, n), generator=g) * 2 - 1).to(torch.bfloat16)
    ref = a.double() @ b.double()
    bd = b.to(DEV) if layout == 0 else b.t().contiguous().to(DEV).t()      # [n, k] storage seen as [k, n]
    out = rt.gemm_bf16(a.to(DEV), bd, out_dtype)
    pypto_b200.check_status(DEV)
    assert out.dtype == out_dtype and tuple(out.shape) == (t, n)
    err = (out.cpu().double() - ref).abs()
    bound = 2e-6 * k + (ref.abs() * 2.0 ** -8 if out_dtype == torch.bfloat16 else 0)
    assert bool((err <= bound).all()), float(err.max())


@pytest.mark.parametrize("t,k,n", [(1, 128, 256), (37, 1024, 1024), (300, 1024, 4096)])
def test_gemm_i8_is_exact(t, k, n):
    import pypto_b200
    from pypto_b200 import _runtime as rt
    g = torch.Generator().manual_seed(t + k + n)
    a = torch.randint(-128, 128, (t, k), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (k, n), generator=g, dtype=torch.int8)
    out = rt.gemm_i8(a.to(DEV), b.to(DEV))
    pypto_b200.check_status(DEV)
    ref = (a.double() @ b.double()).to(torch.int32)          # |sum| <= 1024 * 2^14 < 2^53: exact in float64
    assert torch.equal(out.cpu(), ref)


def test_gemm_rejects_bad_shapes():
    from pypto_b200 import _runtime as rt
    a = torch.zeros((4, 100), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        rt.gemm_bf16(a, torch.zeros((100, 64), dtype=torch.bfloat16, device=DEV))         # k not a multiple of 64
    with pytest.raises(ValueError):
        rt.gemm_bf16(a[:, :64].contiguous(), torch.zeros((64, 12), dtype=torch.bfloat16, device=DEV))   # n not a multiple of 8
    with pytest.raises(ValueError):
        rt.gemm_i8(torch.zeros((4, 128), dtype=torch.int8, device=DEV), torch.zeros((128, 100), dtype=torch.int8, device=DEV))
    with pytest.raises(ValueError):
        rt.gemm_bf16(a[:, :64].contiguous(), torch.zeros((64, 64), dtype=torch.float32, device=DEV))
