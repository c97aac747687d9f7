"""tcgen05 GEMM numerics against fp32 torch references."""
import pytest
import torch

from owl_engine_b200.ops import gemm_tc, quant as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(s):
    return torch.Generator().manual_seed(s)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 128, 64), (300, 256, 512), (77, 384, 192), (1024, 1024, 1024), (300, 1000, 320),
                                   (2048, 2304, 512), (257, 520, 64)])
def test_dense_gemm(dtype, shape):
    """Shapes with t >= 256 and n >= 512 run the persistent 128 x 256 kernel (ragged edges included)."""
    t, n, k = shape
    x = (torch.randn(t, k, generator=gen(1))).to(dtype)
    w = (torch.randn(n, k, generator=gen(2)) * 0.05).to(dtype)
    out = torch.zeros(t, n, dtype=torch.bfloat16, device=DEV)
    gemm_tc.f16_gemm(x.to(DEV), w.to(DEV), out)
    torch.cuda.synchronize()
    assert gemm_tc.gemm_status() == 0
    want = x.float() @ w.float().t()
    err = (out.float().cpu() - want).norm() / want.norm()
    assert err < 4e-3, err


@pytest.mark.parametrize("group", [128, 32])
@pytest.mark.parametrize("shape", [(128, 128, 128), (200, 256, 512), (37, 3584, 256), (512, 1024, 2176)])
def test_w4a16_gemm(group, shape):
    t, n, k = shape
    c = Q.quantize_w4(torch.randn(n, k, generator=gen(3)) * 0.05, group)
    w = Q.pack_skinny(c).to(DEV)
    x = torch.randn(t, k, generator=gen(4)).to(torch.float16)
    out = torch.zeros(t, n, dtype=torch.bfloat16, device=DEV)
    gemm_tc.w4a16_gemm(w, x.to(DEV), out)
    torch.cuda.synchronize()
    assert gemm_tc.gemm_status() == 0
    want = x.float() @ c.dequant().t()
    err = (out.float().cpu() - want).norm() / want.norm()
    assert err < 4e-3, err


@pytest.mark.parametrize("shape", [(300, 512, 1024), (128, 256, 128), (1024, 1000, 2176), (16, 512, 1024), (32, 5120, 2176)])
def test_e4m3_gemm_and_row_quantisation(shape):
    """kind::f8f6f4 product of row-quantised operands: exact against the dequantised operands, close to the 16-bit product."""
    t, n, k = shape
    x = torch.randn(t, k, generator=gen(5)).to(torch.float16)
    w = (torch.randn(n, k, generator=gen(6)) * 0.05).to(torch.float16)
    xq, sx = gemm_tc.quant_e4m3_rows(x.to(DEV))
    wq, sw = gemm_tc.quant_e4m3_rows(w.to(DEV))
    xd = xq.view(torch.float8_e4m3fn).float().cpu() * sx.cpu()[:, None]
    wd = wq.view(torch.float8_e4m3fn).float().cpu() * sw.cpu()[:, None]
    assert ((xd - x.float()).norm() / x.float().norm()) < 0.04          # e4m3: 3 mantissa bits
    assert torch.allclose(sx.cpu(), x.float().abs().amax(1) / 448, rtol=1e-3)
    out = torch.zeros(t, n, dtype=torch.bfloat16, device=DEV)
    gemm_tc.e4m3_gemm(xq, sx, wq, sw, out)
    torch.cuda.synchronize()
    assert gemm_tc.gemm_status() == 0
    want = xd @ wd.t()
    assert ((out.float().cpu() - want).norm() / want.norm()) < 4e-3
    full = x.float() @ w.float().t()
    assert ((out.float().cpu() - full).norm() / full.norm()) < 0.06


def test_w4a8_prefill_arm_close_to_w4a16():
    from owl_engine_b200.ops import linear

    t, n, k = 256, 512, 1024
    c = Q.quantize_w4(torch.randn(n, k, generator=gen(7)) * 0.05, 128)
    w = Q.pack_skinny(c).to(DEV)
    x = torch.randn(t, k, generator=gen(8)).to(torch.float16).to(DEV)
    o8 = torch.zeros(t, n, dtype=torch.bfloat16, device=DEV)
    linear.w4_gemm(w, x, o8, arm="tc8")
    want = x.float().cpu() @ c.dequant().t()
    assert ((o8.float().cpu() - want).norm() / want.norm()) < 0.06
