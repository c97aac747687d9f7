"""Block-scaled NVFP4 GEMM (``csrc/gemm_nvfp4.cu``) against fp32 products of the dequantised operands."""
import pytest
import torch

from owl_engine_b200.formats import nvfp4

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _deq(codes, scales, k):
    r = codes.shape[0]
    c = torch.stack([codes & 0xF, codes >> 4], dim=-1).view(r, k)
    bs = scales.view(torch.float8_e4m3fn).float()
    return (nvfp4.decode_e2m1(c).view(r, k // 16, 16) * bs[..., None]).view(r, k)


@pytest.mark.parametrize("t,k", [(128, 256), (200, 320), (5, 64)])
def test_quant_rows_matches_host_codec(t, k):
    from owl_engine_b200.ops import nvfp4_tc

    x = (torch.randn(t, k, generator=torch.Generator().manual_seed(1)) * torch.rand(t, 1) * 3).bfloat16()
    codes, sf, sx = nvfp4_tc.quant_rows(x.to(DEV))
    wc, ws, wg = nvfp4.quantize_rows(x.float())
    assert torch.allclose(sx.cpu(), wg, rtol=1e-6)
    assert torch.equal(sf.cpu().view(-1, 512), nvfp4.pack_sf_atoms(ws).view(-1, 512))
    # codes may differ where a value sits on a rounding boundary of the division; the dequantised row must agree closely
    got = _deq(codes.cpu(), ws, k) * sx.cpu()[:, None]
    want = _deq(wc, ws, k) * wg[:, None]
    assert (codes.cpu() != wc).float().mean() < 0.01
    assert ((got - want).norm() / want.norm()) < 0.02
    # fp16 input takes the same path
    c2, _, s2 = nvfp4_tc.quant_rows(x.to(DEV).half())
    assert torch.allclose(s2.cpu(), wg, rtol=1e-3) and (c2.cpu() != wc).float().mean() < 0.02


@pytest.mark.parametrize("t,n,k,rows", [(128, 128, 256, False), (256, 384, 1024, True), (300, 200, 576, False), (2048, 1024, 5120, True)])
def test_gemm_matches_fp32_product_of_the_dequantised_operands(t, n, k, rows):
    from owl_engine_b200.ops import nvfp4_tc, quant as Q

    g = torch.Generator().manual_seed(t + n + k)
    w = torch.randn(n, k, generator=g) * 0.05
    x = (torch.randn(t, k, generator=g) * (torch.rand(t, 1, generator=g) + 0.5)).bfloat16()
    lw = Q.nvfp4_linear(w, DEV)
    if rows:
        lw.row_scale = (torch.rand(n, generator=g) + 0.5).to(DEV)
    xq = nvfp4_tc.quant_rows(x.to(DEV))
    out = torch.full((t, n + 8), 7.0, dtype=torch.bfloat16, device=DEV)[:, :n]
    nvfp4_tc.gemm(lw, x.to(DEV), out, xq=xq)
    torch.cuda.synchronize()
    assert nvfp4_tc.status() == 0
    # oracle from the device's own codes: exact up to fp32 summation order and the bf16 rounding of the result
    xs = torch.zeros(t, k // 16, dtype=torch.uint8)
    atoms = xq[1].cpu().view(-1, 4 * ((k + 255) // 256), 32, 4, 4)           # [block, atom, r%32, r//32, b]
    full = atoms.permute(0, 3, 2, 1, 4).reshape(-1, atoms.shape[1] * 4)     # [rows padded, blocks padded]
    xs[:] = full[:t, :k // 16]
    xd = _deq(xq[0].cpu(), xs, k).double() * xq[2].cpu().double()[:, None]
    wd = _deq(lw.codes.cpu(), lw.scales.cpu().view(n, k // 16), k).double() * lw.alpha
    want = xd @ wd.t()
    if rows:
        want = want * lw.row_scale.cpu().double()[None]
    got = out.double().cpu()
    err = (got - want).abs()
    assert float((err / (want.abs() + 1e-3 * want.abs().max())).max()) < 0.01      # bf16: 2^-9 relative, fp32 sums
    assert float(err.norm() / want.norm()) < 3e-3
    # and the W4A4 product is a usable approximation of the 16-bit one
    ref = x.double() @ w.double().t() * (lw.row_scale.cpu().double()[None] if rows else 1.0)
    assert float((got - ref).norm() / ref.norm()) < 0.2
    assert bool((out._base[:, n:] == 7.0).all())           # nothing written past column N


def test_linear_arm_tc4_routes_long_chunks_to_the_block_scaled_product():
    from owl_engine_b200.ops import linear, nvfp4_tc, quant as Q

    g = torch.Generator().manual_seed(5)
    w = torch.randn(512, 1024, generator=g) * 0.05
    lw = Q.nvfp4_linear(w, DEV)
    for t in (4, 64, 256):
        x = torch.randn(t, 1024, generator=g).bfloat16().to(DEV)
        a = torch.empty(t, 512, dtype=torch.bfloat16, device=DEV)
        b = torch.empty(t, 512, dtype=torch.bfloat16, device=DEV)
        linear.nvfp4_gemm(lw, x, a, arm="tc4")
        linear.nvfp4_gemm(lw, x, b, arm="tc")
        rel = float((a.float() - b.float()).norm() / b.float().norm())
        assert rel < (0.2 if t >= nvfp4_tc.MIN_ROWS else 1e-2), (t, rel)
    assert nvfp4_tc.status() == 0
