"""NVFP4 and GGUF device kernels against the host codecs."""
import numpy as np
import pytest
import torch

from owl_engine_b200.formats import gguf as G
from owl_engine_b200.formats import nvfp4 as NV
from owl_engine_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed=0):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("m", [1, 3, 8])
def test_nvfp4_gemv_dequant_and_act_quant(m):
    n, k = 200, 512
    w = torch.randn(n, k, generator=gen(1)) * 0.05
    q = NV.quantize(w)
    ref = NV.dequantize(q)
    codes, sf = q.codes.to(DEV), q.scales.to(DEV)
    deq = K.nvfp4_dequant(codes, sf, q.global_scale)
    torch.testing.assert_close(deq.float().cpu(), ref, rtol=1e-2, atol=1e-4)
    x = torch.randn(m, k, generator=gen(2)).to(torch.bfloat16)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    K.nvfp4_gemv(codes, sf, q.global_scale, x.to(DEV), out, m)
    want = x.float() @ ref.t()
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    # activation quantisation: same format, the dequantised result matches the host quantiser's
    a = NV.quantize_act(x.float())
    ac, asf = K.nvfp4_quant_act(x.to(DEV), a.global_scale)
    got = NV.dequantize(NV.NvFp4(ac.cpu(), asf.cpu(), a.global_scale, (m, k)))
    assert (asf.cpu() == a.scales).float().mean() > 0.99
    torch.testing.assert_close(got, NV.dequantize(a), rtol=0, atol=0.26 * x.float().abs().max().item() / 6 * 1.01)
    assert (ac.cpu() == a.codes).float().mean() > 0.98


def test_nvfp4_per_row_scales_residual_form_and_act_unpack():
    """Merged projections: rows keep their own tensors' scales; the residual form adds in the epilogue."""
    from owl_engine_b200.ops import quant as Q

    n, k, m = 96, 256, 5
    parts = [torch.randn(32, k, generator=gen(3)) * s for s in (0.02, 0.3, 0.08)]
    qs = [NV.quantize(p) for p in parts]
    ref = torch.cat([NV.dequantize(q) for q in qs])
    w = Q.NvFp4Linear(torch.cat([q.codes for q in qs]).to(DEV), torch.cat([q.scales for q in qs]).to(DEV), 1.0, n, k, 128, "nvfp4",
                      torch.cat([torch.full((32,), q.global_scale) for q in qs]).to(DEV))
    deq = K.nvfp4_linear_dequant(w, torch.empty(n, k, dtype=torch.bfloat16, device=DEV))
    torch.testing.assert_close(deq.float().cpu(), ref, rtol=1e-2, atol=1e-5)
    x = torch.randn(m, k, generator=gen(4)).to(torch.bfloat16)
    res = torch.randn(m, n, generator=gen(5)).to(torch.bfloat16)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    K.nvfp4_linear_gemv(w, x.to(DEV), out, m)
    want = x.float() @ ref.t()
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    K.nvfp4_linear_gemv(w, x.to(DEV), out, m, residual=res.to(DEV))
    torch.testing.assert_close(out.float().cpu(), want + res.float(), rtol=2e-2, atol=2e-2 * (want + res.float()).abs().max().item())


@pytest.mark.parametrize("tname", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "IQ4_NL", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ4_XS",
                                   "IQ3_XXS", "IQ3_S"])
def test_gguf_dequant_and_gemv(tname):
    n, k = 24, 512
    be, bb = G.BLOCK[tname]
    rng = np.random.default_rng(3)
    raw = rng.integers(0, 256, size=(n * k // be, bb), dtype=np.uint8)
    # keep the fp16 scale fields finite and moderate
    def set_f16(col, lo=0.001, hi=0.02):
        raw[:, col:col + 2] = rng.uniform(lo, hi, size=(raw.shape[0],)).astype(np.float16).view(np.uint8).reshape(-1, 2)
    if tname in ("Q8_0", "Q4_0", "Q5_0", "IQ4_NL", "IQ4_XS", "IQ3_XXS", "IQ3_S"):
        set_f16(0)
    elif tname in ("Q4_K", "Q5_K", "Q4_1", "Q5_1"):
        set_f16(0); set_f16(2)
    elif tname == "Q2_K":
        set_f16(80); set_f16(82)
    elif tname == "Q3_K":
        set_f16(108)
    else:
        set_f16(208)
    want = torch.from_numpy(G.dequantize(raw.reshape(-1), tname, n * k)).view(n, k)
    blocks = torch.from_numpy(raw.reshape(-1)).to(DEV)
    tid = G.TYPE_ID[tname]
    got = K.gguf_dequant(blocks, tid, k, n)
    torch.testing.assert_close(got.float().cpu(), want, rtol=1e-2, atol=1e-3 * want.abs().max().item())
    rows = torch.tensor([5, 0, 23], dtype=torch.int32, device=DEV)
    torch.testing.assert_close(K.gguf_dequant(blocks, tid, k, n, rows=rows).float().cpu(), want[[5, 0, 23]], rtol=1e-2,
                               atol=1e-3 * want.abs().max().item())
    m = 3
    x = torch.randn(m, k, generator=gen(4)).to(torch.bfloat16)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    K.gguf_gemv(blocks, tid, n, k, x.to(DEV), out, m)
    ref = x.float() @ want.t()
    torch.testing.assert_close(out.float().cpu(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item())
