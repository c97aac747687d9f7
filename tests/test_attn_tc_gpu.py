"""Fused tcgen05 prefill attention (``csrc/attn_tc.cu``) against an fp32 softmax of the same operands, ragged lengths."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(qg, k, vt, gq, pos0, scale):
    """qg [hkv, rows, hd], k [hkv, ctx, hd], vt [hkv, hd, ctx] (float32 on the CPU)."""
    hkv, rows, hd = qg.shape
    ctx = k.shape[1]
    s = torch.einsum("hrd,hkd->hrk", qg, k) * scale
    lim = pos0 + torch.arange(rows) // gq + 1
    mask = torch.arange(ctx)[None, :] >= lim[:, None]
    s = s.masked_fill(mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hrk,hdk->hrd", p, vt)


@pytest.mark.parametrize("t,pos0,gq,hkv", [(16, 0, 6, 1), (37, 100, 6, 2), (128, 1000, 6, 1), (301, 333, 3, 2), (64, 4040, 6, 4)])
def test_fused_attention_matches_fp32_softmax(t, pos0, gq, hkv):
    from owl_engine_b200.ops import kernels as K

    hd = 256
    g = torch.Generator().manual_seed(t + pos0)
    ctx = pos0 + t
    ctx_pad = (ctx + 63) // 64 * 64
    rows = t * gq
    qg = (torch.randn(hkv, rows, hd, generator=g) * 1.5).bfloat16()
    k = torch.zeros(hkv, ctx_pad, hd, dtype=torch.bfloat16)
    k[:, :ctx] = torch.randn(hkv, ctx, hd, generator=g).bfloat16()
    vt = torch.zeros(hkv, hd, ctx_pad, dtype=torch.float16)
    vt[:, :, :ctx] = torch.randn(hkv, hd, ctx, generator=g).half()
    # a few very large scores so that the running maximum moves late in the row (the O rescale path)
    k[:, ctx // 2] *= 6.0
    k[:, ctx - 1] *= 9.0
    og = torch.full((hkv, rows + 3, hd), 5.0, dtype=torch.bfloat16, device=DEV)[:, :rows].contiguous()
    scale = 1 / math.sqrt(hd)
    dq, dk, dv = qg.to(DEV), k.to(DEV), vt.to(DEV)          # held until the kernel has run
    K.call("owl_attn_tc", K.ptr(dq), K.ptr(dk), K.ptr(dv), K.ptr(og), rows, gq, hkv, ctx_pad, pos0, scale, K.stream())
    torch.cuda.synchronize()
    assert K.all_status()["attn_tc"] == 0
    want = _ref(qg.float(), k.float(), vt.float(), gq, pos0, scale)
    got = og.float().cpu()
    err = (got - want).norm() / want.norm()
    assert err < 8e-3, err
    assert float((got - want).abs().max()) < 0.05 * float(want.abs().max()) + 0.02


def test_prefill_path_uses_the_fused_kernel_and_matches_the_gemm_form():
    from owl_engine_b200.ops import kernels as K

    hq, hkv, hd, t, ctx = 12, 2, 256, 160, 2304
    pages = ctx // 16
    g = torch.Generator(device=DEV).manual_seed(3)
    kp = torch.randint(0, 120, (pages, 16, hkv, hd), dtype=torch.uint8, device=DEV, generator=g)
    vp = torch.randint(0, 120, (pages, 16, hkv, hd), dtype=torch.uint8, device=DEV, generator=g)
    bt = torch.randperm(pages, device=DEV, generator=g).to(torch.int32)
    q = torch.randn(t, hq, hd, device=DEV, generator=g).bfloat16()
    qraw = torch.randn(t, hq * 2 * hd, device=DEV, generator=g).bfloat16()
    ws = K.attn_gemm_ws(DEV, t, ctx, hq, hkv, hd)
    outs = []
    for fused in (True, False):
        K.ATTN_FUSED = fused
        out = torch.empty(t, hq * hd, dtype=torch.bfloat16, device=DEV)
        K.attn_gemm_prefill(q, kp, vp, None, bt, ctx - t, t, hq, hkv, hd, 1 / math.sqrt(hd), ws, qraw, hq * 2 * hd, out)
        torch.cuda.synchronize()
        outs.append(out.float())
    K.ATTN_FUSED = True
    assert K.all_status()["attn_tc"] == 0
    err = (outs[0] - outs[1]).norm() / outs[1].norm()
    assert err < 1e-2, err
