"""The vision tower on this package's kernels (``csrc/vision.cu`` + the dense tcgen05 GEMM) against the fp32 torch tower."""
import dataclasses

import pytest
import torch

from owl_engine_b200.models import vision as V

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


@pytest.mark.parametrize("real_heads", [False, True])
def test_kernel_tower_matches_the_fp32_tower(real_heads):
    # real_heads: head_dim 72 (16 heads of the 27B family's tower), inter not a multiple of 64, two blocks
    sp = dataclasses.replace(V.VisionSpec(), depth=2, out_hidden=512) if real_heads else V.tiny_vision(out_hidden=256)
    w = V.init_vision_weights(sp, seed=1, std=0.05)
    for k in w:                                  # biases and norm weights away from their trivial values
        if k.endswith("bias"):
            w[k] = torch.randn_like(w[k]) * 0.05
        elif "norm" in k and k.endswith("weight"):
            w[k] = 1.0 + torch.randn_like(w[k]) * 0.1
    ref = V.VisionTower(sp, w, device=DEV, dtype=torch.float32)
    ker = V.VisionTowerKernels(sp, w, device=DEV)
    g = torch.Generator().manual_seed(2)
    imgs = [(torch.randn(gh * gw, sp.patch_dim, generator=g), (1, gh, gw)) for gh, gw in [(8, 12), (6, 6), (16, 10)]]
    outs = ker.forward_many(imgs)
    torch.cuda.synchronize()
    for (p, grid), got in zip(imgs, outs):
        want = ref.forward(p, grid)
        assert got.shape == want.shape
        assert _rel(got, want) < 3e-2, _rel(got, want)
    # one image alone gives the same rows as inside the batch up to bf16 rounding along other GEMM tile paths (segments do not
    # leak into each other: a leak would be an error of order one)
    alone = ker.forward(*imgs[1])
    assert _rel(alone, outs[1]) < 2e-2


def test_single_operators_against_torch():
    from owl_engine_b200.ops import kernels as K

    V._bind_vision(K)
    g = torch.Generator(device=DEV).manual_seed(0)
    n, C = 50, 1152
    x = torch.randn(n, C, device=DEV, generator=g).bfloat16()
    w, b = torch.randn(C, device=DEV, generator=g), torch.randn(C, device=DEV, generator=g)
    y = torch.empty_like(x)
    K.call("owl_vis_layernorm", K.ptr(x), C, K.ptr(w), K.ptr(b), K.ptr(y), C, n, C, 1e-6, K.stream())
    want = torch.nn.functional.layer_norm(x.float(), (C,), w, b, 1e-6)
    assert _rel(y, want) < 5e-3
    for act, fn in [(1, lambda t: torch.nn.functional.gelu(t, approximate="tanh")), (2, torch.nn.functional.gelu)]:
        K.call("owl_vis_bias_act", K.ptr(x), C, K.ptr(b), K.ptr(x), C, K.ptr(y), C, n, C, act, K.stream())
        assert _rel(y, fn(x.float() + b) + x.float()) < 5e-3
    # non-causal attention over two segments, head_dim 72
    heads, hd = 4, 72
    qkv = torch.randn(n, 3, heads, hd, device=DEV, generator=g).bfloat16()
    seg = torch.tensor([0, 21, n], dtype=torch.int32, device=DEV)
    out = torch.empty(n, heads * hd, dtype=torch.bfloat16, device=DEV)
    K.call("owl_vis_attn", K.ptr(qkv), K.ptr(out), n, heads, hd, K.ptr(seg), 2, K.stream())
    torch.cuda.synchronize()
    q, k, v = (qkv[:, i].float().permute(1, 0, 2) for i in range(3))
    want = torch.empty(n, heads, hd, device=DEV)
    for lo, hi in [(0, 21), (21, n)]:
        a = torch.nn.functional.scaled_dot_product_attention(q[None, :, lo:hi], k[None, :, lo:hi], v[None, :, lo:hi])[0]
        want[lo:hi] = a.permute(1, 0, 2)
    assert _rel(out.view(n, heads, hd), want) < 1e-2
