"""Boot-time self-check: every kernel family runs once on a tiny input and is compared with an
independent host reference before the engine takes traffic. A wrong build, a mismatched weight
layout or a broken driver shows up here as a named failure instead of as wrong tokens later.

``run_all(device)`` returns ``[(name, ok, detail)]``; ``assert_ok`` raises with the failed names. The
engine runs it when ``EngineConfig.selfcheck`` is set (the server profile key ``probes.selfcheck``).

Reference counterpart: ``crates/kernels/src/ops/oracles/mod.rs:1-24`` (fp8 / int8 KV write, NC
attention, marlin, nvfp4, qknorm_insert, cublas oracles).
"""
from __future__ import annotations

import torch

from . import kernels as K
from . import quant as Q
from . import reference as R


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float().cpu() - b.float().cpu()).norm() / b.float().cpu().norm().clamp_min(1e-9))


def _g(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def check_w4_streaming(dev) -> float:
    c = Q.quantize_w4(torch.randn(128, 256, generator=_g(1)) * 0.05, 128)
    x = torch.randn(2, 256, generator=_g(2)).to(torch.bfloat16)
    xp = torch.empty(2, 512, dtype=torch.uint8, device=dev)
    xs = torch.empty(2, 2, 2, dtype=torch.float32, device=dev)
    K.act_pack(x.to(dev), xp, xs, 2, 256, 128)
    out = torch.zeros(2, 128, dtype=torch.bfloat16, device=dev)
    K.w4a16_skinny(Q.pack_skinny(c).to(dev), xp, xs, out, 2)
    return _rel(out, x.float() @ c.dequant().t())


def check_w4_tcgen05_stream(dev) -> float:
    c = Q.quantize_w4(torch.randn(128, 256, generator=_g(3)) * 0.05, 128)
    x = torch.randn(2, 256, generator=_g(4)).to(torch.bfloat16)
    xt = torch.zeros(K.act_tile_bytes(256, 128), dtype=torch.uint8, device=dev)
    K.act_pack(x.to(dev), xt, None, 2, 256, 128 | K.ACT_TILES)
    out = torch.zeros(2, 128, dtype=torch.bfloat16, device=dev)
    K.w4a16_stream_tc(Q.pack_skinny(c, "block").to(dev), xt, out, 2, K.StreamTcWorkspace(dev, max_n=128))
    return _rel(out, x.float() @ c.dequant().t())


def check_w4_tcgen05_gemm(dev) -> float:
    from . import gemm_tc

    c = Q.quantize_w4(torch.randn(128, 256, generator=_g(5)) * 0.05, 128)
    x = torch.randn(40, 256, generator=_g(6)).to(torch.float16)
    out = torch.zeros(40, 128, dtype=torch.bfloat16, device=dev)
    gemm_tc.w4a16_gemm(Q.pack_skinny(c).to(dev), x.to(dev), out)
    return _rel(out, x.float() @ c.dequant().t())


def check_dense_tcgen05_gemm(dev) -> float:
    from . import gemm_tc

    x = torch.randn(33, 128, generator=_g(7)).to(torch.bfloat16)
    w = torch.randn(64, 128, generator=_g(8)).to(torch.bfloat16)
    out = torch.zeros(33, 64, dtype=torch.bfloat16, device=dev)
    gemm_tc.f16_gemm(x.to(dev), w.to(dev), out)
    return _rel(out, x.float() @ w.float().t())


def check_rmsnorm(dev) -> float:
    h = torch.randn(3, 256, generator=_g(9)).to(torch.bfloat16)
    w = (torch.randn(256, generator=_g(10)) * 0.1).to(torch.bfloat16)
    out = torch.zeros(3, 256, dtype=torch.bfloat16, device=dev)
    K.rmsnorm_pack(h.to(dev), w.to(dev), normed=out, m=3, k=256, group=128)
    return _rel(out, R.rmsnorm(h.float(), w.float()))


def check_fp8_kv_write_and_attention(dev) -> float:
    """qk-norm + RoPE + fp8 insert, then paged attention over the written pages, against the host pipeline."""
    hq, hkv, hd, rot, t = 6, 1, 256, 64, 5
    g = _g(11)
    qkv = (torch.randn(t, 2 * hq * hd + 2 * hkv * hd, generator=g) * 0.5).to(torch.bfloat16)
    qn, kn = (torch.randn(hd, generator=g) * 0.1).to(torch.bfloat16), (torch.randn(hd, generator=g) * 0.1).to(torch.bfloat16)
    inv = R.rope_inv_freq(rot, 1e7)
    section = torch.zeros(rot // 2, dtype=torch.uint8)
    pos3 = torch.arange(t, dtype=torch.int32).repeat(3)
    k_pool = torch.zeros(4, 16, hkv, hd, dtype=torch.uint8, device=dev)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.zeros(t, hq, hd, dtype=torch.bfloat16, device=dev)
    kv_slot = (16 * 2 + torch.arange(t, dtype=torch.int32)).to(dev)          # page 2
    d = qkv.to(dev)
    qn_w = 2 * hq * hd
    K.qknorm_rope_insert(d, d.shape[1], d[:, qn_w:], d.shape[1], d[:, qn_w + hkv * hd:], d.shape[1], qn.to(dev), kn.to(dev),
                         pos3.to(dev), inv.to(dev), section.to(dev), kv_slot, q_out, k_pool, v_pool, t, hq, hkv, hd, rot)
    bt = torch.zeros(1, 4, dtype=torch.int32, device=dev)
    bt[0, 0] = 2
    splits = 1
    part_o = torch.zeros(t * hq * splits * hd, dtype=torch.float32, device=dev)
    part_ml = torch.zeros(t * hq * splits * 2, dtype=torch.float32, device=dev)
    K.paged_attn(q_out, k_pool, v_pool, bt, None,
                 torch.full((1,), t, dtype=torch.int32, device=dev), part_o, part_ml, 1, t, hq, hkv, hd, 4, splits, hd ** -0.5)
    out = torch.zeros(t, hq * hd, dtype=torch.bfloat16, device=dev)
    K.attn_reduce(part_o, part_ml, splits, None, 0, t, hq, out=out)
    # host pipeline
    qraw = qkv[:, :qn_w].float().view(t, hq, 2, hd)[:, :, 0]                   # [value | gate] per head: value half
    kraw = qkv[:, qn_w:qn_w + hkv * hd].float().view(t, hkv, hd)
    vraw = qkv[:, qn_w + hkv * hd:].float().view(t, hkv, hd)
    cos, sin = R.rope_cos_sin(pos3.view(3, t), inv, [0] * (rot // 2))
    qh = R.apply_rope(R.rmsnorm(qraw, qn.float()), cos, sin)
    kh = R.fp8_e4m3_roundtrip(R.apply_rope(R.rmsnorm(kraw, kn.float()), cos, sin))
    want = R.gqa_attention(qh, kh, R.fp8_e4m3_roundtrip(vraw), 0).reshape(t, hq * hd)
    return _rel(out, want)


def check_nvfp4(dev) -> float:
    from ..formats import nvfp4 as NV

    q = NV.quantize(torch.randn(64, 128, generator=_g(12)) * 0.05)
    x = torch.randn(1, 128, generator=_g(13)).to(torch.bfloat16)
    out = torch.zeros(1, 64, dtype=torch.bfloat16, device=dev)
    K.nvfp4_gemv(q.codes.to(dev), q.scales.to(dev), q.global_scale, x.to(dev), out, 1)
    return _rel(out, x.float() @ NV.dequantize(q).t())


def check_topk(dev) -> float:
    logits = (torch.randn(1, 1000, generator=_g(14)) * 3).to(torch.bfloat16)
    val, idx = K.TopK(dev, max_rows=1, k=8)(logits.to(dev), 1, 1000)
    want = torch.topk(logits.float(), 8).values
    return float((val.cpu() - want).abs().max())


CHECKS = [("w4 streaming gemv", check_w4_streaming, 1e-2), ("w4 tcgen05 streaming gemv", check_w4_tcgen05_stream, 1e-2),
          ("w4 tcgen05 gemm", check_w4_tcgen05_gemm, 1e-2), ("dense tcgen05 gemm", check_dense_tcgen05_gemm, 1e-2),
          ("rmsnorm", check_rmsnorm, 1e-2), ("qknorm + rope + fp8 kv write + paged attention", check_fp8_kv_write_and_attention, 6e-2),
          ("nvfp4 gemv", check_nvfp4, 2e-2), ("top-k", check_topk, 1e-6)]


def run_all(device="cuda") -> list[tuple[str, bool, str]]:
    out = []
    for name, fn, tol in CHECKS:
        try:
            err = fn(device)
            torch.cuda.synchronize()
            out.append((name, err <= tol, f"err {err:.3g} (tol {tol:g})"))
        except Exception as e:          # a failing check must not hide the others
            out.append((name, False, f"{type(e).__name__}: {e}"))
    return out


def assert_ok(device="cuda") -> None:
    bad = [f"{n}: {d}" for n, ok, d in run_all(device) if not ok]
    if bad:
        raise RuntimeError("kernel self-check failed:\n  " + "\n  ".join(bad))
