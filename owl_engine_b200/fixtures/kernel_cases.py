"""Small single-kernel cases for profiler captures: each case launches ONE kernel family a few times on inputs larger than
L2 but well under a few GB, then exits.

``python -m owl_engine_b200.fixtures.kernel_cases <case>`` with case in
``gemm16 gemm8 gemm_nvfp4 quant_nvfp4 gemm_w4 gemv attn attn16 attn_prefill_tc attn_tc_only attn_prefill_gemm attn_prefill_fused gdn_decode gdn_scan dflash_attn`` (prints the CUDA-event time per launch; integer arguments of a case may follow its name).
"""
import math
import sys

import torch

from owl_engine_b200.ops import gemm_tc, kernels as K, quant as Q

dev = "cuda"
N_LAUNCH = 6


def timed(fn):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(N_LAUNCH):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / N_LAUNCH


def gemm16():
    t, n, k = 2048, 16384, 5120
    x = torch.randn(t, k, device=dev).half()
    w = (torch.randn(n, k, device=dev) * 0.02).half()
    out = torch.empty(t, n, dtype=torch.bfloat16, device=dev)
    ms = timed(lambda: gemm_tc.f16_gemm(x, w, out))
    return ms, f"{2 * t * n * k / ms / 1e9:.0f} TFLOP/s"


def gemm8():
    t, n, k = 2048, 16384, 5120
    x = torch.randn(t, k, device=dev).half()
    w = (torch.randn(n, k, device=dev) * 0.02).half()
    xq, sx = gemm_tc.quant_e4m3_rows(x)
    wq, sw = gemm_tc.quant_e4m3_rows(w)
    out = torch.empty(t, n, dtype=torch.bfloat16, device=dev)
    ms = timed(lambda: gemm_tc.e4m3_gemm(xq, sx, wq, sw, out))
    return ms, f"{2 * t * n * k / ms / 1e9:.0f} TFLOP/s"


def gemm_nvfp4(t: int = 2048, n: int = 34816, k: int = 5120):
    """The merged gate / up projection of a 2048-token chunk, both operands NVFP4 (block-scaled tensor-core path)."""
    from owl_engine_b200.ops import nvfp4_tc

    w = Q.random_nvfp4(n, k, dev)
    x = torch.randn(t, k, device=dev).bfloat16()
    xq = nvfp4_tc.quant_rows(x)
    out = torch.empty(t, n, dtype=torch.bfloat16, device=dev)
    nvfp4_tc.weight_atoms(w)
    ms = timed(lambda: nvfp4_tc.gemm(w, x, out, xq=xq))
    return ms, f"{2 * t * n * k / ms / 1e9:.0f} TFLOP/s (status {nvfp4_tc.status()})"


def quant_nvfp4(t: int = 2048, k: int = 17408):
    """Activation quantisation of the same path: bf16 rows -> e2m1 codes, e4m3 scale atoms, fp32 row scales."""
    from owl_engine_b200.ops import nvfp4_tc

    x = torch.randn(t, k, device=dev).bfloat16()
    bufs = nvfp4_tc.quant_rows(x)
    ms = timed(lambda: nvfp4_tc.quant_rows(x, *bufs))
    return ms, f"{(t * k * 2 + t * k // 2 + t * k // 16) / ms / 1e9:.3f} TB/s"


def gemm_w4():
    t, n, k = 128, 16384, 5120
    w = Q.random_skinny(n, k, 128, dev)
    x = torch.randn(t, k, device=dev).half()
    out = torch.empty(t, n, dtype=torch.bfloat16, device=dev)
    ms = timed(lambda: gemm_tc.w4a16_gemm(w, x, out))
    return ms, f"{2 * t * n * k / ms / 1e9:.0f} TFLOP/s"


def gemv():
    n, k, m = 34816, 5120, 1
    ws = [Q.random_skinny(n, k, 128, dev, seed=i) for i in range(3)]        # 3 x 95 MB: every launch misses L2
    xp = torch.randint(0, 127, (m, 2 * k), dtype=torch.uint8, device=dev)
    xs = torch.rand(m, k // 128, 2, device=dev)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    i = [0]

    def f():
        K.w4a16_skinny(ws[i[0] % 3], xp, xs, out, m)
        i[0] += 1
    ms = timed(f)
    return ms, f"{ws[0].records.numel() / ms / 1e9:.2f} TB/s"


def gemv_fma(k: int = 5120, n: int = 34816, norm: bool = True):
    """One-token W4A16 projection on the half-precision FMA arm: the gate / up shape with the fused RMSNorm prologue and the
    silu * up epilogue (three weight copies, so every launch misses L2)."""
    ws = [Q.random_skinny(n, k, 128, dev, seed=i) for i in range(3)]
    h = torch.randn(k, device=dev).bfloat16()
    nw = (torch.randn(k, device=dev) * 0.1).bfloat16()
    out = torch.zeros(n // 2, dtype=torch.bfloat16, device=dev)
    i = [0]

    def f():
        K.w4_fma(ws[i[0] % 3], h, out, norm_w=nw if norm else None, epi=K.EPI_SILU_MUL)
        i[0] += 1
    ms = timed(f)
    return ms, f"{ws[0].records.numel() / ms / 1e9:.2f} TB/s"


def gemv_fma_down():
    """The down-projection shape (17408 -> 5120) with the residual epilogue."""
    n, k = 5120, 17408
    ws = [Q.random_skinny(n, k, 128, dev, seed=i) for i in range(4)]
    x = torch.randn(k, device=dev).bfloat16()
    hbuf = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    i = [0]

    def f():
        K.w4_fma(ws[i[0] % 4], x, hbuf, residual=hbuf, epi=K.EPI_RESIDUAL)
        i[0] += 1
    ms = timed(f)
    return ms, f"{ws[0].records.numel() / ms / 1e9:.2f} TB/s"


def attn(kv16: bool = False):
    hq, hkv, hd, ctx, b = 24, 4, 256, 32768, 4                              # 4 sequences x 32k tokens: 268 MB of fp8 KV
    pages = b * ctx // 16
    if kv16:                                                                # the 16-bit pool: 537 MB of fp16 words
        kp = torch.randn(pages, 16, hkv, hd, device=dev).half()
        vp = torch.randn(pages, 16, hkv, hd, device=dev).half()
    else:
        kp = torch.randint(0, 120, (pages, 16, hkv, hd), dtype=torch.uint8, device=dev)
        vp = torch.randint(0, 120, (pages, 16, hkv, hd), dtype=torch.uint8, device=dev)
    bt = torch.arange(pages, dtype=torch.int32, device=dev).view(b, -1).contiguous()
    q = torch.randn(b, hq, hd, device=dev).bfloat16()
    splits = 32
    po = torch.empty(b * hq * splits * hd, device=dev)
    pml = torch.empty(b * hq * splits * 2, device=dev)
    ctxs = torch.full((b,), ctx, dtype=torch.int32, device=dev)
    rows = torch.arange(b, dtype=torch.int32, device=dev)
    ms = timed(lambda: K.paged_attn(q, kp, vp, bt, rows, ctxs, po, pml, b, 1, hq, hkv, hd, bt.shape[1], splits, 1 / math.sqrt(hd)))
    return ms, f"{2 * kp.numel() * kp.element_size() / ms / 1e9:.2f} TB/s of KV"


def attn16():
    return attn(True)


def _prefill_attn_case(ctx: int, t: int):
    hq, hkv, hd = 24, 4, 256
    pages = ctx // 16
    kp = torch.randint(0, 120, (pages, 16, hkv, hd), dtype=torch.uint8, device=dev)
    vp = torch.randint(0, 120, (pages, 16, hkv, hd), dtype=torch.uint8, device=dev)
    bt = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
    q = torch.randn(t, hq, hd, device=dev).bfloat16()
    qraw = torch.randn(t, hq * 2 * hd, device=dev).bfloat16()
    return hq, hkv, hd, kp, vp, bt, q, qraw


def attn_prefill_tc(ctx: int = 8192, t: int = 2048):
    """The last 2048-row chunk of an 8192-token prompt, attention only, on the fused tcgen05 kernel (gather + group + one
    kernel with S and O in tensor memory + gate). ``attn_tc_only`` times the fused kernel alone."""
    K.ATTN_FUSED = True
    hq, hkv, hd, kp, vp, bt, q, qraw = _prefill_attn_case(ctx, t)
    ws = K.attn_gemm_ws(dev, t, ctx, hq, hkv, hd)
    out = torch.empty(t, hq * hd, dtype=torch.float16, device=dev)
    ms = timed(lambda: K.attn_gemm_prefill(q, kp, vp, None, bt[0], ctx - t, t, hq, hkv, hd, 1 / math.sqrt(hd), ws, qraw,
                                           hq * 2 * hd, out))
    flops = 4 * hq * hd * (t * (ctx - t) + t * t / 2)
    return ms, f"{flops / ms / 1e9:.0f} TFLOP/s of causal attention work (status {K.all_status()['attn_tc']})"


def attn_tc_only(ctx: int = 8192, t: int = 2048):
    hq, hkv, hd = 24, 4, 256
    gq = hq // hkv
    qg = torch.randn(hkv, t * gq, hd, device=dev).bfloat16()
    kk = torch.randn(hkv, ctx, hd, device=dev).bfloat16()
    vt = torch.randn(hkv, hd, ctx, device=dev).half()
    og = torch.empty(hkv, t * gq, hd, dtype=torch.bfloat16, device=dev)
    ms = timed(lambda: K.call("owl_attn_tc", K.ptr(qg), K.ptr(kk), K.ptr(vt), K.ptr(og), t * gq, gq, hkv, ctx, ctx - t,
                              1 / math.sqrt(hd), K.stream()))
    flops = 4 * hq * hd * (t * (ctx - t) + t * t / 2)
    return ms, f"{flops / ms / 1e9:.0f} TFLOP/s of causal attention work (status {K.all_status()['attn_tc']})"


def attn_prefill_gemm(ctx: int = 8192, t: int = 2048):
    """The last 2048-row chunk of an 8192-token prompt, attention only, GEMM form (gather + 4 x (GEMM, softmax, GEMM) + gate)."""
    K.ATTN_FUSED = False
    hq, hkv, hd, kp, vp, bt, q, qraw = _prefill_attn_case(ctx, t)
    ws = K.attn_gemm_ws(dev, t, ctx, hq, hkv, hd)
    out = torch.empty(t, hq * hd, dtype=torch.float16, device=dev)
    ms = timed(lambda: K.attn_gemm_prefill(q, kp, vp, None, bt[0], ctx - t, t, hq, hkv, hd, 1 / math.sqrt(hd), ws, qraw,
                                           hq * 2 * hd, out))
    flops = 4 * hq * hd * (t * (ctx - t) + t * t / 2)
    return ms, f"{flops / ms / 1e9:.0f} TFLOP/s of causal attention work"


def attn_prefill_fused(ctx: int = 8192, t: int = 2048):
    """The same chunk on the fused warp-level kernel (8 query rows per group, one KV split)."""
    hq, hkv, hd, kp, vp, bt, q, qraw = _prefill_attn_case(ctx, t)
    ng = t // 8
    po = torch.empty(t * hq * hd, device=dev)
    pml = torch.empty(t * hq * 2, device=dev)
    ctxs = (torch.arange(ng, dtype=torch.int32, device=dev) * 8 + (ctx - t) + 8).contiguous()
    rows = torch.zeros(ng, dtype=torch.int32, device=dev)
    out = torch.empty(t, hq * hd, dtype=torch.float16, device=dev)

    def f():
        K.paged_attn(q, kp, vp, bt, rows, ctxs, po, pml, ng, 8, hq, hkv, hd, bt.shape[1], 1, 1 / math.sqrt(hd))
        K.attn_reduce(po, pml, 1, qraw, hq * 2 * hd, t, hq, out=out)
    ms = timed(f)
    flops = 4 * hq * hd * (t * (ctx - t) + t * t / 2)
    return ms, f"{flops / ms / 1e9:.0f} TFLOP/s of causal attention work"


def gdn_decode():
    nk, nv, b = 16, 48, 8
    conv_dim, value_dim = 2 * nk * 128 + nv * 128, nv * 128
    nq = conv_dim + value_dim
    qkvz = torch.randn(b, nq, device=dev).bfloat16()
    ldab = 96
    ab = torch.randn(b, ldab, device=dev).bfloat16()
    conv_w = torch.randn(conv_dim, 4, device=dev) * 0.2
    a_log, dt_bias, gamma = torch.zeros(nv, device=dev), torch.ones(nv, device=dev), torch.ones(128, device=dev)
    conv_state = torch.zeros(b, conv_dim, 3, device=dev)
    state = torch.zeros(b, nv, 128, 128, device=dev)                        # 25 MB per row, 201 MB in all
    slots = torch.arange(b, dtype=torch.int32, device=dev)
    xp = torch.empty(b, 2 * value_dim, dtype=torch.uint8, device=dev)
    xs = torch.empty(b, value_dim // 128, 2, device=dev)
    ms = timed(lambda: K.gdn_decode(qkvz, nq, ab, ldab, conv_w, a_log, dt_bias, gamma, conv_state, state, slots, xpack=xp, xs=xs,
                                    batch=b, t=1, nk=nk, nv=nv))
    return ms, f"{2 * state.numel() * 4 / ms / 1e9:.2f} TB/s of state (read + write)"


def gdn_scan():
    nk, nv, t = 16, 48, 2048
    conv_dim, value_dim = 2 * nk * 128 + nv * 128, nv * 128
    conv = torch.randn(t, conv_dim, device=dev).bfloat16() * 0.1
    z = torch.randn(t, value_dim, device=dev).bfloat16()
    ldab = 96
    ab = torch.randn(t, ldab, device=dev).bfloat16()
    a_log, dt_bias, gamma = torch.zeros(nv, device=dev), torch.ones(nv, device=dev), torch.ones(128, device=dev)
    state = torch.zeros(2, nv, 128, 128, device=dev)
    out = torch.empty(t, value_dim, dtype=torch.float16, device=dev)
    ms = timed(lambda: K.gdn_scan(conv, z, value_dim, ab, ldab, a_log, dt_bias, gamma, state, 0, out, t, nk, nv, False, 1e-6))
    return ms, f"{ms * 1e3 / t:.3f} us / token"


def dflash_attn():
    from owl_engine_b200.models import dflash2  # noqa: F401  (registers the kernel signatures)

    rows, hq, hkv, hd, cap, splits = 8, 32, 8, 128, 2048, 16
    q = torch.randn(rows, hq, hd, device=dev).bfloat16()
    ks, vs = torch.randn(rows, hkv, hd, device=dev).bfloat16(), torch.randn(rows, hkv, hd, device=dev).bfloat16()
    rk, rv = torch.randn(cap, hkv, hd, device=dev).bfloat16(), torch.randn(cap, hkv, hd, device=dev).bfloat16()
    po, pml = torch.empty(hkv * splits * 32 * hd, device=dev), torch.empty(hkv * splits * 32 * 2, device=dev)
    out = torch.empty(rows, hq * hd, dtype=torch.bfloat16, device=dev)
    plen = torch.tensor([cap], dtype=torch.int32, device=dev)
    ms = timed(lambda: K.call("owl_dflash_nc_attn", K.ptr(q), K.ptr(ks), K.ptr(vs), hkv * hd, K.ptr(rk), K.ptr(rv), K.ptr(plen),
                              K.ptr(po), K.ptr(pml), K.ptr(out), rows, hq, hkv, cap, splits, 1 / math.sqrt(hd), 0, K.stream()))
    return ms, f"{2 * rk.numel() * 2 / ms / 1e9:.3f} TB/s of ring KV"


if __name__ == "__main__":
    case = sys.argv[1]
    ms, note = globals()[case](*[int(a) for a in sys.argv[2:]])      # optional integer arguments of the case, in order
    print(f"{case}: {ms * 1e3:.1f} us per launch, {note}")
