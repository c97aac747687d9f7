"""Numerics of every decode-path CUDA kernel against the fp32 PyTorch reference of the same op."""
import math

import pytest
import torch

from owl_engine_b200.ops import kernels as K
from owl_engine_b200.ops import quant as Q
from owl_engine_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed=0):
    return torch.Generator(device="cpu").manual_seed(seed)


def bf(x):
    return x.to(torch.bfloat16)


# ---------------------------------------------------------------------------------------
def test_pack_roundtrip_cpu_layout():
    c = Q.quantize_w4(torch.randn(64, 256, generator=gen(1)), 128)
    s = Q.pack_skinny(c)
    c2 = Q.unpack_skinny(s)
    assert torch.equal(c.q, c2.q) and torch.equal(c.zeros, c2.zeros) and torch.equal(c.scales, c2.scales)


@pytest.mark.parametrize("group", [128, 32])
def test_act_pack_matches_reference(group):
    m, k = 3, 512
    x = bf(torch.randn(m, k, generator=gen(2)) * 3)
    xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
    K.act_pack(x.to(DEV), xp, xs, m, k, group)
    want_p, want_s = Q.act_pack_ref(x.float(), group)
    assert torch.equal(xp.cpu(), want_p)
    torch.testing.assert_close(xs.cpu(), want_s, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("m", [1, 3, 8, 13, 32])
@pytest.mark.parametrize("group", [128, 32])
@pytest.mark.parametrize("shape", [(64, 256), (5120, 1024), (256, 2176)])
def test_w4a16_skinny(m, group, shape):
    n, k = shape
    w = torch.randn(n, k, generator=gen(3)) * 0.05
    c = Q.quantize_w4(w, group)
    s = Q.pack_skinny(c).to(DEV)
    x = bf(torch.randn(m, k, generator=gen(4)))
    xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
    K.act_pack(x.to(DEV), xp, xs, m, k, group)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    K.w4a16_skinny(s, xp, xs, out, m)
    want = x.float() @ c.dequant().t()
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    if m == 1:   # the tensor-core arm must agree with the dp4a arm (both accumulate exactly in int32)
        out2 = torch.zeros_like(out)
        K.w4a16_skinny(s, xp, xs, out2, m, force_mma=True)
        torch.testing.assert_close(out2.float(), out.float(), rtol=1e-2, atol=1e-3)
    # tighter: relative Frobenius error at bf16-output level
    err = (out.float().cpu() - want).norm() / want.norm()
    assert err < 5e-3, err


@pytest.mark.parametrize("m,group", [(1, 128), (1, 32), (5, 128), (20, 32)])
def test_w4a8_arm_skips_the_low_plane(m, group):
    """Activations packed with ACT_A8 are 8-bit (low plane zero, same container): the W4A8 arm, which skips the low-plane
    products, equals the full kernel on the same pack bit for bit, and both match the fp32 product of the dequantised weights
    with the 8-bit activations."""
    n, k = 512, 1024
    c = Q.quantize_w4(torch.randn(n, k, generator=gen(70)) * 0.05, group)
    s = Q.pack_skinny(c).to(DEV)
    x = bf(torch.randn(m, k, generator=gen(71)))
    xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
    K.act_pack(x.to(DEV), xp, xs, m, k, group | K.ACT_A8)
    planes = xp.view(m, k // 8, 16).cpu()
    assert int(planes[:, :, 4:8].max()) == 0 and int(planes[:, :, 12:16].max()) == 0        # low planes
    full = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    a8 = torch.zeros_like(full)
    K.w4a16_skinny(s, xp, xs, full, m)
    K.w4a16_skinny(s, xp, xs, a8, m, a8=True)
    assert torch.equal(full, a8)
    if m == 1:
        mm = torch.zeros_like(full)
        K.w4a16_skinny(s, xp, xs, mm, m, a8=True, force_mma=True)
        torch.testing.assert_close(mm.float(), a8.float(), rtol=1e-2, atol=1e-3)
    xg = x.float().view(m, k // group, group)
    sc = xg.abs().amax(-1, keepdim=True).clamp_min(1e-30) / 127.0
    x8 = (torch.round(xg / sc).clamp(-127, 127) * sc).view(m, k)
    want = x8 @ c.dequant().t()
    err = (a8.float().cpu() - want).norm() / want.norm()
    assert err < 5e-3, err
    exact = x.float() @ c.dequant().t()
    assert (a8.float().cpu() - exact).norm() / exact.norm() < 2e-2       # 8-bit activations: ~1 % of the product's norm


@pytest.mark.parametrize("ks", [1, 2, 4, 8])
def test_w4a16_skinny_splitk_and_epilogues(ks):
    m, n, k, group = 2, 128, 2048, 128
    w = torch.randn(n, k, generator=gen(5)) * 0.05
    c = Q.quantize_w4(w, group)
    s = Q.pack_skinny(c).to(DEV)
    x = bf(torch.randn(m, k, generator=gen(6)))
    xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
    K.act_pack(x.to(DEV), xp, xs, m, k, group)
    want = x.float() @ c.dequant().t()
    res = bf(torch.randn(m, n, generator=gen(7)))
    out = res.to(DEV).clone()
    K.w4a16_skinny(s, xp, xs, out, m, residual=out, epi=K.EPI_RESIDUAL, tiles_per_cta=ks)
    torch.testing.assert_close(out.float().cpu(), want + res.float(), rtol=2e-2, atol=3e-2)
    out32 = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    K.w4a16_skinny(s, xp, xs, out32, m, epi=K.EPI_F32, tiles_per_cta=ks)
    torch.testing.assert_close(out32.cpu(), want, rtol=2e-3, atol=2e-3)
    # silu-mul epilogue: rows interleaved (8 gate, 8 up)
    sm = torch.zeros(m, n // 2, dtype=torch.bfloat16, device=DEV)
    K.w4a16_skinny(s, xp, xs, sm, m, epi=K.EPI_SILU_MUL, tiles_per_cta=ks)
    gate, up = Q.deinterleave_gate_up(want)
    torch.testing.assert_close(sm.float().cpu(), R.swiglu(gate, up), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("m,gout", [(1, 128), (5, 32), (20, 128)])
def test_w4a16_skinny_fused_silu_pack(m, gout):
    n, k, group = 1024, 512, 128
    c = Q.quantize_w4(torch.randn(n, k, generator=gen(50)) * 0.05, group)
    s = Q.pack_skinny(c).to(DEV)
    x = bf(torch.randn(m, k, generator=gen(51)))
    xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
    K.act_pack(x.to(DEV), xp, xs, m, k, group)
    inter = n // 2
    op = torch.zeros(m, 2 * inter, dtype=torch.uint8, device=DEV)
    oxs = torch.zeros(m, inter // gout, 2, dtype=torch.float32, device=DEV)
    K.w4a16_skinny(s, xp, xs, None, m, epi=K.EPI_SILU_PACK, ldo=inter, out_pack=op, out_xs=oxs, gout=gout)
    sm = torch.zeros(m, inter, dtype=torch.bfloat16, device=DEV)
    K.w4a16_skinny(s, xp, xs, sm, m, epi=K.EPI_SILU_MUL)
    wp, ws = Q.act_pack_ref(sm.float().cpu(), gout)
    assert torch.equal(op.cpu(), wp)
    torch.testing.assert_close(oxs.cpu(), ws, rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("m,group", [(1, 128), (3, 32), (8, 128), (20, 128)])
def test_w4a16_skinny_fused_residual_norm(m, group):
    """Projection + residual + RMSNorm + ActPack in one launch against the two-launch path (same rows, same packing)."""
    n, k = 5120, 1024
    c = Q.quantize_w4(torch.randn(n, k, generator=gen(60)) * 0.05, group)
    s = Q.pack_skinny(c).to(DEV)
    x = bf(torch.randn(m, k, generator=gen(61)))
    xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
    K.act_pack(x.to(DEV), xp, xs, m, k, group)
    res = bf(torch.randn(m, n, generator=gen(62))).to(DEV)
    nw = bf(torch.randn(n, generator=gen(63)) * 0.1).to(DEV)
    count = torch.zeros(1, dtype=torch.int32, device=DEV)
    for it in range(2):          # the second call checks that the counter went back to zero
        h2 = res.clone()
        K.w4a16_skinny(s, xp, xs, h2, m, residual=h2, epi=K.EPI_RESIDUAL)
        xn2 = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
        p2 = torch.zeros(m, 2 * n, dtype=torch.uint8, device=DEV)
        s2 = torch.zeros(m, n // 128, 2, dtype=torch.float32, device=DEV)
        K.rmsnorm_pack(h2, nw, normed=xn2, xpack=p2, xs=s2, m=m, k=n, group=128)
        h1 = res.clone()
        xn1, p1, s1 = torch.zeros_like(xn2), torch.zeros_like(p2), torch.zeros_like(s2)
        K.w4a16_skinny_norm(s, xp, xs, h1, nw, count, m, normed=xn1, norm_pack=p1, norm_xs=s1, group=128)
        torch.cuda.synchronize()
        assert torch.equal(h1, h2)
        assert int(count.item()) == 0
        torch.testing.assert_close(xn1.float(), xn2.float(), rtol=1e-2, atol=1e-2)
        want = R.rmsnorm(h2.float().cpu(), nw.float().cpu(), 1e-6)
        torch.testing.assert_close(xn1.float().cpu(), want, rtol=2e-2, atol=2e-2)
        wp, ws = Q.act_pack_ref(xn1.float().cpu(), 128)
        assert torch.equal(p1.cpu(), wp)
        torch.testing.assert_close(s1.cpu(), ws, rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("m", [1, 5, 16])
def test_bf16_and_w8_skinny(m):
    n, k = 272, 1024
    w = bf(torch.randn(n, k, generator=gen(8)) * 0.05)
    x = bf(torch.randn(m, k, generator=gen(9)))
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    assert torch.equal(Q.unpack_dense_bf16(Q.pack_dense_bf16(w), n, k), w)
    K.dense_skinny(Q.dense_skinny(w, DEV), x.to(DEV), out, m)
    want = x.float() @ w.float().t()
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2)
    q8, s8 = Q.quantize_w8_rows(w.float())
    out8 = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    K.dense_skinny(Q.dense_skinny(w.float(), DEV, int8=True), x.to(DEV), out8, m)
    want8 = x.float() @ (q8.float() * s8[:, None]).t()
    torch.testing.assert_close(out8.float().cpu(), want8, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("with_delta", [False, True])
def test_rmsnorm_pack(with_delta):
    m, k, group = 4, 5120, 128
    h = bf(torch.randn(m, k, generator=gen(10)))
    d = bf(torch.randn(m, k, generator=gen(11))) if with_delta else None
    w = bf(torch.randn(k, generator=gen(12)) * 0.1)
    out_h = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    normed = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
    K.rmsnorm_pack(h.to(DEV), w.to(DEV), delta=d.to(DEV) if with_delta else None, out_h=out_h if with_delta else None,
                   normed=normed, xpack=xp, xs=xs, m=m, k=k, group=group)
    hh = bf(h.float() + d.float()) if with_delta else h
    if with_delta:
        assert torch.equal(out_h.cpu(), hh)
    want = R.rmsnorm(hh, w)
    torch.testing.assert_close(normed.float().cpu(), want, rtol=1e-2, atol=1e-2)
    wp, ws = Q.act_pack_ref(normed.float().cpu(), group)
    assert torch.equal(xp.cpu(), wp)
    torch.testing.assert_close(xs.cpu(), ws, rtol=1e-5, atol=1e-3)


def test_silu_mul_embed_argmax():
    m, inter = 3, 1024
    gu = bf(torch.randn(m, 2 * inter, generator=gen(13)))
    out = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    K.silu_mul(gu.to(DEV), m, inter, out=out)
    gate, up = Q.deinterleave_gate_up(gu.float())
    torch.testing.assert_close(out.float().cpu(), R.swiglu(gate, up), rtol=1e-2, atol=1e-2)
    table = bf(torch.randn(100, 64, generator=gen(14)))
    ids = torch.tensor([5, 99, 0], dtype=torch.int32)
    e = torch.empty(3, 64, dtype=torch.bfloat16, device=DEV)
    K.embed(ids.to(DEV), table.to(DEV), e, 3)
    assert torch.equal(e.cpu(), table[ids.long()])
    v = 151936
    logits = bf(torch.randn(2, v, generator=gen(15)))
    sv = torch.empty(2 * 64, dtype=torch.float32, device=DEV)
    si = torch.empty(2 * 64, dtype=torch.int32, device=DEV)
    oi = torch.empty(2, dtype=torch.int32, device=DEV)
    K.argmax(logits.to(DEV), 2, v, v, sv, si, 64, oi)
    assert oi.cpu().tolist() == logits.float().argmax(-1).tolist()


# ---------------------------------------------------------------------------------------
def _gdn_setup(nk, nv, t, batch, seed):
    g = gen(seed)
    kd = vd = 128
    kdim, vdim = nk * kd, nv * vd
    conv_dim = 2 * kdim + vdim
    rows = batch * t
    qkvz = bf(torch.randn(rows, conv_dim + vdim, generator=g))
    ab = bf(torch.randn(rows, 2 * nv, generator=g))
    conv_w = torch.randn(conv_dim, 4, generator=g) * 0.3
    a_log = torch.log(torch.empty(nv).uniform_(1, 8, generator=g))
    dt_bias = torch.ones(nv)
    gamma = 1 + 0.1 * torch.randn(vd, generator=g)
    slots = 3
    conv_state = torch.randn(slots, conv_dim, 3, generator=g)
    state = torch.randn(slots, nv, kd, vd, generator=g) * 0.1
    return dict(qkvz=qkvz, ab=ab, conv_w=conv_w, a_log=a_log, dt_bias=dt_bias, gamma=gamma, conv_state=conv_state,
                state=state, nk=nk, nv=nv, kdim=kdim, vdim=vdim, conv_dim=conv_dim)


def _gdn_ref(s, rows_sel, slot, t):
    nk, nv, kdim, vdim = s["nk"], s["nv"], s["kdim"], s["vdim"]
    x = s["qkvz"][rows_sel].float()
    y, new_hist = R.causal_conv1d(x[:, :s["conv_dim"]], s["conv_w"], s["conv_state"][slot])
    q = R.l2norm(y[:, :kdim].view(t, nk, 128)).repeat_interleave(nv // nk, 1)
    k = R.l2norm(y[:, kdim:2 * kdim].view(t, nk, 128)).repeat_interleave(nv // nk, 1)
    v = y[:, 2 * kdim:].view(t, nv, 128)
    ab = s["ab"][rows_sel].float()
    g, beta = R.gdn_gating(ab[:, :nv], ab[:, nv:], s["a_log"], s["dt_bias"])
    o, st = R.gdn_recurrent(q, k, v, g, beta, s["state"][slot])
    z = x[:, s["conv_dim"]:].view(t, nv, 128)
    return R.gated_rmsnorm(o, z, s["gamma"]).reshape(t, vdim), st, new_hist


@pytest.mark.parametrize("nk,nv", [(2, 6), (2, 2)])
@pytest.mark.parametrize("t", [1, 4])
def test_gdn_decode(nk, nv, t):
    batch = 2
    s = _gdn_setup(nk, nv, t, batch, 20)
    d = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in s.items()}
    slots = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
    out = torch.zeros(batch * t, s["vdim"], dtype=torch.bfloat16, device=DEV)
    xp = torch.zeros(batch * t, 2 * s["vdim"], dtype=torch.uint8, device=DEV)
    xs = torch.zeros(batch * t, s["vdim"] // 128, 2, dtype=torch.float32, device=DEV)
    K.gdn_decode(d["qkvz"], d["qkvz"].shape[1], d["ab"], 2 * nv, d["conv_w"], d["a_log"], d["dt_bias"], d["gamma"],
                 d["conv_state"], d["state"], slots, out=out, xpack=xp, xs=xs, batch=batch, t=t, nk=nk, nv=nv)
    torch.cuda.synchronize()
    for b, slot in enumerate([2, 0]):
        rows = slice(b * t, (b + 1) * t)
        want, st, hist = _gdn_ref(s, rows, slot, t)
        torch.testing.assert_close(out[rows].float().cpu(), want, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(d["state"][slot].cpu(), st, rtol=1e-3, atol=1e-3)
        torch.testing.assert_close(d["conv_state"][slot].cpu(), hist, rtol=0, atol=0)
    # untouched slot stays untouched
    assert torch.equal(d["state"][1].cpu(), s["state"][1])
    wp, ws = Q.act_pack_ref(out.float().cpu(), 128)
    assert torch.equal(xp.cpu(), wp)
    torch.testing.assert_close(xs.cpu(), ws, rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("t,use_state,split", [(70, True, None), (33, False, None), (5, False, None), (2, True, None),
                                               (64, False, "chunked"), (70, True, "chunked"), (200, True, None),
                                               (333, False, None)])
def test_gdn_prefill_conv_and_scan(t, use_state, split):
    """t >= 128 (or split="chunked") runs the chunk-64 WY scan on tensor cores, 32 <= t < 128 the column-split serial scan."""
    nk, nv = 2, 6
    s = _gdn_setup(nk, nv, t, 1, 21)
    if not use_state:
        s["conv_state"].zero_()
        s["state"].zero_()
    d = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in s.items()}
    slot = 1
    conv_out = torch.empty(t, s["conv_dim"], dtype=torch.bfloat16, device=DEV)
    ld = d["qkvz"].shape[1]
    K.gdn_conv_fwd(d["qkvz"], ld, d["conv_w"], d["conv_state"], slot, conv_out, t, nk, nv, use_state)
    out = torch.empty(t, s["vdim"], dtype=torch.bfloat16, device=DEV)
    z = d["qkvz"][:, s["conv_dim"]:]
    K.gdn_scan(conv_out, z, ld, d["ab"], 2 * nv, d["a_log"], d["dt_bias"], d["gamma"], d["state"], slot, out, t, nk, nv,
               use_state, split=split)
    torch.cuda.synchronize()
    want, st, hist = _gdn_ref(s, slice(0, t), slot, t)
    if split == "chunked" or t >= K.GDN_CHUNKED_FROM:
        # bf16 operands of the chunk products: judged on the norm, with a loose bound on any single element
        got = out.float().cpu()
        assert (got - want).norm() / want.norm() < 1e-2
        torch.testing.assert_close(got, want, rtol=1e-1, atol=1e-1)
        assert (d["state"][slot].cpu() - st).norm() / st.norm() < 1e-2
    else:
        torch.testing.assert_close(out.float().cpu(), want, rtol=3e-2, atol=3e-2)
        torch.testing.assert_close(d["state"][slot].cpu(), st, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(d["conv_state"][slot].cpu(), hist, rtol=0, atol=0)


# ---------------------------------------------------------------------------------------
def _attn_case(batch, t, ctx_lens, hq=6, hkv=1, hd=256, seed=30):
    g = gen(seed)
    n_pages = 64
    max_blocks = 16
    k_pool = torch.zeros(n_pages, 16, hkv, hd, dtype=torch.uint8)
    v_pool = torch.zeros(n_pages, 16, hkv, hd, dtype=torch.uint8)
    perm = torch.randperm(n_pages, generator=g)
    bt = torch.zeros(batch, max_blocks, dtype=torch.int32)
    ks, vs = [], []
    nxt = 0
    for b in range(batch):
        n = ctx_lens[b]
        kk = torch.randn(n, hkv, hd, generator=g)
        vv = torch.randn(n, hkv, hd, generator=g)
        k8, v8 = kk.clamp(-448, 448).to(torch.float8_e4m3fn), vv.clamp(-448, 448).to(torch.float8_e4m3fn)
        ks.append(k8.float())
        vs.append(v8.float())
        for pg in range((n + 15) // 16):
            page = int(perm[nxt]); nxt += 1
            bt[b, pg] = page
            lo, hi = pg * 16, min(n, pg * 16 + 16)
            k_pool[page, :hi - lo] = k8[lo:hi].view(torch.uint8)
            v_pool[page, :hi - lo] = v8[lo:hi].view(torch.uint8)
    q = bf(torch.randn(batch * t, hq, hd, generator=g))
    return q, k_pool, v_pool, bt, ks, vs, max_blocks


@pytest.mark.parametrize("t,ctx_lens,splits", [(1, [37, 200], 3), (1, [16, 1], 1), (4, [50, 130], 2), (8, [97, 8], 4),
                                               (2, [33, 64], 5)])
def test_paged_attention(t, ctx_lens, splits):
    hq, hkv, hd = 6, 1, 256
    batch = len(ctx_lens)
    q, k_pool, v_pool, bt, ks, vs, max_blocks = _attn_case(batch, t, ctx_lens)
    rows = batch * t
    part_o = torch.zeros(rows * hq * splits * hd, dtype=torch.float32, device=DEV)
    part_ml = torch.zeros(rows * hq * splits * 2, dtype=torch.float32, device=DEV)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    K.paged_attn(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), bt.to(DEV), None, ctx, part_o, part_ml, batch, t, hq, hkv, hd,
                 max_blocks, splits, 1.0 / math.sqrt(hd))
    out = torch.empty(rows, hq * hd, dtype=torch.bfloat16, device=DEV)
    K.attn_reduce(part_o, part_ml, splits, None, 0, rows, hq, out=out)
    torch.cuda.synchronize()
    for b in range(batch):
        want = R.gqa_attention(q[b * t:(b + 1) * t].float(), ks[b], vs[b], ctx_lens[b] - t)
        got = out[b * t:(b + 1) * t].float().cpu().view(t, hq, hd)
        torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("t,ctx_lens,splits", [(1, [37, 200], 3), (4, [50, 130], 2), (8, [97, 8], 1)])
def test_paged_attention_16bit_pool(t, ctx_lens, splits):
    """The same attention over a 16-bit pool (fp16 words): K / V are used as stored, so the fp32 reference on the
    fp16-rounded values is matched more tightly than with the 8-bit pools."""
    hq, hkv, hd = 6, 1, 256
    batch = len(ctx_lens)
    q, k8, v8, bt, ks, vs, max_blocks = _attn_case(batch, t, ctx_lens)
    k_pool = k8.view(torch.float8_e4m3fn).float().half()        # the case's values (exact in fp16), as a 16-bit pool
    v_pool = v8.view(torch.float8_e4m3fn).float().half()
    rows = batch * t
    part_o = torch.zeros(rows * hq * splits * hd, dtype=torch.float32, device=DEV)
    part_ml = torch.zeros(rows * hq * splits * 2, dtype=torch.float32, device=DEV)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    K.paged_attn(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), bt.to(DEV), None, ctx, part_o, part_ml, batch, t, hq, hkv, hd,
                 max_blocks, splits, 1.0 / math.sqrt(hd))
    out = torch.empty(rows, hq * hd, dtype=torch.bfloat16, device=DEV)
    K.attn_reduce(part_o, part_ml, splits, None, 0, rows, hq, out=out)
    o8 = torch.empty_like(out)
    K.paged_attn(q.to(DEV), k8.to(DEV), v8.to(DEV), bt.to(DEV), None, ctx, part_o, part_ml, batch, t, hq, hkv, hd,
                 max_blocks, splits, 1.0 / math.sqrt(hd))
    K.attn_reduce(part_o, part_ml, splits, None, 0, rows, hq, out=o8)
    torch.cuda.synchronize()
    assert torch.equal(out, o8)          # same values in both pools: the two formats feed the MMA identical fp16 operands
    for b in range(batch):
        want = R.gqa_attention(q[b * t:(b + 1) * t].float(), ks[b], vs[b], ctx_lens[b] - t)
        got = out[b * t:(b + 1) * t].float().cpu().view(t, hq, hd)
        torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)


def test_qknorm_rope_insert():
    rows, hq, hkv, hd, rot = 5, 6, 2, 256, 64
    g = gen(40)
    qraw = bf(torch.randn(rows, hq * 2 * hd, generator=g))
    kraw = bf(torch.randn(rows, hkv * hd, generator=g))
    vraw = bf(torch.randn(rows, hkv * hd, generator=g))
    qw, kw = bf(torch.randn(hd, generator=g) * 0.1), bf(torch.randn(hd, generator=g) * 0.1)
    pos = torch.tensor([0, 1, 2, 1000, 200000], dtype=torch.int32)
    pos3 = torch.stack([pos, pos + 3, pos + 7]).contiguous()
    inv = R.rope_inv_freq(rot, 1e7)
    section = [0 if j % 3 == 0 or (j % 3 == 2 and j >= 30) else j % 3 for j in range(32)]
    kv_slot = torch.tensor([17, 0, 35, -1, 63], dtype=torch.int32)
    k_pool = torch.zeros(4, 16, hkv, hd, dtype=torch.uint8, device=DEV)
    v_pool = torch.zeros(4, 16, hkv, hd, dtype=torch.uint8, device=DEV)
    q_out = torch.empty(rows, hq, hd, dtype=torch.bfloat16, device=DEV)
    K.qknorm_rope_insert(qraw.to(DEV), hq * 2 * hd, kraw.to(DEV), hkv * hd, vraw.to(DEV), hkv * hd, qw.to(DEV),
                         kw.to(DEV), pos3.to(DEV), inv.to(DEV), torch.tensor(section, dtype=torch.uint8, device=DEV),
                         kv_slot.to(DEV), q_out, k_pool, v_pool, rows, hq, hkv, hd, rot)
    torch.cuda.synchronize()
    cos, sin = R.rope_cos_sin(pos3, inv, section)
    q = qraw.float().view(rows, hq, 2 * hd)[..., :hd]
    want_q = R.apply_rope(R.rmsnorm(q, qw), cos, sin)
    torch.testing.assert_close(q_out.float().cpu(), want_q, rtol=2e-2, atol=2e-2)
    want_k = R.apply_rope(R.rmsnorm(kraw.float().view(rows, hkv, hd), kw), cos, sin)
    kp = k_pool.view(-1, hkv, hd).cpu().view(torch.float8_e4m3fn).float()
    vp = v_pool.view(-1, hkv, hd).cpu().view(torch.float8_e4m3fn).float()
    for r in range(rows):
        s = int(kv_slot[r])
        if s < 0:
            continue
        torch.testing.assert_close(kp[s], want_k[r], rtol=0.07, atol=0.02)
        torch.testing.assert_close(vp[s], vraw[r].float().view(hkv, hd), rtol=0.07, atol=0.02)
    assert torch.count_nonzero(kp[1]) == 0
    # 16-bit pool: fp16 words holding the bf16-rounded values
    k16 = torch.zeros(4, 16, hkv, hd, dtype=torch.float16, device=DEV)
    v16 = torch.zeros_like(k16)
    K.qknorm_rope_insert(qraw.to(DEV), hq * 2 * hd, kraw.to(DEV), hkv * hd, vraw.to(DEV), hkv * hd, qw.to(DEV),
                         kw.to(DEV), pos3.to(DEV), inv.to(DEV), torch.tensor(section, dtype=torch.uint8, device=DEV),
                         kv_slot.to(DEV), q_out, k16, v16, rows, hq, hkv, hd, rot)
    torch.cuda.synchronize()
    kp, vp = k16.view(-1, hkv, hd).float().cpu(), v16.view(-1, hkv, hd).float().cpu()
    for r in range(rows):
        s = int(kv_slot[r])
        if s < 0:
            continue
        torch.testing.assert_close(kp[s], want_k[r], rtol=1e-2, atol=1e-2)
        assert torch.equal(vp[s], vraw[r].float().view(hkv, hd))                 # bf16 inputs are stored exactly
    assert torch.count_nonzero(kp[1]) == 0 and torch.equal(kp, kp.bfloat16().float())


def test_zz_skinny_status_clean_after_all():
    torch.cuda.synchronize()
    assert K.skinny_status() == 0


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,v,k", [(1, 151936, 32), (3, 5000, 16), (2, 40, 32)])
def test_topk_with_repetition_penalty(m, v, k):
    logits = bf(torch.randn(m, v, generator=gen(21)) * 4)
    hist = torch.stack([torch.randperm(v, generator=gen(22 + r))[:12] for r in range(m)]).to(torch.int32)
    hlen = torch.tensor([12, 5, 0][:m], dtype=torch.int32)
    pen = 1.3
    tk = K.TopK(DEV, max_rows=4, k=k)
    val, idx = tk(logits.to(DEV), m, v, hist=hist.to(DEV), hist_len=hlen.to(DEV), penalty=pen)
    ref = logits.float().clone()
    for r in range(m):
        for t in hist[r, :int(hlen[r])].tolist():
            ref[r, t] = ref[r, t] / pen if ref[r, t] > 0 else ref[r, t] * pen
    kk = min(k, v)
    want_v, want_i = torch.topk(ref, kk, dim=-1)
    torch.testing.assert_close(val.cpu()[:, :kk], want_v, rtol=0, atol=0)
    # equal values may come in any index order in torch; ours breaks ties by the lowest index
    assert torch.equal(torch.gather(ref, 1, idx.cpu()[:, :kk].long()), want_v)
    if kk < k:
        assert (idx.cpu()[:, kk:] == -1).all()
    mv, mi = K.topk_merge(torch.cat([val - 1000, val], 1).contiguous(), torch.cat([idx, idx], 1).contiguous(), kk)
    torch.testing.assert_close(mv.cpu(), want_v[:, :kk], rtol=0, atol=0)


def test_boot_selfcheck_passes():
    from owl_engine_b200.ops import selfcheck

    res = selfcheck.run_all(DEV)
    assert all(ok for _, ok, _ in res), res
