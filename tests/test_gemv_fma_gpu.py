"""One-token W4A16 projection on the half-precision FMA arm (``csrc/gemv_fma.cu``) against fp32 PyTorch: every prologue
(plain activations, fused RMSNorm), every epilogue (store, residual, silu * up), the dense side rows and both CTA shapes."""
import pytest
import torch

from owl_engine_b200.ops import kernels as K
from owl_engine_b200.ops import quant as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed=0):
    return torch.Generator(device="cpu").manual_seed(seed)


def _weight(n, k, seed=3):
    w = torch.randn(n, k, generator=gen(seed)) * 0.05
    c = Q.quantize_w4(w, 128)
    return c, Q.pack_skinny(c).to(DEV)


@pytest.mark.parametrize("shape", [(64, 256), (5120, 1024), (256, 2176), (1040, 5120), (4864, 6144)])
@pytest.mark.parametrize("vc", [2, 4])
def test_w4_fma_plain_store(shape, vc):
    n, k = shape
    c, s = _weight(n, k)
    x = (torch.randn(k, generator=gen(4)) * 3.0).to(torch.bfloat16)
    x[5] = 40.0                                     # an outlier sets the row scale; small values must survive it
    out = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    K.w4_fma(s, x.to(DEV), out, groups_per_cta=vc)
    want = c.dequant() @ x.float()
    err = (out.float().cpu() - want).norm() / want.norm()
    assert err < 5e-3, err
    assert K.fma_status() == 0


@pytest.mark.parametrize("vc", [2, 4])
def test_w4_fma_norm_prologue_and_side_rows(vc):
    n, k, rows = 2048, 5120, 96
    c, s = _weight(n, k, 5)
    h = (torch.randn(k, generator=gen(6)) * 2.0).to(torch.bfloat16)
    nw = (torch.randn(k, generator=gen(7)) * 0.1).to(torch.bfloat16)
    ab = (torch.randn(rows, k, generator=gen(8)) * 0.05).to(torch.bfloat16)
    out = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    ab_out = torch.zeros(rows, dtype=torch.bfloat16, device=DEV)
    xn_out = torch.zeros(k, dtype=torch.bfloat16, device=DEV)
    K.w4_fma(s, h.to(DEV), out, norm_w=nw.to(DEV), ab_w=ab.to(DEV), ab_out=ab_out, ab_rows=rows, x_out=xn_out, eps=1e-6,
             groups_per_cta=vc)
    hf = h.float()
    xn = (hf * torch.rsqrt((hf * hf).mean() + 1e-6) * (1.0 + nw.float())).to(torch.bfloat16)
    torch.testing.assert_close(xn_out.cpu().float(), xn.float(), rtol=1e-2, atol=1e-2)
    want = c.dequant() @ xn.float()
    err = (out.float().cpu() - want).norm() / want.norm()
    assert err < 5e-3, err
    want_ab = ab.float() @ xn.float()
    err_ab = (ab_out.float().cpu() - want_ab).norm() / want_ab.norm()
    assert err_ab < 5e-3, err_ab


def test_w4_fma_residual_and_silu_epilogues():
    n, k = 5120, 2176
    c, s = _weight(n, k, 9)
    x = torch.randn(k, generator=gen(10)).to(torch.bfloat16)
    res = torch.randn(n, generator=gen(11)).to(torch.bfloat16)
    hbuf = res.clone().to(DEV)
    K.w4_fma(s, x.to(DEV), hbuf, residual=hbuf, epi=K.EPI_RESIDUAL)       # in place: h += W x
    want = res.float() + c.dequant() @ x.float()
    torch.testing.assert_close(hbuf.float().cpu(), want, rtol=2e-2, atol=2e-2)
    # merged gate / up rows, interleaved in eights
    i = 1024
    gate, up = torch.randn(i, k, generator=gen(12)) * 0.05, torch.randn(i, k, generator=gen(13)) * 0.05
    cg = Q.quantize_w4(Q.interleave_gate_up(gate, up), 128)
    act = torch.zeros(i, dtype=torch.bfloat16, device=DEV)
    K.w4_fma(Q.pack_skinny(cg).to(DEV), x.to(DEV), act, epi=K.EPI_SILU_MUL)
    y = cg.dequant() @ x.float()
    g, u = Q.deinterleave_gate_up(y[None])
    want = (torch.nn.functional.silu(g) * u)[0]
    err = (act.float().cpu() - want).norm() / want.norm()
    assert err < 1e-2, err


def test_w4_fma_matches_integer_arm():
    """The two one-token arms read the same records: their outputs agree to bf16 rounding."""
    n, k = 4096, 5120
    c, s = _weight(n, k, 14)
    x = torch.randn(1, k, generator=gen(15)).to(torch.bfloat16).to(DEV)
    xp = torch.empty(1, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(1, k // 128, 2, dtype=torch.float32, device=DEV)
    K.act_pack(x, xp, xs, 1, k, 128)
    a = torch.zeros(1, n, dtype=torch.bfloat16, device=DEV)
    b = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    K.w4a16_skinny(s, xp, xs, a, 1)
    K.w4_fma(s, x[0], b)
    err = (a[0].float() - b.float()).norm() / a.float().norm()
    assert err < 5e-3, err
    assert K.fma_status() == 0


def test_w4_fma_rejects_bad_shapes():
    c, s = _weight(64, 256)
    x = torch.zeros(256, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception):
        K.w4_fma(s, x, out, epi=K.EPI_RESIDUAL)          # residual missing
    with pytest.raises(Exception):
        K.w4_fma(s, x, out, groups_per_cta=3)


@pytest.mark.parametrize("parts", [1, 4])
def test_w4_fma_push_pull_protocol_world_of_one(parts):
    """``parts`` > 1 also cuts every row tile of the row-parallel launch into k parts that land in slots of their own.
    The tensor-parallel pairing on one GPU: the row-parallel launch stores its partial sums, two per 8-byte word together
    with the number of the exchange, into slot 0 of a local word buffer; the column-parallel launch polls the words it
    needs for that number, adds the slot to the residual stream (stored into a second buffer), normalises in its prologue
    and advances the call site's sequence word. Two rounds, so the numbers advance."""
    import ctypes

    from owl_engine_b200.parallel import symm  # noqa: F401  (registers the signature)

    hdim, kdim, n2 = 5120, 2176, 1024
    cr, wr = _weight(hdim, kdim, 21)          # row-parallel: kdim -> hidden
    cc, wc = _weight(n2, hdim, 22)            # column-parallel: hidden -> n2
    words = torch.zeros(parts, hdim // 2, 2, dtype=torch.int32, device=DEV)
    count = torch.zeros(1, dtype=torch.int32, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    arr = lambda t: (ctypes.c_void_p * 8)(t.data_ptr())
    nw = (torch.randn(hdim, generator=gen(23)) * 0.1).to(torch.bfloat16).to(DEV)
    h = torch.randn(hdim, generator=gen(24)).to(torch.bfloat16)
    h_in, h_out = h.clone().to(DEV), torch.zeros(hdim, dtype=torch.bfloat16, device=DEV)
    want_h = h.float()
    for rnd in range(2):
        x = torch.randn(kdim, generator=gen(30 + rnd)).to(torch.bfloat16)
        out = torch.zeros(n2, dtype=torch.bfloat16, device=DEV)
        K.call("owl_w4_fma_tp", K.ptr(wr.records), K.ptr(x.to(DEV)), None, None, hdim, kdim, 0, 0.0, 1, 1, arr(words),
               K.ptr(seq), None, None, None, None, None, 0, 0, 1, parts, 1 << 20, 0, 0, K.stream())
        torch.cuda.synchronize()
        assert int(seq.item()) == rnd and bool((words[..., 1] == rnd + 1).all())      # the producer leaves the word alone
        K.call("owl_w4_fma_tp", K.ptr(wc.records), K.ptr(h_in), K.ptr(nw), K.ptr(out), n2, hdim, 0, 1e-6, 1, 0, None,
               K.ptr(seq), K.ptr(words), K.ptr(count), K.ptr(h_out), None, None, 0, 0, 1, parts, 1 << 20, 0, 0, K.stream())
        torch.cuda.synchronize()
        assert int(seq.item()) == rnd + 1 and int(count.item()) == 0
        part = cr.dequant() @ x.float()
        want_h = (want_h + part).to(torch.bfloat16).float()
        torch.testing.assert_close(h_out.float().cpu(), want_h, rtol=2e-2, atol=6e-2)
        hn = h_out.float().cpu()
        xn = (hn * torch.rsqrt((hn * hn).mean() + 1e-6) * (1.0 + nw.float().cpu())).to(torch.bfloat16).float()
        want = cc.dequant() @ xn
        err = (out.float().cpu() - want).norm() / want.norm()
        assert err < 5e-3, err
        h_in, h_out = h_out, h_in
        want_h = h_in.float().cpu()
    assert K.fma_status() == 0
    # words nobody writes: the bounded wait runs out, the kernel finishes and reports it (nothing hangs)
    seq.fill_(99)
    out = torch.zeros(n2, dtype=torch.bfloat16, device=DEV)
    K.call("owl_w4_fma_tp", K.ptr(wc.records), K.ptr(h_in), K.ptr(nw), K.ptr(out), n2, hdim, 0, 1e-6, 1, 0, None,
           K.ptr(seq), K.ptr(words), K.ptr(count), K.ptr(h_out), None, None, 0, 0, 1, parts, 2000, 0, 0, K.stream())
    torch.cuda.synchronize()
    assert K.fma_status() == 3        # OWL_ERR_WAIT_PEER
    assert K.fma_status() == 0        # read clears it
    assert int(seq.item()) == 100 and int(count.item()) == 0       # the call site's word still advances
