"""tcgen05 integer weight-streaming kernel (decode shapes) against the fp32 reference."""
import pytest
import torch

from owl_engine_b200.ops import kernels as K
from owl_engine_b200.ops import quant as Q
from owl_engine_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed=0):
    return torch.Generator(device="cpu").manual_seed(seed)


def setup(m, n, k, group, seed=3):
    w = torch.randn(n, k, generator=gen(seed)) * 0.05
    c = Q.quantize_w4(w, group)
    s = Q.pack_skinny(c, "block").to(DEV)
    x = (torch.randn(m, k, generator=gen(seed + 1))).to(torch.bfloat16)
    xt = torch.zeros(K.act_tile_bytes(k, group), dtype=torch.uint8, device=DEV)
    K.act_pack(x.to(DEV), xt, None, m, k, group | K.ACT_TILES)
    return c, s, x, xt, x.float() @ c.dequant().t()


@pytest.mark.parametrize("group", [128, 32])
def test_act_pack_tile_layout(group):
    m, k = 5, 512
    x = (torch.randn(m, k, generator=gen(2)) * 3).to(torch.bfloat16)
    xt = torch.zeros(K.act_tile_bytes(k, group), dtype=torch.uint8, device=DEV)
    K.act_pack(x.to(DEV), xt, None, m, k, group | K.ACT_TILES)
    want = Q.act_pack_tiles_ref(x.float(), group)
    bt = 2048 + 64 * (128 // group)
    got = xt.cpu().view(-1, bt)
    assert torch.equal(got[:, :2048], want.view(-1, bt)[:, :2048])
    torch.testing.assert_close(got[:, 2048:].contiguous().view(torch.float32), want.view(-1, bt)[:, 2048:].contiguous().view(torch.float32),
                               rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("group", [128, 32])
@pytest.mark.parametrize("shape", [(64, 256), (5120, 1024), (256, 2176), (1040, 640)])
def test_stream_tc_matches_reference(m, group, shape):
    n, k = shape
    c, s, x, xt, want = setup(m, n, k, group)
    ws = K.StreamTcWorkspace(DEV)
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    K.w4a16_stream_tc(s, xt, out, m, ws, epi=K.EPI_F32)
    torch.cuda.synchronize()
    assert K.stream_tc_status() == 0
    assert int(ws.counters.abs().sum()) == 0          # tickets are left at zero
    err = (out.cpu() - want).norm() / want.norm()
    assert err < 2e-3, err
    # the legacy streaming kernel accumulates the same integers: results agree to fp32 rounding
    ref = torch.zeros_like(out)
    xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
    xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
    K.act_pack(x.to(DEV), xp, xs, m, k, group)
    K.w4a16_skinny(Q.pack_skinny(c).to(DEV), xp, xs, ref, m, epi=K.EPI_F32)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4 * want.abs().max().item())


@pytest.mark.parametrize("ctas", [1, 3, 16, 296])
def test_stream_tc_split_and_epilogues(ctas):
    """Different stream-K splits (CTA counts) give the same numbers; every epilogue."""
    m, n, k, group = 2, 384, 2048, 128
    c, s, x, xt, want = setup(m, n, k, group, seed=5)
    ws = K.StreamTcWorkspace(DEV, ctas=ctas)
    res = torch.randn(m, n, generator=gen(7)).to(torch.bfloat16)
    out = res.to(DEV).clone()
    K.w4a16_stream_tc(s, xt, out, m, ws, residual=out, epi=K.EPI_RESIDUAL)
    torch.testing.assert_close(out.float().cpu(), want + res.float(), rtol=2e-2, atol=3e-2)
    out32 = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    K.w4a16_stream_tc(s, xt, out32, m, ws, epi=K.EPI_F32)
    torch.testing.assert_close(out32.cpu(), want, rtol=2e-3, atol=2e-3)
    sm = torch.zeros(m, n // 2, dtype=torch.bfloat16, device=DEV)
    K.w4a16_stream_tc(s, xt, sm, m, ws, epi=K.EPI_SILU_MUL)
    gate, up = Q.deinterleave_gate_up(want)
    torch.testing.assert_close(sm.float().cpu(), R.swiglu(gate, up), rtol=2e-2, atol=2e-2)
    ob = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    K.w4a16_stream_tc(s, xt, ob, m, ws, pdl=True)
    torch.testing.assert_close(ob.float().cpu(), want, rtol=2e-2, atol=2e-2)
    torch.cuda.synchronize()
    assert K.stream_tc_status() == 0 and int(ws.counters.abs().sum()) == 0


def test_stream_tc_is_deterministic():
    m, n, k = 4, 5120, 6144
    c, s, x, xt, want = setup(m, n, k, 128, seed=9)
    ws = K.StreamTcWorkspace(DEV)
    outs = []
    for _ in range(3):
        o = torch.zeros(m, n, dtype=torch.float32, device=DEV)
        K.w4a16_stream_tc(s, xt, o, m, ws, epi=K.EPI_F32)
        outs.append(o)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
