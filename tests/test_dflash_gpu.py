"""DFlash2 block draft on a GPU: kernels and the whole propose / encode path against the fp32 reference in
``models/dflash2.py``; speculative decoding with the draft reproduces plain greedy decoding."""
import math

import pytest
import torch

from owl_engine_b200.models import dflash2 as D
from owl_engine_b200.ops import kernels as K
from owl_engine_b200.ops import quant as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    return ((a - b).norm() / b.norm().clamp_min(1e-6)).item()


def test_grouped_conv_matches_reference():
    g = torch.Generator().manual_seed(0)
    t, h, block = 8, 256, 8
    x = torch.randn(t, h, generator=g).bfloat16()
    delta = (torch.randn(t, 4 * (h // 16), generator=g) * 0.3).bfloat16()
    base = torch.randn(2, 2, h, generator=g).bfloat16()
    dx, dd, db = x.to(DEV), delta.to(DEV), base.to(DEV)
    for side in (0, 1):
        out = torch.empty(t, h, dtype=torch.bfloat16, device=DEV)
        K.call("owl_dflash_conv", K.ptr(dx), K.ptr(dd), K.ptr(db), side, block, h, t, K.ptr(out), 0, K.stream())
        torch.cuda.synchronize()
        want = D._conv_ref(x.float(), delta.float(), base.float(), side, block)
        assert rel_err(out.float().cpu(), want) < 0.01


@pytest.mark.parametrize("n_prefix", [0, 5, 64])
def test_nc_attention_matches_reference(n_prefix):
    g = torch.Generator().manual_seed(1)
    rows, hq, hkv, hd, cap = 8, 4, 2, 128, 64
    q = torch.randn(rows, hq, hd, generator=g).bfloat16()
    ks, vs = torch.randn(rows, hkv, hd, generator=g).bfloat16(), torch.randn(rows, hkv, hd, generator=g).bfloat16()
    rk, rv = torch.randn(cap, hkv, hd, generator=g).bfloat16(), torch.randn(cap, hkv, hd, generator=g).bfloat16()
    splits = 4
    part_o = torch.zeros(hkv * splits * 32 * hd, device=DEV)
    part_ml = torch.zeros(hkv * splits * 32 * 2, device=DEV)
    out = torch.zeros(rows, hq * hd, dtype=torch.bfloat16, device=DEV)
    plen = torch.tensor([n_prefix], dtype=torch.int32, device=DEV)
    dq, dk, dv, drk, drv = q.to(DEV), ks.to(DEV), vs.to(DEV), rk.to(DEV), rv.to(DEV)
    K.call("owl_dflash_nc_attn", K.ptr(dq), K.ptr(dk), K.ptr(dv), hkv * hd, K.ptr(drk), K.ptr(drv),
           K.ptr(plen), K.ptr(part_o), K.ptr(part_ml), K.ptr(out), rows, hq, hkv, cap, splits, 1 / math.sqrt(hd), 0, K.stream())
    torch.cuda.synchronize()
    kk = torch.cat([rk[:n_prefix], ks]).float().repeat_interleave(hq // hkv, 1)
    vv = torch.cat([rv[:n_prefix], vs]).float().repeat_interleave(hq // hkv, 1)
    att = (torch.einsum("qhd,khd->hqk", q.float(), kk) / math.sqrt(hd)).softmax(-1)
    want = torch.einsum("hqk,khd->qhd", att, vv).reshape(rows, -1)
    assert rel_err(out.float().cpu(), want) < 0.01


def test_selector_walk_matches_reference():
    g = torch.Generator().manual_seed(2)
    s, k, r, vocab = 7, 16, 64, 300
    cand = torch.stack([torch.randperm(vocab, generator=g)[:k] for _ in range(s)]).int()
    unary = torch.randn(s, k, generator=g)
    proj = torch.randn(s, r, generator=g).bfloat16()
    a_tab, b_tab = torch.randn(vocab, r, generator=g).bfloat16(), torch.randn(vocab, r, generator=g).bfloat16()
    anchor = 17
    out = torch.zeros(s, dtype=torch.int32, device=DEV)
    scores = torch.zeros(s * k * k, device=DEV)
    dc, du, dp, da, db = cand.to(DEV), unary.to(DEV), proj.to(DEV), a_tab.to(DEV), b_tab.to(DEV)
    danc = torch.tensor([anchor], dtype=torch.int32, device=DEV)
    K.call("owl_dflash_select", K.ptr(dc), K.ptr(du), K.ptr(dp), r, K.ptr(danc), K.ptr(da), K.ptr(db), s, k, r,
           K.ptr(out), K.ptr(scores), 0, K.stream())
    torch.cuda.synchronize()
    toks, idx = [], 0
    for e in range(s):
        pred = anchor if e == 0 else int(cand[e - 1, idx])
        sc = unary[e] + (a_tab[pred].float()[None] * proj[e].float()[None] * b_tab[cand[e].long()].float()).sum(-1)
        idx = int(sc.argmax())
        toks.append(int(cand[e, idx]))
    assert out.cpu().tolist() == toks


def _tiny():
    spec = D.tiny_spec()
    dense = D.random_dense(spec, seed=4)
    g = torch.Generator().manual_seed(5)
    embed = (torch.randn(spec.vocab, spec.hidden, generator=g) * 0.5).bfloat16()
    head = (torch.randn(spec.vocab, spec.hidden, generator=g) * 0.05).bfloat16()
    dw = D.weights_from_dense(spec, dense, DEV)
    draft = D.DFlash2(spec, dw, embed.to(DEV), Q.dense_skinny(head, DEV), DEV, max_encode=128)
    ref = D.RefDraft(spec, dense, embed, head)
    return spec, draft, ref, g


@pytest.mark.parametrize("n_ctx", [40, 90])
def test_encode_and_propose_match_reference(n_ctx):
    """n_ctx = 90 wraps the 64-slot ring; the second encode call takes the few-row path."""
    spec, draft, ref, g = _tiny()
    taps = (torch.randn(n_ctx, len(spec.taps) * spec.hidden, generator=g) * 0.7).bfloat16()
    cut = n_ctx - 7
    draft.encode(taps[:cut].to(DEV), 0)
    draft.encode(taps[cut:].to(DEV), cut)
    ref.encode(taps.float().view(n_ctx, len(spec.taps), spec.hidden), 0)
    anchor = 11
    got = draft.propose(anchor, n_ctx)
    torch.cuda.synchronize()
    want_hidden = ref.hidden(anchor, n_ctx)
    assert rel_err(draft.hidden.float().cpu(), want_hidden) < 0.05
    toks, _, _ = ref.select(draft.hidden.float().cpu(), anchor)
    assert got == toks
    draft.capture()
    assert draft.propose(anchor, n_ctx) == got


def test_speculative_decoding_with_the_block_draft_reproduces_greedy():
    from owl_engine_b200.engine import spec as S
    from owl_engine_b200.engine.core import Engine, EngineConfig

    cfg = EngineConfig(model="test-hybrid", snap_cut=True, n_pages=128, n_slots=4, n_snap_rows=2, max_seqs=4, max_seq=512, prefill_chunk=64)
    eng = Engine(cfg)
    eng.runner.uniform_rows = True      # the plain baseline uses the arithmetic a speculating engine switches to
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, eng.spec.vocab, (70,), generator=g).tolist()
    plain = eng.generate(prompt, 24)
    dspec = D.DraftSpec(hidden=eng.spec.hidden, n_layers=2, hq=4, hkv=2, hd=128, inter=512, vocab=eng.spec.vocab, rank=64,
                        window=64, mask_token_id=eng.spec.vocab - 1, taps=(1, 3))
    dw = D.weights_from_dense(dspec, D.random_dense(dspec, seed=1), eng.device)
    draft = D.DFlash2(dspec, dw, eng.weights.embed, eng.weights.lm_head, eng.device, max_encode=64)
    runner = S.SpecRunner(S.DFlash2Draft(draft, eng.runner), depth=7, degrade_below=-1.0)
    out = S.generate_spec(eng, prompt, 24, runner)
    assert out == plain
    assert runner.stats.rounds > 0 and runner.stats.drafted == 7 * runner.stats.rounds
