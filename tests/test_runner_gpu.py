"""GPU runner vs the fp32 CPU reference model (prefill chunks, eager decode, graph decode)."""
import pytest
import torch

from owl_engine_b200.models import hybrid as H
from owl_engine_b200.ops import kernels as K
from owl_engine_b200.models.reference import RefModel, init_weights
from owl_engine_b200.models.spec import test_hybrid as make_spec

pytestmark = pytest.mark.gpu
DEV = "cuda"


def build(arm="baseline", n_layers=4, group=128, layout="slice", kv_dtype="fp8", quant="w4a16"):
    spec = make_spec(n_layers=n_layers)
    dense = init_weights(spec, seed=3, std=0.05)
    hw, equiv = H.weights_from_dense(spec, dense, DEV, group=group, layout=layout, quant=quant)
    pool = H.StatePool(spec, DEV, n_pages=32, n_slots=4, kv_dtype=kv_dtype)
    run = H.HybridRunner(spec, hw, pool, max_seqs=4, max_blocks=16, prefill_gemm=arm, pdl=True)
    ref = RefModel(spec, equiv, kv_fp8=kv_dtype == "fp8")
    return spec, run, ref


# Teacher-forced decode against the fp32 model: the error grows with the step (recurrent state, KV rounding). The fp16 FMA
# projection adds 1.4e-3 of its own per projection (measured against a float64 product: 2.1e-3, where rounding the exact
# result to bf16 alone gives 1.6e-3), so the bound is a little wider than the prefill bound of 0.05.
DECODE_TOL = 0.06


def rel_err(a, b):
    return ((a - b).norm() / b.norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("arm,layout", [("baseline", "slice"), ("tc", "slice"), ("tc", "block")])
def test_prefill_then_decode_matches_reference(arm, layout):
    """layout "block": decode GEMVs run on the tcgen05 streaming kernel, producers write ActPack tiles."""
    spec, run, ref = build(arm, layout=layout)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab, (37,), generator=g)
    seq_row, slot = 1, 2
    run.block_table[seq_row, :8] = torch.tensor([5, 9, 2, 30, 11, 12, 13, 14], dtype=torch.int32, device=DEV)
    ids = prompt.to(torch.int32).to(DEV)
    # two chunks: 21 + 16 tokens
    run.prefill_chunk_forward(ids[:21], 0, seq_row, slot, want_logits=False)
    tok = run.prefill_chunk_forward(ids[21:], 21, seq_row, slot)
    torch.cuda.synchronize()
    st = ref.new_state()
    hr = ref.forward(prompt, st)
    want_logits = ref.logits(hr[-1:])
    got_logits = run.logits[:1].float().cpu()
    assert rel_err(got_logits, want_logits) < 0.05
    assert rel_err(run.h[:1].float().cpu(), hr[-1:]) < 0.05
    # decode 6 steps, teacher-forced with the reference's greedy tokens
    lay = H.StepLayout(1, 1)
    v = run.views(lay)
    nxt = int(want_logits.argmax(-1))
    for step in range(6):
        pos = 37 + step
        v["ids"][0] = nxt
        v["pos3"][:] = pos
        v["kv_slot"][0] = int(run.block_table[seq_row, pos // 16]) * 16 + pos % 16
        v["ctx"][0] = pos + 1
        v["gslot"][0] = slot
        v["bt_row"][0] = seq_row
        if step < 3:
            run.step_forward(lay, ctx_hint=64)
        else:
            run.capture(1, 1, ctx_hint=64).replay()
        torch.cuda.synchronize()
        hr = ref.forward(torch.tensor([nxt]), st)
        want = ref.logits(hr)
        assert rel_err(run.logits[:1].float().cpu(), want) < DECODE_TOL, step
        nxt = int(want.argmax(-1))


@pytest.mark.parametrize("layout", ["slice", "block"])
def test_batched_decode_and_self_feeding_graph(layout):
    spec, run, ref = build(layout=layout)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g) for n in (9, 20)]
    rows, slots = [0, 2], [1, 3]
    pages = [[3, 4, 5, 6], [10, 11, 12, 13]]
    states, first = [], []
    for p, r, s, pg in zip(prompts, rows, slots, pages):
        run.block_table[r, :4] = torch.tensor(pg, dtype=torch.int32, device=DEV)
        run.pool.reset_slot(s)
        run.prefill_chunk_forward(p.to(torch.int32).to(DEV), 0, r, s)
        torch.cuda.synchronize()
        st = ref.new_state()
        want = ref.logits(ref.forward(p, st)[-1:])
        states.append(st)
        first.append(int(want.argmax(-1)))
    lay = H.StepLayout(2, 1)
    v = run.views(lay)
    for b in range(2):
        pos = prompts[b].shape[0]
        v["ids"][b] = first[b]
        v["pos3"][b::2] = pos
        v["kv_slot"][b] = pages[b][pos // 16] * 16 + pos % 16
        v["ctx"][b] = pos + 1
        v["gslot"][b] = slots[b]
        v["bt_row"][b] = rows[b]
    graph = run.capture(2, 1, ctx_hint=64, advance=True)
    toks = [list(first), ]
    ref_next = list(first)
    for step in range(5):
        graph.replay()
        torch.cuda.synchronize()
        got = run.out_tok[:2].cpu().tolist()
        for b in range(2):
            hr = states[b].__class__ and ref.forward(torch.tensor([ref_next[b]]), states[b])
            want = ref.logits(hr)
            assert rel_err(run.logits[b:b + 1].float().cpu(), want) < 0.05, (step, b)
            # the graph feeds its own argmax forward: keep the reference on the same tokens
            ref_next[b] = got[b]
        assert v["ids"].cpu().tolist() == got


def test_sequence_parallel_prefill_protocol_on_one_gpu():
    """The tensor-parallel prefill path (GEMM + reduce-scatter epilogue, owner-side sum + norm + all-gather, GEMM that
    waits per row tile) with a world of one on plain device memory: same kernels, flags and sequence numbers."""
    from owl_engine_b200.ops import gemm_tc
    from owl_engine_b200.parallel.symm import PrefillPipe, SymmetricWorkspace

    spec, run, ref = build("tc")
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, spec.vocab, (250,), generator=g)
    ids = prompt.to(torch.int32).to(DEV)
    run.block_table[1, :16] = torch.arange(16, dtype=torch.int32, device=DEV)
    run.prefill_chunk_forward(ids, 0, 1, 1)
    torch.cuda.synchronize()
    h_plain, l_plain = run.h[:1].float().cpu(), run.logits[:1].float().cpu()
    run.pf_pipe = PrefillPipe.local(spec.hidden, 256, DEV)
    run.SP_FROM = 128
    outs = []
    for slot in (2, 3):                         # twice: sequence numbers advance, flags are reused
        run.prefill_chunk_forward(ids, 0, 1, slot)
        torch.cuda.synchronize()
        outs.append((run.h[:1].float().cpu(), run.logits[:1].float().cpu()))
    assert gemm_tc.gemm_status() == 0 and SymmetricWorkspace.status() == 0
    assert rel_err(outs[0][0], h_plain) < 0.02 and rel_err(outs[0][1], l_plain) < 0.02
    assert torch.equal(outs[0][0], outs[1][0])
    a, b = run.pool.rec_state[0][1].float(), run.pool.rec_state[0][2].float()
    assert rel_err(b, a) < 0.02
    st = ref.new_state()
    hr = ref.forward(prompt, st)
    assert rel_err(outs[0][0], hr[-1:]) < 0.05


@pytest.mark.parametrize("kv_dtype", ["fp8", "int8", "bf16"])
def test_gemm_form_prefill_attention_matches_the_fused_kernel_and_the_reference(kv_dtype):
    """Long-context prefill attention as tcgen05 GEMMs (page gather -> S = Q K^T -> causal softmax -> O = P V -> gate) against
    the fused warp-level kernel on the same pool and against the fp32 model; two chunks, so the second one attends to pages
    written by the first."""
    g = torch.Generator().manual_seed(0)
    outs = {}
    for arm in ("gemm", "gemm_flat", "fused"):
        spec, run, ref = build("tc", kv_dtype=kv_dtype)
        run.ATTN_GEMM_FROM = 128 if arm != "fused" else 0
        if arm == "gemm_flat":       # one GEMM pair per q head instead of per kv head
            run._attn_ws = K.attn_gemm_ws(DEV, 216, 256, spec.hq, spec.hkv, spec.hd)
            run._attn_ws["grouped"] = False
        prompt = torch.randint(0, spec.vocab, (256,), generator=torch.Generator().manual_seed(1))
        seq_row, slot = 1, 2
        run.block_table[seq_row, :16] = torch.arange(16, 32, dtype=torch.int32, device=DEV).flip(0)
        ids = prompt.to(torch.int32).to(DEV)
        run.prefill_chunk_forward(ids[:216], 0, seq_row, slot, want_logits=False)
        run.prefill_chunk_forward(ids[216:], 216, seq_row, slot)           # a 40-row tail chunk over 256 keys
        torch.cuda.synchronize()
        outs[arm] = run.logits[:1].float().cpu()
        if arm != "fused":
            assert run._attn_ws is not None
            from owl_engine_b200.ops import gemm_tc
            assert gemm_tc.gemm_status() == 0
    want = ref.logits(ref.forward(prompt, ref.new_state())[-1:])
    assert rel_err(outs["gemm"], outs["fused"]) < 0.02 and rel_err(outs["gemm_flat"], outs["fused"]) < 0.02
    assert rel_err(outs["gemm"], want) < 0.05


def test_w4a8_decode_arm_tracks_the_reference():
    """8-bit decode activations (``act_bits = 8``): greedy decode steps stay close to the fp32 model (looser than the 15-bit
    arm), eager and captured."""
    spec, run, ref = build("tc")
    run.act_bits = 8
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab, (37,), generator=g)
    seq_row, slot = 1, 2
    run.block_table[seq_row, :8] = torch.tensor([5, 9, 2, 30, 11, 12, 13, 14], dtype=torch.int32, device=DEV)
    run.prefill_chunk_forward(prompt.to(torch.int32).to(DEV), 0, seq_row, slot)
    st = ref.new_state()
    want = ref.logits(ref.forward(prompt, st)[-1:])
    lay = H.StepLayout(1, 1)
    v = run.views(lay)
    nxt = int(want.argmax(-1))
    for step in range(4):
        pos = 37 + step
        v["ids"][0] = nxt
        v["pos3"][:] = pos
        v["kv_slot"][0] = int(run.block_table[seq_row, pos // 16]) * 16 + pos % 16
        v["ctx"][0] = pos + 1
        v["gslot"][0] = slot
        v["bt_row"][0] = seq_row
        if step < 2:
            run.step_forward(lay, ctx_hint=64)
        else:
            run.capture(1, 1, ctx_hint=64).replay()
        torch.cuda.synchronize()
        want = ref.logits(ref.forward(torch.tensor([nxt]), st))
        assert rel_err(run.logits[:1].float().cpu(), want) < 0.12, step
        nxt = int(want.argmax(-1))


@pytest.mark.parametrize("kv_dtype", ["int8", "bf16"])
def test_int8_and_16bit_kv_pools_match_reference(kv_dtype):
    """int8 KV pool (per token, per head scales) and the 16-bit pool (fp16 words holding bf16-rounded values): prefill in two
    chunks, then eager and graph decode steps against the fp32 model with an unquantised cache; the stored values are the keys
    the kernel was given."""
    spec, run, ref = build("tc", kv_dtype=kv_dtype)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab, (37,), generator=g)
    seq_row, slot = 1, 2
    run.block_table[seq_row, :8] = torch.tensor([5, 9, 2, 30, 11, 12, 13, 14], dtype=torch.int32, device=DEV)
    ids = prompt.to(torch.int32).to(DEV)
    run.prefill_chunk_forward(ids[:21], 0, seq_row, slot, want_logits=False)
    run.prefill_chunk_forward(ids[21:], 21, seq_row, slot)
    torch.cuda.synchronize()
    st = ref.new_state()
    hr = ref.forward(prompt, st)
    want = ref.logits(hr[-1:])
    assert rel_err(run.logits[:1].float().cpu(), want) < 0.05
    if kv_dtype == "int8":
        ks = run.pool.k_scale[0, 5]                              # page 5 holds positions 0..15
        assert (ks > 0).all() and (run.pool.k_pool[0, 5].view(torch.int8).abs().amax(-1) == 127).all()
    else:
        kp = run.pool.k_pool[0, 5]                               # fp16 words, every one exactly a bf16 value
        assert kp.dtype == torch.float16 and torch.equal(kp.float(), kp.float().bfloat16().float()) and kp.abs().max() > 0
        assert rel_err(run.logits[:1].float().cpu(), want) < 0.03
    lay = H.StepLayout(1, 1)
    v = run.views(lay)
    nxt = int(want.argmax(-1))
    for step in range(4):
        pos = 37 + step
        v["ids"][0] = nxt
        v["pos3"][:] = pos
        v["kv_slot"][0] = int(run.block_table[seq_row, pos // 16]) * 16 + pos % 16
        v["ctx"][0] = pos + 1
        v["gslot"][0] = slot
        v["bt_row"][0] = seq_row
        if step < 2:
            run.step_forward(lay, ctx_hint=64)
        else:
            run.capture(1, 1, ctx_hint=64).replay()
        torch.cuda.synchronize()
        hr = ref.forward(torch.tensor([nxt]), st)
        want = ref.logits(hr)
        assert rel_err(run.logits[:1].float().cpu(), want) < DECODE_TOL, step
        nxt = int(want.argmax(-1))


@pytest.mark.parametrize("arm", ["tc", "tc8"])
def test_nvfp4_weights_prefill_and_decode_match_reference(arm):
    """NVFP4 weights as stored (e2m1 codes, e4m3 block scales, per-tensor scale): prefill through the dequantise-once
    GEMM (bf16, or re-quantised e4m3 rows), decode through ActPack -> bf16 -> streaming NVFP4 GEMV, against the fp32 model
    running on the dequantised weights."""
    spec, run, ref = build(arm, quant="nvfp4")
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab, (150,), generator=g)
    seq_row, slot = 1, 2
    run.block_table[seq_row, :12] = torch.arange(3, 15, dtype=torch.int32, device=DEV)
    ids = prompt.to(torch.int32).to(DEV)
    run.prefill_chunk_forward(ids[:128], 0, seq_row, slot, want_logits=False)      # 128 rows: the dense / e4m3 GEMM
    run.prefill_chunk_forward(ids[128:], 128, seq_row, slot)                        # 22 rows
    torch.cuda.synchronize()
    st = ref.new_state()
    hr = ref.forward(prompt, st)
    want = ref.logits(hr[-1:])
    tol = 0.05 if arm == "tc" else 0.12
    assert rel_err(run.logits[:1].float().cpu(), want) < tol
    lay = H.StepLayout(1, 1)
    v = run.views(lay)
    nxt = int(want.argmax(-1))
    for step in range(3):
        pos = 150 + step
        v["ids"][0] = nxt
        v["pos3"][:] = pos
        v["kv_slot"][0] = int(run.block_table[seq_row, pos // 16]) * 16 + pos % 16
        v["ctx"][0] = pos + 1
        v["gslot"][0] = slot
        v["bt_row"][0] = seq_row
        if step < 2:
            run.step_forward(lay, ctx_hint=256)
        else:
            run.capture(1, 1, ctx_hint=256).replay()
        torch.cuda.synchronize()
        hr = ref.forward(torch.tensor([nxt]), st)
        want = ref.logits(hr)
        assert rel_err(run.logits[:1].float().cpu(), want) < tol, step
        nxt = int(want.argmax(-1))


def test_act_unpack_inverts_act_pack():
    from owl_engine_b200.ops import kernels as K

    g = torch.Generator().manual_seed(9)
    m, k = 5, 512
    x = (torch.randn(m, k, generator=g) * 3).bfloat16().to(DEV)
    for group in (128, 32):
        xp = torch.empty(m, 2 * k, dtype=torch.uint8, device=DEV)
        xs = torch.empty(m, k // group, 2, dtype=torch.float32, device=DEV)
        K.act_pack(x, xp, xs, m, k, group)
        out = torch.zeros(m, k, dtype=torch.bfloat16, device=DEV)
        K.act_unpack(xp, xs, out, m, k, group)
        torch.cuda.synchronize()
        assert rel_err(out.float().cpu(), x.float().cpu()) < 3e-3


def test_nvfp4_checkpoint_loader_weights_run_through_the_per_row_scale_kernels():
    """Weights built by the checkpoint loader from an NVFP4 source (merged projections carry one scale per row) run prefill
    and decode; against the directly quantised model only the quantisation differs (per-tensor vs merged scales), which at
    4 bits with one mantissa bit is a visible but bounded difference (the exact checks of the per-row kernels are in
    test_lowbit_gpu)."""
    from owl_engine_b200.formats import loader as L

    spec = make_spec(n_layers=4)
    dense = init_weights(spec, seed=3, std=0.05)
    hw = L.build_weights(spec, L.NvFp4Provider(dense, 128), DEV)
    assert hw.layers[0].gate_up.layout == "nvfp4" and hw.layers[0].gate_up.row_scale is not None
    pool = H.StatePool(spec, DEV, n_pages=32, n_slots=4)
    run = H.HybridRunner(spec, hw, pool, max_seqs=4, max_blocks=16, prefill_gemm="tc")
    _, run2, _ = build("tc", quant="nvfp4")
    ids = torch.randint(0, spec.vocab, (140,), generator=torch.Generator().manual_seed(2)).to(torch.int32).to(DEV)
    outs = []
    for r in (run, run2):
        r.block_table[1, :12] = torch.arange(3, 15, dtype=torch.int32, device=DEV)
        r.prefill_chunk_forward(ids, 0, 1, 2)
        lay = H.StepLayout(1, 1)
        v = r.views(lay)
        v["ids"][0] = 5; v["pos3"][:] = 140; v["kv_slot"][0] = int(r.block_table[1, 140 // 16]) * 16 + 140 % 16
        v["ctx"][0] = 141; v["gslot"][0] = 2; v["bt_row"][0] = 1
        r.step_forward(lay, ctx_hint=256)
        torch.cuda.synchronize()
        outs.append(r.logits[:1].float().cpu())
    assert torch.isfinite(outs[0]).all() and rel_err(outs[0], outs[1]) < 0.5


@pytest.mark.parametrize("arm,tol", [("tcr", 0.03), ("tc8r", 0.35)])   # e4m3 on both operands of every projection of every layer
def test_wide_batched_step_on_the_resident_dense_weights_matches_the_streaming_arm(arm, tol):
    """16+ rows with a resident dense weight copy: the step multiplies it on the persistent tcgen05 GEMM (fp16, or e4m3
    rows with per-token activation scales); logits agree with the integer weight-streaming arm on the same rows."""
    b = 24
    spec = make_spec(n_layers=4)
    dense = init_weights(spec, seed=3, std=0.05)
    outs, runs = [], []
    for a in (arm, "tc"):
        hw, _ = H.weights_from_dense(spec, dense, DEV)
        pool = H.StatePool(spec, DEV, n_pages=64, n_slots=b)
        r = H.HybridRunner(spec, hw, pool, max_seqs=b, max_blocks=4, prefill_gemm=a)
        lay = H.StepLayout(b, 1)
        v = r.views(lay)
        r.block_table[:, 0] = torch.arange(b, dtype=torch.int32, device=DEV)
        v["ids"].copy_(torch.randint(0, spec.vocab, (b,), generator=torch.Generator().manual_seed(4)).to(torch.int32))
        v["pos3"][:] = 0
        v["kv_slot"].copy_(torch.arange(b, dtype=torch.int32) * 16)
        v["ctx"][:] = 1
        v["gslot"].copy_(torch.arange(b, dtype=torch.int32))
        v["bt_row"].copy_(torch.arange(b, dtype=torch.int32))
        r.step_forward(lay, ctx_hint=64)
        torch.cuda.synchronize()
        outs.append(r.logits[:b].float().cpu())
        runs.append(r)
    assert runs[0]._x16h is not None and runs[1]._x16h is None
    assert rel_err(outs[0], outs[1]) < tol
