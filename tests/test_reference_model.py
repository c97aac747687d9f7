"""CPU reference model: parity with HF transformers Qwen3.5 and self-consistency."""
import pytest
import torch

from owl_engine_b200.models.reference import RefModel, init_weights
from owl_engine_b200.models.spec import ModelSpec, tiny_hybrid
from owl_engine_b200.ops import reference as R


def small_spec():
    return ModelSpec(name="s", vocab=257, hidden=64, inter=128, n_layers=4, hq=4, hkv=2, hd=32, rotary_dim=8,
                     rope_theta=1e7, nk=2, kd=16, nv=4, vd=16)


def hf_model(spec, weights):
    m = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    cfg = m.Qwen3_5TextConfig(
        vocab_size=spec.vocab, hidden_size=spec.hidden, intermediate_size=spec.inter, num_hidden_layers=spec.n_layers,
        num_attention_heads=spec.hq, num_key_value_heads=spec.hkv, head_dim=spec.hd,
        linear_num_key_heads=spec.nk, linear_num_value_heads=spec.nv, linear_key_head_dim=spec.kd,
        linear_value_head_dim=spec.vd, linear_conv_kernel_dim=4, rms_norm_eps=spec.eps,
        layer_types=["full_attention" if spec.is_full(i) else "linear_attention" for i in range(spec.n_layers)],
        rope_parameters={"rope_type": "default", "rope_theta": spec.rope_theta,
                         "partial_rotary_factor": spec.rotary_dim / spec.hd, "mrope_section": [2, 1, 1]},
        tie_word_embeddings=False, attn_implementation="eager")
    model = m.Qwen3_5ForCausalLM(cfg).float().eval()
    missing, unexpected = model.load_state_dict(weights, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in k or "inv_freq" in k for k in missing), missing
    return model


def test_hf_parity_prefill_logits():
    spec = small_spec()
    w = init_weights(spec, seed=1, std=0.1)
    hf = hf_model(spec, w)
    ids = torch.randint(0, spec.vocab, (19,), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    ref = RefModel(spec, w)
    st = ref.new_state()
    got = ref.logits(ref.forward(ids, st))
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)


def test_chunked_equals_recurrent_and_decode_equals_prefill():
    spec = small_spec()
    w = init_weights(spec, seed=2, std=0.1)
    ids = torch.randint(0, spec.vocab, (70,), generator=torch.Generator().manual_seed(3))
    a = RefModel(spec, w)
    b = RefModel(spec, w, chunked_gdn=True)
    sa, sb = a.new_state(), b.new_state()
    ha, hb = a.forward(ids, sa), b.forward(ids, sb)
    torch.testing.assert_close(ha, hb, rtol=1e-3, atol=1e-3)
    # token-by-token decode reproduces the prefill hidden states
    sc = a.new_state()
    hc = torch.cat([a.forward(ids[i:i + 1], sc) for i in range(20)])
    torch.testing.assert_close(hc, ha[:20], rtol=1e-3, atol=1e-3)
    # chunked prefill (two pieces) equals one piece
    sd = a.new_state()
    hd = torch.cat([a.forward(ids[:33], sd), a.forward(ids[33:], sd)])
    torch.testing.assert_close(hd, ha, rtol=1e-3, atol=1e-3)


def test_gdn_chunk_matches_hf_chunk_rule():
    m = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    g = torch.Generator().manual_seed(5)
    t, h, kd, vd = 130, 3, 16, 24
    q, k = R.l2norm(torch.randn(t, h, kd, generator=g)), R.l2norm(torch.randn(t, h, kd, generator=g))
    v = torch.randn(t, h, vd, generator=g)
    gl = -torch.rand(t, h, generator=g)
    beta = torch.rand(t, h, generator=g)
    s0 = torch.randn(h, kd, vd, generator=g) * 0.1
    want_o, want_s = m.torch_chunk_gated_delta_rule(q[None], k[None], v[None], gl[None], beta[None],
                                                    initial_state=s0[None], output_final_state=True)
    for fn in (R.gdn_recurrent, R.gdn_chunked):
        o, s = fn(q, k, v, gl, beta, s0)
        torch.testing.assert_close(o, want_o[0], rtol=1e-3, atol=1e-3)
        torch.testing.assert_close(s, want_s[0], rtol=1e-3, atol=1e-3)


@pytest.mark.slow
def test_tiny_hybrid_greedy_is_deterministic():
    spec = tiny_hybrid()
    spec = ModelSpec(**{**spec.__dict__, "n_layers": 4, "vocab": 4096})
    w = init_weights(spec, seed=0)
    ref = RefModel(spec, w)
    prompt = torch.randint(0, spec.vocab, (16,), generator=torch.Generator().manual_seed(0))
    t1, _ = ref.generate(prompt, 4)
    t2, _ = ref.generate(prompt, 4, prefill_chunk=5)
    assert t1.tolist() == t2.tolist()
