"""The DFlash2 draft as a GGUF container: facts, 1-based taps, name table, refusals, and a round trip of the weights."""
import numpy as np
import pytest
import torch

from owl_engine_b200.formats import dflash_gguf as DG
from owl_engine_b200.formats import gguf
from owl_engine_b200.models import dflash2 as D
from owl_engine_b200.models.spec import test_hybrid as make_spec


def dense_weights(spec, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g) * 0.05
    h = spec.hidden
    d = {"fc.weight": r(h, h * len(spec.taps)), "hidden_norm.weight": 1 + r(h), "norm.weight": 1 + r(h)}
    for i in range(spec.n_layers):
        p = f"layers.{i}."
        d[p + "input_layernorm.weight"], d[p + "post_attention_layernorm.weight"] = 1 + r(h), 1 + r(h)
        d[p + "self_attn.q_proj.weight"], d[p + "self_attn.k_proj.weight"] = r(spec.hq * spec.hd, h), r(spec.hkv * spec.hd, h)
        d[p + "self_attn.v_proj.weight"], d[p + "self_attn.o_proj.weight"] = r(spec.hkv * spec.hd, h), r(h, spec.hq * spec.hd)
        d[p + "self_attn.q_norm.weight"], d[p + "self_attn.k_norm.weight"] = 1 + r(spec.hd), 1 + r(spec.hd)
        for c in ("attention_conv", "mlp_conv"):
            d[p + c + ".base_kernel"], d[p + c + ".kernel_projection.weight"] = r(2, 2, h), r(4 * spec.groups, h)
        d[p + "mlp.gate_proj.weight"], d[p + "mlp.up_proj.weight"] = r(spec.inter, h), r(spec.inter, h)
        d[p + "mlp.down_proj.weight"] = r(h, spec.inter)
    d["selector.hidden_projection.weight"] = r(spec.rank, h)
    d["selector.predecessor_codebook"], d["selector.successor_codebook"] = r(spec.vocab, spec.rank), r(spec.vocab, spec.rank)
    return d


def write(path, spec, dense, *, meta_over=None, drop=()):
    tensors = {}
    for k, t in dense.items():
        name = DG.gguf_name(k)
        if name in drop:
            continue
        a = np.ascontiguousarray(t.float().numpy())
        if a.ndim == 2 and a.shape[1] % 256 == 0 and "codebook" in k:
            tensors[name] = (a.shape, "Q4_K", gguf.quantize_q4_k(a))
        elif a.ndim == 2 and a.shape[1] % 32 == 0:
            tensors[name] = (a.shape, "Q8_0", gguf.quantize_q8_0(a))
        else:
            tensors[name] = (a.shape, "F32", a.view(np.uint8).reshape(-1))
    meta = {"general.architecture": "dflash", "dflash.embedding_length": spec.hidden, "dflash.feed_forward_length": spec.inter,
            "dflash.block_count": spec.n_layers, "dflash.attention.head_count": spec.hq, "dflash.attention.head_count_kv": spec.hkv,
            "dflash.attention.key_length": spec.hd, "dflash.attention.value_length": spec.hd, "dflash.block_size": spec.block,
            "dflash.selector_rank": spec.rank, "dflash.selector_top_k": spec.top_k, "dflash.mask_token_id": spec.mask_token_id,
            "dflash.target_layers": [t + 1 for t in spec.taps], "dflash.attention.sliding_window": spec.window}
    meta.update(meta_over or {})
    gguf.write_gguf(path, meta, tensors)


@pytest.fixture
def target():
    return make_spec(n_layers=8, hidden=256, vocab=512)


def test_round_trip_of_facts_and_weights(tmp_path, target):
    spec = D.DraftSpec(hidden=256, n_layers=2, hq=4, hkv=2, hd=128, inter=512, vocab=512, rank=256, window=64, taps=(2, 6),
                       mask_token_id=511)
    dense = dense_weights(spec)
    write(tmp_path / "draft.gguf", spec, dense)
    f = gguf.GgufFile(tmp_path / "draft.gguf")
    got = DG.draft_spec(f, target)
    assert got == spec                                              # taps come back 0-based
    w = DG.draft_dense(f, got)
    assert set(w) == set(dense)
    for k in dense:
        tol = 0.12 if "codebook" in k else 0.02
        assert ((w[k].float() - dense[k]).norm() / dense[k].norm()).item() < tol, k
    dspec, dw = DG.load_draft(tmp_path / "draft.gguf", target, "cpu")
    assert len(dw.layers) == 2 and dw.a_tab.shape == (512, 256) and dw.fc.shape == (256, 512)


def test_refusals(tmp_path, target):
    spec = D.DraftSpec(hidden=256, n_layers=2, hq=4, hkv=2, hd=128, inter=512, vocab=512, rank=256, window=64, taps=(2, 6))
    dense = dense_weights(spec)
    cases = [({"general.architecture": "qwen35"}, "dflash"),
             ({"dflash.target_layers": [0, 3]}, "normalised twice"),
             ({"dflash.target_layers": [3]}, "one tap per layer"),
             ({"dflash.target_layers": [7, 3]}, "strictly increasing"),
             ({"dflash.target_layers": [3, 9]}, "strictly increasing"),
             ({"dflash.embedding_length": 128}, "not a draft of this model family"),
             ({"dflash.attention.causal": True}, "causal"),
             ({"dflash.mask_token_id": 9999}, "mask token"),
             ({"dflash.block_size": 12}, "block_size")]
    for i, (over, needle) in enumerate(cases):
        p = tmp_path / f"d{i}.gguf"
        write(p, spec, dense, meta_over=over)
        with pytest.raises(DG.DraftLoadError, match=needle):
            DG.draft_spec(gguf.GgufFile(p), target)
    write(tmp_path / "m.gguf", spec, dense, drop=("blk.1.ffn_conv_base", "selector_hidden.weight"))
    f = gguf.GgufFile(tmp_path / "m.gguf")
    with pytest.raises(DG.DraftLoadError, match="blk.1.ffn_conv_base"):
        DG.draft_dense(f, DG.draft_spec(f, target))
    with pytest.raises(DG.DraftLoadError):
        DG.gguf_name("layers.0.self_attn.rotary.inv_freq")
