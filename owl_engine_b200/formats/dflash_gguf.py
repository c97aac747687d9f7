"""The DFlash2 draft model as a GGUF file (``general.architecture = "dflash"``).

A draft file differs from a language-model file in three ways, which is why it has a reader of its own:

* **facts** come from ``dflash.*`` metadata (no gated-delta-net keys): widths, head geometry, block size, selector rank and
  top-k, the mask token, and ``dflash.target_layers`` -- the target layers whose outputs feed the draft, **1-based** in the file
  and 0-based here. They must be as many as the draft has layers, strictly increasing and inside the target; a file whose
  list contains 0 has been normalised twice and would silently shift every tap by one layer, so it is refused;
* **names**: HF-style keys of the draft (``layers.N.self_attn.q_proj.weight``) map to ``blk.N.attn_q.weight`` etc. by a closed
  table (an unknown key is an error, nothing falls through);
* **types**: projections are block-quantised (Q4_K / Q6_K / Q8_0) in the file; the draft's kernels stream bf16 records, so
  everything is dequantised once at load (the draft is read once per proposal, 3.8 GB in bf16 at 27B scale).

The draft shares the target's embedding table, final norm and lm_head, so the file holds none of them.

Reference counterpart: ``crates/models/src/formats/gguf/draft.rs:1-275`` (name table, fc layout, code books) and
``draft_meta.rs:80-250`` (facts, 1-based taps, refusals).
"""
from __future__ import annotations


from ..models import dflash2 as D
from . import gguf


class DraftLoadError(ValueError):
    pass


_LAYER = {
    "attention_conv.base_kernel": "attn_conv_base", "attention_conv.kernel_projection.weight": "attn_conv_proj.weight",
    "mlp_conv.base_kernel": "ffn_conv_base", "mlp_conv.kernel_projection.weight": "ffn_conv_proj.weight",
    "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
    "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
    "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight",
}
_TOP = {
    "fc.weight": "fc.weight", "hidden_norm.weight": "enc.output_norm.weight", "norm.weight": "output_norm.weight",
    "selector.hidden_projection.weight": "selector_hidden.weight", "selector.predecessor_codebook": "selector_predecessor.weight",
    "selector.successor_codebook": "selector_successor.weight",
}


def gguf_name(key: str) -> str:
    """The draft's own key -> the tensor name in the file."""
    if key in _TOP:
        return _TOP[key]
    if key.startswith("layers."):
        _, idx, tail = key.split(".", 2)
        if idx.isdigit() and tail in _LAYER:
            return f"blk.{idx}.{_LAYER[tail]}"
    raise DraftLoadError(f"GGUF draft: no file tensor is defined for the key {key!r}")


def draft_spec(f: gguf.GgufFile, target) -> D.DraftSpec:
    """``dflash.*`` metadata -> ``DraftSpec``, checked against the target model's description (``models.spec.ModelSpec``)."""
    m = f.meta
    where = f"GGUF draft {f.path}"
    arch = m.get("general.architecture")
    if arch != "dflash":
        raise DraftLoadError(f"{where}: general.architecture = {arch!r}; a draft file says \"dflash\" (language models load "
                             "through the model path)")

    def need(k):
        if "dflash." + k not in m:
            raise DraftLoadError(f"{where}: metadata key dflash.{k} is missing")
        return m["dflash." + k]

    hidden, inter, layers = int(need("embedding_length")), int(need("feed_forward_length")), int(need("block_count"))
    hq, hkv = int(need("attention.head_count")), int(need("attention.head_count_kv"))
    hd, vd = int(need("attention.key_length")), int(need("attention.value_length"))
    block, rank, top_k = int(need("block_size")), int(need("selector_rank")), int(need("selector_top_k"))
    if hidden != target.hidden:
        raise DraftLoadError(f"{where}: hidden {hidden} but the target's is {target.hidden}: not a draft of this model family")
    if hd != vd:
        raise DraftLoadError(f"{where}: key_length {hd} != value_length {vd}")
    if min(layers, hq, hkv) <= 0 or hq % hkv:
        raise DraftLoadError(f"{where}: head / layer geometry (layers {layers}, hq {hq}, hkv {hkv})")
    if not (2 <= block <= 8):
        raise DraftLoadError(f"{where}: block_size {block}: the verify step holds 1 anchor + at most 7 drafts")
    if m.get("dflash.attention.causal", False):
        raise DraftLoadError(f"{where}: dflash.attention.causal = true; the draft attends to its whole block")
    raw = m.get("dflash.target_layers")
    if not raw:
        raise DraftLoadError(f"{where}: dflash.target_layers is missing (which target layers feed the draft)")
    raw = [int(x) for x in raw]
    if len(raw) != layers:
        raise DraftLoadError(f"{where}: {len(raw)} target layers for {layers} draft layers (one tap per layer)")
    if any(x <= 0 for x in raw):
        raise DraftLoadError(f"{where}: dflash.target_layers = {raw} contains 0: the file counts from 1, so it has been normalised "
                             "twice (every tap would be one layer off)")
    taps = tuple(x - 1 for x in raw)
    if any(b <= a for a, b in zip(taps, taps[1:])) or taps[-1] >= target.n_layers:
        raise DraftLoadError(f"{where}: taps {list(taps)} are not strictly increasing inside the target's {target.n_layers} layers")
    mask = int(m.get("dflash.mask_token_id", target.vocab - 1))
    if not (0 <= mask < target.vocab):
        raise DraftLoadError(f"{where}: mask token {mask} outside the vocabulary of {target.vocab}")
    window = int(m.get("dflash.attention.sliding_window", 2048))
    return D.DraftSpec(hidden=hidden, n_layers=layers, hq=hq, hkv=hkv, hd=hd, inter=inter, vocab=target.vocab, block=block,
                       top_k=top_k, rank=rank, window=window, mask_token_id=mask,
                       rope_theta=float(m.get("dflash.rope.freq_base", 1e7)),
                       eps=float(m.get("dflash.attention.layer_norm_rms_epsilon", 1e-6)), taps=taps)


def draft_keys(spec: D.DraftSpec) -> list[str]:
    keys = list(_TOP)
    for i in range(spec.n_layers):
        keys += [f"layers.{i}.{t}" for t in _LAYER]
    return keys


def draft_dense(f: gguf.GgufFile, spec: D.DraftSpec) -> dict:
    """Every tensor of the draft under its own key, dequantised (what ``models.dflash2.weights_from_dense`` takes)."""
    h = spec.hidden
    want = {"fc.weight": (h, h * len(spec.taps)), "selector.hidden_projection.weight": (spec.rank, h),
            "selector.predecessor_codebook": (spec.vocab, spec.rank), "selector.successor_codebook": (spec.vocab, spec.rank)}
    out, missing = {}, []
    for key in draft_keys(spec):
        name = gguf_name(key)
        if name not in f.tensors:
            missing.append(name)
            continue
        t = f.dequant(name)
        if key in want and tuple(t.shape) != want[key]:
            raise DraftLoadError(f"GGUF draft {f.path}: {name} is {tuple(t.shape)}, expected {want[key]}")
        out[key] = t
    if missing:
        raise DraftLoadError(f"GGUF draft {f.path}: missing tensors " + ", ".join(missing[:8]))
    return out


def load_draft(path, target, device) -> tuple[D.DraftSpec, D.DraftWeights]:
    f = gguf.GgufFile(path)
    spec = draft_spec(f, target)
    return spec, D.weights_from_dense(spec, draft_dense(f, spec), device)
