"""HF ``config.json`` (Qwen3.5 / Qwen3.8 text config) -> ``ModelSpec``."""
from __future__ import annotations

from .spec import ModelSpec


def spec_from_hf_config(cfg: dict) -> ModelSpec:
    t = cfg.get("text_config", cfg)
    rope = t.get("rope_parameters") or t.get("rope_scaling") or {}
    hd = t.get("head_dim") or t["hidden_size"] // t["num_attention_heads"]
    types = t.get("layer_types")
    full_every = 4
    if types and "full_attention" in types:
        full_every = types.index("full_attention") + 1
    return ModelSpec(name=cfg.get("_name_or_path", t.get("model_type", "qwen3_5")), vocab=t["vocab_size"],
                     hidden=t["hidden_size"], inter=t["intermediate_size"], n_layers=t["num_hidden_layers"],
                     hq=t["num_attention_heads"], hkv=t["num_key_value_heads"], hd=hd,
                     rotary_dim=int(hd * rope.get("partial_rotary_factor", t.get("partial_rotary_factor", 0.25))),
                     rope_theta=float(rope.get("rope_theta", t.get("rope_theta", 1e7))),
                     nk=t.get("linear_num_key_heads", 16), kd=t.get("linear_key_head_dim", 128),
                     nv=t.get("linear_num_value_heads", 48), vd=t.get("linear_value_head_dim", 128),
                     conv_k=t.get("linear_conv_kernel_dim", 4), full_every=full_every, eps=t.get("rms_norm_eps", 1e-6),
                     tied=bool(t.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False))))
