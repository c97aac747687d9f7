"""``--check`` preflight: checkpoint facts from headers only, by the loader's own rules; every problem in one run."""
import json
import os

import numpy as np
import torch

from owl_engine_b200.formats import gguf, loader, preflight as PF, safetensors as st
from owl_engine_b200.models.reference import init_weights
from owl_engine_b200.models.spec import test_hybrid as make_spec


def _hf_dir(path, spec, dense, config=True, drop=()):
    os.makedirs(path, exist_ok=True)
    st.save_file({k: v.to(torch.bfloat16) for k, v in dense.items() if k not in drop}, os.path.join(path, "model.safetensors"))
    cfg = {"vocab_size": spec.vocab, "hidden_size": spec.hidden, "intermediate_size": spec.inter, "num_hidden_layers": spec.n_layers,
           "num_attention_heads": spec.hq, "num_key_value_heads": spec.hkv, "head_dim": spec.hd, "linear_num_key_heads": spec.nk,
           "linear_num_value_heads": spec.nv, "linear_key_head_dim": spec.kd, "linear_value_head_dim": spec.vd}
    open(os.path.join(path, "config.json"), "w").write(json.dumps(cfg if config else {}))


def test_a_good_directory_passes_and_a_broken_one_lists_everything(tmp_path):
    spec = make_spec(n_layers=4, vocab=512)
    dense = init_weights(spec, seed=1, std=0.05)
    good = str(tmp_path / "good")
    _hf_dir(good, spec, dense)
    items = PF.check_model(good, "safetensors", "w4a16", "test-hybrid", 4096)
    assert all(i.ok for i in items), [i.line() for i in items]
    text = "\n".join(i.line() for i in items)
    assert "safetensors checkpoint" in text and "tensors present" in text and "geometry equals test-hybrid" in text
    bad = str(tmp_path / "bad")
    wrong = dict(dense)
    wrong["model.layers.0.mlp.down_proj.weight"] = torch.zeros(spec.hidden, spec.inter + 16)
    _hf_dir(bad, spec, wrong, drop=("model.layers.1.linear_attn.A_log", "model.layers.3.self_attn.q_norm.weight"))
    items = PF.check_model(bad, "safetensors", "w4a16", "test-hybrid", 10 ** 7)
    fails = [i.text for i in items if not i.ok]
    assert len(fails) == 3
    assert any("2 tensors missing" in f and "A_log" in f for f in fails)
    assert any("down_proj" in f and "shapes differ" in f for f in fails)
    assert any("exceeds the trained context" in f for f in fails)
    assert PF.check_model(bad, "safetensors", "w4a16", "test-hybrid", 10 ** 6, yarn_factor=4.0)[-1].ok


def test_format_and_path_mismatches_fail_here_not_at_boot(tmp_path):
    spec = make_spec(n_layers=4, vocab=512)
    d = str(tmp_path / "hf")
    _hf_dir(d, spec, init_weights(spec, seed=1, std=0.05))
    assert "is a safetensors checkpoint" in PF.check_model(d, "awq", "w4a16", "test-hybrid", 512)[0].text
    assert not PF.check_model(d, "gguf", "gguf", "test-hybrid", 512)[0].ok
    assert "does not exist" in PF.check_model(str(tmp_path / "nope"), "safetensors", "w4a16", "test-hybrid", 512)[0].text
    other = make_spec(n_layers=4, vocab=512, hidden=128)
    d2 = str(tmp_path / "other")
    _hf_dir(d2, other, init_weights(other, seed=1, std=0.05))
    items = PF.check_model(d2, "safetensors", "w4a16", "test-hybrid", 512)
    assert any((not i.ok) and "geometry differs" in i.text and "hidden 128" in i.text for i in items)
    assert PF.check_model("", "random", "w4a16", "qwen3.8-27b", 512)[0].ok


def test_gguf_model_draft_and_projector(tmp_path):
    from test_dflash_gguf import dense_weights, write as write_draft
    from test_vision_weights import _mmproj_file

    from owl_engine_b200.models import dflash2 as D
    from owl_engine_b200.models import vision as V

    spec = make_spec(n_layers=4, vocab=512)
    dense = init_weights(spec, seed=3, std=0.05)
    tensors = {}
    for k, v in dense.items():
        a = v.float().numpy()
        a = np.ascontiguousarray(a.reshape(a.shape[0], -1) if a.ndim == 3 else a)
        tensors[loader.gguf_name(k)] = (tuple(a.shape), "F32", a.view(np.uint8).reshape(-1))
    meta = {"general.architecture": "qwen35", "qwen35.embedding_length": spec.hidden, "qwen35.feed_forward_length": spec.inter,
            "qwen35.block_count": spec.n_layers, "qwen35.attention.head_count": spec.hq, "qwen35.attention.head_count_kv": spec.hkv,
            "qwen35.ssm.group_count": spec.nk, "qwen35.ssm.time_step_rank": spec.nv, "qwen35.vocab_size": spec.vocab}
    model = tmp_path / "m.gguf"
    gguf.write_gguf(model, meta, tensors)
    items = PF.check_model(str(model), "gguf", "gguf", "test-hybrid", 512)
    assert all(i.ok for i in items), [i.line() for i in items]
    assert not all(i.ok for i in PF.check_model(str(model), "gguf", "w4a16", "test-hybrid", 512))
    # the projector file next to it
    assert not PF.check_vision(True, "gguf", str(model), "", spec.hidden)[0].ok                 # none there yet
    vs = V.tiny_vision(out_hidden=spec.hidden)
    _mmproj_file(tmp_path / "mmproj-x.gguf", vs, V.init_vision_weights(vs, seed=1))
    v = PF.check_vision(True, "gguf", str(model), "", spec.hidden)
    assert v[0].ok and "mmproj-x.gguf" in v[0].text
    assert not PF.check_vision(True, "gguf", str(model), "", spec.hidden * 2)[0].ok             # outputs the wrong width
    assert PF.check_vision(False, "gguf", str(model), "", spec.hidden) == []
    # the draft container
    target = make_spec(n_layers=8, hidden=256, vocab=512)
    ds = D.DraftSpec(hidden=256, n_layers=2, hq=4, hkv=2, hd=128, inter=512, vocab=512, rank=256, window=64, taps=(2, 6), mask_token_id=511)
    write_draft(tmp_path / "draft.gguf", ds, dense_weights(ds))
    d = PF.check_draft("dflash2", str(tmp_path / "draft.gguf"), target)
    assert d[0].ok and "taps [2, 6]" in d[0].text
    write_draft(tmp_path / "draft2.gguf", ds, dense_weights(ds), meta_over={"dflash.target_layers": [0, 3]})
    assert "normalised twice" in PF.check_draft("dflash2", str(tmp_path / "draft2.gguf"), target)[0].text
    assert PF.check_draft("none", "", target) == [] and PF.check_draft("mtp", "", target)[0].ok


def test_check_exit_code_and_lines(tmp_path, capsys):
    from owl_engine_b200.server import main as M

    root = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "configs", "full.toml"))
    prof = tmp_path / "p.toml"
    prof.write_text(f'extends = ["{root}"]\n[model]\nname = "test-hybrid"\npath = "{tmp_path / "missing"}"\nformat = "safetensors"\n')
    assert M.main(["-p", str(prof), "--check"]) == 1
    assert "[check] FAIL model:" in capsys.readouterr().out
    assert M.main(["-p", root, "--check"]) == 0
