"""Profiles: extends chains, strict keys, --set / --explain / --check, the intent layer, every shipped profile and part."""
import json
from pathlib import Path

import pytest

from owl_engine_b200.utils import config as C
from owl_engine_b200.utils.memory import estimate

ROOT = Path(__file__).resolve().parents[1] / "configs"


def test_full_profile_loads_and_every_schema_key_is_documented():
    cfg = C.load(ROOT / "full.toml")
    for sec, keys in C.SCHEMA.items():
        if sec in C.OPTIONAL_SECTIONS:
            continue
        assert set(keys) == set(cfg.values[sec]), sec


def test_extends_chain_set_and_explain(tmp_path):
    cfg = C.load(ROOT / "qwen38_27b-b200_tp8.toml", sets=["runtime.max_batch=16", "log.level=\"info\""])
    assert cfg.get("parallel.mode") == "tp" and len(cfg.get("parallel.device")) == 8
    assert cfg.get("runtime.max_batch") == 16 and cfg.get("log.level") == "info"
    text = cfg.explain("runtime.max_batch")
    assert "--set" in text and "full.toml" in text
    est = estimate(cfg)
    assert est["tp"] == 8 and est["kv_tokens"] > 1_000_000 and est["weights_bytes"] < 6e9
    assert json.loads(cfg.to_json())["model"]["name"] == "qwen3.8-27b"


def test_refusals(tmp_path):
    base = f'extends = ["{ROOT / "full.toml"}"]\n'
    (tmp_path / "a.toml").write_text(base + "[runtime]\nbogus = 1\n")
    with pytest.raises(C.ConfigError, match="unknown key runtime.bogus"):
        C.load(tmp_path / "a.toml")
    (tmp_path / "b.toml").write_text(base + "[nosuch]\nx = 1\n")
    with pytest.raises(C.ConfigError, match="unknown section"):
        C.load(tmp_path / "b.toml")
    (tmp_path / "c.toml").write_text(base + "[store.kv]\nkv_dtype = \"fp4\"\n")
    with pytest.raises(C.ConfigError, match="kv_dtype"):
        C.load(tmp_path / "c.toml")
    (tmp_path / "d.toml").write_text("[runtime]\nmax_seq = 1\n")
    with pytest.raises(C.ConfigError, match="missing"):
        C.load(tmp_path / "d.toml")
    (tmp_path / "e.toml").write_text('extends = ["f.toml"]\n')
    (tmp_path / "f.toml").write_text('extends = ["e.toml"]\n')
    with pytest.raises(C.ConfigError, match="cycle"):
        C.load(tmp_path / "e.toml")
    with pytest.raises(C.ConfigError, match="layer"):
        C.load(ROOT / "full.toml", sets=['parallel.mode="layer"'])
    with pytest.raises(C.ConfigError, match="allowed|2, 4 or 8"):
        C.load(ROOT / "full.toml", sets=['parallel.mode="tp"', 'parallel.device=["0","1","2"]'])


def test_intent_layer_and_max_context(tmp_path):
    (tmp_path / "i.toml").write_text(f'extends = ["{ROOT / "full.toml"}"]\n[intent]\nhardware = "b200x4"\n'
                                     'goal = "throughput"\ncontext = "max"\n')
    cfg = C.load(tmp_path / "i.toml")
    assert cfg.get("parallel.mode") == "tp" and cfg.get("runtime.max_batch") == 32
    assert cfg.get("runtime.max_seq") % 16 == 0 and cfg.get("runtime.max_seq") > 100_000
    assert "derived:intent" in cfg.explain("runtime.max_batch")


def test_cli_check(capsys):
    assert C.main_cli(["-p", str(ROOT / "qwen38_27b-b200.toml"), "--check", "--explain", "store.vram_budget"]) == 0
    out = capsys.readouterr().out
    assert "kv_pages" in out and "vram_budget" in out
    assert C.main_cli(["-p", str(ROOT / "full.toml"), "--set", "runtime.nope=1"]) == 2


def test_every_shipped_profile_and_part_loads(tmp_path):
    import glob
    import os

    root = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "configs"))
    leaves = sorted(glob.glob(os.path.join(root, "*.toml")))
    assert len(leaves) >= 7
    for leaf in leaves:
        C.load(leaf)
    parts = sorted(glob.glob(os.path.join(root, "parts", "*", "*.toml")))
    assert len(parts) >= 20
    for part in parts:
        if os.path.basename(part) in ("disk-tier.toml",):
            continue                                       # needs a directory and the host tier from the leaf (checked below)
        p = tmp_path / "one.toml"
        p.write_text(f'extends = ["{root}/full.toml", "{part}"]\n')
        C.load(str(p))
    p = tmp_path / "disk.toml"
    p.write_text(f'extends = ["{root}/full.toml", "{root}/parts/feature/agent.toml", "{root}/parts/feature/disk-tier.toml"]\n'
                 f'[store]\ndisk_dir = "{tmp_path}"\n')
    cfg = C.load(str(p))
    assert cfg.get("store.snap_disk_mb") == 16384 and cfg.get("store.evict_policy") == "lrfu"


def test_memory_model_counts_resident_copies_draft_vision_and_state_rows():
    base = estimate(C.load(str(ROOT / "full.toml")))
    tcr = estimate(C.load(str(ROOT / "full.toml"), ['kernel.prefill_gemm="tcr"']))
    tc8r = estimate(C.load(str(ROOT / "full.toml"), ['kernel.prefill_gemm="tc8r"']))
    assert base["resident_copies_bytes"] == 0 and tcr["resident_copies_bytes"] == 2 * tc8r["resident_copies_bytes"]
    assert 40e9 < tcr["resident_copies_bytes"] < 60e9                                   # an fp16 copy of a 27B model's projections
    assert base["kv_pool_bytes"] - tcr["kv_pool_bytes"] == tcr["resident_copies_bytes"]
    dfl = estimate(C.load(str(ROOT / "full.toml"), ['spec.kind="dflash2"', "spec.depth=7"]))
    assert 3e9 < dfl["draft_bytes"] < 5e9 and dfl["state_rows"] == base["state_rows"] + 7   # batched verify scratch rows
    vis = estimate(C.load(str(ROOT / "full.toml"), ["vision.enabled=true"]))
    assert vis["vision_bytes"] > 0 and vis["kv_pool_bytes"] < base["kv_pool_bytes"]
    snap = estimate(C.load(str(ROOT / "full.toml"), ["store.gdn.snap_max=8", "store.snap_host_mb=4096", "store.host_cache_mb=1024"]))
    assert snap["state_rows"] == base["state_rows"] + 6 and snap["pinned_host_bytes"] == 5120 << 20
