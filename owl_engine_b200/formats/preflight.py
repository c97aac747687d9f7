"""Preflight: what ``--check`` can say about a profile's checkpoints before anything is loaded.

Everything here reads headers only (safetensors JSON headers, GGUF metadata and tensor infos, ``config.json``) and uses the
loader's own rules -- the same kind detection, the same name tables, the same geometry sources -- so that "the check passed, the
boot failed" cannot come from two copies of a rule. Problems are collected, not raised: one run shows all of them.

    model       the path exists; its detected kind agrees with ``[model] format`` and ``quant``; the geometry the checkpoint
                declares equals the named model's; every tensor the weight builder will ask for exists with the shape the
                geometry implies; the context asked for fits the trained context (times the YaRN factor)
    draft       ``[spec] draft_path``: a DFlash2 GGUF container is read for its facts (``formats/dflash_gguf.py``); a
                safetensors directory must hold the draft's / the MTP head's tensors
    vision      a GGUF model's projector file resolves (``formats/vision_weights.py``) and describes a tower that fits the
                text model's hidden size; an HF directory holds ``visual.*`` tensors

Reference counterpart: ``crates/engine/src/preflight.rs:1-60`` (check items from the loader's own facts; the server only
prints them).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

from ..models.spec import PRESETS, ModelSpec


@dataclass
class CheckItem:
    ok: bool
    where: str        # "model" | "draft" | "vision"
    text: str

    def line(self) -> str:
        return f"[check] {self.where}: {self.text}" if self.ok else f"[check] FAIL {self.where}: {self.text}"


def needed_tensors(spec: ModelSpec) -> dict:
    """HF name -> expected shape (None: only presence is checked) of everything ``formats.loader.build_weights`` reads."""
    h, need = spec.hidden, {}
    need["model.embed_tokens.weight"] = (spec.vocab, h)
    need["model.norm.weight"] = (h,)
    for i in range(spec.n_layers):
        p = f"model.layers.{i}."
        need[p + "input_layernorm.weight"] = need[p + "post_attention_layernorm.weight"] = (h,)
        need[p + "mlp.gate_proj.weight"] = need[p + "mlp.up_proj.weight"] = (spec.inter, h)
        need[p + "mlp.down_proj.weight"] = (h, spec.inter)
        if spec.is_full(i):
            a = p + "self_attn."
            need[a + "q_proj.weight"] = (2 * spec.hq * spec.hd, h)
            need[a + "k_proj.weight"] = need[a + "v_proj.weight"] = (spec.hkv * spec.hd, h)
            need[a + "o_proj.weight"] = (h, spec.hq * spec.hd)
            need[a + "q_norm.weight"] = need[a + "k_norm.weight"] = (spec.hd,)
        else:
            a = p + "linear_attn."
            need[a + "in_proj_qkv.weight"] = (spec.conv_dim, h)
            need[a + "in_proj_z.weight"] = (spec.value_dim, h)
            need[a + "in_proj_a.weight"] = need[a + "in_proj_b.weight"] = (spec.nv, h)
            need[a + "conv1d.weight"] = None
            need[a + "A_log"] = need[a + "dt_bias"] = (spec.nv,)
            need[a + "norm.weight"] = (spec.vd,)
            need[a + "out_proj.weight"] = (h, spec.value_dim)
    return need


_GEOM = ("hidden", "inter", "n_layers", "hq", "hkv", "hd", "nk", "nv", "kd", "vd", "vocab")


def _geometry_diff(got: ModelSpec, want: ModelSpec) -> list[str]:
    return [f"{k} {getattr(got, k)} (checkpoint) != {getattr(want, k)} ({want.name})" for k in _GEOM if getattr(got, k) != getattr(want, k)]


def check_model(path: str, fmt: str, quant: str, name: str, max_seq: int, yarn_factor: float = 1.0) -> list[CheckItem]:
    from . import gguf, loader

    out: list[CheckItem] = []
    add = lambda ok, text: out.append(CheckItem(ok, "model", text))
    if fmt == "random" or not path:
        add(True, f"random-init weights of {name} (no checkpoint)")
        return out
    p = Path(path)
    if not p.exists():
        add(False, f"{p} does not exist")
        return out
    try:
        kind = loader.detect_kind(p)
    except FileNotFoundError as ex:
        add(False, str(ex))
        return out
    want_kind = {"w4a16": "awq"}.get(fmt, fmt)
    if kind != want_kind:
        add(False, f"[model] format = {fmt!r} but {p} is a {kind} checkpoint")
        return out
    if (kind == "gguf") != (quant == "gguf") and kind == "gguf":
        add(False, f"a GGUF file needs [model] quant = \"gguf\" (profile says {quant!r})")
    if kind == "nvfp4" and quant != "nvfp4":
        add(False, f"an NVFP4 checkpoint needs [model] quant = \"nvfp4\" (profile says {quant!r})")
    add(True, f"{p} is a {kind} checkpoint")
    # geometry
    spec = None
    try:
        if kind == "gguf":
            f = gguf.GgufFile(p)
            spec = gguf.spec_from_meta(f.meta)
        elif (p / "config.json").exists() and json.loads((p / "config.json").read_text()):
            from ..models.config_json import spec_from_hf_config

            spec = spec_from_hf_config(json.loads((p / "config.json").read_text()))
    except (KeyError, TypeError, ValueError) as ex:
        add(False, f"the checkpoint's model description cannot be read: {ex!r}")
    preset = PRESETS[name]() if name in PRESETS else None
    if spec is not None and preset is not None:
        diff = _geometry_diff(spec, preset)
        add(not diff, "geometry equals " + name if not diff else "geometry differs: " + "; ".join(diff))
    spec = spec or preset
    if spec is None:
        add(False, f"no model description: {name!r} is not a known model and the checkpoint declares none")
        return out
    # tensors
    need = needed_tensors(spec)
    missing, wrong = [], []
    if kind == "gguf":
        for hf, shape in need.items():
            g = loader.gguf_name(hf)
            t = f.tensors.get(g)
            if t is None:
                if hf != "lm_head.weight":
                    missing.append(g)
            elif shape is not None and len(shape) == 2 and tuple(t.shape) != tuple(shape):
                wrong.append(f"{g} {tuple(t.shape)} != {shape}")
    else:
        from .safetensors import SafeDir

        src = SafeDir(p)
        infos = {k: sf.header[k] for sf in src.files.values() for k in sf.keys()}
        for hf, shape in need.items():
            alts = [hf, hf.replace(".weight", ".weight_packed")] if kind == "awq" else [hf]
            hit = next((a for a in alts if a in infos), None)
            if hit is None:
                missing.append(hf)
            elif shape is not None and hit == hf and kind == "safetensors" and tuple(infos[hit]["shape"]) != tuple(shape):
                wrong.append(f"{hf} {tuple(infos[hit]['shape'])} != {shape}")
        if not spec.tied and "lm_head.weight" not in infos:
            out.append(CheckItem(True, "model", "no lm_head.weight: the output head shares the embedding table"))
    add(not missing, f"all {len(need)} tensors present" if not missing else
        f"{len(missing)} tensors missing: " + ", ".join(missing[:6]) + (" ..." if len(missing) > 6 else ""))
    if wrong:
        add(False, "shapes differ from the geometry: " + "; ".join(wrong[:6]))
    limit = int(spec.max_position * max(1.0, yarn_factor))
    add(max_seq <= limit, f"runtime.max_seq {max_seq} within the trained context {spec.max_position}" +
        (f" x YaRN {yarn_factor:g}" if yarn_factor > 1 else "") if max_seq <= limit else
        f"runtime.max_seq {max_seq} exceeds the trained context {spec.max_position}" +
        (f" x YaRN {yarn_factor:g} = {limit}" if yarn_factor > 1 else "; set [model.rope] yarn_factor"))
    return out


def check_draft(kind: str, draft_path: str, target: ModelSpec | None) -> list[CheckItem]:
    out: list[CheckItem] = []
    add = lambda ok, text: out.append(CheckItem(ok, "draft", text))
    if kind == "none":
        return out
    if not draft_path:
        add(True, f"{kind} draft with random-init weights (no draft_path)")
        return out
    p = Path(draft_path)
    if not p.exists():
        add(False, f"{p} does not exist")
        return out
    if kind == "dflash2" and p.suffix == ".gguf":
        from . import dflash_gguf, gguf

        if target is None:
            add(False, "the target model is unknown, the draft cannot be checked against it")
            return out
        try:
            f = gguf.GgufFile(p)
            ds = dflash_gguf.draft_spec(f, target)
            missing = [dflash_gguf.gguf_name(k) for k in dflash_gguf.draft_keys(ds) if dflash_gguf.gguf_name(k) not in f.tensors]
            add(not missing, f"DFlash2 container: {ds.n_layers} layers, taps {list(ds.taps)}, block {ds.block}" if not missing
                else "DFlash2 container lacks " + ", ".join(missing[:6]))
        except (ValueError, KeyError) as ex:
            add(False, str(ex))
        return out
    from .safetensors import SafeDir

    try:
        keys = set(SafeDir(p).keys())
    except FileNotFoundError as ex:
        add(False, str(ex))
        return out
    want = "fc.weight" if kind == "dflash2" else "fc"
    has = any(k == want or k.startswith("fc") for k in keys)
    add(has, f"{kind} draft directory with {len(keys)} tensors" if has else f"{p} holds no {kind} draft tensors (no fc weight)")
    return out


def check_vision(enabled: bool, model_fmt: str, model_path: str, vision_path: str, hidden: int | None) -> list[CheckItem]:
    out: list[CheckItem] = []
    add = lambda ok, text: out.append(CheckItem(ok, "vision", text))
    if not enabled:
        return out
    from . import vision_weights as VW

    try:
        if model_fmt == "gguf" and model_path:
            from . import gguf

            f = gguf.GgufFile(VW.resolve_mmproj(model_path, vision_path or None))
            vs = VW.mmproj_spec(f)
            fits = hidden is None or vs.out_hidden == hidden
            add(fits, f"projector file {f.path.name}: {vs.depth} blocks, hidden {vs.hidden}, output {vs.out_hidden}" if fits else
                f"projector file {f.path.name} outputs {vs.out_hidden} but the text model's hidden size is {hidden}")
            return out
        src_dir = vision_path or model_path
        if not src_dir:
            add(True, "random-init vision tower (no checkpoint)")
            return out
        from .safetensors import SafeDir

        n = sum(1 for k in SafeDir(src_dir).keys() if "visual." in k)
        add(n > 0, f"{n} visual.* tensors in {src_dir}" if n else f"{src_dir} holds no visual.* tensors")
    except (ValueError, FileNotFoundError) as ex:
        add(False, str(ex))
    return out


def check_profile(cfg) -> list[CheckItem]:
    """Every check of a loaded profile (``utils.config.OwlConfig``), in report order."""
    v = cfg.values
    m = v["model"]
    items = check_model(m["path"], m["format"], m["quant"], m["name"], v["runtime"]["max_seq"], v["model.rope"]["yarn_factor"])
    target = PRESETS[m["name"]]() if m["name"] in PRESETS else None
    items += check_draft(v["spec"]["kind"], v["spec"]["draft_path"], target)
    items += check_vision(v["vision"]["enabled"], m["format"], m["path"], v["vision"]["path"], target.hidden if target else None)
    return items
