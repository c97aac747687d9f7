"""Memory model: what a profile costs in device memory and how much context it can hold.

``estimate`` splits the declared budget ``V_avail = total * vram_budget - vram_reserve`` into
weights, GDN state rows, graph / workspace reserve and the KV pool, exactly the decomposition
the store's ``MemoryPlan`` enforces at boot; ``solve_max_context`` answers ``context = "max"``.

Reference counterpart: ``crates/shared/src/config/memory.rs`` and ``crates/store/src/budget.rs``.
"""
from __future__ import annotations

from ..models.spec import PRESETS, ModelSpec

B200_HBM_BYTES = 183_359 * (1 << 20)       # nvidia-smi total on a B200
WORKSPACE_RESERVE = 3 << 30                # graphs, prefill workspace, split-KV partials, allocator slack


def weight_bytes(spec: ModelSpec, quant: str, group: int, head_int8: bool) -> int:
    h = spec.hidden
    per_w4 = 0.5 + (4.0 / group)            # nibble + (fp16 scale, fp16 zero) per group
    lin_mlp = 3 * spec.inter * h
    lin_gdn = (spec.conv_dim + spec.value_dim) * h + spec.value_dim * h
    lin_full = (2 * spec.hq * spec.hd + 2 * spec.hkv * spec.hd) * h + spec.hq * spec.hd * h
    params = spec.n_layers * lin_mlp + spec.n_gdn * lin_gdn + spec.n_full * lin_full
    if quant in ("w4a16", "w4a8", "gguf"):
        body = params * per_w4
    elif quant == "nvfp4":
        body = params * (0.5 + 1.0 / 16)
    else:
        body = params * 2
    small = spec.n_gdn * 2 * spec.nv * h * 2
    embed = spec.vocab * h * 2
    head = 0 if spec.tied else spec.vocab * h * (1 if head_int8 else 2)
    return int(body + small + embed + head)


def linear_params(spec: ModelSpec) -> int:
    """Parameters of the quantised projections (what a resident dense copy of the weights duplicates)."""
    h = spec.hidden
    lin_mlp = 3 * spec.inter * h
    lin_gdn = (spec.conv_dim + spec.value_dim) * h + spec.value_dim * h
    lin_full = (2 * spec.hq * spec.hd + 2 * spec.hkv * spec.hd) * h + spec.hq * spec.hd * h
    return spec.n_layers * lin_mlp + spec.n_gdn * lin_gdn + spec.n_full * lin_full


def draft_bytes(kind: str, spec: ModelSpec) -> int:
    """Device memory of the draft model: the MTP head is one full-attention layer plus a [H, 2H] mix in int4 / bf16; the
    DFlash2 draft is five bf16 layers, the tap projection and two selector code books (about 3.8 GB at 27B scale)."""
    h = spec.hidden
    if kind == "mtp":
        layer = (2 * spec.hq * spec.hd + 2 * spec.hkv * spec.hd + spec.hq * spec.hd) * h + 3 * spec.inter * h
        return int(layer * 0.53 + 2 * h * h * 2)
    if kind == "dflash2":
        from ..models.dflash2 import DraftSpec

        d = DraftSpec(hidden=h, vocab=spec.vocab, inter=spec.inter)
        return int(d.params() * 2)
    return 0


VISION_TOWER_BYTES = 900 << 20             # the 27-block tower in bf16 with its padded matrices


def model_spec(cfg) -> ModelSpec:
    """The geometry a profile talks about: the named model when the name is known, else what the checkpoint declares
    (``config.json`` of an HF directory, the metadata of a GGUF file)."""
    import json
    from pathlib import Path

    from .config import ConfigError

    m = cfg.values["model"]
    if m["name"] in PRESETS:
        return PRESETS[m["name"]]()
    p = Path(m["path"]) if m["path"] else None
    try:
        if p is not None and p.is_file() and p.suffix == ".gguf":
            from ..formats import gguf

            return gguf.spec_from_meta(gguf.GgufFile(p).meta)
        if p is not None and (p / "config.json").exists():
            from ..models.config_json import spec_from_hf_config

            return spec_from_hf_config(json.loads((p / "config.json").read_text()))
    except (KeyError, TypeError, ValueError, OSError) as e:
        raise ConfigError(f"model.path = {m['path']!r}: the checkpoint's model description cannot be read ({e!r})") from None
    raise ConfigError(f"model.name = {m['name']!r} is not a known model ({', '.join(sorted(PRESETS))}) and model.path names no "
                      "checkpoint that declares its geometry")


def estimate(cfg) -> dict:
    v = cfg.values
    spec = model_spec(cfg)
    world = max(1, len(v["parallel"]["device"])) if v["parallel"]["mode"] == "tp" else 1
    rspec = spec.sharded(0, world) if world > 1 else spec
    total = B200_HBM_BYTES
    avail = int(total * v["store"]["vram_budget"]) - (v["store"]["vram_reserve_mb"] << 20)
    kv_elem = {"fp8": 1, "int8": 1, "bf16": 2, "f16": 2}[v["store.kv"]["kv_dtype"]]
    w = weight_bytes(rspec, v["model"]["quant"], v["model"]["group"], v["model"]["head_quant"] != "bf16")
    # the prefill arms with resident dense weights keep a second copy of every projection: fp16 (tcr) or e4m3 (tc8r)
    arm = v["kernel"]["prefill_gemm"]
    resident = linear_params(rspec) * {"tcr": 2, "tc8r": 1}.get(arm, 0)
    sp = v["spec"]
    spec_on = sp["kind"] != "none" or sp["lookup"]
    spec_rows = min(v["runtime"]["max_batch"], 8) if spec_on else 1
    # state rows: one per sequence slot, the snapshot rows (at least two), the scratch rows of speculative verify steps
    slots = v["store.gdn"]["gdn_slots"] + max(2, v["store.gdn"]["snap_max"]) + spec_rows
    gdn = slots * rspec.gdn_state_bytes()
    draft = draft_bytes(sp["kind"], spec)                     # the draft models are not sharded
    vision = VISION_TOWER_BYTES if v["vision"]["enabled"] else 0
    kv_per_tok = rspec.kv_bytes_per_token(kv_elem)
    pool = avail - w - resident - gdn - draft - vision - WORKSPACE_RESERVE
    block = v["store"]["block_tokens"]
    pages = max(0, pool // (kv_per_tok * block))
    host = (v["store"]["host_cache_mb"] + v["store"]["snap_host_mb"]) << 20
    return {"model": spec.name, "tp": world, "total_bytes": total, "avail_bytes": avail, "weights_bytes": w,
            "resident_copies_bytes": int(resident), "gdn_state_bytes": gdn, "state_rows": slots, "draft_bytes": draft,
            "vision_bytes": vision, "workspace_reserve_bytes": WORKSPACE_RESERVE, "kv_pool_bytes": max(0, pool),
            "kv_bytes_per_token": kv_per_tok, "kv_pages": int(pages), "kv_tokens": int(pages * block),
            "pinned_host_bytes": host, "disk_bytes": (v["store"]["disk_cache_mb"] + v["store"]["snap_disk_mb"]) << 20,
            "fits": pool > 0 and pages * block >= v["runtime"]["max_seq"],
            "max_seq": v["runtime"]["max_seq"]}


def solve_max_context(cfg) -> int:
    """Largest max_seq (multiple of the block size) one sequence per slot can reach in the pool."""
    e = estimate(cfg)
    block = cfg.values["store"]["block_tokens"]
    per = e["kv_tokens"] // max(1, cfg.values["store.gdn"]["gdn_slots"])
    return max(block, min(per, 1 << 20) // block * block)
