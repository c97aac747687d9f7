"""Profile / configuration system.

One ledger (``OwlConfig``) built from four layers, later layers win:

1. the schema's own table carries **no defaults**: every key must be supplied by a profile
   (``configs/full.toml`` annotates and supplies all of them),
2. the profile file and its ``extends = [...]`` chain (resolved depth-first, relative to the
   including file, cycles refused),
3. an optional site file (``--site``),
4. ``--set section.key=value`` overrides.

After merging, the *intent layer* (``[intent] model / hardware / goal / context``) derives
low-level keys that the user did not set explicitly; every key remembers where its value came
from (``explain``). Unknown sections or keys, missing keys, wrong types and values outside an
enum are errors -- the server refuses to start. Nothing is read from the environment.

Reference counterpart: ``crates/shared/src/config/{mod,intent,memory,resolve}.rs`` and the key set
of ``configs/full.toml``; ``device`` accepts 0, 2, 4 or 8 entries here (the reference: 0 or 2).
"""
from __future__ import annotations

import copy
import json
import tomllib
from dataclasses import dataclass, field
from pathlib import Path


class ConfigError(ValueError):
    pass


class Enum:
    def __init__(self, *values):
        self.values = values

    def __repr__(self):
        return "one of " + "|".join(map(str, self.values))


class ListOf:
    def __init__(self, elem, lengths=None):
        self.elem, self.lengths = elem, lengths


# section -> key -> type spec (python type, Enum, ListOf)
SCHEMA: dict = {
    "intent": {"model": str, "hardware": str, "goal": Enum("", "latency", "throughput", "context"),
               "context": (int, str)},
    "server": {"bind": str, "request_dump_dir": str, "template_path": str, "template_vars": str,
               "queue_timeout_ms": int, "keepalive_ms": int},
    "runtime": {"admission_on_full": str, "default_max_new": int, "max_new_cap": int, "max_seq": int,
                "prefill_chunk": int, "max_batch": int},
    "parallel": {"mode": Enum("single", "tp", "layer"), "device": ListOf(str, lengths=(0, 1, 2, 4, 8)),
                 "tp_ar": Enum("nccl", "fused", "push", "multimem"), "tp_ar_f8": bool, "tp_comm": Enum("p2p", "nccl", "host"),
                 "tp_vocab_split": bool, "tp_fused_gemm": bool},
    "model": {"name": str, "path": str, "format": Enum("safetensors", "awq", "w4a16", "nvfp4", "gguf", "random"),
              "quant": Enum("bf16", "w4a16", "w4a8", "nvfp4", "gguf"), "group": Enum(32, 128),
              "head_quant": Enum("bf16", "rtn-int8-row"), "embed_quant": Enum("bf16", "int8-row")},
    "model.rope": {"yarn_factor": float, "original_max": int, "beta_fast": float, "beta_slow": float,
                   "attention_factor": float},
    "store": {"prefix_cache": bool, "host_cache_mb": int, "snap_host_mb": int, "disk_cache_mb": int,
              "snap_disk_mb": int, "disk_dir": str, "vram_budget": float, "vram_reserve_mb": int, "no_reclaim": bool,
              "block_tokens": Enum(16, 32), "evict_policy": str},
    "store.kv": {"kv_dtype": Enum("fp8", "int8", "bf16", "f16"), "draft_kv_dtype": Enum("bf16", "fp8")},
    "store.gdn": {"gdn_slots": int, "snap_decode_stride": int, "snap_spec_rollback": bool, "snap_max": int, "snap_msg_min_gap": int,
                  "snap_msg_recent": int, "snap_session_cap": int, "snap_structural_reserve": int},
    "spec": {"depth": int, "draft_path": str, "kind": Enum("none", "mtp", "dflash2"), "lookup": bool, "lookup_nmin": int,
             "lookup_nmax": int, "lookup_nstrong": int, "lookup_agree": int, "mtp_window": int, "mtp_sink": int, "mtp_ring": bool, "adaptive_depth": bool,
             "depth_min": int, "depth_switch_ctx": int, "tp_draft": bool, "degrade_after": int, "probe_every": int, "q_alpha": float,
             "q_floor": float, "force_accept": int},
    "vision": {"enabled": bool, "path": str, "max_pixels": int, "image_evict": bool, "image_evict_pad": str},
    "sampling": {"mode": Enum("greedy", "sampling"), "temp": float, "topk": int, "topp": float, "rep_penalty": float},
    "load": {"verify": bool, "staging_mb": int, "repack": Enum("auto", "device", "cpu"), "dump": bool},
    "kvmem": {"select_decode": bool, "index": bool, "workspace_per_req": int, "select_sink": int, "select_recent": int,
              "select_query_tokens": int, "score_mode": Enum("cosine-max", "dot-max", "dot-mean"), "recall_every": int,
              "gqa_aggregation": Enum("max", "mean")},
    "kernel": {"prefill_gemm": Enum("tc", "tcr", "tc8", "tc8r", "tc4", "baseline"), "decode_arm": Enum("paged"), "gdn_chunked": bool,
               "gdn_fused_decode": bool, "pdl": bool, "attn_splits": int, "selfcheck": bool},
    "probes": {"step_profile": bool, "perf_level": Enum("off", "counters", "host", "gpu"), "debug": bool,
               "step_gate": Enum("off", "sticky", "single"), "step_gate_ms": int, "raw_completion": bool,
               "prompt_dump": bool},
    "cuda": {"graph": bool, "launch_sync": bool, "trace_ring": int, "pinned_segment_mb": int},
    "log": {"level": Enum("error", "warn", "info", "debug", "trace"), "tags_allow": ListOf(str),
            "tags_deny": ListOf(str), "file": str, "max_mb": int, "keep": int, "timestamp": bool},
}
OPTIONAL_SECTIONS = {"intent"}


def _check_type(path: str, value, spec):
    if isinstance(spec, Enum):
        if value not in spec.values:
            raise ConfigError(f"{path} = {value!r}: expected {spec}")
        return
    if isinstance(spec, ListOf):
        if not isinstance(value, list):
            raise ConfigError(f"{path}: expected a list")
        for v in value:
            _check_type(path + "[]", v, spec.elem)
        if spec.lengths is not None and len(value) not in spec.lengths:
            raise ConfigError(f"{path}: {len(value)} entries, allowed {spec.lengths}")
        return
    if isinstance(spec, tuple):
        if not isinstance(value, spec) or isinstance(value, bool):
            raise ConfigError(f"{path} = {value!r}: expected {'/'.join(t.__name__ for t in spec)}")
        return
    if spec is float and isinstance(value, int) and not isinstance(value, bool):
        return
    if spec is int and isinstance(value, bool):
        raise ConfigError(f"{path} = {value!r}: expected int")
    if not isinstance(value, spec):
        raise ConfigError(f"{path} = {value!r}: expected {spec.__name__}")


def _flatten(tree: dict) -> dict:
    """Nested TOML tables -> {"model": {...}, "model.rope": {...}} following the schema's section names."""
    out: dict = {}
    for sec, body in tree.items():
        if not isinstance(body, dict) or (sec not in SCHEMA and not any(s.startswith(sec + ".") for s in SCHEMA)):
            raise ConfigError(f"unknown section or top-level key: {sec}")
        plain = {}
        for k, v in body.items():
            if f"{sec}.{k}" in SCHEMA:
                if not isinstance(v, dict):
                    raise ConfigError(f"[{sec}.{k}] must be a table")
                out[f"{sec}.{k}"] = dict(v)
            else:
                plain[k] = v
        if plain or sec in SCHEMA:
            out.setdefault(sec, {}).update(plain)
    return out


@dataclass
class OwlConfig:
    values: dict = field(default_factory=dict)         # section -> key -> value
    provenance: dict = field(default_factory=dict)     # "section.key" -> [(source, value), ...] oldest first
    files: list = field(default_factory=list)

    def get(self, dotted: str):
        sec, key = dotted.rsplit(".", 1)
        return self.values[sec][key]

    def section(self, name: str) -> dict:
        return self.values[name]

    def explain(self, dotted: str) -> str:
        if dotted not in self.provenance:
            raise ConfigError(f"unknown key {dotted}")
        lines = [f"{dotted} = {self.get(dotted)!r}"]
        for src, val in self.provenance[dotted]:
            lines.append(f"  {val!r:<24} from {src}")
        return "\n".join(lines)

    def to_json(self) -> str:
        return json.dumps(self.values, indent=1, sort_keys=True)

    def to_toml(self) -> str:
        out = []
        for sec in sorted(self.values):
            out.append(f"[{sec}]")
            for k, v in sorted(self.values[sec].items()):
                out.append(f"{k} = {json.dumps(v)}")
            out.append("")
        return "\n".join(out)


def _load_chain(path: Path, seen: tuple, cfg: OwlConfig) -> None:
    path = path.resolve()
    if path in seen:
        raise ConfigError("extends cycle: " + " -> ".join(str(p) for p in seen + (path,)))
    try:
        raw = tomllib.loads(path.read_text())
    except FileNotFoundError:
        raise ConfigError(f"profile not found: {path}") from None
    except tomllib.TOMLDecodeError as e:
        raise ConfigError(f"{path}: {e}") from None
    for ext in raw.pop("extends", []):
        _load_chain(path.parent / ext, seen + (path,), cfg)
    cfg.files.append(str(path))
    for sec, kv in _flatten(raw).items():
        _apply(cfg, sec, kv, str(path))


def _apply(cfg: OwlConfig, sec: str, kv: dict, source: str) -> None:
    if sec not in SCHEMA:
        raise ConfigError(f"{source}: unknown section [{sec}]")
    for k, v in kv.items():
        if k not in SCHEMA[sec]:
            raise ConfigError(f"{source}: unknown key {sec}.{k}")
        cfg.values.setdefault(sec, {})[k] = copy.deepcopy(v)
        cfg.provenance.setdefault(f"{sec}.{k}", []).append((source, copy.deepcopy(v)))


def _parse_set(expr: str):
    if "=" not in expr:
        raise ConfigError(f"--set expects section.key=value, got {expr!r}")
    dotted, raw = expr.split("=", 1)
    if "." not in dotted:
        raise ConfigError(f"--set key must be section.key, got {dotted!r}")
    try:
        val = tomllib.loads(f"v = {raw}")["v"]
    except tomllib.TOMLDecodeError:
        val = raw                      # bare string
    sec, key = dotted.strip().rsplit(".", 1)
    return sec, key, val


# ---- intent layer ---------------------------------------------------------------------------
HARDWARE = {
    "b200x1": {"parallel.mode": "single", "parallel.device": []},
    "b200x2": {"parallel.mode": "tp", "parallel.device": ["0", "1"]},
    "b200x4": {"parallel.mode": "tp", "parallel.device": ["0", "1", "2", "3"]},
    "b200x8": {"parallel.mode": "tp", "parallel.device": [str(i) for i in range(8)]},
}
GOALS = {
    "latency": {"runtime.max_batch": 1, "runtime.prefill_chunk": 2048},
    "throughput": {"runtime.max_batch": 32, "runtime.prefill_chunk": 2048},
    "context": {"runtime.max_batch": 1, "runtime.prefill_chunk": 2048, "store.host_cache_mb": 65536},
}


def _derive_intent(cfg: OwlConfig) -> None:
    intent = cfg.values.get("intent", {})
    derived: dict = {}
    if intent.get("model"):
        derived["model.name"] = intent["model"]
    hw = intent.get("hardware")
    if hw:
        if hw not in HARDWARE:
            raise ConfigError(f"intent.hardware = {hw!r}: known {sorted(HARDWARE)}")
        derived.update(HARDWARE[hw])
    if intent.get("goal"):
        derived.update(GOALS[intent["goal"]])
    ctx = intent.get("context")
    if isinstance(ctx, int) and ctx > 0:
        derived["runtime.max_seq"] = ctx
    for dotted, v in derived.items():
        sec, key = dotted.rsplit(".", 1)
        explicit = [s for s, _ in cfg.provenance.get(dotted, []) if not s.endswith("full.toml")]
        if explicit:
            continue                   # an explicit setting beats a derived one
        _apply(cfg, sec, {key: v}, "derived:intent")


def load(profile: str | Path, sets: list[str] | None = None, site: str | Path | None = None) -> OwlConfig:
    cfg = OwlConfig()
    _load_chain(Path(profile), (), cfg)
    if site:
        _load_chain(Path(site), (), cfg)
    for expr in sets or []:
        sec, key, val = _parse_set(expr)
        _apply(cfg, sec, {key: val}, "--set")
    _derive_intent(cfg)
    validate(cfg)
    if cfg.values.get("intent", {}).get("context") == "max":
        from .memory import solve_max_context

        cfg.values["runtime"]["max_seq"] = solve_max_context(cfg)
        cfg.provenance.setdefault("runtime.max_seq", []).append(("derived:intent.context=max",
                                                                 cfg.values["runtime"]["max_seq"]))
    return cfg


def validate(cfg: OwlConfig) -> None:
    for sec, keys in SCHEMA.items():
        if sec not in cfg.values:
            if sec in OPTIONAL_SECTIONS:
                continue
            raise ConfigError(f"missing section [{sec}] (every key must come from a profile; see configs/full.toml)")
        for k, spec in keys.items():
            if k not in cfg.values[sec]:
                if sec in OPTIONAL_SECTIONS:
                    continue
                raise ConfigError(f"missing key {sec}.{k}")
            _check_type(f"{sec}.{k}", cfg.values[sec][k], spec)
    v = cfg.values
    if v["parallel"]["mode"] == "layer":
        raise ConfigError("parallel.mode = \"layer\" (pipeline split) is reserved and not implemented")
    if v["parallel"]["mode"] == "tp" and len(v["parallel"]["device"]) not in (2, 4, 8):
        raise ConfigError("parallel.mode = \"tp\" needs 2, 4 or 8 entries in parallel.device")
    if v["parallel"]["mode"] == "single" and len(v["parallel"]["device"]) > 1:
        raise ConfigError("parallel.mode = \"single\" takes at most one device")
    if not (0.05 <= v["store"]["vram_budget"] <= 1.0):
        raise ConfigError("store.vram_budget must be a fraction in [0.05, 1.0]")
    if v["runtime"]["prefill_chunk"] % 16 or v["runtime"]["prefill_chunk"] <= 0:
        raise ConfigError("runtime.prefill_chunk must be a positive multiple of 16")
    if v["store.gdn"]["gdn_slots"] < 1:
        raise ConfigError("store.gdn.gdn_slots must be >= 1 (it is the concurrency ceiling)")
    adm = v["runtime"]["admission_on_full"]
    if adm not in ("reject", "queue") and not (adm.startswith("queue:") and adm[6:].isdigit()):
        raise ConfigError("runtime.admission_on_full must be reject | queue | queue:<ms>")
    if v["spec"]["kind"] != "none" and v["spec"]["depth"] < 1:
        raise ConfigError("spec.depth must be >= 1 when a draft head is configured")
    _validate_honoured(v)
    from .memory import model_spec

    model_spec(cfg)            # an unknown model name without a checkpoint that declares the geometry is refused here


def _validate_honoured(v: dict) -> None:
    """Keys whose value this build cannot honour are refused here, never ignored (the reference's loader rule): a profile
    that asks for something that is not built must not start and then behave as if the key were not there."""
    def refuse(cond: bool, msg: str) -> None:
        if cond:
            raise ConfigError(msg)

    st, sp, km, kn = v["store"], v["spec"], v["kvmem"], v["kernel"]
    pol, _, lam = st["evict_policy"].partition(":")
    ok = (pol == "lru" and not lam) or pol == "lrfu"
    if ok and lam:
        try:
            ok = float(lam) >= 0
        except ValueError:
            ok = False
    refuse(not ok, f"store.evict_policy = {st['evict_policy']!r}: expected lru | lrfu | lrfu:<lambda >= 0>")
    refuse(st["snap_disk_mb"] > 0 and not (st["host_cache_mb"] and st["disk_cache_mb"] and st["disk_dir"]),
           "store.snap_disk_mb needs the disk tier: set store.host_cache_mb, store.disk_cache_mb and store.disk_dir")
    refuse(min(st["host_cache_mb"], st["snap_host_mb"], st["disk_cache_mb"], st["snap_disk_mb"]) < 0, "store.*_mb must be >= 0")
    g = v["store.gdn"]
    refuse(g["snap_decode_stride"] < 0 or g["snap_msg_min_gap"] < 0 or g["snap_msg_recent"] < 0 or g["snap_session_cap"] < 0
           or g["snap_structural_reserve"] < 0, "store.gdn.snap_* must be >= 0")
    refuse(v["model"]["embed_quant"] != "bf16", "model.embed_quant = \"int8-row\": the int8 embedding table is not built; use bf16")
    r = v["model.rope"]
    refuse(r["yarn_factor"] < 1.0, "model.rope.yarn_factor must be >= 1.0 (1.0 = off)")
    refuse(r["original_max"] < 0 or r["beta_fast"] <= 0 or r["beta_slow"] <= 0 or r["attention_factor"] <= 0,
           "model.rope: original_max >= 0 and beta_fast, beta_slow, attention_factor > 0")
    refuse(v["store.kv"]["draft_kv_dtype"] == "fp8" and sp["kind"] != "mtp",
           "store.kv.draft_kv_dtype = \"fp8\" applies to the MTP head's KV pool: set spec.kind = \"mtp\" or leave it at bf16")
    refuse(sp["mtp_window"] != 0 or sp["mtp_ring"], "spec.mtp_window / spec.mtp_ring: the windowed MTP attention and its ring "
           "pool are not built; the MTP head attends to the whole context (mtp_window = 0, mtp_ring = false)")
    refuse(sp["tp_draft"], "spec.tp_draft = true: the draft models are not tensor-parallel in this build")
    refuse(sp["q_alpha"] != 1.0 or sp["q_floor"] != 0.0, "spec.q_alpha / spec.q_floor: served speculative rounds accept by greedy "
           "agreement, so a calibration of the draft distribution has nothing to act on; leave them at 1.0 / 0.0")
    refuse(sp["adaptive_depth"] and sp["kind"] != "mtp", "spec.adaptive_depth applies to the MTP head only")
    refuse(sp["depth_min"] < 1 or sp["depth_min"] > 7 or sp["depth"] > 7, "spec.depth and spec.depth_min are at most 7 (and depth_min >= 1)")
    refuse(sp["degrade_after"] < 0 or sp["probe_every"] < 1, "spec.degrade_after >= 0 and spec.probe_every >= 1")
    refuse(sp["force_accept"] > 7, "spec.force_accept is at most 7 (-1 = off)")
    refuse(not (1 <= sp["lookup_nmin"] <= sp["lookup_nmax"]) or sp["lookup_nstrong"] < sp["lookup_nmin"] or sp["lookup_agree"] < 0,
           "spec.lookup_*: 1 <= lookup_nmin <= lookup_nmax, lookup_nstrong >= lookup_nmin, lookup_agree >= 0")
    if km["select_decode"]:
        refuse(km["score_mode"] != "cosine-max", f"kvmem.score_mode = {km['score_mode']!r}: the GPU block scorer implements "
               "cosine-max only")
        refuse(km["gqa_aggregation"] != "max", "kvmem.gqa_aggregation = \"mean\": the GPU block scorer aggregates by max only")
        refuse(km["recall_every"] < 1, "kvmem.recall_every must be >= 1")
        refuse(not (1 <= km["select_query_tokens"] <= 64), "kvmem.select_query_tokens must be in 1..64")
    refuse(not kn["gdn_fused_decode"], "kernel.gdn_fused_decode = false: the unfused one-token GDN path is not built")
    refuse(kn["attn_splits"] < 0 or kn["attn_splits"] > 64, "kernel.attn_splits must be in 0..64 (0 = from the context length)")
    cu = v["cuda"]
    refuse(cu["launch_sync"] and cu["graph"], "cuda.launch_sync = true synchronises after every launch, which a graph capture "
           "forbids: set cuda.graph = false with it")
    refuse(not cu["graph"] and sp["kind"] in ("mtp", "dflash2"), "cuda.graph = false: the draft models' proposal chains exist "
           "only as captured graphs; run them with cuda.graph = true or use lookup drafting")
    refuse(cu["trace_ring"] < 0 or cu["pinned_segment_mb"] < 1, "cuda.trace_ring >= 0 and cuda.pinned_segment_mb >= 1")
    refuse(v["load"]["staging_mb"] < 0, "load.staging_mb must be >= 0 (0 = no bound)")
    lg = v["log"]
    refuse((lg["max_mb"] or lg["keep"]) and not lg["file"], "log.max_mb / log.keep rotate log.file: set log.file")
    refuse(v["probes"]["step_gate_ms"] < 0, "probes.step_gate_ms must be >= 0")


def main_cli(argv: list[str] | None = None) -> int:
    """``-p profile [--set k=v]... [--check] [--print-config [--format json]] [--explain key]``."""
    import argparse

    ap = argparse.ArgumentParser(prog="owl-b200-config")
    ap.add_argument("-p", "--profile", required=True)
    ap.add_argument("--site")
    ap.add_argument("--set", action="append", default=[])
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--print-config", action="store_true")
    ap.add_argument("--format", default="toml", choices=["toml", "json"])
    ap.add_argument("--explain")
    a = ap.parse_args(argv)
    try:
        cfg = load(a.profile, a.set, a.site)
    except ConfigError as e:
        print(f"config error: {e}")
        return 2
    if a.explain:
        print(cfg.explain(a.explain))
    if a.print_config:
        print(cfg.to_json() if a.format == "json" else cfg.to_toml())
    if a.check:
        from .memory import estimate

        print(json.dumps(estimate(cfg), indent=1))
    return 0
