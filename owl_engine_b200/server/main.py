"""Server entry point: ``python -m owl_engine_b200.server.main -p <profile.toml> [--set k=v]...
[--check] [--print-config [--format json]] [--explain key] [--log-level l] [--perf-dump dir]``.

Boot order: load + validate the profile (refuse on any config error), short-circuit for
``--check / --print-config / --explain``, take the GPU lock, start the engine thread (weights:
random-init of the named shape, or a checkpoint directory / GGUF file), then bind the listener.
Exit codes follow the engine's ``ServiceExit`` (0 normal, 1 fatal, 70 panic), 2 for config errors.

Reference counterpart: ``apps/server/src/{main,config}.rs``.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import sys

from ..utils import config as C
from ..utils import log
from ..utils.memory import estimate


def parallel_plan(cfg: C.OwlConfig, env=None) -> dict:
    """``[parallel]`` against the launch environment: which rank this process is, which communicator arm it builds.
    Every key is either honoured or refused here, before anything is allocated (the rule of the reference's profile
    loader: refuse, never ignore). ``mode = "tp"`` needs one process per GPU (``torchrun --nproc-per-node N``)."""
    import os

    env = os.environ if env is None else env
    p = cfg.values["parallel"]
    world, rank = int(env.get("WORLD_SIZE", "1")), int(env.get("RANK", "0"))
    local = int(env.get("LOCAL_RANK", rank))
    if p["mode"] == "layer":
        raise C.ConfigError("parallel.mode = \"layer\" is reserved: layer-split serving is not built")
    if p["mode"] == "single":
        if world > 1:
            raise C.ConfigError(f"parallel.mode = \"single\" but the launcher started {world} ranks; use a tp profile "
                                "or start one process")
        return {"world": 1, "rank": 0, "local": 0, "comm_mode": None}
    want = len(p["device"]) or world
    if world == 1:
        raise C.ConfigError(f"parallel.mode = \"tp\" serves with one process per GPU: start it as "
                            f"python -m torch.distributed.run --nproc-per-node {max(want, 2)} --master-addr 127.0.0.1 "
                            "-m owl_engine_b200.server.main -p <profile>")
    if want != world:
        raise C.ConfigError(f"parallel.device names {want} GPUs but the launcher started {world} ranks")
    if world not in (2, 4, 8):
        raise C.ConfigError(f"tensor parallelism is built for 2, 4 or 8 ranks, not {world}")
    if p["tp_ar_f8"]:
        raise C.ConfigError("parallel.tp_ar_f8 = true: the e4m3-payload all-reduce is not built; set it to false")
    if p["tp_comm"] == "host":
        comm_mode = "host"          # staged through pinned host memory (GPU pairs without peer access)
    elif p["tp_comm"] == "nccl" or p["tp_ar"] == "nccl":
        comm_mode = "nccl"
    else:
        comm_mode = "push" if p["tp_ar"] == "push" else "fused"
    return {"world": world, "rank": rank, "local": local, "comm_mode": comm_mode, "multimem": p["tp_ar"] == "multimem",
            "vocab_split": bool(p["tp_vocab_split"]), "fused_gemm": bool(p["tp_fused_gemm"])}


def open_tokenizer(cfg: C.OwlConfig):
    """The profile's tokenizer: the checkpoint's ``tokenizer.json`` when the model path has one, else the byte-level one."""
    from ..engine.tokenizer import ByteTokenizer, HfTokenizer

    v = cfg.values
    path = v["model"]["path"]
    try:
        return HfTokenizer(path) if path and v["model"]["format"] != "gguf" else ByteTokenizer()
    except Exception:   # noqa: BLE001  (no tokenizer files next to the weights)
        return ByteTokenizer()


def load_vision_checkpoint(model_format: str, model_path: str, vision_path: str, default_spec, over: dict):
    """(spec, weights) of the vision tower. A GGUF language model takes its tower from the projector file next to it
    (``mmproj*.gguf``, or the file ``[vision] path`` names); otherwise ``[vision] path`` (or the model directory) is an HF
    safetensors directory whose ``[model.]visual.*`` tensors and ``config.json`` ``vision_config`` describe it. Without any
    checkpoint the tower is random-init with the default geometry (``weights = None``)."""
    import json as _json
    import os

    from ..formats import vision_weights as VW

    if model_format == "gguf" and model_path:
        return VW.load_mmproj(model_path, vision_path or None, **over)
    src_dir = vision_path or (model_path if model_path and os.path.isdir(model_path) else "")
    if not src_dir:
        return default_spec, None
    from ..formats.safetensors import SafeDir

    src = SafeDir(src_dir)
    w = VW.from_hf({k: src.get(k) for k in src.keys() if "visual." in k})
    if not w:
        raise VW.VisionLoadError(f"{src_dir}: no visual.* tensors (vision is enabled but this checkpoint has no tower)")
    spec = default_spec
    cfg_json = os.path.join(src_dir, "config.json")
    if os.path.exists(cfg_json):
        vc = _json.load(open(cfg_json)).get("vision_config")
        if vc:
            spec = VW.spec_from_hf(vc, **over)
    VW.check_complete(spec, w)
    return spec, w


def evict_pad_token(cfg: C.OwlConfig, tok) -> int:
    """``[vision] image_evict_pad``: the filler that page-aligns a droppable segment must be exactly one token. An empty
    setting tries an ideographic full stop, a space, then a newline."""
    text = cfg.values["vision"]["image_evict_pad"]
    for cand in ([text] if text else ["\u3002", " ", "\n"]):
        ids = tok.encode(cand)
        if len(ids) == 1:
            return int(ids[0])
    raise C.ConfigError(f"vision.image_evict_pad = {text!r} is {len(tok.encode(text))} tokens for this tokenizer; it must be exactly one")


def apply_process_switches(cfg: C.OwlConfig) -> None:
    """Profile keys that switch process-wide behaviour of the kernel launcher and the debugging aids."""
    from ..ops import kernels as K
    from ..utils.stepgate import GATE

    v = cfg.values
    K.LAUNCH_SYNC = bool(v["cuda"]["launch_sync"])
    K.set_trace_ring(v["cuda"]["trace_ring"])
    if not v["kernel"]["gdn_chunked"]:
        K.GDN_CHUNKED_FROM = 0            # prefill runs the serial / column-split recurrence instead of the chunked form
    GATE.configure(v["probes"]["step_gate"], v["probes"]["step_gate_ms"])


def boot_facts(eng, v: dict, plan: dict) -> list[str]:
    """What an operator wants to see once at boot: the memory governor's arithmetic, the kernel arms in use, the pools."""
    led, r, c = eng.ledger, eng.runner, eng.cfg
    by = {k: f"{b / 2**30:.2f} GiB" for k, b in sorted(led.by_class().items(), key=lambda kv: -kv[1])}
    lines = [f"[vram-gov] total {led._total() / 2**30:.1f} GiB x budget {led.budget_frac:.2f} - reserve {led.reserve >> 20} MiB = "
             f"{led.avail / 2**30:.2f} GiB; in use {led.used() / 2**30:.2f} GiB {by}",
             f"[kernel-env] sm_100a; decode projection arm {getattr(r, 'decode_gemv', '?')}, prefill GEMM {c.prefill_gemm}, "
             f"graphs {'on' if c.cuda_graph else 'off'}, dependent launch {'on' if c.pdl else 'off'}, kv {c.kv_dtype}, "
             f"weights {c.quant} g{c.group}",
             f"[pools] {c.n_pages} KV pages of 16 tokens ({c.n_pages * 16} tokens), {c.n_slots} sequence slots, "
             f"{c.n_snap_rows} snapshot rows, host tier {c.host_cache_mb} MiB, disk tier {c.disk_cache_mb} MiB, "
             f"snapshot tiers {c.snap_host_mb} / {c.snap_disk_mb} MiB"]
    if plan.get("world", 1) > 1:
        comm = getattr(eng, "comm", None)
        lines.append(f"[parallel] rank {plan['rank']} of {plan['world']}, collectives {getattr(comm, 'mode', '?')}, "
                     f"vocabulary split {'on' if c.vocab_split else 'off'}, fused prefill GEMM + collective "
                     f"{'on' if getattr(r, 'sp_prefill', False) else 'off'}")
    return lines


def build_engine_factory(cfg: C.OwlConfig, plan: dict | None = None, msg_open_ids: tuple = ()):
    v = cfg.values
    plan = plan or {"world": 1, "rank": 0, "local": 0, "comm_mode": None}

    def build():
        import torch

        from ..engine.core import Engine, EngineConfig
        from ..models.spec import PRESETS

        comm = None
        if plan["world"] > 1:
            from ..parallel.comm import TpComm

            hidden = PRESETS[v["model"]["name"]]().hidden if v["model"]["name"] in PRESETS else 5120
            comm = TpComm.from_env(plan["comm_mode"], hidden=hidden, big_elems=v["runtime"]["prefill_chunk"] * hidden,
                                   use_multimem=plan["multimem"])
        else:
            torch.cuda.set_device(plan["local"])
        dev = torch.device(f"cuda:{torch.cuda.current_device()}")
        est = estimate(cfg)
        km, st, sg, rp = v["kvmem"], v["store"], v["store.gdn"], v["model.rope"]
        ecfg = EngineConfig(model=v["model"]["name"], group=v["model"]["group"],
                            quant="nvfp4" if v["model"]["quant"] == "nvfp4" else "w4a16",
                            act_bits=8 if v["model"]["quant"] == "w4a8" else 15,
                            kvmem_budget=km["workspace_per_req"] if km["select_decode"] else 0,
                            kvmem_sink=km["select_sink"], kvmem_recent=km["select_recent"],
                            lm_head_int8=v["model"]["head_quant"] != "bf16",
                            n_pages=min(est["kv_pages"], max(1024, (v["runtime"]["max_seq"] // 16 + 64) * v["store.gdn"]["gdn_slots"])),
                            n_slots=v["store.gdn"]["gdn_slots"], n_snap_rows=max(2, v["store.gdn"]["snap_max"]),
                            max_seqs=max(v["store.gdn"]["gdn_slots"], v["runtime"]["max_batch"]), max_seq=v["runtime"]["max_seq"],
                            prefill_chunk=v["runtime"]["prefill_chunk"], pdl=v["kernel"]["pdl"],
                            prefill_gemm=v["kernel"]["prefill_gemm"], host_cache_mb=v["store"]["host_cache_mb"],
                            disk_cache_mb=v["store"]["disk_cache_mb"], disk_dir=v["store"]["disk_dir"],
                            kv_dtype=v["store.kv"]["kv_dtype"], vocab_split=plan.get("vocab_split", True),
                            prefix_cache=st["prefix_cache"], no_reclaim=st["no_reclaim"], evict_policy=st["evict_policy"],
                            snap_host_mb=st["snap_host_mb"], snap_disk_mb=st["snap_disk_mb"],
                            msg_open_ids=tuple(msg_open_ids) if st["prefix_cache"] and sg["snap_max"] > 0 else (),
                            snap_msg_min_gap=sg["snap_msg_min_gap"], snap_msg_recent=sg["snap_msg_recent"],
                            snap_decode_stride=sg["snap_decode_stride"] if st["prefix_cache"] and sg["snap_max"] > 0 else 0,
                            snap_spec_rollback=sg["snap_spec_rollback"], snap_session_cap=sg["snap_session_cap"], snap_structural_reserve=sg["snap_structural_reserve"],
                            attn_splits=v["kernel"]["attn_splits"], cuda_graph=v["cuda"]["graph"],
                            pinned_segment_mb=v["cuda"]["pinned_segment_mb"],
                            rope_yarn=(rp["yarn_factor"], rp["original_max"], rp["beta_fast"], rp["beta_slow"],
                                       rp["attention_factor"]) if rp["yarn_factor"] > 1.0 else None,
                            kvmem_query_tokens=km["select_query_tokens"], kvmem_recall_every=km["recall_every"],
                            # speculative rounds of several decoding turns run as one batched verify: one scratch state row each
                            spec_rows=min(v["runtime"]["max_batch"], 8) if (v["spec"]["kind"] != "none" or v["spec"]["lookup"]) else 1)
        if v["kernel"]["selfcheck"]:
            from ..ops import selfcheck

            selfcheck.assert_ok(dev)       # refuse to serve on a build whose kernels disagree with the host oracles
        if v["model"]["format"] == "random" or not v["model"]["path"]:
            eng = Engine(ecfg, comm=comm)
        else:
            from ..formats.loader import load_model

            spec, weights = load_model(v["model"]["path"], dev, spec=PRESETS.get(v["model"]["name"], lambda: None)(),
                                       rank=plan["rank"], world=plan["world"], group=v["model"]["group"],
                                       lm_head_int8=ecfg.lm_head_int8, vocab_split=plan.get("vocab_split", True),
                                       verify=v["load"]["verify"], dump=v["load"]["dump"], staging_mb=v["load"]["staging_mb"],
                                       repack=v["load"]["repack"])
            eng = Engine(ecfg, spec=spec, weights=weights, comm=comm)
        if comm is not None:
            eng.runner.sp_prefill = plan["fused_gemm"]
        if v["cuda"]["graph"] and comm is None:
            # single-GPU profiles capture their graphs at boot; tensor-parallel ranks keep capturing a shape at its first
            # use, in lockstep through the mirrored step calls (a capture's warm-up step runs the collectives)
            from ..engine.graph_fleet import GraphFleet

            sp = v["spec"]
            spec_on = sp["kind"] != "none" or sp["lookup"]
            buckets, bk = [], 512             # the context buckets a step can fall into (`Engine._ctx_bucket`)
            while bk < 2 * v["runtime"]["max_seq"]:
                buckets.append(bk)
                bk *= 2
            fleet = GraphFleet(eng, max_batch=v["runtime"]["max_batch"], spec_depths=(max(1, min(7, sp["depth"] or 3)),) if spec_on else (),
                               spec_rows=ecfg.spec_rows, ctx_buckets=tuple(buckets))
            rep = fleet.assemble()
            eng.graph_fleet = fleet
            log.info("boot.graphs", f"{rep['states']} in {rep['capture_ms']:.0f} ms, {rep['bytes'] >> 20} MiB")
        try:
            for line in boot_facts(eng, v, plan):
                log.info("boot", line)
        except Exception as ex:   # noqa: BLE001  (a report line must never cost the boot)
            log.warn("boot", f"boot facts unavailable: {ex!r}")
        if comm is not None and plan["rank"] == 0:
            from ..engine.tp_serve import MirroredEngine, leader_ring

            return MirroredEngine(eng, leader_ring(plan["world"]))
        return eng
    return build


def build_spec_factory(cfg: C.OwlConfig):
    """``[spec]`` section -> a factory ``engine -> SpecRunner`` (None when speculative decoding is off)."""
    sp = cfg.values["spec"]
    if sp["kind"] == "none" and not sp["lookup"]:
        return None
    def make(engine):
        from ..engine.spec import LookupDraft, MtpDraft, SpecRunner
        from ..models.mtp import MtpHead

        lookup = LookupDraft(sp["lookup_nmin"], sp["lookup_nmax"], sp["lookup_nstrong"], sp["lookup_agree"]) if sp["lookup"] else None
        if sp["kind"] in ("mtp", "dflash2") and getattr(engine, "comm", None) is not None:
            # the draft models are not tensor-parallel: with them in the loop a forced-acceptance run at 4 ranks did not
            # reproduce plain decoding, so the profile is refused instead of served wrong (lookup drafting works at any size)
            raise ValueError(f"[spec] kind = {sp['kind']!r} is not available under tensor parallelism; use lookup drafting "
                             "or serve the profile on one GPU")
        if sp["kind"] == "mtp":
            weights = None
            if sp["draft_path"]:
                from ..formats.safetensors import SafeDir

                src = SafeDir(sp["draft_path"])
                weights = {k: src.get(k) for k in src.keys()}
            draft = MtpDraft(MtpHead(engine.runner, weights=weights, kv_dtype=cfg.values["store.kv"]["draft_kv_dtype"]), lookup)
        elif sp["kind"] == "dflash2":
            from ..engine.spec import DFlash2Draft
            from ..models import dflash2 as D

            ts = engine.spec
            n = ts.n_layers
            taps = D.DraftSpec.taps if n >= 62 else tuple(sorted({max(0, n * (2 * i + 1) // 10 - 1) for i in range(5)}))
            dspec = D.DraftSpec(hidden=ts.hidden, vocab=ts.vocab, inter=ts.inter, taps=taps, mask_token_id=ts.vocab - 1,
                                rope_theta=ts.rope_theta)
            if sp["draft_path"].endswith(".gguf"):
                from ..formats import dflash_gguf

                dspec, dw = dflash_gguf.load_draft(sp["draft_path"], ts, engine.device)     # facts from the file's dflash.* keys
            elif sp["draft_path"]:
                from ..formats.safetensors import SafeDir

                src = SafeDir(sp["draft_path"])
                dw = D.weights_from_dense(dspec, {k: src.get(k) for k in src.keys()}, engine.device)
            else:
                dw = D.random_weights(dspec, engine.device)
            head = D.DFlash2(dspec, dw, engine.weights.embed, engine.weights.lm_head, engine.device)
            draft = DFlash2Draft(head, engine.runner, lookup)
        else:
            draft = lookup
        return SpecRunner(draft, depth=max(1, min(7, sp["depth"] or 3)),
                          depth_min=sp["depth_min"] if sp["adaptive_depth"] else None, switch_ctx=sp["depth_switch_ctx"],
                          degrade_after=sp["degrade_after"], probe_every=sp["probe_every"], force_accept=sp["force_accept"])
    return make


def _leave_group(engine) -> None:
    """End of a tensor-parallel rank: drop the captured graphs and the symmetric workspace, then leave the process group
    together with the other ranks (no rank exits while a peer may still touch its memory)."""
    comm = getattr(engine, "comm", None)
    if comm is None:
        return
    import torch
    import torch.distributed as dist

    engine.runner.graphs.clear()
    torch.cuda.synchronize()
    try:
        comm.barrier()
    except Exception:    # noqa: BLE001  (a peer that already died cannot be waited for)
        pass
    comm.symm = None
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.destroy_process_group()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="owl-b200-server")
    ap.add_argument("-p", "--profile", required=True)
    ap.add_argument("--site")
    ap.add_argument("--set", action="append", default=[])
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--print-config", action="store_true")
    ap.add_argument("--format", default="toml", choices=["toml", "json"])
    ap.add_argument("--explain")
    ap.add_argument("--log-level")
    ap.add_argument("--perf-dump")
    a = ap.parse_args(argv)
    try:
        cfg = C.load(a.profile, a.set, a.site)
    except C.ConfigError as e:
        print(f"config error: {e}", file=sys.stderr)
        return 2
    if a.explain:
        print(cfg.explain(a.explain))
    if a.print_config:
        print(cfg.to_json() if a.format == "json" else cfg.to_toml())
    if a.check:
        from ..formats.preflight import check_profile

        print(json.dumps(estimate(cfg), indent=1))
        items = check_profile(cfg)
        for it in items:
            print(it.line())
        if not all(it.ok for it in items):
            return 1
    if a.explain or a.print_config or a.check:
        return 0
    try:
        plan = parallel_plan(cfg)
    except C.ConfigError as e:
        print(f"config error: {e}", file=sys.stderr)
        return 2
    lv = cfg.values["log"]
    log.LOG.configure(a.log_level or lv["level"], lv["tags_allow"], lv["tags_deny"], lv["timestamp"], path=lv["file"] or None,
                      max_mb=lv["max_mb"], keep=lv["keep"])
    from ..engine.sampler import SamplingParams
    from ..engine.service import EngineService
    from ..utils.metrics import METRICS
    from .chat_tpl import ChatTemplate
    from .http import App, serve

    METRICS.set_level(cfg.values["probes"]["perf_level"])
    v = cfg.values
    apply_process_switches(cfg)
    tok = open_tokenizer(cfg)
    try:
        pad_id = evict_pad_token(cfg, tok) if v["vision"]["image_evict"] else 0
    except C.ConfigError as e:
        print(f"config error: {e}", file=sys.stderr)
        return 2
    # the chat format's message-open marker: where conversations fork, so where recurrent-state snapshots are worth taking
    msg_open_ids = tuple(tok.encode("<|im_start|>"))
    if plan["rank"] > 0:
        # follower rank of a tensor-parallel job: no listener, no scheduler; apply the leader's step descriptors
        from ..engine.tp_serve import follower_loop, follower_ring

        engine = build_engine_factory(cfg, plan, msg_open_ids)()
        make_spec = build_spec_factory(cfg)
        spec_runner = make_spec(engine) if make_spec else None
        ring = follower_ring(plan["rank"])
        n = follower_loop(engine, ring, spec_runner)
        log.info("tp.follower", f"rank {plan['rank']}: applied {n} descriptors, leaving")
        ring.free()
        _leave_group(engine)
        return 0
    svc = EngineService(build_engine_factory(cfg, plan, msg_open_ids), max_batch=v["runtime"]["max_batch"],
                        on_full=v["runtime"]["admission_on_full"], spec_runner=build_spec_factory(cfg),
                        running_kw={"park_sessions": bool(v["vision"]["image_evict"]), "max_parked": max(1, v["store.gdn"]["gdn_slots"] // 2),
                                    "evict_pad_id": pad_id, "step_profile": bool(v["probes"]["step_profile"]),
                                    # requests that name no session continue the parked conversation whose prompt they repeat
                                    "auto_sessions": bool(v["vision"]["image_evict"])})
    client = svc.boot()
    vision = None
    if v["vision"]["enabled"]:
        import torch

        from ..models.spec import PRESETS
        from ..models.vision import VisionSpec
        from .http import Vision

        hidden = PRESETS[v["model"]["name"]]().hidden if v["model"]["name"] in PRESETS else 5120
        over = {"max_pixels": v["vision"]["max_pixels"]} if v["vision"]["max_pixels"] else {}
        vspec, vweights = VisionSpec(out_hidden=hidden, **over), None
        try:
            vspec, vweights = load_vision_checkpoint(v["model"]["format"], v["model"]["path"], v["vision"]["path"], vspec, over)
        except ValueError as e:
            print(f"config error: {e}", file=sys.stderr)
            return 2
        # the tower runs on the package's own kernels (csrc/vision.cu + the dense tcgen05 GEMM); the eager PyTorch tower is its
        # test oracle
        from ..models.vision import VisionTowerKernels

        vision = Vision(VisionTowerKernels(vspec, vweights, device=f"cuda:{torch.cuda.current_device()}"),
                        getattr(tok, "image_pad_id", None) or 0)
    s = v["sampling"]
    app = App(client, tok, v["model"]["name"], ChatTemplate(v["server"]["template_path"], v["server"]["template_vars"]),
              SamplingParams(s["mode"], s["temp"], s["topk"], s["topp"], s["rep_penalty"]), v["runtime"]["default_max_new"],
              v["runtime"]["max_new_cap"], v["server"]["queue_timeout_ms"], v["server"]["keepalive_ms"],
              max_concurrent=v["store.gdn"]["gdn_slots"], vision=vision, request_dump_dir=v["server"]["request_dump_dir"],
              prompt_dump=v["probes"]["prompt_dump"], raw_completion=v["probes"]["raw_completion"])
    host, _, port = v["server"]["bind"].rpartition(":")

    async def run():
        server = await serve(app, host or "0.0.0.0", int(port))
        async with server:
            while svc.exit is None and not app.stop.is_set():
                await asyncio.sleep(0.2)

    try:
        asyncio.run(run())
    except KeyboardInterrupt:
        pass
    ex = svc.shutdown()
    if svc.re is not None:
        _leave_group(svc.re.e)
    if a.perf_dump:
        import os
        os.makedirs(a.perf_dump, exist_ok=True)
        open(os.path.join(a.perf_dump, "perf.json"), "w").write(METRICS.dump_json())
        open(os.path.join(a.perf_dump, "perf.csv"), "w").write(METRICS.dump_csv())
    return ex.code


if __name__ == "__main__":
    sys.exit(main())
