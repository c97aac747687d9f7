"""Long-context agent session through the serving engine (``RunningEngine`` with parked sessions).

    turn 0      the client sends a random prompt of ``--prompt`` tokens (chunked prefill: time to first token), ``--gen``
                tokens follow; the finished turn parks its sequence (pages + recurrent state row) under the session name
    turn k      the client sends its whole history plus ``--append`` new tokens; the engine recognises the parked sequence,
                prefills only the new tail (the hit rate is cached / prompt tokens), ``--gen`` tokens follow
    --image-turn / --drop-turn   a ``--patches``-patch image runs through the vision tower and its merged embeddings enter
                the turn's text as a droppable segment (padded to page boundaries by the engine); at the drop turn the
                client's history no longer contains it and the engine unlinks exactly those pages (leave-gap deletion)
    afterwards  the session is released (its exact prefix is published), and a second session with the same first
                ``--prompt`` tokens measures the cross-session prefix hit; with a device pool smaller than the session
                (``--kv-gb``) cold blocks have moved to the pinned-host tier and to disk in between and come back here.

Prints one JSON line (rank 0). Under ``torchrun`` every rank runs the same calls on its weight shard.

``python -m owl_engine_b200.fixtures.agent_session --prompt 131072 --turns 8 --append 2048 --gen 32 --kv-gb 16 --quant w4a8``

Reference counterpart: the agent-session gates of ``crates/engine/tests`` (prefix publish / adopt, tier round trips,
``img_evict`` leave-gap) run as one scenario.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time

import torch

PAGE = 16


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompt", type=int, default=131072)
    ap.add_argument("--turns", type=int, default=8)
    ap.add_argument("--append", type=int, default=2048)
    ap.add_argument("--gen", type=int, default=32)
    ap.add_argument("--kv-gb", type=float, default=16.0, help="device KV pool per rank")
    ap.add_argument("--host-gb", type=float, default=8.0)
    ap.add_argument("--disk-gb", type=float, default=16.0)
    ap.add_argument("--quant", default="w4a8", choices=["w4a16", "w4a8", "nvfp4"])
    ap.add_argument("--prefill-gemm", default="tc8r")
    ap.add_argument("--image-turn", type=int, default=2)
    ap.add_argument("--drop-turn", type=int, default=5)
    ap.add_argument("--patches", type=int, default=1024)
    ap.add_argument("--churn", type=int, default=0,
                    help="tokens of an unrelated prompt served between the session's end and the second session: with a device "
                         "pool smaller than both, the first session's published blocks move to the host tier and to disk")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--comm", default="fused")
    a = ap.parse_args()

    from ..engine.core import Engine, EngineConfig
    from ..models import vision as V
    from ..ops import kernels as K
    from ..parallel.comm import TpComm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    comm = TpComm.from_env(a.comm, hidden=5120, big_elems=2048 * 5120) if world > 1 else None
    rank = comm.rank if comm else 0
    if comm is None:
        torch.cuda.set_device(0)

    def sync():
        if comm:
            comm.barrier()
        torch.cuda.synchronize()

    total = a.prompt + a.turns * (a.append + a.gen) + a.gen + 4096
    disk_dir = tempfile.mkdtemp(prefix=f"owl_agent_r{rank}_")
    # bytes of one KV page on this rank: probe a throw-away config through the engine's own plan
    cfg = EngineConfig(model="qwen3.8-27b", group=128, n_pages=64, n_slots=4, n_snap_rows=a.turns + 3, max_seqs=4, max_seq=total,
                       lm_head_int8=True, prefill_gemm=a.prefill_gemm, n_layers=a.layers,
                       quant="nvfp4" if a.quant == "nvfp4" else "w4a16", act_bits=8 if a.quant == "w4a8" else 15,
                       host_cache_mb=int(a.host_gb * 1024), disk_cache_mb=int(a.disk_gb * 1024), disk_dir=disk_dir)
    from ..models.spec import PRESETS

    sp = PRESETS[cfg.model]()
    n_full = sum(1 for i in range(a.layers or sp.n_layers) if (i + 1) % 4 == 0)
    hkv_local = max(1, sp.hkv // world)
    page_bytes = n_full * 2 * hkv_local * sp.hd * PAGE          # fp8: one byte per element
    cfg.n_pages = max(256, int(a.kv_gb * (1 << 30)) // page_bytes)
    eng = Engine(cfg, comm=comm)
    hidden = eng.spec.hidden
    g = torch.Generator().manual_seed(11)
    rnd = lambda n: torch.randint(0, eng.spec.vocab - 8, (n,), generator=g).tolist()
    pad_id = eng.spec.vocab - 1

    # the image: patches -> vision tower -> merged embeddings (patches / 4 rows of the text hidden size)
    side = int(round(a.patches ** 0.5))
    vs = V.tiny_vision(out_hidden=hidden)
    tower = V.VisionTower(vs, V.init_vision_weights(vs, seed=3), device=eng.device, dtype=torch.float32)
    patches = torch.randn(side * side, vs.patch_dim, generator=g).to(eng.device)
    grid = (1, side, side)
    t0 = time.perf_counter()
    emb = tower.forward(patches, grid).to(torch.bfloat16)
    torch.cuda.synchronize()
    tower_ms = (time.perf_counter() - t0) * 1e3
    n_img = emb.shape[0]

    from ..engine.running import RunningEngine, TurnOpts

    re_ = RunningEngine(eng, max_batch=4, park_sessions=True, max_parked=2, evict_pad_id=pad_id - 1)

    def run_turn(tokens, session, images=None, spans=None):
        """Submit the client's full history as one turn of ``session``; returns (generated tokens, facts)."""
        opts = TurnOpts(max_new=a.gen, ignore_eos=True, session=session, images=list(images or []),
                        image_pad_id=pad_id if images else None, evict_spans=list(spans or []))
        sync()
        t0 = time.perf_counter()
        tid = re_.submit(tokens, opts)
        turn = re_.turns[tid]
        out, ttft, t_first, usage = [], None, None, {}
        while not re_.idle():
            if not re_.pump():
                break
            while not turn.sink.empty():
                ev = turn.sink.get()
                if ev[0] == "token":
                    if ttft is None:
                        torch.cuda.synchronize()
                        t_first = time.perf_counter()
                        ttft = t_first - t0
                    out.append(ev[2])
                elif ev[0] == "completed":
                    usage = ev[3]
                elif ev[0] == "failed":
                    raise RuntimeError(ev[2])
        sync()
        dt = time.perf_counter() - (t_first or t0)
        fresh = len(tokens) - usage.get("cached_tokens", 0)
        return out, {"prompt_tokens": len(tokens), "cached_tokens": usage.get("cached_tokens", 0),
                     "hit_rate": round(usage.get("cached_tokens", 0) / len(tokens), 4), "prefilled": fresh,
                     "ttft_s": round(ttft, 3), "prefill_tok_s": round(fresh / ttft, 1),
                     "decode_tok_s": round((len(out) - 1) / dt, 1) if len(out) > 1 and dt > 0 else None}

    turns = []
    prompt = rnd(a.prompt)
    history = list(prompt)
    gen, facts = run_turn(history, "agent")
    turns.append({"turn": 0, **facts})
    history += gen
    images, spans, img_at = [], [], None
    for k in range(1, a.turns + 1):
        note = {}
        new = rnd(a.append)
        if k == a.image_turn:
            img_at = len(history) + len(new) // 2
            new = new[:len(new) // 2] + [pad_id] * n_img + new[len(new) // 2:]
            images = [(emb, grid, V.fingerprint(b"agent-session-image"))]
            spans = [(img_at, img_at + n_img)]
            note["image_rows"] = n_img
        if k == a.drop_turn and img_at is not None:
            # the client drops the screenshot from its history: the server unlinks exactly those pages
            history = history[:img_at] + history[img_at + n_img:]
            images, spans, img_at = [], [], None
            note["client_dropped_rows"] = n_img
        history += new
        drops0 = re_.gap_drops
        gen, facts = run_turn(history, "agent", images, spans)
        history += gen
        turns.append({"turn": k, **facts, **note, "resumed": re_.resumed, "gap_drops": re_.gap_drops - drops0})
    facts_live = eng.rel.facts()
    if "agent" in re_.parked:
        re_._release_parked("agent", publish=True)           # the session ends: its exact prefix becomes content-addressable
    churn = None
    if a.churn > 0:
        _, churn = run_turn(rnd(a.churn), "other")
        if "other" in re_.parked:
            re_._release_parked("other", publish=True)
        churn["tiers"] = {k: v for k, v in eng.rel.facts().items() if k != "last_verdict"}
    # a second session on the same first prompt: adopted blocks, recall from the lower tiers, time to first token
    prompt2 = prompt + rnd(a.append)
    rec0, hits0 = eng.rel.recalled, eng.prefix_hits
    gen2, facts2 = run_turn(prompt2, "agent-2")
    recalled = eng.rel.recalled - rec0
    res = {"what": "agent session through RunningEngine (parked session resume, leave-gap image drop, prefix tree, tiers)",
           "tp": world, "quant": a.quant, "prefill_gemm": a.prefill_gemm, "kv_pool_gb": a.kv_gb,
           "kv_pages": cfg.n_pages, "page_bytes": page_bytes, "vision_tower_ms": round(tower_ms, 1), "turns": turns,
           "tiers_after_session": {k: v for k, v in facts_live.items() if k != "last_verdict"},
           "churn_session": churn,
           "second_session": {**facts2, "recalled_blocks": recalled, "prefix_hits": eng.prefix_hits - hits0},
           "tiers_final": {k: v for k, v in eng.rel.facts().items() if k != "last_verdict"}}
    status = K.all_status()
    if comm:
        status = {k: int(comm.max_over_ranks(float(abs(v)))) for k, v in status.items()}
    res["kernel_status"] = status
    if rank == 0:
        print(json.dumps(res))
    for name in list(re_.parked):
        re_._release_parked(name, publish=False)
    eng.close()
    if comm is not None:
        import torch.distributed as dist

        eng.runner.graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        comm.symm = None
        torch.cuda.synchronize()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
