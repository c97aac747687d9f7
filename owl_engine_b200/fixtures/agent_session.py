"""Long-context agent session: one large prompt, then turns that each append new tokens to the parked sequence.

    turn 0      a random prompt of ``--prompt`` tokens is prefilled in chunks (time to first token), ``--gen`` tokens follow
    turn k      ``--append`` new tokens extend the live sequence (only the new tail is prefilled), ``--gen`` tokens follow
    --image-turn / --drop-turn   a ``--patches``-patch image runs through the vision tower and its merged embeddings enter
                the turn's text, padded to page boundaries; a later turn unlinks exactly those pages (leave-gap deletion)
    afterwards  the sequence is published, a second sequence with the same first ``--prompt`` tokens measures the prefix
                hit (blocks adopted, tokens prefilled, time to first token); with a device pool smaller than the session
                (``--kv-gb``) cold blocks have moved to the pinned-host tier and to disk in between and come back here,
                which gives the recall latency.

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
    cfg = EngineConfig(model="qwen3.8-27b", group=128, n_pages=64, n_slots=4, n_snap_rows=4, max_seqs=4, max_seq=total,
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

    turns = []
    prompt = rnd(a.prompt)
    sid = eng.add_sequence(prompt)
    sync()
    t0 = time.perf_counter()
    tok = eng.prefill(sid)
    sync()
    ttft = time.perf_counter() - t0

    def decode(n):
        sync()
        t1 = time.perf_counter()
        for _ in range(n):
            eng.decode_step([sid])
        sync()
        return n / (time.perf_counter() - t1)

    turns.append({"turn": 0, "new_tokens": a.prompt, "ttft_s": round(ttft, 3), "prefill_tok_s": round(a.prompt / ttft, 1),
                  "decode_tok_s": round(decode(a.gen), 1), "ctx": eng.seqs[sid].n_cached})
    img_range = None
    for k in range(1, a.turns + 1):
        seq = eng.seqs[sid]
        new = rnd(a.append)
        images = None
        note = {}
        if k == a.image_turn:
            # pad so that the image's rows start and end on page boundaries of the live sequence
            base = len(seq.tokens)
            lead = (-base) % PAGE
            tail = (-(base + lead + n_img)) % PAGE
            new = rnd(lead) + [pad_id] * n_img + rnd(tail) + new
            images = [(emb, grid, V.fingerprint(b"agent-session-image"))]
            img_range = (base + lead, base + lead + n_img + tail)
            note["image_rows"] = n_img
        if k == a.drop_turn and img_range is not None:
            sync()
            t1 = time.perf_counter()
            removed = eng.drop_ranges(sid, [img_range])
            sync()
            note["dropped_tokens"] = removed
            note["drop_ms"] = round((time.perf_counter() - t1) * 1e3, 3)
        sync()
        t1 = time.perf_counter()
        eng.extend_sequence(sid, new, images=images, image_pad_id=pad_id if images else None)
        sync()
        dt = time.perf_counter() - t1
        turns.append({"turn": k, "new_tokens": len(new), "ttft_s": round(dt, 3), "prefill_tok_s": round(len(new) / dt, 1),
                      "decode_tok_s": round(decode(a.gen), 1), "ctx": eng.seqs[sid].n_cached, **note})
    facts_live = eng.rel.facts()
    eng.free_sequence(sid, publish=True)
    # a second session on the same prefix: adopted blocks, recall from the lower tiers, time to first token
    prompt2 = prompt + rnd(a.append)
    lookups0, hits0, rec0 = eng.prefix_lookups, eng.prefix_hits, eng.rel.recalled
    sync()
    t1 = time.perf_counter()
    sid2 = eng.add_sequence(prompt2)
    sync()
    adopt_s = time.perf_counter() - t1
    reused = eng.seqs[sid2].reused
    t1 = time.perf_counter()
    eng.prefill(sid2)
    sync()
    ttft2 = time.perf_counter() - t1
    recalled = eng.rel.recalled - rec0
    res = {"what": "agent session", "tp": world, "quant": a.quant, "prefill_gemm": a.prefill_gemm, "kv_pool_gb": a.kv_gb,
           "kv_pages": cfg.n_pages, "page_bytes": page_bytes, "vision_tower_ms": round(tower_ms, 1), "turns": turns,
           "tiers_after_session": {k: v for k, v in facts_live.items() if k != "last_verdict"},
           "second_session": {"prompt": len(prompt2), "reused_tokens": reused, "hit_rate": round(reused / len(prompt2), 4),
                              "adopt_s": round(adopt_s, 3), "recalled_blocks": recalled,
                              "recall_ms_per_block": round(adopt_s * 1e3 / recalled, 3) if recalled else None,
                              "ttft_s": round(adopt_s + ttft2, 3), "prefix_hits": eng.prefix_hits - hits0,
                              "lookups": eng.prefix_lookups - lookups0},
           "tiers_final": {k: v for k, v in eng.rel.facts().items() if k != "last_verdict"}}
    status = K.all_status()
    if comm:
        status = {k: int(comm.max_over_ranks(float(abs(v)))) for k, v in status.items()}
    res["kernel_status"] = status
    if rank == 0:
        print(json.dumps(res))
    eng.free_sequence(sid2, publish=False)
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
