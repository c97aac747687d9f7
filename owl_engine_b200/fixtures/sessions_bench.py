"""Concurrent sessions through the serving path: ``n`` turns with random prompts of ``lo..hi`` tokens are submitted at once
to a ``RunningEngine`` (admission, chunked prefill, cross-session batched decode), each generates ``out`` tokens.

``run_sessions`` returns the aggregate output rate (generated tokens of all sessions over the wall time from the first
submit to the last completion, host-timed around a device synchronise on both sides), the prompt rate, and the median
time to the first token. Under tensor parallelism every rank calls it with the same arguments (same seed, same turns):
the ranks' engines step in lockstep and meet in the kernels' collectives.

``python -m owl_engine_b200.fixtures.sessions_bench [--sessions 32] [--lo 1024] [--hi 8192] [--out 256] [--quant w4a16|nvfp4]``
(under ``torchrun`` for more than one GPU) prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def run_sessions(eng, n: int = 32, lo: int = 1024, hi: int = 8192, out: int = 256, max_batch: int = 32, seed: int = 7,
                 breakdown: bool = False, prefill_every: int = 8) -> dict:
    """``breakdown``: time every step kind (begin / prefill / decode) with a device synchronise after each step, which
    attributes the wall time but serialises host and device (the rates of such a run are not the headline)."""
    import queue

    from ..engine.running import RunningEngine, TurnOpts

    re = RunningEngine(eng, max_batch=max_batch, on_full="queue", prefill_every=prefill_every)
    kinds: dict = {}
    if breakdown:
        for kind in ("begin", "prefill", "decode"):
            inner = getattr(re, "_do_" + kind)

            def timed(step, inner=inner, kind=kind):
                torch.cuda.synchronize()
                t1 = time.perf_counter()
                inner(step)
                torch.cuda.synchronize()
                rec = kinds.setdefault(kind, [0, 0.0, 0])
                rec[0] += 1
                rec[1] += time.perf_counter() - t1
                rec[2] += len(step.turns)
            setattr(re, "_do_" + kind, timed)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n,), generator=g).tolist()
    prompts = [torch.randint(0, eng.spec.vocab, (ln,), generator=g).tolist() for ln in lens]
    sinks = [queue.Queue() for _ in prompts]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p, s in zip(prompts, sinks):
        re.submit(p, TurnOpts(max_new=out, ignore_eos=True), sink=s)
    first, done, n_tok = {}, 0, 0
    while done < n:
        if not re.pump():
            break
        now = time.perf_counter()
        for i, s in enumerate(sinks):
            while not s.empty():
                ev = s.get()
                if ev[0] == "token":
                    n_tok += 1
                    first.setdefault(i, now - t0)
                elif ev[0] in ("completed", "failed"):
                    done += 1
                    if ev[0] == "failed":
                        raise RuntimeError(f"session {i} failed: {ev[2]}")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    ttft = sorted(first.values())
    return {"sessions": n, "prompt_tokens": sum(lens), "output_tokens": n_tok, "seconds": round(dt, 3),
            "output_tok_s": round(n_tok / dt, 1), "total_tok_s": round((n_tok + sum(lens)) / dt, 1),
            "ttft_p50_s": round(ttft[len(ttft) // 2], 3) if ttft else None, "max_batch": max_batch,
            "prefix_hits": eng.prefix_hits, "prefill_every": prefill_every,
            **({"steps": {k: {"n": v[0], "ms_total": round(v[1] * 1e3, 1), "ms_avg": round(v[1] * 1e3 / v[0], 2),
                              "turns_avg": round(v[2] / v[0], 1)} for k, v in kinds.items()}} if breakdown else {})}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sessions", type=int, default=32)
    ap.add_argument("--lo", type=int, default=1024)
    ap.add_argument("--hi", type=int, default=8192)
    ap.add_argument("--out", type=int, default=256)
    ap.add_argument("--quant", default="w4a16", choices=["w4a16", "nvfp4", "w4a8"])
    ap.add_argument("--comm", default="fused")
    ap.add_argument("--prefill-gemm", default="tc")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--prefill-every", type=int, default=8, help="decode beats between prefill chunks (8: the latency policy; 1: throughput)")
    ap.add_argument("--breakdown", action="store_true", help="time each step kind (adds a device synchronise per step)")
    a = ap.parse_args()
    from ..engine.core import Engine, EngineConfig
    from ..ops import kernels as K
    from ..parallel.comm import TpComm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    comm = TpComm.from_env(a.comm, hidden=5120, big_elems=2048 * 5120) if world > 1 else None
    if comm is None:
        torch.cuda.set_device(0)
    n_pages = a.sessions * (a.hi + a.out + 64) // 16 + 256
    cfg = EngineConfig(model="qwen3.8-27b", group=128, n_pages=n_pages, n_slots=a.sessions, n_snap_rows=2, max_seqs=a.sessions,
                       max_seq=a.hi + a.out + 64, lm_head_int8=True, prefill_gemm=a.prefill_gemm, n_layers=a.layers,
                       quant="nvfp4" if a.quant == "nvfp4" else "w4a16", act_bits=8 if a.quant == "w4a8" else 15)
    eng = Engine(cfg, comm=comm)
    res = run_sessions(eng, a.sessions, a.lo, a.hi, a.out, max_batch=min(32, a.sessions), breakdown=a.breakdown,
                       prefill_every=a.prefill_every)
    status = K.all_status()
    if comm is not None:
        res["seconds"] = round(comm.max_over_ranks(res["seconds"]), 3)
        res["output_tok_s"] = round(res["output_tokens"] / res["seconds"], 1)
        status = {k: int(comm.max_over_ranks(float(abs(v)))) for k, v in status.items()}
    res.update(tp=world, quant=a.quant, kernel_status=status, comm=(comm.mode if comm else "none"))
    if (comm.rank if comm else 0) == 0:
        print(json.dumps(res))
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
