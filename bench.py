#!/usr/bin/env python
"""Headline benchmark: 27B hybrid decode (output tokens/s) at TP = number of GPUs.

Workload (the reference's headline configuration, random-init weights, synthetic prompt):
27B hybrid (hidden 5120, 64 layers 3 GDN : 1 full attention, SwiGLU 17408, vocab 151936),
AWQ-style int4 W4A16 weights (group 128, asymmetric, fp16 scales / zero points), fp8 e4m3 paged KV
(block 16), batch 1, 2048-token random prompt, greedy decode under CUDA-graph replay.

``python bench.py --gpus N --steps K --warmup W`` (N > 1 under torchrun, one rank per GPU):
prefill the prompt, run W untimed decode steps, then time exactly K decode steps twice:

* ``value`` / ``ms_per_step``: device time of K replays of the self-feeding decode graph (CUDA
  events on the launching stream, barrier + synchronize on both sides, max over ranks);
* ``e2e``: the same K steps through ``Engine.decode_step`` -- every step copies its inputs from
  pinned host memory, replays the graph and reads the sampled token back to the host.

Every decode step streams the full ~14.5 GB of weights, far more than the 126 MB L2, so no L2
flush is needed between timed iterations. ``--impl reference`` reports that the reference
(a Rust workspace) cannot be installed in this environment.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_TOK_S = 48.8   # reference: 27B AWQ W4A16 bare decode on 1x3090 Ti (AGENTS.md:152)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        clocks, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                clocks.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        clocks.sort()
        med = clocks[len(clocks) // 2] if clocks else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(clocks)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result marked invalid)")
    ap.add_argument("--gemv", default="fma", choices=["fma", "dp4a", "tc"],
                    help="W4 decode arm: the half-precision FMA projection with fused norm / residual / activation (fma), the "
                         "integer streaming kernels (dp4a) or the tcgen05 streaming kernel (tc)")
    ap.add_argument("--sp-prefill", type=int, default=-1, choices=[-1, 0, 1],
                    help="N > 1: prefill through the GEMM-fused reduce-scatter / all-gather path (1), the all-reduce path (0), "
                         "or the runner's default (-1)")
    ap.add_argument("--prefill-gemm", default="tcr", choices=["tc", "tcr", "tc8", "tc8r", "baseline"],
                    help="prefill GEMM arm: 16-bit tcgen05 (tc), e4m3 tcgen05 W4A8 (tc8), the same with resident dequantised "
                         "weights (tcr, tc8r), dequant + library GEMM (baseline)")
    ap.add_argument("--head", default="int8", choices=["int8", "bf16"],
                    help="lm_head storage: per-row int8 (W8A16; the reference's default, profiles/full.toml:144 "
                         "head_quant = rtn-int8-row) or bf16")
    ap.add_argument("--sessions", type=int, default=32,
                    help="after the single-stream measurement, run this many concurrent sessions (random prompts of 1k-8k tokens, "
                         "--session-out tokens each) through the serving path and report the aggregate rate under \"extra\" "
                         "(0 = skip)")
    ap.add_argument("--session-out", type=int, default=256)
    ap.add_argument("--comm", default="fused", choices=["nccl", "fused", "push"],
                    help="TP collectives: our symmetric-memory kernels (fused) or the NCCL baseline arm")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "reference is a Rust/CUDA cargo workspace (no setup.py/pyproject, no cargo "
                                         "in the image, no sm_100 arch arm): pip install reports 'not installable'"}))
        return

    import torch

    from owl_engine_b200.engine.core import Engine, EngineConfig
    from owl_engine_b200.models import hybrid as H
    from owl_engine_b200.ops import kernels as K
    from owl_engine_b200.parallel.comm import TpComm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    comm = TpComm.from_env(args.comm, hidden=5120, big_elems=2048 * 5120) if world > 1 else None
    rank = comm.rank if comm else 0
    if comm is None:
        torch.cuda.set_device(0)
    dev = torch.device(f"cuda:{torch.cuda.current_device()}")
    warmup = max(3, args.warmup)
    steps = args.steps

    # pages for the warm-up prompt and the timed prompt side by side, plus the generated tokens
    n_pages = max(1024, 2 * (args.prompt_len + 2 * (warmup + steps) + 64) // 16 + 64)
    n_slots, max_seq = 2, args.prompt_len + 2 * (warmup + steps) + 64
    if args.sessions > 0:        # room for the concurrent-session run that follows the headline measurement
        n_slots = max(2, args.sessions)
        max_seq = max(max_seq, 8192 + args.session_out + 64)
        n_pages = max(n_pages, args.sessions * (8192 + args.session_out + 64) // 16 + 256)
    cfg = EngineConfig(model="qwen3.8-27b", group=128, n_pages=n_pages, n_slots=n_slots, max_seqs=n_slots,
                       max_seq=max_seq, n_layers=args.layers,
                       decode_gemv=args.gemv, prefill_gemm=args.prefill_gemm, lm_head_int8=args.head == "int8")
    eng = Engine(cfg, comm=comm)
    if args.sp_prefill >= 0:
        eng.runner.sp_prefill = bool(args.sp_prefill)
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, eng.spec.vocab, (args.prompt_len,), generator=g).tolist()

    def sync_all():
        if comm:
            comm.barrier()
        torch.cuda.synchronize()

    # ---- prefill (TTFT) -------------------------------------------------------------------
    # An untimed first prompt pays the first-call costs of a fresh process (kernel attributes, scratch allocation, TMA
    # descriptor entry point); the timed prompt is a different random prompt of the same length, so nothing is cached.
    warm_prompt = torch.randint(0, eng.spec.vocab, (args.prompt_len,), generator=g).tolist()
    sid0 = eng.add_sequence(warm_prompt)
    sync_all()
    t0 = time.perf_counter()
    eng.prefill(sid0)
    torch.cuda.synchronize()
    ttft_cold_ms = (time.perf_counter() - t0) * 1e3
    eng.free_sequence(sid0, publish=False)
    sid = eng.add_sequence(prompt)
    sync_all()
    t0 = time.perf_counter()
    eng.prefill(sid)
    torch.cuda.synchronize()
    ttft_ms = (time.perf_counter() - t0) * 1e3
    if comm:
        ttft_ms = comm.max_over_ranks(ttft_ms)
    # the same prompt length on the arm that keeps NO resident dense copy of the weights (dequantise once per call into a
    # shared scratch, then the dense GEMM): what time to first token costs without the extra memory of "tcr" / "tc8r"
    ttft_tc_ms = None
    if args.prefill_gemm in ("tcr", "tc8r"):
        eng.runner.prefill_gemm = "tc"
        p3 = torch.randint(0, eng.spec.vocab, (args.prompt_len,), generator=g).tolist()
        for timed in (False, True):
            s3 = eng.add_sequence(p3 if timed else p3[::-1], reuse=False)
            sync_all()
            t0 = time.perf_counter()
            eng.prefill(s3)
            torch.cuda.synchronize()
            ttft_tc_ms = (time.perf_counter() - t0) * 1e3
            eng.free_sequence(s3, publish=False)
        if comm:
            ttft_tc_ms = comm.max_over_ranks(ttft_tc_ms)
        eng.runner.prefill_gemm = args.prefill_gemm

    # ---- count our kernel launches per decode step ---------------------------------------
    launches = {"n": 0}
    orig_call = K.call

    def counting_call(name, *a):
        launches["n"] += 1
        return orig_call(name, *a)

    K.call = counting_call
    lay = H.StepLayout(1, 1)
    v = eng.runner.views(lay)
    saved = eng.runner.inp.clone()
    v["gslot"].fill_(-1); v["kv_slot"].fill_(-1); v["ctx"].fill_(1); v["bt_row"].zero_()
    eng.runner.step_forward(lay, ctx_hint=eng._ctx_bucket(args.prompt_len + 1), advance=True)
    torch.cuda.synchronize()
    eng.runner.inp.copy_(saved)
    K.call = orig_call
    launches_per_step = launches["n"] + 1   # argmax is two kernels behind one call

    # ---- end-to-end arm: host-fed steps through the public API ---------------------------
    for _ in range(warmup):
        eng.decode_step([sid])
    sync_all()
    itl = []
    h2d0, d2h0 = eng.h2d_bytes, eng.d2h_bytes
    t0 = time.perf_counter()
    for _ in range(steps):
        ts = time.perf_counter()
        eng.decode_step([sid])
        itl.append((time.perf_counter() - ts) * 1e3)
    sync_all()
    e2e_s = time.perf_counter() - t0
    if comm:
        e2e_s = comm.max_over_ranks(e2e_s)
    itl.sort()

    # ---- device-timed arm: self-feeding graph, K replays ----------------------------------
    seq = eng.seqs[sid]
    eng._ensure_pages(seq, seq.n_cached + warmup + steps + 2)
    pos = seq.n_cached
    hi = eng.h_inp_np
    hi[lay.ids] = seq.tokens[-1]
    hi[lay.pos3:lay.pos3 + 3] = pos
    hi[lay.kv_slot] = seq.pages[pos // 16] * 16 + pos % 16
    hi[lay.ctx] = pos + 1
    hi[lay.gslot] = seq.slot
    hi[lay.bt_row] = seq.row
    eng.runner.inp[:lay.size].copy_(eng.h_inp[:lay.size])
    graph = eng.runner.capture(1, 1, ctx_hint=eng._ctx_bucket(pos + warmup + steps + 1), advance=True)
    for _ in range(warmup):
        graph.replay()
    sync_all()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    sync_all()
    dev_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else {}
    if comm:
        dev_ms = comm.max_over_ranks(dev_ms)

    # ---- throughput: concurrent sessions through the serving path (does not change `value`) ---------------------------
    extra = None
    if args.sessions > 0:
        from owl_engine_b200.fixtures.sessions_bench import run_sessions

        eng.free_sequence(sid, publish=False)
        extra = run_sessions(eng, args.sessions, 1024, 8192, args.session_out, max_batch=min(32, args.sessions))
        if comm:
            extra["seconds"] = round(comm.max_over_ranks(extra["seconds"]), 3)
            extra["output_tok_s"] = round(extra["output_tokens"] / extra["seconds"], 1)
            extra["total_tok_s"] = round((extra["output_tokens"] + extra["prompt_tokens"]) / extra["seconds"], 1)
        extra["what"] = (f"{args.sessions} concurrent sessions, random prompts of 1024-8192 tokens, {args.session_out} output tokens "
                         "each, through RunningEngine (admission, chunked prefill, batched decode); host-timed, max over ranks")

    # every bounded-wait status word of the native library (0 = no wait ran out anywhere), worst over the ranks
    status = K.all_status()
    if comm:
        status = {k: int(comm.max_over_ranks(float(abs(v)))) for k, v in status.items()}
    bad_status = {k: v for k, v in status.items() if v}
    if rank == 0:
        ms_per_step = dev_ms / steps
        value = 1000.0 / ms_per_step
        e2e_value = steps / e2e_s
        out = {
            "metric": "27B hybrid output tok/s (box, max over ranks) + p50 TTFT/ITL",
            "value": round(value, 2), "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / BASELINE_TOK_S, 3), "dtype": "bf16 activations / int4 W4A16 weights / fp8 KV",
            "data": "synthetic (random prompt ids, random-init weights)",
            "impl": "ours",
            "config": {"model": "qwen3.8-27b hybrid (64 layers, hidden 5120, vocab 151936)", "global_batch": 1,
                       "seq_len": args.prompt_len, "generated": steps, "parallelism": f"tp{world}",
                       "weights": "int4 g128 asym (W4A16)",
                       "lm_head": "int8 per row, W8A16 (reference default head_quant = rtn-int8-row)" if args.head == "int8" else "bf16", "kv": "fp8 e4m3 paged, block 16",
                       "l2": "inputs larger than L2: every step streams the full weight set "
                             f"({eng.weights.streamed_bytes() / 1e9:.1f} GB per rank)",
                       "comm": comm.mode if world > 1 else "none",
                       "comm_proof": (getattr(comm, "proof", {}).get("ok") if world > 1 else None),
                       "sp_prefill": bool(world > 1 and eng.runner._pipe() is not None), "cuda_graph": True, "decode_gemv": args.gemv,
                       "prefill_gemm": args.prefill_gemm,
                       "resident_copies_gb": round(eng.ledger.by_class().get("resident copies", 0) / 1e9, 2)},
            "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s",
                    "h2d_bytes_per_step": (eng.h2d_bytes - h2d0) // steps,
                    "d2h_bytes_per_step": (eng.d2h_bytes - d2h0) // steps,
                    "p50_itl_ms": round(itl[len(itl) // 2], 4), "ttft_ms": round(ttft_ms, 2),
                    "ttft_first_call_ms": round(ttft_cold_ms, 2),
                    "ttft_ms_without_resident_copies": None if ttft_tc_ms is None else round(ttft_tc_ms, 2)},
            "gpu_launches": launches_per_step * steps,
            "launches_per_step": launches_per_step,
            "clocks": clocks,
            "kernel_status": status,
            "extra": extra,
        }
        if args.layers is not None:
            out["invalid"] = "debug run with fewer layers"
        if bad_status:
            out["invalid"] = f"a bounded wait ran out inside a kernel: {bad_status}"
        print(json.dumps(out))
    if comm:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
