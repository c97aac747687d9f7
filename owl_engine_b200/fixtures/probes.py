"""Communication probes, one rank per GPU (run under ``torchrun --nproc-per-node N``):

* ``ar``    latency of the one-shot all-reduce + residual + RMSNorm kernel over peer memory against the NCCL
            all-reduce followed by the separate norm kernel, for decode-shaped payloads ``[rows, hidden]``;
* ``p2p``   peer copy bandwidth (copy engine) between rank 0 and every other rank;
* ``ab``    the decode benchmark's comm arms side by side (``bench.py --comm fused`` vs ``--comm nccl``).

All times are CUDA-event device times, maximum over ranks.

Reference counterpart: ``tools/fixture`` CUDA probes (AR latency, P2P write / overlap, NCCL AR comparator,
TP A/B script).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

import torch


def _time(fn, iters: int, warmup: int = 5) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3          # microseconds


def probe_ar(hidden: int, rows_list: list[int], iters: int) -> list[dict]:
    import torch.distributed as dist

    from ..ops import kernels as K
    from ..parallel.comm import TpComm

    comm = TpComm.from_env("fused", hidden=hidden, big_elems=hidden * max(rows_list))
    dev = torch.device(f"cuda:{torch.cuda.current_device()}")
    w = torch.zeros(hidden, dtype=torch.bfloat16, device=dev)
    out = []
    for rows in rows_list:
        h = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=dev)
        xn = torch.zeros_like(h)
        part = comm.symm.partial(0)
        part[:rows].normal_()
        fused = _time(lambda: comm.symm.ar_residual_norm(0, h, rows, w, normed=xn, group=128, eps=1e-6), iters)
        buf = torch.randn(rows, hidden, dtype=torch.bfloat16, device=dev)
        def nccl():
            dist.all_reduce(buf)
            K.rmsnorm_pack(h, w, delta=buf, out_h=h, normed=xn, m=rows, k=hidden, group=128)
        lib = _time(nccl, iters)
        out.append({"rows": rows, "bytes": rows * hidden * 2, "fused_us": round(comm.max_over_ranks(fused), 2),
                    "nccl_plus_norm_us": round(comm.max_over_ranks(lib), 2)})
    return out


def probe_p2p(mbytes: int, iters: int) -> list[dict]:
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    out = []
    if rank == 0:
        src = torch.empty(mbytes << 20, dtype=torch.uint8, device="cuda:0")
        for peer in range(1, world):
            dst = torch.empty(mbytes << 20, dtype=torch.uint8, device=f"cuda:{peer}")
            us = _time(lambda: dst.copy_(src, non_blocking=True), iters)
            out.append({"peer": peer, "gb_s": round((mbytes << 20) / us / 1e3, 1)})
    dist.barrier()
    return out


def probe_ab(gpus: int, steps: int) -> list[dict]:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    rows = []
    for arm in ("fused", "nccl"):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
               "--master-port", "29533", os.path.join(root, "bench.py"), "--gpus", str(gpus), "--steps", str(steps), "--comm", arm]
        r = subprocess.run(cmd, capture_output=True, text=True)
        line = [l for l in r.stdout.splitlines() if l.startswith("{")]
        rows.append({"comm": arm, **({k: json.loads(line[-1])[k] for k in ("value", "ms_per_step")} if line else {"error": r.stderr[-300:]})})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="owl-b200-probes")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a1 = sub.add_parser("ar"); a1.add_argument("--hidden", type=int, default=5120); a1.add_argument("--rows", type=int, nargs="+", default=[1, 8, 32]); a1.add_argument("--iters", type=int, default=200)
    a2 = sub.add_parser("p2p"); a2.add_argument("--mbytes", type=int, default=256); a2.add_argument("--iters", type=int, default=20)
    a3 = sub.add_parser("ab"); a3.add_argument("--gpus", type=int, default=2); a3.add_argument("--steps", type=int, default=64)
    a = ap.parse_args(argv)
    rows = probe_ar(a.hidden, a.rows, a.iters) if a.cmd == "ar" else probe_p2p(a.mbytes, a.iters) if a.cmd == "p2p" else probe_ab(a.gpus, a.steps)
    if int(os.environ.get("RANK", "0")) == 0:
        for r in rows:
            print(json.dumps(r))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
