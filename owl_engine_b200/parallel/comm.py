"""Tensor-parallel communicator of one rank.

Two arms, selected per call site by ``mode``:

* ``"nccl"``  -- the baseline: ``torch.distributed`` all-reduce (NCCL over NVLink / NVSwitch),
  capturable in CUDA graphs, followed by a separate residual add.
* ``"push"``  -- ``"fused"`` plus the GEMV-fused transfer for decode: the row-parallel GEMV's epilogue writes
  its partial sums into every rank's slot buffer over NVLink (peer stores, tile by tile while the matrix
  streams) and the consumer kernel reduces local memory only (``csrc/gemv.cu`` EPI_PUSH +
  ``owl_push_residual_norm``);
* ``"host"``  -- the fallback for GPU pairs that may not map each other's memory (``parallel/peer.py``): payloads
  cross through pinned host memory and a ``gloo`` all-reduce; not capturable, the runner steps eagerly;
* ``"fused"`` -- the product path: hand-written kernels over symmetric (peer-mapped) memory
  (``parallel/symm.py`` + ``csrc/comm.cu``): one-shot all-reduce fused with the residual add for
  decode-size payloads, reduce-scatter / all-gather fused into the GEMM epilogue / prologue for
  prefill-size payloads.

Reference counterpart: the in-house 2-rank all-reduce (``crates/backends/cuda/src/comm/ar.rs``,
``crates/kernels/cu/comm/*.cu``) injected after every row-parallel node
(``crates/models/src/interpreters/eval.rs:1154-1419``). The reference is world = 2 only and has
no GEMM/collective fusion.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


class TpComm:
    def __init__(self, rank: int, world: int, device, mode: str = "nccl", group=None, hidden: int = 5120,
                 big_elems: int = 2048 * 5120, use_multimem: bool = False):
        self.rank, self.world, self.device, self.mode = rank, world, device, mode
        self.group = group
        self.symm = None
        self.relay = None
        self.capturable = mode != "host"
        if mode == "host" and world > 1:
            from .peer import HostRelay

            self.relay = HostRelay()
        if mode in ("fused", "push") and world > 1:
            from .symm import SymmetricWorkspace

            self.symm = SymmetricWorkspace(rank, world, device, group, hidden=hidden, big_elems=big_elems,
                                           use_multimem=use_multimem)

    @classmethod
    def from_env(cls, mode: str = "nccl", **kw) -> "TpComm | None":
        """Build from torchrun's environment (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*)."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world == 1:
            return None
        rank = int(os.environ["RANK"])
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        prove = kw.pop("prove", True)
        comm = cls(rank, world, torch.device(f"cuda:{local}"), mode, **kw)
        if prove:
            comm.self_proof()
        return comm

    def self_proof(self, rows: int = 4, prefill_rows: int = 256) -> dict:
        """Post-assembly proof of the hand-written collectives against the library ones, on random data: the one-shot
        all-reduce + residual + norm of the decode path, the in-place all-reduce of prefill-size payloads, and the fused
        GEMM + reduce-scatter -> sum + norm + all-gather -> GEMM pipeline. Every rank must agree and every status word must
        be clean; otherwise ALL ranks drop to the library arm (``mode = "nccl"``) before a model is built on top, so a world
        size or topology the kernels were not proven on costs speed, not correctness. Returns the facts it measured.
        (Reference counterpart: the produced == consumed self-proof after staging assembly,
        ``crates/backends/cuda/src/comm/ar.rs``.)"""
        facts = {"mode": self.mode, "world": self.world, "ok": True}
        s = self.symm
        if s is None:
            return facts
        from ..ops import gemm_tc, kernels as K

        dev, H = self.device, s.hidden

        def rnd(*shape, seed, scale=1.0):
            g = torch.Generator(device=dev).manual_seed(seed)
            return torch.randn(*shape, device=dev, generator=g) * scale

        def rel(a, b):
            return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6))

        def nccl_sum(x):
            y = x.float().clone()
            dist.all_reduce(y, group=self.group)
            return y

        try:
            # decode-size: partial sums in the symmetric buffer -> h += sum, normalised rows out
            for which in (0, 1):
                part = rnd(rows, H, seed=100 + which + 10 * self.rank).bfloat16()
                h = rnd(rows, H, seed=7 + which).bfloat16()                       # replicated residual stream
                nw = rnd(H, seed=9, scale=0.1).bfloat16()
                want = h.float() + nccl_sum(part)
                s.partial(which)[:rows].copy_(part)
                xn = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)
                s.ar_residual_norm(which, h, rows, nw, normed=xn)
                facts[f"ar_norm_{which}"] = rel(h, want)
                wn = want * torch.rsqrt(want.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())
                facts[f"ar_norm_{which}_normed"] = rel(xn, wn)
            # prefill-size in-place all-reduce
            n = min(s.big_elems // H, 64)
            y = rnd(n, H, seed=300 + self.rank).bfloat16()
            want = nccl_sum(y)
            s.allreduce_(y)
            facts["ar_inplace"] = rel(y, want)
            pipe = s.prefill
            if pipe is not None and pipe.rows >= prefill_rows:
                t, kd = prefill_rows, 256
                act = rnd(t, kd, seed=400 + self.rank, scale=0.3).half()
                wd = rnd(H, kd, seed=500 + self.rank, scale=0.05).half()
                wg = rnd(512, H, seed=600, scale=0.02).half()
                ln = torch.zeros(H, dtype=torch.bfloat16, device=dev)
                yd = torch.empty(t, H, dtype=torch.bfloat16, device=dev)
                gemm_tc.f16_gemm(act, wd, yd)
                hsum = nccl_sum(yd)
                xw = (hsum * torch.rsqrt(hsum.pow(2).mean(-1, keepdim=True) + 1e-6)).half()
                gw = torch.empty(t, 512, dtype=torch.bfloat16, device=dev)
                gemm_tc.f16_gemm(xw, wg, gw)
                pipe.h.zero_()
                pipe.gemm_rs(act, wd, t)
                pipe.reduce_norm_gather(t, ln, out_dtype=torch.float16)
                go = torch.empty(t, 512, dtype=torch.bfloat16, device=dev)
                pipe.gemm_ag(wg, go, t)
                torch.cuda.synchronize(dev)
                facts["sp_gathered"] = rel(pipe.x(t, torch.float16), xw)
                facts["sp_gemm"] = rel(go, gw)
                pipe.h.zero_()
            torch.cuda.synchronize(dev)
            facts["status"] = [int(s.status()), int(gemm_tc.gemm_status())]
            ok = all(v < 0.03 for k, v in facts.items() if isinstance(v, float)) and not any(facts["status"])
        except Exception as ex:          # a failed launch is a failed proof
            facts["error"] = repr(ex)
            ok = False
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        facts["ok"] = bool(flag.item())
        if not facts["ok"]:
            from ..utils.log import LOG

            LOG.warn("comm.proof", f"rank {self.rank}: own collectives failed their proof at world {self.world} "
                                   f"({facts}); falling back to the library arm")
            self.symm, self.mode = None, "nccl"
        self.proof = facts
        return facts

    # row-parallel projection output: h[:m] += sum over ranks of partial[:m]
    def allreduce_add_residual(self, partial: torch.Tensor, h: torch.Tensor, m: int) -> None:
        if self.symm is not None:
            self.symm.allreduce_add_residual(partial, h, m)
            return
        if self.relay is not None:
            self.relay.allreduce_(partial[:m])
            h[:m].add_(partial[:m])
            return
        dist.all_reduce(partial[:m], group=self.group)
        h[:m].add_(partial[:m])

    def allreduce_prefill(self, y: torch.Tensor) -> None:
        if self.symm is not None and self.symm.can_reduce(y):
            self.symm.allreduce_(y)
            return
        if self.relay is not None:
            self.relay.allreduce_(y)
            return
        dist.all_reduce(y, group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)

    def max_over_ranks(self, value: float) -> float:
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())
