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
        return cls(rank, world, torch.device(f"cuda:{local}"), mode, **kw)

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
