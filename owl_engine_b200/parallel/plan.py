"""Tensor-parallel plan: pure shard arithmetic and the per-tensor rule table.

``TpPlan`` answers "which slice of this dimension does rank r of w hold"; ``rule_of`` maps a
weight name to how it is cut (Megatron column / row split, segmented column split for merged
projections, per-head split, replicate). Everything is world-generic (2 / 4 / 8 ...).

Reference counterpart: ``crates/models/src/plan/tp.rs:35-177`` (``shard_range``,
``segmented_ranges``) and ``crates/models/src/plan/rules.rs:174-239`` (the rule table). The
reference assembles world = 2 only; here any world that divides the head counts works, and
kv heads are replicated when world > hkv.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import torch


@dataclass(frozen=True)
class TpPlan:
    rank: int
    world: int

    def shard_range(self, n: int) -> tuple[int, int]:
        assert n % self.world == 0, (n, self.world)
        per = n // self.world
        return self.rank * per, (self.rank + 1) * per

    def segmented_ranges(self, segments: list[int]) -> list[tuple[int, int]]:
        """For a dimension that is the concatenation of ``segments``, the (start, end) pairs
        this rank owns: each segment is cut independently."""
        out, base = [], 0
        for seg in segments:
            lo, hi = self.shard_range(seg)
            out.append((base + lo, base + hi))
            base += seg
        return out


class Rule(Enum):
    REPLICATE = "replicate"
    COL = "uniform_col"          # split output rows evenly
    ROW = "uniform_row"          # split input columns evenly -> partial sums -> all-reduce
    SEG_COL = "segmented_col"    # output rows are a concat of segments, each split
    PER_HEAD = "per_head"        # first dim indexed by head
    KV_COL = "kv_col"            # k/v projection rows: split by kv head, replicated when world > hkv
    Q_COL = "q_col"              # q rows are per-head [q|gate] pairs: cut whole heads


def rule_of(name: str) -> Rule:
    n = name
    if n.endswith(("gate_proj.weight", "up_proj.weight", "in_proj_z.weight")):
        return Rule.COL
    if n.endswith(("down_proj.weight", "o_proj.weight", "out_proj.weight")):
        return Rule.ROW
    if n.endswith("q_proj.weight"):
        return Rule.Q_COL
    if n.endswith(("k_proj.weight", "v_proj.weight")):
        return Rule.KV_COL
    if n.endswith(("in_proj_qkv.weight", "conv1d.weight")):
        return Rule.SEG_COL
    if n.endswith(("in_proj_a.weight", "in_proj_b.weight", "A_log", "dt_bias")):
        return Rule.PER_HEAD
    return Rule.REPLICATE      # norms, embed, lm_head (vocab split is a separate opt-in)


def shard_tensor(name: str, t: torch.Tensor, full_spec, plan: TpPlan) -> torch.Tensor:
    """Cut one HF-named tensor of the unsharded model for ``plan.rank``."""
    if plan.world == 1:
        return t
    r = rule_of(name)
    sp = full_spec
    if r is Rule.REPLICATE:
        return t
    if r is Rule.COL or r is Rule.PER_HEAD:
        lo, hi = plan.shard_range(t.shape[0])
        return t[lo:hi].contiguous()
    if r is Rule.ROW:
        lo, hi = plan.shard_range(t.shape[1])
        return t[:, lo:hi].contiguous()
    if r is Rule.Q_COL:
        lo, hi = plan.shard_range(sp.hq)
        return t[lo * 2 * sp.hd:hi * 2 * sp.hd].contiguous()
    if r is Rule.KV_COL:
        if sp.hkv % plan.world == 0:
            lo, hi = plan.shard_range(sp.hkv)
        else:
            rep = plan.world // sp.hkv
            lo = plan.rank // rep
            hi = lo + 1
        return t[lo * sp.hd:hi * sp.hd].contiguous()
    if r is Rule.SEG_COL:
        segs = [sp.key_dim, sp.key_dim, sp.value_dim]
        parts = [t[lo:hi] for lo, hi in plan.segmented_ranges(segs)]
        return torch.cat(parts).contiguous()
    raise AssertionError(r)


def shard_dense_for_rank(spec, dense: dict) -> dict:
    """``spec`` is the per-rank (sharded) view; ``dense`` holds the full model. Returns the
    rank's slices (identity when world == 1 or when ``dense`` is already sharded)."""
    if spec.tp_world == 1:
        return dense
    from dataclasses import replace

    w = spec.tp_world
    hkv_full = spec.hkv * w if spec.kv_replicas == 1 else w // spec.kv_replicas
    full = replace(spec, inter=spec.inter * w, hq=spec.hq * w, hkv=hkv_full, nk=spec.nk * w, nv=spec.nv * w,
                   tp_rank=0, tp_world=1, kv_replicas=1)
    plan = TpPlan(spec.tp_rank, w)
    return {k: shard_tensor(k, v, full, plan) for k, v in dense.items()}
