"""Test kit: deterministic RNG, tolerant comparison with a diff report, resource gating.

Reference counterpart: ``crates/shared/src/testkit/*`` (splitmix64 ``Rng``, ``allclose`` /
``DiffReport``, ``resources.toml`` needs) and the ``#[owl_test(gpu, needs=...)]`` macro.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

MASK = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int):
        self.s = seed & MASK

    def next_u64(self) -> int:
        self.s = (self.s + 0x9E3779B97F4A7C15) & MASK
        z = self.s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
        return z ^ (z >> 31)

    def uniform(self) -> float:
        return (self.next_u64() >> 11) / float(1 << 53)

    def tensor(self, *shape, scale: float = 1.0) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        return torch.tensor([(self.uniform() * 2 - 1) * scale for _ in range(n)], dtype=torch.float32).view(*shape)


@dataclass
class DiffReport:
    ok: bool
    max_abs: float
    max_rel: float
    rel_fro: float
    worst_index: tuple
    n_bad: int

    def __str__(self):
        return (f"{'OK' if self.ok else 'MISMATCH'} max_abs={self.max_abs:.3e} max_rel={self.max_rel:.3e} "
                f"rel_fro={self.rel_fro:.3e} worst@{self.worst_index} bad={self.n_bad}")


def allclose(got: torch.Tensor, want: torch.Tensor, rtol: float = 1e-3, atol: float = 1e-5) -> DiffReport:
    g, w = got.detach().float().cpu(), want.detach().float().cpu()
    diff = (g - w).abs()
    bad = diff > (atol + rtol * w.abs())
    idx = tuple(int(i) for i in torch.unravel_index(diff.argmax(), diff.shape)) if diff.numel() else ()
    return DiffReport(ok=not bool(bad.any()), max_abs=float(diff.max()) if diff.numel() else 0.0,
                      max_rel=float((diff / w.abs().clamp_min(1e-12)).max()) if diff.numel() else 0.0,
                      rel_fro=float(diff.norm() / w.norm().clamp_min(1e-12)), worst_index=idx, n_bad=int(bad.sum()))


def need(resource: str) -> str | None:
    """Path of an optional test resource (``OWL_B200_RES_<NAME>``), or None: tests skip, never pass silently."""
    return os.environ.get("OWL_B200_RES_" + resource.upper().replace("-", "_").replace(":", "_"))
