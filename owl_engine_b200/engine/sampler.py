"""Host sampler: repetition penalty -> temperature -> top-k -> top-p -> multinomial (xorshift64*).

Works on the candidate list the device returns (top-k logits of a row, k <= 32), so only a few
hundred bytes cross PCIe per sampled token. The RNG stream is a pure function of (seed, turn, step)
so a request with a seed is reproducible regardless of batching. ``accept_rejection`` is the exact
speculative-sampling rule (accept with min(1, p/q), else resample from the residual).

Reference counterpart: ``crates/engine/src/sampler.rs`` and ``exec/proposal_q.rs:417-476``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

MASK = (1 << 64) - 1


class XorShift64Star:
    def __init__(self, seed: int):
        self.s = (seed & MASK) or 0x9E3779B97F4A7C15

    def next_u64(self) -> int:
        x = self.s
        x ^= x >> 12
        x ^= (x << 25) & MASK
        x ^= x >> 27
        self.s = x
        return (x * 0x2545F4914F6CDD1D) & MASK

    def uniform(self) -> float:
        return (self.next_u64() >> 11) / float(1 << 53)


def step_seed(seed: int, turn: int, step: int) -> int:
    z = (seed * 0x9E3779B97F4A7C15 + turn * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & MASK
    z ^= z >> 31
    return z or 1


@dataclass
class SamplingParams:
    mode: str = "greedy"           # greedy | sampling
    temp: float = 1.0
    topk: int = 20
    topp: float = 0.95
    rep_penalty: float = 1.0
    seed: int = 0


def apply_rep_penalty(cands: list[tuple[int, float]], history: set, penalty: float) -> list[tuple[int, float]]:
    if penalty == 1.0 or not history:
        return cands
    return [(t, (l / penalty if l > 0 else l * penalty) if t in history else l) for t, l in cands]


def distribution(cands: list[tuple[int, float]], p: SamplingParams) -> list[tuple[int, float]]:
    """(token, probability) after temperature, top-k and top-p, sorted by probability (descending)."""
    c = sorted(cands, key=lambda x: (-x[1], x[0]))[:max(1, p.topk)]        # equal logits: the smaller id first, whatever order they came in
    t = max(p.temp, 1e-5)
    m = c[0][1]
    w = [math.exp((l - m) / t) for _, l in c]
    z = sum(w)
    pr = [x / z for x in w]
    keep, acc = [], 0.0
    for (tok, _), q in zip(c, pr):
        keep.append((tok, q))
        acc += q
        if acc >= p.topp:
            break
    z = sum(q for _, q in keep)
    return [(tok, q / z) for tok, q in keep]


def sample(cands: list[tuple[int, float]], p: SamplingParams, turn: int, step: int, history: set | None = None) -> int:
    if p.mode == "greedy" or p.temp <= 0:
        return max(apply_rep_penalty(cands, history or set(), p.rep_penalty), key=lambda x: (x[1], -x[0]))[0]
    dist = distribution(apply_rep_penalty(cands, history or set(), p.rep_penalty), p)
    u = XorShift64Star(step_seed(p.seed, turn, step)).uniform()
    acc = 0.0
    for tok, q in dist:
        acc += q
        if u < acc:
            return tok
    return dist[-1][0]


def accept_rejection(draft_tok: int, p_target: dict, q_draft: dict, rng: XorShift64Star) -> tuple[bool, int]:
    """Exact speculative sampling for one position: returns (accepted, token)."""
    pt, qd = p_target.get(draft_tok, 0.0), max(q_draft.get(draft_tok, 0.0), 1e-12)
    if rng.uniform() < min(1.0, pt / qd):
        return True, draft_tok
    resid = {t: max(0.0, v - q_draft.get(t, 0.0)) for t, v in p_target.items()}
    z = sum(resid.values())
    if z <= 0:
        return False, max(p_target, key=p_target.get)
    u, acc = rng.uniform() * z, 0.0
    for t, v in resid.items():
        acc += v
        if u < acc:
            return False, t
    return False, t
