"""Coverage probe of the KV selection layer: does scoring blocks through the Mean-K index reproduce where attention goes?

    truth   rotated queries x the sequence's rotated keys -> softmax per (query, head) -> attention mass per block
    index   de-rotated queries x block means of de-rotated keys -> one score per block (``select.score_blocks``)
    curve   the share of the true attention mass that the k best-SCORED blocks hold, for k = 1, 2, 4, 8, ...

A curve near the oracle's (the k blocks of largest true mass) means the index is a usable selector; a curve near ``k / blocks``
(chance) means scores and attention disagree -- the first suspects are then the rotary pairing convention of the de-rotation
and the layout of the index. The probe is read-only: it reads pages and the query the step left behind, the model runs once.

Reference counterpart: ``crates/engine/src/exec/coverage.rs:1-45`` (the question, truth / index / curve, the query window).
"""
from __future__ import annotations

import torch

from . import select as S


def block_mass(q: torch.Tensor, k: torch.Tensor, block: int, scale: float | None = None) -> torch.Tensor:
    """True attention mass per block. ``q``: [nq, hq, hd] rotated queries (all at or after the last key); ``k``: [T, hkv, hd]
    rotated keys of the context. Softmax per (query, query head) over all T keys; returns [ceil(T / block)] with the mass
    summed over a block's keys and averaged over queries and heads (sums to 1)."""
    nq, hq, hd = q.shape
    t, hkv, _ = k.shape
    rep = hq // hkv
    scale = hd ** -0.5 if scale is None else scale
    qf = q.float().view(nq, hkv, rep, hd)
    logits = torch.einsum("qgrd,tgd->qgrt", qf, k.float()) * scale
    p = logits.softmax(-1).mean(dim=(0, 1, 2))                       # [T]
    nb = (t + block - 1) // block
    pad = torch.zeros(nb * block - t, dtype=p.dtype)
    return torch.cat([p, pad]).view(nb, block).sum(-1)


def coverage_curve(mass: torch.Tensor, scores: torch.Tensor, ks=(1, 2, 4, 8, 16, 32)) -> dict:
    """Share of the true mass inside the k best-scored blocks, next to the oracle (k blocks of largest mass) and chance."""
    nb = mass.numel()
    by_score = torch.argsort(scores[:nb].float(), descending=True)
    by_mass = torch.argsort(mass, descending=True)
    out = {}
    for k in ks:
        kk = min(k, nb)
        out[k] = {"index": float(mass[by_score[:kk]].sum()), "oracle": float(mass[by_mass[:kk]].sum()), "chance": kk / nb}
    return out


def probe(q_rot: torch.Tensor, qpos: torch.Tensor, k_rot: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, block: int,
          ks=(1, 2, 4, 8, 16, 32)) -> dict:
    """The whole probe on host tensors: ``q_rot`` [nq, hq, hd] at positions ``qpos`` [nq], ``k_rot`` [T, hkv, hd] at positions
    0 .. T-1. Returns the curve and the rank correlation between scores and mass."""
    half = rotary_dim // 2
    t = k_rot.shape[0]

    def cs(pos):
        ang = pos.float()[:, None] * inv_freq.float()[None, :half]
        return ang.cos(), ang.sin()
    kc, ks_ = cs(torch.arange(t))
    k_de = S.derope(k_rot.float(), kc, ks_)
    nb_full = t // block
    index = S.mean_k_index(k_de[:nb_full * block].view(nb_full, block, *k_de.shape[1:]))
    if t % block:
        index = torch.cat([index, k_de[nb_full * block:].mean(0, keepdim=True)])
    qc, qs = cs(qpos)
    q_de = S.derope(q_rot.float(), qc, qs)
    scores = S.score_blocks(q_de, index)
    mass = block_mass(q_rot, k_rot, block)
    r = torch.argsort(torch.argsort(scores)).float()
    m = torch.argsort(torch.argsort(mass)).float()
    rho = float(torch.corrcoef(torch.stack([r, m]))[0, 1]) if mass.numel() > 2 else 1.0
    return {"blocks": int(mass.numel()), "curve": coverage_curve(mass, scores, ks), "spearman": rho}
