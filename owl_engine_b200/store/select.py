"""KV-cache virtualisation (KVMem-style block selection).

For long contexts the per-turn device working set is bounded: a *Mean-K index* keeps, per block,
layer and kv head, the mean of the block's de-rotated keys; ``score_blocks`` scores every block
against the current (de-rotated) queries and ``select`` keeps the sink blocks, the most recent
blocks and the top-k scored ones, up to ``workspace`` tokens. The result is a *view* page table
that replaces the sequence's block table for that step.

Reference counterpart: ``crates/store/src/select.rs`` (``score_blocks``, ``select``),
``crates/kernels/cu/elems/{mean_k,page_softmax}.cu`` (GPU index + scoring).
"""
from __future__ import annotations

import torch


def mean_k_index(k_blocks: torch.Tensor) -> torch.Tensor:
    """k_blocks: [n_blocks, block, hkv, hd] de-rotated keys -> [n_blocks, hkv, hd] block means."""
    return k_blocks.float().mean(dim=1)


def derope(k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Inverse of the partial rotate-half RoPE (k: [T, H, hd]; cos/sin: [T, half])."""
    half = cos.shape[-1]
    x1, x2, rest = k[..., :half], k[..., half:2 * half], k[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c + x2 * s, x2 * c - x1 * s, rest], dim=-1)


def score_blocks(q: torch.Tensor, index: torch.Tensor, mode: str = "cosine-max", gqa: str = "max") -> torch.Tensor:
    """q: [nq, hq, hd] recent queries (de-rotated); index: [n_blocks, hkv, hd]. Returns [n_blocks]."""
    nq, hq, hd = q.shape
    nb, hkv, _ = index.shape
    rep = hq // hkv
    qf = q.float().view(nq, hkv, rep, hd)
    kf = index.float()
    if mode.startswith("cosine"):
        qf = torch.nn.functional.normalize(qf, dim=-1)
        kf = torch.nn.functional.normalize(kf, dim=-1)
    s = torch.einsum("qgrd,bgd->bqgr", qf, kf)               # [nb, nq, hkv, rep]
    s = s.amax(-1) if gqa == "max" else s.mean(-1)           # over the q heads of a kv head
    s = s.amax(1) if mode.endswith("max") else s.mean(1)     # over queries
    return s.amax(-1)                                         # over kv heads


def select(scores: torch.Tensor, n_blocks: int, budget_blocks: int, sink: int = 2, recent: int = 4) -> list[int]:
    """Block ids kept for this step, ascending (causal order is preserved in the view)."""
    if n_blocks <= budget_blocks:
        return list(range(n_blocks))
    keep = set(range(min(sink, n_blocks))) | set(range(max(0, n_blocks - recent), n_blocks))
    room = budget_blocks - len(keep)
    if room > 0:
        masked = scores[:n_blocks].clone()
        for b in keep:
            masked[b] = float("-inf")
        top = torch.topk(masked, min(room, n_blocks - len(keep))).indices.tolist()
        keep |= set(top)
    return sorted(keep)


def view_table(block_table_row: torch.Tensor, kept: list[int]) -> torch.Tensor:
    """Page table of the selected blocks (what the attention kernel walks instead of the full row)."""
    return block_table_row[torch.tensor(kept, dtype=torch.long, device=block_table_row.device)]


# ---- GPU index + scoring (csrc/kvmem.cu) ----------------------------------------------------------------------------
def _K():
    import ctypes

    from ..ops import kernels as K

    if "owl_mean_k_block" not in K._SIGS:
        P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        K.register("owl_mean_k_block", [P, P, P, P, P, I, I, I, I, P, P])
        K.register("owl_mean_k_block_fmt", [P, P, I, P, P, P, P, I, I, I, I, P, P])
        K.register("owl_kvscore", [P, P, P, P, I, I, I, I, I, I, P, P])
        K.register("owl_kvscore_softmax", [P, I, F, P, P])
    return K


def mean_k_blocks_gpu(k_pool_layer: torch.Tensor, pages: torch.Tensor, pos0: torch.Tensor, n_valid: torch.Tensor,
                      inv_freq: torch.Tensor, rotary_dim: int, out: torch.Tensor, k_scale: torch.Tensor | None = None) -> torch.Tensor:
    """Block means of de-rotated keys straight from the paged pool of one layer -> ``out[:len(pages)]``. The pool format is
    read off the tensors: fp16 words (16-bit pool), int8 with ``k_scale`` [pages, 16, hkv], else e4m3."""
    K = _K()
    _, _, hkv, hd = k_pool_layer.shape
    n = pages.numel()
    fmt = 2 if k_pool_layer.dtype == torch.float16 else (1 if k_scale is not None else 0)
    K.call("owl_mean_k_block_fmt", K.ptr(k_pool_layer), K.ptr(k_scale), fmt, K.ptr(pages), K.ptr(pos0), K.ptr(n_valid),
           K.ptr(inv_freq), rotary_dim, n, hkv, hd, K.ptr(out), K.stream())
    return out[:n]


def score_blocks_gpu(q: torch.Tensor, qpos: torch.Tensor, index: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """Cosine-max block scores of rotated queries ``q`` bf16 [nq, hq, hd] against the index float [nb, hkv, hd]."""
    K = _K()
    nq, hq, hd = q.shape
    nb, hkv, _ = index.shape
    out = torch.empty(nb, dtype=torch.float32, device=q.device) if out is None else out
    K.call("owl_kvscore", K.ptr(q), K.ptr(qpos), K.ptr(index), K.ptr(inv_freq), rotary_dim, nq, hq, hkv, hd, nb, K.ptr(out),
           K.stream())
    return out[:nb]


def softmax_scores_gpu(scores: torch.Tensor, temp: float = 1.0) -> torch.Tensor:
    K = _K()
    out = torch.empty_like(scores)
    K.call("owl_kvscore_softmax", K.ptr(scores), scores.numel(), float(temp), K.ptr(out), K.stream())
    return out
