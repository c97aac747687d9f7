"""Int4 weight quantisation, the "skinny tile" repacker and the ActPack activation format.

Canonical W4 form (what the checkpoint readers produce, whatever the on-disk format):
``q`` uint8 ``[N, K]`` with values 0..15, ``scales`` fp16 ``[N, K/G]``, ``zeros`` uint8
``[N, K/G]`` (asymmetric: ``w = (q - z) * s``; symmetric formats use ``z = 8``), G in {32, 128}.

``pack_skinny`` rearranges that into the layout the sm_100a kernels stream (see
``csrc/gemv.cu``); ``unpack_skinny`` is its inverse and exists for tests.

Reference counterpart: the Marlin repack (``crates/kernels/src/family/marlin/repack.rs``,
``crates/kernels/cu/load/*.cu``) and the AWQ source reader (``crates/models/src/formats/awq.rs``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class W4Canonical:
    q: torch.Tensor        # uint8 [N, K], 0..15
    scales: torch.Tensor   # fp16 [N, K/G]
    zeros: torch.Tensor    # uint8 [N, K/G]
    group: int

    @property
    def shape(self):
        return tuple(self.q.shape)

    def dequant(self, dtype=torch.float32) -> torch.Tensor:
        n, k = self.q.shape
        g = self.group
        w = self.q.view(n, k // g, g).to(torch.float32) - self.zeros.view(n, k // g, 1).to(torch.float32)
        w = w * self.scales.view(n, k // g, 1).to(torch.float32)
        return w.view(n, k).to(dtype)


def quantize_w4(w: torch.Tensor, group: int = 128, symmetric: bool = False) -> W4Canonical:
    """Round-to-nearest group quantisation of a dense ``[N, K]`` weight."""
    n, k = w.shape
    assert k % group == 0
    wf = w.to(torch.float32).view(n, k // group, group)
    if symmetric:
        amax = wf.abs().amax(-1, keepdim=True).clamp_min(1e-8)
        scale = (amax / 7.0).to(torch.float16).to(torch.float32).clamp_min(1e-8)
        zero = torch.full_like(scale, 8.0)
    else:
        mx, mn = wf.amax(-1, keepdim=True), wf.amin(-1, keepdim=True)
        scale = ((mx - mn).clamp_min(1e-8) / 15.0).to(torch.float16).to(torch.float32).clamp_min(1e-8)
        zero = (-mn / scale).round().clamp(0, 15)
    q = (wf / scale + zero).round().clamp(0, 15).to(torch.uint8)
    return W4Canonical(q.view(n, k), scale.view(n, k // group).to(torch.float16),
                       zero.view(n, k // group).to(torch.uint8), group)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Merged gate/up rows in "interleaved-8" order: per 16 rows, 8 gate rows then 8 up rows."""
    i, k = gate.shape
    assert up.shape == gate.shape and i % 8 == 0
    return torch.stack([gate.view(i // 8, 8, k), up.view(i // 8, 8, k)], dim=1).reshape(2 * i, k)


def deinterleave_gate_up(y: torch.Tensor):
    """Inverse of the interleaved-8 order on the last dim of an activation ``[..., 2I]``."""
    lead = y.shape[:-1]
    i2 = y.shape[-1]
    v = y.reshape(*lead, i2 // 16, 2, 8)
    return v[..., 0, :].reshape(*lead, i2 // 2), v[..., 1, :].reshape(*lead, i2 // 2)


@dataclass
class W4Skinny:
    """Device-ready W4 weight: tile stream + (scale, zero) table."""
    tiles: torch.Tensor   # uint8 [N/16, K/128, 1024]
    sz: torch.Tensor      # fp16 [N/16, K/G, 16, 2]
    n: int
    k: int
    group: int

    def to(self, device):
        return W4Skinny(self.tiles.to(device), self.sz.to(device), self.n, self.k, self.group)

    @property
    def nbytes(self) -> int:
        return self.tiles.numel() + self.sz.numel() * 2


def pack_skinny(c: W4Canonical) -> W4Skinny:
    n, k = c.q.shape
    assert n % 16 == 0 and k % 128 == 0, (n, k)
    nt, kt = n // 16, k // 128
    # q[nt*16 + half*8 + g, kt*128 + w*32 + t*8 + i] -> tiles[nt, kt, half, g, t, w, i]
    v = c.q.view(nt, 2, 8, kt, 4, 4, 8).permute(0, 3, 1, 2, 5, 4, 6).contiguous()
    lo, hi = v[..., 0::2], v[..., 1::2]
    tiles = (lo | (hi << 4)).to(torch.uint8).reshape(nt, kt, 1024)
    kg = k // c.group
    sz = torch.stack([c.scales.view(nt, 16, kg).permute(0, 2, 1),
                      c.zeros.view(nt, 16, kg).permute(0, 2, 1).to(torch.float16)], dim=-1).contiguous()
    return W4Skinny(tiles, sz, n, k, c.group)


def unpack_skinny(s: W4Skinny) -> W4Canonical:
    nt, kt = s.n // 16, s.k // 128
    b = s.tiles.view(nt, kt, 2, 8, 4, 4, 4)
    v = torch.stack([b & 0xF, b >> 4], dim=-1).reshape(nt, kt, 2, 8, 4, 4, 8)
    q = v.permute(0, 2, 3, 1, 5, 4, 6).reshape(s.n, s.k).contiguous()
    kg = s.k // s.group
    scales = s.sz[..., 0].permute(0, 2, 1).reshape(s.n, kg).contiguous()
    zeros = s.sz[..., 1].permute(0, 2, 1).reshape(s.n, kg).to(torch.uint8).contiguous()
    return W4Canonical(q, scales, zeros, s.group)


def random_skinny(n: int, k: int, group: int, device, std: float = 0.02, seed: int = 0) -> W4Skinny:
    """Random W4 weight generated directly in the device layout (benchmark initialisation).

    Equivalent to quantising N(0, std) weights: nibbles are drawn from a rounded normal around
    the zero-point 8 with a scale chosen so the dequantised values have standard deviation std.
    """
    gen = torch.Generator(device=device).manual_seed(seed)
    nt, kt = n // 16, k // 128
    vals = (torch.randn(nt, kt, 2048, device=device, generator=gen) * 2.5 + 8.0).round().clamp_(0, 15).to(torch.uint8)
    tiles = (vals[..., 0::2] | (vals[..., 1::2] << 4)).contiguous()
    kg = k // group
    sz = torch.empty(nt, kg, 16, 2, dtype=torch.float16, device=device)
    sz[..., 0] = (std / 2.5) * (1.0 + 0.1 * torch.rand(nt, kg, 16, device=device, generator=gen))
    sz[..., 1] = torch.randint(7, 10, (nt, kg, 16), device=device, generator=gen).to(torch.float16)
    return W4Skinny(tiles, sz, n, k, group)


# ---- ActPack -----------------------------------------------------------------------------
_PERM = [0, 4, 1, 5, 2, 6, 3, 7]


def act_pack_ref(x: torch.Tensor, group: int):
    """fp32 reference of the ActPack producer: returns (xpack fp16 [M,K], xs fp32 [M,K/G,2])."""
    m, k = x.shape
    v = x.to(torch.float32).clamp(-65504, 65504).view(m, k // 8, 8)[..., _PERM].clone()
    v[..., [2, 3, 6, 7]] *= 0.0625
    h = v.to(torch.float16)
    hf = h.to(torch.float32)
    eff = hf.clone()
    eff[..., [2, 3, 6, 7]] *= 16.0
    cpg = group // 8
    s_st = hf.sum(-1).view(m, k // group, cpg).sum(-1)
    s_eff = eff.sum(-1).view(m, k // group, cpg).sum(-1)
    return h.view(m, k), torch.stack([s_eff, 1024.0 * s_st], dim=-1)


def quantize_w8_rows(w: torch.Tensor):
    """Per-row symmetric int8 (lm_head / embedding tables): returns (int8 [N,K], fp32 scale [N])."""
    wf = w.to(torch.float32)
    s = wf.abs().amax(-1).clamp_min(1e-8) / 127.0
    q = (wf / s[:, None]).round().clamp(-127, 127).to(torch.int8)
    return q, s
