"""NVFP4 codec: e2m1 values, one e4m3 scale per 16 elements, one fp32 scale per tensor.

``w ~= e2m1(code) * e4m3(block_scale) * global_scale`` with ``global_scale = amax / (6 * 448)`` so
the largest block scale is representable. Storage: two codes per byte (low nibble first), block
scales as e4m3 bytes ``[N, K/16]``. ``quantize`` / ``dequantize`` are the CPU oracles; the device
layout for the block-scaled tensor-core path is produced by ``pack_for_mma``.

Reference counterpart: ``crates/kernels/cu/nvfp4/{nvfp4_quant_act,nvfp4_gemm}.cu`` and the NVFP4
pack transform of ``crates/models/src/formats/transform.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])     # round-to-nearest thresholds


@dataclass
class NvFp4:
    codes: torch.Tensor        # uint8 [N, K/2]: element 2i in the low nibble, 2i+1 in the high nibble
    scales: torch.Tensor       # uint8 view of e4m3 [N, K/16]
    global_scale: float
    shape: tuple


def encode_e2m1(x: torch.Tensor) -> torch.Tensor:
    mag = torch.bucketize(x.abs(), _BOUNDS, right=False).to(torch.uint8)
    return mag | ((x < 0).to(torch.uint8) << 3)


def decode_e2m1(c: torch.Tensor) -> torch.Tensor:
    v = E2M1[(c & 7).long()]
    return torch.where((c & 8) != 0, -v, v)


def quantize(w: torch.Tensor) -> NvFp4:
    n, k = w.shape
    assert k % 16 == 0
    wf = w.float()
    gs = float(wf.abs().max().clamp_min(1e-12)) / (6.0 * 448.0)
    blocks = wf.view(n, k // 16, 16)
    bs = (blocks.abs().amax(-1) / 6.0 / gs).clamp(max=448.0)
    bs8 = bs.to(torch.float8_e4m3fn)
    bsf = bs8.float().clamp_min(2.0 ** -9)
    codes = encode_e2m1(blocks / (bsf[..., None] * gs)).view(n, k)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return NvFp4(packed.contiguous(), bs8.view(torch.uint8).contiguous(), gs, (n, k))


def dequantize(q: NvFp4) -> torch.Tensor:
    n, k = q.shape
    codes = torch.stack([q.codes & 0xF, q.codes >> 4], dim=-1).view(n, k)
    bs = q.scales.view(torch.float8_e4m3fn).float()
    return (decode_e2m1(codes).view(n, k // 16, 16) * bs[..., None]).view(n, k) * q.global_scale


def quantize_act(x: torch.Tensor) -> NvFp4:
    """Per-token-block activation quantisation (same format) for the W4A4 tensor-core path."""
    return quantize(x)


def pack_sf_atoms(scales: torch.Tensor) -> torch.Tensor:
    """Scale-factor layout of the block-scaled MMA (``tcgen05.mma kind::mxf4nvf4 block16``). ``scales``: e4m3 bytes
    ``[R, K/16]``. The scales of a 128-row x 4-block (64 k) tile are one 512-byte atom, row r / block b of the tile at byte
    ``(r % 32) * 16 + (r // 32) * 4 + b``; atoms are ordered ``[ceil(R/128)][4 * ceil(K/256)]``, rows and k padded with zero
    bytes (e4m3 +0: a padded block contributes nothing). Works on any device; returns uint8 ``[blocks, atoms, 512]``."""
    r, nb = scales.shape
    rb, ka = (r + 127) // 128, 4 * ((nb + 15) // 16)
    s = torch.zeros(rb * 128, ka * 4, dtype=torch.uint8, device=scales.device)
    s[:r, :nb] = scales.view(torch.uint8)
    s = s.view(rb, 4, 32, ka, 4)                               # [block, r//32, r%32, atom, b]
    return s.permute(0, 3, 2, 1, 4).contiguous().view(rb, ka, 512)


def pack_for_mma(q: NvFp4):
    """(codes, scale atoms) of a quantised matrix for the block-scaled GEMM; codes stay row-major."""
    return q.codes, pack_sf_atoms(q.scales)


def quantize_rows(x: torch.Tensor):
    """Activation quantisation of the block-scaled GEMM (host oracle of ``owl_nvfp4_quant_rows``): every row has its own
    fp32 scale ``amax_row / (6 * 448)``. Returns (codes ``[T, K/2]``, e4m3 bytes ``[T, K/16]``, fp32 scales ``[T]``)."""
    qs = [quantize(x[t:t + 1]) for t in range(x.shape[0])]
    return (torch.cat([q.codes for q in qs]), torch.cat([q.scales for q in qs]),
            torch.tensor([q.global_scale for q in qs], dtype=torch.float32))
