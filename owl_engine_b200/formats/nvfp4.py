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


def pack_for_mma(q: NvFp4):
    """Scale-factor layout of the block-scaled MMA (``tcgen05.mma kind::mxf4nvf4 block16``): scales
    of a 128-row x 4-block tile are stored as 32 rows x 16 bytes (row r of the tile at
    ``[r % 32][(r // 32) * 4 + block]``), tiles ordered [N/128][K/64]. Codes stay row-major."""
    n, k = q.shape
    nb = k // 16
    assert n % 128 == 0 and nb % 4 == 0
    s = q.scales.view(n // 128, 4, 32, nb // 4, 4)             # [tile, r//32, r%32, kb, blk]
    s = s.permute(0, 3, 2, 1, 4).contiguous()                  # [tile, kb, r%32, r//32, blk]
    return q.codes, s.view(n // 128, nb // 4, 512)
