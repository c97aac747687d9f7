"""Readers of pre-quantised int4 checkpoints, all mapped onto ``ops.quant.W4Canonical``.

* compressed-tensors AWQ (pack-quantized, asymmetric, group 32 or 128): ``weight_packed`` int32
  ``[out, in/8]`` (nibble i of a word = column 8j+i), ``weight_scale`` bf16/f16 ``[out, in/G]``,
  ``weight_zero_point`` int32 ``[out/8, in/G]`` (packed along the output dim), ``weight_shape``.
* compressed-tensors W4A16 symmetric (no zero point tensor; stored values are offset by 8).
* AutoAWQ GEMM layout: ``qweight`` int32 ``[in, out/8]``, ``qzeros`` ``[in/G, out/8]``, ``scales``
  ``[in/G, out]`` with the interleaved nibble order 0,2,4,6,1,3,5,7.

Reference counterpart: ``crates/models/src/formats/{awq,w4a16,kind}.rs``.
"""
from __future__ import annotations

import torch

from ..ops.quant import W4Canonical

_AWQ_ORDER = [0, 2, 4, 6, 1, 3, 5, 7]


def _unpack_i32(packed: torch.Tensor, dim: int, order=None) -> torch.Tensor:
    """int32 words -> 8 nibbles each along `dim` (word i -> positions 8i..8i+7)."""
    p = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, dtype=torch.int64) * 4
    x = ((p.unsqueeze(-1) >> shifts) & 0xF).to(torch.uint8)            # [..., 8]
    if order is not None:
        inv = torch.empty(8, dtype=torch.long)
        inv[torch.tensor(order)] = torch.arange(8)
        x = x[..., inv]
    if dim == -1 or dim == packed.dim() - 1:
        return x.reshape(*packed.shape[:-1], packed.shape[-1] * 8)
    assert dim == 0
    return x.permute(0, 2, 1).reshape(packed.shape[0] * 8, packed.shape[1])


def from_compressed_tensors(src, prefix: str) -> W4Canonical:
    """``src.get(name)`` tensor source; ``prefix`` like ``model.layers.0.mlp.down_proj``."""
    packed = src.get(prefix + ".weight_packed")
    scale = src.get(prefix + ".weight_scale")
    shape = src.get(prefix + ".weight_shape").tolist() if (prefix + ".weight_shape") in src else \
        [packed.shape[0], packed.shape[1] * 8]
    n, k = int(shape[0]), int(shape[1])
    q = _unpack_i32(packed, -1)[:n, :k].contiguous()
    group = k // scale.shape[1]
    if (prefix + ".weight_zero_point") in src:
        z = _unpack_i32(src.get(prefix + ".weight_zero_point"), 0)[:n].contiguous()
    else:
        z = torch.full((n, k // group), 8, dtype=torch.uint8)          # symmetric: stored q = w/s + 8
    return W4Canonical(q, scale.to(torch.float16).contiguous(), z, group)


def from_autoawq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor) -> W4Canonical:
    k = qweight.shape[0]
    q = _unpack_i32(qweight, -1, _AWQ_ORDER).t().contiguous()           # [out, in]
    z = _unpack_i32(qzeros, -1, _AWQ_ORDER).t().contiguous()            # [out, in/G]
    return W4Canonical(q, scales.t().to(torch.float16).contiguous(), z, k // qzeros.shape[0])


def to_compressed_tensors(c: W4Canonical, prefix: str) -> dict:
    """Inverse of ``from_compressed_tensors`` (used to write test / synthetic checkpoints)."""
    n, k = c.q.shape
    sh = torch.arange(8, dtype=torch.int64) * 4
    wp = (c.q.view(n, k // 8, 8).to(torch.int64) << sh).sum(-1)
    wp = torch.where(wp >= 2**31, wp - 2**32, wp).to(torch.int32)
    zt = c.zeros.view(n // 8, 8, -1).permute(0, 2, 1).to(torch.int64)
    zp = (zt << sh).sum(-1)
    zp = torch.where(zp >= 2**31, zp - 2**32, zp).to(torch.int32)
    return {prefix + ".weight_packed": wp, prefix + ".weight_scale": c.scales.to(torch.bfloat16)
            if False else c.scales, prefix + ".weight_zero_point": zp,
            prefix + ".weight_shape": torch.tensor([n, k], dtype=torch.int64)}
