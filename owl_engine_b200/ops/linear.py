"""Prefill-shape linear layers over quantised weights.

``w4_gemm`` computes ``out[T, N] = x[T, K] @ dequant(w)^T`` for a ``W4Skinny`` weight with one of
two arms:

* ``"tc"``        the product path: the tcgen05 / TMEM W4A16 GEMM (``csrc/gemm_tc.cu``), weights
                  dequantised inside the kernel;
* ``"baseline"``  dequantise to a dense bf16 scratch matrix, then the library GEMM
                  (``torch.matmul`` = cuBLAS). This is the comparison arm, like the reference's
                  range-dequant -> cuBLAS arm (``crates/kernels/cu/gguf/gguf_smem.cu:415-552``).
"""
from __future__ import annotations

import torch

from . import kernels as K

_scratch: dict = {}


def _dense_scratch(n: int, k: int, device) -> torch.Tensor:
    key = (str(device),)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n * k:
        buf = torch.empty(n * k, dtype=torch.bfloat16, device=device)
        _scratch[key] = buf
    return buf[:n * k].view(n, k)


def w4_gemm(w, x: torch.Tensor, out: torch.Tensor, arm: str = "tc") -> torch.Tensor:
    if arm == "baseline":
        dense = K.w4_dequant(w, _dense_scratch(w.n, w.k, x.device))
        torch.matmul(x, dense.t(), out=out)
        return out
    if arm == "tc":
        from . import gemm_tc

        return gemm_tc.w4a16_gemm(w, x, out)
    raise ValueError(f"unknown prefill GEMM arm {arm!r}")


_w16: dict = {}


def dense_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, arm: str = "tc") -> torch.Tensor:
    """out[T, N] (bf16) = x @ w^T for a small dense bf16 weight (GDN a/b projections, draft heads)."""
    if arm == "baseline":
        torch.matmul(x.to(w.dtype), w.t(), out=out)
        return out
    from . import gemm_tc

    if x.dtype != w.dtype:
        key = (w.data_ptr(), x.dtype)
        wc = _w16.get(key)
        if wc is None:
            wc = w.to(x.dtype)
            _w16[key] = wc
        w = wc
    return gemm_tc.f16_gemm(x, w, out)
