"""Prefill-shape linear layers over quantised weights.

``w4_gemm`` computes ``out[T, N] = x[T, K] @ dequant(w)^T`` for a ``W4Skinny`` weight with one of
two arms:

* ``"tc"``        the product path, both steps our own sm_100a kernels: for short chunks (fewer than
                  ``DEQUANT_FROM`` tokens) the tcgen05 / TMEM W4A16 GEMM that dequantises inside the kernel
                  (``csrc/gemm_tc.cu``); for long chunks the weight is dequantised ONCE into a dense
                  scratch matrix (``csrc/dequant.cu``, runs at copy bandwidth) and the dense tcgen05 GEMM
                  multiplies it -- the in-kernel dequantisation repeats per 128-token tile and caps
                  the fused kernel near 300 TFLOP/s, the dense kernel runs at 750-1000;
* ``"tc8"``       the W4A8 arm on tensor cores: like ``"tc"``, but for long chunks the dequantised weight is
                  re-quantised per output row to e4m3 and the activations per token, and the product runs as
                  ``tcgen05.mma kind::f8f6f4`` at twice the 16-bit rate (the reference's W4A8 arm quantises
                  activations per token to int8 for IMMA, ``crates/kernels/cu/elems/quant_i8_act.cu:80-98``; int4
                  values times a group scale do not survive an integer MMA without a per-group epilogue, an
                  8-bit float product with per-row scales does);
* ``"tcr"`` / ``"tc8r"``  the same two arms with the dequantised (fp16) resp. re-quantised (e4m3) weight kept RESIDENT
                  on the weight object after its first use: 4 resp. 2 extra bytes per weight in HBM (54 / 27 GB for the
                  27B model on one GPU, which 180 GB leave room for) buy back the per-call dequantisation pass;
* ``"baseline"``  dequantise to a dense bf16 scratch matrix, then the library GEMM
                  (``torch.matmul`` = cuBLAS). This is the comparison arm, like the reference's
                  range-dequant -> cuBLAS arm (``crates/kernels/cu/gguf/gguf_smem.cu:415-552``).
"""
from __future__ import annotations

import torch

from . import kernels as K

_scratch: dict = {}
DEQUANT_FROM = 128      # tokens per chunk from which dequantise-once + dense GEMM wins
SKINNY_UPTO = 32        # rows up to which the decode-shape weight-streaming kernel is used instead of a GEMM


def _dense_scratch(n: int, k: int, device, dtype=torch.bfloat16) -> torch.Tensor:
    key = (str(device), dtype)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n * k:
        led = _ledger(device)
        led.release(f"dequant scratch {dtype}")
        _scratch.pop(key, None)
        buf = None
        buf = led.alloc(f"dequant scratch {dtype}", "workspace", (n * k,), dtype)
        _scratch[key] = buf
    return buf[:n * k].view(n, k)


def _ledger(device):
    from ..utils.ledger import ledger_for

    return ledger_for(device)


def _fp8_scratch(tag: str, r: int, k: int, device):
    key = (tag, str(device))
    buf = _scratch.get(key)
    if buf is None or buf[0].numel() < r * k or buf[1].numel() < r:
        led = _ledger(device)
        led.release(f"e4m3 scratch {tag}")
        buf = (led.alloc(f"e4m3 scratch {tag}", "workspace", (r * k,), torch.uint8), torch.empty(r, dtype=torch.float32, device=device))
        _scratch[key] = buf
    return buf[0][:r * k].view(r, k), buf[1][:r]


def w4_gemm(w, x: torch.Tensor, out: torch.Tensor, arm: str = "tc") -> torch.Tensor:
    arm = "tc" if arm == "tc4" else arm                    # the 4-bit float product exists for NVFP4 weights only
    if arm == "baseline":
        dense = K.w4_dequant(w, _dense_scratch(w.n, w.k, x.device))
        torch.matmul(x, dense.t(), out=out)
        return out
    resident = arm in ("tcr", "tc8r")
    if arm in ("tc8", "tc8r") and x.shape[0] >= DEQUANT_FROM and w.k % 128 == 0:
        from . import gemm_tc

        cached = getattr(w, "_owl_e4m3", None) if resident else None
        if cached is None:
            dense = K.w4_dequant(w, _dense_scratch(w.n, w.k, x.device, torch.float16))
            cached = gemm_tc.quant_e4m3_rows(dense) if resident else gemm_tc.quant_e4m3_rows(dense, *_fp8_scratch("w", w.n, w.k, x.device))
            if resident:
                _ledger(x.device).track("resident e4m3 weight copy", "resident copies", cached[0])
                w._owl_e4m3 = cached
        wq, sw = cached
        xq, sx = gemm_tc.quant_e4m3_rows(x, *_fp8_scratch("x", x.shape[0], w.k, x.device))
        return gemm_tc.e4m3_gemm(xq, sx, wq, sw, out)
    if arm in ("tc", "tc8", "tcr", "tc8r"):
        from . import gemm_tc

        if x.shape[0] <= SKINNY_UPTO and w.layout == "slice":
            # a handful of rows (the tail chunk after the last block boundary): the weight-streaming kernel
            t, k = x.shape
            xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
            xp = torch.empty(t, 2 * k, dtype=torch.uint8, device=x.device)
            xs = torch.empty(t, k // w.group, 2, dtype=torch.float32, device=x.device)
            K.act_pack(xb, xp, xs, t, k, w.group)
            K.w4a16_skinny(w, xp, xs, out, t, ldo=out.stride(0))
            return out
        if x.shape[0] >= DEQUANT_FROM:
            return gemm_tc.f16_gemm(x, w4_dense(w, x.dtype, x.device, resident=resident), out)
        return gemm_tc.w4a16_gemm(w, x, out)
    raise ValueError(f"unknown prefill GEMM arm {arm!r}")


def nvfp4_gemm(w, x: torch.Tensor, out: torch.Tensor, arm: str = "tc") -> torch.Tensor:
    """out[T, N] = x @ dequant(NVFP4 w)^T for a prefill chunk: the weight is dequantised once (bf16) and multiplied on the
    dense tcgen05 GEMM; ``"tc8"`` re-quantises rows to e4m3 and runs the 8-bit float product at twice the rate; ``"tc4"``
    (W4A4) quantises the chunk's activations to NVFP4 with one scale per token and multiplies codes by codes on the
    block-scaled tensor-core path (``ops/nvfp4_tc.py``), with no dense copy of the weight at all; a handful of rows take the
    streaming GEMV."""
    from . import gemm_tc

    t = x.shape[0]
    if arm == "tc4":
        from . import nvfp4_tc

        if t >= nvfp4_tc.MIN_ROWS and w.k % 64 == 0:
            return nvfp4_tc.gemm(w, x, out)
    arm = {"tcr": "tc", "tc8r": "tc8", "tc4": "tc"}.get(arm, arm)       # no resident copies on this path
    if arm != "baseline" and t <= 8:
        K.nvfp4_linear_gemv(w, x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16), out, t)
        return out
    dense = K.nvfp4_linear_dequant(w, _dense_scratch(w.n, w.k, x.device, torch.bfloat16))
    if arm == "baseline":
        torch.matmul(x.to(torch.bfloat16), dense.t(), out=out)
        return out
    if arm == "tc8" and t >= DEQUANT_FROM and w.k % 128 == 0:
        wq, sw = gemm_tc.quant_e4m3_rows(dense, *_fp8_scratch("w", w.n, w.k, x.device))
        xq, sx = gemm_tc.quant_e4m3_rows(x, *_fp8_scratch("x", t, w.k, x.device))
        return gemm_tc.e4m3_gemm(xq, sx, wq, sw, out)
    return gemm_tc.f16_gemm(x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16), dense, out)


def w4_e4m3(w, device):
    """Resident per-row e4m3 copy of a W4 weight: (bytes [N, K], fp32 row scales [N]), created on first use."""
    from . import gemm_tc

    cached = getattr(w, "_owl_e4m3", None)
    if cached is None:
        dense = K.w4_dequant(w, _dense_scratch(w.n, w.k, device, torch.float16))
        _ledger(device).check("resident e4m3 weight copy", w.n * w.k)
        cached = gemm_tc.quant_e4m3_rows(dense)
        _ledger(device).track("resident e4m3 weight copy", "resident copies", cached[0])
        w._owl_e4m3 = cached
    return cached


def w4_dense(w, dtype, device, resident: bool = False) -> torch.Tensor:
    """The weight dequantised into the shared dense scratch matrix (valid until the next call on this stream), or, with
    ``resident``, into a matrix of its own that stays attached to the weight."""
    if resident:
        d = getattr(w, "_owl_dense", None)
        if d is None or d.dtype != dtype:
            # 4x the int4 bytes: a named, budget-checked entry of the device ledger (a profile whose budget cannot hold
            # the copies is refused here, at the first chunk, instead of running the device out of memory later)
            d = K.w4_dequant(w, _ledger(device).alloc("resident dense weight copy", "resident copies", (w.n, w.k), dtype))
            w._owl_dense = d
        return d
    return K.w4_dequant(w, _dense_scratch(w.n, w.k, device, dtype))


def dense_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, arm: str = "tc") -> torch.Tensor:
    """out[T, N] (bf16) = x @ w^T for a small dense bf16 weight (GDN a/b projections, draft heads)."""
    if arm == "baseline":
        torch.matmul(x.to(w.dtype), w.t(), out=out)
        return out
    from . import gemm_tc

    if x.dtype != w.dtype:
        # the converted copy lives on the weight tensor itself (a cache keyed by address would hand a stale copy to the
        # next tensor allocated at that address)
        cache = getattr(w, "_owl_cast", None)
        if cache is None or cache.dtype != x.dtype:
            cache = w.to(x.dtype)
            w._owl_cast = cache
        w = cache
    return gemm_tc.f16_gemm(x, w, out)
