"""Python entry points of the tcgen05 / TMEM GEMM kernels (``csrc/gemm_tc.cu``)."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_void_p

import torch

from . import kernels as K

K.register("owl_w4a16_gemm_tc", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
K.register("owl_f16_gemm_persist", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
K.register("owl_f16_gemm_tc", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
K.register("owl_e4m3_gemm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
K.register("owl_quant_e4m3_rows", [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])


K.register("owl_gemm_dense_set_scratch", [c_void_p, ctypes.c_longlong])
_scratch: dict = {}
KS_SCRATCH_BYTES = 160 * 128 * 256 * 4


def ensure_scratch(device) -> None:
    """Give the dense GEMM its split-K scratch on ``device`` (21 MB, once): a ledger entry of the caller, registered with
    the native library, which never allocates by itself. Called before the first dense GEMM of a device, i.e. before any
    stream capture that contains one."""
    key = str(device)
    if key in _scratch:
        return
    from ..utils.ledger import ledger_for

    dev = torch.device(device)
    buf = ledger_for(dev).alloc("dense GEMM split-K scratch", "workspace", (KS_SCRATCH_BYTES,), torch.uint8)
    with torch.cuda.device(dev):
        K.call("owl_gemm_dense_set_scratch", K.ptr(buf), buf.numel())
    _scratch[key] = buf


def quant_e4m3_rows(x: torch.Tensor, out: torch.Tensor | None = None, scales: torch.Tensor | None = None):
    """Per-row e4m3 quantisation of a 16-bit matrix: returns (bytes [R, K], fp32 scales [R]) with x ~= scale * q."""
    assert x.dtype in (torch.float16, torch.bfloat16) and x.stride(-1) == 1
    r, k = x.shape
    out = torch.empty(r, k, dtype=torch.uint8, device=x.device) if out is None else out
    scales = torch.empty(r, dtype=torch.float32, device=x.device) if scales is None else scales
    K.call("owl_quant_e4m3_rows", K.ptr(x), x.stride(0), int(x.dtype == torch.float16), K.ptr(out), out.stride(0), K.ptr(scales),
           r, k, K.stream())
    return out, scales


def e4m3_gemm(xq: torch.Tensor, sx: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[T, N] (bf16) = (sx[:, None] * sw[None]) * (xq @ wq^T) with e4m3 operands (``tcgen05.mma kind::f8f6f4``)."""
    assert xq.dtype == torch.uint8 and wq.dtype == torch.uint8 and out.dtype == torch.bfloat16
    ensure_scratch(xq.device)
    t, k = xq.shape
    K.call("owl_e4m3_gemm", K.ptr(xq), xq.stride(0), K.ptr(sx), K.ptr(wq), wq.stride(0), K.ptr(sw), K.ptr(out), t, wq.shape[0], k,
           out.stride(0), K.stream())
    return out


def w4a16_gemm(w, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[T, N] (bf16) = x[T, K] (fp16) @ dequant(w)^T on the tcgen05 path."""
    assert x.dtype == torch.float16 and out.dtype == torch.bfloat16 and x.stride(-1) == 1 and out.stride(-1) == 1
    t = x.shape[0]
    K.call("owl_w4a16_gemm_tc", K.ptr(x), x.stride(0), K.ptr(w.records), K.ptr(out), t, w.n, w.k, out.stride(0), w.group,
           w.layout_id, K.stream())
    return out


def f16_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, force_small: bool = False, force_persist: bool = False) -> torch.Tensor:
    """out[T, N] (bf16) = x[T, K] @ w[N, K]^T with fp16 or bf16 operands on the tcgen05 path."""
    assert x.dtype == w.dtype and x.dtype in (torch.float16, torch.bfloat16) and out.dtype == torch.bfloat16
    ensure_scratch(x.device)
    t, k = x.shape
    # long chunks x wide weights: the persistent 128 x 256 kernel; otherwise the 128 x 128 kernel (two CTAs per SM)
    entry = "owl_f16_gemm_persist" if (force_persist or (t >= 256 and w.shape[0] >= 512 and not force_small)) else "owl_f16_gemm_tc"
    K.call(entry, K.ptr(x), x.stride(0), K.ptr(w), w.stride(0), K.ptr(out), t, w.shape[0], k, out.stride(0),
           1 if x.dtype == torch.bfloat16 else 0, K.stream())
    return out


def gemm_status() -> int:
    f = K.fn("owl_gemm_status")
    f.argtypes = []
    g = K.fn("owl_gemm_dense_status")
    g.argtypes = []
    return f() or g()
