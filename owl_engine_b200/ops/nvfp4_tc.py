"""NVFP4 x NVFP4 products on the block-scaled tensor-core path (``csrc/gemm_nvfp4.cu``, ``tcgen05.mma kind::mxf4nvf4``).

The weight's e2m1 codes are read as the checkpoint stores them; its e4m3 block scales are re-ordered ONCE into the MMA's
atom order (``formats/nvfp4.pack_sf_atoms``, 1/8 of the code bytes, a ledger entry) and kept on the weight object. The
activations of a prefill chunk are quantised per call to the same format with one fp32 scale per token row
(``owl_nvfp4_quant_rows``) into a per-device scratch.

Reference counterpart: ``crates/kernels/cu/nvfp4/nvfp4_gemm.cu`` + ``nvfp4_quant_act.cu`` (W4A4 from 128 rows up).
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import kernels as K

K.register("owl_nvfp4_quant_rows", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
K.register("owl_nvfp4_gemm", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_int, c_void_p])

MIN_ROWS = 128          # rows from which the W4A4 product is used (below: the 16-bit arms)
_scratch: dict = {}


def sf_bytes(rows: int, k: int) -> int:
    return ((rows + 127) // 128) * ((k + 255) // 256) * 2048


def weight_atoms(w) -> torch.Tensor:
    """The weight's block scales in atom order (created on first use, tracked in the device ledger)."""
    a = getattr(w, "_owl_sf_atoms", None)
    if a is None:
        from ..formats import nvfp4
        from ..utils.ledger import ledger_for

        a = nvfp4.pack_sf_atoms(w.scales.view(w.n, w.k // 16))
        ledger_for(w.codes.device).track("nvfp4 scale atoms", "resident copies", a)
        w._owl_sf_atoms = a
    return a


def quant_rows(x: torch.Tensor, codes: torch.Tensor | None = None, sf: torch.Tensor | None = None, sx: torch.Tensor | None = None):
    """x bf16 or fp16 ``[T, K]`` -> (codes uint8 ``[T, K/2]``, scale atoms uint8, fp32 row scales ``[T]``). ``sf`` must have been
    zero-filled once (the k padding of the atoms is never written)."""
    assert x.dtype in (torch.bfloat16, torch.float16) and x.stride(-1) == 1
    t, k = x.shape
    codes = torch.empty(t, k // 2, dtype=torch.uint8, device=x.device) if codes is None else codes
    sf = torch.zeros(sf_bytes(t, k), dtype=torch.uint8, device=x.device) if sf is None else sf
    sx = torch.empty(t, dtype=torch.float32, device=x.device) if sx is None else sx
    K.call("owl_nvfp4_quant_rows", K.ptr(x), x.stride(0), int(x.dtype == torch.float16), K.ptr(codes), K.ptr(sf), K.ptr(sx), t, k, K.stream())
    return codes, sf, sx


def _act_scratch(t: int, k: int, device):
    """Per-device activation scratch, grown on demand (ledger entry "nvfp4 act scratch"); the atom buffer is re-zeroed when
    k changes, since another k leaves other padding positions unwritten."""
    from ..utils.ledger import ledger_for

    key = str(device)
    ent = _scratch.get(key)
    need_c, need_s = t * (k // 2), sf_bytes(t, k)
    if ent is None or ent["codes"].numel() < need_c or ent["sf"].numel() < need_s or ent["sx"].numel() < t:
        led = ledger_for(device)
        if ent is not None:
            led.release("nvfp4 act scratch")
            need_c, need_s, t_cap = max(need_c, ent["codes"].numel()), max(need_s, ent["sf"].numel()), max(t, ent["sx"].numel())
        else:
            t_cap = t
        codes = led.alloc("nvfp4 act scratch", "workspace", (need_c + need_s,), torch.uint8)
        ent = {"codes": codes[:need_c], "sf": codes[need_c:], "sx": torch.empty(t_cap, dtype=torch.float32, device=device), "k": -1}
        _scratch[key] = ent
    if ent["k"] != k:
        ent["sf"].zero_()
        ent["k"] = k
    return ent["codes"][:t * (k // 2)].view(t, k // 2), ent["sf"], ent["sx"][:t]


def gemm(w, x: torch.Tensor, out: torch.Tensor, xq=None) -> torch.Tensor:
    """out[T, N] (bf16) = x @ dequant(w)^T with both operands in NVFP4. ``xq``: an already quantised activation triple
    (several projections of one input share it)."""
    assert out.dtype == torch.bfloat16 and out.stride(-1) == 1 and w.k % 64 == 0
    t = x.shape[0]
    if xq is None:
        xq = quant_rows(x, *_act_scratch(t, w.k, x.device))
    codes, sf, sx = xq
    K.call("owl_nvfp4_gemm", K.ptr(codes), K.ptr(sf), K.ptr(sx), K.ptr(w.codes), K.ptr(weight_atoms(w)), float(w.alpha),
           K.ptr(w.row_scale) if w.row_scale is not None else None, K.ptr(out), t, w.n, w.k, out.stride(0), K.stream())
    return out


def status() -> int:
    f = K.fn("owl_gemm_nvfp4_status")
    f.argtypes = []
    return int(f())
