"""GGUF container reader, block codecs (CPU oracles), writer for tests, meta -> ModelSpec.

Supported tensor types: F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS,
IQ3_XXS, IQ3_S (codebooks in ``gguf_grids.py``). The IQ2 / IQ1 families need further grids that are not bundled;
such tensors raise ``UnsupportedGgufType`` with the type name instead of decoding wrongly.

``q4k_to_w4`` maps Q4_K super-blocks onto the engine's int4 form without dequantising: every
32-value sub-block becomes a group with scale ``d * sc`` and (fractional) zero point
``dmin * m / (d * sc)``, so the nibbles are streamed as they are.

Reference counterpart: ``crates/models/src/formats/gguf/*.rs`` (container, meta, weight source,
host dequant tables) and ``crates/kernels/cu/gguf/gguf.cuh`` (block layouts).
"""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..ops.quant import W4Canonical

GGML_TYPES = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2_K",
              11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 15: "Q8_K", 16: "IQ2_XXS", 17: "IQ2_XS", 18: "IQ3_XXS",
              19: "IQ1_S", 20: "IQ4_NL", 21: "IQ3_S", 22: "IQ2_S", 23: "IQ4_XS", 24: "I8", 25: "I16", 26: "I32",
              27: "I64", 28: "F64", 29: "IQ1_M", 30: "BF16"}
TYPE_ID = {v: k for k, v in GGML_TYPES.items()}
# name -> (elements per block, bytes per block)
BLOCK = {"F32": (1, 4), "F16": (1, 2), "BF16": (1, 2), "Q8_0": (32, 34), "Q4_0": (32, 18), "Q4_1": (32, 20), "Q5_0": (32, 22),
         "Q5_1": (32, 24), "Q2_K": (256, 84), "Q3_K": (256, 110), "Q4_K": (256, 144), "Q5_K": (256, 176), "Q6_K": (256, 210),
         "IQ4_NL": (32, 18), "IQ4_XS": (256, 136), "IQ3_XXS": (256, 98), "IQ3_S": (256, 110), "I8": (1, 1), "I32": (1, 4)}
KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


class UnsupportedGgufType(NotImplementedError):
    pass


@dataclass
class GgufTensor:
    name: str
    shape: tuple          # logical shape, outermost first (GGUF stores innermost first)
    type: str
    offset: int
    nbytes: int


class GgufFile:
    def __init__(self, path: str | Path):
        """Memory-map the file and read its header. A truncated or corrupted header is reported as one ``ValueError`` naming
        the file, whatever the reader stumbled over; tensors whose data would lie outside the file are refused here too."""
        try:
            self._parse(path)
        except UnsupportedGgufType:
            raise
        except (struct.error, OverflowError, TypeError, IndexError, KeyError, UnicodeDecodeError, RuntimeError, MemoryError) as e:
            raise ValueError(f"{path}: truncated or corrupted GGUF header ({type(e).__name__}: {e})") from None
        size = len(self.mm)
        for t in self.tensors.values():
            if t.offset < 0 or t.nbytes < 0 or t.offset + t.nbytes > size:
                raise ValueError(f"{path}: tensor {t.name} ({t.nbytes} bytes at {t.offset}) lies outside the file ({size} bytes)")

    def _parse(self, path: str | Path) -> None:
        self.path = Path(path)
        self.mm = np.memmap(self.path, dtype=np.uint8, mode="r")
        self.pos = 0
        if bytes(self.mm[:4]) != b"GGUF":
            raise ValueError("not a GGUF file")
        self.pos = 4
        self.version = self._u32()
        n_tensors, n_kv = self._u64(), self._u64()
        self.meta: dict = {}
        for _ in range(n_kv):
            k = self._str()
            self.meta[k] = self._value(self._u32())
        self.tensors: dict[str, GgufTensor] = {}
        infos = []
        for _ in range(n_tensors):
            name = self._str()
            nd = self._u32()
            dims = [self._u64() for _ in range(nd)]
            t = self._u32()
            off = self._u64()
            infos.append((name, tuple(reversed(dims)), t, off))
        align = int(self.meta.get("general.alignment", 32))
        self.data_start = (self.pos + align - 1) // align * align
        for name, shape, t, off in infos:
            tn = GGML_TYPES.get(t, f"type{t}")
            n = math.prod(int(d) for d in shape) if shape else 1          # Python integers: a corrupted dimension cannot wrap
            be, bb = BLOCK.get(tn, (1, 0))
            if len(shape) > 4 or any(d <= 0 for d in shape) or n >= 1 << 48 or n % be:
                raise ValueError(f"{path}: tensor {name} has the impossible shape {tuple(shape)} for type {tn}")
            self.tensors[name] = GgufTensor(name, shape, tn, self.data_start + off, n // be * bb)

    # -- primitive readers ---------------------------------------------------------------------
    def _take(self, fmt: str):
        n = struct.calcsize(fmt)
        v = struct.unpack_from(fmt, self.mm, self.pos)[0]
        self.pos += n
        return v

    def _u32(self): return self._take("<I")
    def _u64(self): return self._take("<Q")

    def _str(self) -> str:
        n = self._u64()
        s = bytes(self.mm[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def _value(self, t: int):
        fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
        if t in fmt:
            return self._take(fmt[t])
        if t == 8:
            return self._str()
        if t == 9:
            et, n = self._u32(), self._u64()
            return [self._value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {t}")

    # -- tensors -------------------------------------------------------------------------------
    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return self.mm[t.offset:t.offset + t.nbytes]

    def dequant(self, name: str) -> torch.Tensor:
        t = self.tensors[name]
        return torch.from_numpy(dequantize(self.raw(name), t.type, int(np.prod(t.shape)))).view(*t.shape)


# ---- codecs ------------------------------------------------------------------------------------
def _f16(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


def _k_scales(sc: np.ndarray):
    """12 packed bytes -> (8 six-bit scales, 8 six-bit mins), vectorised over blocks [nb, 12]."""
    s = np.zeros(sc.shape[:-1] + (8,), dtype=np.float32)
    m = np.zeros_like(s)
    for j in range(4):
        s[..., j] = sc[..., j] & 63
        m[..., j] = sc[..., j + 4] & 63
    for j in range(4, 8):
        s[..., j] = (sc[..., j + 4] & 0xF) | ((sc[..., j - 4] >> 6) << 4)
        m[..., j] = (sc[..., j + 4] >> 4) | ((sc[..., j] >> 6) << 4)
    return s, m


def dequantize(raw: np.ndarray, tname: str, n: int) -> np.ndarray:
    if tname == "F32":
        return raw.view(np.float32).copy()
    if tname == "F16":
        return _f16(raw)
    if tname == "BF16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    if tname not in BLOCK:
        raise UnsupportedGgufType(f"GGUF tensor type {tname}: codebook / layout not bundled")
    be, bb = BLOCK[tname]
    nb = n // be
    b = raw.reshape(nb, bb)
    if tname == "Q8_0":
        return (_f16(b[:, :2].copy()) * b[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)
    if tname == "Q4_0":
        d = _f16(b[:, :2].copy())
        qs = b[:, 2:]
        x = np.concatenate([(qs & 0xF).astype(np.float32) - 8, (qs >> 4).astype(np.float32) - 8], axis=1)
        return (x * d).reshape(-1)
    if tname == "Q4_1":
        d, m = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
        qs = b[:, 4:]
        x = np.concatenate([(qs & 0xF).astype(np.float32), (qs >> 4).astype(np.float32)], axis=1)
        return (x * d + m).reshape(-1)
    if tname in ("Q5_0", "Q5_1"):
        off = 2 if tname == "Q5_0" else 4
        d = _f16(b[:, 0:2].copy())
        qh = b[:, off:off + 4].copy().view(np.uint32)                       # [nb, 1]: bit j = fifth bit of element j
        qs = b[:, off + 4:]
        j = np.arange(16, dtype=np.uint32)
        lo = (qs & 0xF).astype(np.int32) | ((((qh >> j) & 1) << 4).astype(np.int32))
        hi = (qs >> 4).astype(np.int32) | ((((qh >> (j + 16)) & 1) << 4).astype(np.int32))
        x = np.concatenate([lo, hi], axis=1).astype(np.float32)
        if tname == "Q5_0":
            return ((x - 16.0) * d).reshape(-1)
        return (x * d + _f16(b[:, 2:4].copy())).reshape(-1)
    if tname == "Q2_K":
        # scales[16] (low nibble scale, high nibble min) | qs[64] (2 bits) | d | dmin; two halves of 128, each 4 shifts x 2 x 16
        sc = b[:, 0:16]
        qs = b[:, 16:80].reshape(nb, 2, 32)
        d, dmin = _f16(b[:, 80:82].copy()), _f16(b[:, 82:84].copy())
        out = np.zeros((nb, 2, 4, 32), dtype=np.float32)
        for h in range(2):
            for j in range(4):
                q = ((qs[:, h] >> (2 * j)) & 3).astype(np.float32)             # [nb, 32]
                for half in range(2):
                    s8 = sc[:, h * 8 + j * 2 + half]
                    dl = d[:, 0] * (s8 & 0xF)
                    ml = dmin[:, 0] * (s8 >> 4)
                    out[:, h, j, half * 16:(half + 1) * 16] = dl[:, None] * q[:, half * 16:(half + 1) * 16] - ml[:, None]
        return out.reshape(-1)
    if tname == "Q3_K":
        # hmask[32] | qs[64] | scales[12] (sixteen 6-bit scales) | d
        hm = b[:, 0:32]
        qs = b[:, 32:96].reshape(nb, 2, 32)
        sc12 = b[:, 96:108].astype(np.uint32)
        d = _f16(b[:, 108:110].copy())[:, 0]
        aux = sc12[:, 0:4] | (sc12[:, 4:8] << 8)
        a0 = sc12[:, 0] | (sc12[:, 1] << 8) | (sc12[:, 2] << 16) | (sc12[:, 3] << 24)
        a1 = sc12[:, 4] | (sc12[:, 5] << 8) | (sc12[:, 6] << 16) | (sc12[:, 7] << 24)
        tmp = sc12[:, 8] | (sc12[:, 9] << 8) | (sc12[:, 10] << 16) | (sc12[:, 11] << 24)
        k1, k2 = np.uint32(0x03030303), np.uint32(0x0f0f0f0f)
        w = [(a0 & k2) | (((tmp >> 0) & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
             ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)]
        scales = np.stack([((w[i] >> (8 * j)) & 0xFF) for i in range(4) for j in range(4)], axis=1).astype(np.int32) - 32   # [nb, 16]
        del aux
        out = np.zeros((nb, 2, 4, 32), dtype=np.float32)
        is_ = 0
        for h in range(2):
            for j in range(4):
                m = np.uint8(1 << (h * 4 + j))
                q = ((qs[:, h] >> (2 * j)) & 3).astype(np.int32) - np.where(hm & m, 0, 4)
                for half in range(2):
                    dl = d * scales[:, is_]
                    is_ += 1
                    out[:, h, j, half * 16:(half + 1) * 16] = dl[:, None] * q[:, half * 16:(half + 1) * 16]
        return out.reshape(-1)
    if tname == "IQ3_XXS":
        # d | qs[64] (grid indices, 8 per 32 values) | 8 x u32 (four 7-bit sign fields, top 4 bits = sub-block scale)
        from .gguf_grids import IQ3XXS_GRID, KSIGNS

        d = _f16(b[:, 0:2].copy())[:, 0]
        q3 = b[:, 2:66].reshape(nb, 8, 8)
        aux = b[:, 66:98].copy().view(np.uint32).reshape(nb, 8)
        out = np.zeros((nb, 8, 4, 8), dtype=np.float32)
        bit = (1 << np.arange(8)).astype(np.uint8)
        for ib in range(8):
            db = d * (0.5 + (aux[:, ib] >> 28).astype(np.float32)) * 0.5
            for l in range(4):
                signs = KSIGNS[(aux[:, ib] >> (7 * l)) & 127]                       # [nb]
                g = np.concatenate([IQ3XXS_GRID[q3[:, ib, 2 * l]], IQ3XXS_GRID[q3[:, ib, 2 * l + 1]]], axis=1).astype(np.float32)
                sg = np.where(signs[:, None] & bit[None, :], -1.0, 1.0)
                out[:, ib, l] = db[:, None] * g * sg
        return out.reshape(-1)
    if tname == "IQ3_S":
        # d | qs[64] | qh[8] | signs[32] | scales[4]
        from .gguf_grids import IQ3S_GRID

        d = _f16(b[:, 0:2].copy())[:, 0]
        qs = b[:, 2:66].reshape(nb, 8, 8).astype(np.int32)
        qh = b[:, 66:74].astype(np.int32)
        signs = b[:, 74:106].reshape(nb, 8, 4)
        scl = b[:, 106:110]
        out = np.zeros((nb, 8, 4, 8), dtype=np.float32)
        bit = (1 << np.arange(8)).astype(np.uint8)
        for ib in range(8):
            nib = (scl[:, ib // 2] >> (4 * (ib % 2))) & 0xF
            db = d * (1 + 2 * nib.astype(np.float32))
            for l in range(4):
                i1 = qs[:, ib, 2 * l] | ((qh[:, ib] << (8 - 2 * l)) & 256)
                i2 = qs[:, ib, 2 * l + 1] | ((qh[:, ib] << (7 - 2 * l)) & 256)
                g = np.concatenate([IQ3S_GRID[i1], IQ3S_GRID[i2]], axis=1).astype(np.float32)
                sg = np.where(signs[:, ib, l][:, None] & bit[None, :], -1.0, 1.0)
                out[:, ib, l] = db[:, None] * g * sg
        return out.reshape(-1)
    if tname == "IQ4_NL":
        d = _f16(b[:, :2].copy())
        qs = b[:, 2:]
        x = np.concatenate([KVALUES_IQ4NL[qs & 0xF], KVALUES_IQ4NL[qs >> 4]], axis=1)
        return (x * d).reshape(-1)
    if tname == "Q4_K":
        d, dmin = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
        s, m = _k_scales(b[:, 4:16])
        qs = b[:, 16:].reshape(nb, 4, 32)
        q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)
        return (d[:, :, None] * s[:, :, None] * q - dmin[:, :, None] * m[:, :, None]).reshape(-1)
    if tname == "Q5_K":
        d, dmin = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
        s, m = _k_scales(b[:, 4:16])
        qh = b[:, 16:48]
        qs = b[:, 48:].reshape(nb, 4, 32)
        lo, hi = (qs & 0xF).astype(np.int32), (qs >> 4).astype(np.int32)
        for j in range(4):
            lo[:, j] += ((qh >> (2 * j)) & 1).astype(np.int32) * 16
            hi[:, j] += ((qh >> (2 * j + 1)) & 1).astype(np.int32) * 16
        q = np.stack([lo, hi], axis=2).reshape(nb, 8, 32).astype(np.float32)
        return (d[:, :, None] * s[:, :, None] * q - dmin[:, :, None] * m[:, :, None]).reshape(-1)
    if tname == "Q6_K":
        ql, qh = b[:, :128].reshape(nb, 2, 64), b[:, 128:192].reshape(nb, 2, 32)
        sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(nb, 2, 8)
        d = _f16(b[:, 208:210].copy())
        out = np.zeros((nb, 2, 128), dtype=np.float32)
        l = np.arange(32)
        isx = l // 16
        for h in range(2):
            q1 = ((ql[:, h, :32] & 0xF) | (((qh[:, h] >> 0) & 3) << 4)).astype(np.int32) - 32
            q2 = ((ql[:, h, 32:] & 0xF) | (((qh[:, h] >> 2) & 3) << 4)).astype(np.int32) - 32
            q3 = ((ql[:, h, :32] >> 4) | (((qh[:, h] >> 4) & 3) << 4)).astype(np.int32) - 32
            q4 = ((ql[:, h, 32:] >> 4) | (((qh[:, h] >> 6) & 3) << 4)).astype(np.int32) - 32
            out[:, h, 0:32] = sc[:, h][:, isx + 0] * q1
            out[:, h, 32:64] = sc[:, h][:, isx + 2] * q2
            out[:, h, 64:96] = sc[:, h][:, isx + 4] * q3
            out[:, h, 96:128] = sc[:, h][:, isx + 6] * q4
        return (out * d[:, :, None]).reshape(-1)
    if tname == "IQ4_XS":
        d = _f16(b[:, 0:2].copy())
        sh = b[:, 2:4].copy().view(np.uint16).astype(np.int32)          # [nb, 1]
        sl = b[:, 4:8].astype(np.int32)
        qs = b[:, 8:].reshape(nb, 8, 16)
        ib = np.arange(8)
        ls = ((sl[:, ib // 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)
        dl = d * (ls.astype(np.float32) - 32)
        x = np.concatenate([KVALUES_IQ4NL[qs & 0xF], KVALUES_IQ4NL[qs >> 4]], axis=2)
        return (x * dl[:, :, None]).reshape(-1)
    raise UnsupportedGgufType(tname)


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    b = w.reshape(-1, 32).astype(np.float32)
    d = np.abs(b).max(1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(b / np.where(d > 0, d, 1)), 0).astype(np.int8)
    out = np.zeros((b.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """Simple (round-to-nearest, min/max per sub-block) Q4_K encoder for synthetic checkpoints."""
    b = w.reshape(-1, 8, 32).astype(np.float32)
    nb = b.shape[0]
    mn = np.minimum(b.min(2), 0.0)
    sc = (b.max(2) - mn) / 15.0
    d = sc.max(1, keepdims=True) / 63.0
    dmin = (-mn).max(1, keepdims=True) / 63.0
    d16, dm16 = d.astype(np.float16), dmin.astype(np.float16)
    df, dmf = d16.astype(np.float32), dm16.astype(np.float32)
    s6 = np.clip(np.round(np.where(df > 0, sc / np.where(df > 0, df, 1), 0)), 0, 63).astype(np.uint8)
    m6 = np.clip(np.round(np.where(dmf > 0, -mn / np.where(dmf > 0, dmf, 1), 0)), 0, 63).astype(np.uint8)
    es, em = df * s6, dmf * m6
    q = np.clip(np.round(np.where(es[:, :, None] > 0, (b + em[:, :, None]) / np.where(es > 0, es, 1)[:, :, None], 0)),
                0, 15).astype(np.uint8)
    out = np.zeros((nb, 144), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = dm16.view(np.uint8).reshape(nb, 2)
    scb = np.zeros((nb, 12), dtype=np.uint8)
    for j in range(4):
        scb[:, j] = (s6[:, j] & 63) | ((s6[:, j + 4] >> 4) << 6)
        scb[:, j + 4] = (m6[:, j] & 63) | ((m6[:, j + 4] >> 4) << 6)
        scb[:, j + 8] = (s6[:, j + 4] & 0xF) | ((m6[:, j + 4] & 0xF) << 4)
    out[:, 4:16] = scb
    qq = q.reshape(nb, 4, 2, 32)
    out[:, 16:] = (qq[:, :, 0] | (qq[:, :, 1] << 4)).reshape(nb, 128)
    return out.reshape(-1)


def q4k_to_w4(raw: np.ndarray, n_rows: int, k: int) -> W4Canonical:
    """Q4_K tensor [n_rows, k] -> W4 canonical with group 32 (no dequantisation of the nibbles)."""
    nb = n_rows * k // 256
    b = raw.reshape(nb, 144)
    d, dmin = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
    s, m = _k_scales(b[:, 4:16])
    qs = b[:, 16:].reshape(nb, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(n_rows, k)
    es = (d * s).reshape(n_rows, k // 32)
    em = (dmin * m).reshape(n_rows, k // 32)
    safe = np.where(es > 0, es, 1e-7)                    # a dead sub-block keeps only its (tiny) offset
    zero = em / safe
    return W4Canonical(torch.from_numpy(q.astype(np.uint8)), torch.from_numpy(safe.astype(np.float16)),
                       torch.from_numpy(np.clip(zero, 0, 65504).astype(np.float16)), 32)


# ---- writer (tests / synthetic checkpoints) ---------------------------------------------------
def write_gguf(path, meta: dict, tensors: dict, align: int = 32) -> None:
    """``tensors``: name -> (shape, type name, raw bytes as np.uint8)."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<IQ", 10, v) if v >= 2**32 else struct.pack("<II", 4, v)
        if isinstance(v, float):
            return struct.pack("<If", 6, v)
        if isinstance(v, str):
            return struct.pack("<I", 8) + s(v)
        if isinstance(v, list):
            et = 8 if v and isinstance(v[0], str) else 6 if v and isinstance(v[0], float) else 5
            body = b"".join(s(x) if et == 8 else struct.pack("<f" if et == 6 else "<i", x) for x in v)
            return struct.pack("<IIQ", 9, et, len(v)) + body
        raise TypeError(type(v))

    meta = dict(meta)
    meta.setdefault("general.alignment", align)
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, v in meta.items():
        head += s(k) + val(v)
    off = 0
    infos, blobs = b"", []
    for name, (shape, tname, raw) in tensors.items():
        infos += s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape))
        infos += struct.pack("<IQ", TYPE_ID[tname], off)
        pad = (-len(raw)) % align
        blobs.append(bytes(raw) + b"\0" * pad)
        off += len(raw) + pad
    pre = head + infos
    pre += b"\0" * ((-len(pre)) % align)
    with open(path, "wb") as f:
        f.write(pre)
        for b in blobs:
            f.write(b)


# ---- metadata -> model spec, tokenizer --------------------------------------------------------
def spec_from_meta(meta: dict):
    from ..models.spec import ModelSpec

    arch = meta.get("general.architecture", "qwen35")
    g = lambda k, d=None: meta.get(f"{arch}.{k}", d)
    hd = int(g("attention.key_length", 256))
    return ModelSpec(name=meta.get("general.name", arch), vocab=int(g("vocab_size", len(meta.get("tokenizer.ggml.tokens", [])) or 151936)),
                     hidden=int(g("embedding_length")), inter=int(g("feed_forward_length")), n_layers=int(g("block_count")),
                     hq=int(g("attention.head_count")), hkv=int(g("attention.head_count_kv")), hd=hd,
                     rotary_dim=int(g("rope.dimension_count", hd // 4)), rope_theta=float(g("rope.freq_base", 1e7)),
                     nk=int(g("ssm.group_count", 16)), kd=int(g("ssm.state_size", 128)),
                     nv=int(g("ssm.time_step_rank", 48)), vd=int(g("ssm.state_size", 128)),
                     full_every=int(g("full_attention_interval", 4)), eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)))


def tokenizer_from_meta(meta: dict) -> dict:
    return {"model": meta.get("tokenizer.ggml.model", "gpt2"), "tokens": meta.get("tokenizer.ggml.tokens", []),
            "merges": meta.get("tokenizer.ggml.merges", []), "eos": meta.get("tokenizer.ggml.eos_token_id"),
            "bos": meta.get("tokenizer.ggml.bos_token_id"), "chat_template": meta.get("tokenizer.chat_template", "")}
