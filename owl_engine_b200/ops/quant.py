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
    zeros: torch.Tensor    # uint8 [N, K/G] (fp16 with fractional values for GGUF K-quant sources)
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


K_SLICES = 8   # record streams are stored slice-major: [slice][row tile][record in slice]


def _slice_bounds(kt: int):
    return [(w * kt) // K_SLICES for w in range(K_SLICES + 1)]


def to_slice_major(rec: torch.Tensor) -> torch.Tensor:
    """[NT, KT, REC] -> flat bytes ordered [slice w][nt][kt in slice w] (slice w = record columns
    [w*KT/8, (w+1)*KT/8)), so that one warp of the streaming kernel reads one contiguous range."""
    nt, kt, r = rec.shape
    b = _slice_bounds(kt)
    return torch.cat([rec[:, b[w]:b[w + 1], :].reshape(-1) for w in range(K_SLICES)])


def from_slice_major(flat: torch.Tensor, nt: int, kt: int, r: int) -> torch.Tensor:
    b = _slice_bounds(kt)
    out = torch.empty(nt, kt, r, dtype=flat.dtype, device=flat.device)
    off = 0
    for w in range(K_SLICES):
        n = nt * (b[w + 1] - b[w]) * r
        out[:, b[w]:b[w + 1], :] = flat[off:off + n].view(nt, b[w + 1] - b[w], r)
        off += n
    return out


def record_offset(nt_total: int, kt_total: int, rec_bytes: int, nt: int, kt: int) -> int:
    """Byte offset of record (nt, kt) in a slice-major stream (host mirror of the device formula)."""
    b = _slice_bounds(kt_total)
    w = max(i for i in range(K_SLICES) if b[i] <= kt and b[i] < b[i + 1] or i == 0)
    while not (b[w] <= kt < b[w + 1]):
        w += 1
    return (nt_total * b[w] + nt * (b[w + 1] - b[w]) + (kt - b[w])) * rec_bytes


# Inside a 32-bit word of 8 nibbles, k_local j sits at nibble position _NIB_OF_K[j], so that
# (q & 0x000F000F) yields the pair (k0, k1), (q & 0x00F000F0) the pair (k2, k3), and the same on
# q >> 8 the pairs (k4, k5), (k6, k7): dequantised halves come out in k order.
_NIB_OF_K = [0, 4, 1, 5, 2, 6, 3, 7]
_K_OF_NIB = [0, 2, 4, 6, 1, 3, 5, 7]


@dataclass
class W4Skinny:
    """Device-ready W4 weight: a flat stream of ``N/16 x K/128`` records of ``1024 + 64*(128/G)``
    bytes. Each record is 1024 bytes of nibbles followed by the (scale, zero) half2 pairs of its
    groups. ``layout`` is the record order: "slice" (k-slice major, read by the legacy streaming
    kernels) or "block" ([128-row block][k-record][row tile], row tiles padded to a multiple of 8
    with zero records; read by the tcgen05 streaming kernel as one contiguous run per CTA)."""
    records: torch.Tensor
    n: int
    k: int
    group: int
    layout: str = "slice"

    def to(self, device):
        return W4Skinny(self.records.to(device), self.n, self.k, self.group, self.layout)

    @property
    def layout_id(self) -> int:
        return 1 if self.layout == "block" else 0

    @property
    def nbytes(self) -> int:
        return self.records.numel()

    @property
    def rec_bytes(self) -> int:
        return 1024 + 64 * (128 // self.group)


@dataclass
class NvFp4Linear:
    """Device-ready NVFP4 weight as stored in the checkpoint: e2m1 codes ``[N, K/2]`` (two per byte, low nibble first),
    e4m3 block scales ``[N, K/16]`` and the per-tensor scale ``alpha``. Row order is the model's (gate / up rows interleaved
    in eights for the merged MLP projection, like every other weight format here)."""
    codes: torch.Tensor
    scales: torch.Tensor
    alpha: float
    n: int
    k: int
    group: int = 128          # ActPack group of the activations this weight is fed from
    layout: str = "nvfp4"
    row_scale: torch.Tensor = None   # fp32 [N] (multiplied with alpha): set when rows of several tensors were merged

    @property
    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel()


def nvfp4_linear(w: torch.Tensor, device, group: int = 128) -> NvFp4Linear:
    """Quantise a dense ``[N, K]`` weight to NVFP4 (CPU oracle codec) and move it to the device."""
    from ..formats import nvfp4

    q = nvfp4.quantize(w.float())
    return NvFp4Linear(q.codes.to(device), q.scales.to(device), q.global_scale, w.shape[0], w.shape[1], group)


def random_nvfp4(n: int, k: int, device, std: float = 0.02, seed: int = 0, group: int = 128) -> NvFp4Linear:
    """Random NVFP4 weight generated directly on the device (benchmark initialisation): uniform codes, block scales near one
    e4m3 value, ``alpha`` chosen so that the dequantised values have standard deviation about ``std``."""
    gen = torch.Generator(device=device).manual_seed(seed)
    codes = torch.randint(0, 256, (n, k // 2), device=device, generator=gen, dtype=torch.uint8)
    sc = (torch.rand(n, k // 16, device=device, generator=gen) * 64.0 + 192.0).to(torch.float8_e4m3fn).view(torch.uint8)
    # e2m1 magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}: rms 2.97; mean block scale 224
    return NvFp4Linear(codes, sc, std / (2.97 * 224.0), n, k, group)


def to_block_major(rec: torch.Tensor) -> torch.Tensor:
    """[NT, KT, REC] -> flat bytes ordered [row block][kt][row tile in block (8)], zero records appended
    so that NT becomes a multiple of 8."""
    nt, kt, r = rec.shape
    nrb = (nt + 7) // 8
    if nrb * 8 != nt:
        rec = torch.cat([rec, torch.zeros(nrb * 8 - nt, kt, r, dtype=rec.dtype, device=rec.device)])
    return rec.view(nrb, 8, kt, r).permute(0, 2, 1, 3).reshape(-1).contiguous()


def from_block_major(flat: torch.Tensor, nt: int, kt: int, r: int) -> torch.Tensor:
    nrb = (nt + 7) // 8
    return flat.view(nrb, kt, 8, r).permute(0, 2, 1, 3).reshape(nrb * 8, kt, r)[:nt].contiguous()


def pack_skinny(c: W4Canonical, layout: str = "slice") -> W4Skinny:
    n, k = c.q.shape
    assert n % 16 == 0 and k % 128 == 0, (n, k)
    nt, kt = n // 16, k // 128
    # q[nt*16 + half*8 + g, kt*128 + w*32 + t*8 + j] -> tiles[nt, kt, half, g, t, w, nibble NIB[j]]
    v = c.q.view(nt, 2, 8, kt, 4, 4, 8).permute(0, 3, 1, 2, 5, 4, 6)[..., _K_OF_NIB].contiguous()
    lo, hi = v[..., 0::2], v[..., 1::2]
    tiles = (lo | (hi << 4)).to(torch.uint8).reshape(nt, kt, 1024)
    kg = k // c.group
    gpt = 128 // c.group
    sz = torch.stack([c.scales.view(nt, 16, kg).permute(0, 2, 1),
                      c.zeros.view(nt, 16, kg).permute(0, 2, 1).to(torch.float16)], dim=-1).contiguous()
    szb = sz.view(torch.uint8).reshape(nt, kt, gpt * 64)
    rec = torch.cat([tiles, szb], dim=-1)
    return W4Skinny(to_block_major(rec) if layout == "block" else to_slice_major(rec), n, k, c.group, layout)


def unpack_skinny(s: W4Skinny) -> W4Canonical:
    nt, kt = s.n // 16, s.k // 128
    gpt = 128 // s.group
    rec = (from_block_major if s.layout == "block" else from_slice_major)(s.records, nt, kt, s.rec_bytes)
    b = rec[..., :1024].reshape(nt, kt, 2, 8, 4, 4, 4)
    sz = rec[..., 1024:].contiguous().view(torch.float16).reshape(nt, kt * gpt, 16, 2)
    v = torch.stack([b & 0xF, b >> 4], dim=-1).reshape(nt, kt, 2, 8, 4, 4, 8)[..., _NIB_OF_K]
    q = v.permute(0, 2, 3, 1, 5, 4, 6).reshape(s.n, s.k).contiguous()
    kg = s.k // s.group
    scales = sz[..., 0].permute(0, 2, 1).reshape(s.n, kg).contiguous()
    zeros = sz[..., 1].permute(0, 2, 1).reshape(s.n, kg).contiguous()
    if bool((zeros == zeros.round()).all()):      # integer zero points (AWQ); GGUF-derived ones are fractional
        zeros = zeros.to(torch.uint8)
    return W4Canonical(q, scales, zeros, s.group)


def random_skinny(n: int, k: int, group: int, device, std: float = 0.02, seed: int = 0, layout: str = "slice") -> W4Skinny:
    """Random W4 weight generated directly in the device layout (benchmark initialisation).

    Equivalent to quantising N(0, std) weights: nibbles are drawn from a rounded normal around
    the zero-point 8 with a scale chosen so the dequantised values have standard deviation std.
    """
    gen = torch.Generator(device=device).manual_seed(seed)
    nt, kt = n // 16, k // 128
    if layout == "block":
        nt = (nt + 7) // 8 * 8        # padded row tiles are never stored, so their content is free
    vals = (torch.randn(nt, kt, 2048, device=device, generator=gen) * 2.5 + 8.0).round().clamp_(0, 15).to(torch.uint8)
    tiles = (vals[..., 0::2] | (vals[..., 1::2] << 4)).contiguous()
    kg = k // group
    gpt = 128 // group
    sz = torch.empty(nt, kg, 16, 2, dtype=torch.float16, device=device)
    sz[..., 0] = (std / 2.5) * (1.0 + 0.1 * torch.rand(nt, kg, 16, device=device, generator=gen))
    sz[..., 1] = torch.randint(7, 10, (nt, kg, 16), device=device, generator=gen).to(torch.float16)
    szb = sz.view(torch.uint8).reshape(nt, kt, gpt * 64)
    # a random stream is layout-agnostic: any record order is an equally random weight
    return W4Skinny(torch.cat([tiles, szb], dim=-1).reshape(-1).contiguous(), n, k, group, layout)


def pack_dense_bf16(w: torch.Tensor) -> torch.Tensor:
    """Dense bf16 ``[N, K]`` -> skinny records ``[N/16, K/64, 2048]`` bytes (see csrc/gemv.cu):
    uint4 #((s*2+half)*32 + g*4+t) holds row half*8+g, k = s*32 + t*8 .. +7."""
    n, k = w.shape
    assert n % 16 == 0 and k % 64 == 0, (n, k)
    v = w.to(torch.bfloat16).view(n // 16, 2, 8, k // 64, 2, 4, 8)      # nt, half, g, kt, s, t, e
    v = v.permute(0, 3, 4, 1, 2, 5, 6).contiguous()                      # nt, kt, s, half, g, t, e
    return to_slice_major(v.view(torch.uint8).reshape(n // 16, k // 64, 2048))


def unpack_dense_bf16(rec: torch.Tensor, n: int, k: int) -> torch.Tensor:
    rec = from_slice_major(rec, n // 16, k // 64, 2048)
    v = rec.contiguous().view(torch.bfloat16).reshape(n // 16, k // 64, 2, 2, 8, 4, 8)
    return v.permute(0, 3, 4, 1, 2, 5, 6).reshape(n, k)


def pack_dense_int8(q: torch.Tensor) -> torch.Tensor:
    """int8 ``[N, K]`` -> records ``[N/16, K/128, 2048]``: uint4 #((s*2+half)*32 + g*4+t) holds
    row half*8+g, k = s*64 + t*16 .. +15."""
    n, k = q.shape
    assert n % 16 == 0 and k % 128 == 0, (n, k)
    v = q.view(n // 16, 2, 8, k // 128, 2, 4, 16).permute(0, 3, 4, 1, 2, 5, 6).contiguous()
    return to_slice_major(v.view(torch.uint8).reshape(n // 16, k // 128, 2048))


@dataclass
class DenseSkinny:
    """Dense weight in skinny-record layout. ``kind`` is "bf16" or "int8" (``row_scale`` set)."""
    records: torch.Tensor
    n: int
    k: int
    kind: str = "bf16"
    row_scale: torch.Tensor = None

    @property
    def nbytes(self) -> int:
        return self.records.numel()

    @property
    def shape(self):
        return (self.n, self.k)


def dense_skinny(w: torch.Tensor, device=None, int8: bool = False) -> DenseSkinny:
    n, k = w.shape
    if int8:
        q, s = quantize_w8_rows(w)
        d = DenseSkinny(pack_dense_int8(q), n, k, "int8", s)
    else:
        d = DenseSkinny(pack_dense_bf16(w), n, k, "bf16")
    if device is not None:
        d.records = d.records.to(device)
        if d.row_scale is not None:
            d.row_scale = d.row_scale.to(device)
    return d


# ---- ActPack -----------------------------------------------------------------------------
def act_pack_ref(x: torch.Tensor, group: int):
    """fp32 reference of the ActPack producer (see ``csrc/actpack.cuh``).

    Returns ``(xpack uint8 [M, 2K], xs fp32 [M, K/G, 2])``. Activations are 15-bit fixed point,
    ``x = sx * (128 h + l)`` (h signed byte, l in 0..127), one scale per (token, group). Every run of
    8 consecutive k is one 16-byte chunk ``[h(a) x4 | l(a) x4 | h(c) x4 | l(c) x4]`` where for weight
    byte b, a = x[{0,4,1,5}[b]] (low nibble) and c = x[{2,6,3,7}[b]] (high nibble);
    ``xs = (sx, xsum)``."""
    m, k = x.shape
    v = x.to(torch.float32).view(m, k // 8, 8)
    a, c = v[..., [0, 4, 1, 5]], v[..., [2, 6, 3, 7]]
    cpg = group // 8
    amax = torch.maximum(a.abs(), c.abs()).amax(-1).view(m, k // group, cpg).amax(-1)
    sx = amax.clamp_min(1e-30) * torch.tensor(1.0 / 16383.0, dtype=torch.float32)
    inv = (1.0 / sx).repeat_interleave(cpg, dim=1)[..., None]
    qa = torch.round(a * inv).to(torch.int32)
    qc = torch.round(c * inv).to(torch.int32)
    planes = torch.stack([(qa >> 7) & 0xFF, qa & 0x7F, (qc >> 7) & 0xFF, qc & 0x7F], dim=2)   # [m, chunks, 4, 4]
    xpack = planes.to(torch.uint8).reshape(m, 2 * k)
    xsum = (a + c).sum(-1).view(m, k // group, cpg).sum(-1)
    return xpack, torch.stack([sx, xsum], dim=-1)


def act_pack_tiles_ref(x: torch.Tensor, group: int) -> torch.Tensor:
    """ActPack of ``x`` [M <= 8, K] in the tile layout (see ``csrc/actpack.cuh``): per 128-k record
    ``[4 steps][2 k halves][16 columns][16 B]`` + ``[128/G groups][8 tokens]`` float2 (sx, xsum); flat uint8.
    Bytes of token slots >= M are zero here (the kernels leave them untouched)."""
    m, k = x.shape
    assert m <= 8
    xp, xs = act_pack_ref(x, group)
    gpt = 128 // group
    kt_n = k // 128
    chunks = xp.view(m, kt_n, 4, 4, 4, 4)                     # m, kt, w, t, plane(ha,la,hc,lc), 4 bytes
    tile = torch.zeros(kt_n, 4, 2, 16, 16, dtype=torch.uint8)  # kt, w, k half, column, byte
    for mm in range(m):
        for t in range(4):
            kc, off = t >> 1, (t & 1) * 8
            tile[:, :, kc, mm, off:off + 4] = chunks[mm, :, :, t, 0]          # h(a)
            tile[:, :, kc, mm, off + 4:off + 8] = chunks[mm, :, :, t, 2]      # h(c)
            tile[:, :, kc, 8 + mm, off:off + 4] = chunks[mm, :, :, t, 1]      # l(a)
            tile[:, :, kc, 8 + mm, off + 4:off + 8] = chunks[mm, :, :, t, 3]  # l(c)
    sc = torch.zeros(kt_n, gpt, 8, 2, dtype=torch.float32)
    sc[:, :, :m] = xs.view(m, kt_n, gpt, 2).permute(1, 2, 0, 3)
    return torch.cat([tile.reshape(kt_n, 2048), sc.view(torch.uint8).reshape(kt_n, gpt * 64)], dim=1).reshape(-1)


def act_unpack_ref(xpack: torch.Tensor, xs: torch.Tensor, group: int) -> torch.Tensor:
    """Inverse of ``act_pack_ref`` up to the fixed-point rounding: fp32 activations [M, K]."""
    m = xpack.shape[0]
    p = xpack.view(m, -1, 4, 4).to(torch.int32)
    def val(h, l):
        h = torch.where(h >= 128, h - 256, h)
        return (h * 128 + l).to(torch.float32)
    cpg = group // 8
    sx = xs[..., 0].repeat_interleave(cpg, dim=1)[..., None]
    a, c = val(p[:, :, 0], p[:, :, 1]) * sx, val(p[:, :, 2], p[:, :, 3]) * sx
    out = torch.empty(m, p.shape[1], 8)
    out[..., [0, 4, 1, 5]] = a
    out[..., [2, 6, 3, 7]] = c
    return out.reshape(m, -1)


def quantize_w8_rows(w: torch.Tensor):
    """Per-row symmetric int8 (lm_head / embedding tables): returns (int8 [N,K], fp32 scale [N])."""
    wf = w.to(torch.float32)
    s = wf.abs().amax(-1).clamp_min(1e-8) / 127.0
    q = (wf / s[:, None]).round().clamp(-127, 127).to(torch.int8)
    return q, s
