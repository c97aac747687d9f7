"""Thin Python bindings of the sm_100a kernel launchers (``libowl_b200_cuda.so``).

Every function takes torch CUDA tensors, launches on the current torch stream (so torch CUDA
graph capture records the launch) and raises ``NativeError`` on a rejected shape or a launch
failure. There is no fallback: CPU numerics live in ``ops/reference.py``.
"""
from __future__ import annotations

import collections
import ctypes
import os
from ctypes import c_longlong, c_float, c_int, c_void_p

import torch

from .. import _native

_P = c_void_p
_I = c_int
_F = c_float

_SIGS = {
    "owl_w4a16_skinny": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "owl_w4a16_skinny_a8": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "owl_w4a16_skinny_norm": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "owl_w4a16_stream_tc": [_P, _P, _P, _P, _P, c_longlong, _P, c_longlong, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "owl_bf16_skinny": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "owl_w8a16_skinny": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "owl_rmsnorm_pack": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _I, _I, _P],
    "owl_act_pack": [_P, _I, _P, _P, _I, _I, _I, _I, _P],
    "owl_silu_mul": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "owl_sigmoid_gate": [_P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "owl_embed": [_P, _P, _P, _I, _I, _I, _I, _P],
    "owl_argmax": [_P, _I, _I, _I, _P, _P, _I, _P, _I, _P, _I, _P],
    "owl_gdn_decode": [_P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _I, _P],
    "owl_gdn_conv_fwd": [_P, _I, _P, _P, _I, _P, _I, _I, _I, _I, _P],
    "owl_gdn_scan": [_P, _P, _I, _P, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _F, _I, _P],
    "owl_qknorm_rope_insert": [_P, _I, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F,
                               _F, _I, _P],
    "owl_paged_attn": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "owl_qknorm_rope_insert_f16": [_P, _I, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F,
                                   _F, _I, _P],
    "owl_paged_attn_f16": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "owl_qknorm_rope_insert_i8": [_P, _I, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F,
                                  _F, _I, _P],
    "owl_paged_attn_i8": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "owl_decode_advance": [_P, _P, _P, _I, _I, _I, _P],
    "owl_w4_dequant": [_P, _P, _I, _I, _I, _I, _I, _P],
    "owl_attn_reduce": [_P, _P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P],
}
_bound: dict = {}


def fn(name: str):
    f = _bound.get(name)
    if f is None:
        lib = _native.cuda()
        f = getattr(lib, name)
        sig = _SIGS.get(name)
        if sig is not None:
            f.argtypes = sig
        f.restype = c_int
        _bound[name] = f
    return f


def register(name: str, sig: list) -> None:
    _SIGS[name] = sig


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# Ring of the most recent native launches (entry name + raw arguments), formatted on demand by ``recent_launches``:
# what ran last is the first question after a wrong token or a status word, and a captured graph hides it from the host.
_LAUNCHES: collections.deque = collections.deque(maxlen=2048)
_launch_seq = 0
LAUNCH_SYNC = False       # debugging: wait for every launch and read the bounded-wait status words after it (no graph capture then)


def set_trace_ring(n: int) -> None:
    """Capacity of the launch ring (``[cuda] trace_ring``; 0 keeps the default of 2048 entries)."""
    global _LAUNCHES
    _LAUNCHES = collections.deque(_LAUNCHES, maxlen=n if n > 0 else 2048)


def call(name: str, *args) -> None:
    global _launch_seq
    if args and name not in _SIGS:
        # without argument types ctypes would pass 64-bit pointers as 32-bit ints: the module that registers this entry's
        # signature has not been imported
        raise RuntimeError(f"{name}: no ctypes signature registered (import the module that binds it first)")
    rc = fn(name)(*args)
    _launch_seq += 1
    _LAUNCHES.append((_launch_seq, name, args))
    if rc != 0:
        _native.check(rc, name)
    if LAUNCH_SYNC:
        # the failing launch is the one that just ran: a device fault surfaces here with the entry's name instead of at
        # some later synchronisation point
        try:
            torch.cuda.synchronize()
        except RuntimeError as ex:
            raise RuntimeError(f"{name} (launch {_launch_seq}): {ex}") from None
        bad = {k: v for k, v in all_status().items() if v}
        if bad:
            raise RuntimeError(f"{name} (launch {_launch_seq}): a bounded wait ran out {bad}")


def launch_seq() -> int:
    """Sequence number of the newest launch (a mark for ``launches_since``)."""
    return _launch_seq


def launches_since(mark: int) -> list[str]:
    """Entry names of the launches made after ``mark`` that are still in the ring, oldest first."""
    return [name for seq, name, _ in _LAUNCHES if seq > mark]


def recent_launches(n: int = 256) -> list[dict]:
    """The last ``n`` launches: sequence number, entry, stream handle and the small integer arguments (shapes, modes)."""
    out = []
    for seq, name, args in list(_LAUNCHES)[-n:]:
        ints = [a for a in args[:-1] if type(a) is int and -(1 << 31) <= a < (1 << 31)]
        out.append({"seq": seq, "entry": name, "stream": args[-1] if args and isinstance(args[-1], int) else None, "ints": ints})
    return out


EPI_STORE, EPI_RESIDUAL, EPI_SILU_MUL, EPI_F32, EPI_SILU_PACK = 0, 1, 2, 3, 4


def w4a16_skinny(w, xpack, xs, out, m: int, *, residual=None, epi: int = EPI_STORE, ldo: int | None = None,
                 out_pack=None, out_xs=None, gout: int = 128, tiles_per_cta: int = 0, pdl: bool = False,
                 force_mma: bool = False, a8: bool = False) -> None:
    """out[m, :] = dequant(w) @ x for m <= 32 rows. ``w`` is a ``W4Skinny``. One token runs on the
    dp4a arm unless ``force_mma`` (A/B runs and tests of the tensor-core arm). ``a8``: the activations were packed with
    ``ACT_A8`` (8-bit), the kernel skips the all-zero low plane (the W4A8 arm)."""
    if ldo is None:
        ldo = out.shape[-1] if out is not None else w.n
    assert w.layout == "slice", "w4a16_skinny reads slice-major records"
    if a8:
        call("owl_w4a16_skinny_a8", ptr(w.records), ptr(xpack), ptr(xs), ptr(out), ptr(residual), m, w.n, w.k, ldo, w.group,
             epi, int(force_mma), int(pdl), stream())
        return
    if force_mma:
        tiles_per_cta = -tiles_per_cta - 1
    call("owl_w4a16_skinny", ptr(w.records), ptr(xpack), ptr(xs), ptr(out), ptr(residual), ptr(out_pack), ptr(out_xs),
         m, w.n, w.k, ldo, w.group, epi, gout, tiles_per_cta, int(pdl), stream())


def w4a16_skinny_norm(w, xpack, xs, h, norm_w, count, m: int, *, normed=None, norm_pack=None, norm_xs=None,
                      group: int = 128, eps: float = 1e-6, one_plus_w: bool = True, pdl: bool = False,
                      force_mma: bool = False) -> None:
    """h[m, :] += dequant(w) @ x, and the CTA that finishes last writes rmsnorm(h) * (norm_w or 1 + norm_w) as bf16
    (``normed``) and / or ActPack (``norm_pack`` / ``norm_xs``): the row projection, the residual add and the next
    block's norm in one launch. ``count``: one int32 on the device, zero before the first call (the kernel zeroes it)."""
    assert w.layout == "slice" and h.shape[-1] == w.n and h.is_contiguous()
    call("owl_w4a16_skinny_norm", ptr(w.records), ptr(xpack), ptr(xs), ptr(h), ptr(h), ptr(norm_w), ptr(normed),
         ptr(norm_pack), ptr(norm_xs), ptr(count), m, w.n, w.k, w.n, w.group, group, eps, int(one_plus_w), int(force_mma),
         int(pdl), stream())


class StreamTcWorkspace:
    """Scratch for the split-K partial sums and arrival tickets of ``w4a16_stream_tc``. One per
    stream of launches (launches on one stream are ordered; concurrent streams need their own).
    ``ctas`` = 0 lets the launcher use every CTA slot of the device."""

    def __init__(self, device, max_n: int = 65536, ctas: int = 0):
        props = torch.cuda.get_device_properties(device)
        self.ctas = ctas
        nrb = (max_n + 127) // 128
        slots = (ctas or 2 * props.multi_processor_count) + 2 * nrb     # row blocks x slots never exceeds this
        self.scratch = torch.empty(slots * 128 * 8, dtype=torch.float32, device=device)
        self.counters = torch.zeros(nrb * 4, dtype=torch.int32, device=device)


ACT_TILES = 0x1000     # OR into a producer's ``group`` argument: write ActPack in the tile layout
ACT_A8 = 0x2000        # OR into a producer's ``group`` argument: round the activations to 8 bits (low plane zero)


def act_tile_bytes(k: int, group: int) -> int:
    """Size of an ActPack tile-layout buffer for a K-wide activation (any number of tokens <= 8)."""
    return (k // 128) * (2048 + 64 * (128 // (group & ~ACT_TILES)))


def w4a16_stream_tc(w, xtiles, out, m: int, ws: StreamTcWorkspace, *, residual=None, epi: int = EPI_STORE,
                    ldo: int | None = None, pdl: bool = False) -> None:
    """out[m, :] = dequant(w) @ x for m <= 8 rows on the tcgen05 integer path (``csrc/gemv_tc.cu``).
    ``xtiles``: the activations as written by a producer called with ``group | ACT_TILES``."""
    if ldo is None:
        ldo = out.shape[-1]
    assert w.layout == "block", "w4a16_stream_tc reads block-major records (quant.pack_skinny(..., layout='block'))"
    call("owl_w4a16_stream_tc", ptr(w.records), ptr(xtiles), ptr(out), ptr(residual), ptr(ws.scratch),
         ws.scratch.numel() * 4, ptr(ws.counters), ws.counters.numel() * 4, m, w.n, w.k, ldo, w.group, epi, ws.ctas,
         int(pdl), stream())


def stream_tc_status() -> int:
    f = fn("owl_stream_tc_status")
    f.argtypes = []
    return f()


def dense_skinny(w, x, out, m: int, *, residual=None, epi: int = EPI_STORE, ldo: int | None = None,
                 tiles_per_cta: int = 0, pdl: bool = False) -> None:
    """out[m, :] = W @ x for a ``DenseSkinny`` weight (bf16 records or int8 records + row scale)."""
    if ldo is None:
        ldo = out.shape[-1]
    if w.kind == "int8":
        call("owl_w8a16_skinny", ptr(w.records), ptr(w.row_scale), ptr(x), ptr(out), m, w.n, w.k, ldo, epi,
             tiles_per_cta, int(pdl), stream())
    else:
        call("owl_bf16_skinny", ptr(w.records), ptr(x), ptr(out), ptr(residual), m, w.n, w.k, ldo, epi, tiles_per_cta,
             int(pdl), stream())


register("owl_w4_fma", [_P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P])


def w4_fma(w, x, out, *, norm_w=None, residual=None, epi: int = EPI_STORE, ab_w=None, ab_out=None, ab_rows: int = 0, x_out=None,
           eps: float = 1e-6, one_plus_w: bool = True, groups_per_cta: int = 0, pdl: bool = False) -> None:
    """One token: ``out = epilogue(dequant(w) @ prologue(x))`` on the half-precision FMA arm (``csrc/gemv_fma.cu``).

    ``x`` bf16 ``[K]``: the activations, or with ``norm_w`` the residual stream, which the kernel RMS-normalises itself
    (``* (1 + norm_w)``). ``epi``: ``EPI_STORE``, ``EPI_RESIDUAL`` (``out = residual + y``) or ``EPI_SILU_MUL`` (``out[N/2]``).
    ``ab_w`` bf16 ``[ab_rows, K]``: dense rows multiplied with the same activations into ``ab_out``. ``x_out`` bf16 ``[K]``
    receives the activations the kernel consumed (the normalised row)."""
    assert w.layout == "slice" and w.group == 128, "w4_fma reads slice-major group-128 records"
    call("owl_w4_fma", ptr(w.records), ptr(x), ptr(norm_w), ptr(out), ptr(residual), ptr(ab_w), ptr(ab_out), ab_rows,
         ptr(x_out), w.n, w.k, int(norm_w is not None), epi, eps, int(one_plus_w), groups_per_cta, int(pdl), stream())


def fma_status() -> int:
    """First bounded-wait failure recorded by the FMA-arm projection kernels (0 = none); clears it."""
    f = fn("owl_fma_status")
    f.argtypes = []
    return f()


_STATUS_WORDS = {"skinny": "owl_skinny_status", "fma": "owl_fma_status", "stream_tc": "owl_stream_tc_status",
                 "gemm": "owl_gemm_status", "gemm_dense": "owl_gemm_dense_status", "gemm_nvfp4": "owl_gemm_nvfp4_status", "attn_tc": "owl_attn_tc_status", "comm": "owl_comm_status"}


def all_status() -> dict:
    """Every bounded-wait status word of the native library, read and cleared: ``{name: code}`` with 0 = no wait ran out
    since the last read. A non-zero word means a kernel gave up on a copy, an MMA or a peer flag and finished on stale
    data, so whatever that step produced must be discarded."""
    out = {}
    for name, sym in _STATUS_WORDS.items():
        f = fn(sym)
        f.argtypes = []
        out[name] = int(f())
    return out


def skinny_status() -> int:
    """First bounded-wait failure recorded by a weight-streaming kernel (0 = none); clears it."""
    f = fn("owl_skinny_status")
    f.argtypes = []
    return f()


def _is_f16(t) -> int:
    return int(t is not None and t.dtype == torch.float16)


def rmsnorm_pack(h, w, *, delta=None, out_h=None, normed=None, xpack=None, xs=None, m: int, k: int, group: int = 128,
                 eps: float = 1e-6, one_plus_w: bool = True, pdl: bool = False) -> None:
    """``normed`` may be bf16 or fp16 (the tcgen05 W4A16 GEMM takes fp16 activations)."""
    call("owl_rmsnorm_pack", ptr(h), ptr(delta), ptr(w), ptr(out_h), ptr(normed), ptr(xpack), ptr(xs), m, k, group,
         eps, int(one_plus_w), _is_f16(normed), int(pdl), stream())


register("owl_l2_prefetch", [_P, c_longlong, _I, _P])


def l2_prefetch(t: torch.Tensor, nbytes: int | None = None, ctas: int = 0) -> None:
    """Ask the memory system to bring the first ``nbytes`` of ``t`` into L2 (fire and forget, current stream)."""
    total = t.numel() * t.element_size()
    call("owl_l2_prefetch", ptr(t), min(total, nbytes) if nbytes is not None else total, ctas, stream())


def act_pack(x, xpack, xs, m: int, k: int, group: int = 128, ldx: int | None = None, pdl: bool = False) -> None:
    call("owl_act_pack", ptr(x), ldx if ldx is not None else k, ptr(xpack), ptr(xs), m, k, group, int(pdl), stream())


def silu_mul(gate_up, m: int, inter: int, *, out=None, xpack=None, xs=None, group: int = 128, pdl: bool = False):
    call("owl_silu_mul", ptr(gate_up), ptr(out), ptr(xpack), ptr(xs), m, inter, group, _is_f16(out), int(pdl),
         stream())


def sigmoid_gate(attn, qraw, ldq: int, hd: int, m: int, hdim_total: int, *, out=None, xpack=None, xs=None,
                 group: int = 128, pdl: bool = False):
    call("owl_sigmoid_gate", ptr(attn), ptr(qraw), ldq, hd, ptr(out), ptr(xpack), ptr(xs), m, hdim_total, group,
         int(pdl), stream())


def embed(ids, table, out, m: int, pdl: bool = False) -> None:
    call("owl_embed", ptr(ids), ptr(table), ptr(out), m, table.shape[1], table.shape[0], int(pdl), stream())


def argmax(logits, m: int, vocab: int, ld: int, scratch_val, scratch_idx, nparts: int, out_idx, vocab_offset: int = 0,
           pdl: bool = False, out_val=None) -> None:
    call("owl_argmax", ptr(logits), m, vocab, ld, ptr(scratch_val), ptr(scratch_idx), nparts, ptr(out_idx),
         vocab_offset, ptr(out_val), int(pdl), stream())


def gdn_decode(qkvz, ld: int, ab, ldab: int, conv_w, a_log, dt_bias, gamma, conv_state, state, slots, *, out=None,
               xpack=None, xs=None, batch: int, t: int, nk: int, nv: int, group: int = 128, eps: float = 1e-6,
               pdl: bool = False, tlen=None) -> None:
    """``tlen`` (int32 [batch], optional): sequence b consumes only its first ``tlen[b]`` rows (batched fold after a verify)."""
    call("owl_gdn_decode", ptr(qkvz), ld, ptr(ab), ldab, ptr(conv_w), ptr(a_log), ptr(dt_bias), ptr(gamma),
         ptr(conv_state), ptr(state), ptr(slots), ptr(out), ptr(xpack), ptr(xs), batch, t, nk, nv, group, eps,
         ptr(tlen), int(pdl), stream())


def gdn_conv_fwd(x, ld: int, conv_w, conv_state, slot: int, out, t: int, nk: int, nv: int, use_state: bool) -> None:
    call("owl_gdn_conv_fwd", ptr(x), ld, ptr(conv_w), ptr(conv_state), slot, ptr(out), t, nk, nv, int(use_state),
         stream())


register("owl_gdn_scan_split", [_P, _P, _I, _P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _P])
_scan_scratch: dict = {}
GDN_SPLIT_FROM = 32      # tokens from which the column-split scan (4 CTAs per head + norm kernel) is used
GDN_CHUNKED_FROM = 128   # tokens from which the chunked (WY) tensor-core scan is used (0 = never)
register("owl_gdn_chunk_work_bytes", [_I, _I, _P])
register("owl_gdn_chunk_scan", [_P, _P, _I, _P, _P, _P, _I, _P, _P, c_longlong, _I, _I, _I, _I, _P])
register("owl_gdn_norm_gate", [_P, _P, _I, _P, _P, _I, _I, _F, _I, _P])
_chunk_work: dict = {}


def gdn_scan(qkv, z, ldz: int, ab, ldab: int, a_log, dt_bias, gamma, state, slot: int, out, t: int, nk: int, nv: int,
             use_state: bool, eps: float = 1e-6, split: bool | None = None) -> None:
    """Gated delta rule over ``t`` tokens of one sequence (prefill). Long chunks run the column-split kernel,
    which needs a fp32 scratch of t * nv * 128 floats (cached per device)."""
    if split is None and GDN_CHUNKED_FROM and t >= GDN_CHUNKED_FROM:
        split = "chunked"
    if split is None:
        split = t >= GDN_SPLIT_FROM
    if split == "chunked":
        # chunk-64 WY form on tensor cores (csrc/gdn_chunk.cu): prep kernel over all chunks, recurrence over chunks, gated norm
        key = str(qkv.device)
        nb = c_longlong(0)
        call("owl_gdn_chunk_work_bytes", t, nv, ctypes.addressof(nb))
        need = int(nb.value)
        raw, work = _chunk_work.get(key, (None, None))
        if raw is None or raw.numel() < t * nv * 128 or work.numel() < need:
            raw = torch.empty(max(t * nv * 128, 0 if raw is None else raw.numel()), dtype=torch.float32, device=qkv.device)
            work = torch.empty(max(need, 0 if work is None else work.numel()), dtype=torch.uint8, device=qkv.device)
            _chunk_work[key] = (raw, work)
        call("owl_gdn_chunk_scan", ptr(qkv), ptr(ab), ldab, ptr(a_log), ptr(dt_bias), ptr(state), slot, ptr(raw), ptr(work),
             work.numel(), t, nk, nv, int(use_state), stream())
        call("owl_gdn_norm_gate", ptr(raw), ptr(z), ldz, ptr(gamma), ptr(out), t, nv, eps, _is_f16(out), stream())
        return
    if not split:
        call("owl_gdn_scan", ptr(qkv), ptr(z), ldz, ptr(ab), ldab, ptr(a_log), ptr(dt_bias), ptr(gamma), ptr(state), slot,
             ptr(out), t, nk, nv, int(use_state), eps, _is_f16(out), stream())
        return
    key = str(qkv.device)
    buf = _scan_scratch.get(key)
    if buf is None or buf.numel() < t * nv * 128:
        buf = torch.empty(t * nv * 128, dtype=torch.float32, device=qkv.device)
        _scan_scratch[key] = buf
    call("owl_gdn_scan_split", ptr(qkv), ptr(z), ldz, ptr(ab), ldab, ptr(a_log), ptr(dt_bias), ptr(gamma), ptr(state), slot,
         ptr(out), ptr(buf), t, nk, nv, int(use_state), eps, _is_f16(out), stream())


def qknorm_rope_insert(qraw, ldq: int, kraw, ldk: int, vraw, ldv: int, qnorm_w, knorm_w, pos3, inv_freq, section,
                       kv_slot, q_out, k_pool, v_pool, rows: int, hq: int, hkv: int, hd: int, rot: int,
                       eps: float = 1e-6, rope_scale: float = 1.0, pdl: bool = False, scales=None) -> None:
    """``scales`` = (k_scale, v_scale) fp32 [pages, 16, hkv] selects the int8 pool form."""
    if k_pool.dtype == torch.float16:
        call("owl_qknorm_rope_insert_f16", ptr(qraw), ldq, ptr(kraw), ldk, ptr(vraw), ldv, ptr(qnorm_w), ptr(knorm_w),
             ptr(pos3), ptr(inv_freq), ptr(section), ptr(kv_slot), ptr(q_out), ptr(k_pool), ptr(v_pool), rows, hq, hkv,
             hd, rot, eps, rope_scale, int(pdl), stream())
        return
    if scales is not None:
        call("owl_qknorm_rope_insert_i8", ptr(qraw), ldq, ptr(kraw), ldk, ptr(vraw), ldv, ptr(qnorm_w), ptr(knorm_w),
             ptr(pos3), ptr(inv_freq), ptr(section), ptr(kv_slot), ptr(q_out), ptr(k_pool), ptr(v_pool), ptr(scales[0]),
             ptr(scales[1]), rows, hq, hkv, hd, rot, eps, rope_scale, int(pdl), stream())
        return
    call("owl_qknorm_rope_insert", ptr(qraw), ldq, ptr(kraw), ldk, ptr(vraw), ldv, ptr(qnorm_w), ptr(knorm_w),
         ptr(pos3), ptr(inv_freq), ptr(section), ptr(kv_slot), ptr(q_out), ptr(k_pool), ptr(v_pool), rows, hq, hkv,
         hd, rot, eps, rope_scale, int(pdl), stream())


def paged_attn(q, k_pool, v_pool, block_table, bt_row, ctx_len, part_o, part_ml, groups: int, t: int, hq: int,
               hkv: int, hd: int, max_blocks: int, splits: int, scale: float, pdl: bool = False, per_pages: int = 0,
               scales=None) -> None:
    """``per_pages`` > 0 fixes the pages per KV split (must satisfy splits * per_pages >= pages of the longest row)."""
    if k_pool.dtype == torch.float16:
        call("owl_paged_attn_f16", ptr(q), ptr(k_pool), ptr(v_pool), ptr(block_table), ptr(bt_row), ptr(ctx_len), ptr(part_o),
             ptr(part_ml), groups, t, hq, hkv, hd, max_blocks, splits, per_pages, scale, int(pdl), stream())
        return
    if scales is not None:
        call("owl_paged_attn_i8", ptr(q), ptr(k_pool), ptr(v_pool), ptr(scales[0]), ptr(scales[1]), ptr(block_table),
             ptr(bt_row), ptr(ctx_len), ptr(part_o), ptr(part_ml), groups, t, hq, hkv, hd, max_blocks, splits, per_pages, scale,
             int(pdl), stream())
        return
    call("owl_paged_attn", ptr(q), ptr(k_pool), ptr(v_pool), ptr(block_table), ptr(bt_row), ptr(ctx_len), ptr(part_o),
         ptr(part_ml), groups, t, hq, hkv, hd, max_blocks, splits, per_pages, scale, int(pdl), stream())


def attn_reduce(part_o, part_ml, splits: int, qraw, ldq: int, rows: int, hq: int, *, out=None, xpack=None, xs=None,
                group: int = 128, pdl: bool = False) -> None:
    call("owl_attn_reduce", ptr(part_o), ptr(part_ml), splits, ptr(qraw), ldq, ptr(out), ptr(xpack), ptr(xs), rows, hq,
         group, _is_f16(out), int(pdl), stream())


register("owl_kv_pages_gather", [_P, _P, _P, _I, _I, _P, _I, _P, _P])
register("owl_kv_pages_scatter", [_P, _P, _P, _I, _I, _P, _I, _P, _P])
register("owl_kv_gather", [_P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P])
register("owl_causal_softmax", [_P, _I, _I, _I, _I, _F, _I, _P, _P])
register("owl_attn_gate", [_P, _P, _I, _I, _P, _I, _I, _I, _I, _P, _P])
register("owl_q_group", [_P, _P, _I, _I, _I, _I, _P])
register("owl_f16_gemm_persist_f16out", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P])


def attn_gemm_prefill(q, k_pool, v_pool, scales, bt_row, pos0: int, t: int, hq: int, hkv: int, hd: int, scale: float, ws: dict,
                      qraw, ldq: int, out) -> None:
    """Causal attention of a prefill chunk as tcgen05 GEMMs (long contexts): the sequence's paged K / V are gathered once into
    dense k-major operands (K bf16, V transposed fp16), then per q head S = Q K^T (fp16 scores), a causal softmax in place,
    O = P V; the sigmoid gate of the q projection closes it. ``q``: bf16 [t, hq, hd] after norm and rotary; ``bt_row``: the
    sequence's block-table row; ``ws``: scratch tensors kept by the caller (``attn_gemm_ws``); ``out``: [t, hq * hd] bf16 / fp16."""
    from . import gemm_tc  # noqa: F401  (binds the dense GEMM entries this path calls)

    ctx = pos0 + t
    ctx_pad = (ctx + 63) // 64 * 64
    fmt = 2 if k_pool.dtype == torch.float16 else (1 if scales is not None else 0)
    kb, vt, o = ws["k"][:hkv * ctx_pad * hd], ws["vt"][:hkv * hd * ctx_pad], ws["o"][:t * hq * hd]
    call("owl_kv_gather", ptr(k_pool), ptr(v_pool), ptr(scales[0]) if scales else None, ptr(scales[1]) if scales else None, fmt,
         ptr(bt_row), ctx, ctx_pad, hkv, hd, ptr(kb), ptr(vt), stream())
    gq, st = hq // hkv, stream()
    inv = ws["inv"][:hq * t]            # 1 / softmax denominator per (head, token), applied with the gate
    if ATTN_FUSED and ws.get("grouped", True) and hd == 256:
        # one fused kernel for all kv heads: S and O in tensor memory, online softmax between the two products, key tiles
        # past a row tile's causal limit skipped (csrc/attn_tc.cu); the output is normalised already
        qg, og = ws["qg"][:hq * t * hd], ws["og"][:hq * t * hd]
        call("owl_q_group", ptr(q), ptr(qg), t, hq, hkv, hd, st)
        call("owl_attn_tc", ptr(qg), ptr(kb), ptr(vt), ptr(og), t * gq, gq, hkv, ctx_pad, pos0, float(scale), st)
        call("owl_attn_gate", ptr(og), ptr(qraw), ldq, hd, ptr(out), t, hq * hd, _is_f16(out), gq, None, st)
        return
    if ws["s"] is None:
        ws["s"] = torch.zeros(ws["t"] * gq * ws["ctx"], dtype=torch.float16, device=q.device)
    s = ws["s"][:t * ctx_pad]
    if ws.get("grouped", True):
        # the gq q heads of a kv head as consecutive rows: one GEMM pair per kv head, K and V^T read once for all of them
        qg, og = ws["qg"][:hq * t * hd], ws["og"][:hq * t * hd]
        s = ws["s"][:t * gq * ctx_pad]
        call("owl_q_group", ptr(q), ptr(qg), t, hq, hkv, hd, st)
        for kh in range(hkv):
            call("owl_f16_gemm_persist_f16out", qg.data_ptr() + kh * t * gq * hd * 2, hd, kb.data_ptr() + kh * ctx_pad * hd * 2, hd,
                 ptr(s), t * gq, ctx_pad, hd, ctx_pad, 1, st)
            call("owl_causal_softmax", ptr(s), t * gq, ctx_pad, ctx_pad, pos0, scale, gq, inv.data_ptr() + kh * t * gq * 4, st)
            call("owl_f16_gemm_persist", ptr(s), ctx_pad, vt.data_ptr() + kh * hd * ctx_pad * 2, ctx_pad,
                 og.data_ptr() + kh * t * gq * hd * 2, t * gq, hd, ctx_pad, hd, 0, st)
        call("owl_attn_gate", ptr(og), ptr(qraw), ldq, hd, ptr(out), t, hq * hd, _is_f16(out), gq, ptr(inv), st)
        return
    for h in range(hq):
        kh = h // gq
        call("owl_f16_gemm_persist_f16out", q.data_ptr() + h * hd * 2, hq * hd, kb.data_ptr() + kh * ctx_pad * hd * 2, hd, ptr(s),
             t, ctx_pad, hd, ctx_pad, 1, st)
        call("owl_causal_softmax", ptr(s), t, ctx_pad, ctx_pad, pos0, scale, 1, inv.data_ptr() + h * t * 4, st)
        call("owl_f16_gemm_persist", ptr(s), ctx_pad, vt.data_ptr() + kh * hd * ctx_pad * 2, ctx_pad, o.data_ptr() + h * hd * 2,
             t, hd, ctx_pad, hq * hd, 0, st)
    call("owl_attn_gate", ptr(o), ptr(qraw), ldq, hd, ptr(out), t, hq * hd, _is_f16(out), 0, ptr(inv), st)


ATTN_FUSED = os.environ.get("OWL_ATTN_TC", "1") == "1"      # long-context prefill attention: the fused tcgen05 kernel (0: GEMM form)
register("owl_attn_tc", [_P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P])


def attn_gemm_ws(device, t: int, max_ctx: int, hq: int, hkv: int, hd: int) -> dict:
    """Scratch of ``attn_gemm_prefill`` for chunks of up to ``t`` rows over up to ``max_ctx`` keys."""
    cp = (max_ctx + 63) // 64 * 64
    return {"k": torch.zeros(hkv * cp * hd, dtype=torch.bfloat16, device=device),
            "vt": torch.zeros(hkv * hd * cp, dtype=torch.float16, device=device),
            # fp16 scores of the GEMM form (rows x keys): the fused kernel keeps them in tensor memory and needs no such buffer
            "s": None if ATTN_FUSED and hd == 256 else torch.zeros(t * (hq // hkv) * cp, dtype=torch.float16, device=device),
            "o": torch.zeros(t * hq * hd, dtype=torch.bfloat16, device=device),
            "qg": torch.zeros(t * hq * hd, dtype=torch.bfloat16, device=device),
            "og": torch.zeros(t * hq * hd, dtype=torch.bfloat16, device=device),
            "inv": torch.zeros(t * hq, dtype=torch.float32, device=device), "t": t, "ctx": cp, "grouped": True}


register("owl_topk", [_P, _I, _I, _I, _I, _P, _P, _I, _F, _I, _P, _P, _I, _P, _P, _P])
register("owl_topk_merge", [_P, _P, _I, _I, _I, _P, _P, _P])


class TopK:
    """Device top-k (k <= 32) of logits rows with an optional repetition penalty (``csrc/sample.cu``)."""

    def __init__(self, device, max_rows: int = 32, k: int = 32, parts: int = 64):
        self.k, self.parts = k, parts
        self.sval = torch.empty(max_rows * parts * k, dtype=torch.float32, device=device)
        self.sidx = torch.empty(max_rows * parts * k, dtype=torch.int32, device=device)
        self.val = torch.empty(max_rows, k, dtype=torch.float32, device=device)
        self.idx = torch.empty(max_rows, k, dtype=torch.int32, device=device)

    def __call__(self, logits, m: int, vocab: int, *, hist=None, hist_len=None, penalty: float = 1.0, vocab_offset: int = 0):
        call("owl_topk", ptr(logits), logits.stride(0), m, vocab, self.k, ptr(hist), ptr(hist_len),
             hist.stride(0) if hist is not None else 0, float(penalty), vocab_offset, ptr(self.sval), ptr(self.sidx),
             self.parts, ptr(self.val), ptr(self.idx), stream())
        return self.val[:m], self.idx[:m]


def topk_merge(cand_val, cand_idx, k: int):
    """Global top-k of concatenated per-rank candidates ``[M, n]`` (vocab-split head)."""
    m, n = cand_val.shape
    ov = torch.empty(m, k, dtype=torch.float32, device=cand_val.device)
    oi = torch.empty(m, k, dtype=torch.int32, device=cand_val.device)
    call("owl_topk_merge", ptr(cand_val), ptr(cand_idx), m, n, k, ptr(ov), ptr(oi), stream())
    return ov, oi


register("owl_nvfp4_gemv", [_P, _P, _F, _P, _I, _P, _I, _I, _I, _I, _P])
register("owl_nvfp4_gemv_res", [_P, _P, _F, _P, _I, _P, _I, _P, _I, _I, _I, _P])
register("owl_nvfp4_gemv_rows", [_P, _P, _F, _P, _P, _I, _P, _I, _P, _I, _I, _I, _P])
register("owl_nvfp4_dequant_rows", [_P, _P, _F, _P, _I, _P, c_longlong, _P])
register("owl_act_unpack", [_P, _P, _P, _I, _I, _I, _I, _I, _P])
register("owl_add_rows", [_P, _I, _P, _I, _P, _I, _I, _I, _P])
register("owl_nvfp4_dequant", [_P, _P, _F, _P, c_longlong, _P])
register("owl_nvfp4_quant_act", [_P, _F, _P, _P, c_longlong, _P])
register("owl_gguf_dequant", [_P, _I, _I, _P, _I, _P, _P])
register("owl_gguf_gemv", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P])


def nvfp4_gemv(codes, scales, alpha: float, x, out, m: int) -> None:
    """out[m, N] = alpha * x . dequant(NVFP4 W)^T for m <= 8 (``csrc/lowbit.cu``). codes uint8 [N, K/2], scales e4m3 bytes [N, K/16]."""
    n, k = codes.shape[0], codes.shape[1] * 2
    call("owl_nvfp4_gemv", ptr(codes), ptr(scales), float(alpha), ptr(x), x.stride(0), ptr(out), out.stride(0), m, n, k, stream())


def nvfp4_gemv_res(codes, scales, alpha: float, x, out, residual, m: int) -> None:
    """out = residual + alpha * x . dequant(W)^T (m <= 8); ``residual`` may be ``out``."""
    n, k = codes.shape[0], codes.shape[1] * 2
    call("owl_nvfp4_gemv_res", ptr(codes), ptr(scales), float(alpha), ptr(x), x.stride(0), ptr(out), out.stride(0), ptr(residual),
         m, n, k, stream())


def nvfp4_linear_gemv(w, x, out, m: int, residual=None) -> None:
    """``out[:m] = (residual +) x . dequant(w)^T`` for an ``NvFp4Linear`` (m <= 8), per-row scales included."""
    if w.row_scale is not None:
        call("owl_nvfp4_gemv_rows", ptr(w.codes), ptr(w.scales), float(w.alpha), ptr(w.row_scale), ptr(x), x.stride(0), ptr(out),
             out.stride(0), ptr(residual), m, w.n, w.k, stream())
    elif residual is not None:
        nvfp4_gemv_res(w.codes, w.scales, w.alpha, x, out, residual, m)
    else:
        nvfp4_gemv(w.codes, w.scales, w.alpha, x, out, m)


def nvfp4_linear_dequant(w, out):
    """Dense bf16 ``[N, K]`` copy of an ``NvFp4Linear``."""
    if w.row_scale is not None:
        call("owl_nvfp4_dequant_rows", ptr(w.codes), ptr(w.scales), float(w.alpha), ptr(w.row_scale), w.k, ptr(out), w.n * w.k,
             stream())
        return out
    return nvfp4_dequant(w.codes, w.scales, w.alpha, out)


def act_unpack(xpack, xs, out, m: int, k: int, group: int = 128) -> None:
    """ActPack rows (row layout) -> bf16 or fp16 (by ``out.dtype``) ``out[:m, :k]``."""
    call("owl_act_unpack", ptr(xpack), ptr(xs), ptr(out), out.stride(0), m, k, group, _is_f16(out), stream())


def add_rows(a, b, out, m: int, n: int) -> None:
    """``out[:m, :n] = a[:m, :n] + b[:m, :n]`` (bf16)."""
    call("owl_add_rows", ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out), out.stride(0), m, n, stream())


def nvfp4_dequant(codes, scales, alpha: float, out=None):
    n, k = codes.shape[0], codes.shape[1] * 2
    if out is None:
        out = torch.empty(n, k, dtype=torch.bfloat16, device=codes.device)
    call("owl_nvfp4_dequant", ptr(codes), ptr(scales), float(alpha), ptr(out), n * k, stream())
    return out


def nvfp4_quant_act(x, global_scale: float):
    """bf16 [M, K] -> (codes uint8 [M, K/2], e4m3 block scales uint8 [M, K/16]) for the given global scale."""
    m, k = x.shape
    codes = torch.empty(m, k // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(m, k // 16, dtype=torch.uint8, device=x.device)
    call("owl_nvfp4_quant_act", ptr(x), float(global_scale), ptr(codes), ptr(sf), m * k, stream())
    return codes, sf


register("owl_gguf_set_grids", [_P, _P])
_gguf_grids_on: set = set()


def _gguf_grids(device) -> None:
    """Upload the IQ3 codebooks to ``device`` once (the kernels index them by the blocks' grid numbers)."""
    key = str(device)
    if key in _gguf_grids_on:
        return
    from ..formats.gguf_grids import IQ3S_GRID, IQ3XXS_GRID

    a, b = IQ3XXS_GRID.tobytes(), IQ3S_GRID.tobytes()
    with torch.cuda.device(device):
        call("owl_gguf_set_grids", ctypes.cast(ctypes.c_char_p(a), c_void_p), ctypes.cast(ctypes.c_char_p(b), c_void_p))
    _gguf_grids_on.add(key)


def gguf_dequant(blocks, type_id: int, k: int, n_rows: int, rows=None, out=None):
    """GGUF blocks (uint8, ``n_src_rows * K / elems`` blocks) -> bf16 [R, K]; ``rows`` int32 picks source rows (embedding lookup)."""
    _gguf_grids(blocks.device)
    r = n_rows if rows is None else rows.numel()
    if out is None:
        out = torch.empty(r, k, dtype=torch.bfloat16, device=blocks.device)
    call("owl_gguf_dequant", ptr(blocks), type_id, k, ptr(rows), r, ptr(out), stream())
    return out


def gguf_gemv(blocks, type_id: int, n: int, k: int, x, out, m: int) -> None:
    _gguf_grids(blocks.device)
    call("owl_gguf_gemv", ptr(blocks), type_id, ptr(x), x.stride(0), ptr(out), out.stride(0), m, n, k, stream())


def w4_dequant(w, out=None):
    """Dense bf16 (or fp16, by ``out.dtype``) [N, K] copy of a ``W4Skinny`` weight."""
    if out is None:
        out = torch.empty(w.n, w.k, dtype=torch.bfloat16, device=w.records.device)
    call("owl_w4_dequant", ptr(w.records), ptr(out), w.n, w.k, w.group, w.layout_id, _is_f16(out), stream())
    return out


def decode_advance(inp, tok, block_table, max_blocks: int, b: int, pdl: bool = False) -> None:
    call("owl_decode_advance", ptr(inp), ptr(tok), ptr(block_table), max_blocks, b, int(pdl), stream())
