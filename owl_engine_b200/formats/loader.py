"""Checkpoint loading: detect the source kind, read every tensor as-is, build device weights.

A *provider* answers two questions for an HF-style tensor name: ``w4(name)`` (the int4 canonical
form of a linear weight, read without re-quantisation when the checkpoint already is int4) and
``dense(name)`` (norms, embeddings, small projections). ``build_weights`` merges projections the
kernels want merged (q|k|v, qkv|z, interleaved gate|up), cuts them for the TP rank and packs the
skinny record streams.

Sources: HF directory with bf16 safetensors (quantised on load, RTN), compressed-tensors AWQ /
W4A16 directories (loaded as-is), GGUF files (Q4_K loaded as-is with group 32; other GGUF types are
dequantised and re-quantised to int4 g32 with a warning; norm weights have the +1 that GGUF bakes in
removed). Reference counterpart: ``crates/engine/src/loader.rs``, ``crates/models/src/formats/
{load,kind,sharded}.rs`` and ``formats/gguf/{keys,source,shard}.rs``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..models import hybrid as H
from ..models.spec import ModelSpec
from ..ops import quant as Q
from ..parallel.plan import Rule, TpPlan, rule_of
from ..utils import log
from . import awq, gguf
from .safetensors import SafeDir


def detect_kind(path: str | Path) -> str:
    p = Path(path)
    if p.is_file() and p.suffix == ".gguf":
        return "gguf"
    cfg = p / "config.json"
    if cfg.exists():
        qc = json.loads(cfg.read_text()).get("quantization_config", {})
        fmt = (qc.get("format") or qc.get("quant_method") or "").lower()
        if "pack" in fmt or "awq" in fmt or "compressed" in fmt:
            return "awq"
        if "nvfp4" in fmt or "modelopt" in fmt:
            return "nvfp4"
    if list(p.glob("*.safetensors")):
        names = SafeDir(p).keys()
        if any(k.endswith(".weight_packed") for k in names):
            return "awq"
        return "safetensors"
    raise FileNotFoundError(f"cannot tell what kind of checkpoint {p} is")


class DenseProvider:
    """bf16 / fp32 tensors (dict or SafeDir); linear weights are quantised on load."""

    def __init__(self, src, group: int = 128):
        self.src, self.group = src, group

    def _get(self, name):
        return self.src[name] if isinstance(self.src, dict) else self.src.get(name)

    def dense(self, name: str) -> torch.Tensor:
        return self._get(name)

    def w4(self, name: str) -> Q.W4Canonical:
        return Q.quantize_w4(self._get(name).float(), self.group)

    def has(self, name: str) -> bool:
        return name in self.src if isinstance(self.src, dict) else name in self.src


class AwqProvider(DenseProvider):
    def w4(self, name: str) -> Q.W4Canonical:
        prefix = name[:-len(".weight")]
        if (prefix + ".weight_packed") in self.src:
            return awq.from_compressed_tensors(self.src, prefix)
        return super().w4(name)


# HF name fragment -> GGUF name (llama.cpp-style key convention)
_GGUF_LAYER = {
    "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "post_attention_norm.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight",
    "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
    "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
    "linear_attn.in_proj_qkv.weight": "attn_qkv.weight", "linear_attn.in_proj_z.weight": "attn_gate.weight",
    "linear_attn.in_proj_a.weight": "ssm_alpha.weight", "linear_attn.in_proj_b.weight": "ssm_beta.weight",
    "linear_attn.conv1d.weight": "ssm_conv1d.weight", "linear_attn.A_log": "ssm_a", "linear_attn.dt_bias": "ssm_dt.bias",
    "linear_attn.norm.weight": "ssm_norm.weight", "linear_attn.out_proj.weight": "ssm_out.weight",
}
_GGUF_TOP = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
_PLUS_ONE_NORMS = ("input_layernorm.weight", "post_attention_layernorm.weight", "q_norm.weight", "k_norm.weight",
                   "model.norm.weight")


def gguf_name(hf: str) -> str:
    if hf in _GGUF_TOP:
        return _GGUF_TOP[hf]
    parts = hf.split(".")
    assert parts[0] == "model" and parts[1] == "layers", hf
    return f"blk.{parts[2]}." + _GGUF_LAYER[".".join(parts[3:])]


class GgufProvider:
    """Tensors of a GGUF file under their HF names, in the model's (grouped) value-head order: converted checkpoints store the
    gated-delta-net's value heads tiled (``formats/gguf_shard.py``), which is undone here when the tensor is read, on the raw
    blocks for quantised types. ``general`` metadata key ``owl.vhead_order = "grouped"`` marks a file that is in model order
    already. ``read_shard`` reads one rank's window of a tensor without materialising the rest."""

    def __init__(self, f: gguf.GgufFile):
        self.f = f
        self.dims = None
        self.tiled = str(f.meta.get("owl.vhead_order", "tiled")) != "grouped"

    def set_dims(self, spec) -> None:
        from .gguf_shard import GdnDims

        self.dims = GdnDims(spec.nk, spec.nv, spec.kd, spec.vd)

    def _plan(self, g: str, sel=None):
        """Read plan of GGUF tensor ``g`` (None: take it whole, as stored)."""
        from . import gguf_shard as S

        if self.dims is None or (not self.tiled and sel is None):
            return None
        t = self.f.tensors[g]
        shape = tuple(t.shape) if len(t.shape) == 2 else (int(np.prod(t.shape)), 1) if len(t.shape) == 1 else None
        if shape is None or S.role(g, sel) == S.REPLICATE:
            return None
        dims = self.dims if self.tiled else S.GdnDims(self.dims.nk, self.dims.nk, self.dims.kd, self.dims.vd * self.dims.vpr)
        return S.plan(g, shape, gguf.BLOCK.get(t.type, (1, 0))[0], dims, sel)

    def read_shard(self, name: str, sel) -> torch.Tensor:
        """Dequantised window of rank ``sel.rank`` (value heads in grouped order): equals the matching block of ``dense``."""
        from . import gguf_shard as S

        g = gguf_name(name)
        t = self.f.tensors[g]
        p = self._plan(g, sel)
        if p is None:
            return self.f.dequant(g)
        be, bb = gguf.BLOCK.get(t.type, (1, 0))
        if be == 1:
            x = self.f.dequant(g)
            x = x.reshape(x.shape[0], -1) if x.dim() > 1 else x
            return torch.from_numpy(np.ascontiguousarray(S.apply_dense(x.numpy(), p)))
        shape = tuple(t.shape)
        raw = S.apply_raw(self.f.raw(g), shape, be, bb, p)
        return torch.from_numpy(gguf.dequantize(raw.reshape(-1), t.type, p.shape[0] * p.shape[1])).view(*p.shape)

    def has(self, name: str) -> bool:
        try:
            return gguf_name(name) in self.f.tensors
        except (KeyError, AssertionError):
            return False

    def dense(self, name: str) -> torch.Tensor:
        from . import gguf_shard as S

        g = gguf_name(name)
        t = self.f.dequant(g)
        p = self._plan(g)
        if p is not None:
            shp = t.shape
            x = S.apply_dense(t.reshape(shp[0], -1).numpy() if t.dim() > 1 else t.numpy(), p)
            t = torch.from_numpy(np.ascontiguousarray(x)).view(*shp)
        if name.endswith(_PLUS_ONE_NORMS):
            t = t - 1.0                     # GGUF stores gamma with the +1 baked in; kernels apply (1 + w)
        if name.endswith("A_log"):
            t = torch.log(-t) if (t < 0).all() else t     # some converters store A = -exp(A_log)
        return t

    def w4_shard(self, name: str, full: ModelSpec, plan: TpPlan):
        """One rank's part of a Q4_K tensor, cut on the raw blocks of the memory-mapped file (row windows, block-aligned
        column windows, value heads in grouped order) BEFORE the conversion to the int4 form, so a rank neither reads nor
        converts the other ranks' parts. Returns None when the tensor has no raw plan that equals the canonical cut (another
        block type, kv heads replicated over ranks, a column cut inside a super-block): the caller then reads it whole and
        slices the int4 form. ``tests/test_loader.py`` checks that both routes give the same tensors."""
        from . import gguf_shard as S

        g = gguf_name(name)
        t = self.f.tensors[g]
        if plan.world == 1 or t.type != "Q4_K" or self.dims is None:
            return None
        r = rule_of(name)
        if r is Rule.KV_COL and full.hkv % plan.world:
            return None
        if r is Rule.Q_COL and full.hq % plan.world:
            return None
        try:
            p = self._plan(g, S.ShardSel(plan.rank, plan.world))
        except S.ShardError:
            return None
        if p is None:
            return None
        raw = S.apply_raw(self.f.raw(g), tuple(t.shape), *gguf.BLOCK["Q4_K"], p)
        self.shard_reads = getattr(self, "shard_reads", 0) + 1
        return gguf.q4k_to_w4(raw.reshape(-1), p.shape[0], p.shape[1])

    def w4(self, name: str) -> Q.W4Canonical:
        from . import gguf_shard as S

        g = gguf_name(name)
        t = self.f.tensors[g]
        if t.type == "Q4_K":
            raw = self.f.raw(g)
            try:
                p = self._plan(g)
            except S.ShardError:
                # a 256-element super-block spans two value heads that the tiled order separates (ssm_out with 128-wide
                # heads): the columns are reordered after the conversion, on the 32-element groups of the int4 form, which is
                # just as exact
                p = None
                c = gguf.q4k_to_w4(raw, t.shape[0], t.shape[1])
                sub = S.plan(g, tuple(t.shape), c.group, self.dims, None)
                atoms = torch.from_numpy(np.asarray(sub.col_atoms))
                cols = torch.from_numpy(S.head_rows(np.asarray(sub.col_atoms), c.group))
                return Q.W4Canonical(c.q[:, cols].contiguous(), c.scales[:, atoms].contiguous(), c.zeros[:, atoms].contiguous(),
                                     c.group)
            if p is not None:
                raw = S.apply_raw(raw, tuple(t.shape), *gguf.BLOCK["Q4_K"], p).reshape(-1)
            return gguf.q4k_to_w4(raw, t.shape[0], t.shape[1])
        log.warn("load.gguf", f"{g}: {t.type} is dequantised and re-quantised to int4 g32")
        return Q.quantize_w4(self.dense(name).float(), 32)


@dataclass
class NvCanonical:
    """NVFP4 tensor as stored (ModelOpt layout): e2m1 codes ``[N, K/2]`` (two per byte), e4m3 block scales ``[N, K/16]`` and one
    fp32 scale per ROW (a per-tensor scale broadcast, so that rows of different tensors can be stacked)."""
    codes: torch.Tensor
    scales: torch.Tensor
    row_scale: torch.Tensor
    group: int = 128

    @property
    def shape(self):
        return (self.codes.shape[0], self.codes.shape[1] * 2)


class NvFp4Provider(DenseProvider):
    """ModelOpt NVFP4 checkpoints: ``<name>`` uint8 packed codes, ``<name>_scale`` e4m3 block scales, ``<name>_scale_2`` the
    fp32 per-tensor scale (``crates/models/src/formats`` NVFP4 source in the reference); everything else is 16-bit."""

    def w4(self, name: str) -> NvCanonical:
        codes = self._get(name)
        if codes.dtype not in (torch.uint8, torch.int8):
            from . import nvfp4

            q = nvfp4.quantize(codes.float())                # an unquantised tensor inside a quantised checkpoint
            return NvCanonical(q.codes, q.scales, torch.full((codes.shape[0],), q.global_scale), self.group)
        sc = self._get(name + "_scale")
        g2 = self._get(name + "_scale_2").float().reshape(-1)
        return NvCanonical(codes.view(torch.uint8), sc.view(torch.uint8), g2.expand(codes.shape[0]).contiguous(), self.group)


def open_source(path: str | Path, group: int = 128):
    kind = detect_kind(path)
    if kind == "gguf":
        f = gguf.GgufFile(path)
        return kind, GgufProvider(f), f
    d = SafeDir(path)
    if kind == "nvfp4":
        return kind, NvFp4Provider(d, group), d
    return kind, (AwqProvider(d, group) if kind == "awq" else DenseProvider(d, group)), d


# ---- canonical-form surgery --------------------------------------------------------------------
def cat_rows(parts: list):
    if isinstance(parts[0], NvCanonical):
        return NvCanonical(torch.cat([p.codes for p in parts]), torch.cat([p.scales for p in parts]),
                           torch.cat([p.row_scale for p in parts]), parts[0].group)
    g = parts[0].group
    assert all(p.group == g and p.q.shape[1] == parts[0].q.shape[1] for p in parts)
    return Q.W4Canonical(torch.cat([p.q for p in parts]), torch.cat([p.scales for p in parts]),
                         torch.cat([p.zeros for p in parts]), g)


def rows(c, idx):
    if isinstance(c, NvCanonical):
        return NvCanonical(c.codes[idx].contiguous(), c.scales[idx].contiguous(), c.row_scale[idx].contiguous(), c.group)
    return Q.W4Canonical(c.q[idx].contiguous(), c.scales[idx].contiguous(), c.zeros[idx].contiguous(), c.group)


def cols(c, lo: int, hi: int):
    if isinstance(c, NvCanonical):
        assert lo % 16 == 0 and hi % 16 == 0, "column cut must fall on a scale block boundary"
        return NvCanonical(c.codes[:, lo // 2:hi // 2].contiguous(), c.scales[:, lo // 16:hi // 16].contiguous(), c.row_scale,
                           c.group)
    g = c.group
    assert lo % g == 0 and hi % g == 0, "column cut must fall on a quantisation group boundary"
    return Q.W4Canonical(c.q[:, lo:hi].contiguous(), c.scales[:, lo // g:hi // g].contiguous(),
                         c.zeros[:, lo // g:hi // g].contiguous(), g)


def shard_w4(name: str, c, full: ModelSpec, plan: TpPlan):
    if plan.world == 1:
        return c
    r = rule_of(name)
    n, k = c.shape
    if r is Rule.COL:
        lo, hi = plan.shard_range(n)
        return rows(c, slice(lo, hi))
    if r is Rule.ROW:
        lo, hi = plan.shard_range(k)
        return cols(c, lo, hi)
    if r is Rule.Q_COL:
        lo, hi = plan.shard_range(full.hq)
        return rows(c, slice(lo * 2 * full.hd, hi * 2 * full.hd))
    if r is Rule.KV_COL:
        if full.hkv % plan.world == 0:
            lo, hi = plan.shard_range(full.hkv)
        else:
            lo = plan.rank // (plan.world // full.hkv)
            hi = lo + 1
        return rows(c, slice(lo * full.hd, hi * full.hd))
    if r is Rule.SEG_COL:
        idx = torch.cat([torch.arange(lo, hi) for lo, hi in plan.segmented_ranges([full.key_dim, full.key_dim, full.value_dim])])
        return rows(c, idx)
    return c


def interleave_rows(gate, up):
    def il(a, b):
        i = a.shape[0]
        return torch.stack([a.view(i // 8, 8, -1), b.view(i // 8, 8, -1)], dim=1).reshape(2 * i, -1)
    if isinstance(gate, NvCanonical):
        return NvCanonical(il(gate.codes, up.codes), il(gate.scales, up.scales),
                           il(gate.row_scale[:, None], up.row_scale[:, None]).reshape(-1), gate.group)
    return Q.W4Canonical(il(gate.q, up.q), il(gate.scales, up.scales), il(gate.zeros, up.zeros), gate.group)


class LoadError(ValueError):
    pass


class Stager:
    """Host-to-device upload through a bounded pinned staging buffer (``[load] staging_mb``): a tensor larger than the bound
    crosses in slices of its first dimension, so loading never pins more host memory than the bound, whatever the
    checkpoint's largest tensor is. 0 = unbounded (one copy per tensor straight from pageable memory)."""

    def __init__(self, device, staging_mb: int = 0):
        self.device = torch.device(device)
        self.cap = int(staging_mb) << 20
        self.buf = None
        self.uploads = self.slices = 0

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        self.uploads += 1
        nb = t.numel() * t.element_size()
        if self.cap == 0 or self.device.type != "cuda" or nb == 0 or t.device.type != "cpu":
            self.slices += 1
            return t.to(self.device)
        t = t.contiguous()
        if self.buf is None:
            self.buf = torch.empty(self.cap, dtype=torch.uint8).pin_memory()
        out = torch.empty_like(t, device=self.device)
        flat_src, flat_dst = t.view(-1).view(torch.uint8), out.view(-1).view(torch.uint8)
        for lo in range(0, nb, self.cap):
            n = min(self.cap, nb - lo)
            self.buf[:n].copy_(flat_src[lo:lo + n])
            flat_dst[lo:lo + n].copy_(self.buf[:n], non_blocking=True)
            torch.cuda.current_stream().synchronize()          # the staging buffer is reused by the next slice
            self.slices += 1
        return out


def tensor_table(hw, keep_tensors: bool = False) -> list[dict]:
    """Every tensor of a weight set with its place in the tree, dtype, shape and bytes (``[load] dump``)."""
    rows, seen = [], set()

    def walk(prefix, obj, depth=0):
        if id(obj) in seen or depth > 6:
            return
        seen.add(id(obj))
        if isinstance(obj, torch.Tensor):
            rows.append({"name": prefix, "dtype": str(obj.dtype).replace("torch.", ""), "shape": list(obj.shape),
                         "bytes": obj.numel() * obj.element_size(), "device": str(obj.device),
                         **({"tensor": obj} if keep_tensors else {})})
        elif isinstance(obj, dict):
            for k, v in obj.items():
                walk(f"{prefix}.{k}", v, depth + 1)
        elif isinstance(obj, (list, tuple)):
            for i, v in enumerate(obj):
                walk(f"{prefix}[{i}]", v, depth + 1)
        elif hasattr(obj, "__dict__") and not isinstance(obj, type):
            for k, v in vars(obj).items():
                if not k.startswith("_") and not callable(v):
                    walk(f"{prefix}.{k}" if prefix else k, v, depth + 1)
    walk("", hw)
    return rows


def verify_weights(hw, spec: ModelSpec) -> dict:
    """Post-load checks (``[load] verify``): the layer list matches the model description, every floating-point tensor
    (norms, scales, dense matrices, biases) is finite, and the per-layer vectors have the widths the kernels index with.
    Raises ``LoadError`` naming every offender; returns counts."""
    bad = []
    if len(hw.layers) != spec.n_layers:
        bad.append(f"{len(hw.layers)} layers loaded, the model description has {spec.n_layers}")
    for i, lw in enumerate(hw.layers):
        want = "full" if spec.is_full(i) else "gdn"
        if lw.kind != want:
            bad.append(f"layer {i}: loaded as {lw.kind}, the model description says {want}")
        for nm in ("ln1", "ln2"):
            t = getattr(lw, nm)
            if t.numel() != spec.hidden:
                bad.append(f"layer {i}.{nm}: {t.numel()} elements, hidden is {spec.hidden}")
        if lw.kind == "full" and (lw.q_norm.numel() != spec.hd or lw.k_norm.numel() != spec.hd):
            bad.append(f"layer {i}: q / k norm widths {lw.q_norm.numel()} / {lw.k_norm.numel()}, head width is {spec.hd}")
    checked = 0
    table = tensor_table(hw, keep_tensors=True)
    for r in table:
        t = r["tensor"]
        if t.is_floating_point() and t.numel():
            checked += 1
            if not bool(torch.isfinite(t.float() if t.element_size() == 1 else t).all()):
                bad.append(f"{r['name']}: non-finite values")
    n = len(table)
    if bad:
        raise LoadError("checkpoint verification failed:\n  " + "\n  ".join(bad[:32]))
    return {"tensors": n, "float_tensors_checked": checked}


def build_weights(full: ModelSpec, provider, device, rank: int = 0, world: int = 1, lm_head_int8: bool = False,
                  vocab_split: bool = True, staging_mb: int = 0, repack: str = "auto") -> H.HybridWeights:
    """Read every tensor through ``provider`` and produce the rank's device weights. ``repack``: where the canonical int4
    form is packed into the kernels' record layout: ``"cpu"`` (pack on the host, upload the records), ``"device"`` (upload
    the canonical tensors, pack with device ops: the host does not become the bottleneck of a large checkpoint), ``"auto"``
    = device on a GPU, cpu otherwise. Uploads go through ``Stager`` (``staging_mb``)."""
    from ..parallel.plan import shard_tensor

    if repack == "auto":
        repack = "device" if torch.device(device).type == "cuda" else "cpu"
    spec = full.sharded(rank, world) if world > 1 else full
    plan = TpPlan(rank, world)
    put = Stager(device, staging_mb)
    bf = lambda t: put(t.to(torch.bfloat16))
    f32 = lambda t: put(t.float())
    dn = lambda name: shard_tensor(name, provider.dense(name), full, plan)
    def w4(name):
        if world > 1 and hasattr(provider, "w4_shard"):
            c = provider.w4_shard(name, full, plan)          # the rank's window straight from the file's blocks
            if c is not None:
                return c
        return shard_w4(name, provider.w4(name), full, plan)
    def pack(c):
        if isinstance(c, NvCanonical):
            n, k = c.shape
            return Q.NvFp4Linear(put(c.codes), put(c.scales), 1.0, n, k, c.group, "nvfp4", put(c.row_scale.float()))
        if repack == "device":
            c = Q.W4Canonical(put(c.q), put(c.scales), put(c.zeros), c.group)
            return Q.pack_skinny(c)
        return Q.pack_skinny(c).to(device)
    layers, group = [], None
    for i in range(full.n_layers):
        p = f"model.layers.{i}."
        gate, up = w4(p + "mlp.gate_proj.weight"), w4(p + "mlp.up_proj.weight")
        group = gate.group
        lw = H.LayerWeights(kind="full" if full.is_full(i) else "gdn", ln1=bf(dn(p + "input_layernorm.weight")),
                            ln2=bf(dn(p + "post_attention_layernorm.weight")), gate_up=pack(interleave_rows(gate, up)),
                            down=pack(w4(p + "mlp.down_proj.weight")))
        if lw.kind == "gdn":
            a = p + "linear_attn."
            lw.qkvz = pack(cat_rows([w4(a + "in_proj_qkv.weight"), w4(a + "in_proj_z.weight")]))
            ab = torch.cat([dn(a + "in_proj_a.weight"), dn(a + "in_proj_b.weight")]).to(torch.bfloat16)
            lw.ab_dense = put(H._pad16_rows(ab))
            lw.ab = Q.dense_skinny(lw.ab_dense, device)
            lw.conv_w = f32(dn(a + "conv1d.weight").reshape(spec.conv_dim, spec.conv_k))
            lw.a_log, lw.dt_bias = f32(dn(a + "A_log")), f32(dn(a + "dt_bias"))
            lw.gamma = f32(provider.dense(a + "norm.weight"))
            lw.out_proj = pack(w4(a + "out_proj.weight"))
        else:
            a = p + "self_attn."
            lw.qkv = pack(cat_rows([w4(a + "q_proj.weight"), w4(a + "k_proj.weight"), w4(a + "v_proj.weight")]))
            lw.q_norm, lw.k_norm = bf(provider.dense(a + "q_norm.weight")), bf(provider.dense(a + "k_norm.weight"))
            lw.o_proj = pack(w4(a + "o_proj.weight"))
        layers.append(lw)
    emb = provider.dense("model.embed_tokens.weight").to(torch.bfloat16)
    head = emb if (full.tied or not provider.has("lm_head.weight")) else provider.dense("lm_head.weight").to(torch.bfloat16)
    hw = H.HybridWeights(spec=spec, embed=put(emb), final_norm=bf(provider.dense("model.norm.weight")),
                         lm_head=None, layers=layers, group=group)
    vrows = full.vocab
    if vocab_split and world > 1 and full.vocab % (16 * world) == 0:
        vrows = full.vocab // world
        hw.vocab_offset = rank * vrows
    hw.lm_head = Q.dense_skinny(put(head[hw.vocab_offset:hw.vocab_offset + vrows].contiguous()), device,
                                int8=lm_head_int8)
    return hw


def load_model(path: str | Path, device, spec: ModelSpec | None = None, rank: int = 0, world: int = 1, group: int = 128,
               **kw):
    """Open a checkpoint (any supported kind) and build the rank's weights. Returns (spec, weights)."""
    kind, provider, handle = open_source(path, group)
    if spec is None:
        if kind == "gguf":
            spec = gguf.spec_from_meta(handle.meta)
        else:
            from ..models.config_json import spec_from_hf_config

            spec = spec_from_hf_config(json.loads((Path(path) / "config.json").read_text()))
    if kind == "gguf":
        provider.set_dims(spec)
    verify, dump = kw.pop("verify", False), kw.pop("dump", False)
    hw = build_weights(spec, provider, device, rank, world, **kw)
    if verify:
        facts = verify_weights(hw, hw.spec)
        log.info("load.verify", f"{facts['tensors']} tensors, {facts['float_tensors_checked']} floating-point ones finite")
    if dump:
        for r in tensor_table(hw):
            log.info("load.dump", f"{r['name']:<48s} {r['dtype']:<10s} {str(r['shape']):<20s} {r['bytes']:>12d} B  {r['device']}")
    return spec, hw
