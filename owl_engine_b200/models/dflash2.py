"""DFlash2 block draft: a small bf16 transformer that reads the target's hidden states at a few tap layers and proposes
a whole block of draft tokens (1 anchor + ``block - 1`` masked rows) in ONE forward.

    memory  = hidden_norm(fc(concat of the tap hiddens))           per target position
    encode  : per draft layer  k = rope(k_norm(k_proj(memory))), v = v_proj(memory) -> ring KV (window of recent positions)
    propose : x = embed([anchor, MASK x (block-1)])
              per layer (two-stream residual):
                  h = input_ln(x + residual); (ci, delta) = attn_conv.prepare(h)
                  a = o_proj(nc_attention(q, k, v of ci; ring prefix + own block, not causal)); a = attn_conv.finish(a, delta)
                  n = post_ln(a + residual);  (ci2, delta2) = mlp_conv.prepare(n); x = mlp_conv.finish(mlp(ci2), delta2)
              hidden = norm(x + residual)
              candidates = top-16 of the TARGET lm_head on hidden[1:]; drafts = selector walk over the candidates

The grouped convolution mixes each row with its predecessor inside the block with per-row, per-group coefficients
(``kernel_projection``); the selector scores candidate pairs of neighbouring slots with two low-rank codebooks and walks
greedily. Reference: ``crates/models/src/layers/dflash2.rs:1-40`` (layer), ``:155-165`` (conv prepare / finish),
``:325-418`` (encode / propose attention), ``:518-562`` (layer forward), ``:1199-1225`` (propose block);
kernels ``crates/kernels/cu/dflash/*.cu``, ``cu/attn/naive_attn_nc.cu``. Here every projection of the 8-row block is a
weight-streaming kernel over bf16 records, the encode path uses the dense tcgen05 GEMM, and the whole propose is one
CUDA graph.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field

import torch

from ..ops import kernels as K
from ..ops import quant as Q

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
K.register("owl_dflash_conv", [_P, _P, _P, _I, _I, _I, _I, _P, _I, _P])
K.register("owl_dflash_norm_rope", [_P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _F, _I, _P])
K.register("owl_dflash_nc_attn", [_P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P])
K.register("owl_dflash_select", [_P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _P, _P, _I, _P])


@dataclass
class DraftSpec:
    hidden: int = 5120
    n_layers: int = 5
    hq: int = 32
    hkv: int = 8
    hd: int = 128
    inter: int = 17408
    vocab: int = 151936
    block: int = 8                 # 1 anchor + 7 drafts
    top_k: int = 16
    rank: int = 256
    window: int = 2048             # ring capacity (sliding window of the draft attention)
    mask_token_id: int = 0
    rope_theta: float = 1e7
    eps: float = 1e-6
    taps: tuple = (5, 19, 33, 47, 61)      # target layers whose outputs feed the draft (0-based)

    @property
    def depth(self) -> int:
        return self.block - 1

    @property
    def groups(self) -> int:
        return self.hidden // 16

    def params(self) -> int:
        h = self.hidden
        per = h * self.hq * self.hd * 2 + h * self.hkv * self.hd * 2 + 3 * h * self.inter + 2 * 4 * self.groups * h
        return self.n_layers * per + h * h * len(self.taps) + 2 * self.vocab * self.rank + self.rank * h


def tiny_spec(hidden: int = 256, vocab: int = 512) -> DraftSpec:
    return DraftSpec(hidden=hidden, n_layers=2, hq=4, hkv=2, hd=128, inter=2 * hidden, vocab=vocab, rank=64, window=64,
                     mask_token_id=vocab - 1, taps=(0, 2))


def random_dense(spec: DraftSpec, seed: int = 0, std: float = 0.05) -> dict:
    """fp32 CPU weights under the checkpoint's key names."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g) * std
    h, w = spec.hidden, {}
    w["fc.weight"] = r(h, h * len(spec.taps)) / math.sqrt(len(spec.taps))
    w["hidden_norm.weight"] = 1 + r(h)
    w["norm.weight"] = 1 + r(h)
    for i in range(spec.n_layers):
        p = f"layers.{i}."
        w[p + "input_layernorm.weight"] = 1 + r(h)
        w[p + "post_attention_layernorm.weight"] = 1 + r(h)
        w[p + "self_attn.q_proj.weight"] = r(spec.hq * spec.hd, h)
        w[p + "self_attn.k_proj.weight"] = r(spec.hkv * spec.hd, h)
        w[p + "self_attn.v_proj.weight"] = r(spec.hkv * spec.hd, h)
        w[p + "self_attn.o_proj.weight"] = r(h, spec.hq * spec.hd)
        w[p + "self_attn.q_norm.weight"] = 1 + r(spec.hd)
        w[p + "self_attn.k_norm.weight"] = 1 + r(spec.hd)
        for c in ("attention_conv", "mlp_conv"):
            base = r(2, 2, h)
            base[:, 0] += 1.0                                   # tap 0 starts as the identity
            w[p + c + ".base_kernel"] = base
            w[p + c + ".kernel_projection.weight"] = r(4 * spec.groups, h)
        w[p + "mlp.gate_proj.weight"] = r(spec.inter, h)
        w[p + "mlp.up_proj.weight"] = r(spec.inter, h)
        w[p + "mlp.down_proj.weight"] = r(h, spec.inter)
    w["selector.hidden_projection.weight"] = r(spec.rank, h)
    w["selector.predecessor_codebook"] = r(spec.vocab, spec.rank)
    w["selector.successor_codebook"] = r(spec.vocab, spec.rank)
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


# ---- fp32 reference -------------------------------------------------------------------------------------------------
def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, theta):
    """x [T, heads, hd], rotate-half over the full head dim."""
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = pos.float()[:, None] * inv[None]
    cos, sin = ang.cos()[:, None], ang.sin()[:, None]
    a, b = x[..., :hd // 2], x[..., hd // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)


def _conv_ref(x, delta, base, side, block):
    t, h = x.shape
    g = h // 16
    d = delta.view(t, 2, 2, g)[:, side]                           # [T, tap, G]
    coeff = base[side][None] + d.repeat_interleave(16, dim=-1)    # [T, tap, H]
    prev = torch.cat([torch.zeros(1, h), x[:-1]], 0)
    mask = ((torch.arange(t) % block) >= 1).float()[:, None]
    return coeff[:, 0] * x + coeff[:, 1] * prev * mask


class RefDraft:
    """Plain fp32 implementation of encode / propose (numeric anchor for the CUDA path)."""

    def __init__(self, spec: DraftSpec, w: dict, embed: torch.Tensor, lm_head: torch.Tensor):
        self.spec, self.w, self.embed, self.lm_head = spec, w, embed.float(), lm_head.float()
        self.k = [torch.zeros(0, spec.hkv, spec.hd) for _ in range(spec.n_layers)]
        self.v = [torch.zeros(0, spec.hkv, spec.hd) for _ in range(spec.n_layers)]

    def memory(self, taps: torch.Tensor) -> torch.Tensor:
        """taps [T, n_taps, hidden] -> [T, hidden]"""
        sp = self.spec
        return _rms(taps.reshape(taps.shape[0], -1) @ self.w["fc.weight"].t(), self.w["hidden_norm.weight"], sp.eps)

    def encode(self, taps: torch.Tensor, pos0: int) -> None:
        sp = self.spec
        mem = self.memory(taps)
        pos = torch.arange(pos0, pos0 + mem.shape[0])
        for i in range(sp.n_layers):
            p = f"layers.{i}.self_attn."
            k = (mem @ self.w[p + "k_proj.weight"].t()).view(-1, sp.hkv, sp.hd)
            k = _rope(_rms(k, self.w[p + "k_norm.weight"], sp.eps), pos, sp.rope_theta)
            v = (mem @ self.w[p + "v_proj.weight"].t()).view(-1, sp.hkv, sp.hd)
            self.k[i] = torch.cat([self.k[i], k])[-sp.window:]
            self.v[i] = torch.cat([self.v[i], v])[-sp.window:]

    def hidden(self, anchor: int, pos0: int) -> torch.Tensor:
        sp, w = self.spec, self.w
        ids = torch.tensor([anchor] + [sp.mask_token_id] * sp.depth)
        pos = torch.arange(pos0, pos0 + sp.block)
        x, res = self.embed[ids], None
        for i in range(sp.n_layers):
            p = f"layers.{i}."
            res = x if res is None else res + x
            h = _rms(res, w[p + "input_layernorm.weight"], sp.eps)
            delta = h @ w[p + "attention_conv.kernel_projection.weight"].t()
            ci = _conv_ref(h, delta, w[p + "attention_conv.base_kernel"], 0, sp.block)
            q = (ci @ w[p + "self_attn.q_proj.weight"].t()).view(-1, sp.hq, sp.hd)
            k = (ci @ w[p + "self_attn.k_proj.weight"].t()).view(-1, sp.hkv, sp.hd)
            v = (ci @ w[p + "self_attn.v_proj.weight"].t()).view(-1, sp.hkv, sp.hd)
            q = _rope(_rms(q, w[p + "self_attn.q_norm.weight"], sp.eps), pos, sp.rope_theta)
            k = _rope(_rms(k, w[p + "self_attn.k_norm.weight"], sp.eps), pos, sp.rope_theta)
            kk = torch.cat([self.k[i], k]).repeat_interleave(sp.hq // sp.hkv, dim=1)
            vv = torch.cat([self.v[i], v]).repeat_interleave(sp.hq // sp.hkv, dim=1)
            att = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(sp.hd)
            a = torch.einsum("hqk,khd->qhd", att.softmax(-1), vv).reshape(sp.block, -1) @ w[p + "self_attn.o_proj.weight"].t()
            a = _conv_ref(a, delta, w[p + "attention_conv.base_kernel"], 1, sp.block)
            res = res + a
            n = _rms(res, w[p + "post_attention_layernorm.weight"], sp.eps)
            d2 = n @ w[p + "mlp_conv.kernel_projection.weight"].t()
            c2 = _conv_ref(n, d2, w[p + "mlp_conv.base_kernel"], 0, sp.block)
            m = (torch.nn.functional.silu(c2 @ w[p + "mlp.gate_proj.weight"].t()) * (c2 @ w[p + "mlp.up_proj.weight"].t())) \
                @ w[p + "mlp.down_proj.weight"].t()
            x = _conv_ref(m, d2, w[p + "mlp_conv.base_kernel"], 1, sp.block)
        return _rms(res + x, w["norm.weight"], sp.eps)

    def select(self, hidden: torch.Tensor, anchor: int):
        sp, w = self.spec, self.w
        logits = hidden[1:] @ self.lm_head.t()
        unary, cand = logits.topk(sp.top_k, dim=-1)
        proj = hidden[1:] @ w["selector.hidden_projection.weight"].t()
        a_tab, b_tab = w["selector.predecessor_codebook"], w["selector.successor_codebook"]
        toks, idx = [], 0
        for e in range(sp.depth):
            pred = anchor if e == 0 else int(cand[e - 1, idx])
            score = unary[e] + (a_tab[pred][None] * proj[e][None] * b_tab[cand[e]]).sum(-1)
            idx = int(score.argmax())
            toks.append(int(cand[e, idx]))
        return toks, cand, unary

    def propose(self, anchor: int, pos0: int):
        return self.select(self.hidden(anchor, pos0), anchor)[0]


# ---- device model ---------------------------------------------------------------------------------------------------
@dataclass
class DraftLayer:
    ln1: torch.Tensor
    ln2: torch.Tensor
    qkv: Q.DenseSkinny            # rows: q | k | v  (one stream for the three projections of the block)
    kv_dense: torch.Tensor        # [2 * hkv * hd, hidden] bf16 row-major (encode path, dense GEMM)
    o_proj: Q.DenseSkinny
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    conv_a_base: torch.Tensor
    conv_a_proj: Q.DenseSkinny
    conv_m_base: torch.Tensor
    conv_m_proj: Q.DenseSkinny
    gate_up: Q.DenseSkinny        # gate / up rows interleaved in eights (the order the activation kernel reads)
    down: Q.DenseSkinny


@dataclass
class DraftWeights:
    fc: torch.Tensor              # [hidden, n_taps * hidden] bf16 (dense GEMM / streaming)
    fc_rec: Q.DenseSkinny
    hidden_norm: torch.Tensor
    norm: torch.Tensor
    layers: list = field(default_factory=list)
    sel_proj: Q.DenseSkinny = None
    a_tab: torch.Tensor = None
    b_tab: torch.Tensor = None

    def nbytes(self) -> int:
        n = self.fc.numel() * 2 + self.fc_rec.nbytes + self.a_tab.numel() * 4 + self.sel_proj.nbytes
        for l in self.layers:
            n += l.qkv.nbytes + l.o_proj.nbytes + l.gate_up.nbytes + l.down.nbytes + l.conv_a_proj.nbytes + \
                l.conv_m_proj.nbytes + l.kv_dense.numel() * 2
        return n


def weights_from_dense(spec: DraftSpec, w: dict, device) -> DraftWeights:
    bf = lambda t: t.to(torch.bfloat16).to(device).contiguous()
    rec = lambda t: Q.dense_skinny(t.to(torch.bfloat16), device)
    out = DraftWeights(fc=bf(w["fc.weight"]), fc_rec=rec(w["fc.weight"]), hidden_norm=bf(w["hidden_norm.weight"]),
                       norm=bf(w["norm.weight"]))
    for i in range(spec.n_layers):
        p = f"layers.{i}."
        q, k, v = (w[p + f"self_attn.{n}_proj.weight"] for n in "qkv")
        out.layers.append(DraftLayer(
            ln1=bf(w[p + "input_layernorm.weight"]), ln2=bf(w[p + "post_attention_layernorm.weight"]),
            qkv=rec(torch.cat([q, k, v], 0)), kv_dense=bf(torch.cat([k, v], 0)), o_proj=rec(w[p + "self_attn.o_proj.weight"]),
            q_norm=bf(w[p + "self_attn.q_norm.weight"]), k_norm=bf(w[p + "self_attn.k_norm.weight"]),
            conv_a_base=bf(w[p + "attention_conv.base_kernel"]), conv_a_proj=rec(w[p + "attention_conv.kernel_projection.weight"]),
            conv_m_base=bf(w[p + "mlp_conv.base_kernel"]), conv_m_proj=rec(w[p + "mlp_conv.kernel_projection.weight"]),
            gate_up=rec(Q.interleave_gate_up(w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"])),   # order of silu_mul
            down=rec(w[p + "mlp.down_proj.weight"])))
    out.sel_proj = rec(w["selector.hidden_projection.weight"])
    out.a_tab, out.b_tab = bf(w["selector.predecessor_codebook"]), bf(w["selector.successor_codebook"])
    return out


def random_weights(spec: DraftSpec, device, seed: int = 0) -> DraftWeights:
    """Random-init weights generated on the device tensor by tensor (the 27B-size draft never exists in fp32)."""
    g = torch.Generator(device="cpu").manual_seed(seed)

    def r(*s, std=0.02, one=False):
        t = torch.randn(*s, generator=g, dtype=torch.float32) * std
        return (1 + t if one else t).to(torch.bfloat16)

    h = spec.hidden
    d = {"fc.weight": r(h, h * len(spec.taps)), "hidden_norm.weight": r(h, one=True), "norm.weight": r(h, one=True)}
    for i in range(spec.n_layers):
        p = f"layers.{i}."
        d[p + "input_layernorm.weight"], d[p + "post_attention_layernorm.weight"] = r(h, one=True), r(h, one=True)
        d[p + "self_attn.q_proj.weight"], d[p + "self_attn.k_proj.weight"] = r(spec.hq * spec.hd, h), r(spec.hkv * spec.hd, h)
        d[p + "self_attn.v_proj.weight"], d[p + "self_attn.o_proj.weight"] = r(spec.hkv * spec.hd, h), r(h, spec.hq * spec.hd)
        d[p + "self_attn.q_norm.weight"], d[p + "self_attn.k_norm.weight"] = r(spec.hd, one=True), r(spec.hd, one=True)
        for c in ("attention_conv", "mlp_conv"):
            base = r(2, 2, h).float()
            base[:, 0] += 1.0
            d[p + c + ".base_kernel"], d[p + c + ".kernel_projection.weight"] = base.to(torch.bfloat16), r(4 * spec.groups, h)
        d[p + "mlp.gate_proj.weight"], d[p + "mlp.up_proj.weight"] = r(spec.inter, h), r(spec.inter, h)
        d[p + "mlp.down_proj.weight"] = r(h, spec.inter)
    d["selector.hidden_projection.weight"] = r(spec.rank, h)
    d["selector.predecessor_codebook"], d["selector.successor_codebook"] = r(spec.vocab, spec.rank), r(spec.vocab, spec.rank)
    return weights_from_dense(spec, d, device)


class DFlash2:
    """The draft on the GPU for ONE sequence at a time (ring KV per layer); ``embed`` / ``lm_head`` are the target's."""

    SPLITS = 16

    def __init__(self, spec: DraftSpec, weights: DraftWeights, embed: torch.Tensor, lm_head, device, *, max_encode: int = 2048,
                 pdl: bool = True):
        self.spec, self.w, self.embed, self.lm_head, self.device, self.pdl = spec, weights, embed, lm_head, device, pdl
        sp, B = spec, spec.block
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=device)
        f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=device)
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=device)
        self.ring_k = [bf(sp.window, sp.hkv, sp.hd) for _ in range(sp.n_layers)]
        self.ring_v = [bf(sp.window, sp.hkv, sp.hd) for _ in range(sp.n_layers)]
        self.n_seen = 0                                    # positions encoded so far (host mirror)
        self.prefix_len = i32(1)                           # min(n_seen, window), read by the attention kernel
        self.inv_freq = (1.0 / (sp.rope_theta ** (torch.arange(0, sp.hd, 2, dtype=torch.float32) / sp.hd))).to(device)
        nqkv = (sp.hq + 2 * sp.hkv) * sp.hd
        self.ids, self.pos, self.anchor = i32(B), i32(B), i32(1)
        self.x, self.res, self.h, self.ci = bf(B, sp.hidden), bf(B, sp.hidden), bf(B, sp.hidden), bf(B, sp.hidden)
        self.delta = bf(B, 4 * sp.groups)
        self.qkv, self.q, self.k = bf(B, nqkv), bf(B, sp.hq, sp.hd), bf(B, sp.hkv, sp.hd)
        self.att, self.a = bf(B, sp.hq * sp.hd), bf(B, sp.hidden)
        self.gu, self.act, self.m = bf(B, 2 * sp.inter), bf(B, sp.inter), bf(B, sp.hidden)
        self.part_o, self.part_ml = f32(sp.hkv * self.SPLITS * 32 * sp.hd), f32(sp.hkv * self.SPLITS * 32 * 2)
        self.hidden = bf(B, sp.hidden)
        self.logits = bf(B, lm_head.n)
        self.topk = K.TopK(device, max_rows=B, k=sp.top_k)
        self.proj = bf(B, sp.rank)
        self.drafts = i32(sp.depth)
        self.scores = f32(sp.depth * sp.top_k * sp.top_k)
        # encode workspace
        self.max_encode = max_encode
        self.e_mem, self.e_memn = bf(max_encode, sp.hidden), bf(max_encode, sp.hidden)
        self.e_kv = bf(max_encode, 2 * sp.hkv * sp.hd)
        self.e_pos, self.e_slot = i32(max_encode), i32(max_encode)
        self.graph = None

    # -- encode: target tap hiddens -> ring KV ------------------------------------------------------------------------
    def reset(self) -> None:
        self.n_seen = 0
        self.prefix_len.zero_()

    def encode(self, taps: torch.Tensor, pos0: int) -> None:
        """taps bf16 [T, n_taps * hidden] (tap hiddens of T consecutive positions starting at pos0, concatenated per row)."""
        from ..ops import gemm_tc

        sp, w = self.spec, self.w
        t = taps.shape[0]
        assert t <= self.max_encode and taps.shape[1] == sp.hidden * len(sp.taps)
        mem, memn, kv = self.e_mem[:t], self.e_memn[:t], self.e_kv[:t]
        if t <= 32:
            K.dense_skinny(w.fc_rec, taps, mem, t)
        else:
            gemm_tc.f16_gemm(taps, w.fc, mem)
        K.rmsnorm_pack(mem, w.hidden_norm, normed=memn, m=t, k=sp.hidden, eps=sp.eps, one_plus_w=False)
        lo = max(0, t - sp.window)          # rows older than the window would only race with their successors for a slot
        n = t - lo
        self.e_pos[:n] = torch.arange(pos0 + lo, pos0 + t, dtype=torch.int32, device=self.device)
        self.e_slot[:n] = self.e_pos[:n] % sp.window
        nk = sp.hkv * sp.hd
        kv = kv[:n]
        for i, lw in enumerate(w.layers):
            gemm_tc.f16_gemm(memn[lo:], lw.kv_dense, kv, force_small=True)
            K.call("owl_dflash_norm_rope", K.ptr(kv), kv.stride(0), K.ptr(kv[:, nk:]), kv.stride(0), K.ptr(lw.k_norm),
                   K.ptr(self.e_pos), K.ptr(self.inv_freq), None, K.ptr(self.ring_k[i]), K.ptr(self.ring_v[i]),
                   K.ptr(self.e_slot), n, sp.hkv, sp.eps, 0, K.stream())
        self.n_seen = pos0 + t
        self.prefix_len.fill_(min(self.n_seen, sp.window))

    # -- propose ------------------------------------------------------------------------------------------------------
    def _gemv(self, w, x, out, m):
        K.dense_skinny(w, x, out, m, pdl=self.pdl)

    def _conv(self, x, delta, base, side, out):
        sp = self.spec
        K.call("owl_dflash_conv", K.ptr(x), K.ptr(delta), K.ptr(base), side, sp.block, sp.hidden, sp.block, K.ptr(out),
               int(self.pdl), K.stream())

    def _forward(self) -> None:
        """ids / pos / anchor -> drafts (all device buffers; capturable)."""
        sp, w, B, pdl = self.spec, self.w, self.spec.block, int(self.pdl)
        K.embed(self.ids, self.embed, self.x, B, pdl=self.pdl)
        nq, nk = sp.hq * sp.hd, sp.hkv * sp.hd
        first = True
        for i, lw in enumerate(w.layers):
            if first:
                self.res.copy_(self.x)
                K.rmsnorm_pack(self.res, lw.ln1, normed=self.h, m=B, k=sp.hidden, eps=sp.eps, one_plus_w=False, pdl=self.pdl)
                first = False
            else:
                K.rmsnorm_pack(self.res, lw.ln1, delta=self.x, out_h=self.res, normed=self.h, m=B, k=sp.hidden, eps=sp.eps,
                               one_plus_w=False, pdl=self.pdl)
            self._gemv(lw.conv_a_proj, self.h, self.delta, B)
            self._conv(self.h, self.delta, lw.conv_a_base, 0, self.ci)
            self._gemv(lw.qkv, self.ci, self.qkv, B)
            K.call("owl_dflash_norm_rope", K.ptr(self.qkv), self.qkv.stride(0), None, 0, K.ptr(lw.q_norm), K.ptr(self.pos),
                   K.ptr(self.inv_freq), K.ptr(self.q), None, None, None, B, sp.hq, sp.eps, pdl, K.stream())
            K.call("owl_dflash_norm_rope", K.ptr(self.qkv[:, nq:]), self.qkv.stride(0), None, 0, K.ptr(lw.k_norm),
                   K.ptr(self.pos), K.ptr(self.inv_freq), K.ptr(self.k), None, None, None, B, sp.hkv, sp.eps, pdl, K.stream())
            K.call("owl_dflash_nc_attn", K.ptr(self.q), K.ptr(self.k), K.ptr(self.qkv[:, nq + nk:]), self.qkv.stride(0),
                   K.ptr(self.ring_k[i]), K.ptr(self.ring_v[i]), K.ptr(self.prefix_len), K.ptr(self.part_o),
                   K.ptr(self.part_ml), K.ptr(self.att), B, sp.hq, sp.hkv, sp.window, self.SPLITS, 1.0 / math.sqrt(sp.hd), pdl,
                   K.stream())
            self._gemv(lw.o_proj, self.att, self.a, B)
            self._conv(self.a, self.delta, lw.conv_a_base, 1, self.x)
            K.rmsnorm_pack(self.res, lw.ln2, delta=self.x, out_h=self.res, normed=self.h, m=B, k=sp.hidden, eps=sp.eps,
                           one_plus_w=False, pdl=self.pdl)
            self._gemv(lw.conv_m_proj, self.h, self.delta, B)
            self._conv(self.h, self.delta, lw.conv_m_base, 0, self.ci)
            self._gemv(lw.gate_up, self.ci, self.gu, B)
            K.silu_mul(self.gu, B, sp.inter, out=self.act, pdl=self.pdl)
            self._gemv(lw.down, self.act, self.m, B)
            self._conv(self.m, self.delta, lw.conv_m_base, 1, self.x)
        K.rmsnorm_pack(self.res, w.norm, delta=self.x, out_h=self.res, normed=self.hidden, m=B, k=sp.hidden, eps=sp.eps,
                       one_plus_w=False, pdl=self.pdl)
        d = sp.depth
        K.dense_skinny(self.lm_head, self.hidden[1:], self.logits, d, pdl=self.pdl)
        val, idx = self.topk(self.logits, d, self.lm_head.n)
        self._gemv(w.sel_proj, self.hidden[1:], self.proj, d)
        K.call("owl_dflash_select", K.ptr(idx), K.ptr(val), K.ptr(self.proj), self.proj.stride(0), K.ptr(self.anchor),
               K.ptr(w.a_tab), K.ptr(w.b_tab), d, sp.top_k, sp.rank, K.ptr(self.drafts), K.ptr(self.scores), pdl, K.stream())

    def capture(self) -> None:
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._forward()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._forward()
        self.graph = g

    def propose(self, anchor: int, pos0: int, depth: int | None = None) -> list[int]:
        """Draft tokens for the positions after ``pos0`` (the anchor's position)."""
        sp = self.spec
        self.ids[0] = anchor
        self.ids[1:] = sp.mask_token_id
        self.anchor[0] = anchor
        self.pos.copy_(torch.arange(pos0, pos0 + sp.block, dtype=torch.int32, device=self.device))
        if self.graph is not None:
            self.graph.replay()
        else:
            self._forward()
        return self.drafts[:depth or sp.depth].tolist()
