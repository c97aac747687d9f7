"""The never-optimised fp32 CPU reference model of the hybrid (the numeric anchor).

``RefModel`` runs prefill and decode for one sequence with explicit state (KV lists for the
full-attention layers, conv + recurrent state for the GDN layers). It is the oracle of the
GPU runner and the "CPU f32 reference-numerics path" benchmark configuration.

Weight names follow HF ``Qwen3_5ForCausalLM`` (``model.layers.N.linear_attn.in_proj_qkv.weight``
...), so a real checkpoint or an HF module's ``state_dict()`` can be passed in as-is.

Reference counterpart: ``crates/models/src/reference.rs`` (sync reducer) and
``crates/backends/cpu/src/ops.rs`` (naive ops).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..ops import reference as R
from .spec import ModelSpec, mrope_section_map


def init_weights(spec: ModelSpec, seed: int = 0, std: float = 0.02, dtype=torch.float32) -> dict:
    """Random-init N(0, std) weights with HF names. Norm weights are zero-centred (stored as
    w with the op using 1+w) except the GDN gated norm (plain gamma, initialised to 1)."""
    g = torch.Generator().manual_seed(seed)
    w: dict[str, torch.Tensor] = {}

    def rnd(*shape):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    w["model.embed_tokens.weight"] = rnd(spec.vocab, spec.hidden)
    if not spec.tied:
        w["lm_head.weight"] = rnd(spec.vocab, spec.hidden)
    w["model.norm.weight"] = torch.zeros(spec.hidden, dtype=dtype)
    for i in range(spec.n_layers):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = rnd(spec.hidden)
        w[p + "post_attention_layernorm.weight"] = rnd(spec.hidden)
        if spec.is_full(i):
            a = p + "self_attn."
            w[a + "q_proj.weight"] = rnd(2 * spec.hq * spec.hd, spec.hidden)
            w[a + "k_proj.weight"] = rnd(spec.hkv * spec.hd, spec.hidden)
            w[a + "v_proj.weight"] = rnd(spec.hkv * spec.hd, spec.hidden)
            w[a + "o_proj.weight"] = rnd(spec.hidden, spec.hq * spec.hd)
            w[a + "q_norm.weight"] = rnd(spec.hd)
            w[a + "k_norm.weight"] = rnd(spec.hd)
        else:
            a = p + "linear_attn."
            w[a + "in_proj_qkv.weight"] = rnd(spec.conv_dim, spec.hidden)
            w[a + "in_proj_z.weight"] = rnd(spec.value_dim, spec.hidden)
            w[a + "in_proj_a.weight"] = rnd(spec.nv, spec.hidden)
            w[a + "in_proj_b.weight"] = rnd(spec.nv, spec.hidden)
            w[a + "conv1d.weight"] = (torch.randn(spec.conv_dim, 1, spec.conv_k, generator=g) * 0.2).to(dtype)
            w[a + "A_log"] = torch.log(torch.empty(spec.nv).uniform_(1.0, 16.0, generator=g)).to(dtype)
            w[a + "dt_bias"] = torch.ones(spec.nv, dtype=dtype)
            w[a + "norm.weight"] = torch.ones(spec.vd, dtype=dtype)
            w[a + "out_proj.weight"] = rnd(spec.hidden, spec.value_dim)
        m = p + "mlp."
        w[m + "gate_proj.weight"] = rnd(spec.inter, spec.hidden)
        w[m + "up_proj.weight"] = rnd(spec.inter, spec.hidden)
        w[m + "down_proj.weight"] = rnd(spec.hidden, spec.inter)
    return w


@dataclass
class RefState:
    """Per-sequence state of the reference model."""
    pos: int = 0
    k: dict = field(default_factory=dict)       # layer -> [S, hkv, hd]
    v: dict = field(default_factory=dict)
    conv: dict = field(default_factory=dict)    # layer -> [conv_dim, 3]
    rec: dict = field(default_factory=dict)     # layer -> [nv, kd, vd]


class RefModel:
    def __init__(self, spec: ModelSpec, weights: dict, *, kv_fp8: bool = False, chunked_gdn: bool = False,
                 linear_hook=None):
        """``kv_fp8`` rounds K/V through e4m3 like the paged pool. ``linear_hook(name, x)`` may
        return an override for a projection (used to model quantised weights)."""
        self.spec = spec
        self.w = {k: v.float() for k, v in weights.items()}
        self.kv_fp8 = kv_fp8
        self.chunked_gdn = chunked_gdn
        self.linear_hook = linear_hook
        self.inv_freq, self.rope_scale = R.rope_inv_freq(spec.rotary_dim, spec.rope_theta), 1.0
        if getattr(spec, "rope_yarn", None):
            factor, orig, bf, bs, af = spec.rope_yarn
            self.inv_freq, self.rope_scale = R.rope_yarn(spec.rotary_dim, spec.rope_theta, factor, orig or spec.max_position, bf, bs, af)
        self.section = mrope_section_map(spec)

    # -- helpers -------------------------------------------------------------------------
    def lin(self, name: str, x: torch.Tensor) -> torch.Tensor:
        if self.linear_hook is not None:
            y = self.linear_hook(name, x)
            if y is not None:
                return y
        return x @ self.w[name].t()

    def new_state(self) -> RefState:
        return RefState()

    # -- layers --------------------------------------------------------------------------
    def full_attn(self, i: int, x: torch.Tensor, st: RefState, pos3: torch.Tensor) -> torch.Tensor:
        sp, a = self.spec, f"model.layers.{i}.self_attn."
        t = x.shape[0]
        qg = self.lin(a + "q_proj.weight", x).view(t, sp.hq, 2 * sp.hd)
        q, gate = qg[..., :sp.hd], qg[..., sp.hd:]
        k = self.lin(a + "k_proj.weight", x).view(t, sp.hkv, sp.hd)
        v = self.lin(a + "v_proj.weight", x).view(t, sp.hkv, sp.hd)
        q = R.rmsnorm(q, self.w[a + "q_norm.weight"], sp.eps)
        k = R.rmsnorm(k, self.w[a + "k_norm.weight"], sp.eps)
        cos, sin = R.rope_cos_sin(pos3, self.inv_freq, self.section, self.rope_scale)
        q, k = R.apply_rope(q, cos, sin), R.apply_rope(k, cos, sin)
        if self.kv_fp8:
            k, v = R.fp8_e4m3_roundtrip(k), R.fp8_e4m3_roundtrip(v)
        past = st.k[i].shape[0] if i in st.k else 0
        st.k[i] = torch.cat([st.k[i], k]) if past else k
        st.v[i] = torch.cat([st.v[i], v]) if past else v
        o = R.gqa_attention(q, st.k[i], st.v[i], past)
        o = o.reshape(t, sp.hq * sp.hd) * torch.sigmoid(gate.reshape(t, sp.hq * sp.hd))
        return self.lin(a + "o_proj.weight", o)

    def gdn(self, i: int, x: torch.Tensor, st: RefState) -> torch.Tensor:
        sp, a = self.spec, f"model.layers.{i}.linear_attn."
        t = x.shape[0]
        qkv = self.lin(a + "in_proj_qkv.weight", x)
        z = self.lin(a + "in_proj_z.weight", x).view(t, sp.nv, sp.vd)
        av = self.lin(a + "in_proj_a.weight", x)
        bv = self.lin(a + "in_proj_b.weight", x)
        y, st.conv[i] = R.causal_conv1d(qkv, self.w[a + "conv1d.weight"].view(sp.conv_dim, sp.conv_k),
                                        st.conv.get(i))
        kdim = sp.key_dim
        q = R.l2norm(y[:, :kdim].view(t, sp.nk, sp.kd))
        k = R.l2norm(y[:, kdim:2 * kdim].view(t, sp.nk, sp.kd))
        v = y[:, 2 * kdim:].view(t, sp.nv, sp.vd)
        rep = sp.nv // sp.nk
        q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
        g, beta = R.gdn_gating(av, bv, self.w[a + "A_log"], self.w[a + "dt_bias"])
        s0 = st.rec.get(i)
        if s0 is None:
            s0 = torch.zeros(sp.nv, sp.kd, sp.vd)
        fn = R.gdn_chunked if (self.chunked_gdn and t > 1) else R.gdn_recurrent
        o, st.rec[i] = fn(q, k, v, g, beta, s0)
        o = R.gated_rmsnorm(o, z, self.w[a + "norm.weight"], sp.eps)
        return self.lin(a + "out_proj.weight", o.reshape(t, sp.value_dim))

    def mlp(self, i: int, x: torch.Tensor) -> torch.Tensor:
        m = f"model.layers.{i}.mlp."
        return self.lin(m + "down_proj.weight", R.swiglu(self.lin(m + "gate_proj.weight", x),
                                                         self.lin(m + "up_proj.weight", x)))

    # -- model ---------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, st: RefState, pos3: torch.Tensor | None = None, *, taps=None,
                embeds: torch.Tensor | None = None) -> torch.Tensor:
        """Run ``ids`` ([T]) through the model starting at ``st.pos``; returns the final
        hidden states [T, hidden] (before the last norm). ``taps`` (dict) collects the
        hidden state after the listed layers (speculative draft heads)."""
        sp = self.spec
        t = ids.shape[0]
        if pos3 is None:
            p = torch.arange(st.pos, st.pos + t)
            pos3 = torch.stack([p, p, p])
        h = self.w["model.embed_tokens.weight"][ids] if embeds is None else embeds.float()
        for i in range(sp.n_layers):
            p = f"model.layers.{i}."
            x = R.rmsnorm(h, self.w[p + "input_layernorm.weight"], sp.eps)
            h = h + (self.full_attn(i, x, st, pos3) if sp.is_full(i) else self.gdn(i, x, st))
            x = R.rmsnorm(h, self.w[p + "post_attention_layernorm.weight"], sp.eps)
            h = h + self.mlp(i, x)
            if taps is not None and i in taps:
                taps[i] = h.clone()
        st.pos += t
        return h

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        x = R.rmsnorm(h, self.w["model.norm.weight"], self.spec.eps)
        head = self.w["model.embed_tokens.weight"] if self.spec.tied else self.w["lm_head.weight"]
        return self.lin("lm_head.weight", x) if not self.spec.tied else x @ head.t()

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n_new: int, st: RefState | None = None, prefill_chunk: int = 0):
        """Greedy decode; returns (tokens [n_new], state)."""
        st = st or self.new_state()
        if prefill_chunk and prompt.shape[0] > prefill_chunk:
            h = None
            for s in range(0, prompt.shape[0], prefill_chunk):
                h = self.forward(prompt[s:s + prefill_chunk], st)
        else:
            h = self.forward(prompt, st)
        out = []
        tok = int(self.logits(h[-1:]).argmax(-1))
        out.append(tok)
        for _ in range(n_new - 1):
            h = self.forward(torch.tensor([tok]), st)
            tok = int(self.logits(h).argmax(-1))
            out.append(tok)
        return torch.tensor(out), st
