"""Plain PyTorch (fp32) reference implementations of every op. They are the numeric oracle of
the CUDA kernels and the building blocks of the CPU reference model.

Formulas follow the HF ``transformers`` Qwen3.5 modelling code (the same gold standard the
reference uses in ``crates/models/src/layers/*.py``) and ``crates/backends/cpu/src/ops.rs``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, one_plus_w: bool = True) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y * ((1.0 + w.float()) if one_plus_w else w.float())


def rope_inv_freq(rotary_dim: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.int64).float() / rotary_dim))


def rope_yarn(rotary_dim: int, theta: float, factor: float, original_max: int, beta_fast: float = 32.0, beta_slow: float = 1.0,
              attention_factor: float = 1.0) -> tuple[torch.Tensor, float]:
    """YaRN context extension: per-frequency blend of the original rotary frequencies (dimensions that turn more than
    ``beta_fast`` times within the trained context keep theirs) and frequencies divided by ``factor`` (dimensions that turn
    less than ``beta_slow`` times), linear in between; cos / sin are multiplied by ``(0.1 ln(factor) + 1) * attention_factor``.
    Returns (inv_freq [rotary_dim / 2], scale). ``factor <= 1`` is plain rope.

    Reference counterpart: ``[model.rope]`` of ``profiles/full.toml:147-155`` (YaRN keys; the same formula as the HF
    ``yarn`` rope type)."""
    base = rope_inv_freq(rotary_dim, theta)
    if factor <= 1.0:
        return base, float(attention_factor)

    def turn_dim(n_rot: float) -> float:              # the (fractional) frequency index that makes n_rot turns in original_max
        return rotary_dim * math.log(original_max / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

    lo = max(math.floor(turn_dim(beta_fast)), 0)
    hi = min(math.ceil(turn_dim(beta_slow)), rotary_dim - 1)
    if lo == hi:
        hi += 0.001
    ramp = ((torch.arange(rotary_dim // 2, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)
    keep = 1.0 - ramp                                 # 1 = extrapolate (original frequency), 0 = interpolate (divided by factor)
    inv = base / factor * (1 - keep) + base * keep
    return inv, float((0.1 * math.log(factor) + 1.0) * attention_factor)


def rope_cos_sin(pos3: torch.Tensor, inv_freq: torch.Tensor, section: list[int], scale: float = 1.0):
    """pos3: int [3, T]. Returns cos, sin of shape [T, rotary_dim/2] (fp32 angle as in HF)."""
    sec = torch.tensor(section, dtype=torch.long)
    pos = pos3.float()[sec, :].t()                      # [T, half]
    ang = pos * inv_freq.float()[None, :]
    return ang.cos() * scale, ang.sin() * scale


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, H, hd]; rotate-half over the first 2*half dims, the rest pass through."""
    half = cos.shape[-1]
    x1, x2, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


def gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos0: int) -> torch.Tensor:
    """Causal GQA. q: [T, hq, hd]; k, v: [S, hkv, hd] (S = cached + new); row t sees
    keys 0..q_pos0+t. Returns [T, hq, hd]."""
    t, hq, hd = q.shape
    s, hkv, _ = k.shape
    rep = hq // hkv
    kf = k.float().repeat_interleave(rep, dim=1)
    vf = v.float().repeat_interleave(rep, dim=1)
    scores = torch.einsum("thd,shd->hts", q.float(), kf) / math.sqrt(hd)
    idx_q = torch.arange(t)[:, None] + q_pos0
    idx_k = torch.arange(s)[None, :]
    scores = scores.masked_fill((idx_k > idx_q)[None], float("-inf"))
    p = scores.softmax(-1)
    return torch.einsum("hts,shd->thd", p, vf)


def fp8_e4m3_roundtrip(x: torch.Tensor) -> torch.Tensor:
    """Value after a saturating cast to e4m3 (the KV pool storage) and back."""
    return x.float().clamp(-448, 448).to(torch.float8_e4m3fn).float()


def causal_conv1d(x: torch.Tensor, w: torch.Tensor, hist: torch.Tensor | None):
    """Depthwise causal conv, kernel 4, no bias, then SiLU. x: [T, C]; w: [C, 4];
    hist: [C, 3] (x[t-3], x[t-2], x[t-1]) or None. Returns (y [T, C], new_hist [C, 3])."""
    t, c = x.shape
    h = hist.float() if hist is not None else torch.zeros(c, 3)
    full = torch.cat([h.t(), x.float()], dim=0)          # [T+3, C]
    y = sum(full[j:j + t] * w.float()[:, j][None, :] for j in range(4))
    return F.silu(y), full[-3:].t().contiguous()


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gdn_gating(a: torch.Tensor, b: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor):
    g = -torch.exp(a_log.float()) * F.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float())


def gdn_recurrent(q, k, v, g, beta, state):
    """Serial gated delta rule. q,k: [T, nv, kd] (already l2-normed, GVA-expanded);
    v: [T, nv, vd]; g, beta: [T, nv]; state: [nv, kd, vd] fp32 (updated copy returned)."""
    t = q.shape[0]
    s = state.float().clone()
    scale = 1.0 / math.sqrt(q.shape[-1])
    out = torch.zeros(t, v.shape[1], v.shape[2])
    for i in range(t):
        s = s * torch.exp(g[i])[:, None, None]
        kv = torch.einsum("hk,hkv->hv", k[i].float(), s)
        delta = beta[i][:, None] * (v[i].float() - kv)
        s = s + torch.einsum("hk,hv->hkv", k[i].float(), delta)
        out[i] = torch.einsum("hk,hkv->hv", q[i].float() * scale, s)
    return out, s


def gdn_chunked(q, k, v, g, beta, state, chunk: int = 64):
    """Chunked (WY representation) gated delta rule; same contract as ``gdn_recurrent``."""
    t, h, kd = q.shape
    vd = v.shape[-1]
    pad = (chunk - t % chunk) % chunk
    qf, kf, vf = (F.pad(x.float().transpose(0, 1), (0, 0, 0, pad)) for x in (q, k, v))   # [h, T', d]
    gf, bf = (F.pad(x.float().t(), (0, pad)) for x in (g, beta))                           # [h, T']
    n = (t + pad) // chunk
    qf = qf * (1.0 / math.sqrt(kd))
    qc, kc, vc = (x.view(h, n, chunk, -1) for x in (qf, kf, vf))
    gc = gf.view(h, n, chunk).cumsum(-1)
    bc = bf.view(h, n, chunk)
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()
    kb, vb = kc * bc[..., None], vc * bc[..., None]
    eye = torch.eye(chunk)
    a = -((kb @ kc.transpose(-1, -2)) * decay).masked_fill(torch.triu(torch.ones(chunk, chunk, dtype=torch.bool)), 0)
    # (I - A)^-1 by forward substitution
    tmat = torch.linalg.solve_triangular(eye - a, eye.expand_as(a).contiguous(), upper=False)
    u = tmat @ vb
    w = tmat @ (kb * gc.exp()[..., None])
    s = state.float().clone()
    out = torch.zeros(h, n, chunk, vd)
    strict = torch.triu(torch.ones(chunk, chunk, dtype=torch.bool), diagonal=1)
    for i in range(n):
        attn = ((qc[:, i] @ kc[:, i].transpose(-1, -2)) * decay[:, i]).masked_fill(strict, 0)
        v_new = u[:, i] - w[:, i] @ s
        out[:, i] = (qc[:, i] * gc[:, i, :, None].exp()) @ s + attn @ v_new
        s = s * gc[:, i, -1, None, None].exp() + \
            (kc[:, i] * (gc[:, i, -1, None] - gc[:, i]).exp()[..., None]).transpose(-1, -2) @ v_new
    out = out.view(h, n * chunk, vd)[:, :t].transpose(0, 1).contiguous()
    return out, s


def gated_rmsnorm(o: torch.Tensor, z: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """rmsnorm(o) * gamma * silu(z) over the last dim (per head)."""
    of = o.float()
    y = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps)
    return y * gamma.float() * F.silu(z.float())


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate.float()) * up.float()


def layernorm(x, w, b, eps=1e-6):
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps)


def gelu_tanh(x):
    return F.gelu(x.float(), approximate="tanh")


def gelu_erf(x):
    return F.gelu(x.float())
