"""Vision tower (Qwen3.5-VL style ViT), image preprocessing and multimodal position ids.

Pipeline for one image:

    decode (PNG / raw RGB) -> smart_resize (both sides multiples of patch * merge, pixel budget)
    -> bicubic resample -> normalise -> patchify [n_patches, 3 * t_patch * patch * patch]
    -> patch embed (the Conv3d is a linear map on flattened patches) + learned position table
       (48 x 48, bilinearly resampled to the image's grid) -> ``depth`` blocks of
       LayerNorm -> qkv(+bias) -> 2-D axial RoPE -> non-causal attention -> proj,
       LayerNorm -> fc1 -> GELU(tanh) -> fc2
    -> merger: LayerNorm -> 2 x 2 spatial merge -> fc1 -> GELU(erf) -> fc2 -> text hidden size

The merged embeddings replace the ``<|image_pad|>`` rows of the text embedding (``scatter_images``),
and ``mrope_positions`` assigns (t, h, w) position ids: text tokens advance all three together, an
image occupies one temporal step and a (h, w) grid, the text after it resumes at max + 1.

The tower runs once per image, outside the decode loop, on dense library kernels (cuBLAS GEMMs and
torch's fused attention); the per-token hot path of the engine never touches it. ``ImageCache``
keeps the merged embeddings of the last few images by content fingerprint.

Reference counterpart: ``crates/models/src/layers/vision.rs:12-54``, ``vlm/mod.rs``,
``vlm/preprocess.rs``, ``apps/server/src/vision_processor.rs:1-20``, ``crates/engine/src/vision/vlm.rs``.
"""
from __future__ import annotations

import hashlib
import math
from collections import OrderedDict
from dataclasses import dataclass

import torch
import torch.nn.functional as F

IMAGE_MEAN = (0.5, 0.5, 0.5)
IMAGE_STD = (0.5, 0.5, 0.5)


@dataclass
class VisionSpec:
    hidden: int = 1152
    depth: int = 27
    heads: int = 16
    inter: int = 4304
    patch: int = 16
    t_patch: int = 2
    merge: int = 2
    pos_grid: int = 48
    out_hidden: int = 5120
    min_pixels: int = 56 * 56
    max_pixels: int = 1280 * 28 * 28
    eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def patch_dim(self) -> int:
        return 3 * self.t_patch * self.patch * self.patch


def tiny_vision(out_hidden: int = 256) -> VisionSpec:
    return VisionSpec(hidden=64, depth=2, heads=4, inter=128, patch=16, t_patch=2, merge=2, pos_grid=8, out_hidden=out_hidden)


# ---- preprocessing ----------------------------------------------------------------------------
def smart_resize(h: int, w: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """Round both sides to multiples of ``factor`` keeping the aspect ratio and the pixel budget."""
    if max(h, w) / max(1, min(h, w)) > 200:
        raise ValueError("aspect ratio above 200")
    hb, wb = max(factor, round(h / factor) * factor), max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb, wb = math.ceil(h * beta / factor) * factor, math.ceil(w * beta / factor) * factor
    return hb, wb


def preprocess(rgb, spec: VisionSpec) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """``rgb``: uint8 [H, W, 3] (numpy or tensor). Returns ``(patches [n, patch_dim] fp32, (t, gh, gw))``; patches are
    ordered so that each 2 x 2 merge window is contiguous (the merger reshapes without a gather)."""
    img = torch.as_tensor(rgb).permute(2, 0, 1).float()[None] / 255.0
    h, w = img.shape[-2:]
    f = spec.patch * spec.merge
    hb, wb = smart_resize(h, w, f, spec.min_pixels, spec.max_pixels)
    img = F.interpolate(img, size=(hb, wb), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 1)
    mean, std = torch.tensor(IMAGE_MEAN).view(1, 3, 1, 1), torch.tensor(IMAGE_STD).view(1, 3, 1, 1)
    img = (img - mean) / std
    frames = img.repeat(spec.t_patch, 1, 1, 1)                       # a still image fills the temporal patch
    gh, gw, p, m = hb // spec.patch, wb // spec.patch, spec.patch, spec.merge
    x = frames.view(1, spec.t_patch, 3, gh // m, m, p, gw // m, m, p)   # t, tp, c, bh, mh, ph, bw, mw, pw
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                            # t, bh, bw, mh, mw, c, tp, ph, pw
    return x.reshape(gh * gw, spec.patch_dim).contiguous(), (1, gh, gw)


def fingerprint(data: bytes) -> int:
    return int.from_bytes(hashlib.blake2b(data, digest_size=8).digest(), "little")


# ---- the tower --------------------------------------------------------------------------------
def init_vision_weights(spec: VisionSpec, seed: int = 0, std: float = 0.02) -> dict:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g) * std
    w = {"patch_embed.weight": r(spec.hidden, spec.patch_dim), "patch_embed.bias": torch.zeros(spec.hidden),
         "pos_embed": r(spec.pos_grid * spec.pos_grid, spec.hidden)}
    for i in range(spec.depth):
        b = f"blocks.{i}."
        w.update({b + "norm1.weight": torch.ones(spec.hidden), b + "norm1.bias": torch.zeros(spec.hidden),
                  b + "norm2.weight": torch.ones(spec.hidden), b + "norm2.bias": torch.zeros(spec.hidden),
                  b + "qkv.weight": r(3 * spec.hidden, spec.hidden), b + "qkv.bias": torch.zeros(3 * spec.hidden),
                  b + "proj.weight": r(spec.hidden, spec.hidden), b + "proj.bias": torch.zeros(spec.hidden),
                  b + "fc1.weight": r(spec.inter, spec.hidden), b + "fc1.bias": torch.zeros(spec.inter),
                  b + "fc2.weight": r(spec.hidden, spec.inter), b + "fc2.bias": torch.zeros(spec.hidden)})
    mh = spec.hidden * spec.merge * spec.merge
    w.update({"merger.norm.weight": torch.ones(spec.hidden), "merger.norm.bias": torch.zeros(spec.hidden),
              "merger.fc1.weight": r(mh, mh), "merger.fc1.bias": torch.zeros(mh),
              "merger.fc2.weight": r(spec.out_hidden, mh), "merger.fc2.bias": torch.zeros(spec.out_hidden)})
    return w


class VisionTower:
    def __init__(self, spec: VisionSpec, weights: dict | None = None, device="cpu", dtype=torch.float32):
        self.spec, self.device, self.dtype = spec, torch.device(device), dtype
        self.w = {k: v.to(self.device, dtype) for k, v in (weights or init_vision_weights(spec)).items()}

    def _pos_table(self, gh: int, gw: int) -> torch.Tensor:
        """The learned pos_grid x pos_grid table resampled bilinearly (4 taps) to the image's patch grid, in merge-window order."""
        sp = self.spec
        t = self.w["pos_embed"].view(1, sp.pos_grid, sp.pos_grid, sp.hidden).permute(0, 3, 1, 2).float()
        t = F.interpolate(t, size=(gh, gw), mode="bilinear", align_corners=True)[0].permute(1, 2, 0)   # gh, gw, C
        m = sp.merge
        return t.view(gh // m, m, gw // m, m, sp.hidden).permute(0, 2, 1, 3, 4).reshape(gh * gw, sp.hidden).to(self.dtype)

    def _rope(self, gh: int, gw: int) -> tuple[torch.Tensor, torch.Tensor]:
        """2-D axial RoPE: half of the rotary pairs turn with the row index, half with the column index."""
        sp = self.spec
        d = sp.head_dim // 2                 # rotary pairs
        inv = 1.0 / (10000.0 ** (torch.arange(0, d // 2, dtype=torch.float32) / (d // 2)))
        m = sp.merge
        hh = torch.arange(gh).view(gh // m, m, 1, 1).expand(gh // m, m, gw // m, m).permute(0, 2, 1, 3).reshape(-1)
        ww = torch.arange(gw).view(1, 1, gw // m, m).expand(gh // m, m, gw // m, m).permute(0, 2, 1, 3).reshape(-1)
        ang = torch.cat([hh[:, None].float() * inv[None], ww[:, None].float() * inv[None]], dim=1)   # n, d
        ang = torch.cat([ang, ang], dim=1)                                                            # rotate-half layout
        return ang.cos().to(self.device, self.dtype), ang.sin().to(self.device, self.dtype)

    @staticmethod
    def _rot(x, cos, sin):
        d = x.shape[-1] // 2
        xr = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
        return x * cos[None] + xr * sin[None]

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grid: tuple[int, int, int]) -> torch.Tensor:
        """``patches`` [n, patch_dim] in merge-window order -> merged embeddings [n / merge^2, out_hidden]."""
        sp, w = self.spec, self.w
        _, gh, gw = grid
        x = patches.to(self.device, self.dtype) @ w["patch_embed.weight"].t() + w["patch_embed.bias"]
        x = x + self._pos_table(gh, gw).to(self.device)
        cos, sin = self._rope(gh, gw)
        n, hd = x.shape[0], sp.head_dim
        for i in range(sp.depth):
            b = f"blocks.{i}."
            y = F.layer_norm(x, (sp.hidden,), w[b + "norm1.weight"], w[b + "norm1.bias"], sp.eps)
            qkv = (y @ w[b + "qkv.weight"].t() + w[b + "qkv.bias"]).view(n, 3, sp.heads, hd).permute(1, 2, 0, 3)
            q, k, v = self._rot(qkv[0], cos, sin), self._rot(qkv[1], cos, sin), qkv[2]
            a = F.scaled_dot_product_attention(q[None], k[None], v[None])[0]          # non-causal, one image = one segment
            x = x + a.permute(1, 0, 2).reshape(n, sp.hidden) @ w[b + "proj.weight"].t() + w[b + "proj.bias"]
            y = F.layer_norm(x, (sp.hidden,), w[b + "norm2.weight"], w[b + "norm2.bias"], sp.eps)
            y = F.gelu(y @ w[b + "fc1.weight"].t() + w[b + "fc1.bias"], approximate="tanh")
            x = x + y @ w[b + "fc2.weight"].t() + w[b + "fc2.bias"]
        y = F.layer_norm(x, (sp.hidden,), w["merger.norm.weight"], w["merger.norm.bias"], sp.eps)
        y = y.view(n // (sp.merge * sp.merge), -1)
        y = F.gelu(y @ w["merger.fc1.weight"].t() + w["merger.fc1.bias"])
        return y @ w["merger.fc2.weight"].t() + w["merger.fc2.bias"]

    def n_tokens(self, grid: tuple[int, int, int]) -> int:
        return grid[0] * grid[1] * grid[2] // (self.spec.merge ** 2)


class VisionTowerKernels:
    """The tower on this package's own kernels: every matrix product on the dense tcgen05 GEMM (bf16 operands), everything
    between them one fused pass each (``csrc/vision.cu``: LayerNorm, bias + GELU / residual epilogues, bilinear position
    resampling, 2-D rotary, non-causal tensor-core attention per image). Weights are converted once: bf16 matrices with the k
    dimension padded to a multiple of 64 (the GEMM's tile), fp32 vectors. Same interface and results (to bf16 rounding) as
    ``VisionTower``; several images run as one batch of segments."""

    def __init__(self, spec: VisionSpec, weights: dict | None = None, device="cuda"):
        from ..ops import kernels as K

        _bind_vision(K)
        self.spec, self.device = spec, torch.device(device)
        w = weights or init_vision_weights(spec)
        self.inter_p = (spec.inter + 63) // 64 * 64
        self.m, self.v = {}, {}
        for k, t in w.items():
            t = t.float()
            if t.dim() == 2 and k != "pos_embed":
                if k.endswith("fc1.weight") and "merger" not in k:
                    t = torch.cat([t, torch.zeros(self.inter_p - spec.inter, t.shape[1])])          # extra rows: gelu(0) = 0
                if k.endswith("fc2.weight") and "merger" not in k:
                    t = torch.cat([t, torch.zeros(t.shape[0], self.inter_p - spec.inter)], dim=1)   # and they meet zero columns
                self.m[k] = t.to(self.device, torch.bfloat16).contiguous()
            else:
                if k.endswith("fc1.bias") and "merger" not in k:
                    t = torch.cat([t, torch.zeros(self.inter_p - spec.inter)])
                self.v[k] = t.to(self.device).contiguous()

    def _gemm(self, x, name, out=None):
        from ..ops import gemm_tc

        w = self.m[name]
        out = torch.empty(x.shape[0], w.shape[0], dtype=torch.bfloat16, device=self.device) if out is None else out
        return gemm_tc.f16_gemm(x, w, out)

    @torch.no_grad()
    def forward_many(self, images: list) -> list:
        """``images``: [(patches [n_i, patch_dim], (t, gh, gw))]; returns the merged embeddings of each, bf16."""
        from ..ops import kernels as K

        sp, dev, st = self.spec, self.device, K.stream
        C, hd = sp.hidden, sp.head_dim
        x_in = torch.cat([p.to(dev, torch.bfloat16) for p, _ in images]).contiguous()
        n = x_in.shape[0]
        offs = [0]
        for p, _ in images:
            offs.append(offs[-1] + p.shape[0])
        seg = torch.tensor(offs, dtype=torch.int32, device=dev)
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=dev)
        x, y, qkv, att, mid = bf(n, C), bf(n, C), bf(n, 3 * C), bf(n, C), bf(n, self.inter_p)
        self._gemm(x_in, "patch_embed.weight", x)
        K.call("owl_vis_bias_act", K.ptr(x), C, K.ptr(self.v["patch_embed.bias"]), None, 0, K.ptr(x), C, n, C, 0, st())
        for i, (_, (_, gh, gw)) in enumerate(images):
            K.call("owl_vis_pos_embed", x.data_ptr() + offs[i] * C * 2, C, K.ptr(self.v["pos_embed"]), sp.pos_grid, gh, gw, sp.merge, C, st())
        for li in range(sp.depth):
            b = f"blocks.{li}."
            K.call("owl_vis_layernorm", K.ptr(x), C, K.ptr(self.v[b + "norm1.weight"]), K.ptr(self.v[b + "norm1.bias"]), K.ptr(y), C,
                   n, C, sp.eps, st())
            self._gemm(y, b + "qkv.weight", qkv)
            K.call("owl_vis_bias_act", K.ptr(qkv), 3 * C, K.ptr(self.v[b + "qkv.bias"]), None, 0, K.ptr(qkv), 3 * C, n, 3 * C, 0, st())
            for i, (_, (_, gh, gw)) in enumerate(images):
                K.call("owl_vis_rope", K.ptr(qkv), sp.heads, hd, offs[i], gh, gw, sp.merge, st())
            K.call("owl_vis_attn", K.ptr(qkv), K.ptr(att), n, sp.heads, hd, K.ptr(seg), len(images), st())
            self._gemm(att, b + "proj.weight", y)
            K.call("owl_vis_bias_act", K.ptr(y), C, K.ptr(self.v[b + "proj.bias"]), K.ptr(x), C, K.ptr(x), C, n, C, 0, st())
            K.call("owl_vis_layernorm", K.ptr(x), C, K.ptr(self.v[b + "norm2.weight"]), K.ptr(self.v[b + "norm2.bias"]), K.ptr(y), C,
                   n, C, sp.eps, st())
            self._gemm(y, b + "fc1.weight", mid)
            K.call("owl_vis_bias_act", K.ptr(mid), self.inter_p, K.ptr(self.v[b + "fc1.bias"]), None, 0, K.ptr(mid), self.inter_p, n,
                   self.inter_p, 1, st())
            self._gemm(mid, b + "fc2.weight", y)
            K.call("owl_vis_bias_act", K.ptr(y), C, K.ptr(self.v[b + "fc2.bias"]), K.ptr(x), C, K.ptr(x), C, n, C, 0, st())
        K.call("owl_vis_layernorm", K.ptr(x), C, K.ptr(self.v["merger.norm.weight"]), K.ptr(self.v["merger.norm.bias"]), K.ptr(y), C, n,
               C, sp.eps, st())
        mh = C * sp.merge * sp.merge
        ym = y.view(n // (sp.merge * sp.merge), mh)
        h1 = self._gemm(ym, "merger.fc1.weight")
        K.call("owl_vis_bias_act", K.ptr(h1), mh, K.ptr(self.v["merger.fc1.bias"]), None, 0, K.ptr(h1), mh, h1.shape[0], mh, 2, st())
        out = self._gemm(h1, "merger.fc2.weight")
        K.call("owl_vis_bias_act", K.ptr(out), sp.out_hidden, K.ptr(self.v["merger.fc2.bias"]), None, 0, K.ptr(out), sp.out_hidden,
               out.shape[0], sp.out_hidden, 0, st())
        m2 = sp.merge * sp.merge
        return [out[offs[i] // m2:offs[i + 1] // m2] for i in range(len(images))]

    def forward(self, patches: torch.Tensor, grid: tuple[int, int, int]) -> torch.Tensor:
        return self.forward_many([(patches, grid)])[0]

    def n_tokens(self, grid: tuple[int, int, int]) -> int:
        return grid[0] * grid[1] * grid[2] // (self.spec.merge ** 2)


def _bind_vision(K) -> None:
    import ctypes

    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    K.register("owl_vis_layernorm", [P, I, P, P, P, I, I, I, F, P])
    K.register("owl_vis_bias_act", [P, I, P, P, I, P, I, I, I, I, P])
    K.register("owl_vis_pos_embed", [P, I, P, I, I, I, I, I, P])
    K.register("owl_vis_rope", [P, I, I, I, I, I, I, P])
    K.register("owl_vis_attn", [P, P, I, I, I, P, I, P])


# ---- text side --------------------------------------------------------------------------------
def scatter_images(embeds: torch.Tensor, ids: torch.Tensor, image_pad_id: int, image_embeds: list[torch.Tensor]) -> torch.Tensor:
    """Overwrite the rows of ``embeds`` whose token is the image pad with the images' merged embeddings, in order."""
    pos = (ids == image_pad_id).nonzero().flatten()
    allv = torch.cat(image_embeds) if image_embeds else embeds[:0]
    if pos.numel() != allv.shape[0]:
        raise ValueError(f"{pos.numel()} image-pad tokens but {allv.shape[0]} image embeddings")
    embeds[pos] = allv.to(embeds.dtype).to(embeds.device)
    return embeds


def mrope_positions(ids: list[int], image_pad_id: int, grids: list[tuple[int, int, int]], merge: int = 2):
    """(t, h, w) position ids [3, n] and the position the next token continues from. Text advances all
    three components together; image k occupies a (t, gh/merge, gw/merge) block starting at the current
    position; the text after it resumes at (largest id used) + 1."""
    n = len(ids)
    pos = torch.zeros(3, n, dtype=torch.int32)
    cur, i, k = 0, 0, 0
    while i < n:
        if ids[i] != image_pad_id:
            pos[:, i] = cur
            cur += 1
            i += 1
            continue
        t, gh, gw = grids[k]
        h, w = gh // merge, gw // merge
        cnt = t * h * w
        if ids[i:i + cnt] != [image_pad_id] * cnt:
            raise ValueError("image-pad run shorter than the image's token count")
        tt = torch.arange(t).view(t, 1, 1).expand(t, h, w).reshape(-1)
        hh = torch.arange(h).view(1, h, 1).expand(t, h, w).reshape(-1)
        ww = torch.arange(w).view(1, 1, w).expand(t, h, w).reshape(-1)
        pos[0, i:i + cnt], pos[1, i:i + cnt], pos[2, i:i + cnt] = cur + tt, cur + hh, cur + ww
        cur += max(t, h, w)
        i += cnt
        k += 1
    return pos, cur


class ImageCache:
    """Merged embeddings of recent images by content fingerprint (LRU)."""

    def __init__(self, cap: int = 8):
        self.cap, self.items = cap, OrderedDict()
        self.hits = self.misses = 0

    def get(self, tower: VisionTower, data: bytes, decode) -> tuple[torch.Tensor, tuple[int, int, int], int]:
        fp = fingerprint(data)
        if fp in self.items:
            self.items.move_to_end(fp)
            self.hits += 1
            return (*self.items[fp], fp)
        self.misses += 1
        patches, grid = preprocess(decode(data), tower.spec)
        emb = tower.forward(patches, grid)
        self.items[fp] = (emb, grid)
        while len(self.items) > self.cap:
            self.items.popitem(last=False)
        return emb, grid, fp
