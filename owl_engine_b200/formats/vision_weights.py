"""Vision-tower checkpoints: HF safetensors names and the GGUF ``mmproj`` container, both mapped onto the tower's own keys.

The tower (``models/vision.py``) names its tensors ``patch_embed.{weight,bias}``, ``pos_embed``, ``blocks.<i>.{norm1,norm2,qkv,
proj,fc1,fc2}.{weight,bias}`` and ``merger.{norm,fc1,fc2}.{weight,bias}``.

* **HF** (``[model.]visual.*`` inside the language model's safetensors): ``patch_embed.proj.weight`` is a Conv3d kernel
  ``[out, in, t, p, p]`` and flattens to ``[out, in * t * p * p]`` (the order the preprocessor writes patches in);
  ``blocks.<i>.attn.qkv / attn.proj / mlp.linear_fc1 / mlp.linear_fc2`` and ``merger.linear_fc1 / linear_fc2`` lose their
  module path.
* **mmproj** (llama.cpp's projector file next to a GGUF language model; ``general.architecture = "clip"``,
  ``clip.projector_type = "qwen3vl_merger"``): hyper-parameters come from ``clip.vision.*`` metadata, except the side of the
  position table (rows of ``v.position_embd.weight``) and the temporal patch size (whether ``v.patch_embd.weight.1`` exists).
  The Conv3d kernel is stored as one 4-D tensor per time slice; HF order interleaves the slices per input channel
  (``stack`` on a new axis after ``in``), it does not append them. Anything the tower cannot represent is refused loudly: a
  different projector, deepstack layers, a normalisation other than mean = std = 0.5, a non-square position table.

Reference counterpart: ``crates/models/src/formats/gguf/mmproj.rs:1-420`` (facts, key map, time-slice merge, path resolution),
``crates/models/src/layers/vision.rs`` (HF key surface).
"""
from __future__ import annotations

import math
from pathlib import Path

import torch

from ..models.vision import IMAGE_MEAN, IMAGE_STD, VisionSpec
from . import gguf


class VisionLoadError(ValueError):
    pass


_HF_LOCAL = {"attn.qkv": "qkv", "attn.proj": "proj", "mlp.linear_fc1": "fc1", "mlp.linear_fc2": "fc2", "norm1": "norm1",
             "norm2": "norm2"}
_HF_TOP = {"patch_embed.proj.bias": "patch_embed.bias", "pos_embed.weight": "pos_embed", "merger.norm.weight": "merger.norm.weight",
           "merger.norm.bias": "merger.norm.bias", "merger.linear_fc1.weight": "merger.fc1.weight",
           "merger.linear_fc1.bias": "merger.fc1.bias", "merger.linear_fc2.weight": "merger.fc2.weight",
           "merger.linear_fc2.bias": "merger.fc2.bias"}
_MM_LOCAL = {"norm1": "ln1", "norm2": "ln2", "qkv": "attn_qkv", "proj": "attn_out", "fc1": "ffn_up", "fc2": "ffn_down"}
_MM_TOP = {"patch_embed.bias": "v.patch_embd.bias", "pos_embed": "v.position_embd.weight", "merger.norm.weight": "v.post_ln.weight",
           "merger.norm.bias": "v.post_ln.bias", "merger.fc1.weight": "mm.0.weight", "merger.fc1.bias": "mm.0.bias",
           "merger.fc2.weight": "mm.2.weight", "merger.fc2.bias": "mm.2.bias"}


def tower_key(hf_key: str) -> str | None:
    """HF tensor name -> the tower's key (None: not a vision tensor)."""
    k = hf_key
    for pre in ("model.visual.", "visual."):
        if k.startswith(pre):
            k = k[len(pre):]
            break
    else:
        return None
    if k == "patch_embed.proj.weight":
        return "patch_embed.weight"
    if k in _HF_TOP:
        return _HF_TOP[k]
    if k.startswith("blocks."):
        _, idx, rest = k.split(".", 2)
        mod, _, leaf = rest.rpartition(".")
        if mod in _HF_LOCAL and leaf in ("weight", "bias"):
            return f"blocks.{idx}.{_HF_LOCAL[mod]}.{leaf}"
    raise VisionLoadError(f"vision checkpoint: no place in the tower for {hf_key!r}")


def from_hf(tensors: dict) -> dict:
    """``{HF name: tensor}`` (other tensors are skipped) -> the tower's weight dict."""
    out = {}
    for name, t in tensors.items():
        key = tower_key(name)
        if key is None:
            continue
        if key == "patch_embed.weight" and t.dim() == 5:
            t = t.reshape(t.shape[0], -1)                 # [out, in, t, p, p] -> [out, in * t * p * p]
        out[key] = t
    return out


def spec_from_hf(vision_config: dict, **over) -> VisionSpec:
    """``vision_config`` of an HF ``config.json`` -> ``VisionSpec``."""
    c = vision_config
    n_pos = int(c.get("num_position_embeddings", 2304))
    side = math.isqrt(n_pos)
    if side * side != n_pos:
        raise VisionLoadError(f"num_position_embeddings = {n_pos} is not a square")
    return VisionSpec(hidden=c["hidden_size"], depth=c["depth"], heads=c["num_heads"], inter=c["intermediate_size"],
                      patch=c.get("patch_size", 16), t_patch=c.get("temporal_patch_size", 2), merge=c.get("spatial_merge_size", 2),
                      pos_grid=side, out_hidden=c["out_hidden_size"], **over)


def check_complete(spec: VisionSpec, w: dict) -> None:
    """Every tensor the tower reads is there with the shape it indexes with."""
    from ..models.vision import init_vision_weights

    want = {k: tuple(v.shape) for k, v in init_vision_weights(spec).items()}
    missing = sorted(set(want) - set(w))
    wrong = sorted(f"{k}: {tuple(w[k].shape)} instead of {want[k]}" for k in want if k in w and tuple(w[k].shape) != want[k])
    if missing or wrong:
        raise VisionLoadError("vision tower checkpoint incomplete: missing " + ", ".join(missing[:8] or ["-"]) +
                              "; wrong shapes " + "; ".join(wrong[:8] or ["-"]))


# ---- mmproj -----------------------------------------------------------------------------------------------------------------
def resolve_mmproj(text_model: str | Path, explicit: str | Path | None = None) -> Path:
    """The projector file of a GGUF language model: ``explicit`` when given, else the only ``mmproj*.gguf`` in the same
    directory; none or several are refused with the candidates listed."""
    if explicit:
        p = Path(explicit)
        if not p.is_file():
            raise VisionLoadError(f"[vision] path is not a file: {p}")
        return p
    d = Path(text_model).parent
    cands = sorted(p for p in d.iterdir() if p.name.startswith("mmproj") and p.suffix == ".gguf" and p.is_file())
    if not cands:
        raise VisionLoadError(f"vision is enabled but {d} holds no mmproj*.gguf; set [vision] path")
    if len(cands) > 1:
        raise VisionLoadError(f"{d} holds {len(cands)} projector files ({', '.join(c.name for c in cands)}); name one in [vision] path")
    return cands[0]


def mmproj_spec(f: gguf.GgufFile, **over) -> VisionSpec:
    m = f.meta
    where = f"mmproj {f.path}"

    def need(key):
        if key not in m:
            raise VisionLoadError(f"{where}: metadata key {key} is missing")
        return m[key]

    arch = m.get("general.architecture")
    if arch != "clip":
        raise VisionLoadError(f"{where}: general.architecture = {arch!r}, a projector file says \"clip\"")
    if not m.get("clip.has_vision_encoder", False):
        raise VisionLoadError(f"{where}: clip.has_vision_encoder is not true")
    proj = need("clip.projector_type")
    if proj != "qwen3vl_merger":
        raise VisionLoadError(f"{where}: clip.projector_type = {proj!r}; only qwen3vl_merger is supported")
    if not m.get("clip.use_gelu", False):
        raise VisionLoadError(f"{where}: clip.use_gelu is not true (the tower's MLP uses GELU)")
    if any(m.get("clip.vision.is_deepstack_layers", []) or []):
        raise VisionLoadError(f"{where}: deepstack layers are not supported")
    for key, want in (("clip.vision.image_mean", IMAGE_MEAN), ("clip.vision.image_std", IMAGE_STD)):
        got = m.get(key)
        if got is not None and any(abs(float(a) - float(b)) > 1e-6 for a, b in zip(got, want)):
            raise VisionLoadError(f"{where}: {key} = {list(got)} but the preprocessor normalises with {list(want)}")
    hidden, heads = int(need("clip.vision.embedding_length")), int(need("clip.vision.attention.head_count"))
    depth, inter = int(need("clip.vision.block_count")), int(need("clip.vision.feed_forward_length"))
    out_hidden, patch = int(need("clip.vision.projection_dim")), int(need("clip.vision.patch_size"))
    merge = int(need("clip.vision.spatial_merge_size"))
    eps = float(m.get("clip.vision.attention.layer_norm_epsilon", 1e-6))
    if min(hidden, heads, depth, out_hidden, patch, merge) <= 0 or hidden % heads or not (eps > 0 and math.isfinite(eps)):
        raise VisionLoadError(f"{where}: inconsistent hyper-parameters (hidden {hidden}, heads {heads}, depth {depth}, eps {eps})")
    pos = f.tensors.get("v.position_embd.weight")
    if pos is None or len(pos.shape) != 2 or pos.shape[1] != hidden:
        raise VisionLoadError(f"{where}: v.position_embd.weight is missing or not [positions, {hidden}]")
    side = math.isqrt(pos.shape[0])
    if side * side != pos.shape[0]:
        raise VisionLoadError(f"{where}: {pos.shape[0]} position rows are not a square table")
    p0 = f.tensors.get("v.patch_embd.weight")
    if p0 is None or len(p0.shape) != 4 or p0.shape[0] != hidden or p0.shape[2] != patch or p0.shape[3] != patch or p0.shape[1] != 3:
        raise VisionLoadError(f"{where}: v.patch_embd.weight is missing or not [{hidden}, 3, {patch}, {patch}]")
    p1 = f.tensors.get("v.patch_embd.weight.1")
    if p1 is not None and tuple(p1.shape) != tuple(p0.shape):
        raise VisionLoadError(f"{where}: the two time slices of the patch kernel differ in shape")
    return VisionSpec(hidden=hidden, depth=depth, heads=heads, inter=inter, patch=patch, t_patch=2 if p1 is not None else 1,
                      merge=merge, pos_grid=side, out_hidden=out_hidden, eps=eps, **over)


def mmproj_name(key: str) -> str:
    """The tower's key -> the projector file's tensor name."""
    if key in _MM_TOP:
        return _MM_TOP[key]
    if key.startswith("blocks."):
        _, idx, mod, leaf = key.split(".")
        return f"v.blk.{idx}.{_MM_LOCAL[mod]}.{leaf}"
    raise KeyError(key)


def mmproj_weights(f: gguf.GgufFile, spec: VisionSpec) -> dict:
    """Every tensor of the tower, dequantised to fp32 (the tower is prefill-only and under 1 GB; projector files mix F16,
    F32 and Q8_0)."""
    from ..models.vision import init_vision_weights

    out = {}
    for key in init_vision_weights(VisionSpec(hidden=8, depth=spec.depth, heads=1, inter=8, pos_grid=1, out_hidden=8)):
        if key == "patch_embed.weight":
            a = f.dequant("v.patch_embd.weight").float()
            if spec.t_patch == 2:
                a = torch.stack([a, f.dequant("v.patch_embd.weight.1").float()], dim=2)      # [out, in, t, p, p]
            out[key] = a.reshape(a.shape[0], -1).contiguous()
            continue
        name = mmproj_name(key)
        if name not in f.tensors:
            raise VisionLoadError(f"mmproj {f.path}: tensor {name} (the tower's {key}) is missing")
        out[key] = f.dequant(name).float()
    check_complete(spec, out)
    return out


def load_mmproj(text_model: str | Path, explicit: str | Path | None = None, **over):
    """(spec, weights) of the projector file that belongs to a GGUF language model."""
    f = gguf.GgufFile(resolve_mmproj(text_model, explicit))
    spec = mmproj_spec(f, **over)
    return spec, mmproj_weights(f, spec)
