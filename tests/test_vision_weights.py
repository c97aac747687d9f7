"""Vision-tower checkpoints: HF names and the GGUF projector file ("mmproj") against the tower's own weight dict."""
import numpy as np
import pytest
import torch

from owl_engine_b200.formats import gguf
from owl_engine_b200.formats import vision_weights as VW
from owl_engine_b200.models import vision as V


def _mmproj_file(path, spec, w, *, meta_over=None, drop=(), q8=("blocks.0.fc1.weight",)):
    """Write the tower's weights the way the converter lays out a projector file: one 4-D kernel per time slice, F16 / F32 /
    Q8_0 mixed."""
    tensors = {}
    for key, t in w.items():
        a = t.float().numpy()
        if key == "patch_embed.weight":
            k5 = a.reshape(spec.hidden, 3, spec.t_patch, spec.patch, spec.patch)
            for ti in range(spec.t_patch):
                s = np.ascontiguousarray(k5[:, :, ti])
                tensors["v.patch_embd.weight" + ("" if ti == 0 else f".{ti}")] = (s.shape, "F32", s.view(np.uint8).reshape(-1))
            continue
        name = VW.mmproj_name(key)
        if name in drop:
            continue
        if key in q8:
            tensors[name] = (a.shape, "Q8_0", gguf.quantize_q8_0(a))
        elif a.ndim == 2:
            h = np.ascontiguousarray(a.astype(np.float16))
            tensors[name] = (a.shape, "F16", h.view(np.uint8).reshape(-1))
        else:
            tensors[name] = (a.shape, "F32", np.ascontiguousarray(a).view(np.uint8).reshape(-1))
    meta = {"general.architecture": "clip", "clip.has_vision_encoder": True, "clip.projector_type": "qwen3vl_merger",
            "clip.use_gelu": True, "clip.vision.block_count": spec.depth, "clip.vision.embedding_length": spec.hidden,
            "clip.vision.feed_forward_length": spec.inter, "clip.vision.attention.head_count": spec.heads,
            "clip.vision.projection_dim": spec.out_hidden, "clip.vision.patch_size": spec.patch,
            "clip.vision.spatial_merge_size": spec.merge, "clip.vision.image_mean": [0.5, 0.5, 0.5],
            "clip.vision.image_std": [0.5, 0.5, 0.5]}
    meta.update(meta_over or {})
    gguf.write_gguf(path, meta, tensors)


def test_mmproj_round_trip_gives_the_same_tower(tmp_path):
    spec = V.tiny_vision(out_hidden=96)
    w = V.init_vision_weights(spec, seed=4, std=0.05)
    (tmp_path / "model.gguf").write_bytes(b"")
    _mmproj_file(tmp_path / "mmproj-tiny-f16.gguf", spec, w)
    got_spec, got = VW.load_mmproj(tmp_path / "model.gguf")
    assert (got_spec.hidden, got_spec.depth, got_spec.heads, got_spec.inter, got_spec.patch, got_spec.t_patch, got_spec.merge,
            got_spec.pos_grid, got_spec.out_hidden) == (spec.hidden, spec.depth, spec.heads, spec.inter, spec.patch, spec.t_patch,
                                                        spec.merge, spec.pos_grid, spec.out_hidden)
    assert torch.equal(got["patch_embed.weight"], w["patch_embed.weight"])          # the time slices interleave per channel
    assert set(got) == set(w)
    rgb = torch.randint(0, 255, (70, 90, 3), generator=torch.Generator().manual_seed(0), dtype=torch.uint8)
    patches, grid = V.preprocess(rgb, spec)
    a = V.VisionTower(spec, w).forward(patches, grid)
    b = V.VisionTower(got_spec, got).forward(patches, grid)
    assert ((a - b).norm() / a.norm()).item() < 5e-3                                 # fp16 / Q8_0 storage only


def test_mmproj_resolution_and_refusals(tmp_path):
    spec = V.tiny_vision(out_hidden=96)
    w = V.init_vision_weights(spec, seed=4)
    model = tmp_path / "model.gguf"
    model.write_bytes(b"")
    with pytest.raises(VW.VisionLoadError, match="no mmproj"):
        VW.resolve_mmproj(model)
    _mmproj_file(tmp_path / "mmproj-a.gguf", spec, w)
    assert VW.resolve_mmproj(model).name == "mmproj-a.gguf"
    _mmproj_file(tmp_path / "mmproj-b.gguf", spec, w, meta_over={"clip.projector_type": "pixtral"})
    with pytest.raises(VW.VisionLoadError, match="2 projector files"):
        VW.resolve_mmproj(model)
    assert VW.resolve_mmproj(model, tmp_path / "mmproj-b.gguf").name == "mmproj-b.gguf"
    with pytest.raises(VW.VisionLoadError, match="qwen3vl_merger"):
        VW.load_mmproj(model, tmp_path / "mmproj-b.gguf")
    _mmproj_file(tmp_path / "mmproj-c.gguf", spec, w, meta_over={"clip.vision.image_mean": [0.48, 0.45, 0.40]})
    with pytest.raises(VW.VisionLoadError, match="image_mean"):
        VW.load_mmproj(model, tmp_path / "mmproj-c.gguf")
    _mmproj_file(tmp_path / "mmproj-d.gguf", spec, w, drop=("v.blk.1.attn_out.bias",))
    with pytest.raises(VW.VisionLoadError, match="v.blk.1.attn_out.bias"):
        VW.load_mmproj(model, tmp_path / "mmproj-d.gguf")
    _mmproj_file(tmp_path / "mmproj-e.gguf", spec, w, meta_over={"general.architecture": "qwen35"})
    with pytest.raises(VW.VisionLoadError, match="clip"):
        VW.load_mmproj(model, tmp_path / "mmproj-e.gguf")


def test_hf_names_map_onto_the_tower():
    spec = V.tiny_vision(out_hidden=96)
    w = V.init_vision_weights(spec, seed=2)
    hf = {"model.language_model.embed_tokens.weight": torch.zeros(4, 4)}
    back = {"qkv": "attn.qkv", "proj": "attn.proj", "fc1": "mlp.linear_fc1", "fc2": "mlp.linear_fc2", "norm1": "norm1", "norm2": "norm2"}
    for k, t in w.items():
        if k == "patch_embed.weight":
            hf["model.visual.patch_embed.proj.weight"] = t.view(spec.hidden, 3, spec.t_patch, spec.patch, spec.patch)
        elif k == "patch_embed.bias":
            hf["model.visual.patch_embed.proj.bias"] = t
        elif k == "pos_embed":
            hf["model.visual.pos_embed.weight"] = t
        elif k.startswith("blocks."):
            _, i, mod, leaf = k.split(".")
            hf[f"model.visual.blocks.{i}.{back[mod]}.{leaf}"] = t
        else:
            hf["model.visual." + k.replace("merger.fc", "merger.linear_fc")] = t
    got = VW.from_hf(hf)
    assert set(got) == set(w) and all(torch.equal(got[k], w[k]) for k in w)
    VW.check_complete(spec, got)
    assert VW.tower_key("visual.blocks.3.attn.proj.bias") == "blocks.3.proj.bias" and VW.tower_key("lm_head.weight") is None
    with pytest.raises(VW.VisionLoadError):
        VW.tower_key("model.visual.deepstack_merger_list.0.norm.weight")
    del got["blocks.1.fc2.bias"]
    with pytest.raises(VW.VisionLoadError, match="blocks.1.fc2.bias"):
        VW.check_complete(spec, got)
    s = VW.spec_from_hf({"hidden_size": 1152, "depth": 27, "num_heads": 16, "intermediate_size": 4304, "out_hidden_size": 5120,
                         "num_position_embeddings": 2304})
    assert s.pos_grid == 48 and s.head_dim == 72
