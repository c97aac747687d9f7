"""Checkpoints of every supported kind load into identical device weights (CPU tensors here)."""
import json

import numpy as np
import pytest
import torch

from owl_engine_b200.formats import awq, gguf, loader, safetensors as st
from owl_engine_b200.models.reference import init_weights
from owl_engine_b200.models.spec import test_hybrid as make_spec
from owl_engine_b200.ops import quant as Q


def _linear_names(spec):
    for i in range(spec.n_layers):
        p = f"model.layers.{i}."
        yield from (p + "mlp." + n + "_proj.weight" for n in ("gate", "up", "down"))
        if spec.is_full(i):
            yield from (p + "self_attn." + n + "_proj.weight" for n in "qkvo")
        else:
            yield from (p + "linear_attn." + n + ".weight" for n in ("in_proj_qkv", "in_proj_z", "out_proj"))


def test_awq_directory_loads_as_is_and_matches_dense_path(tmp_path):
    spec = make_spec(n_layers=4, vocab=512)
    dense = init_weights(spec, seed=1, std=0.05)
    tensors = {}
    for k, v in dense.items():
        tensors[k] = v
    for name in _linear_names(spec):
        c = Q.quantize_w4(dense[name], 32)
        tensors.pop(name)
        tensors.update(awq.to_compressed_tensors(c, name[:-len(".weight")]))
    st.save_file(tensors, tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps({"quantization_config": {"format": "pack-quantized"}}))
    assert loader.detect_kind(tmp_path) == "awq"
    kind, prov, _ = loader.open_source(tmp_path)
    hw = loader.build_weights(spec, prov, "cpu")
    hw2 = loader.build_weights(spec, loader.DenseProvider(dense, 32), "cpu")
    for a, b in zip(hw.layers, hw2.layers):
        assert torch.equal(a.gate_up.records, b.gate_up.records) and torch.equal(a.down.records, b.down.records)
        if a.kind == "gdn":
            assert torch.equal(a.qkvz.records, b.qkvz.records)
        else:
            assert torch.equal(a.qkv.records, b.qkv.records)
    assert hw.group == 32


def test_tp_shards_tile_the_full_weight():
    spec = make_spec(n_layers=4, vocab=512)
    dense = init_weights(spec, seed=2, std=0.05)
    prov = loader.DenseProvider(dense, 128)
    full = loader.build_weights(spec, prov, "cpu")
    parts = [loader.build_weights(spec, prov, "cpu", rank=r, world=2, vocab_split=True) for r in range(2)]
    assert parts[0].spec.inter * 2 == spec.inter and parts[1].vocab_offset == 256
    # row-parallel down_proj: the two column shards concatenate to the full canonical weight
    f = Q.unpack_skinny(full.layers[0].down)
    ps = [Q.unpack_skinny(p.layers[0].down) for p in parts]
    assert torch.equal(torch.cat([p.q for p in ps], dim=1), f.q)
    # column-parallel (interleaved) gate_up: row shards concatenate
    f = Q.unpack_skinny(full.layers[0].gate_up)
    ps = [Q.unpack_skinny(p.layers[0].gate_up) for p in parts]
    assert torch.equal(torch.cat([p.q for p in ps], dim=0), f.q)


def _to_file_order(g: str, a: np.ndarray, spec) -> np.ndarray:
    """What the converter does to a tensor of the gated-delta-net: value heads from the model's grouped order to the tiled one."""
    from owl_engine_b200.formats import gguf_shard as S

    dims = S.GdnDims(spec.nk, spec.nv, spec.kd, spec.vd)
    inv = np.argsort(S.grouped_head_order(dims))            # file position f holds grouped head inv[f]
    name = g.split(".")[2]
    r = S.role(g)
    if r == S.ROWS_HEAD:
        w = a.shape[0] // spec.nv
        return a[S.head_rows(inv, w)]
    if r == S.SEGS:
        kq = spec.nk * spec.kd
        return np.concatenate([a[:2 * kq], a[2 * kq:][S.head_rows(inv, spec.vd)]])
    if r == S.COLS_HEAD:
        return a[:, S.head_rows(inv, spec.vd)]
    return a


@pytest.mark.parametrize("order", ["grouped", "tiled"])
def test_gguf_q4k_file_loads(tmp_path, order):
    """``tiled``: the file stores the value heads the way the llama.cpp converter writes them; the loader undoes it."""
    spec = make_spec(n_layers=4, vocab=512)
    dense = init_weights(spec, seed=3, std=0.05)
    tensors = {}
    lin = set(_linear_names(spec))
    for k, v in dense.items():
        g = loader.gguf_name(k)
        a = v.float().numpy()
        a = np.ascontiguousarray(a.reshape(a.shape[0], -1) if a.ndim == 3 else a)
        if order == "tiled" and g.startswith("blk."):
            a = np.ascontiguousarray(_to_file_order(g, a, spec))
        if k.endswith(loader._PLUS_ONE_NORMS):
            a = a + 1.0
        if k in lin:
            tensors[g] = (tuple(a.shape), "Q4_K", gguf.quantize_q4_k(a))
        else:
            a = np.ascontiguousarray(a.reshape(a.shape[0], -1) if a.ndim == 3 else a)
            tensors[g] = (tuple(a.shape), "F32", a.view(np.uint8).reshape(-1))
    meta = {"general.architecture": "qwen35", "qwen35.embedding_length": spec.hidden,
            "qwen35.feed_forward_length": spec.inter, "qwen35.block_count": spec.n_layers,
            "qwen35.attention.head_count": spec.hq, "qwen35.attention.head_count_kv": spec.hkv,
            "qwen35.ssm.group_count": spec.nk, "qwen35.ssm.time_step_rank": spec.nv, "qwen35.vocab_size": spec.vocab}
    if order == "grouped":
        meta["owl.vhead_order"] = "grouped"
    gguf.write_gguf(tmp_path / "m.gguf", meta, tensors)
    got_spec, hw = loader.load_model(tmp_path / "m.gguf", "cpu")
    assert got_spec.hidden == spec.hidden and got_spec.nv == spec.nv and hw.group == 32
    c = Q.unpack_skinny(hw.layers[0].down)
    w = dense["model.layers.0.mlp.down_proj.weight"]
    assert ((c.dequant() - w).norm() / w.norm()) < 0.15
    torch.testing.assert_close(hw.layers[0].ln1.float(), dense["model.layers.0.input_layernorm.weight"], atol=1e-2, rtol=1e-2)
    # a gated-delta-net layer's tensors come out in the model's head order whichever order the file uses
    kind, prov, f = loader.open_source(tmp_path / "m.gguf")
    prov.set_dims(spec)
    for name in ("linear_attn.in_proj_z.weight", "linear_attn.out_proj.weight", "linear_attn.in_proj_qkv.weight"):
        k = f"model.layers.0.{name}"
        got = prov.w4(k).dequant()
        assert ((got - dense[k]).norm() / dense[k].norm()) < 0.15, (order, name)
    for name in ("linear_attn.A_log", "linear_attn.dt_bias", "linear_attn.in_proj_a.weight"):
        k = f"model.layers.0.{name}"
        if name.endswith("A_log"):
            continue
        torch.testing.assert_close(prov.dense(k).float().view(-1), dense[k].float().view(-1), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("order", ["grouped", "tiled"])
def test_gguf_ranks_read_their_part_from_the_raw_blocks(tmp_path, order):
    """Under tensor parallelism a rank cuts its window out of the file's Q4_K blocks before converting them; the result must
    be the tensor that slicing the fully loaded int4 form gives, for every projection, and the built weights must be equal."""
    from owl_engine_b200.parallel.plan import TpPlan

    spec = make_spec(n_layers=4, vocab=512, mult=2)            # head counts a world of 2 divides (ssm_out heads: 128 wide)
    dense = init_weights(spec, seed=5, std=0.05)
    lin = set(_linear_names(spec))
    tensors = {}
    for k, v in dense.items():
        g = loader.gguf_name(k)
        a = v.float().numpy()
        a = np.ascontiguousarray(a.reshape(a.shape[0], -1) if a.ndim == 3 else a)
        if order == "tiled" and g.startswith("blk."):
            a = np.ascontiguousarray(_to_file_order(g, a, spec))
        if k.endswith(loader._PLUS_ONE_NORMS):
            a = a + 1.0
        tensors[g] = (tuple(a.shape), "Q4_K", gguf.quantize_q4_k(a)) if k in lin else (tuple(a.shape), "F32", a.view(np.uint8).reshape(-1))
    meta = {"general.architecture": "qwen35", "qwen35.embedding_length": spec.hidden,
            "qwen35.feed_forward_length": spec.inter, "qwen35.block_count": spec.n_layers,
            "qwen35.attention.head_count": spec.hq, "qwen35.attention.head_count_kv": spec.hkv,
            "qwen35.ssm.group_count": spec.nk, "qwen35.ssm.time_step_rank": spec.nv, "qwen35.vocab_size": spec.vocab}
    if order == "grouped":
        meta["owl.vhead_order"] = "grouped"
    gguf.write_gguf(tmp_path / "m.gguf", meta, tensors)
    _, prov, _ = loader.open_source(tmp_path / "m.gguf")
    prov.set_dims(spec)
    raw_route = 0
    for rank in range(2):
        plan = TpPlan(rank, 2)
        for name in sorted(lin):
            want = loader.shard_w4(name, prov.w4(name), spec, plan)
            got = prov.w4_shard(name, spec, plan)
            if got is None:
                continue                                   # no raw plan (e.g. a super-block spanning two heads): whole read + slice
            raw_route += 1
            assert got.q.shape == want.q.shape, name
            assert torch.equal(got.q, want.q) and torch.equal(got.scales, want.scales) and torch.equal(got.zeros, want.zeros), name
    assert raw_route >= len(lin)                           # most projections take the raw route on both ranks
    # the rank's built weights are the same whichever route read them
    a = loader.build_weights(spec, prov, "cpu", rank=1, world=2)
    reads = prov.shard_reads
    prov.w4_shard = lambda *args, **kw: None
    b = loader.build_weights(spec, prov, "cpu", rank=1, world=2)
    assert reads > 0
    for la, lb in zip(a.layers, b.layers):
        for nm in ("gate_up", "down", "qkvz", "out_proj", "qkv", "o_proj"):
            ta, tb = getattr(la, nm, None), getattr(lb, nm, None)
            if ta is not None:
                assert torch.equal(ta.records, tb.records), nm
