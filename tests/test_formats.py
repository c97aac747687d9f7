import numpy as np
import pytest
import torch

from owl_engine_b200.formats import awq, gguf, nvfp4, safetensors as st
from owl_engine_b200.ops import quant as Q


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4, 2).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
         "d": torch.randn(8).to(torch.float8_e4m3fn)}
    st.save_file(t, tmp_path / "m.safetensors", {"format": "pt"})
    d = st.SafeDir(tmp_path)
    assert set(d.keys()) == set(t)
    for k in t:
        assert torch.equal(d.get(k).view(torch.uint8) if t[k].dtype == torch.float8_e4m3fn else d.get(k),
                           t[k].view(torch.uint8) if t[k].dtype == torch.float8_e4m3fn else t[k])


@pytest.mark.parametrize("group", [32, 128])
def test_awq_compressed_tensors_roundtrip(tmp_path, group):
    c = Q.quantize_w4(torch.randn(64, 256), group)
    st.save_file(awq.to_compressed_tensors(c, "l.down_proj"), tmp_path / "q.safetensors")
    c2 = awq.from_compressed_tensors(st.SafeDir(tmp_path), "l.down_proj")
    assert torch.equal(c.q, c2.q) and torch.equal(c.zeros, c2.zeros) and c2.group == group
    torch.testing.assert_close(c2.dequant(), c.dequant())


def test_autoawq_layout():
    c = Q.quantize_w4(torch.randn(16, 256), 128)
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    def pack(x):   # x [rows, cols] uint8, pack along cols in AutoAWQ order
        v = x.view(x.shape[0], -1, 8)[..., order].to(torch.int64)
        w = (v << (torch.arange(8) * 4)).sum(-1)
        return torch.where(w >= 2**31, w - 2**32, w).to(torch.int32)
    c2 = awq.from_autoawq(pack(c.q.t().contiguous()), pack(c.zeros.t().contiguous()), c.scales.t().contiguous())
    assert torch.equal(c2.q, c.q) and torch.equal(c2.zeros, c.zeros)


def test_nvfp4_codec():
    w = torch.randn(128, 256) * 0.05
    q = nvfp4.quantize(w)
    d = nvfp4.dequantize(q)
    assert ((d - w).norm() / w.norm()) < 0.12
    vals = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.5, -6.0])
    assert torch.equal(nvfp4.decode_e2m1(nvfp4.encode_e2m1(vals)), vals)
    codes, sf = nvfp4.pack_for_mma(q)
    assert sf.shape == (1, 4, 512)


def test_gguf_container_and_codecs(tmp_path):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((64, 256)) * 0.05).astype(np.float32)
    tensors = {"a.f32": ((64, 256), "F32", w.view(np.uint8).reshape(-1)),
               "a.q8": ((64, 256), "Q8_0", gguf.quantize_q8_0(w)),
               "a.q4k": ((64, 256), "Q4_K", gguf.quantize_q4_k(w))}
    meta = {"general.architecture": "qwen35", "general.name": "t", "qwen35.embedding_length": 256,
            "qwen35.feed_forward_length": 512, "qwen35.block_count": 4, "qwen35.attention.head_count": 6,
            "qwen35.attention.head_count_kv": 1, "tokenizer.ggml.tokens": ["a", "b", "c"], "tokenizer.ggml.eos_token_id": 2}
    gguf.write_gguf(tmp_path / "m.gguf", meta, tensors)
    f = gguf.GgufFile(tmp_path / "m.gguf")
    assert f.meta["qwen35.block_count"] == 4 and f.tensors["a.q4k"].shape == (64, 256)
    assert torch.equal(f.dequant("a.f32"), torch.from_numpy(w))
    assert (f.dequant("a.q8") - torch.from_numpy(w)).abs().max() < 2e-3
    dq = f.dequant("a.q4k")
    assert ((dq - torch.from_numpy(w)).norm() / np.linalg.norm(w)) < 0.12
    c = gguf.q4k_to_w4(f.raw("a.q4k"), 64, 256)
    torch.testing.assert_close(c.dequant(), dq, rtol=2e-2, atol=2e-3)
    spec = gguf.spec_from_meta(f.meta)
    assert spec.hidden == 256 and spec.n_layers == 4 and gguf.tokenizer_from_meta(f.meta)["eos"] == 2


def test_gguf_other_codecs_shapes():
    rng = np.random.default_rng(1)
    for t in ["Q4_0", "Q5_K", "Q6_K", "IQ4_NL", "IQ4_XS"]:
        be, bb = gguf.BLOCK[t]
        raw = rng.integers(0, 255, size=bb * 4, dtype=np.uint8)
        d16 = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
        if t == "Q6_K":
            raw.reshape(4, bb)[:, 208:210] = d16
        else:
            raw.reshape(4, bb)[:, 0:2] = d16
            if t == "Q5_K":
                raw.reshape(4, bb)[:, 2:4] = d16
        out = gguf.dequantize(raw, t, be * 4)
        assert out.shape == (be * 4,) and np.isfinite(out).all()
    with pytest.raises(gguf.UnsupportedGgufType):
        gguf.dequantize(np.zeros(10, dtype=np.uint8), "IQ3_S", 256)


def test_awq_forge_converts_a_dense_checkpoint(tmp_path):
    import json
    import torch
    from owl_engine_b200.forge import awq as forge
    from owl_engine_b200.formats import awq as A
    from owl_engine_b200.formats import safetensors as ST

    g = torch.Generator().manual_seed(0)
    src = tmp_path / "src"; src.mkdir()
    w = (torch.randn(64, 128, generator=g) * 0.05)
    dense = {"model.layers.0.mlp.down_proj.weight": w.to(torch.bfloat16),
             "model.layers.0.input_layernorm.weight": torch.ones(128, dtype=torch.bfloat16),
             "lm_head.weight": torch.randn(32, 128, generator=g).to(torch.bfloat16)}
    ST.save_file(dense, src / "model.safetensors")
    (src / "config.json").write_text(json.dumps({"hidden_size": 128}))
    rep = forge.convert(src, tmp_path / "rtn", group=32)
    assert rep["quantized"] == 1 and rep["bytes_after"] < rep["bytes_before"]
    out = ST.SafeDir(tmp_path / "rtn")
    assert "lm_head.weight" in out and "model.layers.0.mlp.down_proj.weight_packed" in out
    c = A.from_compressed_tensors(out, "model.layers.0.mlp.down_proj")
    err = (c.dequant() - w.to(torch.bfloat16).float()).abs().max() / w.abs().max()
    assert err < 0.08
    assert json.loads((tmp_path / "rtn" / "config.json").read_text())["quantization_config"]["config_groups"]["group_0"]["weights"]["group_size"] == 32
    # activation-aware mode: channels with large activations get finer resolution -> lower output error
    x = torch.randn(256, 128, generator=g)
    x[:, :8] *= 30.0
    forge.convert(src, tmp_path / "awq", group=32, mode="awq", calib={"model.layers.0.mlp.down_proj": x})
    o2 = ST.SafeDir(tmp_path / "awq")
    c2 = A.from_compressed_tensors(o2, "model.layers.0.mlp.down_proj")
    sinv = o2.get("model.layers.0.mlp.down_proj.input_scale_inv").float()
    ref = x @ w.to(torch.bfloat16).float().t()
    e_rtn = (x @ c.dequant().t() - ref).pow(2).mean()
    e_awq = ((x * sinv) @ c2.dequant().t() - ref).pow(2).mean()
    assert e_awq <= e_rtn * 1.02


def test_nvfp4_checkpoint_source_and_row_surgery():
    """ModelOpt-style NVFP4 tensors (packed codes, e4m3 block scales, fp32 per-tensor scale) keep their values through the
    loader's row / column / interleave surgery: the per-tensor scale travels as a per-row scale."""
    import torch

    from owl_engine_b200.formats import loader as L, nvfp4

    g = torch.Generator().manual_seed(0)
    dense = {n: torch.randn(r, 64, generator=g) * s for n, r, s in (("q.weight", 32, 0.05), ("k.weight", 16, 0.2), ("g.weight", 16, 0.1),
                                                                    ("u.weight", 16, 0.4))}
    src = {}
    for n, w in dense.items():
        q = nvfp4.quantize(w)
        src[n], src[n + "_scale"] = q.codes, q.scales.view(torch.float8_e4m3fn)
        src[n + "_scale_2"] = torch.tensor(q.global_scale)
        dense[n] = nvfp4.dequantize(q)
    prov = L.NvFp4Provider(src, 128)

    def deq(c):
        n, k = c.shape
        q = nvfp4.NvFp4(c.codes, c.scales, 1.0, (n, k))
        return nvfp4.dequantize(q) * c.row_scale[:, None]

    qk = L.cat_rows([prov.w4("q.weight"), prov.w4("k.weight")])
    assert torch.allclose(deq(qk), torch.cat([dense["q.weight"], dense["k.weight"]]), rtol=1e-6, atol=1e-8)
    assert torch.allclose(deq(L.cols(qk, 16, 48)), torch.cat([dense["q.weight"], dense["k.weight"]])[:, 16:48], rtol=1e-6, atol=1e-8)
    assert torch.allclose(deq(L.rows(qk, slice(8, 40))), torch.cat([dense["q.weight"], dense["k.weight"]])[8:40], rtol=1e-6, atol=1e-8)
    gu = L.interleave_rows(prov.w4("g.weight"), prov.w4("u.weight"))
    from owl_engine_b200.ops import quant as Q
    assert torch.allclose(deq(gu), Q.interleave_gate_up(dense["g.weight"], dense["u.weight"]), rtol=1e-6, atol=1e-8)
