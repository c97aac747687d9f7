"""Checkpoint containers and codecs against host references: safetensors, AWQ / compressed-tensors, NVFP4, GGUF blocks and grids, the AWQ converter, shard plans."""
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
        gguf.dequantize(np.zeros(10, dtype=np.uint8), "IQ2_XS", 256)


def _scalar_decode(raw, t):
    """Element-by-element decoders written straight from the block layouts (independent of the vectorised codecs)."""
    from owl_engine_b200.formats.gguf_grids import IQ3S_GRID, IQ3XXS_GRID, KSIGNS

    f16 = lambda b: float(np.frombuffer(bytes(b), dtype=np.float16)[0])
    be, bb = gguf.BLOCK[t]
    out = []
    for blk in raw.reshape(-1, bb):
        b = [int(x) for x in blk]
        y = [0.0] * be
        if t == "Q4_1":
            d, m = f16(blk[0:2]), f16(blk[2:4])
            for j in range(16):
                y[j], y[j + 16] = d * (b[4 + j] & 15) + m, d * (b[4 + j] >> 4) + m
        elif t in ("Q5_0", "Q5_1"):
            o = 2 if t == "Q5_0" else 4
            d = f16(blk[0:2])
            qh = b[o] | (b[o + 1] << 8) | (b[o + 2] << 16) | (b[o + 3] << 24)
            for j in range(16):
                lo = (b[o + 4 + j] & 15) | (((qh >> j) & 1) << 4)
                hi = (b[o + 4 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4)
                if t == "Q5_0":
                    y[j], y[j + 16] = d * (lo - 16), d * (hi - 16)
                else:
                    m = f16(blk[2:4])
                    y[j], y[j + 16] = d * lo + m, d * hi + m
        elif t == "Q2_K":
            d, dmin = f16(blk[80:82]), f16(blk[82:84])
            i, is_ = 0, 0
            for h in range(2):
                q = b[16 + 32 * h:16 + 32 * h + 32]
                for j in range(4):
                    for half in range(2):
                        sc = b[is_]
                        is_ += 1
                        for l in range(16):
                            y[i] = d * (sc & 15) * ((q[half * 16 + l] >> (2 * j)) & 3) - dmin * (sc >> 4)
                            i += 1
        elif t == "Q3_K":
            d = f16(blk[108:110])
            sc = b[96:108]
            scales = []
            for k in range(16):
                low = (sc[k] & 15) if k < 8 else (sc[k - 8] >> 4)
                hi = (sc[8 + k % 4] >> (2 * (k // 4))) & 3
                scales.append((low | (hi << 4)) - 32)
            i, is_, m = 0, 0, 1
            for h in range(2):
                q = b[32 + 32 * h:32 + 32 * h + 32]
                for j in range(4):
                    for half in range(2):
                        dl = d * scales[is_]
                        is_ += 1
                        for l in range(16):
                            ll = half * 16 + l
                            y[i] = dl * (((q[ll] >> (2 * j)) & 3) - (0 if b[ll] & m else 4))
                            i += 1
                    m <<= 1
        elif t == "IQ3_XXS":
            d = f16(blk[0:2])
            for ib in range(8):
                aux = b[66 + 4 * ib] | (b[67 + 4 * ib] << 8) | (b[68 + 4 * ib] << 16) | (b[69 + 4 * ib] << 24)
                db = d * (0.5 + (aux >> 28)) * 0.5
                for l in range(4):
                    signs = int(KSIGNS[(aux >> (7 * l)) & 127])
                    g = list(IQ3XXS_GRID[b[2 + 8 * ib + 2 * l]]) + list(IQ3XXS_GRID[b[2 + 8 * ib + 2 * l + 1]])
                    for j in range(8):
                        y[32 * ib + 8 * l + j] = db * int(g[j]) * (-1 if signs & (1 << j) else 1)
        elif t == "IQ3_S":
            d = f16(blk[0:2])
            for ib in range(8):
                db = d * (1 + 2 * ((b[106 + ib // 2] >> (4 * (ib % 2))) & 15))
                qh = b[66 + ib]
                for l in range(4):
                    i1 = b[2 + 8 * ib + 2 * l] | ((qh << (8 - 2 * l)) & 256)
                    i2 = b[2 + 8 * ib + 2 * l + 1] | ((qh << (7 - 2 * l)) & 256)
                    g = list(IQ3S_GRID[i1]) + list(IQ3S_GRID[i2])
                    signs = b[74 + 4 * ib + l]
                    for j in range(8):
                        y[32 * ib + 8 * l + j] = db * int(g[j]) * (-1 if signs & (1 << j) else 1)
        out += y
    return np.asarray(out, dtype=np.float32)


@pytest.mark.parametrize("t", ["Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K", "IQ3_XXS", "IQ3_S"])
def test_gguf_new_codecs_against_scalar_decoders(t):
    be, bb = gguf.BLOCK[t]
    rng = np.random.default_rng(11)
    raw = rng.integers(0, 256, size=(6, bb), dtype=np.uint8)
    for col in {"Q4_1": (0, 2), "Q5_0": (0,), "Q5_1": (0, 2), "Q2_K": (80, 82), "Q3_K": (108,), "IQ3_XXS": (0,), "IQ3_S": (0,)}[t]:
        raw[:, col:col + 2] = rng.uniform(0.01, 0.1, size=(6,)).astype(np.float16).view(np.uint8).reshape(-1, 2)
    got = gguf.dequantize(raw.reshape(-1), t, 6 * be)
    want = _scalar_decode(raw, t)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


def test_iq3_grids_are_well_formed():
    from owl_engine_b200.formats import gguf_grids as GR

    assert GR.IQ3XXS_GRID.shape == (256, 4) and set(np.unique(GR.IQ3XXS_GRID)) == {4, 12, 20, 28, 36, 44, 52, 62}
    assert GR.IQ3S_GRID.shape == (512, 4) and set(np.unique(GR.IQ3S_GRID)) == {1, 3, 5, 7, 9, 11, 13, 15}
    assert len({bytes(r) for r in GR.IQ3XXS_GRID}) == 256 and len({bytes(r) for r in GR.IQ3S_GRID}) == 512     # no duplicate entry
    assert all(bin(int(v)).count("1") % 2 == 0 for v in GR.KSIGNS)


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


def test_gguf_shard_plans_keep_the_contiguous_block_invariant():
    """What rank r reads equals a contiguous block of the fully loaded tensor in grouped head order, for every role; what cannot
    be cut exactly is refused."""
    from owl_engine_b200.formats import gguf_shard as S

    dims = S.GdnDims(nk=4, nv=12, kd=8, vd=32)
    order = S.grouped_head_order(dims)
    assert sorted(order.tolist()) == list(range(12))
    assert order[:3].tolist() == [0, 4, 8]                  # the three value heads of key head 0 sit 4 apart in the file
    rng = np.random.default_rng(0)
    inv = np.argsort(order)

    def tiled_rows(a, width):       # grouped -> file order
        return a[S.head_rows(inv, width)]

    cases = {
        "blk.0.ffn_up.weight": (rng.standard_normal((64, 96)).astype(np.float32), None),
        "blk.0.attn_gate.weight": (rng.standard_normal((12 * 32, 64)).astype(np.float32), "rows_head"),
        "blk.0.ssm_a": (rng.standard_normal((12, 1)).astype(np.float32), "rows_head"),
        "blk.0.attn_qkv.weight": (rng.standard_normal((2 * 32 + 12 * 32, 64)).astype(np.float32), "segs"),
        "blk.0.ffn_down.weight": (rng.standard_normal((16, 128)).astype(np.float32), None),
        "blk.0.ssm_out.weight": (rng.standard_normal((16, 12 * 32)).astype(np.float32), "cols_head"),
        "blk.0.attn_norm.weight": (rng.standard_normal((64, 1)).astype(np.float32), None),
    }
    for key, (full, kind) in cases.items():
        if kind == "rows_head":
            filed = tiled_rows(full, full.shape[0] // 12)
        elif kind == "segs":
            filed = np.concatenate([full[:64], tiled_rows(full[64:], 32)])
        elif kind == "cols_head":
            filed = full[:, S.head_rows(inv, 32)]
        else:
            filed = full
        whole = S.apply_dense(filed, S.plan(key, full.shape, 1, dims, None))
        assert np.array_equal(whole, full), key
        for world in (2, 4):
            parts = [S.apply_dense(filed, S.plan(key, full.shape, 1, dims, S.ShardSel(r, world))) for r in range(world)]
            r = S.role(key)
            if r == S.REPLICATE:
                assert all(np.array_equal(p, full) for p in parts)
            elif r in (S.COLS, S.COLS_HEAD):
                assert np.array_equal(np.concatenate(parts, axis=1), full), (key, world)
            elif r == S.SEGS:
                kq = 32
                for seg, (lo, hi) in enumerate([(0, kq), (kq, 2 * kq), (2 * kq, full.shape[0])]):
                    n = (hi - lo) // world
                    got = []
                    for p in parts:
                        o = [0, kq // world, 2 * kq // world][seg]
                        got.append(p[o:o + n])
                    assert np.array_equal(np.concatenate(got), full[lo:hi]), (key, world, seg)
            else:
                assert np.array_equal(np.concatenate(parts), full), (key, world)
    # raw blocks: a column window of a block-quantised tensor is a window of blocks
    w = (rng.standard_normal((8, 512)) * 0.05).astype(np.float32)
    raw = gguf.quantize_q8_0(w)
    pl = S.plan("blk.0.ffn_down.weight", (8, 512), 32, dims, S.ShardSel(1, 2))
    cut = S.apply_raw(raw, (8, 512), 32, 34, pl)
    assert np.array_equal(gguf.dequantize(cut.reshape(-1), "Q8_0", 8 * 256).reshape(8, 256),
                          gguf.dequantize(raw, "Q8_0", 8 * 512).reshape(8, 512)[:, 256:])
    # refusals
    with pytest.raises(S.ShardError):
        S.plan("blk.0.ffn_up.weight", (66, 96), 1, dims, S.ShardSel(0, 4))            # rows not divisible
    with pytest.raises(S.ShardError):
        S.plan("blk.0.ffn_down.weight", (16, 96), 32, dims, S.ShardSel(0, 2))         # cut inside a block
    with pytest.raises(S.ShardError):
        S.plan("blk.0.ssm_out.weight", (16, 12 * 32), 256, dims, None)                # a block spans two heads
    with pytest.raises(S.ShardError):
        S.plan("blk.0.ssm_a", (12, 1), 1, S.GdnDims(4, 12, 8, 32), S.ShardSel(0, 5))  # heads not divisible
    assert S.role("output.weight") == S.REPLICATE and S.role("output.weight", S.ShardSel(0, 2, head_split=True)) == S.ROWS
