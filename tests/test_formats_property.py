"""Round-trip properties of the checkpoint containers and codecs on random shapes and values."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from owl_engine_b200.formats import gguf, safetensors as sf
from owl_engine_b200.ops import quant as Q


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 6), st.integers(1, 4), st.floats(0.01, 50.0), st.integers(0, 2 ** 31 - 1))
def test_gguf_block_codecs_bound_their_error(rows, blocks, scale, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, blocks * 256)) * scale).astype(np.float32)
    q8 = gguf.dequantize(gguf.quantize_q8_0(w), "Q8_0", w.size).reshape(w.shape)
    # one fp16 scale per 32 values, 8-bit codes: half a code step, plus the scale's own fp16 rounding (2^-11 relative) on up
    # to 127 steps
    amax = np.abs(w).reshape(rows, -1, 32).max(-1, keepdims=True)
    assert np.all(np.abs(q8.reshape(rows, -1, 32) - w.reshape(rows, -1, 32)) <= amax / 127 * 0.57 + 1e-6 * scale)
    q4 = gguf.dequantize(gguf.quantize_q4_k(w), "Q4_K", w.size).reshape(w.shape)
    rel = np.linalg.norm(q4 - w) / np.linalg.norm(w)
    assert rel < 0.12                                                  # 4-bit with 6-bit sub-block scales on gaussian data
    # the int4 form read from the Q4_K blocks dequantises to the same values as the block decoder
    c = gguf.q4k_to_w4(gguf.quantize_q4_k(w), rows, blocks * 256)
    assert np.allclose(c.dequant().numpy(), q4, rtol=2e-3, atol=2e-3 * scale)


@settings(max_examples=25, deadline=None)
@given(specs=st.lists(st.tuples(st.sampled_from(["F32", "F16", "Q8_0"]), st.integers(1, 5), st.integers(1, 3)), min_size=1, max_size=6),
       meta=st.dictionaries(st.text("abc.", min_size=1, max_size=8),
                            st.one_of(st.integers(0, 2 ** 40), st.floats(-1e3, 1e3, width=32), st.text("abcdefgh ", max_size=12), st.booleans(),
                                      st.lists(st.integers(-5, 5), min_size=1, max_size=4)), max_size=5))
def test_gguf_container_round_trips_metadata_and_tensors(tmp_path_factory, specs, meta):
    path = tmp_path_factory.mktemp("g") / "t.gguf"
    rng = np.random.default_rng(0)
    tensors, want = {}, {}
    for i, (tname, r, b) in enumerate(specs):
        a = rng.standard_normal((r, b * 32)).astype(np.float32)
        if tname == "F32":
            raw, back = a.view(np.uint8).reshape(-1), a
        elif tname == "F16":
            h = a.astype(np.float16)
            raw, back = h.view(np.uint8).reshape(-1), h.astype(np.float32)
        else:
            raw = gguf.quantize_q8_0(a)
            back = gguf.dequantize(raw, "Q8_0", a.size).reshape(a.shape)
        tensors[f"t{i}.weight"] = (a.shape, tname, raw)
        want[f"t{i}.weight"] = back
    gguf.write_gguf(path, meta, tensors)
    f = gguf.GgufFile(path)
    for k, v in meta.items():
        got = f.meta[k]
        assert (abs(got - v) <= 1e-6 * max(1.0, abs(v))) if isinstance(v, float) else got == v, (k, v, got)
    for name, back in want.items():
        assert tuple(f.tensors[name].shape) == back.shape
        assert np.array_equal(f.dequant(name).numpy(), back)


@settings(max_examples=30, deadline=None)
@given(st.integers(1, 4), st.integers(1, 4), st.sampled_from([32, 128]), st.integers(0, 2 ** 31 - 1))
def test_int4_records_round_trip_through_both_layouts(nt, kt, group, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(nt * 16, kt * 128, generator=g)
    c = Q.quantize_w4(w, group)
    for layout in ("slice", "block"):
        back = Q.unpack_skinny(Q.pack_skinny(c, layout))
        assert torch.equal(back.q, c.q) and torch.equal(back.scales, c.scales) and torch.equal(back.zeros.to(c.zeros.dtype), c.zeros)
    assert ((c.dequant() - w).norm() / w.norm()).item() < 0.16


@settings(max_examples=20, deadline=None)
@given(spec=st.dictionaries(st.text("abcdef._", min_size=1, max_size=10),
                            st.tuples(st.sampled_from(["f32", "bf16", "f16", "u8", "i32"]), st.lists(st.integers(1, 5), min_size=0, max_size=3)),
                            min_size=1, max_size=6))
def test_safetensors_round_trips_every_dtype_and_rank(tmp_path_factory, spec):
    path = tmp_path_factory.mktemp("s") / "m.safetensors"
    dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "u8": torch.uint8, "i32": torch.int32}
    tensors = {}
    for name, (d, shape) in spec.items():
        t = torch.randn(tuple(shape)) * 10 if dt[d].is_floating_point else torch.randint(0, 100, tuple(shape))
        tensors[name] = t.to(dt[d])
    sf.save_file(tensors, path)
    back = sf.SafeFile(path)
    assert set(back.keys()) == set(tensors)
    for name, t in tensors.items():
        got = back.get(name)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)


@settings(max_examples=300, deadline=None)
@given(st.integers(0, 2), st.lists(st.tuples(st.integers(0, 400), st.integers(0, 255)), min_size=1, max_size=6), st.integers(10, 62),
       st.integers(0, 10 ** 6))
def test_damaged_container_files_are_refused_with_a_value_error(mode, flips, big, cut):
    """Truncated files, flipped header bytes and absurd 64-bit counts: the GGUF and safetensors readers either read the file
    or raise ``ValueError`` (``UnsupportedGgufType`` for a type id they do not decode) -- nothing else, and quickly."""
    import os
    import tempfile
    import time

    d = tempfile.mkdtemp(prefix="owl_fuzz_")
    a = np.random.default_rng(0).standard_normal((4, 64)).astype(np.float32)
    gguf.write_gguf(os.path.join(d, "ok.gguf"), {"general.architecture": "qwen35", "x.list": [1, 2, 3], "x.s": "hello", "x.f": 1.5},
                    {"t.weight": (a.shape, "F32", a.view(np.uint8).reshape(-1)), "q.weight": (a.shape, "Q8_0", gguf.quantize_q8_0(a))})
    sf.save_file({"a": torch.from_numpy(a), "b": torch.arange(6).view(2, 3).to(torch.bfloat16)}, os.path.join(d, "ok.safetensors"))
    for name in ("ok.gguf", "ok.safetensors"):
        good = open(os.path.join(d, name), "rb").read()
        b = bytearray(good)
        if mode == 0:
            b = b[:cut % len(b)]
        elif mode == 1:
            for pos, val in flips:
                b[pos % min(len(b), 300)] = val
        else:
            p = flips[0][0] % (min(len(b), 300) - 8)
            b[p:p + 8] = (1 << big).to_bytes(8, "little")
        path = os.path.join(d, "bad" + os.path.splitext(name)[1])
        open(path, "wb").write(bytes(b))
        t0 = time.time()
        try:
            if name.endswith(".gguf"):
                f = gguf.GgufFile(path)
                for n in f.tensors:
                    f.dequant(n)
            else:
                f = sf.SafeFile(path)
                for n in f.keys():
                    f.get(n)
        except (ValueError, gguf.UnsupportedGgufType):
            pass
        assert time.time() - t0 < 2.0
