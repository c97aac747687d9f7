"""Profile keys are honoured or refused: validation refusals, the pieces the keys switch (YaRN rope, speculative depth rules,
loader staging / verification, request dumps, the evict pad token, launch-ring capacity), all without a GPU."""
import json
import math
import os

import pytest
import torch

from owl_engine_b200.utils import config as C

FULL = os.path.join(os.path.dirname(__file__), "..", "configs", "full.toml")


def load(*sets):
    return C.load(FULL, list(sets))


@pytest.mark.parametrize("sets, needle", [
    (["store.evict_policy=\"mru\""], "evict_policy"),
    (["store.evict_policy=\"lrfu:-1\""], "evict_policy"),
    (["store.snap_disk_mb=64"], "snap_disk_mb needs the disk tier"),
    (["model.embed_quant=\"int8-row\""], "embed_quant"),
    (["model.rope.yarn_factor=0.5"], "yarn_factor"),
    (["store.kv.draft_kv_dtype=\"fp8\""], "draft_kv_dtype"),
    (["spec.mtp_window=4032"], "mtp_window"),
    (["spec.mtp_ring=true"], "mtp_ring"),
    (["spec.tp_draft=true"], "tp_draft"),
    (["spec.q_alpha=0.5"], "q_alpha"),
    (["spec.adaptive_depth=true"], "adaptive_depth"),
    (["spec.force_accept=9"], "force_accept"),
    (["kvmem.select_decode=true", "kvmem.score_mode=\"dot-mean\""], "score_mode"),
    (["kvmem.select_decode=true", "kvmem.gqa_aggregation=\"mean\""], "gqa_aggregation"),
    (["kvmem.select_decode=true", "kvmem.select_query_tokens=512"], "select_query_tokens"),
    (["kernel.gdn_fused_decode=false"], "gdn_fused_decode"),
    (["kernel.attn_splits=100"], "attn_splits"),
    (["cuda.launch_sync=true"], "launch_sync"),
    (["cuda.graph=false", "spec.kind=\"mtp\"", "spec.depth=3"], "cuda.graph = false"),
    (["log.max_mb=8"], "log.file"),
    (["load.repack=\"always\""], "load.repack"),
])
def test_values_this_build_cannot_honour_are_refused(sets, needle):
    with pytest.raises(C.ConfigError) as ei:
        load(*sets)
    assert needle in str(ei.value)


def test_values_that_are_honoured_pass():
    cfg = load("store.evict_policy=\"lrfu:0.8\"", "model.rope.yarn_factor=4.0", "cuda.graph=false", "cuda.launch_sync=true",
               "log.file=\"/tmp/owl.log\"", "log.max_mb=8", "log.keep=3", "kvmem.select_decode=true", "kvmem.recall_every=4",
               "spec.kind=\"mtp\"", "spec.depth=5", "spec.adaptive_depth=true", "store.kv.draft_kv_dtype=\"fp8\"",
               "cuda.graph=true", "cuda.launch_sync=false", "load.repack=\"device\"", "load.verify=true")
    assert cfg.get("store.evict_policy") == "lrfu:0.8" and cfg.get("spec.depth_switch_ctx") == 49152


def test_yarn_matches_the_published_formula():
    from owl_engine_b200.ops import reference as R

    inv, scale = R.rope_yarn(64, 1e7, 4.0, 4096)
    base = R.rope_inv_freq(64, 1e7)
    assert torch.allclose(inv[:4], base[:4]) and torch.allclose(inv[-4:], base[-4:] / 4.0)        # fast dims keep, slow dims stretch
    assert torch.all(inv[1:] <= inv[:-1]) and abs(scale - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    same, one = R.rope_yarn(64, 1e7, 1.0, 4096)
    assert torch.equal(same, base) and one == 1.0
    rot = pytest.importorskip("transformers.modeling_rope_utils")

    class Cfg:
        rope_theta, head_dim, hidden_size, num_attention_heads, partial_rotary_factor = 1e7, 64, 256, 4, 1.0
        max_position_embeddings = 16384
        rope_scaling = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 4096, "beta_fast": 32.0, "beta_slow": 1.0}
        rope_parameters = dict(rope_scaling, rope_theta=1e7)

        def standardize_rope_params(self):
            pass
    try:
        hf_inv, hf_scale = rot.ROPE_INIT_FUNCTIONS["yarn"](Cfg(), "cpu")
    except Exception as ex:   # noqa: BLE001  (the library's config protocol changed)
        pytest.skip(f"transformers yarn initialiser not callable with a plain object: {ex}")
    assert torch.allclose(hf_inv, inv, rtol=0, atol=0) and abs(hf_scale - scale) < 1e-12


def test_engine_config_carries_yarn_into_the_model_description():
    from owl_engine_b200.engine.core import Engine, EngineConfig

    e = Engine(EngineConfig(model="test-hybrid", n_pages=32, n_slots=2, max_seqs=2, max_seq=256, rope_yarn=(4.0, 4096, 32.0, 1.0, 1.0)),
               device="cpu")
    assert e.full_spec.rope_yarn == (4.0, 4096, 32.0, 1.0, 1.0)
    assert Engine(EngineConfig(model="test-hybrid", n_pages=32, n_slots=2, max_seqs=2, max_seq=256), device="cpu").full_spec.rope_yarn is None


def test_speculative_depth_and_degrade_rules():
    from owl_engine_b200.engine.spec import SpecRunner

    s = SpecRunner(None, depth=6, depth_min=3, switch_ctx=1000, degrade_after=3, probe_every=5, window=1000)
    assert s.depth_for(999) == 6 and s.depth_for(1000) == 3
    assert SpecRunner(None, depth=2, depth_min=3, switch_ctx=10).depth_for(50) == 2          # never deeper than depth
    assert SpecRunner(None, depth=6).depth_for(10 ** 6) == 6                                    # adaptive off
    for m in (0, 0, 1, 0, 0):
        s._note(m)
    assert s._cool == 0                       # the streak was broken by an accepted draft
    s._note(0)
    assert s._cool == 5 and s._zero_streak == 0
    assert s._accept([5, 6, 7], [5, 6, 9, 1]) == (2, [5, 6, 9])
    f = SpecRunner(None, depth=3, force_accept=2)
    assert f._accept([5, 8, 7], [5, 6, 9, 1]) == (2, [5, 8, 9])      # the drafts are taken whatever the target said
    assert f._accept([5], [4, 6]) == (1, [5, 6])


def test_stager_bounds_and_reproduces(monkeypatch):
    from owl_engine_b200.formats.loader import Stager

    st = Stager("cpu", staging_mb=1)
    t = torch.arange(1 << 19, dtype=torch.float32)            # 2 MiB
    out = st(t)
    assert torch.equal(out, t) and st.uploads == 1


def test_verify_weights_names_the_offender():
    from dataclasses import replace

    from owl_engine_b200.formats import loader as L
    from owl_engine_b200.models import hybrid as H
    from owl_engine_b200.models.spec import PRESETS

    spec = replace(PRESETS["test-hybrid"](), n_layers=4)
    hw = H.random_weights(spec, torch.device("cpu"), group=128, seed=1)
    facts = L.verify_weights(hw, spec)
    assert facts["tensors"] > 20 and facts["float_tensors_checked"] > 8
    names = {r["name"] for r in L.tensor_table(hw)}
    assert any(n.startswith("layers[0].") for n in names) and "final_norm" in names
    hw.layers[1].ln2[3] = float("nan")
    with pytest.raises(L.LoadError) as ei:
        L.verify_weights(hw, spec)
    assert "layers[1].ln2" in str(ei.value)
    with pytest.raises(L.LoadError) as ei:
        L.verify_weights(hw, replace(spec, n_layers=5))
    assert "5" in str(ei.value)


def test_evict_pad_token_must_be_one_token():
    from owl_engine_b200.engine.tokenizer import ByteTokenizer
    from owl_engine_b200.server.main import evict_pad_token

    tok = ByteTokenizer()
    assert evict_pad_token(load("vision.image_evict_pad=\".\""), tok) == ord(".")
    assert evict_pad_token(load("vision.image_evict_pad=\"\""), tok) == ord(" ")         # the ideographic stop is 3 bytes here
    with pytest.raises(C.ConfigError):
        evict_pad_token(load("vision.image_evict_pad=\"..\""), tok)


def test_launch_ring_capacity_follows_the_profile():
    from owl_engine_b200.ops import kernels as K

    old = K._LAUNCHES.maxlen
    try:
        K.set_trace_ring(16)
        assert K._LAUNCHES.maxlen == 16
        K.set_trace_ring(0)
        assert K._LAUNCHES.maxlen == 2048
    finally:
        K.set_trace_ring(old)


def test_http_cpu_face_dumps_requests_and_reuses_a_shared_system_prompt(tmp_path):
    """Through the whole stack on the CPU face: two conversations with one system prompt and different user messages; the
    second is served from the snapshot at the message boundary (``usage.prompt_tokens_details``), bodies are dumped, the
    rendered prompt and the raw completion reach the log, step-profile events reach the metrics store."""
    import asyncio
    import sys

    sys.path.insert(0, os.path.dirname(__file__))
    from owl_engine_b200.engine.core import Engine, EngineConfig
    from owl_engine_b200.engine.service import EngineService
    from owl_engine_b200.engine.tokenizer import ByteTokenizer
    from owl_engine_b200.server.http import App, serve
    from owl_engine_b200.utils.log import LOG
    from owl_engine_b200.utils.metrics import METRICS
    from test_server_http import request

    tok = ByteTokenizer()
    ecfg = EngineConfig(model="test-hybrid", n_pages=256, n_slots=4, n_snap_rows=6, max_seqs=4, max_seq=2048, prefill_chunk=64,
                        msg_open_ids=tuple(tok.encode("<|im_start|>")), snap_msg_min_gap=32, snap_msg_recent=2, snap_decode_stride=1)
    svc = EngineService(lambda: Engine(ecfg, device="cpu"), max_batch=4, running_kw={"step_profile": True})
    client = svc.boot()
    METRICS.set_level("host")
    system = "You are a careful assistant. " * 12

    async def main():
        app = App(client, tok, "test-hybrid", request_dump_dir=str(tmp_path / "dumps"), prompt_dump=True, raw_completion=True)
        server = await serve(app, "127.0.0.1", 0)
        port = server.sockets[0].getsockname()[1]
        async with server:
            out = []
            for user in ("first question, fairly short", "a different second question of another length"):
                body = {"messages": [{"role": "system", "content": system}, {"role": "user", "content": user}],
                        "max_tokens": 8, "ignore_eos": True}
                st, _, raw = await request(port, "POST", "/v1/chat/completions", body)
                assert st == 200
                out.append(json.loads(raw))
            return out
    try:
        first, second = asyncio.run(main())
    finally:
        assert svc.shutdown().code == 0
    cached = lambda r: r["usage"].get("prompt_tokens_details", {}).get("cached_tokens", r["usage"].get("cached_tokens", 0))
    assert cached(first) == 0
    n_sys = len(tok.encode("<|im_start|>system\n" + system))
    assert cached(second) >= n_sys // 16 * 16 - 16 and cached(second) % 16 == 0 and cached(second) > 0
    assert len(os.listdir(tmp_path / "dumps")) == 2
    tail = "\n".join(LOG.tail(200))
    assert "[server.prompt]" in tail and "[server.raw]" in tail
    steps = [e for e in METRICS.events if e["tag"] == "engine.step"]
    assert {"begin", "prefill", "decode"} <= {e["kind"] for e in steps} and all(e["ms"] >= 0 for e in steps)


def test_request_dump_prompt_dump_and_raw_completion(tmp_path):
    from owl_engine_b200.engine.tokenizer import ByteTokenizer
    from owl_engine_b200.server.http import App

    app = App(client=None, tokenizer=ByteTokenizer(), model_name="m", request_dump_dir=str(tmp_path / "dumps"), prompt_dump=True)
    app._dump_request(b'{"messages": []}')
    app._dump_request(b'{"messages": [1]}')
    files = sorted(os.listdir(tmp_path / "dumps"))
    assert len(files) == 2 and json.loads(open(tmp_path / "dumps" / files[1]).read()) == {"messages": [1]}
    assert app.prompt_dump and not app.raw_completion


def test_suffix_lookup_and_head_fusion():
    from owl_engine_b200.engine.spec import fuse_lookup, suffix_lookup

    assert suffix_lookup([1, 2, 3, 4, 9, 1, 2, 3, 4], 3, 2, 8) == ([9, 1, 2], 4)          # extended to the whole earlier run
    assert suffix_lookup([5, 6, 5, 6, 5, 6], 3, 2, 8) == ([5, 6], 4)                      # overlap allowed; what follows is short
    assert suffix_lookup([7, 1, 2, 8, 1, 2, 9, 1, 2], 2, 2, 8) == ([9, 1], 2)             # equal length: the more recent match
    assert suffix_lookup([1, 2, 3, 4, 9, 1, 2, 3, 4], 3, 2, 3)[1] == 3                    # the extension stops at nmax
    assert suffix_lookup([1, 2, 3], 3, 2, 8) is None and suffix_lookup([1, 2], 3, 2, 8) is None
    assert suffix_lookup([4, 4, 4, 4], 2, 1, 8) == ([4], 3)
    draft = [10, 11, 12, 13]
    assert fuse_lookup(draft, [20, 21], 6, 3, 6, 0) == [20, 21, 12, 13]                   # strong: the head is replaced, the tail kept
    assert fuse_lookup(draft, [20, 21], 4, 3, 6, 1) == draft                              # weak and disagreeing: the model's draft stays
    assert fuse_lookup(draft, [10, 21], 4, 3, 6, 1) == [10, 21, 12, 13]                   # weak but agreeing on the first token
    assert fuse_lookup(draft, [20, 21], 2, 3, 6, 0) == draft                              # shorter than nmin never counts
    assert fuse_lookup(draft, [], 9, 3, 6, 0) == draft


def test_lookup_history_buffer_tracks_the_sequence():
    from types import SimpleNamespace

    from owl_engine_b200.engine.spec import LookupDraft

    seq = SimpleNamespace(tokens=[1, 2, 3, 4, 9, 1, 2, 3, 4])
    eng = SimpleNamespace(seqs={0: seq})
    lk = LookupDraft(2, 8)
    assert lk.propose(eng, 0, 3) == [9, 1, 2]
    seq.tokens += [9, 1]
    assert lk.propose(eng, 0, 2) == [2, 3]                  # the buffer grew in place
    seq.tokens[:] = [3, 3, 7, 3, 3]                         # another history under the same id (a rewritten sequence)
    assert lk.propose(eng, 0, 1) == [7] and lk.hits == 3


def test_any_override_of_any_key_loads_or_is_refused_with_a_config_error():
    """Random values for random keys: the loader answers with a validated profile or a ConfigError that names the key,
    never with another exception; what loads also survives the memory model and the preflight."""
    from hypothesis import given, settings, strategies as st

    from owl_engine_b200.formats.preflight import check_profile
    from owl_engine_b200.utils.memory import estimate

    keys = sorted(f"{sec}.{k}" for sec, ks in C.SCHEMA.items() if sec != "intent" for k in ks)
    value = st.one_of(st.booleans(), st.integers(-3, 10 ** 7), st.floats(-2, 8, allow_nan=False), st.text("abclrfutq0123:._-/ ", max_size=10),
                      st.lists(st.text("0123", max_size=2), max_size=9), st.sampled_from(["tp", "fp8", "tcr", "mtp", "queue:50", "lrfu:0.5"]))

    def lit(v):
        if isinstance(v, bool):
            return "true" if v else "false"
        if isinstance(v, str):
            return '"' + v.replace("\\\\", "").replace('"', "") + '"'
        if isinstance(v, list):
            return "[" + ", ".join(lit(x) for x in v) + "]"
        return repr(v)

    @settings(max_examples=400, deadline=None)
    @given(st.lists(st.tuples(st.sampled_from(keys), value), min_size=1, max_size=4))
    def run(overrides):
        sets = [f"{k}={lit(v)}" for k, v in overrides]
        try:
            cfg = C.load(FULL, sets)
        except C.ConfigError as e:
            assert str(e)
            return
        est = estimate(cfg)
        assert est["kv_pool_bytes"] >= 0 and isinstance(est["fits"], bool)
        assert all(isinstance(i.line(), str) for i in check_profile(cfg))
    run()
