"""Tensor-parallel serving, host side (no GPU): the shared-memory descriptor ring between processes, the leader's
mirroring wrapper against a follower loop on a recording engine, and the ``[parallel]`` refusals of the server."""
import multiprocessing as mp
import os

import pytest
import torch

from owl_engine_b200.engine import tp_serve as T
from owl_engine_b200.parallel.ring import RingClosed, RingTimeout, StepRing


def _reader(name, reader, n, q):
    ring = StepRing.open(name, reader, 20.0)
    got = []
    try:
        while True:
            op, args, kw = ring.pop(20.0)
            if op == "shutdown":
                break
            got.append((op, args[0], int(kw["t"].sum()) if "t" in kw else None))
    except RingClosed:
        got.append("closed")
    q.put((reader, got))
    ring.free()


def test_ring_broadcasts_in_order_to_every_reader_process():
    name = f"/owl_test_ring_{os.getpid()}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ring = StepRing.create(name, 3, capacity=4096)          # small ring: the producer must wait for the readers
    procs = [ctx.Process(target=_reader, args=(name, r, 200, q)) for r in range(3)]
    for p in procs:
        p.start()
    for i in range(200):
        ring.push("decode_step", [i, i + 1], t=torch.full((3,), i, dtype=torch.int32))
    ring.push("shutdown")
    out = dict(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(30)
    ring.free()
    want = [("decode_step", [i, i + 1], 3 * i) for i in range(200)]
    assert out[0] == want and out[1] == want and out[2] == want


def test_ring_wraps_grows_reader_buffer_and_times_out():
    name = f"/owl_test_ring2_{os.getpid()}"
    ring = StepRing.create(name, 1, capacity=1 << 20)
    rd = StepRing.open(name, 0, 5.0)
    big = bytes(range(256)) * 700                             # larger than the reader's first buffer
    for _ in range(12):                                       # 12 x 179 KB wraps the 1 MB ring
        ring.push_bytes(big)
        assert rd.pop_bytes(1.0) == big
    with pytest.raises(RingTimeout):
        rd.pop_bytes(0.05)
    with pytest.raises(ValueError):
        ring.push_bytes(bytes(2 << 20))                       # can never fit
    # a reader that stops consuming stalls the producer, which reports it instead of overwriting
    for _ in range(5):
        ring.push_bytes(big)
    with pytest.raises(RingTimeout):
        ring.push_bytes(big, timeout_s=0.05)
    ring.close()
    for _ in range(5):
        assert rd.pop_bytes(1.0) == big                       # queued messages drain after close
    with pytest.raises(RingClosed):
        rd.pop_bytes(1.0)
    rd.free()
    ring.free()


class _Rec:
    """An engine stand-in that records its calls; results are a function of the call sequence only."""

    def __init__(self):
        self.calls, self.seqs, self.comm = [], {}, None

    def prefill_plan(self, sid):
        return [(0, 4), (4, 7)]

    def __getattr__(self, name):
        if name.startswith("_") or name not in T.MIRRORED:
            raise AttributeError(name)

        def f(*a, **kw):
            self.calls.append((name, a, tuple(sorted(kw.items()))))
            if name == "add_sequence":
                return len(self.calls)
            if name == "decode_step":
                return [7] * len(a[0])
            return 5
        return f


class _Spec:
    def __init__(self):
        self.calls = []

    def after_prefill(self, e, sid):
        self.calls.append(("after_prefill", sid))

    def round(self, e, sid):
        self.calls.append(("round", sid))
        return e.decode_step([sid])


def test_leader_mirrors_every_call_to_the_follower():
    name = f"/owl_test_ring3_{os.getpid()}"
    ring = StepRing.create(name, 1)
    rd = StepRing.open(name, 0, 5.0)
    lead, foll = _Rec(), _Rec()
    ls, fs = _Spec(), _Spec()
    me = T.MirroredEngine(lead, ring)
    ms = T.MirroredSpec(ls, ring)
    out = me.generate([1, 2, 3], 3)
    assert out == [5, 7, 7]
    sid = me.add_sequence([4, 5], images=[(torch.ones(2, 4, dtype=torch.bfloat16), (1, 1, 2), 99)], image_pad_id=3)
    ms.after_prefill(me, sid)
    assert ms.round(me, sid) == [7]
    me.set_last_token(sid, 11)
    me.shutdown()
    n = T.follower_loop(foll, rd, fs)
    assert n == len(lead.calls) + 2 - 1          # every leader call, plus the two spec calls, minus the nested decode_step
    strip = lambda calls: [(c[0], str(c[1]), str(c[2])) for c in calls]
    assert strip(foll.calls) == strip(lead.calls)
    assert fs.calls == ls.calls == [("after_prefill", sid), ("round", sid)]
    rd.free()
    ring.free()


def test_parallel_section_is_honoured_or_refused():
    from owl_engine_b200.server.main import parallel_plan
    from owl_engine_b200.utils import config as C

    root = os.path.join(os.path.dirname(__file__), "..", "configs")
    one = C.load(os.path.join(root, "qwen38_27b-b200.toml"), [], None)
    assert parallel_plan(one, {})["world"] == 1
    with pytest.raises(C.ConfigError):
        parallel_plan(one, {"WORLD_SIZE": "2", "RANK": "0"})              # single profile under a 2-rank launcher
    tp8 = C.load(os.path.join(root, "qwen38_27b-b200_tp8.toml"), [], None)
    with pytest.raises(C.ConfigError):
        parallel_plan(tp8, {})                                            # tp profile started as one process
    with pytest.raises(C.ConfigError):
        parallel_plan(tp8, {"WORLD_SIZE": "4", "RANK": "1"})              # 8 devices named, 4 ranks started
    p = parallel_plan(tp8, {"WORLD_SIZE": "8", "RANK": "3", "LOCAL_RANK": "3"})
    assert p["world"] == 8 and p["rank"] == 3 and p["comm_mode"] == "fused" and p["vocab_split"] and p["fused_gemm"]
    f8 = C.load(os.path.join(root, "qwen38_27b-b200_tp8.toml"), ["parallel.tp_ar_f8=true"], None)
    with pytest.raises(C.ConfigError):
        parallel_plan(f8, {"WORLD_SIZE": "8", "RANK": "0"})
    mm = C.load(os.path.join(root, "qwen38_27b-b200_tp8.toml"), ["parallel.tp_ar=multimem"], None)
    assert parallel_plan(mm, {"WORLD_SIZE": "8", "RANK": "0"})["multimem"]
    nc = C.load(os.path.join(root, "qwen38_27b-b200_tp8.toml"), ["parallel.tp_comm=nccl"], None)
    assert parallel_plan(nc, {"WORLD_SIZE": "8", "RANK": "0"})["comm_mode"] == "nccl"
