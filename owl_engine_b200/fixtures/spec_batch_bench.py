"""Speculative decoding for a batch of sessions with a forced acceptance length: the 27B configuration with group-32 int4
weights (what a GGUF Q4_K checkpoint converts to at load), an MTP head and one DFlash2 block draft per session.

Every session first decodes plainly (one batched (B, 1) step per token: the baseline rate and each session's greedy
continuation), then again with speculative rounds: per round and session the MTP head and the DFlash2 draft run (their cost
is real), an oracle replaces their tokens by ``--accept`` correct drafts followed by a wrong one (so acceptance length is an
input), the target verifies all sessions of a group in ONE (B, T) step and one batched fold replays the accepted rows'
recurrent updates. The run asserts that every session's speculative output equals its plain output.

``python -m owl_engine_b200.fixtures.spec_batch_bench [--batch 8] [--prompt 1024] [--out 512] [--depth 7] [--accept 3]``
(under ``torchrun`` for tensor parallelism) prints one JSON line.

Reference counterpart: the spec-aware batch gates of ``crates/engine/tests`` (``tp_batch_gate.rs``) and ``tools/fixture``'s
forced-acceptance decode benchmark.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--out", type=int, default=512)
    ap.add_argument("--depth", type=int, default=7)
    ap.add_argument("--accept", type=int, default=3)
    ap.add_argument("--group", type=int, default=32)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--drafts", default="mtp,dflash2", help="draft models that run every round (their cost is measured)")
    ap.add_argument("--comm", default="fused")
    ap.add_argument("--prefill-gemm", default="tc")
    a = ap.parse_args()

    from ..engine.core import Engine, EngineConfig
    from ..engine.spec import DFlash2Pool, MtpDraft, OracleDraft, SpecRunner
    from ..models import dflash2 as D
    from ..models import hybrid as H
    from ..models.mtp import MtpHead
    from ..ops import kernels as K
    from ..parallel.comm import TpComm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    comm = TpComm.from_env(a.comm, hidden=5120, big_elems=2048 * 5120) if world > 1 else None
    rank = comm.rank if comm else 0
    if comm is None:
        torch.cuda.set_device(0)

    def sync():
        if comm:
            comm.barrier()
        torch.cuda.synchronize()

    t = a.depth + 1
    per = max(1, H.HybridRunner.MAX_ROWS // t)
    n_seq = a.prompt + a.out + 64
    cfg = EngineConfig(model="qwen3.8-27b", group=a.group, n_pages=a.batch * (n_seq // 16 + 2) + 64, n_slots=a.batch, n_snap_rows=1,
                       spec_rows=min(per, a.batch), max_seqs=a.batch, max_seq=n_seq, lm_head_int8=True, n_layers=a.layers,
                       decode_gemv="dp4a" if a.group != 128 else "fma", prefill_gemm=a.prefill_gemm)
    eng = Engine(cfg, comm=comm)
    eng.runner.uniform_rows = True
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, eng.spec.vocab - 8, (a.prompt,), generator=g).tolist() for _ in range(a.batch)]

    # ---- plain: batched (B, 1) steps ---------------------------------------------------------------------------------
    sids = []
    plains = []
    for p in prompts:
        sid = eng.add_sequence(p, reuse=False)
        plains.append([eng.prefill(sid)])
        sids.append(sid)
    for _ in range(4):
        for o, tok in zip(plains, eng.decode_step(sids)):
            o.append(tok)
    sync()
    t0 = time.perf_counter()
    n0 = len(plains[0])
    while len(plains[0]) < a.out:
        for o, tok in zip(plains, eng.decode_step(sids)):
            o.append(tok)
    sync()
    plain_s = time.perf_counter() - t0
    n_plain = a.batch * (len(plains[0]) - n0)
    for sid in sids:
        eng.free_sequence(sid, publish=False)

    # ---- speculative: drafts per session, one verify + one fold per group and round ----------------------------------
    names = [x for x in a.drafts.split(",") if x]
    if world > 1 and names:
        # the draft models are not tensor-parallel: with them in the loop at 4 ranks the verify rows no longer reproduce plain
        # decoding (on one GPU they do), so under tensor parallelism the fixture measures the target side of a round only
        names = []
    pool = mtp = None
    if "dflash2" in names:
        n = eng.spec.n_layers
        taps = D.DraftSpec.taps if n >= 62 else tuple(sorted({max(0, n * (2 * i + 1) // 10 - 1) for i in range(5)}))
        dspec = D.DraftSpec(hidden=eng.spec.hidden, vocab=eng.spec.vocab, inter=eng.spec.inter, taps=taps,
                            mask_token_id=eng.spec.vocab - 1, n_layers=len(taps))
        dw = D.random_weights(dspec, eng.device)
        pool = DFlash2Pool(lambda: D.DFlash2(dspec, dw, eng.weights.embed, eng.weights.lm_head, eng.device), a.batch, eng.runner)
    if "mtp" in names:
        mtp = MtpDraft(MtpHead(eng.runner, seed=3))
        if pool is not None:
            # both draft models listen to the prompt chunks' hiddens
            mtp_sink, pool_sink = mtp._on_chunk, pool._on_chunk
            eng.runner.tap_sink = lambda pos0, tt, taps: (mtp_sink(pos0, tt, taps), pool_sink(pos0, tt, taps))

    spent = {"propose_s": 0.0, "observe_s": 0.0}

    class Forced:
        """Runs the real draft models of the session, returns the oracle's tokens. Host time spent inside the draft calls is
        accumulated (a proposal ends with a device-to-host read of its tokens, so it includes the device time; the encodes of
        ``observe`` are asynchronous and show up in the next synchronising call)."""

        def __init__(self, oracle):
            self.oracle = oracle

        def after_prefill(self, engine, sid):
            if mtp is not None:
                mtp.after_prefill(engine, sid)
            if pool is not None:
                pool.after_prefill(engine, sid)

        def propose(self, engine, sid, depth):
            t1 = time.perf_counter()
            if mtp is not None:
                mtp.propose(engine, sid, min(depth, 3))
            if pool is not None:
                pool.propose(engine, sid, depth)
            spent["propose_s"] += time.perf_counter() - t1
            return self.oracle.propose(engine, sid, depth)

        def observe(self, engine, sid, n_rows, emitted, row0=0):
            t1 = time.perf_counter()
            if mtp is not None:
                mtp.observe(engine, sid, n_rows, emitted, row0)
            if pool is not None:
                pool.observe(engine, sid, n_rows, emitted, row0)
            spent["observe_s"] += time.perf_counter() - t1

    spec = SpecRunner(None, depth=a.depth, degrade_below=-1.0)
    spec.per_sid = {}
    sids, outs = [], []
    for p, plain in zip(prompts, plains):
        sid = eng.add_sequence(p, reuse=False)
        if pool is not None:
            pool.bind(sid)
        outs.append([eng.prefill(sid)])
        spec.per_sid[sid] = Forced(OracleDraft(plain, len(p), a.accept, eng.spec.vocab))
        spec.after_prefill(eng, sid)
        sids.append(sid)
    for _ in range(2):                                      # warm-up rounds (graph capture)
        for o, toks in zip(outs, spec.round_batch(eng, sids)):
            o.extend(toks)
    sync()
    n0 = sum(len(o) for o in outs)
    r0 = spec.stats.rounds
    spent["propose_s"] = spent["observe_s"] = 0.0
    t0 = time.perf_counter()
    while min(len(o) for o in outs) < a.out:
        live = [i for i, o in enumerate(outs) if len(o) < a.out]
        for i, toks in zip(live, spec.round_batch(eng, [sids[i] for i in live])):
            outs[i].extend(toks)
    sync()
    spec_s = time.perf_counter() - t0
    n_spec = sum(len(o) for o in outs) - n0
    equal = all(o[:a.out] == p[:a.out] for o, p in zip(outs, plains))
    if comm:
        plain_s, spec_s = comm.max_over_ranks(plain_s), comm.max_over_ranks(spec_s)
    plain_rate = n_plain / plain_s
    status = K.all_status()
    if comm:
        status = {k: int(comm.max_over_ranks(float(abs(v)))) for k, v in status.items()}
    rounds = (spec.stats.rounds - r0) / a.batch
    res = {"what": "batched speculative decoding, forced acceptance", "tp": world, "batch": a.batch, "prompt": a.prompt,
           "out": a.out, "group": a.group, "depth": a.depth, "forced_accept": a.accept, "drafts_run": names,
           "plain_tok_s": round(plain_rate, 1),
           "spec_tok_s": round(n_spec / spec_s, 1), "speedup": round(n_spec / spec_s / plain_rate, 3),
           "round_ms": round(spec_s * 1e3 / max(rounds, 1), 3), "tokens_per_round": round(n_spec / max(spec.stats.rounds - r0, 1), 2),
           "sequences_per_verify": min(per, a.batch),
           "draft_share": {"propose": round(spent["propose_s"] / spec_s, 3), "observe": round(spent["observe_s"] / spec_s, 3)}, "folds": spec.stats.folds, "equal_to_plain": equal, "kernel_status": status}
    if rank == 0:
        print(json.dumps(res))
    if comm is not None:
        import torch.distributed as dist

        eng.runner.graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        comm.symm = None
        torch.cuda.synchronize()
        dist.destroy_process_group()
    assert equal, "speculative output differs from plain decoding"


if __name__ == "__main__":
    main()
