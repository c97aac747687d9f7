"""Speculative-decoding throughput on the 27B configuration with a forced acceptance length.

The oracle draft replays the model's own greedy continuation, correct for ``accept`` drafts per round and wrong after,
so acceptance length is an input; every run asserts that the speculative output equals plain decoding.
``python -m owl_engine_b200.fixtures.spec_bench [n_layers]`` prints one JSON line (wall-clock tokens/s through the
host-fed engine API, prefix cache warm so that prefill is excluded).
"""
import json
import sys
import time

import torch

from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.engine.spec import OracleDraft, MtpDraft, SpecRunner, generate_spec
from owl_engine_b200.models.mtp import MtpHead
layers = int(sys.argv[1]) if len(sys.argv) > 1 else None
cfg = EngineConfig(model="qwen3.8-27b", group=128, n_pages=512, n_slots=2, max_seqs=2, max_seq=4096, n_layers=layers)
eng = Engine(cfg)
eng.runner.uniform_rows = True
g = torch.Generator().manual_seed(1)
prompt = torch.randint(0, eng.spec.vocab, (2048,), generator=g).tolist()
N = 96
t0 = time.perf_counter(); plain = eng.generate(prompt, N); torch.cuda.synchronize(); t_plain = time.perf_counter() - t0
# time plain decode only (exclude prefill): second run reuses the prefix
t0 = time.perf_counter(); plain2 = eng.generate(prompt, N); torch.cuda.synchronize(); t_plain = time.perf_counter() - t0
assert plain2 == plain
res = {"plain_tok_s": round(N / t_plain, 1)}
for depth, acc in [(3, 3), (3, 2), (3, 1), (7, 7), (7, 4)]:
    spec = SpecRunner(OracleDraft(plain, len(prompt), acc, eng.spec.vocab), depth=depth, degrade_below=-1.0)
    generate_spec(eng, prompt, N, spec)   # warm graphs
    spec = SpecRunner(OracleDraft(plain, len(prompt), acc, eng.spec.vocab), depth=depth, degrade_below=-1.0)
    t0 = time.perf_counter(); got = generate_spec(eng, prompt, N, spec); torch.cuda.synchronize(); dt = time.perf_counter() - t0
    assert got == plain, (depth, acc)
    res[f"d{depth}_a{acc}"] = {"tok_s": round(N / dt, 1), "mean_accept": round(spec.stats.mean_accept, 2), "rounds": spec.stats.rounds, "folds": spec.stats.folds}
head = MtpHead(eng.runner, seed=3)
spec = SpecRunner(MtpDraft(head), depth=3, degrade_below=-1.0)
generate_spec(eng, prompt, N, spec)
spec = SpecRunner(MtpDraft(head), depth=3, degrade_below=-1.0)
t0 = time.perf_counter(); got = generate_spec(eng, prompt, N, spec); torch.cuda.synchronize(); dt = time.perf_counter() - t0
res["mtp_random_head_d3"] = {"tok_s": round(N / dt, 1), "mean_accept": round(spec.stats.mean_accept, 2), "equal": got == plain}
print(json.dumps(res))

# DFlash2 block draft of the 27B family's size (random-init): what a round costs with the real draft in the loop. The draft
# runs (encode of every accepted row + one captured proposal per round) while the oracle supplies the tokens, so the
# acceptance length stays an input.
from owl_engine_b200.engine.spec import DFlash2Draft
from owl_engine_b200.models import dflash2 as D


class _ForcedDFlash(DFlash2Draft):
    def __init__(self, draft, runner, oracle):
        super().__init__(draft, runner)
        self.oracle = oracle

    def propose(self, engine, sid, depth):
        super().propose(engine, sid, depth)
        return self.oracle.propose(engine, sid, depth)


n = eng.spec.n_layers
taps = D.DraftSpec.taps if n >= 62 else tuple(sorted({max(0, n * (2 * i + 1) // 10 - 1) for i in range(5)}))
dspec = D.DraftSpec(hidden=eng.spec.hidden, vocab=eng.spec.vocab, inter=eng.spec.inter, taps=taps, mask_token_id=eng.spec.vocab - 1,
                    n_layers=len(taps))
dw = D.random_weights(dspec, eng.device)
draft = D.DFlash2(dspec, dw, eng.weights.embed, eng.weights.lm_head, eng.device)
ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
adapter = _ForcedDFlash(draft, eng.runner, None)      # built once: attaching the taps drops the runner's captured graphs
for depth, acc in [(7, 7), (7, 4), (7, 3)]:
    for rep in range(2):
        adapter.oracle = OracleDraft(plain, len(prompt), acc, eng.spec.vocab)
        spec = SpecRunner(adapter, depth=depth, degrade_below=-1.0)
        t0 = time.perf_counter(); got = generate_spec(eng, prompt, N, spec); torch.cuda.synchronize(); dt = time.perf_counter() - t0
    res[f"dflash2_d{depth}_a{acc}"] = {"tok_s": round(N / dt, 1), "rounds": spec.stats.rounds, "equal": got == plain}
ev[0].record()
for _ in range(20):
    draft.graph.replay()
ev[1].record(); torch.cuda.synchronize()
res["dflash2_propose_ms"] = round(ev[0].elapsed_time(ev[1]) / 20, 3)
res["dflash2_bytes_gb"] = round(dw.nbytes() / 1e9, 2)
print(json.dumps(res))
