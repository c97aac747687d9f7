"""Cross-session batched decode on the 27B configuration: aggregate tokens/s for 1, 4, 8, 16 and 32 concurrent sequences
(one fused (B, 1) step per token, CUDA-graph replay, host-fed like the serving path).

``python -m owl_engine_b200.fixtures.batch_bench [prompt_len]`` prints one JSON line. Every sequence has its own random prompt of
``prompt_len`` tokens (default 1024); the timed region is 32 decode steps after 4 warm-up steps, CUDA events around the loop.
"""
import json
import sys

import torch

from owl_engine_b200.engine.core import Engine, EngineConfig

plen = int(sys.argv[1]) if len(sys.argv) > 1 else 1024
NMAX = 32
cfg = EngineConfig(model="qwen3.8-27b", group=128, n_pages=NMAX * (plen + 128) // 16 + 64, n_slots=NMAX, n_snap_rows=1, max_seqs=NMAX,
                   max_seq=plen + 128, lm_head_int8=True)
eng = Engine(cfg)
g = torch.Generator().manual_seed(5)
sids = []
for i in range(NMAX):
    sid = eng.add_sequence(torch.randint(0, eng.spec.vocab, (plen,), generator=g).tolist(), reuse=False)
    eng.prefill(sid)
    sids.append(sid)
res = {"prompt_len": plen}
for b in (1, 4, 8, 16, 32):
    use = sids[:b]
    for _ in range(4):
        eng.decode_step(use)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(32):
        eng.decode_step(use)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 32
    res[f"b{b}"] = {"ms_per_step": round(ms, 3), "tok_s": round(b * 1e3 / ms, 1)}
print(json.dumps(res))
