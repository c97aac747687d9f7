"""Cross-session batched decode on the 27B configuration: aggregate tokens/s for 1, 4, 8, 16 and 32 concurrent sequences
(one fused (B, 1) step per token, CUDA-graph replay, host-fed like the serving path).

``python -m owl_engine_b200.fixtures.batch_bench [prompt_len] [prefill_gemm]`` prints one JSON line (``prefill_gemm`` "tcr" keeps
a resident fp16 copy of the weights, which steps of 16+ rows multiply on the dense tcgen05 GEMM). Every sequence has its own random prompt of
``prompt_len`` tokens (default 1024); the timed region is 32 decode steps after 4 warm-up steps, CUDA events around the loop.
"""
import json
import sys

import torch

from owl_engine_b200.engine.core import Engine, EngineConfig

plen = int(sys.argv[1]) if len(sys.argv) > 1 else 1024
arm = sys.argv[2] if len(sys.argv) > 2 else "tc"
NMAX = 32
cfg = EngineConfig(model="qwen3.8-27b", group=128, n_pages=NMAX * (plen + 256) // 16 + 64, n_slots=NMAX, n_snap_rows=1, max_seqs=NMAX,
                   max_seq=plen + 256, lm_head_int8=True, prefill_gemm=arm)
eng = Engine(cfg)
g = torch.Generator().manual_seed(5)
sids = []
for i in range(NMAX):
    sid = eng.add_sequence(torch.randint(0, eng.spec.vocab, (plen,), generator=g).tolist(), reuse=False)
    eng.prefill(sid)
    sids.append(sid)
res = {"prompt_len": plen, "prefill_gemm": arm}
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
