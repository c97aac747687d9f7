"""A short decode run of the 27B shape for launch lists: ``python -m owl_engine_b200.fixtures.decode_step_case
[--layers 8] [--steps 3] [--prompt 256] [--graph 0|1] [--gemv fma|dp4a]``.

Builds the engine on random weights (a slice of ``--layers`` layers keeps the device footprint at a few GB), prefills a
short prompt and runs ``--steps`` decode steps, eagerly by default so that a profiler sees one launch per kernel in
program order. Prints the mean step time measured with CUDA events (meaningful only without a profiler attached)."""
import argparse

import torch

from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.models import hybrid as H


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--prompt", type=int, default=256)
    ap.add_argument("--graph", type=int, default=0)
    ap.add_argument("--gemv", default="fma")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    eng = Engine(EngineConfig(model="qwen3.8-27b", n_pages=256, n_slots=2, max_seqs=2, max_seq=2048, n_layers=a.layers,
                              decode_gemv=a.gemv, lm_head_int8=True, prefill_gemm="tc"))
    g = torch.Generator().manual_seed(0)
    sid = eng.add_sequence(torch.randint(0, eng.spec.vocab, (a.prompt,), generator=g).tolist())
    eng.prefill(sid)
    if a.graph:
        for _ in range(2):
            eng.decode_step([sid])
    torch.cuda.synchronize()
    lay = H.StepLayout(1, 1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        if a.graph:
            eng.decode_step([sid])
        else:
            eng.runner.step_forward(lay, ctx_hint=2048, advance=False)
    e1.record()
    torch.cuda.synchronize()
    print(f"decode_step_case: {a.layers} layers, {e0.elapsed_time(e1) / a.steps * 1e3:.1f} us per step "
          f"({'graph' if a.graph else 'eager'}), status {eng._check_status(force=True) or 'clean'}")


if __name__ == "__main__":
    main()
