"""Timed CPU baseline of the reference-numerics configuration: the tiny Qwen3.5-style hybrid (hidden 1024, 24 layers
[GDN, GDN, GDN, full] x 6, vocab 151936) in fp32 on the host, weights N(0, 0.02) from seed 0, one sequence with a 128-token
prefill of uniform random ids followed by 64 greedy decode steps.

``python -m owl_engine_b200.fixtures.cpu_baseline [--gpu]`` prints one JSON line; ``--gpu`` also runs the same model and
prompt through the GPU engine (W4A16 weights quantised from the same dense tensors) and reports its time and how many of the
64 tokens agree with the fp32 run until the first difference."""
import json
import sys
import time

import torch

from owl_engine_b200.models.reference import RefModel, init_weights
from owl_engine_b200.models.spec import tiny_hybrid


def main():
    spec = tiny_hybrid()
    torch.manual_seed(0)
    t0 = time.perf_counter()
    w = init_weights(spec, seed=0, std=0.02)
    t_init = time.perf_counter() - t0
    ref = RefModel(spec, w)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, spec.vocab, (128,), generator=g)
    st = ref.new_state()
    t0 = time.perf_counter()
    h = ref.forward(prompt, st)
    tok = int(ref.logits(h[-1:]).argmax(-1))
    t_prefill = time.perf_counter() - t0
    out = [tok]
    t0 = time.perf_counter()
    for _ in range(63):
        h = ref.forward(torch.tensor([tok]), st)
        tok = int(ref.logits(h).argmax(-1))
        out.append(tok)
    t_decode = time.perf_counter() - t0
    res = {"model": spec.name, "dtype": "fp32", "device": "cpu", "threads": torch.get_num_threads(), "init_s": round(t_init, 2),
           "prefill_128_s": round(t_prefill, 3), "decode_63_steps_s": round(t_decode, 3),
           "decode_tok_s": round(63 / t_decode, 2), "tokens": out[:8]}
    if "--gpu" in sys.argv and torch.cuda.is_available():
        from owl_engine_b200.engine.core import Engine, EngineConfig
        from owl_engine_b200.models import hybrid as H

        dev = torch.device("cuda:0")
        hw, _ = H.weights_from_dense(spec, w, dev, group=128)
        eng = Engine(EngineConfig(model="tiny-hybrid", n_pages=64, n_slots=2, max_seqs=2, max_seq=512, prefill_chunk=128), spec=spec,
                     weights=hw)
        eng.generate(prompt.tolist(), 8)                       # warm-up: graphs, scratch
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        got = eng.generate(prompt.tolist()[::-1], 64)          # a different prompt of the same length: nothing cached
        torch.cuda.synchronize()
        t_gpu = time.perf_counter() - t0
        same = eng.generate(prompt.tolist(), 64)
        agree = next((i for i, (a, b) in enumerate(zip(same, out)) if a != b), 64)
        res["gpu"] = {"weights": "W4A16 g128 of the same tensors", "prefill_plus_64_tokens_s": round(t_gpu, 4),
                      "tokens_equal_to_fp32_until": agree, "speedup_vs_cpu": round((t_prefill + t_decode) / t_gpu, 1)}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
