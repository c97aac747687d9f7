"""Weight-streaming microbenchmark: the tcgen05 streaming kernel against the legacy integer arms on the 27B layer
shapes, timed as CUDA-graph replays over rotating weight copies (inputs larger than L2).
``python -m owl_engine_b200.fixtures.gemv_bench``
"""
import torch

from owl_engine_b200.ops import kernels as K, quant as Q
dev = 'cuda'
def bench(n, k, m, group=128, reps=24, ncopies=4, old=True):
    xp = torch.randint(0, 127, (m, 2*k), dtype=torch.uint8, device=dev)
    xs = torch.rand(m, k//group, 2, device=dev)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    ws = K.StreamTcWorkspace(dev)
    xt = torch.randint(0, 127, (K.act_tile_bytes(k, group),), dtype=torch.uint8, device=dev)
    res = {}
    arms = [("tc", lambda w: K.w4a16_stream_tc(w, xt, out, m, ws, pdl=True))]
    if old: arms.append(("old", lambda w: K.w4a16_skinny(w, xp, xs, out, m, pdl=True)))
    for name, f in arms:
        lay = 'block' if name == 'tc' else 'slice'
        ws_ = [Q.random_skinny(n, k, group, dev, seed=i, layout=lay) for i in range(ncopies)]
        for i in range(3): f(ws_[i % ncopies])
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(reps): f(ws_[i % ncopies])
        g.replay(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); g.replay(); g.replay(); e1.record(); torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / (2 * reps) * 1e3
        res[name] = (us, ws_[0].records.numel() / us / 1e6)
    print(f"N={n} K={k} M={m} g{group}: " + "  ".join(f"{a} {u:.1f}us {t:.2f}TB/s" for a, (u, t) in res.items()), flush=True)
shapes = [(34816, 5120), (16384, 5120), (14336, 5120), (5120, 6144), (5120, 17408)]
for (n, k) in shapes:
    for m in (1, 8):
        bench(n, k, m)
bench(34816, 5120, 1, group=32)
print("status", K.stream_tc_status(), K.skinny_status())
