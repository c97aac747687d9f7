"""Fused GEMM + collective kernels of the tensor-parallel prefill on the 27B MLP boundary, against the unfused arm.

One iteration = the work between two MLP halves of a layer on T tokens:

    fused    : down_proj GEMM with reduce-scatter epilogue (peer stores from TMEM)  ->  owner-side sum + residual +
               RMSNorm + all-gather by peer stores  ->  gate_up GEMM gated per row tile on the gathered rows
    unfused  : down_proj GEMM  ->  all-reduce (our one-shot kernel, and NCCL)  ->  residual + RMSNorm  ->  gate_up GEMM

Launch under torchrun with 2, 4 or 8 ranks, e.g.
``python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29531 -m
owl_engine_b200.fixtures.tp_gemm_bench``. Rank 0 prints one JSON line: device time per iteration (CUDA events, max over
ranks), achieved FLOP/s, and the roofline = the slower of FLOPs / measured GEMM rate and bytes over NVLink / 770 GB/s.
"""
import json
import os

import torch
import torch.distributed as dist

from owl_engine_b200.ops import gemm_tc, kernels as K
from owl_engine_b200.parallel.comm import TpComm

T, H, INTER = int(os.environ.get("OWL_T", 2048)), 5120, 17408
GEMM_TFLOPS, LINK_GBS = 1426.0, 770.0        # sustained library bf16 GEMM on this GPU type; peer copy per direction


def timed(fn, comm, it=20):
    for _ in range(3):
        fn()
    comm.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(it):
        fn()
    e1.record(); torch.cuda.synchronize()
    return comm.max_over_ranks(e0.elapsed_time(e1) / it)


def main():
    comm = TpComm.from_env("fused", hidden=H, big_elems=T * H)
    dev, W, rank = comm.device, comm.world, comm.rank
    pipe = comm.symm.prefill
    kd = INTER // W                                        # down_proj K and gate_up N / 2 per rank
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    act = (torch.randn(T, kd, device=dev, generator=g) * 0.3).half()
    w_down = (torch.randn(H, kd, device=dev, generator=g) * 0.02).half()
    w_gu = (torch.randn(2 * kd, H, device=dev, generator=g) * 0.02).half()
    ln = torch.zeros(H, dtype=torch.bfloat16, device=dev)
    gu = torch.empty(T, 2 * kd, dtype=torch.bfloat16, device=dev)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    h = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    x = torch.empty(T, H, dtype=torch.float16, device=dev)

    def fused():
        pipe.gemm_rs(act, w_down, T)
        pipe.reduce_norm_gather(T, ln, out_dtype=torch.float16)
        pipe.gemm_ag(w_gu, gu, T)

    def unfused(nccl):
        gemm_tc.f16_gemm(act, w_down, y)
        if nccl:
            dist.all_reduce(y)
        else:
            comm.symm.allreduce_(y)
        K.rmsnorm_pack(h, ln, delta=y, out_h=h, normed=x, m=T, k=H)
        gemm_tc.f16_gemm(x, w_gu, gu)

    def gemms_only():
        gemm_tc.f16_gemm(act, w_down, y)
        gemm_tc.f16_gemm(x, w_gu, gu)

    res = {"world": W, "T": T, "fused_ms": timed(fused, comm), "unfused_own_ar_ms": timed(lambda: unfused(False), comm),
           "unfused_nccl_ms": timed(lambda: unfused(True), comm), "gemms_only_ms": timed(gemms_only, comm)}
    flops = 2 * T * H * kd + 2 * T * 2 * kd * H
    link_bytes = 2 * (W - 1) / W * T * H * 2               # reduce-scatter out + all-gather out, per rank and direction
    roof_ms = max(flops / (GEMM_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e3
    res.update(flops_per_rank=flops, nvlink_bytes_per_rank=int(link_bytes), roofline_ms=round(roof_ms, 4),
               fused_tflops=round(flops / res["fused_ms"] / 1e9, 1), fused_frac_of_roofline=round(roof_ms / res["fused_ms"], 3),
               status=[comm.symm.status(), gemm_tc.gemm_status()])
    # correctness on the way: the gathered GEMM input equals the unfused arm's normalised rows
    h.zero_(); pipe.h.zero_()
    fused(); unfused(False)
    torch.cuda.synchronize()
    a, b = pipe.x(T, torch.float16).float(), x.float()
    res["max_rel_diff_vs_unfused"] = round(((a - b).norm() / b.norm().clamp_min(1e-6)).item(), 5)
    if rank == 0:
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in res.items()}))
    comm.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
