"""Prefill GEMM arms on the 27B layer shapes: the fused W4A16 tcgen05 GEMM, dequantise-once + the dense tcgen05 GEMMs
(persistent 128 x 256 and 128 x 128 tiles) and the library GEMM as yardstick. CUDA-event time per call.
``python -m owl_engine_b200.fixtures.gemm_bench``
"""
import torch

from owl_engine_b200.ops import kernels as K, quant as Q, gemm_tc
dev='cuda'
def t(fn, it=10):
    for _ in range(3): fn()
    torch.cuda.synchronize()
    e0,e1=torch.cuda.Event(enable_timing=True),torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(it): fn()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1)/it
for (n,k) in [(34816,5120),(5120,17408),(16384,5120),(5120,6144)]:
    w=Q.random_skinny(n,k,128,dev)
    for T in (256, 2048):
        x16=torch.randn(T,k,device=dev,dtype=torch.float16); xb=x16.to(torch.bfloat16)
        out=torch.empty(T,n,device=dev,dtype=torch.bfloat16)
        dense=torch.empty(n,k,device=dev,dtype=torch.bfloat16)
        fl=2*T*n*k
        a=t(lambda: gemm_tc.w4a16_gemm(w,x16,out))
        b=t(lambda: K.w4_dequant(w,dense))
        c=t(lambda: gemm_tc.f16_gemm(xb,dense,out))
        c0=t(lambda: gemm_tc.f16_gemm(xb,dense,out,force_small=True))
        d=t(lambda: torch.matmul(xb,dense.t(),out=out))
        # W4A8 arm: rows re-quantised to e4m3, product on kind::f8f6f4
        wq,sw=gemm_tc.quant_e4m3_rows(dense); xq,sx=gemm_tc.quant_e4m3_rows(xb)
        e=t(lambda: gemm_tc.e4m3_gemm(xq,sx,wq,sw,out))
        qw=t(lambda: gemm_tc.quant_e4m3_rows(dense,wq,sw)); qx=t(lambda: gemm_tc.quant_e4m3_rows(xb,xq,sx))
        print(f"N={n} K={k} T={T}: w4 fused {a:.3f} ms ({fl/a/1e9:.0f} TF)  dequant {b:.3f} ms  dense persist {c:.3f} ms ({fl/c/1e9:.0f} TF) small-tile {c0:.3f} ms  cublas {d:.3f} ms ({fl/d/1e9:.0f} TF)  e4m3 {e:.3f} ms ({fl/e/1e9:.0f} TF; quant w {qw:.3f} x {qx:.3f} ms)", flush=True)
print(gemm_tc.gemm_status())
