// Helpers of the GEMM-form prefill attention (long prompts): the two contractions of causal attention run as tcgen05 GEMMs
// (gemm_dense.cu), these kernels do what lies between them.
//
//   owl_kv_gather       paged K / V of one sequence and layer (e4m3, int8 + scales, or fp16 words)
//                         -> K  bf16 [hkv][ctx_pad][hd]   (rows = keys: the B operand of S = Q K^T, k-major)
//                            Vt fp16 [hkv][hd][ctx_pad]   (rows = dims: the B operand of O = P V,   k-major)
//                       ctx_pad is a multiple of 64; the padding columns / rows are written as zeros
//   owl_causal_softmax  S fp16 [rows][ld] -> P fp16 in place: row r sees keys < pos0 + r + 1, softmax(scale * s), zeros elsewhere
//
// Role in the reference: the FlashInfer prefill kernels of crates/kernels/cu/attn (fused form); on this part the tensor cores
// are reached through tcgen05 GEMMs, and below a few thousand keys the fused warp-level kernel of attn.cu stays in use.
#include <cuda_fp8.h>
#include "common.cuh"

namespace owl {

constexpr int AG_PAGE = 16;

template <int FMT>   // 0 e4m3, 1 int8 (+ scale), 2 fp16 words
__device__ __forceinline__ float ag_elem(const uint8_t* row, int d) {
  if (FMT == 2) return __half2float(reinterpret_cast<const __half*>(row)[d]);
  if (FMT == 1) return (float)reinterpret_cast<const int8_t*>(row)[d];
  __nv_fp8_e4m3 v;
  v.__x = row[d];
  return (float)v;
}

// grid (ctx_pad / 16, hkv), block 256 = 16 tokens x 16 lanes of 16 dims (hd = 256). The V tile goes through shared memory so
// that both the pool reads and the transposed stores are contiguous.
template <int FMT>
__global__ void __launch_bounds__(256) kv_gather_kernel(const uint8_t* __restrict__ k_pool, const uint8_t* __restrict__ v_pool,
                                                        const float* __restrict__ k_scale, const float* __restrict__ v_scale,
                                                        const int* __restrict__ bt, int ctx, int ctx_pad, int hkv,
                                                        __nv_bfloat16* __restrict__ kout, __half* __restrict__ vt) {
  constexpr int HD = 256, ESZ = FMT == 2 ? 2 : 1;
  __shared__ __half vs[16][HD + 2];
  const int pg = blockIdx.x, h = blockIdx.y, tok = threadIdx.x >> 4, l16 = threadIdx.x & 15;
  const int key = pg * AG_PAGE + tok;
  const bool live = key < ctx;
  const int page = live ? bt[pg] : 0;
  const size_t slot = (size_t)page * AG_PAGE + tok;
  const uint8_t* kp = k_pool + (slot * hkv + h) * HD * ESZ;
  const uint8_t* vp = v_pool + (slot * hkv + h) * HD * ESZ;
  const float ks = (FMT == 1 && live) ? k_scale[slot * hkv + h] : 1.f;
  const float vsc = (FMT == 1 && live) ? v_scale[slot * hkv + h] : 1.f;
  __nv_bfloat16* ko = kout + ((size_t)h * ctx_pad + key) * HD;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = l16 * 16 + i;
    ko[d] = __float2bfloat16(live ? ag_elem<FMT>(kp, d) * ks : 0.f);
    vs[tok][d] = __float2half_rn(live ? ag_elem<FMT>(vp, d) * vsc : 0.f);
  }
  __syncthreads();
  // transposed store: thread -> (dim, 16 consecutive keys)
  const int d = threadIdx.x;
  __half* vo = vt + ((size_t)h * HD + d) * ctx_pad + (size_t)pg * AG_PAGE;
  __align__(16) __half tmp[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) tmp[i] = vs[i][d];
  reinterpret_cast<uint4*>(vo)[0] = reinterpret_cast<const uint4*>(tmp)[0];
  reinterpret_cast<uint4*>(vo)[1] = reinterpret_cast<const uint4*>(tmp)[1];
}

// one CTA (256 threads) per score row; three passes over the row (max, sum, write)
__global__ void __launch_bounds__(256) causal_softmax_kernel(__half* __restrict__ s, int ld, int ncols, int pos0, float scale_log2,
                                                             int rpt, float* __restrict__ inv_sum) {
  __shared__ float red[32];
  const int r = blockIdx.x;
  __half* row = s + (size_t)r * ld;
  const int limit = min(pos0 + r / rpt + 1, ncols);
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) mx = fmaxf(mx, __half2float(row[c]));
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) sum += exp2f((__half2float(row[c]) - mx) * scale_log2);
  sum = block_sum(sum, red);
  for (int c = threadIdx.x; c < ncols; c += blockDim.x)
    row[c] = __float2half_rn(c < limit ? exp2f((__half2float(row[c]) - mx) * scale_log2) : 0.f);
  if (threadIdx.x == 0) inv_sum[r] = 1.f / sum;
}

// The row staged in shared memory (rows up to ~100 k keys): one vectorised read of the scores, one exponential per element, one
// vectorised write. The probabilities are left UNNORMALISED (largest = 1, which keeps them in the fp16 normal range however many
// keys a row sees); 1 / sum goes to inv_sum[row] and is applied to the output row after O = P V. ld and ncols are multiples of
// 8; dynamic shared memory = ncols halves.
__global__ void __launch_bounds__(512) causal_softmax_smem_kernel(__half* __restrict__ s, int ld, int ncols, int pos0, float scale_log2,
                                                                  int rpt, float* __restrict__ inv_sum) {
  extern __shared__ __align__(16) __half srow[];
  __shared__ float red[32];
  const int r = blockIdx.x;
  __half* row = s + (size_t)r * ld;
  const int limit = min(pos0 + r / rpt + 1, ncols);
  const int nfull = limit >> 3, nv = (limit + 7) >> 3, nv_all = ncols >> 3;   // fully visible chunks / chunks with a visible key / all
  __half2 m2 = __float2half2_rn(-65504.f);
  for (int c = threadIdx.x; c < nv; c += blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(row)[c];
    reinterpret_cast<uint4*>(srow)[c] = u;
    const __half2* h2 = reinterpret_cast<const __half2*>(&u);
    if (c < nfull) {
      m2 = __hmax2(m2, __hmax2(__hmax2(h2[0], h2[1]), __hmax2(h2[2], h2[3])));
    } else {
      const __half* h = reinterpret_cast<const __half*>(&u);
      for (int i = 0; i < limit - c * 8; ++i) m2 = __hmax2(m2, __half2half2(h[i]));
    }
  }
  const float mx = block_max(fmaxf(__low2float(m2), __high2float(m2)), red);
  const float bias = -mx * scale_log2;
  float sum = 0.f;
  for (int c = threadIdx.x; c < nv_all; c += blockDim.x) {
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (c < nv) {
      u = reinterpret_cast<const uint4*>(srow)[c];
      __half2* h2 = reinterpret_cast<__half2*>(&u);
      if (c < nfull) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h2[i]);
          const float e0 = exp2f(fmaf(f.x, scale_log2, bias)), e1 = exp2f(fmaf(f.y, scale_log2, bias));
          sum += e0 + e1;
          h2[i] = __floats2half2_rn(e0, e1);
        }
      } else {
        __half* h = reinterpret_cast<__half*>(&u);
        for (int i = 0; i < 8; ++i) {
          const float e = c * 8 + i < limit ? exp2f(fmaf(__half2float(h[i]), scale_log2, bias)) : 0.f;
          sum += e;
          h[i] = __float2half_rn(e);
        }
      }
    }
    reinterpret_cast<uint4*>(row)[c] = u;
  }
  sum = block_sum(sum, red);
  if (threadIdx.x == 0) inv_sum[r] = 1.f / sum;
}

// y = o * sigmoid(gate): o bf16 [rows][HD], gate from the q projection output ([q_h | gate_h] per head, row stride ldq); y bf16 or
// fp16 [rows][HD]. grid (HD / 8 / 256 rounded up, rows).
__global__ void __launch_bounds__(256) attn_gate_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ qraw,
                                                        int ldq, int D, void* __restrict__ out, int HD, int out_f16, int gq,
                                                        const float* __restrict__ inv_sum) {
  const int row = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= (HD >> 3)) return;
  const int e = c * 8, head = e / D, off = e % D;
  // gq > 0: o is stacked per kv head, [hkv][rows][gq][D] (the grouped GEMM's output); else [rows][HD]
  const __nv_bfloat16* src = gq > 0 ? o + ((((size_t)(head / gq) * gridDim.y + row) * gq + head % gq) * D + off)
                                    : o + (size_t)row * HD + e;
  const uint4 a = *reinterpret_cast<const uint4*>(src);
  // softmax denominator of this (token, head): same stacking as the grouped rows, or [head][rows] for the flat layout
  const float nrm = !inv_sum ? 1.f : gq > 0 ? inv_sum[((size_t)(head / gq) * gridDim.y + row) * gq + head % gq]
                                            : inv_sum[(size_t)head * gridDim.y + row];
  const uint4 g = *reinterpret_cast<const uint4*>(qraw + (size_t)row * ldq + (size_t)head * 2 * D + D + off);
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float y0 = nrm * bf16_lo(aw[i]) / (1.f + __expf(-bf16_lo(gw[i]))), y1 = nrm * bf16_hi(aw[i]) / (1.f + __expf(-bf16_hi(gw[i])));
    r[i] = out_f16 ? pack_f16(y0, y1) : pack_bf16(y0, y1);
  }
  reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + (size_t)row * HD)[c] = make_uint4(r[0], r[1], r[2], r[3]);
}

}  // namespace owl
using namespace owl;

// q bf16 [rows][hq][D] -> qg [hkv][rows][gq][D]: the q heads of one kv head become consecutive rows of one GEMM operand.
__global__ void __launch_bounds__(256) q_group_kernel(const uint4* __restrict__ q, uint4* __restrict__ qg, int hq, int gq, int cpd) {
  const int row = blockIdx.y, rows = gridDim.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= hq * cpd) return;
  const int head = c / cpd, off = c % cpd;
  qg[(((size_t)(head / gq) * rows + row) * gq + head % gq) * cpd + off] = q[(size_t)row * hq * cpd + c];
}

OWL_API int owl_q_group(const void* q, void* qg, int rows, int hq, int hkv, int D, cudaStream_t st) {
  if (rows < 1 || hkv < 1 || hq % hkv || (D & 7) || !q || !qg) return OWL_ERR_BAD_ARG;
  const int cpd = D / 8;
  q_group_kernel<<<dim3((hq * cpd + 255) / 256, rows), 256, 0, st>>>((const uint4*)q, (uint4*)qg, hq, hq / hkv, cpd);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// gq > 0: `o` is the grouped layout [hkv][rows][gq][D]; gq = 0: [rows][HD].
OWL_API int owl_attn_gate(const void* o, const void* qraw, int ldq, int D, void* out, int rows, int HD, int out_f16, int gq,
                          const void* inv_sum, cudaStream_t st) {
  if (rows < 1 || (HD & 7) || (D & 7) || (ldq & 7) || !o || !qraw || !out || gq < 0) return OWL_ERR_BAD_ARG;
  attn_gate_kernel<<<dim3((HD / 8 + 255) / 256, rows), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)qraw, ldq, D, out,
                                                                   HD, out_f16, gq, (const float*)inv_sum);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// bt: the sequence's block-table row (int32 page numbers). fmt: 0 e4m3, 1 int8 with k_scale / v_scale [pages][16][hkv], 2 fp16.
OWL_API int owl_kv_gather(const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale, int fmt, const void* bt,
                          int ctx, int ctx_pad, int hkv, int hd, void* k_out, void* vt_out, cudaStream_t st) {
  if (hd != 256 || ctx < 1 || ctx_pad < ctx || (ctx_pad & 63) || hkv < 1 || fmt < 0 || fmt > 2 || (fmt == 1 && (!k_scale || !v_scale)))
    return OWL_ERR_BAD_ARG;
  const dim3 grid(ctx_pad / AG_PAGE, hkv);
  if (fmt == 0)
    kv_gather_kernel<0><<<grid, 256, 0, st>>>((const uint8_t*)k_pool, (const uint8_t*)v_pool, nullptr, nullptr, (const int*)bt, ctx,
                                              ctx_pad, hkv, (__nv_bfloat16*)k_out, (__half*)vt_out);
  else if (fmt == 1)
    kv_gather_kernel<1><<<grid, 256, 0, st>>>((const uint8_t*)k_pool, (const uint8_t*)v_pool, (const float*)k_scale,
                                              (const float*)v_scale, (const int*)bt, ctx, ctx_pad, hkv, (__nv_bfloat16*)k_out,
                                              (__half*)vt_out);
  else
    kv_gather_kernel<2><<<grid, 256, 0, st>>>((const uint8_t*)k_pool, (const uint8_t*)v_pool, nullptr, nullptr, (const int*)bt, ctx,
                                              ctx_pad, hkv, (__nv_bfloat16*)k_out, (__half*)vt_out);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// s: fp16 [rows][ld]; columns [0, ncols) are rewritten (probabilities, zeros past the causal limit pos0 + r + 1).
// rows_per_tok consecutive rows belong to one query token (the q heads of a kv head stacked per token).
// The probabilities are written unnormalised (row maximum = 1); inv_sum[row] = 1 / (row sum) scales the row of O = P V.
OWL_API int owl_causal_softmax(void* s, int rows, int ld, int ncols, int pos0, float scale, int rows_per_tok, void* inv_sum,
                               cudaStream_t st) {
  if (rows < 1 || ncols < 1 || ld < ncols || pos0 < 0 || rows_per_tok < 1 || !inv_sum) return OWL_ERR_BAD_ARG;
  const size_t smem = (size_t)ncols * 2;
  if (!(ld & 7) && !(ncols & 7) && !(reinterpret_cast<uintptr_t>(s) & 15) && smem <= 200 * 1024) {
    static bool attr_done = false;
    if (!attr_done) {
      if (cudaFuncSetAttribute(causal_softmax_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return OWL_ERR_LAUNCH * 1000;
      attr_done = true;
    }
    causal_softmax_smem_kernel<<<rows, 512, smem, st>>>((__half*)s, ld, ncols, pos0, scale * 1.4426950408889634f, rows_per_tok,
                                                        (float*)inv_sum);
  } else {
    causal_softmax_kernel<<<rows, 256, 0, st>>>((__half*)s, ld, ncols, pos0, scale * 1.4426950408889634f, rows_per_tok, (float*)inv_sum);
  }
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
