// KV-cache selection index on the GPU (long contexts attend to a bounded view of their blocks):
//
//   owl_mean_k_block : per (block, kv head) the mean of the block's keys with the rotary embedding undone, read straight
//                      from the paged e4m3 pool -> float [blocks][hkv][hd]
//   owl_kvscore      : score of every indexed block against the current queries (rotary undone on the fly):
//                      max over queries and q heads of the cosine between query and block mean
//   owl_kvscore_softmax : softmax over the block scores (coverage bookkeeping reads probabilities)
//
// Positions are the text positions of the keys (all three m-RoPE streams equal); blocks holding image patches are
// scored with the same formula. Reference counterpart: crates/kernels/cu/elems/mean_k.cu:27-76,
// cu/elems/page_softmax.cu:44-159, crates/store/src/select.rs (score_blocks).
#include "common.cuh"

namespace owl {

constexpr int KVM_PAGE = 16;

__device__ __forceinline__ float e4m3_to_f(uint8_t v) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(v, __NV_E4M3)));
}

// pool element d of a token row: FMT 0 e4m3, 1 int8 (scaled by the token's scale afterwards), 2 fp16 words
template <int FMT>
__device__ __forceinline__ float kv_elem(const uint8_t* row, int d) {
  if (FMT == 2) return __half2float(reinterpret_cast<const __half*>(row)[d]);
  if (FMT == 1) return (float)reinterpret_cast<const int8_t*>(row)[d];
  return e4m3_to_f(row[d]);
}

// grid (blocks, hkv), hd threads.
template <int FMT>
__global__ void mean_k_block_kernel(const uint8_t* __restrict__ k_pool, const float* __restrict__ k_scale,
                                    const int* __restrict__ pages, const int* __restrict__ pos0,
                                    const int* __restrict__ n_valid, const float* __restrict__ inv_freq, int rotary_dim, int hkv,
                                    int hd, float* __restrict__ out) {
  constexpr int ESZ = FMT == 2 ? 2 : 1;
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x, half = rotary_dim / 2;
  const int n = min(max(n_valid[b], 1), KVM_PAGE);
  const uint8_t* base = k_pool + (((size_t)pages[b] * KVM_PAGE) * hkv + h) * hd * ESZ;
  float acc = 0.f;
  for (int i = 0; i < n; ++i) {
    const uint8_t* kp = base + (size_t)i * hkv * hd * ESZ;
    const float sc = FMT == 1 ? k_scale[((size_t)pages[b] * KVM_PAGE + i) * hkv + h] : 1.f;
    float v = kv_elem<FMT>(kp, d) * sc;
    if (d < rotary_dim) {
      const int j = d < half ? d : d - half;
      float sn, cs;
      sincosf((float)(pos0[b] + i) * inv_freq[j], &sn, &cs);
      const float o = kv_elem<FMT>(kp, d < half ? d + half : d - half) * sc;
      v = d < half ? v * cs + o * sn : v * cs - o * sn;       // inverse rotation
    }
    acc += v;
  }
  out[((size_t)b * hkv + h) * hd + d] = acc / (float)n;
}

// grid (blocks), 256 threads; warp per (query, q head) pair. q: bf16 [nq][hq][hd] AFTER rotary; qpos[nq].
__global__ void __launch_bounds__(256) kvscore_kernel(const __nv_bfloat16* __restrict__ q, const int* __restrict__ qpos,
                                                      const float* __restrict__ index, const float* __restrict__ inv_freq,
                                                      int rotary_dim, int nq, int hq, int hkv, int hd, float* __restrict__ out) {
  __shared__ float red[8];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, half = rotary_dim / 2, rep = hq / hkv;
  float best = -INFINITY;
  for (int pair = warp; pair < nq * hq; pair += 8) {
    const int qi = pair / hq, h = pair % hq;
    const __nv_bfloat16* qv = q + ((size_t)qi * hq + h) * hd;
    const float* kb = index + ((size_t)b * hkv + h / rep) * hd;
    float dot = 0.f, qq = 0.f, kk = 0.f;
    for (int d = lane; d < hd; d += 32) {
      float v = __bfloat162float(qv[d]);
      if (d < rotary_dim) {
        const int j = d < half ? d : d - half;
        float sn, cs;
        sincosf((float)qpos[qi] * inv_freq[j], &sn, &cs);
        const float o = __bfloat162float(qv[d < half ? d + half : d - half]);
        v = d < half ? v * cs + o * sn : v * cs - o * sn;
      }
      const float k = kb[d];
      dot += v * k; qq += v * v; kk += k * k;
    }
    dot = warp_sum(dot); qq = warp_sum(qq); kk = warp_sum(kk);
    best = fmaxf(best, dot * rsqrtf(fmaxf(qq * kk, 1e-20f)));
  }
  if (lane == 0) red[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    out[b] = m;
  }
}

__global__ void __launch_bounds__(1024) kvscore_softmax_kernel(const float* __restrict__ s, int n, float temp, float* __restrict__ out) {
  __shared__ float red[32];
  float m = -INFINITY;
  for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, s[i] * temp);
  m = block_max(m, red);
  float sum = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) sum += __expf(s[i] * temp - m);
  sum = block_sum(sum, red);
  for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = __expf(s[i] * temp - m) / sum;
}

}  // namespace owl
using namespace owl;

// k_pool: one layer's e4m3 pool [pages][16][hkv][hd]; pages / pos0 / n_valid: int32 [blocks]; out float [blocks][hkv][hd].
OWL_API int owl_mean_k_block(const void* k_pool, const void* pages, const void* pos0, const void* n_valid, const void* inv_freq,
                             int rotary_dim, int blocks, int hkv, int hd, void* out, cudaStream_t st) {
  if (blocks < 1 || hkv < 1 || hd < 32 || hd > 1024 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return OWL_ERR_BAD_ARG;
  mean_k_block_kernel<0><<<dim3(blocks, hkv), hd, 0, st>>>((const uint8_t*)k_pool, nullptr, (const int*)pages, (const int*)pos0,
                                                          (const int*)n_valid, (const float*)inv_freq, rotary_dim, hkv, hd,
                                                          (float*)out);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// The same index over the other pool formats: fmt 1 = int8 with k_scale float [pages][16][hkv], fmt 2 = fp16 words.
OWL_API int owl_mean_k_block_fmt(const void* k_pool, const void* k_scale, int fmt, const void* pages, const void* pos0,
                                 const void* n_valid, const void* inv_freq, int rotary_dim, int blocks, int hkv, int hd, void* out,
                                 cudaStream_t st) {
  if (blocks < 1 || hkv < 1 || hd < 32 || hd > 1024 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) || fmt < 0 || fmt > 2 ||
      (fmt == 1 && !k_scale))
    return OWL_ERR_BAD_ARG;
  const dim3 grid(blocks, hkv);
  if (fmt == 0)
    mean_k_block_kernel<0><<<grid, hd, 0, st>>>((const uint8_t*)k_pool, nullptr, (const int*)pages, (const int*)pos0,
                                                (const int*)n_valid, (const float*)inv_freq, rotary_dim, hkv, hd, (float*)out);
  else if (fmt == 1)
    mean_k_block_kernel<1><<<grid, hd, 0, st>>>((const uint8_t*)k_pool, (const float*)k_scale, (const int*)pages, (const int*)pos0,
                                                (const int*)n_valid, (const float*)inv_freq, rotary_dim, hkv, hd, (float*)out);
  else
    mean_k_block_kernel<2><<<grid, hd, 0, st>>>((const uint8_t*)k_pool, nullptr, (const int*)pages, (const int*)pos0,
                                                (const int*)n_valid, (const float*)inv_freq, rotary_dim, hkv, hd, (float*)out);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// q bf16 [nq][hq][hd] (rotated), qpos int32 [nq], index float [blocks][hkv][hd]; out float [blocks].
OWL_API int owl_kvscore(const void* q, const void* qpos, const void* index, const void* inv_freq, int rotary_dim, int nq, int hq,
                        int hkv, int hd, int blocks, void* out, cudaStream_t st) {
  if (blocks < 1 || nq < 1 || hkv < 1 || hq % hkv || rotary_dim > hd || (rotary_dim & 1)) return OWL_ERR_BAD_ARG;
  kvscore_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)q, (const int*)qpos, (const float*)index, (const float*)inv_freq,
                                         rotary_dim, nq, hq, hkv, hd, (float*)out);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

OWL_API int owl_kvscore_softmax(const void* scores, int n, float temp, void* out, cudaStream_t st) {
  if (n < 1) return OWL_ERR_BAD_ARG;
  kvscore_softmax_kernel<<<1, 1024, 0, st>>>((const float*)scores, n, temp, (float*)out);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
