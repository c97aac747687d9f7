// Device side of sampling: exact top-k candidates (k <= 32) of every row's logits, with the
// repetition penalty applied first, so that only k (value, index) pairs per row travel to the host
// sampler instead of the whole vocabulary.
//
//   stage 1  grid (parts, rows): a CTA loads its slice of the row into shared memory, rescales the
//            tokens of the row's history (logit > 0 ? logit / penalty : logit * penalty), then
//            extracts its k largest entries by k rounds of block-wide argmax (ties: lowest index)
//   stage 2  grid (rows): the same extraction over the parts * k survivors
//
// Both stages are exact (no thresholds, no approximate selection) and deterministic.
//
// Role in the reference: crates/kernels/cu/elems/topk32.cu:1-30 (top-32 + repetition penalty) and
// dflash_topk.cu (top-16 for the draft selector); topk_merge_halves.cu for the vocab-split head is
// covered by running stage 2 over the concatenated per-rank candidates.
#include "common.cuh"

namespace owl {

constexpr int TK_THREADS = 256;
constexpr int TK_MAX_K = 32;
constexpr int TK_MAX_SLICE = 8192;      // floats of one stage-1 slice in shared memory
constexpr int TK_MAX_CAND = 4096;       // candidates stage 2 can merge

struct Cand { float v; int i; };

__device__ __forceinline__ Cand cand_max(Cand a, Cand b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// Block-wide argmax over sm[0..n): returns the winner to every thread. red: 8 x Cand scratch.
__device__ __forceinline__ Cand block_argmax(const float* sm, const int* idx, int n, Cand* red) {
  Cand c = {-INFINITY, 0x7fffffff};
  for (int j = threadIdx.x; j < n; j += TK_THREADS) c = cand_max(c, Cand{sm[j], idx ? idx[j] : j});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Cand d = {__shfl_xor_sync(0xffffffffu, c.v, o), __shfl_xor_sync(0xffffffffu, c.i, o)};
    c = cand_max(c, d);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  Cand w = red[0];
#pragma unroll
  for (int k = 1; k < TK_THREADS / 32; ++k) w = cand_max(w, red[k]);
  __syncthreads();
  return w;
}

__global__ void __launch_bounds__(TK_THREADS) topk_stage1(const __nv_bfloat16* __restrict__ logits, int ld, int V, int K,
                                                          const int* __restrict__ hist, const int* __restrict__ hist_len,
                                                          int hist_ld, float penalty, int vocab_offset, float* sval,
                                                          int* sidx) {
  __shared__ float sm[TK_MAX_SLICE];
  __shared__ Cand red[TK_THREADS / 32];
  const int row = blockIdx.y, parts = gridDim.x;
  const int per = (V + parts - 1) / parts, lo = blockIdx.x * per, n = max(0, min(per, V - lo));
  for (int j = threadIdx.x; j < n; j += TK_THREADS) sm[j] = __bfloat162float(logits[(size_t)row * ld + lo + j]);
  __syncthreads();
  if (hist && penalty != 1.f) {
    // the host passes each history token once, so no two threads touch the same entry
    const int hl = hist_len[row];
    for (int j = threadIdx.x; j < hl; j += TK_THREADS) {
      const int t = hist[(size_t)row * hist_ld + j] - vocab_offset - lo;
      if (t >= 0 && t < n) sm[t] = sm[t] > 0.f ? sm[t] / penalty : sm[t] * penalty;
    }
    __syncthreads();
  }
  for (int r = 0; r < K; ++r) {
    const Cand w = block_argmax(sm, nullptr, n, red);
    if (threadIdx.x == 0) {
      const size_t o = ((size_t)row * parts + blockIdx.x) * K + r;
      sval[o] = w.v;
      sidx[o] = w.i == 0x7fffffff ? -1 : w.i + lo + vocab_offset;
      if (w.i != 0x7fffffff) sm[w.i] = -INFINITY;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(TK_THREADS) topk_stage2(const float* __restrict__ sval, const int* __restrict__ sidx,
                                                          int n, int K, float* out_val, int* out_idx) {
  __shared__ float sm[TK_MAX_CAND];
  __shared__ int si[TK_MAX_CAND];
  __shared__ Cand red[TK_THREADS / 32];
  const int row = blockIdx.x;
  for (int j = threadIdx.x; j < n; j += TK_THREADS) {
    sm[j] = sidx[(size_t)row * n + j] < 0 ? -INFINITY : sval[(size_t)row * n + j];
    si[j] = j;
  }
  __syncthreads();
  for (int r = 0; r < K; ++r) {
    const Cand w = block_argmax(sm, si, n, red);
    if (threadIdx.x == 0) {
      const bool any = w.i != 0x7fffffff && w.v > -INFINITY;
      out_val[(size_t)row * K + r] = any ? w.v : -INFINITY;
      out_idx[(size_t)row * K + r] = any ? sidx[(size_t)row * n + w.i] : -1;
      if (w.i != 0x7fffffff) sm[w.i] = -INFINITY;
    }
    __syncthreads();
  }
}

}  // namespace owl
using namespace owl;

// logits bf16 [M][ld] (V valid columns). hist: int32 [M][hist_ld] distinct token ids per row (may be
// null), hist_len int32 [M]. scratch: parts * M * K floats and ints. out: [M][K], sorted descending,
// index -1 / value -inf pads when a row has fewer than K finite entries.
OWL_API int owl_topk(const void* logits, int ld, int M, int V, int K, const void* hist, const void* hist_len,
                     int hist_ld, float penalty, int vocab_offset, void* scratch_val, void* scratch_idx, int parts,
                     void* out_val, void* out_idx, cudaStream_t st) {
  if (M < 1 || V < 1 || K < 1 || K > TK_MAX_K || parts < 1 || (V + parts - 1) / parts > TK_MAX_SLICE ||
      parts * K > TK_MAX_CAND || !logits || !scratch_val || !scratch_idx || !out_val || !out_idx || penalty <= 0.f)
    return OWL_ERR_BAD_ARG;
  topk_stage1<<<dim3(parts, M), TK_THREADS, 0, st>>>((const __nv_bfloat16*)logits, ld, V, K, (const int*)hist,
                                                     (const int*)hist_len, hist_ld, penalty, vocab_offset,
                                                     (float*)scratch_val, (int*)scratch_idx);
  OWL_LAUNCH_CHECK();
  topk_stage2<<<M, TK_THREADS, 0, st>>>((const float*)scratch_val, (const int*)scratch_idx, parts * K, K,
                                        (float*)out_val, (int*)out_idx);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// Merge per-rank candidate lists of a vocab-split head: cand_val / cand_idx [M][n] (n = ranks * K,
// global token ids) -> the global top-K.
OWL_API int owl_topk_merge(const void* cand_val, const void* cand_idx, int M, int n, int K, void* out_val, void* out_idx,
                           cudaStream_t st) {
  if (M < 1 || n < 1 || n > TK_MAX_CAND || K < 1 || K > TK_MAX_K) return OWL_ERR_BAD_ARG;
  topk_stage2<<<M, TK_THREADS, 0, st>>>((const float*)cand_val, (const int*)cand_idx, n, K, (float*)out_val,
                                        (int*)out_idx);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
