// Kernels of the DFlash2 block draft (a small bf16 transformer that proposes 7 tokens in one forward):
//
//   owl_dflash_conv      grouped dynamic 2-tap temporal convolution inside a block of rows
//   owl_dflash_norm_rope per-head RMSNorm + rotate-half RoPE (hd = 128, full rotary), optional write of K and V
//                        rows into the draft's ring KV (window of the most recent positions)
//   owl_dflash_nc_attn   non-causal block attention: every row of the block sees the whole prefix window in the
//                        ring and all rows of its own block; split over the window + owl_dflash_nc_reduce
//   owl_dflash_select    selector lattice score[e,p,c] = unary[e,c] + <A[pred] * proj[e], B[cand[e,c]]> and the
//                        greedy walk through it, one CTA, no host round trip
//
// Math as in the reference's draft kernels (crates/kernels/cu/dflash/dflash_conv.cu:10-40,
// cu/dflash/dflash_select.cu:10-42, cu/attn/naive_attn_nc.cu:66) and layer (crates/models/src/layers/dflash2.rs:1-40);
// the kernels here are written for 148 SMs: the attention splits the window so that a block of 8 rows fills the
// GPU (8 KV heads x 16 splits), one lane per query row, keys broadcast from shared memory.
#include "common.cuh"

namespace owl {

constexpr int DF_GROUP = 16;      // channels per convolution group
constexpr int DF_HD = 128;        // draft head dim
constexpr int DF_MAX_ROWS = 8;    // rows of a block (1 anchor + 7 masked)

// out[t, d] = sum_tap (base[side, tap, d] + delta[t, side, tap, d / 16]) * x[t - tap, d] * [t % block >= tap]
__global__ void __launch_bounds__(256) dflash_conv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                                                          const __nv_bfloat16* __restrict__ base, int side, int block, int H,
                                                          int rows, __nv_bfloat16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int G = H / DF_GROUP;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * H) return;
  const int t = (int)(i / H), d = (int)(i % H), g = d / DF_GROUP;
  float acc = 0.f;
#pragma unroll
  for (int tap = 0; tap < 2; ++tap) {
    if ((t % block) < tap || t < tap) continue;
    const float c = __bfloat162float(base[((size_t)side * 2 + tap) * H + d]) +
                    __bfloat162float(delta[(((size_t)t * 2 + side) * 2 + tap) * G + g]);
    acc += c * __bfloat162float(x[(size_t)(t - tap) * H + d]);
  }
  out[i] = __float2bfloat16(acc);
}

// One CTA (128 threads = head dim) per (row, head). heads_n heads are normalised + rotated; when ring_k is
// given the result goes to ring_k[slot[row]] (and the matching v row is copied to ring_v), else to out.
struct DfNormRopeParams {
  const __nv_bfloat16* x; int ldx;            // [T][ldx], head h at column h * 128
  const __nv_bfloat16* v; int ldv;            // value rows (ring write only)
  const __nv_bfloat16* w;                     // norm weight [128]
  const int* pos; const float* inv_freq;      // [T], [64]
  __nv_bfloat16* out;                         // [T][heads * 128] or null
  __nv_bfloat16* ring_k; __nv_bfloat16* ring_v; const int* slot;   // [cap][heads][128]
  int heads; float eps;
};
__global__ void __launch_bounds__(DF_HD) dflash_norm_rope_kernel(DfNormRopeParams p) {
  __shared__ float red[32];
  __shared__ float row[DF_HD];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const float xv = __bfloat162float(p.x[(size_t)t * p.ldx + h * DF_HD + d]);
  const float ss = block_sum(xv * xv, red);
  const float n = xv * rsqrtf(ss / DF_HD + p.eps) * __bfloat162float(p.w[d]);
  row[d] = __bfloat162float(__float2bfloat16(n));
  __syncthreads();
  const int j = d & 63;
  const float ang = (float)p.pos[t] * p.inv_freq[j];
  float sn, cs;
  sincosf(ang, &sn, &cs);
  const float a = row[d], b = row[d < 64 ? d + 64 : d - 64];
  const float r = d < 64 ? a * cs - b * sn : a * cs + b * sn;
  if (p.ring_k) {
    const size_t o = ((size_t)p.slot[t] * p.heads + h) * DF_HD + d;
    p.ring_k[o] = __float2bfloat16(r);
    p.ring_v[o] = p.v[(size_t)t * p.ldv + h * DF_HD + d];
  } else {
    p.out[((size_t)t * p.heads + h) * DF_HD + d] = __float2bfloat16(r);
  }
}

// Non-causal block attention. grid (Hkv, splits), 256 threads. Lane l of every warp owns query row
// (l / gq) of q head (kvh * gq + l % gq), gq = Hq / Hkv, rows * gq <= 32. The warps walk the keys of the split
// (ring slots [lo, hi) and, in split 0, the block's own keys) with stride 8; keys and values are staged per warp
// in shared memory and read as broadcasts. Partial (m, l, acc) per split go to global memory.
struct DfAttnParams {
  const __nv_bfloat16* q;        // [rows][Hq][128]
  const __nv_bfloat16* kself; const __nv_bfloat16* vself; int ldv;   // [rows][Hkv][128], v rows [rows][ldv]
  const __nv_bfloat16* ring_k; const __nv_bfloat16* ring_v;          // [cap][Hkv][128]
  const int* prefix_len;         // device: number of valid ring slots (min(tokens so far, cap))
  float* part_o; float* part_ml; // [Hkv][splits][32][128], [Hkv][splits][32][2]
  int rows, Hq, Hkv, cap, splits; float scale;
};
__global__ void __launch_bounds__(256) dflash_nc_attn_kernel(DfAttnParams p) {
  __shared__ __align__(16) float s_kv[8][2][DF_HD];    // per warp: key, value
  __shared__ float s_acc[32][DF_HD + 1];
  __shared__ float s_m[32], s_l[32];
  __shared__ uint32_t s_q[32][DF_HD / 2 + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int kvh = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = p.Hq / p.Hkv, nq = p.rows * gq;
  const int n_ring = min(*p.prefix_len, p.cap);
  const int per = (n_ring + p.splits - 1) / p.splits;
  const int lo = split * per, hi = min(n_ring, lo + per);
  const int n_keys = max(0, hi - lo) + (split == 0 ? p.rows : 0);
  // this lane's query vector: packed bf16 pairs in shared memory (row stride 65 words: conflict-free per-lane reads)
  const bool live = lane < nq;
  if (warp == 0) {
    const int r = live ? lane / gq : 0, h = kvh * gq + (live ? lane % gq : 0);
    const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)r * p.Hq + h) * DF_HD);
#pragma unroll
    for (int c = 0; c < DF_HD / 8; ++c) {
      const uint4 u = src[c];
      s_q[lane][c * 4] = u.x; s_q[lane][c * 4 + 1] = u.y; s_q[lane][c * 4 + 2] = u.z; s_q[lane][c * 4 + 3] = u.w;
    }
  }
  __syncthreads();
  const uint32_t* qv = s_q[lane];
  float m = -INFINITY, l = 0.f, acc[DF_HD];
#pragma unroll
  for (int d = 0; d < DF_HD; ++d) acc[d] = 0.f;
  for (int k = warp; k < n_keys; k += 8) {
    const __nv_bfloat16 *kp, *vp;
    if (k < hi - lo) {
      kp = p.ring_k + ((size_t)(lo + k) * p.Hkv + kvh) * DF_HD;
      vp = p.ring_v + ((size_t)(lo + k) * p.Hkv + kvh) * DF_HD;
    } else {
      const int r = k - max(0, hi - lo);
      kp = p.kself + ((size_t)r * p.Hkv + kvh) * DF_HD;
      vp = p.vself + (size_t)r * p.ldv + kvh * DF_HD;
    }
    const uint2 ku = reinterpret_cast<const uint2*>(kp)[lane], vu = reinterpret_cast<const uint2*>(vp)[lane];
    __syncwarp();
    s_kv[warp][0][lane * 4 + 0] = bf16_lo(ku.x); s_kv[warp][0][lane * 4 + 1] = bf16_hi(ku.x);
    s_kv[warp][0][lane * 4 + 2] = bf16_lo(ku.y); s_kv[warp][0][lane * 4 + 3] = bf16_hi(ku.y);
    s_kv[warp][1][lane * 4 + 0] = bf16_lo(vu.x); s_kv[warp][1][lane * 4 + 1] = bf16_hi(vu.x);
    s_kv[warp][1][lane * 4 + 2] = bf16_lo(vu.y); s_kv[warp][1][lane * 4 + 3] = bf16_hi(vu.y);
    __syncwarp();
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < DF_HD; d += 4) {
      const float4 kk = *reinterpret_cast<const float4*>(&s_kv[warp][0][d]);
      s += bf16_lo(qv[d / 2]) * kk.x + bf16_hi(qv[d / 2]) * kk.y + bf16_lo(qv[d / 2 + 1]) * kk.z + bf16_hi(qv[d / 2 + 1]) * kk.w;
    }
    s *= p.scale;
    const float mn = fmaxf(m, s), corr = __expf(m - mn), pr = __expf(s - mn);
    l = l * corr + pr;
    m = mn;
#pragma unroll
    for (int d = 0; d < DF_HD; d += 4) {
      const float4 vv = *reinterpret_cast<const float4*>(&s_kv[warp][1][d]);
      acc[d] = acc[d] * corr + pr * vv.x;
      acc[d + 1] = acc[d + 1] * corr + pr * vv.y;
      acc[d + 2] = acc[d + 2] * corr + pr * vv.z;
      acc[d + 3] = acc[d + 3] * corr + pr * vv.w;
    }
  }
  // merge the 8 warps (one after the other) into shared memory
  if (warp == 0) {
    s_m[lane] = m; s_l[lane] = l;
#pragma unroll
    for (int d = 0; d < DF_HD; ++d) s_acc[lane][d] = acc[d];
  }
  __syncthreads();
  for (int w = 1; w < 8; ++w) {
    if (warp == w && m > -INFINITY) {
      const float mo = s_m[lane], mn = fmaxf(mo, m);
      const float co = mo > -INFINITY ? __expf(mo - mn) : 0.f, cn = __expf(m - mn);
      s_m[lane] = mn;
      s_l[lane] = s_l[lane] * co + l * cn;
#pragma unroll
      for (int d = 0; d < DF_HD; ++d) s_acc[lane][d] = s_acc[lane][d] * co + acc[d] * cn;
    }
    __syncthreads();
  }
  float* po = p.part_o + ((size_t)(kvh * p.splits + split) * 32) * DF_HD;
  for (int i = threadIdx.x; i < 32 * DF_HD; i += blockDim.x) po[i] = s_acc[i / DF_HD][i % DF_HD];
  if (threadIdx.x < 32) {
    float* pm = p.part_ml + ((size_t)(kvh * p.splits + split) * 32 + threadIdx.x) * 2;
    pm[0] = s_m[threadIdx.x];
    pm[1] = s_l[threadIdx.x];
  }
}

// out[r][h][d] (bf16) from the split partials. grid (rows * Hq), 128 threads.
__global__ void __launch_bounds__(DF_HD) dflash_nc_reduce_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                 __nv_bfloat16* __restrict__ out, int rows, int Hq, int Hkv,
                                                                 int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x / Hq, h = blockIdx.x % Hq, d = threadIdx.x;
  const int gq = Hq / Hkv, kvh = h / gq, lane = r * gq + h % gq;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[((size_t)(kvh * splits + s) * 32 + lane) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* ml = part_ml + ((size_t)(kvh * splits + s) * 32 + lane) * 2;
    if (ml[0] == -INFINITY) continue;
    const float c = __expf(ml[0] - m);
    l += ml[1] * c;
    o += part_o[((size_t)(kvh * splits + s) * 32 + lane) * DF_HD + d] * c;
  }
  out[((size_t)r * Hq + h) * DF_HD + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
}

// Selector: S slots, K candidates each, rank R. One CTA of 256 threads; warp per lattice item.
__global__ void __launch_bounds__(256) dflash_select_kernel(const int* __restrict__ cand, const float* __restrict__ unary,
                                                            const __nv_bfloat16* __restrict__ proj, int ldp,
                                                            const int* __restrict__ anchor, const __nv_bfloat16* __restrict__ a_tab,
                                                            const __nv_bfloat16* __restrict__ b_tab, int S, int K, int R,
                                                            int* __restrict__ out_tok, float* __restrict__ scores) {
  extern __shared__ float s_score[];    // [S][K][K]
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, items = S * K * K;
  const int anc = anchor[0];
  for (int it = warp; it < items; it += 8) {
    const int e = it / (K * K), pp = (it / K) % K, c = it % K;
    const int pred = e == 0 ? anc : cand[(e - 1) * K + pp];
    const int cd = cand[e * K + c];
    const __nv_bfloat16 *ar = a_tab + (size_t)pred * R, *br = b_tab + (size_t)cd * R, *pr = proj + (size_t)e * ldp;
    float dot = 0.f;
    for (int r = lane; r < R; r += 32) dot += __bfloat162float(ar[r]) * __bfloat162float(pr[r]) * __bfloat162float(br[r]);
    dot = warp_sum(dot);
    if (lane == 0) {
      const float sc = unary[e * K + c] + dot;
      s_score[it] = sc;
      if (scores) scores[it] = sc;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int idx = 0;
    for (int e = 0; e < S; ++e) {
      const float* row = s_score + (e * K + (e == 0 ? 0 : idx)) * K;
      int best = 0;
      for (int c = 1; c < K; ++c)
        if (row[c] > row[best]) best = c;          // ties: the smaller index
      idx = best;
      out_tok[e] = cand[e * K + best];
    }
  }
}

template <typename... Args>
static int df_launch(void (*kern)(Args...), dim3 grid, dim3 block, size_t smem, int pdl, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

}  // namespace owl
using namespace owl;

// x, out: bf16 [rows][H]; delta: bf16 [rows][2][2][H/16]; base: bf16 [2][2][H].
OWL_API int owl_dflash_conv(const void* x, const void* delta, const void* base, int side, int block, int H, int rows, void* out,
                            int pdl, cudaStream_t st) {
  if (rows < 1 || H < DF_GROUP || (H % DF_GROUP) || block < 1 || (side != 0 && side != 1)) return OWL_ERR_BAD_ARG;
  const size_t n = (size_t)rows * H;
  return df_launch(dflash_conv_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, pdl, st, (const __nv_bfloat16*)x,
                   (const __nv_bfloat16*)delta, (const __nv_bfloat16*)base, side, block, H, rows, (__nv_bfloat16*)out);
}

// Normalise + rotate `heads` heads of x; write to out [T][heads][128], or (ring_k != null) K to ring_k[slot[t]] and the
// v rows to ring_v[slot[t]].
OWL_API int owl_dflash_norm_rope(const void* x, int ldx, const void* v, int ldv, const void* w, const void* pos,
                                 const void* inv_freq, void* out, void* ring_k, void* ring_v, const void* slot, int T, int heads,
                                 float eps, int pdl, cudaStream_t st) {
  if (T < 1 || heads < 1 || (!out && !ring_k) || (ring_k && (!ring_v || !slot || !v))) return OWL_ERR_BAD_ARG;
  DfNormRopeParams p = {};
  p.x = (const __nv_bfloat16*)x; p.ldx = ldx; p.v = (const __nv_bfloat16*)v; p.ldv = ldv; p.w = (const __nv_bfloat16*)w;
  p.pos = (const int*)pos; p.inv_freq = (const float*)inv_freq; p.out = (__nv_bfloat16*)out; p.ring_k = (__nv_bfloat16*)ring_k;
  p.ring_v = (__nv_bfloat16*)ring_v; p.slot = (const int*)slot; p.heads = heads; p.eps = eps;
  return df_launch(dflash_norm_rope_kernel, dim3(T, heads), dim3(DF_HD), 0, pdl, st, p);
}

// part_o: float [Hkv][splits][32][128]; part_ml: float [Hkv][splits][32][2]; out bf16 [rows][Hq][128].
OWL_API int owl_dflash_nc_attn(const void* q, const void* kself, const void* vself, int ldv, const void* ring_k, const void* ring_v,
                               const void* prefix_len, void* part_o, void* part_ml, void* out, int rows, int Hq, int Hkv, int cap,
                               int splits, float scale, int pdl, cudaStream_t st) {
  if (rows < 1 || rows > DF_MAX_ROWS || Hkv < 1 || Hq % Hkv || rows * (Hq / Hkv) > 32 || splits < 1 || splits > 64 || cap < 1)
    return OWL_ERR_BAD_ARG;
  DfAttnParams p = {};
  p.q = (const __nv_bfloat16*)q; p.kself = (const __nv_bfloat16*)kself; p.vself = (const __nv_bfloat16*)vself; p.ldv = ldv;
  p.ring_k = (const __nv_bfloat16*)ring_k; p.ring_v = (const __nv_bfloat16*)ring_v; p.prefix_len = (const int*)prefix_len;
  p.part_o = (float*)part_o; p.part_ml = (float*)part_ml; p.rows = rows; p.Hq = Hq; p.Hkv = Hkv; p.cap = cap;
  p.splits = splits; p.scale = scale;
  int r = df_launch(dflash_nc_attn_kernel, dim3(Hkv, splits), dim3(256), 0, pdl, st, p);
  if (r) return r;
  return df_launch(dflash_nc_reduce_kernel, dim3(rows * Hq), dim3(DF_HD), 0, pdl, st, (const float*)part_o,
                   (const float*)part_ml, (__nv_bfloat16*)out, rows, Hq, Hkv, splits);
}

// cand int32 [S][K], unary float [S][K], proj bf16 [S][ldp], anchor int32 [1] (device), codebooks bf16 [vocab][R];
// out_tok int32 [S]; scores float [S][K][K] or null.
OWL_API int owl_dflash_select(const void* cand, const void* unary, const void* proj, int ldp, const void* anchor,
                              const void* a_tab, const void* b_tab, int S, int K, int R, void* out_tok, void* scores, int pdl,
                              cudaStream_t st) {
  if (S < 1 || S > 15 || K < 1 || K > 32 || R < 1) return OWL_ERR_BAD_ARG;
  const size_t smem = (size_t)S * K * K * sizeof(float);
  if (smem > 48 * 1024) return OWL_ERR_BAD_ARG;
  return df_launch(dflash_select_kernel, dim3(1), dim3(256), smem, pdl, st, (const int*)cand, (const float*)unary,
                   (const __nv_bfloat16*)proj, ldp, (const int*)anchor, (const __nv_bfloat16*)a_tab, (const __nv_bfloat16*)b_tab, S,
                   K, R, (int*)out_tok, (float*)scores);
}
