// Vision-tower operators (ViT blocks of the VLM front end). The matrix products run on the dense tcgen05 GEMM
// (gemm_dense.cu); these kernels are everything around them, each one pass over its rows:
//
//   owl_vis_layernorm   y = (x - mean) / sqrt(var + eps) * w + b                       bf16 rows, fp32 statistics
//   owl_vis_bias_act    y = act(x + bias) (+ residual)    act: none | GELU(tanh) | GELU(erf)   (the epilogue of every Linear)
//   owl_vis_pos_embed   x += bilinear 4-tap resampling of the learned G x G position table at the patch's grid cell
//                       (patches arrive in merge-window order)
//   owl_vis_rope        2-D axial rotary embedding of q and k inside the packed qkv rows (rotate-half layout: the first half
//                       of the rotary pairs turns with the patch's row, the second half with its column)
//   owl_vis_attn        non-causal attention inside each image (variable-length segments), head_dim up to 80 (72 for the
//                       27B family's tower): one warp per 16 query rows, mma.sync m16n8k16 bf16, keys in tiles of 64 through
//                       shared memory, online softmax on the accumulator fragments, P reused as the A operand of P V
//
// Role in the reference: crates/kernels/cu/vis/vision_ops.cu:1-30 (Gelu tanh / erf, BiasAdd, PosEmbedBilinear, AttnFull) and
// cu/vis/layernorm.cu.
#include "common.cuh"
#include "actpack.cuh"

namespace owl {

// ---- LayerNorm: one warp per row ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) vis_layernorm_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const float* __restrict__ w,
                                                            const float* __restrict__ b, __nv_bfloat16* __restrict__ out, int ldo,
                                                            int rows, int C, float eps) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + (size_t)row * ldx;
  float s = 0.f, ss = 0.f;
  for (int c = lane * 8; c < C; c += 256) {
    float v[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(xr + c), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) { s += v[i]; ss = fmaf(v[i], v[i], ss); }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  const float mean = s / (float)C, rstd = rsqrtf(fmaxf(ss / (float)C - mean * mean, 0.f) + eps);
  __nv_bfloat16* orow = out + (size_t)row * ldo;
  for (int c = lane * 8; c < C; c += 256) {
    float v[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(xr + c), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (v[i] - mean) * rstd * w[c + i] + b[c + i];
    *reinterpret_cast<uint4*>(orow + c) = pack_bf16x8(v);
  }
}

// ---- bias + activation (+ residual) ------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_tanh_f(float v) {
  return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}
__device__ __forceinline__ float gelu_erf_f(float v) { return 0.5f * v * (1.f + erff(v * 0.7071067811865476f)); }

// grid (ceil(C / 8 / 256), rows)
__global__ void __launch_bounds__(256) vis_bias_act_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const float* __restrict__ bias,
                                                           const __nv_bfloat16* residual, int ldr, __nv_bfloat16* out, int ldo, int C,
                                                           int act) {
  const int row = blockIdx.y, c = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c >= C) return;
  float v[8], r[8];
  unpack_bf16x8(*reinterpret_cast<const uint4*>(x + (size_t)row * ldx + c), v);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] += bias ? bias[c + i] : 0.f;
    v[i] = act == 1 ? gelu_tanh_f(v[i]) : act == 2 ? gelu_erf_f(v[i]) : v[i];
  }
  if (residual) {
    unpack_bf16x8(*reinterpret_cast<const uint4*>(residual + (size_t)row * ldr + c), r);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] += r[i];
  }
  *reinterpret_cast<uint4*>(out + (size_t)row * ldo + c) = pack_bf16x8(v);
}

// patch index n (merge-window order) -> (row, column) of the gh x gw patch grid
__device__ __forceinline__ void vis_cell(int n, int gw, int merge, int& r, int& c) {
  const int per_win = merge * merge, wins_w = gw / merge;
  const int win = n / per_win, in = n % per_win;
  r = (win / wins_w) * merge + in / merge;
  c = (win % wins_w) * merge + in % merge;
}

// grid (ceil(C / 8 / 256), n). align_corners = true resampling of table [G][G][C] to gh x gw.
__global__ void __launch_bounds__(256) vis_pos_embed_kernel(__nv_bfloat16* x, int ldx, const float* __restrict__ table, int G, int gh,
                                                            int gw, int merge, int C) {
  const int n = blockIdx.y, c = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c >= C) return;
  int r, q;
  vis_cell(n, gw, merge, r, q);
  const float fy = gh > 1 ? (float)r * (float)(G - 1) / (float)(gh - 1) : 0.f, fx = gw > 1 ? (float)q * (float)(G - 1) / (float)(gw - 1) : 0.f;
  const int y0 = min((int)fy, G - 1), x0 = min((int)fx, G - 1), y1 = min(y0 + 1, G - 1), x1 = min(x0 + 1, G - 1);
  const float wy = fy - (float)y0, wx = fx - (float)x0;
  const float* t00 = table + ((size_t)y0 * G + x0) * C + c;
  const float* t01 = table + ((size_t)y0 * G + x1) * C + c;
  const float* t10 = table + ((size_t)y1 * G + x0) * C + c;
  const float* t11 = table + ((size_t)y1 * G + x1) * C + c;
  float v[8];
  __nv_bfloat16* xr = x + (size_t)n * ldx + c;
  unpack_bf16x8(*reinterpret_cast<const uint4*>(xr), v);
#pragma unroll
  for (int i = 0; i < 8; ++i)
    v[i] += (1.f - wy) * ((1.f - wx) * t00[i] + wx * t01[i]) + wy * ((1.f - wx) * t10[i] + wx * t11[i]);
  *reinterpret_cast<uint4*>(xr) = pack_bf16x8(v);
}

// qkv [n][3][heads][hd]: rotate q and k in place. grid (n), block = heads * hd / 2 threads rounded up to 32 (one rotary pair of
// one head each, for q and k). pairs = hd / 2; pair j < pairs / 2 turns with the row index, the others with the column index;
// frequency of pair j: 10000^(-(j mod pairs/2) / (pairs/2)).
__global__ void __launch_bounds__(1024) vis_rope_kernel(__nv_bfloat16* qkv, int heads, int hd, int gw, int merge, int n0) {
  const int n = blockIdx.x, pairs = hd / 2, half = pairs / 2;
  const int idx = threadIdx.x;
  if (idx >= heads * pairs) return;
  const int h = idx / pairs, j = idx % pairs;
  int r, c;
  vis_cell(n - n0, gw, merge, r, c);
  const int f = j % half;
  const float inv = exp2f(-(float)f / (float)half * 13.287712379549449f);      // 10000^(-f / half)
  const float ang = (float)(j < half ? r : c) * inv;
  float sn, cs;
  sincosf(ang, &sn, &cs);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    __nv_bfloat16* v = qkv + (((size_t)n * 3 + which) * heads + h) * hd;
    const float a = __bfloat162float(v[j]), b = __bfloat162float(v[j + pairs]);
    v[j] = __float2bfloat16(a * cs - b * sn);
    v[j + pairs] = __float2bfloat16(b * cs + a * sn);
  }
}

// ---- non-causal attention over segments --------------------------------------------------------------------------------
constexpr int VA_BM = 64, VA_BN = 64, VA_HDP = 80, VA_LDK = VA_HDP + 8, VA_LDV = VA_BN + 8;

__device__ __forceinline__ void va_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (ceil(n / 64), heads), block 128 (4 warps x 16 query rows). seg: int32 [n_seg + 1] row offsets of the images.
__global__ void __launch_bounds__(128) vis_attn_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out, int n,
                                                       int heads, int hd, const int* __restrict__ seg, int n_seg, float scale_log2) {
  __shared__ __align__(16) __nv_bfloat16 ks[VA_BN][VA_LDK];      // keys of the tile, [key][d]
  __shared__ __align__(16) __nv_bfloat16 vt[VA_HDP][VA_LDV];     // values of the tile transposed, [d][key]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int head = blockIdx.y, q0 = blockIdx.x * VA_BM;
  const int kd = (hd + 15) / 16, nd = (hd + 7) / 8;
  const size_t row_stride = (size_t)3 * heads * hd;
  // segment bounds of this thread's two query rows, and of the whole tile
  const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
  auto bounds = [&](int r, int& lo, int& hi) {
    lo = hi = 0;
    if (r >= n) return;
    for (int s = 0; s < n_seg; ++s)
      if (r >= seg[s] && r < seg[s + 1]) { lo = seg[s]; hi = seg[s + 1]; }
  };
  int lo0, hi0, lo1, hi1, tlo, thi;
  bounds(r0, lo0, hi0);
  bounds(r1, lo1, hi1);
  {
    int a, b;
    bounds(q0, tlo, b);
    bounds(min(q0 + VA_BM, n) - 1, a, thi);
  }
  // Q fragments of this warp's 16 rows: a[kk][0..3]
  uint32_t qa[5][4];
#pragma unroll
  for (int kk = 0; kk < 5; ++kk) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = (i & 1) ? r1 : r0, d = kk * 16 + 2 * t + ((i & 2) ? 8 : 0);
      uint32_t v = 0;
      if (kk < kd && r < n && d < hd) v = *reinterpret_cast<const uint32_t*>(qkv + (size_t)r * row_stride + (size_t)head * hd + d);
      qa[kk][i] = v;
    }
  }
  float o[10][4];
#pragma unroll
  for (int j = 0; j < 10; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  for (int k0 = tlo; k0 < thi; k0 += VA_BN) {
    __syncthreads();
    // stage the tile: thread -> (key, 8 dims) chunks
    for (int ch = tid; ch < VA_BN * (VA_HDP / 8); ch += 128) {
      const int key = ch / (VA_HDP / 8), d = (ch % (VA_HDP / 8)) * 8;
      uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
      if (k0 + key < thi && d < hd) {
        const __nv_bfloat16* src = qkv + (size_t)(k0 + key) * row_stride + (size_t)heads * hd + (size_t)head * hd + d;
        kv = *reinterpret_cast<const uint4*>(src);
        vv = *reinterpret_cast<const uint4*>(src + (size_t)heads * hd);
      }
      *reinterpret_cast<uint4*>(&ks[key][d]) = kv;
      const __nv_bfloat16* ve = reinterpret_cast<const __nv_bfloat16*>(&vv);
#pragma unroll
      for (int i = 0; i < 8; ++i) vt[d + i][key] = ve[i];
    }
    __syncthreads();
    // S = Q K^T for 16 rows x 64 keys: 8 key tiles of 8
    float sc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 5; ++kk) {
        if (kk < kd) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&ks[j * 8 + g][kk * 16 + 2 * t]);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&ks[j * 8 + g][kk * 16 + 2 * t + 8]);
          va_mma(sc[j], qa[kk], b0, b1);
        }
      }
    }
    // mask to each row's own image, online softmax
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = k0 + j * 8 + 2 * t + (i & 1);
        const bool vis = (i < 2) ? (key >= lo0 && key < hi0) : (key >= lo1 && key < hi1);
        sc[j][i] = vis ? sc[j][i] * scale_log2 : -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
      mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0m = fmaxf(m0, mx0), n1m = fmaxf(m1, mx1);
    const float f0 = (n0m == -INFINITY) ? 1.f : exp2f(m0 - n0m), f1 = (n1m == -INFINITY) ? 1.f : exp2f(m1 - n1m);
    m0 = n0m; m1 = n1m;
    l0 *= f0; l1 *= f1;
#pragma unroll
    for (int j = 0; j < 10; ++j) { o[j][0] *= f0; o[j][1] *= f0; o[j][2] *= f1; o[j][3] *= f1; }
    uint32_t pa[4][4];                // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = (m0 == -INFINITY) ? 0.f : exp2f(sc[j][0] - m0), p1 = (m0 == -INFINITY) ? 0.f : exp2f(sc[j][1] - m0);
      const float p2 = (m1 == -INFINITY) ? 0.f : exp2f(sc[j][2] - m1), p3 = (m1 == -INFINITY) ? 0.f : exp2f(sc[j][3] - m1);
      l0 += p0 + p1; l1 += p2 + p3;
      pa[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V: 10 dim tiles of 8, 4 k-steps of 16 keys
#pragma unroll
    for (int j = 0; j < 10; ++j) {
      if (j < nd) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&vt[j * 8 + g][kk * 16 + 2 * t]);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&vt[j * 8 + g][kk * 16 + 2 * t + 8]);
          va_mma(o[j], pa[kk], b0, b1);
        }
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
  for (int j = 0; j < 10; ++j) {
    const int d = j * 8 + 2 * t;
    if (j < nd && d < hd) {
      if (r0 < n) *reinterpret_cast<uint32_t*>(out + ((size_t)r0 * heads + head) * hd + d) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
      if (r1 < n) *reinterpret_cast<uint32_t*>(out + ((size_t)r1 * heads + head) * hd + d) = pack_bf16(o[j][2] * i1, o[j][3] * i1);
    }
  }
}

}  // namespace owl
using namespace owl;

OWL_API int owl_vis_layernorm(const void* x, int ldx, const void* w, const void* b, void* out, int ldo, int rows, int C, float eps,
                              cudaStream_t st) {
  if (rows < 1 || C < 8 || (C & 7) || (ldx & 7) || (ldo & 7) || !x || !w || !b || !out) return OWL_ERR_BAD_ARG;
  vis_layernorm_kernel<<<(rows + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (const float*)w, (const float*)b,
                                                       (__nv_bfloat16*)out, ldo, rows, C, eps);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// act: 0 none, 1 GELU(tanh), 2 GELU(erf). bias fp32 [C] or null; residual bf16 [rows][ldr] or null; out may alias x or residual.
OWL_API int owl_vis_bias_act(const void* x, int ldx, const void* bias, const void* residual, int ldr, void* out, int ldo, int rows,
                             int C, int act, cudaStream_t st) {
  if (rows < 1 || C < 8 || (C & 7) || (ldx & 7) || (ldo & 7) || (residual && (ldr & 7)) || act < 0 || act > 2 || !x || !out)
    return OWL_ERR_BAD_ARG;
  vis_bias_act_kernel<<<dim3((C / 8 + 255) / 256, rows), 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (const float*)bias,
                                                                      (const __nv_bfloat16*)residual, ldr, (__nv_bfloat16*)out, ldo, C,
                                                                      act);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// x bf16 [n][ldx] (the n = gh * gw patches of one image, merge-window order) += table fp32 [G * G][C] resampled to gh x gw.
OWL_API int owl_vis_pos_embed(void* x, int ldx, const void* table, int G, int gh, int gw, int merge, int C, cudaStream_t st) {
  if (!x || !table || G < 1 || gh < 1 || gw < 1 || merge < 1 || gh % merge || gw % merge || (C & 7) || (ldx & 7)) return OWL_ERR_BAD_ARG;
  vis_pos_embed_kernel<<<dim3((C / 8 + 255) / 256, gh * gw), 256, 0, st>>>((__nv_bfloat16*)x, ldx, (const float*)table, G, gh, gw, merge,
                                                                          C);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// qkv bf16 [n_total][3][heads][hd]; rows [n0, n0 + gh * gw) are one image's patches (merge-window order).
OWL_API int owl_vis_rope(void* qkv, int heads, int hd, int n0, int gh, int gw, int merge, cudaStream_t st) {
  if (!qkv || heads < 1 || hd < 4 || (hd & 3) || heads * hd / 2 > 1024 || gh % merge || gw % merge || n0 < 0) return OWL_ERR_BAD_ARG;
  const int threads = ((heads * hd / 2 + 31) / 32) * 32;
  vis_rope_kernel<<<gh * gw, threads, 0, st>>>((__nv_bfloat16*)qkv + (size_t)n0 * 3 * heads * hd, heads, hd, gw, merge, 0);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// qkv bf16 [n][3][heads][hd] -> out bf16 [n][heads * hd]; seg int32 [n_seg + 1] (device) row offsets of the images.
OWL_API int owl_vis_attn(const void* qkv, void* out, int n, int heads, int hd, const void* seg, int n_seg, cudaStream_t st) {
  if (!qkv || !out || !seg || n < 1 || heads < 1 || hd < 8 || hd > VA_HDP || (hd & 7) || n_seg < 1) return OWL_ERR_BAD_ARG;
  vis_attn_kernel<<<dim3((n + VA_BM - 1) / VA_BM, heads), 128, 0, st>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)out, n, heads, hd,
                                                                       (const int*)seg, n_seg, rsqrtf((float)hd) * 1.4426950408889634f);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
