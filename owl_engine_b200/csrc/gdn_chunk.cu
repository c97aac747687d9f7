// Chunked (WY representation) gated delta rule for prefill on tensor cores.
//
// The serial rule per v-head   S <- e^{g_t} S;  d_t = beta_t (v_t - k_t^T S);  S += k_t d_t^T;  o_t = scale q_t^T S
// is evaluated 64 tokens at a time. With gc = cumsum(g) inside a chunk, D_ij = e^{gc_i - gc_j},
//   A'  = strictly_lower(beta_i (k_i . k_j) D_ij)          T = (I + A')^-1
//   u   = T (beta v)             w = T (beta e^{gc} k)     attn = lower(scale (q_i . k_j) D_ij)
//   v'  = u - w S                o = (scale e^{gc} q) S + attn v'
//   S  <- e^{gc_last} S + (e^{gc_last - gc} k)^T v'
// (every exponential has a non-positive argument). Two kernels:
//   gdn_chunk_prep_kernel  one CTA per (chunk, v-head), all chunks in parallel: the 64x64 products and the two 64x128
//                          products on mma.sync (bf16 in, fp32 accumulate), the triangular inverse by forward substitution
//                          with one column per thread; writes w, u, scaled q, scaled k^T and attn
//   gdn_chunk_scan_kernel  one CTA per (v-head, half of the value columns), the chunks in order: three small tensor-core
//                          products per chunk against the fp32 state kept in MMA accumulator registers (a bf16 copy in
//                          shared memory is the B operand), operands prefetched one chunk ahead with cp.async
// followed by the gated RMSNorm kernel of gdn.cu. q and k arrive l2-normalised from the convolution kernel.
//
// Reference counterpart: the chunk-64 delta-rule kernels (cumsum, kkt, solve_tril, wu, h, o) that the reference compiles
// ahead of time from a Triton fork (crates/kernels/triton/gdn_chunked_*), launched around a state transpose. Tiles of 64
// rows are below the tcgen05 instruction shapes that pay (M = 128 per CTA), so this family stays on warp-level MMA.
#include "common.cuh"

namespace owl {

constexpr int CK_C = 64;            // chunk length
constexpr int CK_D = 128;           // head dim (k and v)
constexpr int CK_LD = CK_D + 8;     // row stride of [64][128] bf16 tiles (68 words: conflict-free fragment loads)
constexpr int CK_LT = CK_C + 8;     // row stride of [*][64] bf16 tiles
constexpr int CK_NC = 64;           // value columns per CTA of the recurrence kernel

__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// A fragment (16 x 16) of a row-major bf16 tile; B fragment (16 x 8) of a tile stored [n][k]
__device__ __forceinline__ void frag_a(const __nv_bfloat16* s, int ld, int m0, int k0, int g, int t, uint32_t* a) {
  a[0] = *reinterpret_cast<const uint32_t*>(s + (m0 + g) * ld + k0 + 2 * t);
  a[1] = *reinterpret_cast<const uint32_t*>(s + (m0 + g + 8) * ld + k0 + 2 * t);
  a[2] = *reinterpret_cast<const uint32_t*>(s + (m0 + g) * ld + k0 + 2 * t + 8);
  a[3] = *reinterpret_cast<const uint32_t*>(s + (m0 + g + 8) * ld + k0 + 2 * t + 8);
}
__device__ __forceinline__ void frag_b(const __nv_bfloat16* s, int ld, int n0, int k0, int g, int t, uint32_t* b) {
  b[0] = *reinterpret_cast<const uint32_t*>(s + (n0 + g) * ld + k0 + 2 * t);
  b[1] = *reinterpret_cast<const uint32_t*>(s + (n0 + g) * ld + k0 + 2 * t + 8);
}
__device__ __forceinline__ void ck_cp16(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
}

struct GdnChunkParams {
  const __nv_bfloat16* qkv;     // [T][conv_dim]: q | k (nk heads each, l2-normalised) | v (nv heads)
  const __nv_bfloat16* ab;      // [T][ldab]: a (nv) | b (nv)
  const float* a_log; const float* dt_bias;
  float* state;                 // [slots][nv][128 k][128 v]
  float* raw;                   // [T][nv * 128] un-normalised outputs
  __nv_bfloat16* w;             // [Tpad][nv][128]
  float* u;                     // [Tpad][nv][128] (fp32: v' = u - w S cancels)
  __nv_bfloat16* qg;            // [Tpad][nv][128]   scale e^{gc} q
  __nv_bfloat16* kdT;           // [nv][chunks][128][64]   (e^{gc_last - gc} k)^T
  __nv_bfloat16* attn;          // [nv][chunks][64][64]
  float* eglast;                // [nv][chunks]
  int ldab, nk, nv, T, slot, use_state, chunks;
};

// ---- preparation: one CTA per (chunk, v-head), 256 threads -----------------------------------------------------------
struct PrepSmem {
  __nv_bfloat16 k[CK_C][CK_LD];       // k rows
  __nv_bfloat16 q[CK_C][CK_LD];       // q rows; later T as bf16 ([64][CK_LT] inside the same bytes)
  __nv_bfloat16 vbT[CK_D][CK_LT];     // (beta v)^T
  __nv_bfloat16 kgT[CK_D][CK_LT];     // (beta e^{gc} k)^T; first the staging area of the raw v rows ([64][CK_LD])
  float a[CK_C][CK_C + 1];            // A' (strictly lower)
  float g[CK_C], gc[CK_C], beta[CK_C];
};
__global__ void __launch_bounds__(256) gdn_chunk_prep_kernel(GdnChunkParams p) {
  extern __shared__ __align__(16) uint8_t ck_smem[];
  PrepSmem& sm = *reinterpret_cast<PrepSmem*>(ck_smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  const int c = blockIdx.x, h = blockIdx.y, R = p.nv / p.nk, hk = h / R;
  const int K = p.nk * CK_D, V = p.nv * CK_D, conv_dim = 2 * K + V, r0 = c * CK_C;
  const float scale = rsqrtf((float)CK_D);
  __nv_bfloat16(*vraw)[CK_LD] = reinterpret_cast<__nv_bfloat16(*)[CK_LD]>(&sm.kgT[0][0]);
  // 1. tiles (zero rows past T) and per-token scalars
  for (int i = tid; i < CK_C * 16; i += 256) {
    const int t = i >> 4, piece = (i & 15) * 8, r = r0 + t;
    uint4 qv = make_uint4(0, 0, 0, 0), kv = qv, vv = qv;
    if (r < p.T) {
      const __nv_bfloat16* xr = p.qkv + (size_t)r * conv_dim;
      qv = *reinterpret_cast<const uint4*>(xr + hk * CK_D + piece);
      kv = *reinterpret_cast<const uint4*>(xr + K + hk * CK_D + piece);
      vv = *reinterpret_cast<const uint4*>(xr + 2 * K + h * CK_D + piece);
    }
    *reinterpret_cast<uint4*>(&sm.q[t][piece]) = qv;
    *reinterpret_cast<uint4*>(&sm.k[t][piece]) = kv;
    *reinterpret_cast<uint4*>(&vraw[t][piece]) = vv;
  }
  if (tid < CK_C) {
    const int r = r0 + tid;
    float gg = 0.f, bb = 0.f;
    if (r < p.T) {
      const float a = __bfloat162float(p.ab[(size_t)r * p.ldab + h]);
      const float b = __bfloat162float(p.ab[(size_t)r * p.ldab + p.nv + h]);
      gg = -__expf(p.a_log[h]) * softplus_f(a + p.dt_bias[h]);
      bb = sigmoid_f(b);
    }
    sm.g[tid] = gg;
    sm.beta[tid] = bb;
  }
  __syncthreads();
  if (tid == 0) {
    float acc = 0.f;
    for (int i = 0; i < CK_C; ++i) { acc += sm.g[i]; sm.gc[i] = acc; }
    p.eglast[(size_t)h * p.chunks + c] = __expf(acc);
  }
  __syncthreads();
  const float gc_last = sm.gc[CK_C - 1];
  // 2. (beta v)^T, scaled q rows and scaled k^T to global; all read the row tiles
  for (int i = tid; i < CK_D * (CK_C / 2); i += 256) {
    const int d = i / (CK_C / 2), j = (i % (CK_C / 2)) * 2;
    const float v0 = __bfloat162float(vraw[j][d]) * sm.beta[j], v1 = __bfloat162float(vraw[j + 1][d]) * sm.beta[j + 1];
    *reinterpret_cast<uint32_t*>(&sm.vbT[d][j]) = pack_bf16(v0, v1);
    const float k0 = __bfloat162float(sm.k[j][d]), k1 = __bfloat162float(sm.k[j + 1][d]);
    *reinterpret_cast<uint32_t*>(p.kdT + (((size_t)h * p.chunks + c) * CK_D + d) * CK_C + j) =
        pack_bf16(k0 * __expf(gc_last - sm.gc[j]), k1 * __expf(gc_last - sm.gc[j + 1]));
  }
  for (int i = tid; i < CK_C * (CK_D / 2); i += 256) {
    const int t = i / (CK_D / 2), d = (i % (CK_D / 2)) * 2;
    const float e = scale * __expf(sm.gc[t]);
    *reinterpret_cast<uint32_t*>(p.qg + ((size_t)(r0 + t) * p.nv + h) * CK_D + d) =
        pack_bf16(__bfloat162float(sm.q[t][d]) * e, __bfloat162float(sm.q[t][d + 1]) * e);
  }
  __syncthreads();                                     // the raw v rows are consumed: their bytes become kgT
  for (int i = tid; i < CK_D * (CK_C / 2); i += 256) {
    const int d = i / (CK_C / 2), j = (i % (CK_C / 2)) * 2;
    const float k0 = __bfloat162float(sm.k[j][d]) * sm.beta[j] * __expf(sm.gc[j]);
    const float k1 = __bfloat162float(sm.k[j + 1][d]) * sm.beta[j + 1] * __expf(sm.gc[j + 1]);
    *reinterpret_cast<uint32_t*>(&sm.kgT[d][j]) = pack_bf16(k0, k1);
  }
  // 3. k k^T and q k^T (64 x 64 x 128): warp -> rows 16 (warp & 3), columns 32 (warp >> 2)
  {
    const int m0 = (warp & 3) * 16, nh = (warp >> 2) * 32;
    float kk[4][4], qk[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) kk[n][i] = qk[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < CK_D / 16; ++ks) {
      uint32_t ak[4], aq[4];
      frag_a(&sm.k[0][0], CK_LD, m0, ks * 16, g, t4, ak);
      frag_a(&sm.q[0][0], CK_LD, m0, ks * 16, g, t4, aq);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        uint32_t b[2];
        frag_b(&sm.k[0][0], CK_LD, nh + n * 8, ks * 16, g, t4, b);
        mma_bf16(kk[n], ak[0], ak[1], ak[2], ak[3], b[0], b[1]);
        mma_bf16(qk[n], aq[0], aq[1], aq[2], aq[3], b[0], b[1]);
      }
    }
    __nv_bfloat16* at = p.attn + ((size_t)h * p.chunks + c) * CK_C * CK_C;
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = m0 + g + half * 8, j = nh + n * 8 + 2 * t4;
        float av[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int jj = j + e;
          const float dec = jj <= i ? __expf(sm.gc[i] - sm.gc[jj]) : 0.f;
          sm.a[i][jj] = jj < i ? sm.beta[i] * kk[n][half * 2 + e] * dec : 0.f;
          av[e] = scale * qk[n][half * 2 + e] * dec;
        }
        *reinterpret_cast<uint32_t*>(at + i * CK_C + j) = pack_bf16(av[0], av[1]);
      }
  }
  __syncthreads();
  // 4. T = (I + A')^-1 by forward substitution: thread c owns column c (rows above the diagonal are zero)
  __nv_bfloat16(*tb)[CK_LT] = reinterpret_cast<__nv_bfloat16(*)[CK_LT]>(&sm.q[0][0]);
  if (tid < CK_C) {
    float col[CK_C];
#pragma unroll
    for (int i = 0; i < CK_C; ++i) {
      float acc = (i == tid) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) acc -= sm.a[i][j] * col[j];
      col[i] = acc;
    }
#pragma unroll
    for (int i = 0; i < CK_C; ++i) tb[i][tid] = __float2bfloat16(col[i]);
  }
  __syncthreads();
  // 5. u = T (beta v), w = T (beta e^{gc} k)  (64 x 128 x 64): warp -> rows 16 (warp & 3), columns 64 (warp >> 2)
  {
    const int m0 = (warp & 3) * 16, nh = (warp >> 2) * 64;
    float uu[8][4], ww[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) uu[n][i] = ww[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < CK_C / 16; ++ks) {
      uint32_t a[4];
      frag_a(&tb[0][0], CK_LT, m0, ks * 16, g, t4, a);
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        uint32_t bv[2], bk[2];
        frag_b(&sm.vbT[0][0], CK_LT, nh + n * 8, ks * 16, g, t4, bv);
        frag_b(&sm.kgT[0][0], CK_LT, nh + n * 8, ks * 16, g, t4, bk);
        mma_bf16(uu[n], a[0], a[1], a[2], a[3], bv[0], bv[1]);
        mma_bf16(ww[n], a[0], a[1], a[2], a[3], bk[0], bk[1]);
      }
    }
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const size_t o = ((size_t)(r0 + m0 + g + half * 8) * p.nv + h) * CK_D + nh + n * 8 + 2 * t4;
        *reinterpret_cast<float2*>(p.u + o) = make_float2(uu[n][half * 2], uu[n][half * 2 + 1]);
        *reinterpret_cast<uint32_t*>(p.w + o) = pack_bf16(ww[n][half * 2], ww[n][half * 2 + 1]);
      }
  }
}

// ---- the recurrence over chunks: one CTA per (v-head, 64 value columns), 256 threads ----------------------------------
struct ScanBuf {
  __nv_bfloat16 w[CK_C][CK_LD];
  __nv_bfloat16 qg[CK_C][CK_LD];
  __nv_bfloat16 kdT[CK_D][CK_LT];
  __nv_bfloat16 attn[CK_C][CK_LT];
  float u[CK_C][CK_NC + 4];         // this CTA's 64 columns (fp32)
};
struct ScanSmem {
  ScanBuf buf[2];
  __nv_bfloat16 sT[CK_NC][CK_LD];   // state^T as bf16: [value column][k]
  __nv_bfloat16 vnT[CK_NC][CK_LT];  // v'^T: [value column][token]
};
__global__ void __launch_bounds__(256) gdn_chunk_scan_kernel(GdnChunkParams p) {
  extern __shared__ __align__(16) uint8_t ck_smem[];
  ScanSmem& sm = *reinterpret_cast<ScanSmem*>(ck_smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  const int h = blockIdx.x, cb = blockIdx.y * CK_NC, V = p.nv * CK_D;
  // state rows 16 warp .. +15, all 64 columns: 8 n-tiles of accumulator registers
  float S[8][4];
  float* sp = p.state + ((size_t)p.slot * p.nv + h) * CK_D * CK_D;
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int k = warp * 16 + g + half * 8, col = cb + n * 8 + 2 * t4;
      S[n][half * 2] = p.use_state ? sp[(size_t)k * CK_D + col] : 0.f;
      S[n][half * 2 + 1] = p.use_state ? sp[(size_t)k * CK_D + col + 1] : 0.f;
    }
  auto issue = [&](int c) {
    if (c < p.chunks) {
      ScanBuf& b = sm.buf[c & 1];
      const int r0 = c * CK_C;
      for (int i = tid; i < CK_C * 16; i += 256) {
        const int t = i >> 4, piece = (i & 15) * 8;
        const size_t o = ((size_t)(r0 + t) * p.nv + h) * CK_D + piece;
        ck_cp16(&b.w[t][piece], p.w + o);
        ck_cp16(&b.qg[t][piece], p.qg + o);
      }
      for (int i = tid; i < CK_C * 8; i += 256) {
        const int t = i >> 3, piece = (i & 7) * 8;
        ck_cp16(&b.attn[t][piece], p.attn + (((size_t)h * p.chunks + c) * CK_C + t) * CK_C + piece);
      }
      for (int i = tid; i < CK_C * 16; i += 256) {
        const int t = i >> 4, piece = (i & 15) * 4;
        ck_cp16(&b.u[t][piece], p.u + ((size_t)(r0 + t) * p.nv + h) * CK_D + cb + piece);
      }
      for (int i = tid; i < CK_D * 8; i += 256) {
        const int d = i >> 3, piece = (i & 7) * 8;
        ck_cp16(&b.kdT[d][piece], p.kdT + (((size_t)h * p.chunks + c) * CK_D + d) * CK_C + piece);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(0);
  for (int c = 0; c < p.chunks; ++c) {
    ScanBuf& b = sm.buf[c & 1];
    const int r0 = c * CK_C;
    // the state as the B operand of this chunk
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int k = warp * 16 + g + half * 8, col = n * 8 + 2 * t4;
        sm.sT[col][k] = __float2bfloat16(S[n][half * 2]);
        sm.sT[col + 1][k] = __float2bfloat16(S[n][half * 2 + 1]);
      }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                 // chunk c and the state copy are visible; everyone is done with chunk c - 1
    issue(c + 1);
    // v' = u - w S and o = qg S: warp -> rows 16 (warp & 3), columns 32 (warp >> 2); K = 128
    const int m0 = (warp & 3) * 16, nh = (warp >> 2) * 32;
    float pv[4][4], ov[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[n][i] = ov[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < CK_D / 16; ++ks) {
      uint32_t aw[4], aq[4];
      frag_a(&b.w[0][0], CK_LD, m0, ks * 16, g, t4, aw);
      frag_a(&b.qg[0][0], CK_LD, m0, ks * 16, g, t4, aq);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        uint32_t bs[2];
        frag_b(&sm.sT[0][0], CK_LD, nh + n * 8, ks * 16, g, t4, bs);
        mma_bf16(pv[n], aw[0], aw[1], aw[2], aw[3], bs[0], bs[1]);
        mma_bf16(ov[n], aq[0], aq[1], aq[2], aq[3], bs[0], bs[1]);
      }
    }
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = m0 + g + half * 8, col = nh + n * 8 + 2 * t4;
        const float2 uw = *reinterpret_cast<const float2*>(&b.u[i][col]);
        sm.vnT[col][i] = __float2bfloat16(uw.x - pv[n][half * 2]);
        sm.vnT[col + 1][i] = __float2bfloat16(uw.y - pv[n][half * 2 + 1]);
      }
    __syncthreads();
    // o += attn v'  (K = 64 tokens)
#pragma unroll
    for (int ks = 0; ks < CK_C / 16; ++ks) {
      uint32_t a[4];
      frag_a(&b.attn[0][0], CK_LT, m0, ks * 16, g, t4, a);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        uint32_t bv[2];
        frag_b(&sm.vnT[0][0], CK_LT, nh + n * 8, ks * 16, g, t4, bv);
        mma_bf16(ov[n], a[0], a[1], a[2], a[3], bv[0], bv[1]);
      }
    }
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = r0 + m0 + g + half * 8;
        if (r < p.T)
          *reinterpret_cast<float2*>(p.raw + (size_t)r * V + h * CK_D + cb + nh + n * 8 + 2 * t4) =
              make_float2(ov[n][half * 2], ov[n][half * 2 + 1]);
      }
    // S <- e^{gc_last} S + (e^{gc_last - gc} k)^T v': warp -> state rows 16 warp .. +15, all 64 columns
    const float eg = p.eglast[(size_t)h * p.chunks + c];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) S[n][i] *= eg;
#pragma unroll
    for (int ks = 0; ks < CK_C / 16; ++ks) {
      uint32_t a[4];
      frag_a(&b.kdT[0][0], CK_LT, warp * 16, ks * 16, g, t4, a);
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        uint32_t bv[2];
        frag_b(&sm.vnT[0][0], CK_LT, n * 8, ks * 16, g, t4, bv);
        mma_bf16(S[n], a[0], a[1], a[2], a[3], bv[0], bv[1]);
      }
    }
    __syncthreads();                 // all reads of sT and vnT are done before the next chunk rewrites them
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int k = warp * 16 + g + half * 8, col = cb + n * 8 + 2 * t4;
      *reinterpret_cast<float2*>(sp + (size_t)k * CK_D + col) = make_float2(S[n][half * 2], S[n][half * 2 + 1]);
    }
}

}  // namespace owl
using namespace owl;

static long long ck_work_bytes(int T, int nv) {
  const long long chunks = (T + CK_C - 1) / CK_C, tpad = chunks * CK_C;
  return tpad * nv * CK_D * 2 * 4 + (long long)nv * chunks * CK_D * CK_C * 2 + (long long)nv * chunks * CK_C * CK_C * 2 +
         (long long)nv * chunks * 4 + 1024;
}
// Bytes of the work buffer for T tokens and nv value heads -> *out_bytes (long long).
OWL_API int owl_gdn_chunk_work_bytes(int T, int nv, void* out_bytes) {
  if (T < 1 || nv < 1 || !out_bytes) return OWL_ERR_BAD_ARG;
  *reinterpret_cast<long long*>(out_bytes) = ck_work_bytes(T, nv);
  return OWL_OK;
}

// raw: float [T][nv * 128] (un-normalised outputs, input of the gated norm); work: owl_gdn_chunk_work_bytes(T, nv) bytes.
OWL_API int owl_gdn_chunk_scan(const void* qkv, const void* ab, int ldab, const void* a_log, const void* dt_bias, void* state,
                               int slot, void* raw, void* work, long long work_bytes, int T, int nk, int nv, int use_state,
                               cudaStream_t st) {
  if (T < 1 || nk < 1 || nv % nk || !raw || !work || work_bytes < ck_work_bytes(T, nv) ||
      (reinterpret_cast<uintptr_t>(work) & 255))
    return OWL_ERR_BAD_ARG;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(PrepSmem)) != cudaSuccess ||
        cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ScanSmem)) != cudaSuccess)
      return OWL_ERR_LAUNCH * 1000;
    attr = true;
  }
  GdnChunkParams p = {};
  p.qkv = (const __nv_bfloat16*)qkv; p.ab = (const __nv_bfloat16*)ab; p.a_log = (const float*)a_log; p.dt_bias = (const float*)dt_bias;
  p.state = (float*)state; p.raw = (float*)raw; p.ldab = ldab; p.nk = nk; p.nv = nv; p.T = T; p.slot = slot; p.use_state = use_state;
  p.chunks = (T + CK_C - 1) / CK_C;
  const size_t tpad = (size_t)p.chunks * CK_C, rows = tpad * nv * CK_D;
  auto* base = reinterpret_cast<__nv_bfloat16*>(work);
  p.u = reinterpret_cast<float*>(base);                 // 2 * rows bf16-sized elements
  p.w = base + 2 * rows; p.qg = base + 3 * rows;
  p.kdT = base + 4 * rows;
  p.attn = p.kdT + (size_t)nv * p.chunks * CK_D * CK_C;
  p.eglast = reinterpret_cast<float*>(p.attn + (size_t)nv * p.chunks * CK_C * CK_C);
  gdn_chunk_prep_kernel<<<dim3(p.chunks, nv), 256, sizeof(PrepSmem), st>>>(p);
  OWL_LAUNCH_CHECK();
  gdn_chunk_scan_kernel<<<dim3(nv, CK_D / CK_NC), 256, sizeof(ScanSmem), st>>>(p);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
