// Weight-streaming "skinny" GEMMs for decode / verify / small-batch steps (M <= 32 tokens).
//
//   owl_w4a16_skinny : C[M,N] = X[M,K] . dequant(W4)[N,K]^T   (int4, group 32/128, asymmetric)
//   owl_bf16_skinny  : C[M,N] = X[M,K] . W[N,K]^T             (dense bf16 weights)
//   owl_w8a16_skinny : C[M,N] = X[M,K] . (s[n] * W8[N,K])^T   (int8 rows with one scale per row)
//
// These ops are bound by HBM bandwidth, not math: each weight byte is read exactly once, by
// 16-byte streaming loads that bypass L1, with several tiles in flight per warp. The
// contraction itself runs on the warp-level tensor-core path (m16n8k16, fp32 accumulate) so
// that 1..8 tokens cost the same issue slots as one; the weight tile is the 16-row A operand
// and the tokens are the 8-column B operand.
//
// Role in the reference: replaces the Marlin W4A16 decode path and the int8-row / f16 GEMV
// family (crates/kernels/cu/marlin/*, crates/kernels/cu/elems/gemv_i8w_*.cu,
// crates/kernels/cu/elems/gemv_dual_f16.cu).
//
// ---- W4 tile layout ("skinny tiles", produced by the load-time repacker) ---------------
// tile(nt, kt) covers rows nt*16..nt*16+15 and k = kt*128..kt*128+127 and is 64 x uint4:
//   uint4 #L       (L = g*4 + t): row nt*16 + g    ; word w, nibble i <-> k = kt*128 + w*32 + t*8 + i
//   uint4 #(32+L)               : row nt*16 + 8 + g; same k mapping
// tiles are stored [N/16][K/128] so a warp that walks K reads one contiguous stream.
// (scale, zero) pairs are half2 at sz[((nt*KG) + kg)*16 + r], kg = k / G.
//
// ---- activation pack ("ActPack") ----------------------------------------------------------
// The int4 -> fp16 conversion uses the exponent-bias trick: (q & 0x000F000F) | 0x64006400 is
// the half2 (1024+q_lo, 1024+q_hi), and the same with mask 0x00F000F0 is (1024+16 q, ...).
// Instead of subtracting the bias and rescaling per weight, the producer of the activations
// stores them pre-permuted and pre-scaled as fp16:
//   per 8 consecutive k: [x0, x4, x1/16, x5/16, x2, x6, x3/16, x7/16]
// plus per (token, group) two fp32 sums: xsum = sum of effective x, xoff = 1024 * sum of the
// stored halves. Then  sum_k (q_k - z) x_k = acc - xoff - z * xsum  exactly (fp32 accumulate).
#include "common.cuh"

namespace owl {

__device__ __forceinline__ void mma_f16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
  return r;
}

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU_MUL = 2, EPI_F32 = 3 };

struct SkinnyParams {
  const uint4* w;        // weight stream (layout depends on kernel)
  const uint32_t* sz;    // w4: half2 (scale, zero) table; w8: float per-row scale; bf16: unused
  const uint4* x;        // w4: ActPack fp16 [M][K]; bf16/w8: bf16 activations [M][K]
  const float2* xs;      // w4: (xsum, xoff) [M][K/G]
  void* out;             // bf16 [M][ldo] (or fp32 for EPI_F32)
  const __nv_bfloat16* residual;  // EPI_RESIDUAL: out = residual + y (may alias out)
  int M, N, K;
  int ldo;               // output row stride in elements
  int n_tiles;           // N / 16
  int ks;                // K slices per row tile (warps of one CTA that split K)
};

constexpr int SK_WARPS = 8;
constexpr int SK_DEPTH = 4;  // weight tiles in flight per warp

template <int MT>
__device__ __forceinline__ void skinny_epilogue(const SkinnyParams& p, float (&acc)[MT][4], int nt, int ks_idx,
                                                int rt_local, float* red, int epi) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int KS = p.ks;
  if (KS > 1) {
    // red[warp][lane][MT*4]; slice 0 of each row tile sums the others in a fixed order.
    float* mine = red + ((size_t)(threadIdx.x >> 5) * 32 + lane) * (MT * 4);
    if (ks_idx != 0) {
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) mine[m * 4 + i] = acc[m][i];
    }
    __syncthreads();
    if (ks_idx == 0) {
      for (int s = 1; s < KS; ++s) {
        const float* o = red + ((size_t)(rt_local * KS + s) * 32 + lane) * (MT * 4);
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[m][i] += o[m * 4 + i];
      }
    }
  }
  if (ks_idx != 0 || nt >= p.n_tiles) return;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int tok = m * 8 + 2 * t + j;
      if (tok >= p.M) continue;
      const float v_lo = acc[m][j], v_hi = acc[m][2 + j];  // rows g and g+8
      if (epi == EPI_SILU_MUL) {
        // row g = gate_j, row g+8 = up_j of output column nt*8+g
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)tok * p.ldo + nt * 8 + g;
        *o = __float2bfloat16(silu_f(v_lo) * v_hi);
      } else if (epi == EPI_F32) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)tok * p.ldo + nt * 16 + g;
        o[0] = v_lo; o[8] = v_hi;
      } else {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)tok * p.ldo + nt * 16 + g;
        float a = v_lo, b = v_hi;
        if (epi == EPI_RESIDUAL) {
          const __nv_bfloat16* r = p.residual + (size_t)tok * p.ldo + nt * 16 + g;
          a += __bfloat162float(r[0]); b += __bfloat162float(r[8]);
        }
        o[0] = __float2bfloat16(a); o[8] = __float2bfloat16(b);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// W4A16
// ------------------------------------------------------------------------------------------
template <int MT, int G>
__global__ void __launch_bounds__(SK_WARPS * 32) w4a16_skinny_kernel(SkinnyParams p, int epi) {
  __shared__ float red[SK_WARPS * 32 * MT * 4];
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int KS = p.ks, rt_per_cta = SK_WARPS / KS;
  const int ks_idx = wi % KS, rt_local = wi / KS;
  const int nt = blockIdx.x * rt_per_cta + rt_local;
  const int KT = p.K >> 7;
  constexpr int GPT = 128 / G;  // groups per tile
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;

  if (nt < p.n_tiles) {
    const int kt0 = (int)((long long)ks_idx * KT / KS), kt1 = (int)((long long)(ks_idx + 1) * KT / KS);
    const uint4* wp = p.w + ((size_t)nt * KT + kt0) * 64 + lane;
    const uint32_t* szp = p.sz + ((size_t)nt * KT + kt0) * GPT * 16 + g;
    uint4 wlo[SK_DEPTH], whi[SK_DEPTH];
    uint32_t sz0[SK_DEPTH][GPT], sz1[SK_DEPTH][GPT];
    // Prologue: weights do not depend on the previous kernel, start streaming before the
    // programmatic-dependency wait.
#pragma unroll
    for (int d = 0; d < SK_DEPTH; ++d) {
      if (kt0 + d < kt1) {
        wlo[d] = ldg_stream(wp + (size_t)d * 64);
        whi[d] = ldg_stream(wp + (size_t)d * 64 + 32);
#pragma unroll
        for (int q = 0; q < GPT; ++q) {
          sz0[d][q] = ldg_stream_u32(szp + ((size_t)d * GPT + q) * 16);
          sz1[d][q] = ldg_stream_u32(szp + ((size_t)d * GPT + q) * 16 + 8);
        }
      }
    }
    pdl_wait();
    const int KG = p.K / G;
    for (int kt = kt0; kt < kt1; kt += SK_DEPTH) {
#pragma unroll
      for (int d = 0; d < SK_DEPTH; ++d) {
        const int k = kt + d;
        if (k < kt1) {
          // B fragments (activations) for this tile: 4 words x MT token blocks.
          uint4 xb[MT][4];
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const int tok = m * 8 + g;
            if (tok < p.M) {
              const uint4* xp = p.x + ((size_t)tok * p.K + (size_t)k * 128) / 8 + t;
#pragma unroll
              for (int w = 0; w < 4; ++w) xb[m][w] = __ldg(xp + w * 4);
            } else {
#pragma unroll
              for (int w = 0; w < 4; ++w) xb[m][w] = make_uint4(0, 0, 0, 0);
            }
          }
          const uint32_t ql[4] = {wlo[d].x, wlo[d].y, wlo[d].z, wlo[d].w};
          const uint32_t qh[4] = {whi[d].x, whi[d].y, whi[d].z, whi[d].w};
          uint32_t s0[GPT], s1[GPT];
#pragma unroll
          for (int q = 0; q < GPT; ++q) { s0[q] = sz0[d][q]; s1[q] = sz1[d][q]; }
          // refill this slot
          if (k + SK_DEPTH < kt1) {
            wlo[d] = ldg_stream(wp + (size_t)(k - kt0 + SK_DEPTH) * 64);
            whi[d] = ldg_stream(wp + (size_t)(k - kt0 + SK_DEPTH) * 64 + 32);
#pragma unroll
            for (int q = 0; q < GPT; ++q) {
              sz0[d][q] = ldg_stream_u32(szp + ((size_t)(k - kt0 + SK_DEPTH) * GPT + q) * 16);
              sz1[d][q] = ldg_stream_u32(szp + ((size_t)(k - kt0 + SK_DEPTH) * GPT + q) * 16 + 8);
            }
          }
          float c[MT][4];
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            if (w == 0 || G == 32) {
#pragma unroll
              for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int i = 0; i < 4; ++i) c[m][i] = 0.f;
            }
            const uint32_t a0 = lop3_and_or(ql[w], 0x000F000Fu, 0x64006400u);
            const uint32_t a2 = lop3_and_or(ql[w], 0x00F000F0u, 0x64006400u);
            const uint32_t a1 = lop3_and_or(qh[w], 0x000F000Fu, 0x64006400u);
            const uint32_t a3 = lop3_and_or(qh[w], 0x00F000F0u, 0x64006400u);
            const uint32_t ql8 = ql[w] >> 8, qh8 = qh[w] >> 8;
            const uint32_t e0 = lop3_and_or(ql8, 0x000F000Fu, 0x64006400u);
            const uint32_t e2 = lop3_and_or(ql8, 0x00F000F0u, 0x64006400u);
            const uint32_t e1 = lop3_and_or(qh8, 0x000F000Fu, 0x64006400u);
            const uint32_t e3 = lop3_and_or(qh8, 0x00F000F0u, 0x64006400u);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              mma_f16_16816(c[m], a0, a1, a2, a3, xb[m][w].x, xb[m][w].y);
              mma_f16_16816(c[m], e0, e1, e2, e3, xb[m][w].z, xb[m][w].w);
            }
            if (w == 3 || G == 32) {
              const int q = (G == 32) ? w : 0;
              const __half2 h0 = *reinterpret_cast<const __half2*>(&s0[q]);
              const __half2 h1 = *reinterpret_cast<const __half2*>(&s1[q]);
              const float sc0 = __low2float(h0), z0 = __high2float(h0);
              const float sc1 = __low2float(h1), z1 = __high2float(h1);
              const int kg = k * GPT + q;
#pragma unroll
              for (int m = 0; m < MT; ++m) {
                const int tokA = m * 8 + 2 * t;
                float2 sa = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
                if (tokA < p.M) sa = __ldg(p.xs + (size_t)tokA * KG + kg);
                if (tokA + 1 < p.M) sb = __ldg(p.xs + (size_t)(tokA + 1) * KG + kg);
                acc[m][0] += sc0 * (c[m][0] - sa.y - z0 * sa.x);
                acc[m][1] += sc0 * (c[m][1] - sb.y - z0 * sb.x);
                acc[m][2] += sc1 * (c[m][2] - sa.y - z1 * sa.x);
                acc[m][3] += sc1 * (c[m][3] - sb.y - z1 * sb.x);
              }
            }
          }
        }
      }
    }
  } else {
    pdl_wait();
  }
  pdl_launch_dependents();
  skinny_epilogue<MT>(p, acc, nt, ks_idx, rt_local, red, epi);
}

// ------------------------------------------------------------------------------------------
// Dense bf16 weights [N][K] row-major, and int8 rows with per-row fp32 scale.
// Thread (g,t) loads 16 bytes of row g and of row g+8 per 32(bf16)/64(int8)-wide k step; the
// same 8 (16) consecutive k of the token row form the B fragments, so no permutation is needed.
// ------------------------------------------------------------------------------------------
template <int MT, bool W8>
__global__ void __launch_bounds__(SK_WARPS * 32) dense_skinny_kernel(SkinnyParams p, int epi) {
  __shared__ float red[SK_WARPS * 32 * MT * 4];
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int KS = p.ks, rt_per_cta = SK_WARPS / KS;
  const int ks_idx = wi % KS, rt_local = wi / KS;
  const int nt = blockIdx.x * rt_per_cta + rt_local;
  constexpr int KSTEP = W8 ? 64 : 32;           // k covered by one 16-byte load across t = 0..3
  const int KT = p.K / KSTEP;
  const size_t row_u4 = (size_t)p.K / (W8 ? 16 : 8);  // uint4 per weight row
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;

  if (nt < p.n_tiles) {
    const int kt0 = (int)((long long)ks_idx * KT / KS), kt1 = (int)((long long)(ks_idx + 1) * KT / KS);
    const uint4* w0 = p.w + (size_t)(nt * 16 + g) * row_u4 + (size_t)kt0 * 4 + t;
    const uint4* w1 = w0 + 8 * row_u4;
    constexpr int D = 6;
    uint4 wlo[D], whi[D];
#pragma unroll
    for (int d = 0; d < D; ++d)
      if (kt0 + d < kt1) { wlo[d] = ldg_stream(w0 + d * 4); whi[d] = ldg_stream(w1 + d * 4); }
    pdl_wait();
    for (int kt = kt0; kt < kt1; kt += D) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        const int k = kt + d;
        if (k < kt1) {
          const uint4 a = wlo[d], b = whi[d];
          if (k + D < kt1) {
            wlo[d] = ldg_stream(w0 + (size_t)(k - kt0 + D) * 4);
            whi[d] = ldg_stream(w1 + (size_t)(k - kt0 + D) * 4);
          }
          if (!W8) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const int tok = m * 8 + g;
              uint4 xb = make_uint4(0, 0, 0, 0);
              if (tok < p.M) xb = __ldg(p.x + ((size_t)tok * p.K + (size_t)k * 32) / 8 + t);
              mma_bf16_16816(acc[m], a.x, b.x, a.y, b.y, xb.x, xb.y);
              mma_bf16_16816(acc[m], a.z, b.z, a.w, b.w, xb.z, xb.w);
            }
          } else {
            // int8 -> fp16 by byte permute: (w ^ 0x80) is the biased byte b = w + 128, and the
            // half with bit pattern 0x6400 | b equals 1024 + b; subtracting 1152 restores w exactly.
            const uint32_t al[4] = {a.x ^ 0x80808080u, a.y ^ 0x80808080u, a.z ^ 0x80808080u, a.w ^ 0x80808080u};
            const uint32_t bl[4] = {b.x ^ 0x80808080u, b.y ^ 0x80808080u, b.z ^ 0x80808080u, b.w ^ 0x80808080u};
            const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
            auto cvt = [&](uint32_t v, uint32_t sel) -> uint32_t {
              uint32_t r = __byte_perm(v, 0x64646464u, sel);
              __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r), bias);
              return *reinterpret_cast<uint32_t*>(&h);
            };
            auto x16 = [&](uint32_t v) -> uint32_t { return pack_f16(bf16_lo(v), bf16_hi(v)); };
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t fa[4], fb[4];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                fa[u * 2 + 0] = cvt(al[h * 2 + u], 0x4140u);
                fa[u * 2 + 1] = cvt(al[h * 2 + u], 0x4342u);
                fb[u * 2 + 0] = cvt(bl[h * 2 + u], 0x4140u);
                fb[u * 2 + 1] = cvt(bl[h * 2 + u], 0x4342u);
              }
#pragma unroll
              for (int m = 0; m < MT; ++m) {
                const int tok = m * 8 + g;
                uint4 xv = make_uint4(0, 0, 0, 0);
                if (tok < p.M) xv = __ldg(p.x + ((size_t)tok * p.K + (size_t)k * 64) / 8 + t * 2 + h);
                mma_f16_16816(acc[m], fa[0], fb[0], fa[1], fb[1], x16(xv.x), x16(xv.y));
                mma_f16_16816(acc[m], fa[2], fb[2], fa[3], fb[3], x16(xv.z), x16(xv.w));
              }
            }
          }
        }
      }
    }
    if (W8) {
      const float* rs = reinterpret_cast<const float*>(p.sz);
      const float s0 = rs[nt * 16 + g], s1 = rs[nt * 16 + g + 8];
#pragma unroll
      for (int m = 0; m < MT; ++m) { acc[m][0] *= s0; acc[m][1] *= s0; acc[m][2] *= s1; acc[m][3] *= s1; }
    }
  } else {
    pdl_wait();
  }
  pdl_launch_dependents();
  skinny_epilogue<MT>(p, acc, nt, ks_idx, rt_local, red, epi);
}

// Split-K factor: keep at least ~2 waves of 8-warp CTAs in flight when N is small.
static int pick_ks(int n_tiles, int k_units) {
  int ks = 1;
  while (ks < SK_WARPS && (long long)n_tiles * ks < 148LL * 16 && (k_units / (ks * 2)) >= 4) ks *= 2;
  return ks;
}

template <typename K>
static int launch_skinny(K kernel, const SkinnyParams& p, int epi, int pdl, cudaStream_t st) {
  const int rt_per_cta = SK_WARPS / p.ks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.n_tiles + rt_per_cta - 1) / rt_per_cta);
  cfg.blockDim = dim3(SK_WARPS * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p, epi);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

}  // namespace owl

using namespace owl;

// out[M, ldo] (bf16, or fp32 with epi=3). group is 32 or 128. epi: 0 store, 1 residual add,
// 2 silu(gate)*up with gate/up rows interleaved per 16-row tile (rows 0-7 gate, 8-15 up), 3 fp32 store.
OWL_API int owl_w4a16_skinny(const void* wtiles, const void* sz, const void* xpack, const void* xsums, void* out,
                             const void* residual, int M, int N, int K, int ldo, int group, int epi, int ks,
                             int pdl, cudaStream_t st) {
  if (M < 1 || M > 32 || (N & 15) || (K & 127) || (group != 32 && group != 128)) return OWL_ERR_BAD_ARG;
  SkinnyParams p;
  p.w = (const uint4*)wtiles; p.sz = (const uint32_t*)sz; p.x = (const uint4*)xpack; p.xs = (const float2*)xsums;
  p.out = out; p.residual = (const __nv_bfloat16*)residual; p.M = M; p.N = N; p.K = K; p.ldo = ldo;
  p.n_tiles = N / 16;
  p.ks = ks > 0 ? ks : pick_ks(p.n_tiles, K / 128);
  if (p.ks != 1 && p.ks != 2 && p.ks != 4 && p.ks != 8) return OWL_ERR_BAD_ARG;
  const int mt = (M + 7) / 8;
#define OWL_W4_CASE(MTV)                                                                        \
  return group == 128 ? launch_skinny(w4a16_skinny_kernel<MTV, 128>, p, epi, pdl, st)           \
                      : launch_skinny(w4a16_skinny_kernel<MTV, 32>, p, epi, pdl, st)
  if (mt == 1) { OWL_W4_CASE(1); }
  if (mt == 2) { OWL_W4_CASE(2); }
  OWL_W4_CASE(4);
#undef OWL_W4_CASE
}

OWL_API int owl_bf16_skinny(const void* w, const void* x, void* out, const void* residual, int M, int N, int K,
                            int ldo, int epi, int ks, int pdl, cudaStream_t st) {
  if (M < 1 || M > 32 || (N & 15) || (K & 31)) return OWL_ERR_BAD_ARG;
  SkinnyParams p;
  p.w = (const uint4*)w; p.sz = nullptr; p.x = (const uint4*)x; p.xs = nullptr; p.out = out;
  p.residual = (const __nv_bfloat16*)residual; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.n_tiles = N / 16;
  p.ks = ks > 0 ? ks : pick_ks(p.n_tiles, K / 32);
  if (p.ks != 1 && p.ks != 2 && p.ks != 4 && p.ks != 8) return OWL_ERR_BAD_ARG;
  const int mt = (M + 7) / 8;
  if (mt == 1) return launch_skinny(dense_skinny_kernel<1, false>, p, epi, pdl, st);
  if (mt == 2) return launch_skinny(dense_skinny_kernel<2, false>, p, epi, pdl, st);
  return launch_skinny(dense_skinny_kernel<4, false>, p, epi, pdl, st);
}

OWL_API int owl_w8a16_skinny(const void* w, const void* row_scale, const void* x, void* out, int M, int N, int K,
                             int ldo, int epi, int ks, int pdl, cudaStream_t st) {
  if (M < 1 || M > 32 || (N & 15) || (K & 63)) return OWL_ERR_BAD_ARG;
  SkinnyParams p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)row_scale; p.x = (const uint4*)x; p.xs = nullptr; p.out = out;
  p.residual = nullptr; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.n_tiles = N / 16;
  p.ks = ks > 0 ? ks : pick_ks(p.n_tiles, K / 64);
  if (p.ks != 1 && p.ks != 2 && p.ks != 4 && p.ks != 8) return OWL_ERR_BAD_ARG;
  const int mt = (M + 7) / 8;
  if (mt == 1) return launch_skinny(dense_skinny_kernel<1, true>, p, epi, pdl, st);
  if (mt == 2) return launch_skinny(dense_skinny_kernel<2, true>, p, epi, pdl, st);
  return launch_skinny(dense_skinny_kernel<4, true>, p, epi, pdl, st);
}
