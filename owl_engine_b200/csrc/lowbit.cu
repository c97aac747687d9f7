// Other weight formats on the device: NVFP4 (block-scaled e2m1) and the GGUF block quantisations.
//
//   owl_nvfp4_gemv        out[M,N] = alpha * x[M,K] . dequant(W)[N,K]^T   for M <= 8 (decode): one warp per
//                          output row streams 16 codes + 1 scale per lane step, fp32 accumulate
//   owl_nvfp4_dequant     W -> bf16 [N,K] (prefill: feeds the dense tcgen05 GEMM; load-time checks)
//   owl_nvfp4_quant_act   x bf16 [M,K] -> codes + e4m3 block scales with a given global scale (W4A4 operand)
//   owl_gguf_dequant      GGUF blocks (Q8_0, Q4_0/1, Q5_0/1, Q2_K .. Q6_K, IQ4_NL, IQ4_XS, IQ3_XXS, IQ3_S) -> bf16; with a row index
//                          list it is the quantised embedding-table lookup
//   owl_gguf_gemv         out[M,N] = x[M,K] . dequant(blocks)[N,K]^T for M <= 8: one warp per output row,
//                          dequantisation in registers (no dense copy of the weight)
//
// Numerics mirror the host codecs (formats/nvfp4.py, formats/gguf.py), which the tests use as oracles.
//
// Role in the reference: crates/kernels/cu/nvfp4/{nvfp4_gemv,nvfp4_quant_act}.cu,
// cu/gguf/{gguf_gemm,gguf_rows,gguf_smem}.cu.
#include <cuda_fp8.h>
#include "common.cuh"
#include "actpack.cuh"

namespace owl {

// ---- e2m1 / e4m3 ---------------------------------------------------------------------------------
__device__ __forceinline__ float e2m1_to_float(uint32_t c) {       // c: 4 bits, sign | exp(2) | man(1)
  const uint32_t e = (c >> 1) & 3u, m = c & 1u;
  const float mag = e == 0 ? 0.5f * (float)m : __uint_as_float(((e + 126u) << 23) | (m << 22));
  return (c & 8u) ? -mag : mag;
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __nv_fp8_e4m3 v;
  v.__x = b;
  return (float)v;
}
__device__ __forceinline__ uint32_t float_to_e2m1(float x) {       // round to nearest representable magnitude
  const float a = fabsf(x);
  const uint32_t mag = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
  return mag | (x < 0.f ? 8u : 0u);
}

// grid (ceil(N / 8)), block 256: warp w of the CTA owns row blockIdx.x * 8 + w
template <int MT>
__global__ void __launch_bounds__(256) nvfp4_gemv_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf,
                                                         float alpha, const __nv_bfloat16* __restrict__ x, int ldx,
                                                         __nv_bfloat16* out, int ldo, const __nv_bfloat16* residual,
                                                         const float* __restrict__ row_scale, int M, int N, int K) {
  const int lane = threadIdx.x & 31, n = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (n >= N) return;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  const uint8_t* wrow = codes + (size_t)n * (K >> 1);
  const uint8_t* srow = sf + (size_t)n * (K >> 4);
  for (int b = lane; b < (K >> 4); b += 32) {                 // one 16-element block per lane step
    const uint2 q = *reinterpret_cast<const uint2*>(wrow + b * 8);
    const float s = e4m3_to_float(srow[b]);
    float w[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      w[i] = e2m1_to_float((q.x >> (4 * i)) & 15u) * s;
      w[8 + i] = e2m1_to_float((q.y >> (4 * i)) & 15u) * s;
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m >= M) break;
      const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)m * ldx + b * 16);
      float xv[16];
      unpack_bf16x8(xp[0], xv);
      unpack_bf16x8(xp[1], xv + 8);
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[m] = fmaf(w[i], xv[i], acc[m]);
    }
  }
  const float a = row_scale ? alpha * row_scale[n] : alpha;     // merged projections keep one per-tensor scale per row
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m < M)
      out[(size_t)m * ldo + n] = __float2bfloat16(v * a + (residual ? __bfloat162float(residual[(size_t)m * ldo + n]) : 0.f));
  }
}

// x = sx * (128 h + l) per element; chunk byte order as written by actpack_emit
__global__ void __launch_bounds__(256) act_unpack_kernel(const uint4* __restrict__ xpack, const float2* __restrict__ xs,
                                                         __nv_bfloat16* __restrict__ out, int ldo, int nchunks, int cpg, int out_f16) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (c >= nchunks) return;
  const uint4 pk = xpack[(size_t)row * nchunks + c];
  const float sx = xs[(size_t)row * (nchunks / cpg) + c / cpg].x;
  const int klo[4] = {0, 4, 1, 5}, khi[4] = {2, 6, 3, 7};
  float v[8];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int hl = (int)(int8_t)((pk.x >> (8 * b)) & 0xff), ll = (int)((pk.y >> (8 * b)) & 0x7f);
    const int hb = (int)(int8_t)((pk.z >> (8 * b)) & 0xff), lb = (int)((pk.w >> (8 * b)) & 0x7f);
    v[klo[b]] = sx * (float)(hl * 128 + ll);
    v[khi[b]] = sx * (float)(hb * 128 + lb);
  }
  if (out_f16) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = clamp_h(v[i]);
  }
  *reinterpret_cast<uint4*>(out + (size_t)row * ldo + c * 8) = out_f16 ? pack_f16x8(v) : pack_bf16x8(v);
}

// out[m][n] = a[m][n] + b[m][n] (bf16 rows with leading dimensions; the residual epilogue of the GEMM arms)
__global__ void __launch_bounds__(256) add_rows_kernel(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ b,
                                                       int ldb, __nv_bfloat16* __restrict__ out, int ldo, int n8) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (c >= n8) return;
  float x[8], y[8];
  unpack_bf16x8(*reinterpret_cast<const uint4*>(a + (size_t)row * lda + c * 8), x);
  unpack_bf16x8(*reinterpret_cast<const uint4*>(b + (size_t)row * ldb + c * 8), y);
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] += y[i];
  *reinterpret_cast<uint4*>(out + (size_t)row * ldo + c * 8) = pack_bf16x8(x);
}

__global__ void __launch_bounds__(256) nvfp4_dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf,
                                                            float alpha, __nv_bfloat16* out, size_t n_blocks,
                                                            const float* __restrict__ row_scale, int blocks_per_row) {
  const size_t b = (size_t)blockIdx.x * 256 + threadIdx.x;     // one 16-element block per thread
  if (b >= n_blocks) return;
  const uint2 q = *reinterpret_cast<const uint2*>(codes + b * 8);
  const float s = e4m3_to_float(sf[b]) * alpha * (row_scale ? row_scale[b / blocks_per_row] : 1.f);
  float w[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[i] = e2m1_to_float((q.x >> (4 * i)) & 15u) * s;
    w[8 + i] = e2m1_to_float((q.y >> (4 * i)) & 15u) * s;
  }
  uint4* o = reinterpret_cast<uint4*>(out + b * 16);
  o[0] = make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]), pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
  o[1] = make_uint4(pack_bf16(w[8], w[9]), pack_bf16(w[10], w[11]), pack_bf16(w[12], w[13]), pack_bf16(w[14], w[15]));
}

// one 16-element block per thread: block scale = amax / 6 / global (e4m3), codes = round(x / (scale * global))
__global__ void __launch_bounds__(256) nvfp4_quant_kernel(const __nv_bfloat16* __restrict__ x, float global_scale,
                                                          uint8_t* codes, uint8_t* sf, size_t n_blocks) {
  const size_t b = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (b >= n_blocks) return;
  const uint4* xp = reinterpret_cast<const uint4*>(x + b * 16);
  float v[16];
  unpack_bf16x8(xp[0], v);
  unpack_bf16x8(xp[1], v + 8);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float bs = fminf(amax / 6.f / global_scale, 448.f);
  const __nv_fp8_e4m3 s8(bs);
  sf[b] = s8.__x;
  const float inv = 1.f / (fmaxf((float)s8, 0.001953125f) * global_scale);
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    lo |= float_to_e2m1(v[i] * inv) << (4 * i);
    hi |= float_to_e2m1(v[8 + i] * inv) << (4 * i);
  }
  *reinterpret_cast<uint2*>(codes + b * 8) = make_uint2(lo, hi);
}

// ---- GGUF blocks ------------------------------------------------------------------------------------
enum { GG_Q8_0 = 8, GG_Q4_0 = 2, GG_Q4_1 = 3, GG_Q5_0 = 6, GG_Q5_1 = 7, GG_Q2_K = 10, GG_Q3_K = 11, GG_Q4_K = 12, GG_Q5_K = 13,
       GG_Q6_K = 14, GG_IQ3_XXS = 18, GG_IQ4_NL = 20, GG_IQ3_S = 21, GG_IQ4_XS = 23 };

// Codebooks of the IQ3 types (four magnitudes per entry), uploaded once by owl_gguf_set_grids from the host tables.
__device__ uint32_t g_iq3xxs_grid[256];
__device__ uint32_t g_iq3s_grid[512];
__device__ __forceinline__ uint8_t ksign7(int i) { return (uint8_t)(i | ((__popc(i) & 1) << 7)); }   // 7 sign bits + even parity

__device__ __constant__ int8_t c_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

__device__ __forceinline__ float f16_at(const uint8_t* p) {
  return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}
__device__ __forceinline__ void k_scale_min(const uint8_t* sc, int j, float& s, float& m) {   // 12 packed bytes -> pair j
  if (j < 4) { s = (float)(sc[j] & 63); m = (float)(sc[j + 4] & 63); }
  else { s = (float)((sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4)); m = (float)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)); }
}

__host__ __device__ __forceinline__ bool gguf_geom(int type, int& elems, int& bytes) {
  switch (type) {
    case GG_Q8_0: elems = 32; bytes = 34; return true;
    case GG_Q4_0: elems = 32; bytes = 18; return true;
    case GG_IQ4_NL: elems = 32; bytes = 18; return true;
    case GG_Q4_1: elems = 32; bytes = 20; return true;
    case GG_Q5_0: elems = 32; bytes = 22; return true;
    case GG_Q5_1: elems = 32; bytes = 24; return true;
    case GG_Q2_K: elems = 256; bytes = 84; return true;
    case GG_Q3_K: elems = 256; bytes = 110; return true;
    case GG_IQ3_XXS: elems = 256; bytes = 98; return true;
    case GG_IQ3_S: elems = 256; bytes = 110; return true;
    case GG_Q4_K: elems = 256; bytes = 144; return true;
    case GG_Q5_K: elems = 256; bytes = 176; return true;
    case GG_Q6_K: elems = 256; bytes = 210; return true;
    case GG_IQ4_XS: elems = 256; bytes = 136; return true;
  }
  return false;
}

// Element e (0 .. elems-1) of one block.
__device__ __forceinline__ float gguf_elem(int type, const uint8_t* b, int e) {
  switch (type) {
    case GG_Q8_0: return f16_at(b) * (float)(int8_t)b[2 + e];
    case GG_Q4_0: { const uint8_t q = b[2 + (e & 15)]; return f16_at(b) * (float)((int)(e < 16 ? (q & 0xF) : (q >> 4)) - 8); }
    case GG_IQ4_NL: { const uint8_t q = b[2 + (e & 15)]; return f16_at(b) * (float)c_iq4nl[e < 16 ? (q & 0xF) : (q >> 4)]; }
    case GG_Q4_1: { const uint8_t q = b[4 + (e & 15)]; return f16_at(b) * (float)(e < 16 ? (q & 0xF) : (q >> 4)) + f16_at(b + 2); }
    case GG_Q5_0:
    case GG_Q5_1: {
      const int off = type == GG_Q5_0 ? 2 : 4;
      const uint32_t qh = b[off] | (b[off + 1] << 8) | (b[off + 2] << 16) | ((uint32_t)b[off + 3] << 24);
      const uint8_t q = b[off + 4 + (e & 15)];
      const int v = (e < 16 ? (q & 0xF) : (q >> 4)) | (((qh >> e) & 1) << 4);
      return type == GG_Q5_0 ? f16_at(b) * (float)(v - 16) : f16_at(b) * (float)v + f16_at(b + 2);
    }
    case GG_Q2_K: {
      // element e: half h (128), shift pair j, 16-run `half16`; scales[h*8 + j*2 + half16], qs[h*32 + l] >> 2j
      const int h = e >> 7, r = e & 127, j = r >> 5, l = r & 31;
      const uint8_t sc = b[h * 8 + j * 2 + (l >> 4)];
      const int q = (b[16 + h * 32 + l] >> (2 * j)) & 3;
      return f16_at(b + 80) * (float)(sc & 0xF) * (float)q - f16_at(b + 82) * (float)(sc >> 4);
    }
    case GG_Q3_K: {
      const int h = e >> 7, r = e & 127, j = r >> 5, l = r & 31;
      const int is = h * 8 + j * 2 + (l >> 4);                      // one of sixteen 6-bit scales
      const uint8_t* sc = b + 96;
      const int low4 = is < 8 ? (sc[is] & 0xF) : (sc[is - 8] >> 4);
      const int hi2 = (sc[8 + (is & 3)] >> (2 * (is >> 2))) & 3;
      const int scale = (low4 | (hi2 << 4)) - 32;
      const int q = ((b[32 + h * 32 + l] >> (2 * j)) & 3) - ((b[l] & (1 << (h * 4 + j))) ? 0 : 4);
      return f16_at(b + 108) * (float)scale * (float)q;
    }
    case GG_IQ3_XXS: {
      const int ib = e >> 5, r = e & 31, l = r >> 3, jj = r & 7;   // sub-block ib, 8-run l, element jj
      const uint8_t* gas = b + 66 + ib * 4;
      const uint32_t aux = gas[0] | (gas[1] << 8) | (gas[2] << 16) | ((uint32_t)gas[3] << 24);
      const uint32_t grid = g_iq3xxs_grid[b[2 + ib * 8 + 2 * l + (jj >> 2)]];
      const float mag = (float)((grid >> (8 * (jj & 3))) & 0xFF);
      const uint8_t signs = ksign7((aux >> (7 * l)) & 127);
      return f16_at(b) * (0.5f + (float)(aux >> 28)) * 0.5f * mag * ((signs >> jj) & 1 ? -1.f : 1.f);
    }
    case GG_IQ3_S: {
      const int ib = e >> 5, r = e & 31, l = r >> 3, jj = r & 7;
      const int qh = b[66 + ib];
      const int idx = b[2 + ib * 8 + 2 * l + (jj >> 2)] | ((jj < 4 ? (qh << (8 - 2 * l)) : (qh << (7 - 2 * l))) & 256);
      const float mag = (float)((g_iq3s_grid[idx] >> (8 * (jj & 3))) & 0xFF);
      const float d = f16_at(b) * (float)(1 + 2 * ((b[106 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF));
      return d * mag * ((b[74 + ib * 4 + l] >> jj) & 1 ? -1.f : 1.f);
    }
    case GG_Q4_K: {
      const int j = e >> 5, l = e & 31;                 // sub-block j (32 elements): pair (j/2), low nibbles for even j
      float s, m; k_scale_min(b + 4, j, s, m);
      const uint8_t q = b[16 + (j >> 1) * 32 + l];
      return f16_at(b) * s * (float)((j & 1) ? (q >> 4) : (q & 0xF)) - f16_at(b + 2) * m;
    }
    case GG_Q5_K: {
      const int j = e >> 5, l = e & 31;
      float s, m; k_scale_min(b + 4, j, s, m);
      const uint8_t q = b[48 + (j >> 1) * 32 + l];
      const int hi = (b[16 + l] >> j) & 1;
      return f16_at(b) * s * (float)(((j & 1) ? (q >> 4) : (q & 0xF)) + 16 * hi) - f16_at(b + 2) * m;
    }
    case GG_Q6_K: {
      const int h = e >> 7, r = e & 127, part = r >> 5, l = r & 31;     // half h, quarter part, lane l
      const uint8_t* ql = b + h * 64; const uint8_t* qh = b + 128 + h * 32;
      const int lowb = (part & 1) ? ql[32 + l] : ql[l];
      const int q4 = (part & 2) ? (lowb >> 4) : (lowb & 0xF);
      const int q = (q4 | (((qh[l] >> (2 * part)) & 3) << 4)) - 32;
      const float sc = (float)(int8_t)b[192 + h * 8 + (l >> 4) + 2 * part];
      return f16_at(b + 208) * sc * (float)q;
    }
    case GG_IQ4_XS: {
      const int ib = e >> 5, l = e & 31;
      const int sh = b[2] | (b[3] << 8);
      const int ls = ((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
      const uint8_t q = b[8 + ib * 16 + (l & 15)];
      return f16_at(b) * (float)(ls - 32) * (float)c_iq4nl[l < 16 ? (q & 0xF) : (q >> 4)];
    }
  }
  return 0.f;
}

// grid (K / 256 or K / 32 blocks rounded to 256 threads, rows): rows == null -> row r = blockIdx.y
__global__ void __launch_bounds__(256) gguf_dequant_kernel(const uint8_t* __restrict__ blocks, int type, int K,
                                                           const int* __restrict__ rows, __nv_bfloat16* out) {
  int elems, bytes;
  gguf_geom(type, elems, bytes);
  const int k = blockIdx.x * 256 + threadIdx.x;
  if (k >= K) return;
  const int src = rows ? rows[blockIdx.y] : blockIdx.y;
  const uint8_t* b = blocks + ((size_t)src * (K / elems) + k / elems) * bytes;
  out[(size_t)blockIdx.y * K + k] = __float2bfloat16(gguf_elem(type, b, k % elems));
}

template <int MT>
__global__ void __launch_bounds__(256) gguf_gemv_kernel(const uint8_t* __restrict__ blocks, int type,
                                                        const __nv_bfloat16* __restrict__ x, int ldx, __nv_bfloat16* out,
                                                        int ldo, int M, int N, int K) {
  int elems, bytes;
  gguf_geom(type, elems, bytes);
  const int lane = threadIdx.x & 31, n = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (n >= N) return;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  const uint8_t* wrow = blocks + (size_t)n * (K / elems) * bytes;
  for (int k0 = lane * 8; k0 < K; k0 += 256) {           // 8 consecutive k per lane step (inside one block: 8 | 32)
    const uint8_t* b = wrow + (size_t)(k0 / elems) * bytes;
    float w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = gguf_elem(type, b, (k0 % elems) + i);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m >= M) break;
      float xv[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k0), xv);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[m] = fmaf(w[i], xv[i], acc[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m < M) out[(size_t)m * ldo + n] = __float2bfloat16(v);
  }
}

}  // namespace owl
using namespace owl;

static int nvfp4_gemv_launch(const void* codes, const void* sf, float alpha, const void* x, int ldx, void* out, int ldo,
                             const void* residual, int M, int N, int K, cudaStream_t st, const void* row_scale = nullptr) {
  if (M < 1 || M > 8 || N < 1 || (K & 15) || (ldx & 7)) return OWL_ERR_BAD_ARG;
  const dim3 grid((N + 7) / 8);
  const auto *c = (const uint8_t*)codes, *f = (const uint8_t*)sf;
  const auto *xx = (const __nv_bfloat16*)x, *r = (const __nv_bfloat16*)residual;
  const float* rs = (const float*)row_scale;
  if (M == 1) nvfp4_gemv_kernel<1><<<grid, 256, 0, st>>>(c, f, alpha, xx, ldx, (__nv_bfloat16*)out, ldo, r, rs, M, N, K);
  else if (M <= 4) nvfp4_gemv_kernel<4><<<grid, 256, 0, st>>>(c, f, alpha, xx, ldx, (__nv_bfloat16*)out, ldo, r, rs, M, N, K);
  else nvfp4_gemv_kernel<8><<<grid, 256, 0, st>>>(c, f, alpha, xx, ldx, (__nv_bfloat16*)out, ldo, r, rs, M, N, K);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
OWL_API int owl_nvfp4_gemv(const void* codes, const void* sf, float alpha, const void* x, int ldx, void* out, int ldo,
                           int M, int N, int K, cudaStream_t st) {
  return nvfp4_gemv_launch(codes, sf, alpha, x, ldx, out, ldo, nullptr, M, N, K, st);
}
// out = residual + alpha * x . W^T (residual bf16 [M][ldo], may alias out).
OWL_API int owl_nvfp4_gemv_res(const void* codes, const void* sf, float alpha, const void* x, int ldx, void* out, int ldo,
                               const void* residual, int M, int N, int K, cudaStream_t st) {
  if (!residual) return OWL_ERR_BAD_ARG;
  return nvfp4_gemv_launch(codes, sf, alpha, x, ldx, out, ldo, residual, M, N, K, st);
}
// Per-row scales (fp32 [N], multiplied with alpha): rows of a merged projection keep their tensors' own scales.
// residual may be null.
OWL_API int owl_nvfp4_gemv_rows(const void* codes, const void* sf, float alpha, const void* row_scale, const void* x, int ldx,
                                void* out, int ldo, const void* residual, int M, int N, int K, cudaStream_t st) {
  if (!row_scale) return OWL_ERR_BAD_ARG;
  return nvfp4_gemv_launch(codes, sf, alpha, x, ldx, out, ldo, residual, M, N, K, st, row_scale);
}
OWL_API int owl_nvfp4_dequant_rows(const void* codes, const void* sf, float alpha, const void* row_scale, int K, void* out,
                                   long long n_elems, cudaStream_t st) {
  if (n_elems < 16 || (n_elems & 15) || !row_scale || K < 16 || (K & 15)) return OWL_ERR_BAD_ARG;
  const size_t nb = (size_t)n_elems / 16;
  nvfp4_dequant_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, st>>>((const uint8_t*)codes, (const uint8_t*)sf, alpha,
                                                                     (__nv_bfloat16*)out, nb, (const float*)row_scale, K / 16);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
// ActPack rows (15-bit fixed point + per-group scale, row layout) back to bf16 [M][ldo]: the input of the float GEMV arms.
// out: bf16 (out_f16 = 0) or fp16 (out_f16 = 1) [M][ldo].
OWL_API int owl_act_unpack(const void* xpack, const void* xs, void* out, int ldo, int M, int K, int G, int out_f16, cudaStream_t st) {
  if (M < 1 || (K & 7) || (G != 32 && G != 128) || (K % G) || (ldo & 7)) return OWL_ERR_BAD_ARG;
  const int nchunks = K / 8;
  act_unpack_kernel<<<dim3((nchunks + 255) / 256, M), 256, 0, st>>>((const uint4*)xpack, (const float2*)xs, (__nv_bfloat16*)out, ldo,
                                                                     nchunks, G >> 3, out_f16);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
// out = a + b over M rows of N bf16 values (N multiple of 8; out may alias a or b).
OWL_API int owl_add_rows(const void* a, int lda, const void* b, int ldb, void* out, int ldo, int M, int N, cudaStream_t st) {
  if (M < 1 || N < 8 || (N & 7) || (lda & 7) || (ldb & 7) || (ldo & 7)) return OWL_ERR_BAD_ARG;
  add_rows_kernel<<<dim3((N / 8 + 255) / 256, M), 256, 0, st>>>((const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)b, ldb,
                                                               (__nv_bfloat16*)out, ldo, N / 8);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
OWL_API int owl_nvfp4_dequant(const void* codes, const void* sf, float alpha, void* out, long long n_elems, cudaStream_t st) {
  if (n_elems < 16 || (n_elems & 15)) return OWL_ERR_BAD_ARG;
  const size_t nb = (size_t)n_elems / 16;
  nvfp4_dequant_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, st>>>((const uint8_t*)codes, (const uint8_t*)sf, alpha, (__nv_bfloat16*)out, nb,
                                                                     nullptr, 1);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
OWL_API int owl_nvfp4_quant_act(const void* x, float global_scale, void* codes, void* sf, long long n_elems, cudaStream_t st) {
  if (n_elems < 16 || (n_elems & 15) || global_scale <= 0.f) return OWL_ERR_BAD_ARG;
  const size_t nb = (size_t)n_elems / 16;
  nvfp4_quant_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, global_scale, (uint8_t*)codes, (uint8_t*)sf, nb);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
// Uploads the IQ3 codebooks (host tables: 256 and 512 little-endian uint32 entries of four magnitudes) to the current device.
OWL_API int owl_gguf_set_grids(const void* iq3xxs, const void* iq3s) {
  if (!iq3xxs || !iq3s) return OWL_ERR_BAD_ARG;
  if (cudaMemcpyToSymbol(g_iq3xxs_grid, iq3xxs, sizeof(uint32_t) * 256) != cudaSuccess) return OWL_ERR_LAUNCH * 1000;
  if (cudaMemcpyToSymbol(g_iq3s_grid, iq3s, sizeof(uint32_t) * 512) != cudaSuccess) return OWL_ERR_LAUNCH * 1000;
  return OWL_OK;
}

// blocks: [n_src_rows][K / elems] GGUF blocks of `type` (ggml type id). rows: optional int32 [R] source rows.
OWL_API int owl_gguf_dequant(const void* blocks, int type, int K, const void* rows, int R, void* out, cudaStream_t st) {
  int elems, bytes;
  if (!gguf_geom(type, elems, bytes) || K < elems || K % elems || R < 1) return OWL_ERR_BAD_ARG;
  gguf_dequant_kernel<<<dim3((K + 255) / 256, R), 256, 0, st>>>((const uint8_t*)blocks, type, K, (const int*)rows, (__nv_bfloat16*)out);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
OWL_API int owl_gguf_gemv(const void* blocks, int type, const void* x, int ldx, void* out, int ldo, int M, int N, int K,
                          cudaStream_t st) {
  int elems, bytes;
  if (!gguf_geom(type, elems, bytes) || M < 1 || M > 8 || K % elems || (K & 255) || (ldx & 7)) return OWL_ERR_BAD_ARG;
  const dim3 grid((N + 7) / 8);
  if (M == 1) gguf_gemv_kernel<1><<<grid, 256, 0, st>>>((const uint8_t*)blocks, type, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)out, ldo, M, N, K);
  else if (M <= 4) gguf_gemv_kernel<4><<<grid, 256, 0, st>>>((const uint8_t*)blocks, type, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)out, ldo, M, N, K);
  else gguf_gemv_kernel<8><<<grid, 256, 0, st>>>((const uint8_t*)blocks, type, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)out, ldo, M, N, K);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
