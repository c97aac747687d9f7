// Load-time / baseline helpers: expand a W4 skinny-tile weight to dense bf16 [N][K].
// Used by the baseline GEMM arm (dequant -> library GEMM) and by tests; the product prefill
// path dequantises inside the tcgen05 GEMM instead (gemm_tc.cu).
// Reference counterpart: owl_gguf_dequant_range_* + cuBLAS arm (crates/kernels/cu/gguf/gguf_smem.cu).
#include "common.cuh"

#include "records.cuh"

namespace owl {
// grid (K/128, N/16), block 64: thread L handles uint4 #L of the tile (row, 4 words of 8 nibbles).
__global__ void __launch_bounds__(64) w4_dequant_kernel(const uint8_t* __restrict__ records, __nv_bfloat16* out, int N,
                                                        int K, int G, int layout, int f16) {
  const int kt = blockIdx.x, nt = blockIdx.y, L = threadIdx.x;
  const int KT = K >> 7, GPT = 128 / G;
  const int half = L >> 5, g = (L & 31) >> 2, t = L & 3;
  const int row = nt * 16 + half * 8 + g;
  const int REC = 1024 + 64 * GPT;
  const uint8_t* rec = records + record_offset_any(layout, N / 16, KT, nt, kt) * (size_t)REC;
  const uint4 u = reinterpret_cast<const uint4*>(rec)[L];
  const __half2* sz = reinterpret_cast<const __half2*>(rec + 1024);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    const int q = (G == 128) ? 0 : wi;
    const __half2 s = sz[q * 16 + half * 8 + g];
    const float sc = __low2float(s), z = __high2float(s);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int nib = (i >> 1) + (i & 1) * 4;   // k_local i sits at nibble (i/2) + 4*(i%2)
      v[i] = ((float)((w[wi] >> (4 * nib)) & 0xF) - z) * sc;
    }
    uint4 o = f16 ? make_uint4(pack_f16(v[0], v[1]), pack_f16(v[2], v[3]), pack_f16(v[4], v[5]), pack_f16(v[6], v[7]))
                  : make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
    *reinterpret_cast<uint4*>(out + (size_t)row * K + kt * 128 + wi * 32 + t * 8) = o;
  }
}
}  // namespace owl
using namespace owl;

// out: bf16 (f16 = 0) or fp16 (f16 = 1) [N][K].
OWL_API int owl_w4_dequant(const void* records, void* out, int N, int K, int G, int layout, int f16, cudaStream_t st) {
  if ((N & 15) || (K & 127) || (G != 32 && G != 128)) return OWL_ERR_BAD_ARG;
  w4_dequant_kernel<<<dim3(K / 128, N / 16), 64, 0, st>>>((const uint8_t*)records, (__nv_bfloat16*)out, N, K, G, layout, f16);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

namespace owl {
// One CTA per row: amax -> scale = amax / 448, out = e4m3(x / scale). 16-bit input (fp16 or bf16), K multiple of 8.
__global__ void __launch_bounds__(256) quant_e4m3_rows_kernel(const uint16_t* __restrict__ x, int ldx, int f16,
                                                              uint8_t* __restrict__ out, int ldo, float* __restrict__ scales,
                                                              int K) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
  const int nchunks = K >> 3;
  auto unpack = [&](const uint4& u, float* v) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (f16) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
      } else {
        v[2 * i] = bf16_lo(w[i]); v[2 * i + 1] = bf16_hi(w[i]);
      }
    }
  };
  float amax = 0.f;
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
    float v[8];
    unpack(src[c], v);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = block_max(amax, red);
  const float scale = amax > 0.f ? amax / 448.f : 1.f, inv = 1.f / scale;
  if (threadIdx.x == 0) scales[row] = scale;
  uint2* dst = reinterpret_cast<uint2*>(out + (size_t)row * ldo);
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
    float v[8];
    unpack(src[c], v);
    uint32_t q[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_fp8x2_storage_t p2 = __nv_cvt_float2_to_fp8x2(make_float2(v[2 * i] * inv, v[2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      q[i >> 1] |= (uint32_t)p2 << (16 * (i & 1));
    }
    dst[c] = make_uint2(q[0], q[1]);
  }
}
}  // namespace owl

// x: fp16 (f16 = 1) or bf16 [R][ldx]; out: e4m3 bytes [R][ldo]; scales fp32 [R] with x ~= scale * out.
OWL_API int owl_quant_e4m3_rows(const void* x, int ldx, int f16, void* out, int ldo, void* scales, int R, int K,
                                cudaStream_t st) {
  if (R < 1 || K < 8 || (K & 7) || (ldx & 7) || (ldo & 7) || !scales) return OWL_ERR_BAD_ARG;
  owl::quant_e4m3_rows_kernel<<<R, 256, 0, st>>>((const uint16_t*)x, ldx, f16, (uint8_t*)out, ldo, (float*)scales, K);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
