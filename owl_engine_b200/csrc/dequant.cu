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
