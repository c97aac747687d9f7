// ActPack helpers: the fp16 activation format consumed by the W4A16 weight-streaming kernels.
// Per run of 8 consecutive k the stored halves are [x0, x1, x2/16, x3/16, x4, x5, x6/16, x7/16].
#pragma once
#include "common.cuh"

namespace owl {

__device__ __forceinline__ void unpack_bf16x8(const uint4& a, float* v) {
  v[0] = bf16_lo(a.x); v[1] = bf16_hi(a.x); v[2] = bf16_lo(a.y); v[3] = bf16_hi(a.y);
  v[4] = bf16_lo(a.z); v[5] = bf16_hi(a.z); v[6] = bf16_lo(a.w); v[7] = bf16_hi(a.w);
}
__device__ __forceinline__ uint4 pack_bf16x8(const float* v) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ uint4 pack_f16x8(const float* v) {
  return make_uint4(pack_f16(v[0], v[1]), pack_f16(v[2], v[3]), pack_f16(v[4], v[5]), pack_f16(v[6], v[7]));
}
__device__ __forceinline__ float clamp_h(float x) { return fminf(fmaxf(x, -65504.f), 65504.f); }

// v: 8 consecutive activations. Returns the packed chunk; s_stored = sum of the 8 stored
// halves, s_eff = sum of the effective activations (stored * 16 for the pre-scaled slots).
__device__ __forceinline__ uint4 actpack_chunk(const float* v, float& s_stored, float& s_eff) {
  const __half h0 = __float2half_rn(clamp_h(v[0])), h1 = __float2half_rn(clamp_h(v[1]));
  const __half h2 = __float2half_rn(clamp_h(v[2]) * 0.0625f), h3 = __float2half_rn(clamp_h(v[3]) * 0.0625f);
  const __half h4 = __float2half_rn(clamp_h(v[4])), h5 = __float2half_rn(clamp_h(v[5]));
  const __half h6 = __float2half_rn(clamp_h(v[6]) * 0.0625f), h7 = __float2half_rn(clamp_h(v[7]) * 0.0625f);
  const float lo = __half2float(h0) + __half2float(h1) + __half2float(h4) + __half2float(h5);
  const float hi = __half2float(h2) + __half2float(h3) + __half2float(h6) + __half2float(h7);
  s_stored = lo + hi;
  s_eff = lo + 16.f * hi;
  uint4 r;
  r.x = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
  r.y = (uint32_t)__half_as_ushort(h2) | ((uint32_t)__half_as_ushort(h3) << 16);
  r.z = (uint32_t)__half_as_ushort(h4) | ((uint32_t)__half_as_ushort(h5) << 16);
  r.w = (uint32_t)__half_as_ushort(h6) | ((uint32_t)__half_as_ushort(h7) << 16);
  return r;
}
// Sum over `cpg` (4 or 16) consecutive lanes; every lane of the warp must call this.
__device__ __forceinline__ void actpack_group_reduce(float& s_stored, float& s_eff, int cpg) {
  for (int o = cpg >> 1; o > 0; o >>= 1) {
    s_stored += __shfl_xor_sync(0xffffffffu, s_stored, o);
    s_eff += __shfl_xor_sync(0xffffffffu, s_eff, o);
  }
}

}  // namespace owl
