// ActPack: the activation format consumed by the W4A16 weight-streaming kernels (gemv.cu).
//
// The streaming kernels feed the int4 weights to the integer tensor-core path as bytes: one AND
// gives the four low nibbles of a 32-bit weight word, one shift + AND the four high nibbles, and
// that is the entire "dequantisation" (zero point and scale are applied once per group on the
// int32 accumulators). The activations therefore have to be integers too: the producer stores
// every activation as 16-bit fixed point split into a signed high byte and an unsigned low byte,
// x = sx * (256 * h + l), with one scale sx per (token, group of G consecutive k), so two int8
// MMAs per nibble stream accumulate sum_k q_k x_k exactly in int32.
//
// Layout: every run of 8 consecutive k is one 16-byte chunk (same index as the k run). Weight
// byte b (0..3) of the run holds k_lo = {0,4,1,5}[b] in its low nibble and k_hi = {2,6,3,7}[b] in
// its high nibble (the nibble order of the weight records), and the chunk stores
//   bytes  0..3  : h of x[k_lo(b)]      bytes  4..7  : l of x[k_lo(b)]
//   bytes  8..11 : h of x[k_hi(b)]      bytes 12..15 : l of x[k_hi(b)]
// Per (token, group): float2 (sx, xsum) with xsum = sum of the group's activations. Then
//   sum_k (q_k - z) x_k = sx * (256 * acc_h + acc_l) - z * xsum.
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

// Packs 8 consecutive activations. Every lane of the warp must call this; the `cpg` (4 or 16)
// consecutive lanes that hold the chunks of one group cooperate through shuffles. Returns the
// chunk; (sx, xsum) are valid in every lane of the group.
__device__ __forceinline__ uint4 actpack_emit(const float* v, int cpg, float& sx, float& xsum) {
  float pb[4], pl[4];   // pl: activations of the low nibbles, pb: of the high nibbles
  const int klo[4] = {0, 4, 1, 5}, khi[4] = {2, 6, 3, 7};
  float amax = 0.f;
  xsum = 0.f;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    pl[b] = v[klo[b]];
    pb[b] = v[khi[b]];
    amax = fmaxf(amax, fmaxf(fabsf(pb[b]), fabsf(pl[b])));
    xsum += pl[b] + pb[b];
  }
  for (int o = cpg >> 1; o > 0; o >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    xsum += __shfl_xor_sync(0xffffffffu, xsum, o);
  }
  sx = fmaxf(amax, 1e-30f) * (1.f / 32767.f);
  const float inv = 1.f / sx;
  uint32_t hb = 0, lb = 0, hl = 0, ll = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int qb = __float2int_rn(pb[b] * inv), ql = __float2int_rn(pl[b] * inv);
    hb |= (uint32_t)((qb >> 8) & 0xff) << (8 * b);
    lb |= (uint32_t)(qb & 0xff) << (8 * b);
    hl |= (uint32_t)((ql >> 8) & 0xff) << (8 * b);
    ll |= (uint32_t)(ql & 0xff) << (8 * b);
  }
  return make_uint4(hl, ll, hb, lb);
}

}  // namespace owl
