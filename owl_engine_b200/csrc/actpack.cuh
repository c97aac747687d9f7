// ActPack: the activation format consumed by the W4A16 weight-streaming kernels (gemv.cu).
//
// The streaming kernels feed the int4 weights to the integer tensor-core path as bytes: one AND
// gives the four low nibbles of a 32-bit weight word, one shift + AND the four high nibbles, and
// that is the entire "dequantisation" (zero point and scale are applied once per group on the
// int32 accumulators). The activations therefore have to be integers too: the producer stores
// every activation as 15-bit fixed point split into a signed high byte h and a 7-bit low part l
// (0..127, valid both as a signed and as an unsigned byte, which lets one tcgen05 kind::i8 operand
// carry both planes), x = sx * (128 * h + l), with one scale sx per (token, group of G consecutive
// k), so two int8 MMAs per nibble stream accumulate sum_k q_k x_k exactly in int32.
//
// Layout: every run of 8 consecutive k is one 16-byte chunk (same index as the k run). Weight
// byte b (0..3) of the run holds k_lo = {0,4,1,5}[b] in its low nibble and k_hi = {2,6,3,7}[b] in
// its high nibble (the nibble order of the weight records), and the chunk stores
//   bytes  0..3  : h of x[k_lo(b)]      bytes  4..7  : l of x[k_lo(b)]
//   bytes  8..11 : h of x[k_hi(b)]      bytes 12..15 : l of x[k_hi(b)]
// Per (token, group): float2 (sx, xsum) with xsum = sum of the group's activations. Then
//   sum_k (q_k - z) x_k = sx * (128 * acc_h + acc_l) - z * xsum.
#pragma once
#include "common.cuh"

namespace owl {

constexpr int ACT_LO_BITS = 7;            // x_fixed = (h << ACT_LO_BITS) + l
constexpr float ACT_QMAX = 16383.f;       // largest |x_fixed|

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
// With ACT_A8 in the producer's group argument (it arrives here as bit ACT_A8 >> 3 of `cpg`) the activations are rounded to
// 8 bits instead of 15: h = round(x * 127 / amax), l = 0 and sx = amax / (127 * 128), so every consumer reads the same
// format and the W4A8 arm of the streaming kernel may skip the low plane.
constexpr int ACT_A8 = 0x2000;
__device__ __forceinline__ uint4 actpack_emit(const float* v, int cpg, float& sx, float& xsum) {
  const bool a8 = (cpg & (ACT_A8 >> 3)) != 0;
  cpg &= (ACT_A8 >> 3) - 1;
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
  if (a8) {
    const float s8 = fmaxf(amax, 1e-30f) * (1.f / 127.f), inv8 = 1.f / s8;
    uint32_t hb8 = 0, hl8 = 0;
    int qsum = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int qb = __float2int_rn(pb[b] * inv8), ql = __float2int_rn(pl[b] * inv8);
      hb8 |= (uint32_t)(qb & 0xff) << (8 * b);
      hl8 |= (uint32_t)(ql & 0xff) << (8 * b);
      qsum += qb + ql;
    }
    for (int o = cpg >> 1; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
    xsum = s8 * (float)qsum;      // the zero-point term uses the ROUNDED activations: the product is exact for them
    sx = s8 * (1.f / 128.f);
    return make_uint4(hl8, 0u, hb8, 0u);
  }
  sx = fmaxf(amax, 1e-30f) * (1.f / ACT_QMAX);
  const float inv = 1.f / sx;
  uint32_t hb = 0, lb = 0, hl = 0, ll = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int qb = __float2int_rn(pb[b] * inv), ql = __float2int_rn(pl[b] * inv);
    hb |= (uint32_t)((qb >> ACT_LO_BITS) & 0xff) << (8 * b);
    lb |= (uint32_t)(qb & 0x7f) << (8 * b);
    hl |= (uint32_t)((ql >> ACT_LO_BITS) & 0xff) << (8 * b);
    ll |= (uint32_t)(ql & 0x7f) << (8 * b);
  }
  return make_uint4(hl, ll, hb, lb);
}

// ---- where a chunk goes ------------------------------------------------------------------------
// Row layout (default): xpack[token][K/8] chunks and xs[token][K/G], as described above.
// Tile layout (group argument of a producer has ACT_TILES set; at most 8 tokens): the buffer is one
// run per 128-k record kt of
//   [4 MMA steps w][2 k halves][16 columns][16 bytes]   the B operand of the tcgen05 streaming kernel:
//        column = token for the high planes, 8 + token for the low planes; chunk c8 = kt*16 + w*4 + t
//        contributes bytes t*8 .. t*8+7 of step w: {h(a), h(c)} resp. {l(a), l(c)}
//   [128/G groups][8 tokens] float2 (sx, xsum)
// so the consumer fetches everything a weight block needs with one bulk copy. `xs` is unused.
// Tokens 8..15, 16..23, ... go to further buffers of the same size that follow the first one.
constexpr int ACT_TILES = 0x1000;
__host__ __device__ constexpr int actpack_tile_bytes(int G) { return 2048 + 64 * (128 / G); }

// Group argument check of the producers' launchers: 32 / 128, optionally | ACT_TILES.
inline bool actpack_group_ok(int G, int tokens) {
  const int g = G & ~(ACT_TILES | 0x2000);       // 0x2000: ACT_A8
  (void)tokens;
  return g == 32 || g == 128;
}

__device__ __forceinline__ void actpack_store(uint4* xpack, float2* xs, int tiles, int G, int token, int c8, int nchunks,
                                              const uint4& pk, float sx, float xsum) {
  G &= ~ACT_A8;
  const int cpg = G >> 3;
  if (!tiles) {
    xpack[(size_t)token * nchunks + c8] = pk;
    if ((c8 % cpg) == 0) xs[(size_t)token * (nchunks / cpg) + c8 / cpg] = make_float2(sx, xsum);
  } else {
    const int kt = c8 >> 4, w = (c8 >> 2) & 3, t = c8 & 3;
    uint8_t* rec = reinterpret_cast<uint8_t*>(xpack) + ((size_t)(token >> 3) * (nchunks >> 4) + kt) * actpack_tile_bytes(G);
    token &= 7;
    uint8_t* b = rec + w * 512 + (t >> 1) * 256 + token * 16 + (t & 1) * 8;
    *reinterpret_cast<uint2*>(b) = make_uint2(pk.x, pk.z);
    *reinterpret_cast<uint2*>(b + 128) = make_uint2(pk.y, pk.w);
    if ((c8 % cpg) == 0) *reinterpret_cast<float2*>(rec + 2048 + (((c8 & 15) / cpg) * 8 + token) * 8) = make_float2(sx, xsum);
  }
}

}  // namespace owl
