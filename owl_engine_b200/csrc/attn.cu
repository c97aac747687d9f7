// Full-attention kernels for the gated GQA layers (fp8 e4m3 paged KV, page = 16 tokens).
//
//   owl_qknorm_rope_insert : per-head q/k RMSNorm x(1+w), partial rotate-half RoPE (m-RoPE
//                            capable: 3 position streams + per-frequency section map), K/V cast to
//                            e4m3 and scattered into the paged pool, q written as bf16.
//   owl_paged_attn         : split-KV GQA attention over the paged fp8 pool for decode (T=1),
//                            verify (T<=8 rows, causal inside the new rows) and prefill chunks
//                            (issued as groups of <=8 consecutive rows). Tensor-core QK^T and PV
//                            with fp8 -> f16 conversion in registers; one 16-token page per tile.
//   owl_attn_reduce        : merges the split partials, applies the sigmoid output gate and
//                            writes bf16 and/or ActPack for o_proj.
//
// Role in the reference: owl_qknorm_rope_kv_insert_* (crates/kernels/cu/fused/qknorm_insert.cu),
// the XQA / paged-attention-v2 / FlashInfer decode+verify arms (cu/xqa/mha.cu,
// cu/attn/pagedattention_f16.cu, cu/flashinfer/*) and owl_sigmoid_gate_mul_f16.
#include "common.cuh"
#include "actpack.cuh"

namespace owl {

constexpr int PAGE = 16;

// ---------------------------------------------------------------------------------------
// grid (rows, hq + 2*hkv), block 128. head < hq: q; < hq+hkv: k; else v.
// qraw row layout: per q head [q_h (hd) | gate_h (hd)]; kraw/vraw: [hkv][hd].
// ---------------------------------------------------------------------------------------
struct InsertParams {
  const __nv_bfloat16* qraw; int ldq;
  const __nv_bfloat16* kraw; int ldk;
  const __nv_bfloat16* vraw; int ldv;
  const __nv_bfloat16* qnorm_w; const __nv_bfloat16* knorm_w;
  const int* pos3;              // [3][rows] position streams (T,H,W); text rows have all equal
  const float* inv_freq;        // [rot/2]
  const unsigned char* section; // [rot/2] stream index per frequency
  const int* kv_slot;           // [rows] physical token index (page*16 + off); < 0 = skip write
  __nv_bfloat16* q_out;         // [rows][hq][hd]
  uint8_t* k_pool; uint8_t* v_pool;  // [pages][16][hkv][hd] e4m3, or int8 when the scale pools are given
  float* k_scale; float* v_scale;    // int8 pool: [pages][16][hkv] per (token, kv head) scales (null: e4m3 pool)
  int kv16;                          // 16-bit pool: fp16 words holding the bf16-rounded values (exact inside the fp16 range)
  int rows, hq, hkv, hd, rot;
  float eps, rope_scale;        // rope_scale multiplies cos/sin (YaRN attention factor)
};

__global__ void __launch_bounds__(128) qknorm_rope_insert_kernel(InsertParams p) {
  __shared__ float y[256];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
  const int hd = p.hd;
  const bool is_q = head < p.hq, is_k = !is_q && head < p.hq + p.hkv;
  const int kvh = is_q ? 0 : (is_k ? head - p.hq : head - p.hq - p.hkv);
  const __nv_bfloat16* src = is_q ? p.qraw + (size_t)row * p.ldq + (size_t)head * 2 * hd
                           : is_k ? p.kraw + (size_t)row * p.ldk + (size_t)kvh * hd
                                  : p.vraw + (size_t)row * p.ldv + (size_t)kvh * hd;
  const int e0 = tid * 2;
  float a = 0.f, b = 0.f;
  if (e0 < hd) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(src + e0);
    a = bf16_lo(u); b = bf16_hi(u);
  }
  if (is_q || is_k) {
    const float ss = block_sum(a * a + b * b, red);
    const float rinv = rsqrtf(ss / (float)hd + p.eps);
    const __nv_bfloat16* w = is_q ? p.qnorm_w : p.knorm_w;
    if (e0 < hd) {
      a = a * rinv * (1.f + __bfloat162float(w[e0]));
      b = b * rinv * (1.f + __bfloat162float(w[e0 + 1]));
      y[e0] = a; y[e0 + 1] = b;
    }
    __syncthreads();
    const int half = p.rot >> 1;
    if (e0 < p.rot) {
      float o[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int d = e0 + i;
        const int j = d < half ? d : d - half;
        const int pos = p.pos3[(size_t)p.section[j] * p.rows + row];
        float sn, cs;
        sincosf((float)pos * p.inv_freq[j], &sn, &cs);
        sn *= p.rope_scale; cs *= p.rope_scale;
        o[i] = d < half ? y[d] * cs - y[d + half] * sn : y[d] * cs + y[d - half] * sn;
      }
      a = o[0]; b = o[1];
    }
  }
  float amax = 0.f;
  if (!is_q && p.k_scale) {    // int8 pool: one scale per (token, kv head), from the bf16-rounded values
    const float av = e0 < hd ? fmaxf(fabsf(__bfloat162float(__float2bfloat16(a))), fabsf(__bfloat162float(__float2bfloat16(b)))) : 0.f;
    amax = block_max(av, red);
  }
  if (e0 >= hd) return;
  if (is_q) {
    *reinterpret_cast<uint32_t*>(p.q_out + ((size_t)row * p.hq + head) * hd + e0) = pack_bf16(a, b);
  } else {
    const int slot = p.kv_slot[row];
    if (slot < 0) return;
    uint8_t* dst = (is_k ? p.k_pool : p.v_pool) + ((size_t)slot * p.hkv + kvh) * hd + e0;
    // values are rounded to bf16 first so the pool holds cast(bf16(x)) like a two-step pipeline
    const float ar = __bfloat162float(__float2bfloat16(a)), br = __bfloat162float(__float2bfloat16(b));
    if (p.kv16) {
      __half2* d16 = reinterpret_cast<__half2*>((is_k ? p.k_pool : p.v_pool) + (((size_t)slot * p.hkv + kvh) * hd + e0) * 2);
      *d16 = __floats2half2_rn(fminf(fmaxf(ar, -65504.f), 65504.f), fminf(fmaxf(br, -65504.f), 65504.f));
      return;
    }
    if (p.k_scale) {
      const float sc = amax > 0.f ? amax / 127.f : 1.f, inv = 1.f / sc;
      const int qa = max(-127, min(127, __float2int_rn(ar * inv))), qb = max(-127, min(127, __float2int_rn(br * inv)));
      *reinterpret_cast<uint16_t*>(dst) = (uint16_t)(qa & 0xff) | ((uint16_t)(qb & 0xff) << 8);
      if (tid == 0) (is_k ? p.k_scale : p.v_scale)[(size_t)slot * p.hkv + kvh] = sc;
    } else {
      *reinterpret_cast<uint16_t*>(dst) = (uint16_t)f_to_fp8e4m3(ar) | ((uint16_t)f_to_fp8e4m3(br) << 8);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Paged attention. grid (splits, hkv, groups); block = 4 warps.
// A "group" is T consecutive query rows of one sequence; each query row contributes Gq = hq/hkv
// heads (<= 8) = one MMA row group. Warps = RG row groups x TS token splits (RG*TS = 4).
// ---------------------------------------------------------------------------------------
struct AttnParams {
  const __nv_bfloat16* q;       // [groups*T][hq][hd]
  const uint8_t* k_pool; const uint8_t* v_pool;
  const float* k_scale; const float* v_scale;   // int8 pool only
  const int* block_table;       // [seqs][max_blocks]
  const int* bt_row;            // [groups] -> block_table row (nullptr: identity)
  const int* ctx_len;           // [groups] tokens visible to the LAST row of the group
  float* part_o;                // [groups*T][hq][splits][hd]
  float* part_ml;               // [groups*T][hq][splits][2]
  int T, hq, hkv, max_blocks, splits;
  int per_pages;                // > 0: pages per split fixed by the caller (partitions aligned to positions, the same for
                                //      every T); 0: the pages of the longest row divided evenly
  float scale_log2;             // softmax scale * log2(e)
};

constexpr int AT_WARPS = 4;
constexpr int HD = 256;

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two_bytes, __NV_E4M3);
  return *reinterpret_cast<uint32_t*>(&r);
}
// two int8 bytes -> f16x2, exact: (b ^ 0x80) placed under the exponent of 1024, minus 1152
__device__ __forceinline__ uint32_t s8x2_to_f16x2(uint32_t two_bytes) {
  const uint32_t w = __byte_perm(two_bytes ^ 0x8080u, 0x64646464u, 0x4140u);
  const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&w), __half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480)));
  return *reinterpret_cast<const uint32_t*>(&r);
}
// pool formats of the attention kernel
enum { KV_E4M3 = 0, KV_I8 = 1, KV_F16 = 2 };
template <int KV>
__device__ __forceinline__ uint32_t kv2_to_f16x2(uint32_t two_bytes) {
  return KV == KV_I8 ? s8x2_to_f16x2(two_bytes) : e4m3x2_to_f16x2(two_bytes);
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int RG, int KV>
__global__ void __launch_bounds__(AT_WARPS * 32) paged_attn_kernel(AttnParams p) {
  constexpr int TS = AT_WARPS / RG;
  constexpr bool I8 = KV == KV_I8, F16 = KV == KV_F16;
  constexpr int ESZ = F16 ? 2 : 1;             // bytes per pool element
  // cross-warp merge buffers (token splits of the same row group)
  __shared__ float mo[AT_WARPS][8][HD + 1];   // O by [row][dim]
  __shared__ float mml[AT_WARPS][8][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, kvh = blockIdx.y, grp = blockIdx.z;
  const int Gq = p.hq / p.hkv;
  const int rg = warp / TS, ts = warp % TS;  // row group index within the CTA pass, token split
  pdl_launch_dependents();
  pdl_wait();
  const int ctx_last = p.ctx_len[grp];
  const int btr = p.bt_row ? p.bt_row[grp] : grp;
  const int* bt = p.block_table + (size_t)btr * p.max_blocks;

  for (int r0 = 0; r0 < p.T; r0 += RG) {
    const int r = r0 + rg;                       // query row inside the group
    const bool row_ok = r < p.T;
    const int limit = ctx_last - (p.T - 1 - r);  // tokens visible to this row
    const int npages_all = (ctx_last + PAGE - 1) / PAGE;
    const int per = p.per_pages > 0 ? p.per_pages : (npages_all + p.splits - 1) / p.splits;
    const int pg0 = split * per, pg1 = min(npages_all, pg0 + per);

    // Q fragments (f16) for k-steps (blk 0..3, j 0..3): dims blk*64 + t*16 + j*4 + {0,1 | 2,3}
    uint32_t qa0[16], qa2[16];
    {
      const size_t qrow = (size_t)grp * p.T + (row_ok ? r : 0);
      const __nv_bfloat16* qp = p.q + (qrow * p.hq + (size_t)kvh * Gq + g) * HD;
      const bool head_ok = row_ok && g < Gq;
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        uint4 u0 = make_uint4(0, 0, 0, 0), u1 = u0;
        if (head_ok) {
          u0 = *reinterpret_cast<const uint4*>(qp + blk * 64 + t * 16);
          u1 = *reinterpret_cast<const uint4*>(qp + blk * 64 + t * 16 + 8);
        }
        const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          qa0[blk * 4 + j] = pack_f16(bf16_lo(w[j * 2]), bf16_hi(w[j * 2]));
          qa2[blk * 4 + j] = pack_f16(bf16_lo(w[j * 2 + 1]), bf16_hi(w[j * 2 + 1]));
        }
      }
    }
    float m_run = -INFINITY, l_run = 0.f;  // for row g (replicated over t)
    float o[16][4];                         // O^T m-tiles (blk 0..7, ip 0..1)
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    if (row_ok) {
      for (int pg = pg0 + ts; pg < pg1; pg += TS) {
        const int tk0 = pg * PAGE;
        if (tk0 >= limit) break;
        const int page = bt[pg];
        const uint8_t* kp = p.k_pool + (((size_t)page * PAGE) * p.hkv + kvh) * HD * ESZ;
        const uint8_t* vp = p.v_pool + (((size_t)page * PAGE) * p.hkv + kvh) * HD * ESZ;
        const size_t tstride = (size_t)p.hkv * HD * ESZ;
        // ---- S = Q K^T for tokens tk0+g (s0) and tk0+8+g (s1) -----------------------------
        float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
        uint4 ka[4], kb[4];
        uint4 ka2[F16 ? 4 : 1], kb2[F16 ? 4 : 1];   // 16-bit pool: the second 8 of the lane's 16 dims per block
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
          ka[blk] = ldg_stream(reinterpret_cast<const uint4*>(kp + (size_t)g * tstride + (blk * 64 + t * 16) * ESZ));
          kb[blk] = ldg_stream(reinterpret_cast<const uint4*>(kp + (size_t)(g + 8) * tstride + (blk * 64 + t * 16) * ESZ));
          if constexpr (F16) {
            ka2[blk] = ldg_stream(reinterpret_cast<const uint4*>(kp + (size_t)g * tstride + (blk * 64 + t * 16) * ESZ + 16));
            kb2[blk] = ldg_stream(reinterpret_cast<const uint4*>(kp + (size_t)(g + 8) * tstride + (blk * 64 + t * 16) * ESZ + 16));
          }
        }
        // V words for tokens tk0 + {2t, 2t+1, 2t+8, 2t+9}, dims blk*32 + g*4 .. +3
        // (16-bit pool: two words per token and block, x = dims 0,1 and y = dims 2,3 of the lane's four)
        uint32_t va[8], vb[8], vc[8], vd[8];
        uint32_t va2[F16 ? 8 : 1], vb2[F16 ? 8 : 1], vc2[F16 ? 8 : 1], vd2[F16 ? 8 : 1];
#pragma unroll
        for (int blk = 0; blk < 8; ++blk) {
          const size_t doff = (size_t)(blk * 32 + g * 4) * ESZ;
          va[blk] = ldg_stream_u32(reinterpret_cast<const uint32_t*>(vp + (size_t)(2 * t) * tstride + doff));
          vb[blk] = ldg_stream_u32(reinterpret_cast<const uint32_t*>(vp + (size_t)(2 * t + 1) * tstride + doff));
          vc[blk] = ldg_stream_u32(reinterpret_cast<const uint32_t*>(vp + (size_t)(2 * t + 8) * tstride + doff));
          vd[blk] = ldg_stream_u32(reinterpret_cast<const uint32_t*>(vp + (size_t)(2 * t + 9) * tstride + doff));
          if constexpr (F16) {
            va2[blk] = ldg_stream_u32(reinterpret_cast<const uint32_t*>(vp + (size_t)(2 * t) * tstride + doff + 4));
            vb2[blk] = ldg_stream_u32(reinterpret_cast<const uint32_t*>(vp + (size_t)(2 * t + 1) * tstride + doff + 4));
            vc2[blk] = ldg_stream_u32(reinterpret_cast<const uint32_t*>(vp + (size_t)(2 * t + 8) * tstride + doff + 4));
            vd2[blk] = ldg_stream_u32(reinterpret_cast<const uint32_t*>(vp + (size_t)(2 * t + 9) * tstride + doff + 4));
          }
        }
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
          const uint32_t wa[4] = {ka[blk].x, ka[blk].y, ka[blk].z, ka[blk].w};
          const uint32_t wb[4] = {kb[blk].x, kb[blk].y, kb[blk].z, kb[blk].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if constexpr (F16) {     // fp16 words as stored: dims j*4 + {0,1} and {2,3}
              const uint32_t xa[8] = {wa[0], wa[1], wa[2], wa[3], ka2[blk].x, ka2[blk].y, ka2[blk].z, ka2[blk].w};
              const uint32_t xb[8] = {wb[0], wb[1], wb[2], wb[3], kb2[blk].x, kb2[blk].y, kb2[blk].z, kb2[blk].w};
              mma16816(s0, qa0[blk * 4 + j], 0u, qa2[blk * 4 + j], 0u, xa[2 * j], xa[2 * j + 1]);
              mma16816(s1, qa0[blk * 4 + j], 0u, qa2[blk * 4 + j], 0u, xb[2 * j], xb[2 * j + 1]);
            } else {
              mma16816(s0, qa0[blk * 4 + j], 0u, qa2[blk * 4 + j], 0u, kv2_to_f16x2<KV>(wa[j] & 0xffffu),
                       kv2_to_f16x2<KV>(wa[j] >> 16));
              mma16816(s1, qa0[blk * 4 + j], 0u, qa2[blk * 4 + j], 0u, kv2_to_f16x2<KV>(wb[j] & 0xffffu),
                       kv2_to_f16x2<KV>(wb[j] >> 16));
            }
          }
        }
        // s0[0..1]: (row g, tokens tk0+2t, +1); s1[0..1]: (row g, tokens tk0+8+2t, +1)
        float sv[4] = {s0[0], s0[1], s1[0], s1[1]};
        const int tk[4] = {tk0 + 2 * t, tk0 + 2 * t + 1, tk0 + 8 + 2 * t, tk0 + 9 + 2 * t};
        float vsc[4] = {1.f, 1.f, 1.f, 1.f};
        if (I8) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const size_t si = ((size_t)page * PAGE + (tk[i] - tk0)) * p.hkv + kvh;
            sv[i] *= p.k_scale[si];
            vsc[i] = p.v_scale[si];
          }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          sv[i] = tk[i] < limit ? sv[i] * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, sv[i]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);     // finite: token tk0 < limit is visible
        const float alpha = exp2f(m_run - m_new);
        float ps = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) { sv[i] = exp2f(sv[i] - m_new); ps += sv[i]; }
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = l_run * alpha + ps;
        m_run = m_new;
        // P^T as the B operand: b0 = (tokens 2t,2t+1 ; row g), b1 = (tokens 8+2t, 9+2t ; row g)
        const uint32_t pb0 = pack_f16(sv[0] * vsc[0], sv[1] * vsc[1]), pb1 = pack_f16(sv[2] * vsc[2], sv[3] * vsc[3]);
        // rescale factors for the O^T columns (rows 2t, 2t+1)
        const float al0 = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4);
        const float al1 = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
#pragma unroll
        for (int blk = 0; blk < 8; ++blk) {
#pragma unroll
          for (int ip = 0; ip < 2; ++ip) {
            float* c = o[blk * 2 + ip];
            c[0] *= al0; c[1] *= al1; c[2] *= al0; c[3] *= al1;
            // m-tile rows: g -> dim blk*32 + g*4 + ip*2, g+8 -> that + 1
            const uint32_t selA = ip ? 0x0062u : 0x0040u;  // bytes (x.b[2ip], y.b[2ip])
            const uint32_t selB = ip ? 0x0073u : 0x0051u;  // bytes (x.b[2ip+1], y.b[2ip+1])
            uint32_t a0, a1, a2, a3;
            if constexpr (F16) {     // word ip of each token holds dims (2ip, 2ip+1): low halves -> row g, high halves -> row g+8
              const uint32_t wa_ = ip ? va2[blk] : va[blk], wb_ = ip ? vb2[blk] : vb[blk];
              const uint32_t wc_ = ip ? vc2[blk] : vc[blk], wd_ = ip ? vd2[blk] : vd[blk];
              a0 = __byte_perm(wa_, wb_, 0x5410u); a1 = __byte_perm(wa_, wb_, 0x7632u);
              a2 = __byte_perm(wc_, wd_, 0x5410u); a3 = __byte_perm(wc_, wd_, 0x7632u);
            } else {
              a0 = kv2_to_f16x2<KV>(__byte_perm(va[blk], vb[blk], selA) & 0xffffu);
              a1 = kv2_to_f16x2<KV>(__byte_perm(va[blk], vb[blk], selB) & 0xffffu);
              a2 = kv2_to_f16x2<KV>(__byte_perm(vc[blk], vd[blk], selA) & 0xffffu);
              a3 = kv2_to_f16x2<KV>(__byte_perm(vc[blk], vd[blk], selB) & 0xffffu);
            }
            mma16816(c, a0, a1, a2, a3, pb0, pb1);
          }
        }
      }
    }
    // ---- merge the token-split warps of each row group, write the split partial ----------
    // O^T regs: o[blk*2+ip][0..1] = (dim blk*32+g*4+ip*2, rows 2t, 2t+1); [2..3] = dim + 1.
    __syncthreads();
#pragma unroll
    for (int blk = 0; blk < 8; ++blk)
#pragma unroll
      for (int ip = 0; ip < 2; ++ip) {
        const int d = blk * 32 + g * 4 + ip * 2;
        mo[warp][2 * t][d] = o[blk * 2 + ip][0];
        mo[warp][2 * t + 1][d] = o[blk * 2 + ip][1];
        mo[warp][2 * t][d + 1] = o[blk * 2 + ip][2];
        mo[warp][2 * t + 1][d + 1] = o[blk * 2 + ip][3];
      }
    if (t == 0) { mml[warp][g][0] = m_run; mml[warp][g][1] = l_run; }
    __syncthreads();
    // every warp finalises rows of its own row group for a slice of dims
    {
      const int rr = r0 + rg;
      if (rr < p.T) {
        for (int row = 0; row < Gq; ++row) {
          float M = -INFINITY;
          for (int s = 0; s < TS; ++s) M = fmaxf(M, mml[rg * TS + s][row][0]);
          float L = 0.f, w[TS];
          for (int s = 0; s < TS; ++s) {
            const float ms = mml[rg * TS + s][row][0];
            w[s] = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
            L += w[s] * mml[rg * TS + s][row][1];
          }
          const size_t qrow = (size_t)grp * p.T + rr;
          const size_t base = ((qrow * p.hq + (size_t)kvh * Gq + row) * p.splits + split);
          // dims handled by this warp's lanes: ts*(HD/TS) + lane, + 32, ...
          for (int d = ts * (HD / TS) + lane; d < (ts + 1) * (HD / TS); d += 32) {
            float acc = 0.f;
            for (int s = 0; s < TS; ++s) acc += w[s] * mo[rg * TS + s][row][d];
            p.part_o[base * HD + d] = acc;
          }
          if (ts == 0 && lane == 0) { p.part_ml[base * 2] = M; p.part_ml[base * 2 + 1] = L; }
        }
      }
    }
  }
}

// grid (rows, hq), block 256: CTA per (row, head); warp w merges splits w, w+8, ... (loads of
// different splits are independent), lane handles 8 dims; warp 0 combines and finishes.
__global__ void __launch_bounds__(256) attn_reduce_kernel(const float* __restrict__ part_o,
                                                          const float* __restrict__ part_ml, int splits,
                                                          const __nv_bfloat16* __restrict__ qraw, int ldq,
                                                          __nv_bfloat16* out, uint4* xpack, float2* xs, int hq, int G,
                                                          int out_f16) {
  __shared__ float sm_acc[8][HD];
  __shared__ float sm_l[8];
  __shared__ float sm_M;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x, head = blockIdx.y;
  // gate does not depend on the previous kernel's output only when qraw is older; load after the wait
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = ((size_t)row * hq + head) * splits;
  // global max over splits (every warp computes it: splits <= 64 -> two loads per lane)
  float mloc = -INFINITY;
  for (int s = lane; s < splits; s += 32) mloc = fmaxf(mloc, part_ml[(base + s) * 2]);
  const float M = warp_max(mloc);
  float L = 0.f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int s = warp; s < splits; s += 8) {
    const float ms = part_ml[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += w * part_ml[(base + s) * 2 + 1];
    const float4 a = *reinterpret_cast<const float4*>(part_o + (base + s) * HD + lane * 8);
    const float4 b = *reinterpret_cast<const float4*>(part_o + (base + s) * HD + lane * 8 + 4);
    acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * a.z; acc[3] += w * a.w;
    acc[4] += w * b.x; acc[5] += w * b.y; acc[6] += w * b.z; acc[7] += w * b.w;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) sm_acc[warp][lane * 8 + i] = acc[i];
  if (lane == 0) sm_l[warp] = L;
  __syncthreads();
  if (warp != 0) return;
  L = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) L += sm_l[w];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a += sm_acc[w][lane * 8 + i];
    acc[i] = a;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  float v[8];
  if (qraw) {
    const uint4 gq = *reinterpret_cast<const uint4*>(qraw + (size_t)row * ldq + (size_t)head * 2 * HD + HD + lane * 8);
    float gf[8];
    unpack_bf16x8(gq, gf);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = __bfloat162float(__float2bfloat16(acc[i] * inv));
      const float y = a * sigmoid_f(gf[i]);
      v[i] = out_f16 ? __half2float(__float2half_rn(clamp_h(y))) : __bfloat162float(__float2bfloat16(y));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(__float2bfloat16(acc[i] * inv));
  }
  const size_t e = ((size_t)row * hq + head) * HD + lane * 8;
  if (out) *reinterpret_cast<uint4*>(out + e) = out_f16 ? pack_f16x8(v) : pack_bf16x8(v);
  if (xpack) {
    const int tiles = G & ACT_TILES, g = G & ~ACT_TILES;
    float sx, xsum;
    const uint4 pk = actpack_emit(v, g >> 3, sx, xsum);
    actpack_store(xpack, xs, tiles, g, row, head * (HD / 8) + lane, hq * (HD / 8), pk, sx, xsum);
  }
}

}  // namespace owl
using namespace owl;

static int insert_launch(const void* qraw, int ldq, const void* kraw, int ldk, const void* vraw, int ldv, const void* qnorm_w,
                         const void* knorm_w, const void* pos3, const void* inv_freq, const void* section, const void* kv_slot,
                         void* q_out, void* k_pool, void* v_pool, void* k_scale, void* v_scale, int rows, int hq, int hkv, int hd,
                         int rot, float eps, float rope_scale, int pdl, cudaStream_t st, int kv16 = 0) {
  if (rows < 1 || hd > 256 || (hd & 1) || rot > hd || (rot & 3)) return OWL_ERR_BAD_ARG;
  InsertParams p;
  p.qraw = (const __nv_bfloat16*)qraw; p.ldq = ldq; p.kraw = (const __nv_bfloat16*)kraw; p.ldk = ldk;
  p.vraw = (const __nv_bfloat16*)vraw; p.ldv = ldv; p.qnorm_w = (const __nv_bfloat16*)qnorm_w;
  p.knorm_w = (const __nv_bfloat16*)knorm_w; p.pos3 = (const int*)pos3; p.inv_freq = (const float*)inv_freq;
  p.section = (const unsigned char*)section; p.kv_slot = (const int*)kv_slot; p.q_out = (__nv_bfloat16*)q_out;
  p.k_pool = (uint8_t*)k_pool; p.v_pool = (uint8_t*)v_pool; p.k_scale = (float*)k_scale; p.v_scale = (float*)v_scale;
  p.rows = rows; p.hq = hq; p.hkv = hkv; p.hd = hd; p.kv16 = kv16;
  p.rot = rot; p.eps = eps; p.rope_scale = rope_scale;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows, hq + 2 * hkv); cfg.blockDim = dim3(128); cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, qknorm_rope_insert_kernel, p);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

OWL_API int owl_qknorm_rope_insert(const void* qraw, int ldq, const void* kraw, int ldk, const void* vraw, int ldv,
                                   const void* qnorm_w, const void* knorm_w, const void* pos3, const void* inv_freq,
                                   const void* section, const void* kv_slot, void* q_out, void* k_pool, void* v_pool,
                                   int rows, int hq, int hkv, int hd, int rot, float eps, float rope_scale, int pdl,
                                   cudaStream_t st) {
  return insert_launch(qraw, ldq, kraw, ldk, vraw, ldv, qnorm_w, knorm_w, pos3, inv_freq, section, kv_slot, q_out, k_pool, v_pool,
                       nullptr, nullptr, rows, hq, hkv, hd, rot, eps, rope_scale, pdl, st);
}

// int8 KV pool: values rounded to int8 with one fp32 scale per (token, kv head) in k_scale / v_scale [pages][16][hkv].
OWL_API int owl_qknorm_rope_insert_i8(const void* qraw, int ldq, const void* kraw, int ldk, const void* vraw, int ldv,
                                      const void* qnorm_w, const void* knorm_w, const void* pos3, const void* inv_freq,
                                      const void* section, const void* kv_slot, void* q_out, void* k_pool, void* v_pool,
                                      void* k_scale, void* v_scale, int rows, int hq, int hkv, int hd, int rot, float eps,
                                      float rope_scale, int pdl, cudaStream_t st) {
  if (!k_scale || !v_scale) return OWL_ERR_BAD_ARG;
  return insert_launch(qraw, ldq, kraw, ldk, vraw, ldv, qnorm_w, knorm_w, pos3, inv_freq, section, kv_slot, q_out, k_pool, v_pool,
                       k_scale, v_scale, rows, hq, hkv, hd, rot, eps, rope_scale, pdl, st);
}

// 16-bit KV pool: fp16 words holding the bf16-rounded values (what a bf16 pool holds, readable by the fp16 MMA as stored).
OWL_API int owl_qknorm_rope_insert_f16(const void* qraw, int ldq, const void* kraw, int ldk, const void* vraw, int ldv,
                                       const void* qnorm_w, const void* knorm_w, const void* pos3, const void* inv_freq,
                                       const void* section, const void* kv_slot, void* q_out, void* k_pool, void* v_pool,
                                       int rows, int hq, int hkv, int hd, int rot, float eps, float rope_scale, int pdl,
                                       cudaStream_t st) {
  return insert_launch(qraw, ldq, kraw, ldk, vraw, ldv, qnorm_w, knorm_w, pos3, inv_freq, section, kv_slot, q_out, k_pool, v_pool,
                       nullptr, nullptr, rows, hq, hkv, hd, rot, eps, rope_scale, pdl, st, 1);
}

template <int KV>
static int attn_launch(const void* q, const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale,
                       const void* block_table, const void* bt_row, const void* ctx_len, void* part_o, void* part_ml, int groups,
                       int T, int hq, int hkv, int hd, int max_blocks, int splits, int per_pages, float scale, int pdl,
                       cudaStream_t st) {
  if (hd != HD || groups < 1 || T < 1 || T > 8 || hq % hkv || hq / hkv > 8 || splits < 1) return OWL_ERR_BAD_ARG;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.k_pool = (const uint8_t*)k_pool; p.v_pool = (const uint8_t*)v_pool;
  p.k_scale = (const float*)k_scale; p.v_scale = (const float*)v_scale;
  p.block_table = (const int*)block_table; p.bt_row = (const int*)bt_row; p.ctx_len = (const int*)ctx_len;
  p.part_o = (float*)part_o; p.part_ml = (float*)part_ml; p.T = T; p.hq = hq; p.hkv = hkv;
  p.max_blocks = max_blocks; p.splits = splits; p.per_pages = per_pages; p.scale_log2 = scale * 1.4426950408889634f;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, hkv, groups); cfg.blockDim = dim3(AT_WARPS * 32); cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e;
  // per_pages > 0 asks for arithmetic that does not depend on T: one warp per row (no token split inside a CTA)
  if (per_pages > 0) e = cudaLaunchKernelEx(&cfg, paged_attn_kernel<4, KV>, p);
  else if (T == 1) e = cudaLaunchKernelEx(&cfg, paged_attn_kernel<1, KV>, p);
  else if (T == 2) e = cudaLaunchKernelEx(&cfg, paged_attn_kernel<2, KV>, p);
  else e = cudaLaunchKernelEx(&cfg, paged_attn_kernel<4, KV>, p);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

// part_o: float[groups*T*hq*splits*256], part_ml: float[groups*T*hq*splits*2].
OWL_API int owl_paged_attn(const void* q, const void* k_pool, const void* v_pool, const void* block_table,
                           const void* bt_row, const void* ctx_len, void* part_o, void* part_ml, int groups, int T,
                           int hq, int hkv, int hd, int max_blocks, int splits, int per_pages, float scale, int pdl,
                           cudaStream_t st) {
  return attn_launch<KV_E4M3>(q, k_pool, v_pool, nullptr, nullptr, block_table, bt_row, ctx_len, part_o, part_ml, groups, T, hq, hkv,
                            hd, max_blocks, splits, per_pages, scale, pdl, st);
}

// The same attention over an int8 pool with per (token, kv head) scales.
OWL_API int owl_paged_attn_i8(const void* q, const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale,
                              const void* block_table, const void* bt_row, const void* ctx_len, void* part_o, void* part_ml,
                              int groups, int T, int hq, int hkv, int hd, int max_blocks, int splits, int per_pages, float scale,
                              int pdl, cudaStream_t st) {
  if (!k_scale || !v_scale) return OWL_ERR_BAD_ARG;
  return attn_launch<KV_I8>(q, k_pool, v_pool, k_scale, v_scale, block_table, bt_row, ctx_len, part_o, part_ml, groups, T, hq, hkv,
                           hd, max_blocks, splits, per_pages, scale, pdl, st);
}

// The same attention over a 16-bit pool (fp16 words holding bf16-rounded values, written by owl_qknorm_rope_insert_f16).
OWL_API int owl_paged_attn_f16(const void* q, const void* k_pool, const void* v_pool, const void* block_table,
                               const void* bt_row, const void* ctx_len, void* part_o, void* part_ml, int groups, int T,
                               int hq, int hkv, int hd, int max_blocks, int splits, int per_pages, float scale, int pdl,
                               cudaStream_t st) {
  return attn_launch<KV_F16>(q, k_pool, v_pool, nullptr, nullptr, block_table, bt_row, ctx_len, part_o, part_ml, groups, T, hq, hkv,
                             hd, max_blocks, splits, per_pages, scale, pdl, st);
}

OWL_API int owl_attn_reduce(const void* part_o, const void* part_ml, int splits, const void* qraw, int ldq, void* out,
                            void* xpack, void* xs, int rows, int hq, int G, int out_f16, int pdl, cudaStream_t st) {
  if (rows < 1 || splits < 1 || !actpack_group_ok(G, rows)) return OWL_ERR_BAD_ARG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows, hq); cfg.blockDim = dim3(256); cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, attn_reduce_kernel, (const float*)part_o, (const float*)part_ml, splits,
                                     (const __nv_bfloat16*)qraw, ldq, (__nv_bfloat16*)out, (uint4*)xpack, (float2*)xs,
                                     hq, G, out_f16);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}
