// Fused causal attention of a prefill chunk on tcgen05 (sm_100a): S = Q K^T and O = P V both accumulate in tensor memory, the
// online softmax runs between them in registers, key tiles past the causal limit of a row tile are never touched.
//
//   owl_attn_tc : per kv head h and tile of 128 query rows (the gq q heads of a kv head are stacked as consecutive rows, row =
//                 token * gq + head-in-group, so one K / V tile serves all of them)
//                   og[h][row][:] = softmax_k(scale * q[row] . K[h][k]) V[h][k],   k < pos0 + token(row) + 1
//
// Operands (dense, produced once per layer and chunk by owl_kv_gather / owl_q_group from the paged pool of THIS GPU):
//   qg  bf16 [hkv][rows][256]       K  bf16 [hkv][ctx_pad][256]       Vt  fp16 [hkv][256][ctx_pad]       og  bf16 [hkv][rows][256]
// All three are k-major for their MMA, read by plain (non-multicast) TMA with the 128-byte swizzle.
//
// One CTA = one (row tile, kv head), 320 threads, key tiles of 64:
//   warp 0      producer: Q once (64 KB), then K_j (32 KB) and V_j (32 KB) through two-stage rings of their own
//   warp 1      one thread issues S_j = Q K_j^T (16 x M128 N64 K16, bf16) into one of two 64-column S buffers, then
//               O += P_{j-1} V_{j-1} (4 x M128 N256 K16, fp16) into the 256 O columns: S_{j} runs while the softmax of tile j-1
//               is still busy
//   warps 2-9   softmax, two threads per query row (each half of the tile's key columns; the halves' row maxima meet through
//               shared memory at an mbarrier): tcgen05.ld S_j, causal mask on the diagonal tiles, running maximum,
//               P_j = 2^(s - m) as fp16 into swizzled shared memory (the A operand of the second MMA), row sums. The maximum
//               in use only moves when the new one exceeds it by more than 8 (a factor 256, far inside fp16 / fp32 range);
//               then, after the PV product in flight has completed, the warp rescales its O rows in tensor memory
//               (tcgen05.ld / st). At the end O / l goes out as bf16.
// Every wait is bounded; on a timeout the CTA records an error code, the roles leave their loops, copies in flight are waited
// for (bounded) and TMEM is freed.
//
// Role in the reference: the FlashInfer prefill kernels (crates/kernels/cu/flashinfer/README.md:24-31: paged prefill, hd 256,
// GQA 24 / 4, fp8 pool).
#include <cuda.h>
#include "common.cuh"

namespace owl {

__device__ int g_attn_tc_status = 0;

constexpr int AT_BM = 128, AT_BN = 64, AT_HD = 256;
constexpr int AT_Q_BYTES = AT_BM * AT_HD * 2;            // 64 KB: 4 blocks of [128 rows x 128 B]
constexpr int AT_K_BYTES = AT_BN * AT_HD * 2;            // 32 KB: 4 blocks of [64 rows x 128 B]
constexpr int AT_V_BYTES = AT_HD * AT_BN * 2;            // 32 KB: [256 rows x 128 B]
constexpr int AT_P_BYTES = AT_BM * AT_BN * 2;            // 16 KB: [128 rows x 128 B]
constexpr int AT_OFF_K = AT_Q_BYTES, AT_OFF_V = AT_OFF_K + 2 * AT_K_BYTES, AT_OFF_P = AT_OFF_V + 2 * AT_V_BYTES;
constexpr int AT_OFF_CTL = AT_OFF_P + 2 * AT_P_BYTES;    // 224 KB
constexpr int AT_SMEM = AT_OFF_CTL + 2304;          // 231,680 bytes: the dynamic region is declared 1024-aligned
constexpr int AT_THREADS = 320;        // producer warp, MMA warp, 8 softmax warps
constexpr uint32_t AT_COL_S = 0, AT_COL_O = 128;         // TMEM columns: S0, S1 (64 each), O (256)
constexpr float AT_LAZY = 8.f;

struct AtParams {
  __nv_bfloat16* out;
  int rows, gq, pos0, hkv, row_tiles;
  float scale_log2;
};
struct AtCtl {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full[2], p_empty[2], o_done;
  uint64_t pair[4];            // meeting point of the two softmax warps of a lane quarter (64 arrivals per phase)
  uint32_t tmem_base;
  volatile int abort_flag;
  float mx[2][2][AT_BM];       // [tile parity][column half][row]: row maxima of the halves (and, at the end, the halves' sums)
};

static_assert(sizeof(AtCtl) <= 2304, "control block exceeds its reservation");

__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity, AtCtl* c, int code) {
  const uint64_t t0 = global_ns();
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 15u) == 15u && wait_expired(t0)) break;
    if ((i & 255u) == 255u && c->abort_flag) return false;
  }
  c->abort_flag = 1;
  atomicCAS(&g_attn_tc_status, 0, code);
  return false;
}
// The same wait for the hand-offs on the critical path of a tile (scores ready, probabilities ready, the warps' meeting
// point): test_wait polls instead of suspending the thread, whose wake-up costs more than the work it waits for.
__device__ __forceinline__ bool at_spin(uint64_t* bar, uint32_t parity, AtCtl* c, int code) {
  const uint64_t t0 = global_ns();
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 63u) == 63u) {
      if (c->abort_flag) return false;
      if (wait_expired(t0)) break;
    }
  }
  c->abort_flag = 1;
  atomicCAS(&g_attn_tc_status, 0, code);
  return false;
}
// 32 lanes x 32 consecutive 32-bit columns <- 32 registers per thread (lane = TMEM lane)
__device__ __forceinline__ void at_tmem_st_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31]) : "memory");
}

// 2^x on the special-function unit (ex2.approx: 2^-inf = 0, relative error about 2^-22)
__device__ __forceinline__ float at_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(AT_THREADS, 1) attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                const __grid_constant__ CUtensorMap tmK,
                                                                const __grid_constant__ CUtensorMap tmV, AtParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = smem_raw;
  AtCtl* ctl = reinterpret_cast<AtCtl*>(base + AT_OFF_CTL);
  if ((smem_u32(base) & 1023u) != 0u) {              // the swizzled tiles need a 1024-byte aligned base: refuse to run on anything else
    if (threadIdx.x == 0) atomicCAS(&g_attn_tc_status, 0, OWL_ERR_BAD_ARG);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the row tiles with the most key tiles start first
  const int tile = p.row_tiles - 1 - (int)blockIdx.x, kh = blockIdx.y;
  const int row0 = tile * AT_BM;
  const int last_row = min(row0 + AT_BM, p.rows) - 1;
  const int n_kv = (p.pos0 + last_row / p.gq + 1 + AT_BN - 1) / AT_BN;      // key tiles this row tile can see

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->k_full[s], 1); mbar_init(&ctl->k_empty[s], 1);
      mbar_init(&ctl->v_full[s], 1); mbar_init(&ctl->v_empty[s], 1);
      mbar_init(&ctl->s_full[s], 1); mbar_init(&ctl->s_empty[s], 8);
      mbar_init(&ctl->p_full[s], 8); mbar_init(&ctl->p_empty[s], 1);
    }
    mbar_init(&ctl->o_done, 1);
    for (int q = 0; q < 4; ++q) mbar_init(&ctl->pair[q], 64);
    ctl->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&ctl->q_full, AT_Q_BYTES);
      for (int kb = 0; kb < 4; ++kb) tma_load_3d(base + kb * (AT_BM * 128), &tmQ, &ctl->q_full, kb * 64, row0, kh);
      int j = 0;
      for (; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((uint32_t)(j >> 1) & 1u) ^ 1u;
        if (!at_wait(&ctl->k_empty[s], ph, ctl, OWL_ERR_WAIT_MMA)) break;
        mbar_expect_tx(&ctl->k_full[s], AT_K_BYTES);
        uint8_t* ks = base + AT_OFF_K + s * AT_K_BYTES;
        for (int kb = 0; kb < 4; ++kb) tma_load_3d(ks + kb * (AT_BN * 128), &tmK, &ctl->k_full[s], kb * 64, j * AT_BN, kh);
        if (!at_wait(&ctl->v_empty[s], ph, ctl, OWL_ERR_WAIT_MMA)) { ++j; break; }
        mbar_expect_tx(&ctl->v_full[s], AT_V_BYTES);
        tma_load_3d(base + AT_OFF_V + s * AT_V_BYTES, &tmV, &ctl->v_full[s], j * AT_BN, 0, kh);
      }
      if (ctl->abort_flag) {
        // copies already issued still land in this CTA's shared memory: give them a bounded time before the CTA leaves
        for (uint32_t n = 0; n < 256u; ++n)
          if (mbar_try_wait(&ctl->q_full, 0)) break;
        for (int i = max(0, j - 2); i < j; ++i)
          for (uint32_t n = 0; n < 256u; ++n)
            if (mbar_try_wait(&ctl->k_full[i & 1], ((uint32_t)(i >> 1)) & 1u) && mbar_try_wait(&ctl->v_full[i & 1], ((uint32_t)(i >> 1)) & 1u))
              break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_f16(AT_BM, AT_BN, 1), idesc_o = umma_idesc_f16(AT_BM, AT_HD, 0);
      const uint32_t sq = smem_u32(base);
      bool ok = at_wait(&ctl->q_full, 0, ctl, OWL_ERR_WAIT_TMA);
      auto pv = [&](int j) -> bool {        // O (+)= P_j V_j
        const int s = j & 1;
        const uint32_t ph = ((uint32_t)(j >> 1)) & 1u;
        if (!at_spin(&ctl->p_full[s], ph, ctl, OWL_ERR_WAIT_EPI)) return false;
        if (!at_spin(&ctl->v_full[s], ph, ctl, OWL_ERR_WAIT_TMA)) return false;
        tc_fence_after();
        const uint64_t dp = umma_desc_k128(smem_u32(base + AT_OFF_P + s * AT_P_BYTES));
        const uint64_t dv = umma_desc_k128(smem_u32(base + AT_OFF_V + s * AT_V_BYTES));
#pragma unroll
        for (int i = 0; i < 4; ++i)          // 16 keys = 32 bytes of the 128-byte rows per instruction
          tc_mma_f16(tmem + AT_COL_O, dp + (uint64_t)(i * 2), dv + (uint64_t)(i * 2), idesc_o, (j > 0 || i > 0) ? 1u : 0u);
        tc_commit(&ctl->v_empty[s]);
        tc_commit(&ctl->p_empty[s]);
        tc_commit(&ctl->o_done);
        return true;
      };
      for (int j = 0; ok && j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((uint32_t)(j >> 1)) & 1u;
        if (!at_spin(&ctl->k_full[s], ph, ctl, OWL_ERR_WAIT_TMA)) { ok = false; break; }
        if (!at_spin(&ctl->s_empty[s], ph ^ 1u, ctl, OWL_ERR_WAIT_EPI)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sk = smem_u32(base + AT_OFF_K + s * AT_K_BYTES);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const uint64_t dq = umma_desc_k128(sq + kb * (AT_BM * 128)), dk = umma_desc_k128(sk + kb * (AT_BN * 128));
#pragma unroll
          for (int i = 0; i < 4; ++i)
            tc_mma_f16(tmem + AT_COL_S + s * AT_BN, dq + (uint64_t)(i * 2), dk + (uint64_t)(i * 2), idesc_s, (kb > 0 || i > 0) ? 1u : 0u);
        }
        tc_commit(&ctl->k_empty[s]);
        tc_commit(&ctl->s_full[s]);
        if (j > 0 && !pv(j - 1)) { ok = false; break; }
      }
      if (ok && n_kv > 0) pv(n_kv - 1);
    }
  } else {
    // Two warps per TMEM lane quarter: both own the same 32 query rows, each half of a tile's 64 key columns (and half of
    // the O columns when rows are rescaled). They meet once per tile, at an mbarrier of 64 arrivals (a bounded wait like every other), to exchange the
    // row maxima of their halves through shared memory.
    const int q4 = warp & 3, hf = (warp - 2) >> 2;           // lane quarter, column half
    const int r_loc = q4 * 32 + lane, grow = row0 + r_loc;
    const int limit = grow < p.rows ? p.pos0 + grow / p.gq + 1 : 1;      // keys visible to this row (padding rows: one key)
    const uint32_t lane_addr = tmem + ((uint32_t)(q4 * 32) << 16);
    uint8_t* prow_base = base + AT_OFF_P + (r_loc >> 3) * 1024 + (r_loc & 7) * 128;
    float m_used = -INFINITY, l = 0.f;                       // l: this thread's half of the row sum
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      const uint32_t ph = ((uint32_t)(j >> 1)) & 1u;
      if (!__all_sync(0xffffffffu, at_spin(&ctl->s_full[s], ph, ctl, OWL_ERR_WAIT_MMA))) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[32];
      tmem_ld_32x32b_x32(lane_addr + AT_COL_S + s * AT_BN + hf * 32, sv);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->s_empty[s]);
      const int k0 = j * AT_BN + hf * 32;
      // raw scores: the softmax scale (> 0) is folded into the exponent's multiply-add; four independent running maxima
      if (k0 + 32 > limit) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (k0 + c >= limit) sv[c] = 0xff800000u;           // -inf: outside this row's causal limit
      }
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        m4[0] = fmaxf(m4[0], __uint_as_float(sv[c]));     m4[1] = fmaxf(m4[1], __uint_as_float(sv[c + 1]));
        m4[2] = fmaxf(m4[2], __uint_as_float(sv[c + 2])); m4[3] = fmaxf(m4[3], __uint_as_float(sv[c + 3]));
      }
      float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
      ctl->mx[s][hf][r_loc] = mx;
      mbar_arrive(&ctl->pair[q4]);                           // (arrive has release, the wait acquire semantics)
      if (!__all_sync(0xffffffffu, at_spin(&ctl->pair[q4], (uint32_t)j & 1u, ctl, OWL_ERR_WAIT_EPI))) { ok = false; break; }
      mx = fmaxf(mx, ctl->mx[s][hf ^ 1][r_loc]);             // both warps of the row now hold the same maximum
      // Rows whose every key of this tile is masked keep their maximum (a tile past the row's limit inside the row tile).
      const bool grow_m = mx > m_used + AT_LAZY;
      const unsigned any_here = __any_sync(0xffffffffu, grow_m);
      if (any_here) {
        const float m_new = grow_m ? mx : m_used;
        const float f = (m_used == -INFINITY) ? 0.f : at_ex2(m_used - m_new);
        if (j > 0) {
          // the product that still adds to O must have completed before its rows are rescaled
          if (!__all_sync(0xffffffffu, at_wait(&ctl->o_done, ((uint32_t)(j - 1)) & 1u, ctl, OWL_ERR_WAIT_MMA))) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < AT_HD / 64; ++c) {             // this warp's half of the O columns
            uint32_t o[32];
            tmem_ld_32x32b_x32(lane_addr + AT_COL_O + hf * (AT_HD / 2) + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int v = 0; v < 32; ++v) o[v] = __float_as_uint(__uint_as_float(o[v]) * f);
            at_tmem_st_x32(lane_addr + AT_COL_O + hf * (AT_HD / 2) + c * 32, o);
          }
          tc_wait_st();
          tc_fence_before();
        }
        l *= f;
        m_used = m_new;
      }
      // P_j (fp16) into the swizzled A-operand tile; the buffer is free once the product two tiles back has read it
      if (!__all_sync(0xffffffffu, at_spin(&ctl->p_empty[s], ph ^ 1u, ctl, OWL_ERR_WAIT_MMA))) { ok = false; break; }
      uint8_t* prow = prow_base + s * AT_P_BYTES;
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
      const float nm = -m_used;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float e[8];
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          e[v] = at_ex2(fmaf(__uint_as_float(sv[c * 8 + v]), p.scale_log2, nm));
          s4[v & 3] += e[v];
        }
        *reinterpret_cast<uint4*>(prow + (((hf * 4 + c) ^ (r_loc & 7)) << 4)) =
            make_uint4(pack_f16(e[0], e[1]), pack_f16(e[2], e[3]), pack_f16(e[4], e[5]), pack_f16(e[6], e[7]));
      }
      l += (s4[0] + s4[1]) + (s4[2] + s4[3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->p_full[s]);
    }
    // the two halves of every row sum meet; then each warp writes its half of the output columns
    ctl->mx[n_kv & 1][hf][r_loc] = l;                         // the parity buffer the last tile did not use
    if (ok) {
      mbar_arrive(&ctl->pair[q4]);
      ok = __all_sync(0xffffffffu, at_wait(&ctl->pair[q4], (uint32_t)n_kv & 1u, ctl, OWL_ERR_WAIT_EPI));
    }
    l += ctl->mx[n_kv & 1][hf ^ 1][r_loc];
    if (ok && n_kv > 0 && __all_sync(0xffffffffu, at_wait(&ctl->o_done, ((uint32_t)(n_kv - 1)) & 1u, ctl, OWL_ERR_WAIT_MMA))) {
      tc_fence_after();
      const float inv = 1.f / l;
      __nv_bfloat16* orow = p.out + ((size_t)kh * p.rows + grow) * AT_HD + hf * (AT_HD / 2);
#pragma unroll 1
      for (int c = 0; c < AT_HD / 64; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(lane_addr + AT_COL_O + hf * (AT_HD / 2) + c * 32, o);
        tc_wait_ld();
        if (grow < p.rows) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(o[v * 8 + 0]) * inv, __uint_as_float(o[v * 8 + 1]) * inv);
            pk.y = pack_bf16(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv);
            pk.z = pack_bf16(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv);
            pk.w = pack_bf16(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = pk;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AtEncodeFn at_encode() {
  static AtEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AtEncodeFn>(p);
  }
  return fn;
}
// [d2][d1][d0] 16-bit tensor, box d0 = 64 elements (128 bytes, swizzled) x box1 rows x 1
static int at_map(CUtensorMap* m, const void* ptr, CUtensorMapDataType dt, long long d0, long long d1, long long d2, int box1) {
  AtEncodeFn enc = at_encode();
  if (!enc) return OWL_ERR_LAUNCH * 1000 - 1;
  cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2};
  cuuint64_t strides[2] = {(cuuint64_t)d0 * 2, (cuuint64_t)d0 * (cuuint64_t)d1 * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OWL_OK : OWL_ERR_LAUNCH * 1000 - (int)r;
}

}  // namespace owl
using namespace owl;

// qg bf16 [hkv][rows][256] (rows = tokens x gq, token-major), k bf16 [hkv][ctx_pad][256], vt fp16 [hkv][256][ctx_pad],
// og bf16 [hkv][rows][256]. Row r sees keys < pos0 + r / gq + 1 (which must not exceed ctx_pad; ctx_pad a multiple of 64).
OWL_API int owl_attn_tc(const void* qg, const void* k, const void* vt, void* og, int rows, int gq, int hkv, int ctx_pad, int pos0,
                        float scale, cudaStream_t st) {
  if (!qg || !k || !vt || !og || rows < 1 || gq < 1 || hkv < 1 || ctx_pad < 64 || (ctx_pad & 63) || pos0 < 0 ||
      pos0 + (rows - 1) / gq + 1 > ctx_pad || (reinterpret_cast<uintptr_t>(qg) & 15) || (reinterpret_cast<uintptr_t>(k) & 15) ||
      (reinterpret_cast<uintptr_t>(vt) & 15) || (reinterpret_cast<uintptr_t>(og) & 15))
    return OWL_ERR_BAD_ARG;
  CUtensorMap mq, mk, mv;
  int r = at_map(&mq, qg, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, AT_HD, rows, hkv, AT_BM);
  if (r) return r;
  r = at_map(&mk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, AT_HD, ctx_pad, hkv, AT_BN);
  if (r) return r;
  r = at_map(&mv, vt, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, ctx_pad, AT_HD, hkv, AT_HD);
  if (r) return r;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM) != cudaSuccess)
      return OWL_ERR_LAUNCH * 1000;
    attr = true;
  }
  AtParams p = {};
  p.out = (__nv_bfloat16*)og; p.rows = rows; p.gq = gq; p.pos0 = pos0; p.hkv = hkv;
  p.row_tiles = (rows + AT_BM - 1) / AT_BM;
  p.scale_log2 = scale * 1.4426950408889634f;
  attn_tc_kernel<<<dim3(p.row_tiles, hkv), AT_THREADS, AT_SMEM, st>>>(mq, mk, mv, p);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

OWL_API int owl_attn_tc_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_tc_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_attn_tc_status, &zero, sizeof(int));
  return v;
}
