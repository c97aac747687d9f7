// Decode-shape W4A16 weight streaming on the 5th-generation tensor cores (sm_100a).
//
//   owl_w4a16_stream_tc : out[M, N] = ActPack(x)[M, K] . dequant(W4 records)[N, K]^T,  M <= 8
//
// The legacy integer MMA / dp4a streaming kernels (gemv.cu) are bound by instruction issue: every
// nibble costs a CUDA-core or legacy-MMA instruction slot. Here the contraction itself runs on
// tcgen05.mma kind::i8 with BOTH the weight operand and the accumulators in tensor memory, so the
// CUDA cores only split nibbles into bytes (one AND, one shift + AND per 8 weights) and apply
// scales once per group, and shared memory carries the packed bytes once.
//
// Weights are read in the block-major record layout (records.cuh): a block = 128 weight rows x
// 128 k = 8 records = one contiguous run, and consecutive k of a row block follow each other, so
// the whole range of a CTA is one contiguous stream and a ring stage (one block, 8.5 KB) is ONE
// bulk copy (cp.async.bulk, no multicast) issued by the producer warp; stage s always serves the
// same warp group, which releases it as soon as the block sits in its registers.
//
// One warp executes dependent instructions only every few cycles, so the time per block is set by
// the longest per-warp instruction chain and by the number of hand-offs between warps. Blocks are
// therefore dealt round-robin to four independent warp groups (4 warps = the 4 TMEM lane
// quarters); a group does everything for its block and only talks to itself:
//
//   unpack    warp q owns TMEM lanes 32q..32q+31 = two 16-row records. The record's chunk order is
//             the mma fragment order (lane = row % 8 * 4 + k piece), so two 16-byte loads per lane,
//             16 AND / shift ops and one tcgen05.st.16x256b.x4 put a record into the A operand
//             (TMEM lane = weight row, 8 columns per 32-k MMA step). The k order inside an MMA step
//             is the record's own nibble order; the activation tile uses the same order, and a
//             contraction does not care.
//   (B)       the activation producers write ActPack directly as the B operand (columns = token x
//             {high, low} plane, unswizzled K-major core matrices) followed by the per-group
//             activation scales, one 2 KB run per k-record, so the producer warp fetches it with a
//             second bulk copy into the same ring stage: no thread touches activation bytes
//   epilogue  of the group's PREVIOUS block (its MMA ran while this block was unpacked):
//             tcgen05.ld the int32 sums, acc += s * (sx * (128 * acc_h + acc_l) - z * xsum)
//   MMA       a fifth warp per group waits until the four warps have signalled, then issues
//             4 x tcgen05.mma (M128 N16 K32, u8 x s8 -> s32, A from TMEM) and a commit
//
// Work split (stream-K): the (row block, k-record) sequence is cut into equal contiguous ranges,
// one per CTA (one CTA per SM). A CTA flushes its fp32 partial sums whenever its range leaves a
// row block; partials of a row block that several CTAs share go to a scratch buffer and the last
// CTA to arrive (per-warp ticket) adds them in slot order, so the result does not depend on
// timing. Epilogues: bf16 store, residual add, silu(gate) * up, fp32 store.
//
// Every mbarrier wait is bounded; on a timeout the CTA records an error code and every role
// leaves its loop (the rendezvous of a group's four warps is an mbarrier too),
// copies in flight are waited for (bounded) and TMEM is freed before the CTA exits.
//
// Role in the reference: the Marlin W4A16 decode GEMMs (crates/kernels/cu/marlin/*); the
// reference has no tcgen05 path.
#include "common.cuh"
#include "records.cuh"
#include "actpack.cuh"

namespace owl {

__device__ int g_stream_tc_status = 0;

constexpr int VT_NG = 4;                   // warp groups (blocks are dealt round-robin)
constexpr int VT_BTILE = 4 * 512;          // B of one block: 4 steps x (16 columns x 32 bytes)
constexpr int VT_THREADS = (VT_NG * 5 + 1) * 32;
constexpr int VT_W_PROD = VT_NG * 4, VT_W_MMA = VT_NG * 4 + 1;    // warps 0-15 compute, 16 producer, 17-20 MMA issuers
constexpr int VT_TMEM_COLS = 512;          // [0,256): 4 groups x 2 A buffers x 32, [256,512): accumulators
constexpr int VT_ACC0 = 256;

enum { VEPI_STORE = 0, VEPI_RESIDUAL = 1, VEPI_SILU_MUL = 2, VEPI_F32 = 3 };

template <int G> struct VtCfg {
  static constexpr int GPT = 128 / G;                       // scale groups per record
  static constexpr int REC = 1024 + 64 * GPT;
  static constexpr int BLK = 8 * REC;                       // one weight block (one bulk copy)
  static constexpr int ACT = VT_BTILE + 64 * GPT;           // the block's activation tile + (sx, xsum) pairs (one bulk copy)
  static constexpr int STAGE = BLK + ACT;                   // one ring stage
  static constexpr int ACCW = 16 * GPT;                     // accumulator columns per block
  static constexpr int STAGES = 16;                         // multiple of VT_NG: a stage always serves the same group
  static constexpr int OFF_RED = STAGES * STAGE;
  static constexpr int OFF_CTL = OFF_RED + (VT_NG - 1) * 128 * 8 * 4;
  static constexpr int SMEM = OFF_CTL + 512 + 128 /*alignment slack*/;
};

struct VtCtl {
  uint64_t pk_full[20], pk_empty[20];
  uint64_t acc_full[VT_NG], grp[VT_NG], red_full[4], red_empty[4];
  uint32_t tmem_base;
  volatile int abort_flag;
};

struct VtParams {
  const uint8_t* w;       // block-major record stream
  const uint8_t* x;       // ActPack in tile layout (actpack.cuh): K/128 runs of VtCfg::ACT bytes
  void* out;
  const __nv_bfloat16* residual;
  float* scratch;         // [NRB][slots][128][MT] partial sums
  int* counters;          // [NRB][4] arrival tickets, zero between launches
  int M, N, K, ldo;
  int NT, KT, NRB;        // row tiles, k-records, 128-row blocks
  int TB, per, slots;     // total blocks, blocks per CTA, partial slots per row block
};

__device__ __forceinline__ bool vt_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __noinline__ bool vt_wait_slow(uint64_t* bar, uint32_t parity, VtCtl* ctl, int code) {
  // the hinted try_wait parks the warp in hardware until the phase completes: a spinning warp
  // would take issue slots from the warps it is waiting for
  const uint64_t t0 = global_ns();
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 15u) == 15u && wait_expired(t0)) break;
    if ((i & 255u) == 255u && ctl->abort_flag) return false;
  }
  ctl->abort_flag = 1;
  atomicCAS(&g_stream_tc_status, 0, code);
  return false;
}
// Bounded wait; the common case (phase already complete) costs one try_wait.
__device__ __forceinline__ bool vt_wait(uint64_t* bar, uint32_t parity, VtCtl* ctl, int code) {
  if (vt_try_wait(bar, parity)) return true;
  return vt_wait_slow(bar, parity, ctl, code);
}

__device__ __forceinline__ void vt_bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
// Tuning aid, compiled only with -DOWL_VT_TRACE: thread 0 (compute) and the MMA issuer of group 0 in
// CTA 0 keep clock stamps of their first 64 steps in shared memory, copied to a global array at exit.
#ifdef OWL_VT_TRACE
__device__ unsigned g_vt_trace[64 * 16];
#define VT_STAMP(cond, i, pt) do { if (blockIdx.x == 0 && (cond) && (i) < 64) vtrace[(i) * 16 + (pt)] = (unsigned)clock(); } while (0)
#else
#define VT_STAMP(cond, i, pt) do { } while (0)
#endif

__device__ __forceinline__ float vt_silu(float x) { return x / (1.f + __expf(-x)); }

template <int G, int MT>
__global__ void __launch_bounds__(VT_THREADS, 1) stream_tc_kernel(VtParams p, int epi) {
  using C = VtCfg<G>;
  constexpr int GPT = C::GPT, REC = C::REC, S = C::STAGES, ACCW = C::ACCW;
  constexpr int NLD = MT <= 4 ? 4 : 8;     // accumulator columns read per plane
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  uint8_t* pk = base;
  float* red = reinterpret_cast<float*>(base + C::OFF_RED);
  VtCtl* ctl = reinterpret_cast<VtCtl*>(base + C::OFF_CTL);
#ifdef OWL_VT_TRACE
  __shared__ unsigned vtrace[64 * 16];
  for (int i = threadIdx.x; i < 64 * 16; i += VT_THREADS) vtrace[i] = 0;
#endif

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KT = p.KT;
  const int lo = blockIdx.x * p.per, hi = min(lo + p.per, p.TB);
  const int nb = hi - lo;
#ifdef OWL_VT_TRACE
  const bool dry = epi >= 100;   // tuning aid: consumers only release the packed stages
#else
  constexpr bool dry = false;
#endif

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&ctl->pk_full[s], 1); mbar_init(&ctl->pk_empty[s], 4); }
    for (int i = 0; i < VT_NG; ++i) { mbar_init(&ctl->acc_full[i], 1); mbar_init(&ctl->grp[i], 4); }
    for (int i = 0; i < 4; ++i) { mbar_init(&ctl->red_full[i], VT_NG - 1); mbar_init(&ctl->red_empty[i], 1); }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&ctl->tmem_base, VT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == VT_W_PROD) {
    // ------------------------------- producer -------------------------------------------------
    // Weights are static: the first ring fill starts before the previous kernel has finished; the
    // activation tiles (written by that kernel) follow after the dependency wait.
    if (lane == 0) {
      const uint8_t* src = p.w + (size_t)lo * C::BLK;
      int kt = lo % KT, b = 0, s = 0;
      uint32_t ph = 0;
      const int pre = min(nb, S);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&ctl->pk_full[i], (uint32_t)C::STAGE);
        vt_bulk_g2s(pk + (size_t)i * C::STAGE, src + (size_t)i * C::BLK, (uint32_t)C::BLK, &ctl->pk_full[i]);
      }
      pdl_wait();
      for (; b < pre; ++b) {
        vt_bulk_g2s(pk + (size_t)b * C::STAGE + C::BLK, p.x + (size_t)kt * C::ACT, (uint32_t)C::ACT, &ctl->pk_full[b]);
        if (++kt == KT) kt = 0;
      }
      ph = 1u;      // stage 0 comes around again: wait for its first release
      for (; b < nb; ++b) {
        if (!vt_wait(&ctl->pk_empty[s], ph ^ 1u, ctl, OWL_ERR_WAIT_EPI)) break;
        mbar_expect_tx(&ctl->pk_full[s], (uint32_t)C::STAGE);
        vt_bulk_g2s(pk + (size_t)s * C::STAGE, src + (size_t)b * C::BLK, (uint32_t)C::BLK, &ctl->pk_full[s]);
        vt_bulk_g2s(pk + (size_t)s * C::STAGE + C::BLK, p.x + (size_t)kt * C::ACT, (uint32_t)C::ACT, &ctl->pk_full[s]);
        if (++kt == KT) kt = 0;
        if (++s == S) { s = 0; ph ^= 1u; }
      }
      if (ctl->abort_flag) {
        // copies that were issued but will never be consumed: wait (bounded) for them to land
        for (int i = max(0, b - S); i < b; ++i)
          for (uint32_t n = 0; n < 256u; ++n)
            if (mbar_try_wait(&ctl->pk_full[i % S], ((uint32_t)(i / S)) & 1u)) break;
      }
    }
  } else if (warp >= VT_W_MMA) {
    // ------------------------------- MMA issuer of group g -------------------------------------
    // tcgen05.mma issue is slow (about a hundred cycles per instruction for these small tiles), so
    // it has a warp of its own: the compute warps only signal and move on.
    if (lane == 0 && !dry) {
      const int g = warp - VT_W_MMA;
      const uint32_t idesc = umma_idesc_i8(128, 16, 0, 1);
      const uint64_t db_base = umma_desc_k_noswz(smem_u32(pk + C::BLK), 256, 128);
      uint32_t grp_ph = 0;
      int step = 0, s = g;
      for (int b = g; b < nb; b += 4, ++step) {
        const int abuf = step & 1;
        // all four warps of the group: A operand stored, B tile landed, previous sums read out
        if (!vt_wait(&ctl->grp[g], grp_ph, ctl, OWL_ERR_WAIT_EPI)) break;
        grp_ph ^= 1u;
        if (!vt_wait(&ctl->pk_full[s], ((uint32_t)(b / S)) & 1u, ctl, OWL_ERR_WAIT_TMA)) break;   // long complete: orders the tile's arrival before the MMA
        VT_STAMP(g == 0, step, 10);
        tc_fence_after();
        const uint64_t db = db_base + (uint64_t)(s * (C::STAGE >> 4));      // the stage's activation tile
        const uint32_t ta = tmem + (g * 2 + abuf) * 32, td = tmem + VT_ACC0 + g * ACCW;
        if (G == 128) {
          tc_mma_i8_ts(td, ta, db, idesc, 0u);
          tc_mma_i8_ts(td, ta + 8, db + 32, idesc, 1u);
          tc_mma_i8_ts(td, ta + 16, db + 64, idesc, 1u);
          tc_mma_i8_ts(td, ta + 24, db + 96, idesc, 1u);
        } else {
          tc_mma_i8_ts(td, ta, db, idesc, 0u);
          tc_mma_i8_ts(td + 16, ta + 8, db + 32, idesc, 0u);
          tc_mma_i8_ts(td + 32, ta + 16, db + 64, idesc, 0u);
          tc_mma_i8_ts(td + 48, ta + 24, db + 96, idesc, 0u);
        }
        tc_commit(&ctl->acc_full[g]);
        VT_STAMP(g == 0, step, 11);
        s += 4; if (s >= S) s -= S;
      }
    }
  } else {
    // ------------------------------- compute group g -------------------------------------------
    const int g = warp >> 2, q4 = warp & 3, gt = tid & 127, row = q4 * 32 + lane;
    const uint32_t tq = tmem + ((uint32_t)(q4 * 32) << 16);          // this warp's TMEM lane quarter
    const uint32_t t_acc = tq + VT_ACC0 + g * ACCW;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    uint32_t sz_prev[GPT];          // (s, z) of this thread's row for the block whose MMA is in flight
    int prev_s = 0;                 // ring stage of that block (holds its activation scales; released after its MMA)
    bool pend = false;              // a block of this group has its MMA issued and its epilogue pending
    uint32_t acc_ph = 0;            // parity of the next acc_full completion to wait for
    bool ok = true;
    int step = 0;                   // own blocks processed so far

    // Epilogue of the pending block: wait for its MMA, read the sums, scale into acc.
    auto epilogue = [&]() -> bool {
      if (!vt_wait(&ctl->acc_full[g], acc_ph, ctl, OWL_ERR_WAIT_MMA)) return false;
      acc_ph ^= 1u;
      VT_STAMP(tid == 0, step, 4);
      tc_fence_after();
      uint32_t rh[GPT][NLD], rl[GPT][NLD];     // high-plane / low-plane sums of tokens 0..NLD-1
#pragma unroll
      for (int gi = 0; gi < GPT; ++gi) {
        if (NLD == 4) { tmem_ld_32x32b_x4(t_acc + gi * 16, rh[gi]); tmem_ld_32x32b_x4(t_acc + gi * 16 + 8, rl[gi]); }
        else {
          uint32_t r16[16];
          tmem_ld_32x32b_x16(t_acc + gi * 16, r16);
#pragma unroll
          for (int m = 0; m < NLD; ++m) { rh[gi][m] = r16[m]; rl[gi][m] = r16[8 + m]; }
        }
      }
      float2 xv[GPT][MT];
#pragma unroll
      for (int gi = 0; gi < GPT; ++gi)
#pragma unroll
        for (int m = 0; m < MT; ++m)
          xv[gi][m] = *reinterpret_cast<const float2*>(pk + (size_t)prev_s * C::STAGE + C::BLK + VT_BTILE + (gi * 8 + m) * 8);
      tc_wait_ld();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->pk_empty[prev_s]);    // its MMA is done with the activation tile: release the stage
#pragma unroll
      for (int gi = 0; gi < GPT; ++gi) {
        const __half2 h = *reinterpret_cast<const __half2*>(&sz_prev[gi]);
        const float sc = __low2float(h), zz = __high2float(h);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const int v = ((int)rh[gi][m] << 7) + (int)rl[gi][m];
          acc[m] = fmaf(sc, fmaf(xv[gi][m].x, (float)v, -zz * xv[gi][m].y), acc[m]);
        }
      }
      pend = false;
      return true;
    };

    // Final epilogue for this thread's output row of row block rb.
    auto finalize = [&](int rb, const float* v) {
      const int n = rb * 128 + row;
      const bool valid = n < p.N;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float other = __shfl_xor_sync(0xffffffffu, v[m], 8);
        if (!valid || m >= p.M) continue;
        if (epi == VEPI_SILU_MUL) {
          if (!(row & 8))
            reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + (n >> 4) * 8 + (n & 7)] =
                __float2bfloat16(vt_silu(v[m]) * other);
        } else if (epi == VEPI_F32) {
          reinterpret_cast<float*>(p.out)[(size_t)m * p.ldo + n] = v[m];
        } else {
          float a = v[m];
          if (epi == VEPI_RESIDUAL) a += __bfloat162float(p.residual[(size_t)m * p.ldo + n]);
          reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16(a);
        }
      }
    };

    pdl_wait();   // activations, residual and output belong to the previous kernel until now
    // this group's blocks are CTA-local b = g, g + 4, ...
    int b = g, nflush = 0;
    int s = g;                         // ring stage of block b (b % S)
    uint32_t ph = 0;

    for (int seg_lo = lo; seg_lo < hi && ok;) {
      const int rb = seg_lo / KT;
      const int seg_hi = min(hi, (rb + 1) * KT);
      for (; lo + b < seg_hi && !dry; b += 4) {
        const int abuf = step & 1;
        const uint8_t* blk = pk + (size_t)s * C::STAGE;
        VT_STAMP(tid == 0, step, 0);
        if (!vt_wait(&ctl->pk_full[s], ph, ctl, OWL_ERR_WAIT_TMA)) { ok = false; break; }
        VT_STAMP(tid == 0, step, 1);
        // ---- unpack this warp's two records into the A operand -------------------------------
        const uint8_t* rec = blk + (size_t)(2 * q4) * REC + lane * 16;
        const uint4 v0 = *reinterpret_cast<const uint4*>(rec);                // record 2q, row lane / 4
        const uint4 v1 = *reinterpret_cast<const uint4*>(rec + 512);          // record 2q, row 8 + lane / 4
        const uint4 v2 = *reinterpret_cast<const uint4*>(rec + REC);          // record 2q + 1
        const uint4 v3 = *reinterpret_cast<const uint4*>(rec + REC + 512);
        uint32_t sz_cur[GPT];
#pragma unroll
        for (int gi = 0; gi < GPT; ++gi)
          sz_cur[gi] = *reinterpret_cast<const uint32_t*>(blk + (row >> 4) * REC + 1024 + gi * 64 + (row & 15) * 4);
        VT_STAMP(tid == 0, step, 2);
        {
          uint32_t a[16];
          a[0] = v0.x & 0x0f0f0f0fu;  a[1] = (v0.x >> 4) & 0x0f0f0f0fu;  a[2] = v1.x & 0x0f0f0f0fu;  a[3] = (v1.x >> 4) & 0x0f0f0f0fu;
          a[4] = v0.y & 0x0f0f0f0fu;  a[5] = (v0.y >> 4) & 0x0f0f0f0fu;  a[6] = v1.y & 0x0f0f0f0fu;  a[7] = (v1.y >> 4) & 0x0f0f0f0fu;
          a[8] = v0.z & 0x0f0f0f0fu;  a[9] = (v0.z >> 4) & 0x0f0f0f0fu;  a[10] = v1.z & 0x0f0f0f0fu; a[11] = (v1.z >> 4) & 0x0f0f0f0fu;
          a[12] = v0.w & 0x0f0f0f0fu; a[13] = (v0.w >> 4) & 0x0f0f0f0fu; a[14] = v1.w & 0x0f0f0f0fu; a[15] = (v1.w >> 4) & 0x0f0f0f0fu;
          VT_STAMP(tid == 0, step, 12);
          tmem_st_16x256b_x4(tq + (g * 2 + abuf) * 32, a);
          VT_STAMP(tid == 0, step, 13);
          a[0] = v2.x & 0x0f0f0f0fu;  a[1] = (v2.x >> 4) & 0x0f0f0f0fu;  a[2] = v3.x & 0x0f0f0f0fu;  a[3] = (v3.x >> 4) & 0x0f0f0f0fu;
          a[4] = v2.y & 0x0f0f0f0fu;  a[5] = (v2.y >> 4) & 0x0f0f0f0fu;  a[6] = v3.y & 0x0f0f0f0fu;  a[7] = (v3.y >> 4) & 0x0f0f0f0fu;
          a[8] = v2.z & 0x0f0f0f0fu;  a[9] = (v2.z >> 4) & 0x0f0f0f0fu;  a[10] = v3.z & 0x0f0f0f0fu; a[11] = (v3.z >> 4) & 0x0f0f0f0fu;
          a[12] = v2.w & 0x0f0f0f0fu; a[13] = (v2.w >> 4) & 0x0f0f0f0fu; a[14] = v3.w & 0x0f0f0f0fu; a[15] = (v3.w >> 4) & 0x0f0f0f0fu;
          VT_STAMP(tid == 0, step, 14);
          tmem_st_16x256b_x4(tq + ((uint32_t)16 << 16) + (g * 2 + abuf) * 32, a);
        }
        VT_STAMP(tid == 0, step, 3);
        // ---- previous block of this group: its MMA ran meanwhile -----------------------------
        if (pend && !epilogue()) { ok = false; break; }
        VT_STAMP(tid == 0, step, 5);
        tc_wait_st();
        tc_fence_before();
        VT_STAMP(tid == 0, step, 6);
        // tell the group's MMA issuer: A operand stored, previous sums read out
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->grp[g]);
        VT_STAMP(tid == 0, step, 7);
#pragma unroll
        for (int gi = 0; gi < GPT; ++gi) sz_prev[gi] = sz_cur[gi];
        prev_s = s;
        pend = true;
        VT_STAMP(tid == 0, step, 8);
        ++step;
        s += 4; if (s >= S) { s -= S; ph ^= 1u; }
      }
      if (!ok) break;
      if (dry) {
        for (; lo + b < seg_hi; b += 4) {
          if (!vt_wait(&ctl->pk_full[s], ph, ctl, OWL_ERR_WAIT_TMA)) { ok = false; break; }
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->pk_empty[s]);
          s += 4; if (s >= S) { s -= S; ph ^= 1u; }
        }
        seg_lo = seg_hi;
        continue;
      }
      // ---- segment end: drain, combine the groups, flush ----------------------------------------
      if (pend && !epilogue()) { ok = false; break; }
      if (g != 0) {
        if (!vt_wait(&ctl->red_empty[q4], ((uint32_t)nflush & 1u) ^ 1u, ctl, OWL_ERR_WAIT_EPI)) { ok = false; break; }
#pragma unroll
        for (int m = 0; m < MT; ++m) { red[((g - 1) * 128 + row) * 8 + m] = acc[m]; acc[m] = 0.f; }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->red_full[q4]);
      } else {
        if (!vt_wait(&ctl->red_full[q4], (uint32_t)nflush & 1u, ctl, OWL_ERR_WAIT_EPI)) { ok = false; break; }
#pragma unroll
        for (int o = 0; o < VT_NG - 1; ++o)
#pragma unroll
          for (int m = 0; m < MT; ++m) acc[m] += red[(o * 128 + row) * 8 + m];
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->red_empty[q4]);
        const int c0 = (rb * KT) / p.per, c1 = ((rb + 1) * KT - 1) / p.per, cnt = c1 - c0 + 1;
        if (cnt == 1) {
          finalize(rb, acc);
        } else {
          float* mine = p.scratch + (((size_t)rb * p.slots + (blockIdx.x - c0)) * 128 + row) * MT;
#pragma unroll
          for (int m = 0; m < MT; ++m) __stcg(mine + m, acc[m]);
          __threadfence();
          __syncwarp();
          int ticket = 0;
          if (lane == 0) ticket = atomicAdd(&p.counters[rb * 4 + q4], 1);
          ticket = __shfl_sync(0xffffffffu, ticket, 0);
          if (ticket == cnt - 1) {     // last of this row quarter: add all partials in slot order
            __threadfence();
            float tot[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) tot[m] = 0.f;
            for (int sl = 0; sl < cnt; ++sl) {
              const float* o = p.scratch + (((size_t)rb * p.slots + sl) * 128 + row) * MT;
#pragma unroll
              for (int m = 0; m < MT; ++m) tot[m] += __ldcg(o + m);
            }
            finalize(rb, tot);
            if (lane == 0) p.counters[rb * 4 + q4] = 0;
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.f;
      }
      ++nflush;
      seg_lo = seg_hi;
    }
    if (!ok) ctl->abort_flag = 1;
  }

  tc_fence_before();
  __syncthreads();
#ifdef OWL_VT_TRACE
  if (blockIdx.x == 0) for (int i = threadIdx.x; i < 64 * 16; i += VT_THREADS) g_vt_trace[i] = vtrace[i];
#endif
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, VT_TMEM_COLS);
  }
  pdl_launch_dependents();
}

// Stream-K split of TB blocks over at most `ctas` CTAs.
static void vt_plan(int KT, int TB, int ctas, int* grid, int* per, int* slots) {
  int g = ctas < TB ? ctas : TB;
  if (g < 1) g = 1;
  const int pr = (TB + g - 1) / g;
  *grid = (TB + pr - 1) / pr; *per = pr; *slots = (KT - 1) / pr + 2;
}

template <int G, int MT>
static int launch_stream_tc(VtParams p, int epi, int ctas, long long scratch_bytes, long long counter_bytes, int pdl,
                            cudaStream_t st) {
  auto kernel = stream_tc_kernel<G, MT>;
  constexpr int smem = VtCfg<G>::SMEM;
  static int resident = 0;     // CTAs that fit on the device at once (SMs x occupancy)
  if (!resident) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
    int dev = 0, sms = 0, occ = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, VT_THREADS, smem);
    if (e != cudaSuccess || occ < 1 || sms < 1) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
    if (occ > 512 / VT_TMEM_COLS) occ = 512 / VT_TMEM_COLS;     // tensor memory: 512 columns per SM
    resident = sms * occ;
  }
  int grid;
  vt_plan(p.KT, p.TB, ctas > 0 ? ctas : resident, &grid, &p.per, &p.slots);
  if ((long long)p.NRB * p.slots * 128 * MT * 4 > scratch_bytes || (long long)p.NRB * 16 > counter_bytes)
    return OWL_ERR_BAD_ARG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(VT_THREADS);
  cfg.dynamicSmemBytes = smem;
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

template <int G>
static int dispatch_stream_tc(const VtParams& p, int epi, int ctas, long long sb, long long cb, int pdl, cudaStream_t st) {
  if (p.M == 1) return launch_stream_tc<G, 1>(p, epi, ctas, sb, cb, pdl, st);
  if (p.M == 2) return launch_stream_tc<G, 2>(p, epi, ctas, sb, cb, pdl, st);
  if (p.M <= 4) return launch_stream_tc<G, 4>(p, epi, ctas, sb, cb, pdl, st);
  return launch_stream_tc<G, 8>(p, epi, ctas, sb, cb, pdl, st);
}

}  // namespace owl

using namespace owl;


// xpack: activations in the ActPack tile layout (producers called with group | ACT_TILES).
// out[M, ldo] (bf16, fp32 with epi = 3). M <= 8. epi: 0 store, 1 residual add, 2 silu(gate) * up with
// gate / up rows interleaved per 16-row tile (rows 0-7 gate, 8-15 up; out has N/2 columns), 3 fp32.
// ctas: CTAs to split the work over (0 = every CTA slot of the device). scratch holds the split-K
// partial sums: (ctas + 2 * ceil(N/128)) * 128 * 8 floats always suffice; counters: 4 ints per 128
// rows, zero before the first launch and left zero by every launch.
OWL_API int owl_w4a16_stream_tc(const void* records, const void* xpack, void* out,
                                const void* residual, void* scratch, long long scratch_bytes, void* counters,
                                long long counter_bytes, int M, int N, int K, int ldo, int group, int epi, int ctas,
                                int pdl, cudaStream_t st) {
#ifdef OWL_VT_TRACE
  const bool epi_ok = (epi >= 0 && epi <= 3) || epi >= 100;
#else
  const bool epi_ok = epi >= 0 && epi <= 3;
#endif
  if (M < 1 || M > 8 || (group != 32 && group != 128) || !epi_ok || !out || !records || !xpack)
    return OWL_ERR_BAD_ARG;
  if (N < 16 || (N & 15) || K < 128 || (K & 127) || !scratch || !counters) return OWL_ERR_BAD_ARG;
  if (epi == VEPI_RESIDUAL && !residual) return OWL_ERR_BAD_ARG;
  VtParams p = {};
  p.w = (const uint8_t*)records; p.x = (const uint8_t*)xpack;
  p.out = out; p.residual = (const __nv_bfloat16*)residual;
  p.scratch = (float*)scratch; p.counters = (int*)counters;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo;
  p.NT = N / 16; p.KT = K / 128; p.NRB = (p.NT + 7) / 8;
  p.TB = p.NRB * p.KT;
  return group == 128 ? dispatch_stream_tc<128>(p, epi, ctas, scratch_bytes, counter_bytes, pdl, st)
                      : dispatch_stream_tc<32>(p, epi, ctas, scratch_bytes, counter_bytes, pdl, st);
}

#ifdef OWL_VT_TRACE
OWL_API int owl_stream_tc_trace(void* host_dst) {
  return (int)cudaMemcpyFromSymbol(host_dst, g_vt_trace, sizeof(unsigned) * 64 * 16);
}
#endif

OWL_API int owl_stream_tc_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_stream_tc_status, sizeof(int));
  return v;
}
