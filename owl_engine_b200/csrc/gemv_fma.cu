// One-token W4A16 projection on the half-precision FMA pipe, with the producer / consumer glue of a decode
// step folded into its prologue and epilogue.
//
//   owl_w4_fma : y[N] = dequant(W4 g128)[N,K] . x[K]            (one token)
//     prologue : x = the bf16 activation vector as is, or rmsnorm(h) * (1 + w) computed here from the residual
//                stream (every CTA normalises the row itself: 10 KB from L2, no separate norm kernel, no packed
//                activation buffer in global memory)
//     epilogue : bf16 store | residual add (h += y) | silu(gate) * up
//     side job : a few dense bf16 rows (the GDN a / b gate projections) are multiplied by warps of the same
//                grid, so that they need neither a launch nor a forked branch of the step graph
//
// Why this arm exists. One token makes the projection a pure weight stream: 0.53 bytes per weight, every byte
// read once. At 6.4 TB/s an SM receives about 22 bytes per clock, i.e. 44 weights, so the instruction budget is
// about three instructions per weight BYTE and lane. The integer arm (dp4a, issued at a quarter of the rate on
// this part, two 8-bit planes per activation) needs five; the warp-level MMA issues once per ~34 clocks per
// sub-core. This arm needs nine instructions per 32-bit word of eight weights:
//
//   * A nibble masked in place (q & 0x000f000f, q & 0x00f000f0, and the same on q >> 8) IS a pair of fp16
//     subnormals with the values n * 2^-24 and 16 n * 2^-24: no bias to subtract, no conversion. The record
//     layout puts k, k+1 into the two halves of each masked pair.
//   * The activations are stored once per CTA in shared memory as fp16 multiplied by a power of two chosen from
//     the row maximum (|x'| <= 16384), so the products n * x' * 2^-24 sit in the normal fp16 range and the
//     absolute rounding floor (2^-25) is 2^-19 of the largest term. fma.rn.f16x2 without .ftz keeps subnormal
//     inputs; two accumulator pairs per row (the x1 and the x16 pairs) are folded once per group of 128 k, where
//     the group's scale and zero point are applied in fp32:  y += s * (dot - z * sum(x')).
//
// The weight records and their slice-major order are those of the integer arms (gemv.cu): one 1088-byte record =
// 16 rows x 128 k of nibbles + 16 (scale, zero) half2; warp w of a group of eight streams k slice w through its
// own ring of bulk copies.
//
// Role in the reference: the Marlin W4A16 decode GEMV plus the fused add + RMSNorm and activation kernels around
// it (crates/kernels/cu/marlin/*, crates/kernels/cu/elems/add_rmsnorm.cu, exec/phases.rs decode sequence).
#include "common.cuh"

namespace owl {

__device__ int g_fma_status = 0;   // first bounded-wait failure of this file's kernels (0 = none)

enum { FMA_PLAIN = 0, FMA_NORM = 1, FMA_PULL = 2 };
enum { FEPI_STORE = 0, FEPI_RESIDUAL = 1, FEPI_SILU_MUL = 2, FEPI_PUSH = 3 };
constexpr int FM_MAX_RANKS = 8;

constexpr int FM_REC = 1088;          // bytes per record (g128)
constexpr int FM_STAGES = 4;          // records per warp ring: three in flight while one is consumed
constexpr int FM_WARPS = 8;           // warps per group = k slices of the record order
constexpr int FM_RED = 8;             // units of work whose partial sums wait in shared memory for one common barrier

struct FmaParams {
  const uint8_t* w;                 // slice-major record stream
  const __nv_bfloat16* x;           // [K] activations (FMA_PLAIN) or residual stream (FMA_NORM)
  const __nv_bfloat16* norm_w;      // [K] (FMA_NORM)
  __nv_bfloat16* out;               // [N] (FEPI_SILU_MUL: [N/2])
  const __nv_bfloat16* residual;    // [N] (FEPI_RESIDUAL), may alias out
  const __nv_bfloat16* ab_w;        // optional dense rows [ab_rows][K] multiplied with the same x
  __nv_bfloat16* ab_out;            // [ab_rows]
  __nv_bfloat16* x_out;             // optional: the activations this kernel consumed, as bf16 [K] (written by CTA 0)
  int ab_rows;
  int N, K, n_tiles;
  float eps;
  int one_plus;
  int kparts;                       // FEPI_PUSH: every row tile is cut into this many k parts, each a unit of work of its own
  // FEPI_PUSH (row-parallel projection): the partial sums of k part q go into slot [push_rank * kparts + q] of every
  // rank's word buffer [world * kparts][N / 2] with plain (peer) stores while the matrix streams. A word is 8 bytes: two
  // bf16 sums and the sequence number of this exchange (the call site's word + 1). An aligned 8-byte store arrives whole,
  // so the consumer needs no flag, the producer no fence and no count of finished CTAs: a word whose number matches is
  // valid. With one rank this is a local split of the k range: a projection with few row tiles (N = hidden) gets kparts
  // times as many units of work, and the consumer's prologue adds the parts.
  uint2* push_ll[FM_MAX_RANKS];
  const uint32_t* push_seq;         // local: number of the call site's last completed exchange
  int push_rank, push_world;
  // FMA_PULL (the column-parallel projection that follows): every thread polls the words of the chunks it loads until they
  // carry the awaited number (bounded), x = residual stream + the slots in rank order (the same sum, bit for bit, on every
  // rank), then the norm as in FMA_NORM. CTA 0 stores the new residual stream into h_out, a buffer other than x (the
  // other CTAs still read x). The CTA that leaves last writes the awaited number into the call site's word: every CTA of
  // this grid read the word before that, and the next producer of the call site starts after this grid.
  const uint2* pull_ll;             // local [world * kparts][K / 2]
  uint32_t* pull_seq;               // local: the call site's word (the same the producer read)
  int* pull_count;                  // local: CTAs of this launch that left (returns to zero)
  __nv_bfloat16* h_out;
  int pull_world;                   // slots to add (ranks x k parts)
  uint32_t spin_limit;
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float h2_sum(uint32_t v) {
  const __half2 h = *reinterpret_cast<const __half2*>(&v);
  return __low2float(h) + __high2float(h);
}
// 16-byte asynchronous copy global -> shared that bypasses L1 (every weight byte is read once).
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// Named barrier of one 8-warp group; the id is an immediate so that the CTA reserves only the barriers it uses.
template <int VC>
__device__ __forceinline__ void group_barrier(int vc) {
  if (vc == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
  else if (vc == 1) asm volatile("bar.sync 2, 256;" ::: "memory");
  else if (VC > 2 && vc == 2) asm volatile("bar.sync 3, 256;" ::: "memory");
  else if (VC > 2) asm volatile("bar.sync 4, 256;" ::: "memory");
}
__device__ __forceinline__ void bf16x8_to_f(const uint4& a, float* v) {
  v[0] = bf16_lo(a.x); v[1] = bf16_hi(a.x); v[2] = bf16_lo(a.y); v[3] = bf16_hi(a.y);
  v[4] = bf16_lo(a.z); v[5] = bf16_hi(a.z); v[6] = bf16_lo(a.w); v[7] = bf16_hi(a.w);
}

__host__ __device__ constexpr int fma_smem_bytes(int vc, int k) {
  return vc * FM_WARPS * FM_STAGES * FM_REC + k * 2 + (k / 128) * 4 + vc * FM_RED * FM_WARPS * 16 * 4 + 2 * 32 * 4 + 64;
}

// VC groups of eight warps per CTA; the groups share the activation vector and nothing else.
template <int VC, int MODE, int EPI>
__global__ void __launch_bounds__(VC * FM_WARPS * 32, 4 / VC) w4_fma_kernel(FmaParams p) {
  constexpr int NT = VC * FM_WARPS * 32;
  constexpr bool NORMED = MODE != FMA_PLAIN;
  constexpr int FM_CACHE = NORMED ? 2 : 3;   // activation chunks (8 values) kept in registers between the two prologue passes
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring_all = smem;
  uint4* xh4 = reinterpret_cast<uint4*>(smem + VC * FM_WARPS * FM_STAGES * FM_REC);   // fp16 x' [K]
  float* xg = reinterpret_cast<float*>(xh4 + p.K / 8);                             // per 128-k group: sum(x') * 2^-24
  float* red = xg + p.K / 128;                                                     // [VC][FM_RED units][8 warps][16 rows]
  float* pro = red + VC * FM_RED * FM_WARPS * 16;                                  // prologue reductions [2][32]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vc = warp / FM_WARPS, wi = warp % FM_WARPS, g = lane >> 2, t = lane & 3;
  uint8_t* ring = ring_all + (size_t)warp * FM_STAGES * FM_REC;

  // ---- this warp's stream -----------------------------------------------------------------------------------------
  // Warp wi streams k slice wi: records [tile][record in slice], one contiguous run for the whole matrix. A unit of work
  // is one row tile (or, with kparts > 1, one of the k parts of a tile: records [q * rpi / P, (q + 1) * rpi / P) of the
  // tile in every slice); the groups of the grid take contiguous, equally long runs of units.
  const int KT = p.K / 128;
  const int n_groups = gridDim.x * VC, grp = blockIdx.x * VC + vc;
  const int kt0 = (int)((long long)wi * KT / FM_WARPS), kt1 = (int)((long long)(wi + 1) * KT / FM_WARPS);
  const int rpi = kt1 - kt0;
  const int P = EPI == FEPI_PUSH ? p.kparts : 1;
  const int n_units = p.n_tiles * P;
  const int u0 = (int)((long long)grp * n_units / n_groups), u1 = (int)((long long)(grp + 1) * n_units / n_groups);
  // record index (within the slice) where unit u starts
  auto unit_start = [&](int u) { return (u / P) * rpi + (u % P) * rpi / P; };
  const int R0 = unit_start(u0), total = unit_start(u1) - R0;
  const uint8_t* gsrc = p.w + ((size_t)p.n_tiles * kt0 + (size_t)R0) * FM_REC + lane * 16;   // next record to fetch, this lane's word
  const uint32_t ring_s = smem_u32(ring) + lane * 16;
  int to_issue = total;

  // Record j of the stream lives in ring stage j % FM_STAGES; lane L copies the 16-byte words it reads itself (L and
  // 32 + L), lanes 0..3 the scale / zero words. One commit group per record, also past the end, so that the group count
  // stays uniform and "all but the two newest groups are complete" always means "the record about to be read landed".
  auto issue = [&](uint32_t stage_off) {
    if (to_issue > 0) {
      cp_async16(ring_s + stage_off, gsrc);
      cp_async16(ring_s + stage_off + 512, gsrc + 512);
      if (lane < 4) cp_async16(ring_s + stage_off + 1024, gsrc + 1024);
      gsrc += FM_REC;
    }
    --to_issue;
    cp_async_commit();
  };
  // weights do not depend on the previous kernel: start the stream before the dependency wait
#pragma unroll
  for (int j = 0; j < FM_STAGES - 1; ++j) issue(j * FM_REC);

  // ---- prologue: the activation vector as scaled fp16 in shared memory -------------------------------------
  const int nchunks = p.K / 8;
  const uint4* x4 = reinterpret_cast<const uint4*>(p.x);
  const uint4* w4 = reinterpret_cast<const uint4*>(p.norm_w);
  uint4 wc[FM_CACHE], hc[FM_CACHE];
  if (NORMED) {
#pragma unroll
    for (int i = 0; i < FM_CACHE; ++i) {
      const int c = tid + i * NT;
      wc[i] = c < nchunks ? __ldg(w4 + c) : make_uint4(0, 0, 0, 0);
    }
  }
  // the dependent launch may start now: its CTAs take the SMs as this grid's CTAs leave, and fetch weights (which no kernel
  // of a step writes) until this grid has completed; measured +6 % tokens/s over triggering at the end
  pdl_launch_dependents();
  pdl_wait();
  uint32_t want = 0, seq = 0;
  bool dead = false;                      // a wait of this thread ran out: do not wait again
  if (MODE == FMA_PULL) want = __ldcg(p.pull_seq) + 1u;
  if (EPI == FEPI_PUSH) seq = __ldcg(p.push_seq) + 1u;
  // one chunk (8 values) of the input row; FMA_PULL adds the ranks' slots in rank order and rounds to bf16 once
  auto load_x = [&](int c) -> uint4 {
    const uint4 hv = __ldcg(x4 + c);
    if (MODE != FMA_PULL) return hv;
    float a[8];
    bf16x8_to_f(hv, a);
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.pull_world; ++r) {
      // four words of this chunk: (2 sums, number) x 4, valid once all four numbers match
      const uint4* src = reinterpret_cast<const uint4*>(p.pull_ll + (size_t)r * (p.K >> 1)) + 2 * c;
      uint4 u = ld_relaxed_sys_u4(src), v = ld_relaxed_sys_u4(src + 1);
      if (!dead) {
        uint32_t i = 0;
        while (u.y != want || u.w != want || v.y != want || v.w != want) {
          if (++i >= p.spin_limit) { dead = true; atomicCAS(&g_fma_status, 0, OWL_ERR_WAIT_PEER); break; }
          if (i > 64) __nanosleep(32);
          u = ld_relaxed_sys_u4(src); v = ld_relaxed_sys_u4(src + 1);
        }
      }
      sum[0] += bf16_lo(u.x); sum[1] += bf16_hi(u.x); sum[2] += bf16_lo(u.z); sum[3] += bf16_hi(u.z);
      sum[4] += bf16_lo(v.x); sum[5] += bf16_hi(v.x); sum[6] += bf16_lo(v.z); sum[7] += bf16_hi(v.z);
    }
    const uint4 o = make_uint4(pack_bf16(a[0] + sum[0], a[1] + sum[1]), pack_bf16(a[2] + sum[2], a[3] + sum[3]),
                               pack_bf16(a[4] + sum[4], a[5] + sum[5]), pack_bf16(a[6] + sum[6], a[7] + sum[7]));
    if (blockIdx.x == 0) reinterpret_cast<uint4*>(p.h_out)[c] = o;
    return o;
  };
  float ss = 0.f, mx = 0.f;
  auto scan = [&](const uint4& hv, const uint4& wv) {
    float h[8], wf[8];
    bf16x8_to_f(hv, h);
    if (NORMED) {
      bf16x8_to_f(wv, wf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ss = fmaf(h[i], h[i], ss);
        mx = fmaxf(mx, fabsf(h[i] * (p.one_plus ? 1.f + wf[i] : wf[i])));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(h[i]));
    }
  };
#pragma unroll
  for (int i = 0; i < FM_CACHE; ++i) {
    const int c = tid + i * NT;
    hc[i] = c < nchunks ? load_x(c) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int i = 0; i < FM_CACHE; ++i) scan(hc[i], wc[i]);
  for (int c = tid + FM_CACHE * NT; c < nchunks; c += NT)      // (FMA_PULL rows fit the register cache: checked by the launcher)
    scan(__ldcg(x4 + c), NORMED ? __ldg(w4 + c) : make_uint4(0, 0, 0, 0));
  ss = warp_sum(ss);
  mx = warp_max(mx);
  if (lane == 0) { pro[warp] = ss; pro[32 + warp] = mx; }
  __syncthreads();
  ss = warp_sum(lane < VC * FM_WARPS ? pro[lane] : 0.f);
  mx = warp_max(lane < VC * FM_WARPS ? pro[32 + lane] : 0.f);
  const float rinv = NORMED ? rsqrtf(ss / (float)p.K + p.eps) : 1.f;
  // power-of-two scale: 8192 < max |x'| <= 16384
  const float sx = __uint_as_float(__float_as_uint(16384.f / fmaxf(mx * rinv, 1e-30f)) & 0x7f800000u);
  const float unscale = 16777216.f / sx;      // products carry 2^-24 (subnormal nibbles) and sx
  auto emit = [&](int c, const uint4& hv, const uint4& wv) {       // warp-uniform call: c - lane is the same in all lanes
    float h[8], wf[8], s8 = 0.f;
    bf16x8_to_f(hv, h);
    if (NORMED) {
      bf16x8_to_f(wv, wf);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        h[i] = __bfloat162float(__float2bfloat16(h[i] * rinv * (p.one_plus ? 1.f + wf[i] : wf[i])));
    }
    uint32_t pk[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 hh = __floats2half2_rn(h[2 * i] * sx, h[2 * i + 1] * sx);
      pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
      s8 += __low2float(hh) + __high2float(hh);
    }
    s8 += __shfl_xor_sync(0xffffffffu, s8, 8);
    s8 += __shfl_xor_sync(0xffffffffu, s8, 4);
    s8 += __shfl_xor_sync(0xffffffffu, s8, 2);
    s8 += __shfl_xor_sync(0xffffffffu, s8, 1);
    if (c < nchunks) {
      xh4[c] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      if ((c & 15) == 0) xg[c >> 4] = s8 * (1.f / 16777216.f);
      if (p.x_out && blockIdx.x == 0)
        reinterpret_cast<uint4*>(p.x_out)[c] = make_uint4(pack_bf16(h[0], h[1]), pack_bf16(h[2], h[3]),
                                                          pack_bf16(h[4], h[5]), pack_bf16(h[6], h[7]));
    }
  };
#pragma unroll
  for (int i = 0; i < FM_CACHE; ++i)
    if (tid - lane + i * NT < nchunks) emit(tid + i * NT, hc[i], wc[i]);
  for (int c = tid + FM_CACHE * NT; c - lane < nchunks; c += NT) {
    const bool in = c < nchunks;
    emit(c, in ? __ldcg(x4 + c) : make_uint4(0, 0, 0, 0),
         (NORMED && in) ? __ldg(w4 + c) : make_uint4(0, 0, 0, 0));
  }
  __syncthreads();

  // ---- side job: dense rows against the same activations, one warp per row ------------------------------------
  if (p.ab_rows > 0) {
    const int gw = blockIdx.x * (VC * FM_WARPS) + warp, nw = gridDim.x * VC * FM_WARPS;
    const int stride = max(1, nw / p.ab_rows);
    if (gw % stride == 0 && gw / stride < p.ab_rows) {
      const int r = gw / stride;
      const uint4* wr = reinterpret_cast<const uint4*>(p.ab_w + (size_t)r * p.K);
      float a = 0.f;
      for (int c = lane; c < nchunks; c += 32) {
        float wf[8];
        bf16x8_to_f(__ldg(wr + c), wf);
        const uint4 xv = xh4[c];
        const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 xf = __half22float2(xh[i]);
          a = fmaf(wf[2 * i], xf.x, a);
          a = fmaf(wf[2 * i + 1], xf.y, a);
        }
      }
      a = warp_sum(a);
      if (lane == 0) p.ab_out[r] = __float2bfloat16(a / sx);
    }
  }

  // ---- main loop ----------------------------------------------------------------------------------------------
  float acc0 = 0.f, acc1 = 0.f;      // rows g and g + 8 of the current tile, this lane's k runs
  const uint32_t sixteenth = 0x2C002C00u;       // (1/16, 1/16)
  uint32_t st_c = 0, st_i = (FM_STAGES - 1) * FM_REC;        // ring offsets of the record consumed / fetched next
  const uint8_t* ring_l = ring + lane * 16;                   // this lane's weight words of stage 0
  const uint8_t* ring_z = ring + 1024 + g * 4;                // and its rows' (scale, zero) pairs
  const uint4* x_slice = xh4 + kt0 * 16 + t;                  // this lane's activations of the slice's first record
  const float* g_slice = xg + kt0;
  for (int u = u0, item = 0; u < u1; ++u, ++item) {
    const int q = u % P;
    const int ka = q * rpi / P, kb = (q + 1) * rpi / P;
    const uint4* xr = x_slice + ka * 16;
    const float* xs = g_slice + ka;
    for (int kk = ka; kk < kb; ++kk) {
      const uint4 x0 = xr[0], x1 = xr[4], x2 = xr[8], x3 = xr[12];
      const float xsum = *xs;
      xr += 16;
      ++xs;
      cp_async_wait<FM_STAGES - 2>();           // this lane's copies of the record have landed
      __syncwarp();                             // and everybody's (scale words), and everybody left the previous record
      issue(st_i);                              // refill the stage the previous record occupied
      st_i = st_i == (FM_STAGES - 1) * FM_REC ? 0u : st_i + FM_REC;
      const uint4 lo = *reinterpret_cast<const uint4*>(ring_l + st_c), hi = *reinterpret_cast<const uint4*>(ring_l + st_c + 512);
      const uint32_t su0 = *reinterpret_cast<const uint32_t*>(ring_z + st_c), su1 = *reinterpret_cast<const uint32_t*>(ring_z + st_c + 32);
      st_c = st_c == (FM_STAGES - 1) * FM_REC ? 0u : st_c + FM_REC;
      uint32_t a0 = 0u, b0 = 0u, a1 = 0u, b1 = 0u;
#define OWL_FMA_WORD(Q0, Q1, XV)                                                           \
      {                                                                                    \
        uint32_t q0 = (Q0), q1 = (Q1);                                                     \
        a0 = hfma2_u(q0 & 0x000f000fu, (XV).x, a0); b0 = hfma2_u(q0 & 0x00f000f0u, (XV).y, b0); \
        a1 = hfma2_u(q1 & 0x000f000fu, (XV).x, a1); b1 = hfma2_u(q1 & 0x00f000f0u, (XV).y, b1); \
        q0 >>= 8; q1 >>= 8;                                                                \
        a0 = hfma2_u(q0 & 0x000f000fu, (XV).z, a0); b0 = hfma2_u(q0 & 0x00f000f0u, (XV).w, b0); \
        a1 = hfma2_u(q1 & 0x000f000fu, (XV).z, a1); b1 = hfma2_u(q1 & 0x00f000f0u, (XV).w, b1); \
      }
      OWL_FMA_WORD(lo.x, hi.x, x0)
      OWL_FMA_WORD(lo.y, hi.y, x1)
      OWL_FMA_WORD(lo.z, hi.z, x2)
      OWL_FMA_WORD(lo.w, hi.w, x3)
#undef OWL_FMA_WORD
      const float f0 = h2_sum(hfma2_u(b0, sixteenth, a0)), f1 = h2_sum(hfma2_u(b1, sixteenth, a1));
      const float2 s0 = __half22float2(*reinterpret_cast<const __half2*>(&su0));
      const float2 s1 = __half22float2(*reinterpret_cast<const __half2*>(&su1));
      const float xq = xsum * 0.25f;            // four t lanes share z * sum
      acc0 = fmaf(s0.x, fmaf(-s0.y, xq, f0), acc0);
      acc1 = fmaf(s1.x, fmaf(-s1.y, xq, f1), acc1);
    }
    // ---- end of the unit: the 4 t lanes, then this warp's 16 sums wait in shared memory for the other k slices ---------
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    const int bi = item % FM_RED;                 // slot of this unit in the current batch
    float* rmine = red + (size_t)((vc * FM_RED + bi) * FM_WARPS + wi) * 16;
    if (t == 0) { rmine[g] = acc0; rmine[8 + g] = acc1; }
    acc0 = acc1 = 0.f;
    if (bi + 1 < FM_RED && u + 1 < u1) continue;
    // ---- a batch of units is complete (or the group is done): ONE barrier for the whole batch, then the 8 warps share
    // the finishing work. The k slices of a group run unsynchronised in between (a barrier per 5-record tile would keep
    // every warp waiting for the slowest one all the time).
    group_barrier<VC>(vc);
    const int n_batch = bi + 1, ub = u - bi;
    for (int i = wi; i < n_batch; i += FM_WARPS) {
      const float* rb = red + (size_t)((vc * FM_RED + i) * FM_WARPS) * 16;
      const int uu = ub + i, nt = uu / P, qq = uu % P;
      float v = 0.f;
      if (lane < 16) {
#pragma unroll
        for (int sl = 0; sl < FM_WARPS; ++sl) v += rb[sl * 16 + lane];
        v *= unscale;
      }
      if (EPI == FEPI_SILU_MUL) {
        const float up = __shfl_down_sync(0xffffffffu, v, 8);
        if (lane < 8) p.out[nt * 8 + lane] = __float2bfloat16(silu_f(v) * up);
      } else if (EPI == FEPI_PUSH) {
        const float hi = __shfl_down_sync(0xffffffffu, v, 1);
        if (lane < 16 && !(lane & 1)) {
          const uint32_t pk = pack_bf16(v, hi);
          const size_t off = (size_t)(p.push_rank * P + qq) * (p.N >> 1) + nt * 8 + (lane >> 1);
          for (int r = 0; r < p.push_world; ++r)
            asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p.push_ll[r] + off), "r"(pk), "r"(seq) : "memory");
        }
      } else if (lane < 16) {
        if (EPI == FEPI_RESIDUAL) v += __bfloat162float(p.residual[nt * 16 + lane]);
        p.out[nt * 16 + lane] = __float2bfloat16(v);
      }
    }
    if (u + 1 < u1) group_barrier<VC>(vc);        // the next batch reuses the slots
  }
  cp_async_wait<0>();
  if (MODE == FMA_PULL && tid == 0) {
    if (atomicAdd(p.pull_count, 1) == (int)gridDim.x - 1) {
      *p.pull_count = 0;
      *p.pull_seq = want;
    }
  }
}

template <int VC, int MODE, int EPI>
static int launch_fma(const FmaParams& p, int grid, int pdl, cudaStream_t st) {
  auto kernel = w4_fma_kernel<VC, MODE, EPI>;
  static int attr_smem = 0;
  const int smem = fma_smem_bytes(VC, p.K);
  if (smem > attr_smem) {
    const int want = smem > 96 * 1024 ? smem : 96 * 1024;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, want);
    if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
    attr_smem = want;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(VC * FM_WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

template <int VC>
static int dispatch_fma(const FmaParams& p, int mode, int epi, int grid, int pdl, cudaStream_t st) {
#define OWL_FMA_CASE(M, E) if (mode == M && epi == E) return launch_fma<VC, M, E>(p, grid, pdl, st);
  OWL_FMA_CASE(FMA_PLAIN, FEPI_STORE) OWL_FMA_CASE(FMA_PLAIN, FEPI_RESIDUAL) OWL_FMA_CASE(FMA_PLAIN, FEPI_SILU_MUL)
  OWL_FMA_CASE(FMA_PLAIN, FEPI_PUSH)
  OWL_FMA_CASE(FMA_NORM, FEPI_STORE) OWL_FMA_CASE(FMA_NORM, FEPI_RESIDUAL) OWL_FMA_CASE(FMA_NORM, FEPI_SILU_MUL)
  OWL_FMA_CASE(FMA_PULL, FEPI_STORE) OWL_FMA_CASE(FMA_PULL, FEPI_SILU_MUL)
#undef OWL_FMA_CASE
  return OWL_ERR_BAD_ARG;
}

static int fma_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

}  // namespace owl
using namespace owl;

// One token: out = epilogue(dequant(records)[N, K] . prologue(x)). records: slice-major g128 W4 records. mode 0: x is
// the bf16 activation vector; mode 1: x is the residual stream and the kernel multiplies by rmsnorm(x) * (norm_w or
// 1 + norm_w). epi 0: bf16 store, 1: out = residual + y, 2: out[N/2] = silu(gate) * up with gate / up rows interleaved in
// eights. ab_w / ab_out / ab_rows: optional dense bf16 rows [ab_rows][K] multiplied with the same activations.
// x_out: optional bf16 [K], receives the activations the kernel consumed (mode 1: the normalised row). groups_per_cta: 2
// (512 threads, two CTAs per SM) or 4 (1024 threads, one per SM); 0 = chosen from K.
OWL_API int owl_w4_fma(const void* records, const void* x, const void* norm_w, void* out, const void* residual,
                       const void* ab_w, void* ab_out, int ab_rows, void* x_out, int N, int K, int mode, int epi, float eps,
                       int one_plus_w, int groups_per_cta, int pdl, cudaStream_t st) {
  if (!records || !x || !out || (N & 15) || (K & 127) || K < 128 || K > 32768 || mode < 0 || mode > 1 || epi < 0 || epi > 2)
    return OWL_ERR_BAD_ARG;
  if ((mode == FMA_NORM && !norm_w) || (epi == FEPI_RESIDUAL && !residual) || (ab_rows > 0 && (!ab_w || !ab_out)) || ab_rows < 0)
    return OWL_ERR_BAD_ARG;
  FmaParams p = {};
  p.w = (const uint8_t*)records; p.x = (const __nv_bfloat16*)x; p.norm_w = (const __nv_bfloat16*)norm_w;
  p.out = (__nv_bfloat16*)out; p.residual = (const __nv_bfloat16*)residual;
  p.ab_w = (const __nv_bfloat16*)ab_w; p.ab_out = (__nv_bfloat16*)ab_out; p.ab_rows = ab_rows;
  p.x_out = (__nv_bfloat16*)x_out;
  p.N = N; p.K = K; p.n_tiles = N / 16; p.eps = eps; p.one_plus = one_plus_w;
  const int vc = groups_per_cta ? groups_per_cta : (K > 8192 ? 4 : 2);
  if (vc != 2 && vc != 4) return OWL_ERR_BAD_ARG;
  const int grid = fma_sm_count() * (4 / vc);
  if (p.ab_rows > grid * vc * FM_WARPS) return OWL_ERR_BAD_ARG;
  return vc == 4 ? dispatch_fma<4>(p, mode, epi, grid, pdl, st) : dispatch_fma<2>(p, mode, epi, grid, pdl, st);
}

// Split forms of the same launch (one token), across ranks and / or across k parts. push != 0: a row-parallel projection
// whose partial sums are stored into slot [rank * kparts + part] of every rank's word buffer (ll_ptrs: `world` peer-mapped
// bases of [world * kparts][N / 2] 8-byte words, zero before the first call; seq: the call site's local sequence word, zero
// before the first call); x is the plain activation vector. world * kparts <= 8; world = 1 is a local k split.
// push == 0: the column-parallel projection that consumes such a buffer: x is the residual stream, pull_ll the LOCAL word
// buffer, seq the same local word, pull_count a local int (zero before the first call), h_out (a buffer other than x)
// receives x + sum of the slots, and the kernel multiplies by rmsnorm(h_out) * (norm_w or 1 + norm_w); epi 0 or 2 as in
// owl_w4_fma.
OWL_API int owl_w4_fma_tp(const void* records, const void* x, const void* norm_w, void* out, int N, int K, int epi, float eps,
                          int one_plus_w, int push, void* const* ll_ptrs, void* seq, const void* pull_ll, void* pull_count,
                          void* h_out, const void* ab_w, void* ab_out, int ab_rows, int rank, int world, int kparts,
                          unsigned spin_limit, int groups_per_cta, int pdl, cudaStream_t st) {
  if (!records || !x || (N & 15) || (K & 127) || K < 128 || K > 32768 || world < 1 || world > FM_MAX_RANKS || rank < 0 ||
      rank >= world || !seq)
    return OWL_ERR_BAD_ARG;
  FmaParams p = {};
  p.w = (const uint8_t*)records; p.x = (const __nv_bfloat16*)x; p.norm_w = (const __nv_bfloat16*)norm_w;
  p.out = (__nv_bfloat16*)out; p.N = N; p.K = K; p.n_tiles = N / 16; p.eps = eps; p.one_plus = one_plus_w;
  p.ab_w = (const __nv_bfloat16*)ab_w; p.ab_out = (__nv_bfloat16*)ab_out; p.ab_rows = ab_rows;
  const int vc = groups_per_cta ? groups_per_cta : (K > 8192 ? 4 : 2);
  if (vc != 2 && vc != 4) return OWL_ERR_BAD_ARG;
  const int grid = fma_sm_count() * (4 / vc);
  if (ab_rows < 0 || (ab_rows > 0 && (!ab_w || !ab_out)) || ab_rows > grid * vc * FM_WARPS) return OWL_ERR_BAD_ARG;
  if (kparts < 1 || world * kparts > FM_MAX_RANKS) return OWL_ERR_BAD_ARG;
  p.kparts = kparts;
  if (push) {
    if (!ll_ptrs) return OWL_ERR_BAD_ARG;
    for (int r = 0; r < world; ++r) {
      p.push_ll[r] = (uint2*)ll_ptrs[r];
      if (!p.push_ll[r] || (reinterpret_cast<uintptr_t>(p.push_ll[r]) & 15)) return OWL_ERR_BAD_ARG;
    }
    p.push_seq = (const uint32_t*)seq; p.push_rank = rank; p.push_world = world;
    return vc == 4 ? launch_fma<4, FMA_PLAIN, FEPI_PUSH>(p, grid, pdl, st) : launch_fma<2, FMA_PLAIN, FEPI_PUSH>(p, grid, pdl, st);
  }
  if (!out || !norm_w || !pull_ll || !pull_count || !h_out || h_out == x || (epi != FEPI_STORE && epi != FEPI_SILU_MUL) ||
      (reinterpret_cast<uintptr_t>(pull_ll) & 15))
    return OWL_ERR_BAD_ARG;
  if (K / 8 > 2 * vc * FM_WARPS * 32) return OWL_ERR_BAD_ARG;      // the pulled row must fit the prologue's register cache
  p.pull_ll = (const uint2*)pull_ll; p.pull_seq = (uint32_t*)seq; p.pull_count = (int*)pull_count;
  p.h_out = (__nv_bfloat16*)h_out; p.pull_world = world * kparts;
  p.spin_limit = spin_limit ? spin_limit : (1u << 22);
  return vc == 4 ? dispatch_fma<4>(p, FMA_PULL, epi, grid, pdl, st) : dispatch_fma<2>(p, FMA_PULL, epi, grid, pdl, st);
}

// First bounded-wait failure recorded by this file's kernels since the last call (0 = none); clears it.
OWL_API int owl_fma_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_fma_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_fma_status, &zero, sizeof(int));
  return v;
}
