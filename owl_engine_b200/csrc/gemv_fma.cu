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

enum { FMA_PLAIN = 0, FMA_NORM = 1 };
enum { FEPI_STORE = 0, FEPI_RESIDUAL = 1, FEPI_SILU_MUL = 2 };

constexpr int FM_REC = 1088;          // bytes per record (g128)
constexpr int FM_SLOTS = 2;           // chunks in flight per warp
constexpr int FM_CH = 2;              // records per chunk (one bulk copy, one mbarrier)
constexpr int FM_SLOT_BYTES = FM_CH * FM_REC;
constexpr int FM_WARPS = 8;           // warps per group = k slices of the record order

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
};

__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float h2_sum(uint32_t v) {
  const __half2 h = *reinterpret_cast<const __half2*>(&v);
  return __low2float(h) + __high2float(h);
}
__device__ __forceinline__ void bulk_g2s_f(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
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
  return vc * FM_WARPS * FM_SLOTS * FM_SLOT_BYTES + vc * FM_WARPS * FM_SLOTS * 8 + k * 2 + (k / 128) * 4 +
         vc * 2 * FM_WARPS * 16 * 4 + 2 * 32 * 4 + 64;
}

// VC groups of eight warps per CTA; the groups share the activation vector and nothing else.
template <int VC, int MODE, int EPI>
__global__ void __launch_bounds__(VC * FM_WARPS * 32, 4 / VC) w4_fma_kernel(FmaParams p) {
  constexpr int NT = VC * FM_WARPS * 32;
  constexpr int FM_CACHE = MODE == FMA_NORM ? 2 : 3;   // activation chunks (8 values) kept in registers between the two prologue passes
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring_all = smem;
  uint64_t* bars_all = reinterpret_cast<uint64_t*>(smem + VC * FM_WARPS * FM_SLOTS * FM_SLOT_BYTES);
  uint4* xh4 = reinterpret_cast<uint4*>(bars_all + VC * FM_WARPS * FM_SLOTS);      // fp16 x' [K]
  float* xg = reinterpret_cast<float*>(xh4 + p.K / 8);                             // per 128-k group: sum(x') * 2^-24
  float* red = xg + p.K / 128;                                                     // [VC][2][8 warps][16 rows]
  float* pro = red + VC * 2 * FM_WARPS * 16;                                       // prologue reductions [2][32]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vc = warp / FM_WARPS, wi = warp % FM_WARPS, g = lane >> 2, t = lane & 3;
  uint8_t* ring = ring_all + (size_t)warp * FM_SLOTS * FM_SLOT_BYTES;
  uint64_t* bars = bars_all + warp * FM_SLOTS;

  // ---- this warp's stream: k slice wi of the row tiles of its group -----------------------------------------
  const int KT = p.K / 128;
  const int n_groups = gridDim.x * VC, grp = blockIdx.x * VC + vc;
  const int nt0 = (int)((long long)grp * p.n_tiles / n_groups);
  const int n_items = (int)((long long)(grp + 1) * p.n_tiles / n_groups) - nt0;
  const int kt0 = (int)((long long)wi * KT / FM_WARPS), kt1 = (int)((long long)(wi + 1) * KT / FM_WARPS);
  const int rpi = kt1 - kt0;
  const int total = rpi * n_items;
  const uint8_t* wsrc = p.w + ((size_t)p.n_tiles * kt0 + (size_t)nt0 * rpi) * FM_REC;
  const int n_chunks = (total + FM_CH - 1) / FM_CH;

  if (lane == 0) {
    for (int s = 0; s < FM_SLOTS; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  if (lane == 0) {      // weights do not depend on the previous kernel: start the stream before the dependency wait
    for (int c = 0; c < FM_SLOTS && c < n_chunks; ++c) {
      const uint32_t bytes = (uint32_t)min(FM_CH, total - c * FM_CH) * FM_REC;
      mbar_expect_tx(&bars[c], bytes);
      bulk_g2s_f(ring + (size_t)c * FM_SLOT_BYTES, wsrc + (size_t)c * FM_SLOT_BYTES, bytes, &bars[c]);
    }
  }

  // ---- prologue: the activation vector as scaled fp16 in shared memory -------------------------------------
  const int nchunks = p.K / 8;
  const uint4* x4 = reinterpret_cast<const uint4*>(p.x);
  const uint4* w4 = reinterpret_cast<const uint4*>(p.norm_w);
  uint4 wc[FM_CACHE], hc[FM_CACHE];
  if (MODE == FMA_NORM) {
#pragma unroll
    for (int i = 0; i < FM_CACHE; ++i) {
      const int c = tid + i * NT;
      wc[i] = c < nchunks ? __ldg(w4 + c) : make_uint4(0, 0, 0, 0);
    }
  }
  pdl_wait();
  float ss = 0.f, mx = 0.f;
  auto scan = [&](const uint4& hv, const uint4& wv) {
    float h[8], wf[8];
    bf16x8_to_f(hv, h);
    if (MODE == FMA_NORM) {
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
    hc[i] = c < nchunks ? __ldcg(x4 + c) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int i = 0; i < FM_CACHE; ++i) scan(hc[i], wc[i]);
  for (int c = tid + FM_CACHE * NT; c < nchunks; c += NT)
    scan(__ldcg(x4 + c), MODE == FMA_NORM ? __ldg(w4 + c) : make_uint4(0, 0, 0, 0));
  ss = warp_sum(ss);
  mx = warp_max(mx);
  if (lane == 0) { pro[warp] = ss; pro[32 + warp] = mx; }
  __syncthreads();
  ss = warp_sum(lane < VC * FM_WARPS ? pro[lane] : 0.f);
  mx = warp_max(lane < VC * FM_WARPS ? pro[32 + lane] : 0.f);
  const float rinv = MODE == FMA_NORM ? rsqrtf(ss / (float)p.K + p.eps) : 1.f;
  // power-of-two scale: 8192 < max |x'| <= 16384
  const float sx = __uint_as_float(__float_as_uint(16384.f / fmaxf(mx * rinv, 1e-30f)) & 0x7f800000u);
  const float unscale = 16777216.f / sx;      // products carry 2^-24 (subnormal nibbles) and sx
  auto emit = [&](int c, const uint4& hv, const uint4& wv) {       // warp-uniform call: c - lane is the same in all lanes
    float h[8], wf[8], s8 = 0.f;
    bf16x8_to_f(hv, h);
    if (MODE == FMA_NORM) {
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
         (MODE == FMA_NORM && in) ? __ldg(w4 + c) : make_uint4(0, 0, 0, 0));
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
  bool failed = false;
  int item = 0, kk = 0, chunk = 0, in_chunk = 0, slot = 0;
  uint32_t parity = 0;
  const uint8_t* rec_b = ring;
  const uint32_t sixteenth = 0x2C002C00u;       // (1/16, 1/16)
  for (int j = 0; j < total || item < n_items; ++j) {
    if (j < total) {
      const int krec = kt0 + kk;
      const uint4* xr = xh4 + krec * 16 + t;
      const uint4 x0 = xr[0], x1 = xr[4], x2 = xr[8], x3 = xr[12];
      const float xsum = xg[krec];
      if (in_chunk == 0) {
        if (!failed && !mbar_wait(&bars[slot], parity, 1u << 22)) {
          failed = true;
          atomicCAS(&g_fma_status, 0, OWL_ERR_WAIT_TMA);
        }
      }
      const uint4* rec = reinterpret_cast<const uint4*>(rec_b);
      const uint4 lo = rec[lane], hi = rec[32 + lane];
      const uint32_t* szr = reinterpret_cast<const uint32_t*>(rec + 64);
      const uint32_t su0 = szr[g], su1 = szr[8 + g];
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
      {
        const float f0 = h2_sum(hfma2_u(b0, sixteenth, a0)), f1 = h2_sum(hfma2_u(b1, sixteenth, a1));
        const __half2 s0 = *reinterpret_cast<const __half2*>(&su0), s1 = *reinterpret_cast<const __half2*>(&su1);
        acc0 = fmaf(__low2float(s0), fmaf(-__high2float(s0), xsum * 0.25f, f0), acc0);   // four t lanes share z * sum
        acc1 = fmaf(__low2float(s1), fmaf(-__high2float(s1), xsum * 0.25f, f1), acc1);
      }
      rec_b += FM_REC;
      if (++in_chunk == FM_CH || j + 1 == total) {
        __syncwarp();
        const int nc = chunk + FM_SLOTS;
        if (lane == 0 && nc < n_chunks) {
          const uint32_t bytes = (uint32_t)min(FM_CH, total - nc * FM_CH) * FM_REC;
          mbar_expect_tx(&bars[slot], bytes);
          bulk_g2s_f(ring + (size_t)slot * FM_SLOT_BYTES, wsrc + (size_t)nc * FM_SLOT_BYTES, bytes, &bars[slot]);
        }
        ++chunk; in_chunk = 0;
        if (++slot == FM_SLOTS) { slot = 0; parity ^= 1u; }
        rec_b = ring + (size_t)slot * FM_SLOT_BYTES;
      }
      if (++kk < rpi) continue;
      kk = 0;
    }
    // ---- end of a row tile: 4 t lanes, then the 8 k slices through shared memory ------------------------------
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    float* rbuf = red + (size_t)((vc * 2 + (item & 1)) * FM_WARPS) * 16;
    if (t == 0) { rbuf[wi * 16 + g] = acc0; rbuf[wi * 16 + 8 + g] = acc1; }
    acc0 = acc1 = 0.f;
    group_barrier<VC>(vc);
    if (wi == (item & (FM_WARPS - 1))) {
      const int nt = nt0 + item;
      float v = 0.f;
      if (lane < 16) {
#pragma unroll
        for (int s = 0; s < FM_WARPS; ++s) v += rbuf[s * 16 + lane];
        v *= unscale;
      }
      if (EPI == FEPI_SILU_MUL) {
        const float up = __shfl_down_sync(0xffffffffu, v, 8);
        if (lane < 8) p.out[nt * 8 + lane] = __float2bfloat16(silu_f(v) * up);
      } else if (lane < 16) {
        if (EPI == FEPI_RESIDUAL) v += __bfloat162float(p.residual[nt * 16 + lane]);
        p.out[nt * 16 + lane] = __float2bfloat16(v);
      }
    }
    ++item;
  }
  pdl_launch_dependents();
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
  OWL_FMA_CASE(FMA_NORM, FEPI_STORE) OWL_FMA_CASE(FMA_NORM, FEPI_RESIDUAL) OWL_FMA_CASE(FMA_NORM, FEPI_SILU_MUL)
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

// First bounded-wait failure recorded by this file's kernels since the last call (0 = none); clears it.
OWL_API int owl_fma_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_fma_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_fma_status, &zero, sizeof(int));
  return v;
}
