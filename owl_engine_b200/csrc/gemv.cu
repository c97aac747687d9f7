// Weight-streaming "skinny" GEMMs for decode / verify / small-batch steps (M <= 32 tokens).
//
//   owl_w4a16_skinny : C[M,N] = X[M,K] . dequant(W4)[N,K]^T   (int4, group 32/128, asymmetric)
//   owl_bf16_skinny  : C[M,N] = X[M,K] . W[N,K]^T             (dense bf16 weights, tiled)
//   owl_w8a16_skinny : C[M,N] = X[M,K] . (s[n] * W8[N,K])^T   (int8 rows, one scale per row, tiled)
//
// These ops are bound by HBM bandwidth: every weight byte is read exactly once. Each warp owns
// a private ring of shared-memory slots that lane 0 keeps full with bulk asynchronous copies
// (cp.async.bulk + mbarrier complete_tx), so the bytes in flight per SM are set by the ring
// depth (~100 KB/SM) instead of by registers, and the stream never drains between row tiles:
// a CTA is persistent over a contiguous range of 16-row tiles and its 8 warps split K.
// The contraction runs on the warp-level tensor-core path (m16n8k16, fp32 accumulate) so that
// 1..8 tokens cost the same issue slots as one; the weight tile is the 16-row A operand and
// the tokens are the 8-column B operand.
//
// Role in the reference: replaces the Marlin W4A16 decode path and the int8-row / f16 GEMV
// family (crates/kernels/cu/marlin/*, crates/kernels/cu/elems/gemv_i8w_*.cu,
// crates/kernels/cu/elems/gemv_dual_f16.cu).
//
// ---- W4 record layout ("skinny tiles", produced by the load-time repacker) ----------------
// record(nt, kt) covers rows nt*16..+15 and k = kt*128..+127; records are stored
// [N/16][K/128] so all records of a row tile are one contiguous stream. A record is
//   1024 B : 64 x uint4; uint4 #L (L = g*4+t) = row nt*16+g, uint4 #(32+L) = row nt*16+8+g;
//            word w holds k = kt*128 + w*32 + t*8 + j (j = 0..7) at nibble position (j/2) + 4*(j%2),
//            so the four masked pairs of a word come out in k order
//   64 B x (128/G) : per group of the record 16 x half2 (scale, zero), row-major.
//
// ---- dense record layout (bf16: 16 rows x 64 k; int8: 16 rows x 128 k; 2048 B) ---------------
//   uint4 #((s*2 + half)*32 + L): row half*8+g, k = s*KH + t*KV .. +KV-1  (bf16: KH 32, KV 8;
//   int8: KH 64, KV 16)
//
// ---- activation pack ("ActPack", see actpack.cuh) ---------------------------------------------
// The int4 weights go to the integer tensor-core path (m16n8k32, u8 x s8/u8) as bytes: one AND
// extracts the four low nibbles of a weight word, one shift + AND the four high nibbles. The
// producer of the activations stores x as 15-bit fixed point (signed high byte, 7-bit low
// part, one scale per token and group) plus the group sum of x; then
//   sum_k (q_k - z) x_k = sx * (128 * acc_h + acc_l) - z * xsum   with exact int32 accumulation.
#include "common.cuh"
#include "actpack.cuh"

namespace owl {

__device__ int g_skinny_status = 0;   // first bounded-wait failure of any skinny kernel (0 = none)
// Lanes whose token column does not exist read their B fragments / group sums from this zero
// page (pointer step 0) instead of branching around the loads.
__device__ __align__(16) uint4 g_zero_page[32];

__device__ __forceinline__ void mma_f16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// m16n8k32 integer MMAs: A = unsigned weight bytes, B = signed (high plane) or unsigned (low plane)
__device__ __forceinline__ void imma_u8s8(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_u8u8(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {   // unsigned a bytes x signed b bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {   // unsigned x unsigned
  int d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
  return r;
}
// Non-multicast bulk copy global -> this CTA's shared memory, completion on an mbarrier.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU_MUL = 2, EPI_F32 = 3, EPI_SILU_PACK = 4, EPI_PUSH = 5, EPI_RESIDUAL_NORM = 6 };
constexpr int SK_MAX_RANKS = 8;
enum { KIND_W4_G128 = 0, KIND_W4_G32 = 1, KIND_BF16 = 2, KIND_W8 = 3 };

struct SkinnyParams {
  const uint8_t* w;      // record stream
  const float* row_scale;// w8: per-row scale
  const uint4* x;        // w4: ActPack fp16 [M][K]; bf16/w8: bf16 activations [M][K]
  const float2* xs;      // w4: (xsum, xoff) [M][K/G]
  void* out;             // bf16 [M][ldo] (or fp32 for EPI_F32)
  const __nv_bfloat16* residual;  // EPI_RESIDUAL: out = residual + y (may alias out)
  uint4* out_pack;       // EPI_SILU_PACK: ActPack of silu(gate)*up, [M][N/2] fp16
  float2* out_xs;        // EPI_SILU_PACK: [M][N/2/Gout]
  int M, N, K;
  int ldo;               // output row stride in elements
  int n_tiles;           // N / 16
  int tiles_per_cta;     // contiguous row tiles per CTA
  int gout;              // EPI_SILU_PACK: group size of the produced ActPack (32 or 128)
  int force_mma;         // tests / A-B runs: use the tensor-core arm even for one token
  int a8;                // activations were packed with ACT_A8 (low plane all zero): skip its products (W4A8 arm)
  // EPI_PUSH (tensor parallel, row-parallel projection): the partial sums go straight into every rank's
  // reduction buffer (plain peer stores over NVLink), slot [rank] of [world][push_rows][ldo] bf16, so the
  // transfer overlaps the streaming tile by tile; the CTA that finishes last publishes one sequence number per
  // peer and the consumer kernel (comm.cu: owl_push_residual_norm) only reads local memory.
  __nv_bfloat16* push_dst[SK_MAX_RANKS];   // base of the buffer on each rank (peer-mapped)
  uint32_t* push_flag[SK_MAX_RANKS];       // flag word of this call site on each rank, indexed [src rank]
  int* push_count;                         // local: CTAs of this launch that are done (returns to zero)
  uint32_t* push_seq;                      // local: sequence number of this call site
  int push_rank, push_world, push_rows;
  // EPI_RESIDUAL_NORM: out = residual + y, and the CTA that finishes last (push_count) RMS-normalises the M finished rows
  // and packs them for the next projection: the separate norm launch of the step disappears
  const __nv_bfloat16* norm_w;             // [N]
  __nv_bfloat16* normed;                   // optional bf16 [M][N]
  uint4* norm_pack; float2* norm_xs;       // optional ActPack of the normalised rows (row layout or tiles, by norm_g)
  int norm_g, norm_one_plus;
  float norm_eps;
};

constexpr int SK_WARPS = 8;    // warps per CTA = K slices of the record layout
constexpr int SK_SLOTS = 2;    // chunks in flight per warp
constexpr int SK_CHUNK_BYTES = 2176;   // bulk-copy size target (one mbarrier per chunk)

template <int KIND> struct RecInfo;
template <> struct RecInfo<KIND_W4_G128> { static constexpr int BYTES = 1024 + 64, KREC = 128; };
template <> struct RecInfo<KIND_W4_G32> { static constexpr int BYTES = 1024 + 256, KREC = 128; };
template <> struct RecInfo<KIND_BF16> { static constexpr int BYTES = 2048, KREC = 64; };
template <> struct RecInfo<KIND_W8> { static constexpr int BYTES = 2048, KREC = 128; };
template <int KIND> constexpr int chunk_recs() { return SK_CHUNK_BYTES / RecInfo<KIND>::BYTES > 0 ? SK_CHUNK_BYTES / RecInfo<KIND>::BYTES : 1; }

template <int MT, int KIND>
constexpr int skinny_smem_bytes() {
  // rings + barriers + split-K reduction (double buffered) + silu-pack staging (double buffered, bf16)
  return SK_WARPS * SK_SLOTS * chunk_recs<KIND>() * RecInfo<KIND>::BYTES + SK_WARPS * SK_SLOTS * 8 +
         2 * SK_WARPS * 32 * MT * 4 * 4 + 2 * MT * 8 * 128 * 2 + 128;
}

// m16n8k16 with a zero accumulator input (first MMA of a chain).
__device__ __forceinline__ void mma_f16_16816_z(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Records are stored slice-major: the K range is cut into SK_WARPS slices (slice w covers record
// columns [w*KT/8, (w+1)*KT/8)), and inside a slice the order is [row tile][record]. Warp w of a
// CTA that owns row tiles nt0.. therefore reads ONE contiguous byte stream, cut into fixed-size
// chunks that ignore row-tile boundaries (one bulk copy + one mbarrier per chunk).
// SIMT = true (single token only): the contraction runs on the CUDA cores with dp4a instead of the
// warp-level tensor-core path. On sm_100 the legacy mma.sync path issues one m16n8k16/k32 MMA per
// ~34 cycles per SM sub-core, which caps a W4 stream at ~4 TB/s (8 MMAs per 1088-byte record
// whatever the token count); for one token 32 dp4a per lane per record are cheaper than that.
template <int MT, int KIND, bool SIMT, bool A8>
__global__ void __launch_bounds__(SK_WARPS * 32, MT == 1 ? 4 : 2) skinny_stream_kernel(SkinnyParams p, int epi) {
  constexpr int REC = RecInfo<KIND>::BYTES, KREC = RecInfo<KIND>::KREC;
  constexpr bool W4 = KIND == KIND_W4_G128 || KIND == KIND_W4_G32;
  constexpr int G = KIND == KIND_W4_G32 ? 32 : 128;
  constexpr int GPT = 128 / G;
  constexpr int CH = chunk_recs<KIND>();
  constexpr int SLOT_BYTES = CH * REC;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring_all = smem;
  uint64_t* bars_all = reinterpret_cast<uint64_t*>(smem + SK_WARPS * SK_SLOTS * SLOT_BYTES);
  float* red = reinterpret_cast<float*>(bars_all + SK_WARPS * SK_SLOTS);
  __nv_bfloat16* gbuf = reinterpret_cast<__nv_bfloat16*>(red + 2 * SK_WARPS * 32 * MT * 4);

  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  uint8_t* ring = ring_all + (size_t)wi * SK_SLOTS * SLOT_BYTES;
  uint64_t* bars = bars_all + wi * SK_SLOTS;
  const int KT = p.K / KREC;
  const int nt0 = blockIdx.x * p.tiles_per_cta;
  const int n_items = min(p.tiles_per_cta, p.n_tiles - nt0);
  const int kt0 = (int)((long long)wi * KT / SK_WARPS), kt1 = (int)((long long)(wi + 1) * KT / SK_WARPS);
  const int rpi = kt1 - kt0;               // records per row tile for this warp's slice
  const int total = rpi * n_items;         // records this warp streams
  const uint8_t* wsrc = p.w + ((size_t)p.n_tiles * kt0 + (size_t)nt0 * rpi) * REC;   // start of this warp's stream
  const int n_chunks = (total + CH - 1) / CH;

  if (lane == 0) {
    for (int s = 0; s < SK_SLOTS; ++s) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  // Prologue: weights do not depend on the previous kernel, start streaming before the
  // programmatic-dependency wait.
  if (lane == 0) {
    for (int c = 0; c < SK_SLOTS && c < n_chunks; ++c) {
      const uint32_t bytes = (uint32_t)min(CH, total - c * CH) * REC;
      mbar_expect_tx(&bars[c], bytes);
      bulk_g2s(ring + (size_t)c * SLOT_BYTES, wsrc + (size_t)c * SLOT_BYTES, bytes, &bars[c]);
    }
  }
  pdl_wait();

  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;
  bool failed = false;
  constexpr int XSTRIDE = (KIND == KIND_BF16) ? 8 : 16;   // uint4 of x per record and token
  const uint4* xbase[MT];
  const float2 *xsA[MT], *xsB[MT];
  int xstep[MT], sstepA[MT], sstepB[MT];
  const int KG = p.K / G;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const int tok = SIMT ? 0 : m * 8 + g;
    const bool ok = tok < p.M;
    xbase[m] = ok ? p.x + ((size_t)tok * p.K) / 8 + (size_t)kt0 * XSTRIDE + (KIND == KIND_W8 ? t * 2 : t) : g_zero_page;
    xstep[m] = ok ? XSTRIDE : 0;
    const int tokA = SIMT ? 0 : m * 8 + 2 * t;
    const float2* z2 = reinterpret_cast<const float2*>(g_zero_page);
    xsA[m] = (W4 && tokA < p.M) ? p.xs + (size_t)tokA * KG + (size_t)kt0 * GPT : z2;
    xsB[m] = (W4 && tokA + 1 < p.M) ? p.xs + (size_t)(tokA + 1) * KG + (size_t)kt0 * GPT : z2;
    sstepA[m] = (W4 && tokA < p.M) ? GPT : 0;
    sstepB[m] = (W4 && tokA + 1 < p.M) ? GPT : 0;
  }

  int item = 0, kk = 0;       // position of the current record: row tile nt0+item, record kt0+kk
  int chunk = 0, in_chunk = 0, slot = 0;
  uint32_t parity = 0;
  const uint8_t* rec_b = ring;
  for (int j = 0; j < total || item < n_items; ++j) {
    if (j < total) {
      // B fragments first (L1/L2 hits) so they overlap the wait for the weight record.
      uint4 xb[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4* xp = xbase[m] + kk * xstep[m];
        if (W4) {
#pragma unroll
          for (int w = 0; w < 4; ++w) xb[m][w] = __ldg(xp + w * 4);
        } else if (KIND == KIND_BF16) {
          xb[m][0] = __ldg(xp); xb[m][1] = __ldg(xp + 4);
        } else {
          xb[m][0] = __ldg(xp); xb[m][1] = __ldg(xp + 1);       // k-step 0: 16 consecutive x
          xb[m][2] = __ldg(xp + 8); xb[m][3] = __ldg(xp + 9);   // k-step 1 (+64 k)
        }
      }
      float2 sa[MT][GPT], sb[MT][GPT];
      if (W4) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int q = 0; q < GPT; ++q) {
            sa[m][q] = __ldg(xsA[m] + kk * sstepA[m] + q);
            sb[m][q] = __ldg(xsB[m] + kk * sstepB[m] + q);
          }
      }
      if (in_chunk == 0) {
        if (!failed && !mbar_wait(&bars[slot], parity, 1u << 22)) {
          failed = true;
          atomicCAS(&g_skinny_status, 0, OWL_ERR_WAIT_TMA);
        }
      }
      const uint4* rec = reinterpret_cast<const uint4*>(rec_b);
      if (W4) {
        const uint4 lo = rec[lane], hi = rec[32 + lane];
        const uint32_t ql[4] = {lo.x, lo.y, lo.z, lo.w};   // row g:   word w = bytes of k-run (w, t)
        const uint32_t qh[4] = {hi.x, hi.y, hi.z, hi.w};   // row g+8
        const uint32_t* szr = reinterpret_cast<const uint32_t*>(rec + 64);
        uint32_t su0[GPT], su1[GPT];
#pragma unroll
        for (int q = 0; q < GPT; ++q) { su0[q] = szr[q * 16 + g]; su1[q] = szr[q * 16 + 8 + g]; }
        uint32_t nl[4], nh[4], ul[4], uh[4];                // low / high nibbles as bytes, rows g / g+8
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          nl[w] = ql[w] & 0x0F0F0F0Fu; nh[w] = qh[w] & 0x0F0F0F0Fu;
          ul[w] = (ql[w] >> 4) & 0x0F0F0F0Fu; uh[w] = (qh[w] >> 4) & 0x0F0F0F0Fu;
        }
        // xb[m][w] = chunk of k-run (w, t) for token g: .x/.y = high/low byte plane of the
        // activations under the low nibbles, .z/.w = the same for the high nibbles.
        if (SIMT) {
          // one token: per row (g, g+8) and word, 4 dp4a; the partial sums cover this lane's k-runs
          // (quarter t of every word), the four t lanes are summed once per row tile
#pragma unroll
          for (int q = 0; q < GPT; ++q) {
            int h0 = 0, l0 = 0, h1 = 0, l1 = 0;
#pragma unroll
            if (A8) {      // 8-bit activations: the low plane is zero, half the products
#pragma unroll
              for (int w = (G == 128 ? 0 : q); w < (G == 128 ? 4 : q + 1); ++w) {
                h0 = dp4a_us(nl[w], xb[0][w].x, h0); h0 = dp4a_us(ul[w], xb[0][w].z, h0);
                h1 = dp4a_us(nh[w], xb[0][w].x, h1); h1 = dp4a_us(uh[w], xb[0][w].z, h1);
              }
            } else {
#pragma unroll
              for (int w = (G == 128 ? 0 : q); w < (G == 128 ? 4 : q + 1); ++w) {
                h0 = dp4a_us(nl[w], xb[0][w].x, h0); l0 = dp4a_uu(nl[w], xb[0][w].y, l0);
                h0 = dp4a_us(ul[w], xb[0][w].z, h0); l0 = dp4a_uu(ul[w], xb[0][w].w, l0);
                h1 = dp4a_us(nh[w], xb[0][w].x, h1); l1 = dp4a_uu(nh[w], xb[0][w].y, l1);
                h1 = dp4a_us(uh[w], xb[0][w].z, h1); l1 = dp4a_uu(uh[w], xb[0][w].w, l1);
              }
            }
            const __half2 hh0 = *reinterpret_cast<const __half2*>(&su0[q]);
            const __half2 hh1 = *reinterpret_cast<const __half2*>(&su1[q]);
            const float sc0 = __low2float(hh0), z0 = __high2float(hh0);
            const float sc1 = __low2float(hh1), z1 = __high2float(hh1);
            const float xq = 0.25f * sa[0][q].y;    // each of the 4 t lanes carries a quarter of z * xsum
            acc[0][0] = fmaf(sc0, fmaf(sa[0][q].x, (float)(h0 * 128 + l0), -z0 * xq), acc[0][0]);
            acc[0][2] = fmaf(sc1, fmaf(sa[0][q].x, (float)(h1 * 128 + l1), -z1 * xq), acc[0][2]);
          }
        } else if (G == 128) {
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            int ch[4] = {0, 0, 0, 0}, cl[4] = {0, 0, 0, 0};
#pragma unroll
            for (int i = 0; i < 2; ++i) {   // one k32-byte MMA covers words 2i and 2i+1
              imma_u8s8(ch, nl[2 * i], nh[2 * i], nl[2 * i + 1], nh[2 * i + 1], xb[m][2 * i].x, xb[m][2 * i + 1].x);
              imma_u8s8(ch, ul[2 * i], uh[2 * i], ul[2 * i + 1], uh[2 * i + 1], xb[m][2 * i].z, xb[m][2 * i + 1].z);
              if (!A8) {
                imma_u8u8(cl, nl[2 * i], nh[2 * i], nl[2 * i + 1], nh[2 * i + 1], xb[m][2 * i].y, xb[m][2 * i + 1].y);
                imma_u8u8(cl, ul[2 * i], uh[2 * i], ul[2 * i + 1], uh[2 * i + 1], xb[m][2 * i].w, xb[m][2 * i + 1].w);
              }
            }
            const __half2 h0 = *reinterpret_cast<const __half2*>(&su0[0]);
            const __half2 h1 = *reinterpret_cast<const __half2*>(&su1[0]);
            const float sc0 = __low2float(h0), z0 = __high2float(h0);
            const float sc1 = __low2float(h1), z1 = __high2float(h1);
            const float f0 = (float)(ch[0] * 128 + cl[0]), f1 = (float)(ch[1] * 128 + cl[1]);
            const float f2 = (float)(ch[2] * 128 + cl[2]), f3 = (float)(ch[3] * 128 + cl[3]);
            acc[m][0] = fmaf(sc0, fmaf(sa[m][0].x, f0, -z0 * sa[m][0].y), acc[m][0]);
            acc[m][1] = fmaf(sc0, fmaf(sb[m][0].x, f1, -z0 * sb[m][0].y), acc[m][1]);
            acc[m][2] = fmaf(sc1, fmaf(sa[m][0].x, f2, -z1 * sa[m][0].y), acc[m][2]);
            acc[m][3] = fmaf(sc1, fmaf(sb[m][0].x, f3, -z1 * sb[m][0].y), acc[m][3]);
          }
        } else {
          // group 32 = one word per group: the second half of the k32 MMA is fed zeros
#pragma unroll
          for (int q = 0; q < GPT; ++q) {
            const __half2 h0 = *reinterpret_cast<const __half2*>(&su0[q]);
            const __half2 h1 = *reinterpret_cast<const __half2*>(&su1[q]);
            const float sc0 = __low2float(h0), z0 = __high2float(h0);
            const float sc1 = __low2float(h1), z1 = __high2float(h1);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              int ch[4] = {0, 0, 0, 0}, cl[4] = {0, 0, 0, 0};
              imma_u8s8(ch, nl[q], nh[q], 0u, 0u, xb[m][q].x, 0u);
              imma_u8s8(ch, ul[q], uh[q], 0u, 0u, xb[m][q].z, 0u);
              if (!A8) {
                imma_u8u8(cl, nl[q], nh[q], 0u, 0u, xb[m][q].y, 0u);
                imma_u8u8(cl, ul[q], uh[q], 0u, 0u, xb[m][q].w, 0u);
              }
              const float f0 = (float)(ch[0] * 128 + cl[0]), f1 = (float)(ch[1] * 128 + cl[1]);
              const float f2 = (float)(ch[2] * 128 + cl[2]), f3 = (float)(ch[3] * 128 + cl[3]);
              acc[m][0] = fmaf(sc0, fmaf(sa[m][q].x, f0, -z0 * sa[m][q].y), acc[m][0]);
              acc[m][1] = fmaf(sc0, fmaf(sb[m][q].x, f1, -z0 * sb[m][q].y), acc[m][1]);
              acc[m][2] = fmaf(sc1, fmaf(sa[m][q].x, f2, -z1 * sa[m][q].y), acc[m][2]);
              acc[m][3] = fmaf(sc1, fmaf(sb[m][q].x, f3, -z1 * sb[m][q].y), acc[m][3]);
            }
          }
        }
      } else if (KIND == KIND_BF16) {
        const uint4 a0 = rec[0 * 32 + lane], b0 = rec[1 * 32 + lane];
        const uint4 a1 = rec[2 * 32 + lane], b1 = rec[3 * 32 + lane];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float c2[4] = {0.f, 0.f, 0.f, 0.f};
          mma_bf16_16816(acc[m], a0.x, b0.x, a0.y, b0.y, xb[m][0].x, xb[m][0].y);
          mma_bf16_16816(c2, a1.x, b1.x, a1.y, b1.y, xb[m][1].x, xb[m][1].y);
          mma_bf16_16816(acc[m], a0.z, b0.z, a0.w, b0.w, xb[m][0].z, xb[m][0].w);
          mma_bf16_16816(c2, a1.z, b1.z, a1.w, b1.w, xb[m][1].z, xb[m][1].w);
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[m][i] += c2[i];
        }
      } else {
        // int8 -> fp16 by byte permute: (w ^ 0x80) is the biased byte b = w + 128, and the half
        // with bit pattern 0x6400 | b equals 1024 + b; subtracting 1152 restores w exactly.
        const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
        auto cvt = [&](uint32_t v, uint32_t sel) -> uint32_t {
          uint32_t r = __byte_perm(v, 0x64646464u, sel);
          __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r), bias);
          return *reinterpret_cast<uint32_t*>(&h);
        };
        auto x16 = [&](uint32_t v) -> uint32_t { return pack_f16(bf16_lo(v), bf16_hi(v)); };
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint4 a = rec[(s * 2 + 0) * 32 + lane], b = rec[(s * 2 + 1) * 32 + lane];
          const uint32_t al[4] = {a.x ^ 0x80808080u, a.y ^ 0x80808080u, a.z ^ 0x80808080u, a.w ^ 0x80808080u};
          const uint32_t bl[4] = {b.x ^ 0x80808080u, b.y ^ 0x80808080u, b.z ^ 0x80808080u, b.w ^ 0x80808080u};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t fa[4], fb[4];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              fa[u * 2 + 0] = cvt(al[h * 2 + u], 0x4140u);
              fa[u * 2 + 1] = cvt(al[h * 2 + u], 0x4342u);
              fb[u * 2 + 0] = cvt(bl[h * 2 + u], 0x4140u);
              fb[u * 2 + 1] = cvt(bl[h * 2 + u], 0x4342u);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const uint4 xv = xb[m][s * 2 + h];
              mma_f16_16816(acc[m], fa[0], fb[0], fa[1], fb[1], x16(xv.x), x16(xv.y));
              mma_f16_16816(acc[m], fa[2], fb[2], fa[3], fb[3], x16(xv.z), x16(xv.w));
            }
          }
        }
      }
      rec_b += REC;
      if (++in_chunk == CH || j + 1 == total) {
        // every lane has consumed this chunk (its MMAs used the loaded registers): refill the slot
        __syncwarp();
        const int nc = chunk + SK_SLOTS;
        if (lane == 0 && nc < n_chunks) {
          const uint32_t bytes = (uint32_t)min(CH, total - nc * CH) * REC;
          mbar_expect_tx(&bars[slot], bytes);
          bulk_g2s(ring + (size_t)slot * SLOT_BYTES, wsrc + (size_t)nc * SLOT_BYTES, bytes, &bars[slot]);
        }
        ++chunk; in_chunk = 0;
        if (++slot == SK_SLOTS) { slot = 0; parity ^= 1u; }
        rec_b = ring + (size_t)slot * SLOT_BYTES;
      }
      if (++kk < rpi) continue;
      kk = 0;
    }
    // ---- end of a row tile (warps with an empty slice come straight here) -------------------
    const int nt = nt0 + item;
    if (KIND == KIND_W8) {
      const float s0 = p.row_scale[nt * 16 + g], s1 = p.row_scale[nt * 16 + g + 8];
#pragma unroll
      for (int m = 0; m < MT; ++m) { acc[m][0] *= s0; acc[m][1] *= s0; acc[m][2] *= s1; acc[m][3] *= s1; }
    }
    if (SIMT) {
      acc[0][0] += __shfl_xor_sync(0xffffffffu, acc[0][0], 1);
      acc[0][0] += __shfl_xor_sync(0xffffffffu, acc[0][0], 2);
      acc[0][2] += __shfl_xor_sync(0xffffffffu, acc[0][2], 1);
      acc[0][2] += __shfl_xor_sync(0xffffffffu, acc[0][2], 2);
    }
    // split-K reduction across the 8 warps (double buffered: one barrier per item)
    float* rbuf = red + (size_t)(item & 1) * SK_WARPS * 32 * MT * 4;
    float* mine = rbuf + ((size_t)wi * 32 + lane) * (MT * 4);
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i) { mine[m * 4 + i] = acc[m][i]; acc[m][i] = 0.f; }
    __syncthreads();
    const int fin = item & (SK_WARPS - 1);   // rotate the finishing warp
    if (wi == fin) {
      float r[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) r[m][i] = 0.f;
      for (int s = 0; s < SK_WARPS; ++s) {
        const float* o = rbuf + ((size_t)s * 32 + lane) * (MT * 4);
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int i = 0; i < 4; ++i) r[m][i] += o[m * 4 + i];
      }
      const int grp = item >> 4;            // 16 row tiles = 128 silu outputs = one pack group set
      __nv_bfloat16* gb = gbuf + (size_t)(grp & 1) * MT * 8 * 128;

#pragma unroll
      for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int tok = m * 8 + 2 * t + jj;
          const float v_lo = r[m][jj], v_hi = r[m][2 + jj];  // rows g and g+8
          if (epi == EPI_SILU_PACK) {
            gb[(size_t)(m * 8 + 2 * t + jj) * 128 + (item & 15) * 8 + g] = __float2bfloat16(silu_f(v_lo) * v_hi);
          } else if (tok < p.M) {
            if (epi == EPI_SILU_MUL) {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)tok * p.ldo + nt * 8 + g;
              *o = __float2bfloat16(silu_f(v_lo) * v_hi);
            } else if (epi == EPI_F32) {
              float* o = reinterpret_cast<float*>(p.out) + (size_t)tok * p.ldo + nt * 16 + g;
              o[0] = v_lo; o[8] = v_hi;
            } else if (epi == EPI_PUSH) {
              const __nv_bfloat16 a = __float2bfloat16(v_lo), b = __float2bfloat16(v_hi);
              const size_t off = ((size_t)p.push_rank * p.push_rows + tok) * p.ldo + nt * 16 + g;
              for (int r = 0; r < p.push_world; ++r) { p.push_dst[r][off] = a; p.push_dst[r][off + 8] = b; }
            } else {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)tok * p.ldo + nt * 16 + g;
              float a = v_lo, b = v_hi;
              if (epi == EPI_RESIDUAL || epi == EPI_RESIDUAL_NORM) {
                const __nv_bfloat16* rr = p.residual + (size_t)tok * p.ldo + nt * 16 + g;
                a += __bfloat162float(rr[0]); b += __bfloat162float(rr[8]);
              }
              o[0] = __float2bfloat16(a); o[8] = __float2bfloat16(b);
            }
          }
        }
      }
      if (epi == EPI_SILU_PACK && (item & 15) == 15) {
        // 128 activations per token are complete (earlier tiles were finished by other warps
        // before they reached this item's barrier): pack them. Host guarantees tiles_per_cta % 16 == 0.
        __syncwarp();
        const int I = p.N / 2;
        const int col0 = ((nt0 + (item & ~15)) >> 4) * 128;   // first output column of this group
        const int cpg = p.gout >> 3;
        for (int c = lane; c < MT * 8 * 16; c += 32) {
          const int tok = c >> 4, ch = c & 15;
          float v8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v8[i] = __bfloat162float(gb[(size_t)tok * 128 + ch * 8 + i]);
          float sx, xsum;
          const uint4 pk = actpack_emit(v8, cpg, sx, xsum);
          if (tok < p.M) {
            p.out_pack[((size_t)tok * I + col0) / 8 + ch] = pk;
            if ((ch % cpg) == 0) p.out_xs[(size_t)tok * (I / p.gout) + col0 / p.gout + ch / cpg] = make_float2(sx, xsum);
          }
        }
      }
    }
    ++item;
  }
  if (epi == EPI_PUSH) {
    // every thread's peer stores are ordered before the count; the last CTA of the grid tells the peers
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      if (atomicAdd(p.push_count, 1) == (int)gridDim.x - 1) {
        *p.push_count = 0;
        const uint32_t seq = *p.push_seq + 1;
        *p.push_seq = seq;
        __threadfence_system();
        for (int r = 0; r < p.push_world; ++r)
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.push_flag[r] + p.push_rank), "r"(seq) : "memory");
      }
    }
  }
  if (epi == EPI_RESIDUAL_NORM) {
    __shared__ int s_last;
    __shared__ float s_red[32];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int last = atomicAdd(p.push_count, 1) == (int)gridDim.x - 1;
      if (last) *p.push_count = 0;
      s_last = last;
      __threadfence();
    }
    __syncthreads();
    if (s_last) {
      // every CTA's rows are in global memory (fence + count): read them past L1
      const int nchunks = p.N >> 3, tiles = p.norm_g & ACT_TILES, gq = p.norm_g & ~ACT_TILES, cpg = gq >> 3;
      const int nround = (nchunks + 31) & ~31;
      const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(p.out);
      for (int row = 0; row < p.M; ++row) {
        const uint4* hp = reinterpret_cast<const uint4*>(hb + (size_t)row * p.ldo);
        float ss = 0.f;
        for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
          float v[8];
          unpack_bf16x8(__ldcg(hp + c), v);
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
        }
        ss = block_sum(ss, s_red);
        const float rinv = rsqrtf(ss / (float)p.N + p.norm_eps);
        for (int c = threadIdx.x; c < nround; c += blockDim.x) {
          float v[8];
          const bool live = c < nchunks;
          if (live) {
            float wf[8];
            unpack_bf16x8(__ldcg(hp + c), v);
            unpack_bf16x8(reinterpret_cast<const uint4*>(p.norm_w)[c], wf);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              v[i] = __bfloat162float(__float2bfloat16(v[i] * rinv * (p.norm_one_plus ? 1.f + wf[i] : wf[i])));
            if (p.normed) reinterpret_cast<uint4*>(p.normed + (size_t)row * p.N)[c] = pack_bf16x8(v);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
          }
          if (p.norm_pack) {
            float sx, xsum;
            const uint4 pk = actpack_emit(v, cpg, sx, xsum);
            if (live) actpack_store(p.norm_pack, p.norm_xs, tiles, gq, row, c, nchunks, pk, sx, xsum);
          }
        }
      }
    }
  }
  // Dependents are released when this CTA is done streaming: releasing them earlier only parks
  // their CTAs on SM resources this kernel still needs (measured slower).
  pdl_launch_dependents();
}

template <int MT, int KIND, bool SIMT = false, bool A8 = false>
static int launch_skinny(const SkinnyParams& p, int epi, int pdl, cudaStream_t st) {
  auto kernel = skinny_stream_kernel<MT, KIND, SIMT, A8>;
  constexpr int smem = skinny_smem_bytes<MT, KIND>();
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
    attr_done = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.n_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta);
  cfg.blockDim = dim3(SK_WARPS * 32);
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

// Contiguous row tiles per CTA: enough CTAs to fill every SM twice, multiples of 16 for the
// fused pack epilogue.
static int pick_tiles_per_cta(int n_tiles, int epi, int want) {
  int tpc = want > 0 ? want : (n_tiles + 591) / 592;   // ~4 CTAs per SM: the dp4a arm needs the warps
  if (tpc < 1) tpc = 1;
  if (epi == EPI_SILU_PACK) tpc = ((tpc + 15) / 16) * 16;
  return tpc;
}

template <int KIND>
static int dispatch_mt(const SkinnyParams& p, int epi, int pdl, cudaStream_t st) {
  const int mt = (p.M + 7) / 8;
  constexpr bool W4K = KIND == KIND_W4_G128 || KIND == KIND_W4_G32;
  if constexpr (W4K) {
    if (p.a8) {      // W4A8 arm: its own instantiations, so the 15-bit kernels keep their code
      if (p.M == 1 && !p.force_mma) return launch_skinny<1, KIND, true, true>(p, epi, pdl, st);
      if (mt == 1) return launch_skinny<1, KIND, false, true>(p, epi, pdl, st);
      if (mt == 2) return launch_skinny<2, KIND, false, true>(p, epi, pdl, st);
      return launch_skinny<4, KIND, false, true>(p, epi, pdl, st);
    }
  }
  if (W4K && p.M == 1 && !p.force_mma) return launch_skinny<1, KIND, W4K>(p, epi, pdl, st);
  if (mt == 1) return launch_skinny<1, KIND>(p, epi, pdl, st);
  if (mt == 2) return launch_skinny<2, KIND>(p, epi, pdl, st);
  return launch_skinny<4, KIND>(p, epi, pdl, st);
}

}  // namespace owl

using namespace owl;

// out[M, ldo] (bf16, or fp32 with epi=3). group is 32 or 128. epi: 0 store, 1 residual add,
// 2 silu(gate)*up with gate/up rows interleaved per 16-row tile (rows 0-7 gate, 8-15 up), 3 fp32
// store, 4 = 2 but written as ActPack (out_pack/out_xs, group gout) instead of bf16.
OWL_API int owl_w4a16_skinny(const void* records, const void* xpack, const void* xsums, void* out,
                             const void* residual, void* out_pack, void* out_xs, int M, int N, int K, int ldo,
                             int group, int epi, int gout, int tiles_per_cta, int pdl, cudaStream_t st) {
  if (M < 1 || M > 32 || (N & 15) || (K & 127) || (group != 32 && group != 128)) return OWL_ERR_BAD_ARG;
  if (epi == EPI_RESIDUAL && !residual) return OWL_ERR_BAD_ARG;
  if (epi != EPI_SILU_PACK && !out) return OWL_ERR_BAD_ARG;
  if (epi == EPI_SILU_PACK && ((N & 255) || (gout != 32 && gout != 128) || !out_pack || !out_xs)) return OWL_ERR_BAD_ARG;
  SkinnyParams p = {};
  p.w = (const uint8_t*)records; p.x = (const uint4*)xpack; p.xs = (const float2*)xsums;
  p.out = out; p.residual = (const __nv_bfloat16*)residual; p.out_pack = (uint4*)out_pack; p.out_xs = (float2*)out_xs;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.gout = gout;
  p.n_tiles = N / 16;
  p.force_mma = (tiles_per_cta < 0);
  p.tiles_per_cta = pick_tiles_per_cta(p.n_tiles, epi, tiles_per_cta < 0 ? -tiles_per_cta - 1 : tiles_per_cta);
  return group == 128 ? dispatch_mt<KIND_W4_G128>(p, epi, pdl, st) : dispatch_mt<KIND_W4_G32>(p, epi, pdl, st);
}

// W4A8 arm: the same launch for activations packed with ACT_A8 (8-bit, low plane zero): half the integer products.
OWL_API int owl_w4a16_skinny_a8(const void* records, const void* xpack, const void* xsums, void* out, const void* residual,
                                int M, int N, int K, int ldo, int group, int epi, int force_mma, int pdl, cudaStream_t st) {
  if (M < 1 || M > 32 || (N & 15) || (K & 127) || (group != 32 && group != 128) || !out) return OWL_ERR_BAD_ARG;
  if (epi != EPI_STORE && epi != EPI_RESIDUAL && epi != EPI_SILU_MUL && epi != EPI_F32) return OWL_ERR_BAD_ARG;
  if (epi == EPI_RESIDUAL && !residual) return OWL_ERR_BAD_ARG;
  SkinnyParams p = {};
  p.w = (const uint8_t*)records; p.x = (const uint4*)xpack; p.xs = (const float2*)xsums;
  p.out = out; p.residual = (const __nv_bfloat16*)residual;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.n_tiles = N / 16; p.force_mma = force_mma; p.a8 = 1;
  p.tiles_per_cta = pick_tiles_per_cta(p.n_tiles, epi, 0);
  return group == 128 ? dispatch_mt<KIND_W4_G128>(p, epi, pdl, st) : dispatch_mt<KIND_W4_G32>(p, epi, pdl, st);
}

// Row projection with the residual add AND the following RMSNorm + activation packing in one launch (EPI_RESIDUAL_NORM):
// out = residual + W x; the last CTA to finish normalises the M rows of `out` with norm_w and writes `normed` (bf16, optional)
// and / or the ActPack (norm_pack / norm_xs, group norm_g, optionally | ACT_TILES). count: local int, zero before the first call.
OWL_API int owl_w4a16_skinny_norm(const void* records, const void* xpack, const void* xsums, void* out, const void* residual,
                                  const void* norm_w, void* normed, void* norm_pack, void* norm_xs, void* count, int M, int N,
                                  int K, int ldo, int group, int norm_g, float eps, int one_plus_w, int force_mma, int pdl,
                                  cudaStream_t st) {
  if (M < 1 || M > 32 || (N & 127) || (K & 127) || (group != 32 && group != 128) || !out || !residual || !norm_w || !count ||
      ldo != N || !actpack_group_ok(norm_g, M) || (!normed && !norm_pack) || (norm_pack && !norm_xs && !(norm_g & ACT_TILES)))
    return OWL_ERR_BAD_ARG;
  SkinnyParams p = {};
  p.w = (const uint8_t*)records; p.x = (const uint4*)xpack; p.xs = (const float2*)xsums;
  p.out = out; p.residual = (const __nv_bfloat16*)residual;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.n_tiles = N / 16; p.force_mma = force_mma;
  p.tiles_per_cta = pick_tiles_per_cta(p.n_tiles, EPI_RESIDUAL, 0);
  p.push_count = (int*)count;
  p.norm_w = (const __nv_bfloat16*)norm_w; p.normed = (__nv_bfloat16*)normed; p.norm_pack = (uint4*)norm_pack;
  p.norm_xs = (float2*)norm_xs; p.norm_g = norm_g; p.norm_one_plus = one_plus_w; p.norm_eps = eps;
  return group == 128 ? dispatch_mt<KIND_W4_G128>(p, EPI_RESIDUAL_NORM, pdl, st) : dispatch_mt<KIND_W4_G32>(p, EPI_RESIDUAL_NORM, pdl, st);
}

// Tensor-parallel variant for row-parallel projections: the partial sums are written into every rank's
// reduction buffer instead of a local output (see EPI_PUSH). dst_ptrs / flag_ptrs: host arrays of `world`
// peer-mapped device pointers (buffer base [world][push_rows][ldo] bf16; flag words [world] uint32 of this call
// site); count / seq: local device words (zero before the first call).
OWL_API int owl_w4a16_skinny_push(const void* records, const void* xpack, const void* xsums, void* const* dst_ptrs,
                                  void* const* flag_ptrs, void* count, void* seq, int M, int N, int K, int ldo, int group,
                                  int rank, int world, int push_rows, int force_mma, int pdl, cudaStream_t st) {
  if (M < 1 || M > 32 || M > push_rows || (N & 15) || (K & 127) || (group != 32 && group != 128) || world < 2 ||
      world > SK_MAX_RANKS || rank < 0 || rank >= world || !count || !seq)
    return OWL_ERR_BAD_ARG;
  SkinnyParams p = {};
  p.w = (const uint8_t*)records; p.x = (const uint4*)xpack; p.xs = (const float2*)xsums;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.gout = 128;
  p.n_tiles = N / 16;
  p.force_mma = force_mma;
  p.tiles_per_cta = pick_tiles_per_cta(p.n_tiles, EPI_PUSH, 0);
  for (int r = 0; r < world; ++r) { p.push_dst[r] = (__nv_bfloat16*)dst_ptrs[r]; p.push_flag[r] = (uint32_t*)flag_ptrs[r]; }
  p.push_count = (int*)count; p.push_seq = (uint32_t*)seq; p.push_rank = rank; p.push_world = world; p.push_rows = push_rows;
  return group == 128 ? dispatch_mt<KIND_W4_G128>(p, EPI_PUSH, pdl, st) : dispatch_mt<KIND_W4_G32>(p, EPI_PUSH, pdl, st);
}

// w: dense bf16 records [N/16][K/64][2048 B].
OWL_API int owl_bf16_skinny(const void* w, const void* x, void* out, const void* residual, int M, int N, int K,
                            int ldo, int epi, int tiles_per_cta, int pdl, cudaStream_t st) {
  if (M < 1 || M > 32 || (N & 15) || (K & 63) || epi == EPI_SILU_PACK || !out || (epi == EPI_RESIDUAL && !residual))
    return OWL_ERR_BAD_ARG;
  SkinnyParams p = {};
  p.w = (const uint8_t*)w; p.x = (const uint4*)x; p.out = out; p.residual = (const __nv_bfloat16*)residual;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.n_tiles = N / 16;
  p.tiles_per_cta = pick_tiles_per_cta(p.n_tiles, epi, tiles_per_cta);
  return dispatch_mt<KIND_BF16>(p, epi, pdl, st);
}

// w: int8 records [N/16][K/128][2048 B]; row_scale fp32 [N].
OWL_API int owl_w8a16_skinny(const void* w, const void* row_scale, const void* x, void* out, int M, int N, int K,
                             int ldo, int epi, int tiles_per_cta, int pdl, cudaStream_t st) {
  if (M < 1 || M > 32 || (N & 15) || (K & 127) || epi == EPI_SILU_PACK || epi == EPI_RESIDUAL || !out)
    return OWL_ERR_BAD_ARG;
  SkinnyParams p = {};
  p.w = (const uint8_t*)w; p.row_scale = (const float*)row_scale; p.x = (const uint4*)x; p.out = out;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.n_tiles = N / 16;
  p.tiles_per_cta = pick_tiles_per_cta(p.n_tiles, epi, tiles_per_cta);
  return dispatch_mt<KIND_W8>(p, epi, pdl, st);
}

// First bounded-wait failure recorded by a skinny kernel since the last call (0 = none); clears it.
OWL_API int owl_skinny_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_skinny_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_skinny_status, &zero, sizeof(int));
  return v;
}
