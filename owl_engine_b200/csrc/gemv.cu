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
// ---- activation pack ("ActPack") --------------------------------------------------------------
// The int4 -> fp16 conversion uses the exponent-bias trick: (q & 0x000F000F) | 0x64006400 is
// the half2 (1024+q_lo, 1024+q_hi), and the same with mask 0x00F000F0 is (1024+16 q, ...).
// Instead of subtracting the bias and rescaling per weight, the producer of the activations
// stores them pre-permuted and pre-scaled as fp16:
//   per 8 consecutive k: [x0, x1, x2/16, x3/16, x4, x5, x6/16, x7/16]
// plus per (token, group) two fp32 sums: xsum = sum of effective x, xoff = 1024 * sum of the
// stored halves. Then  sum_k (q_k - z) x_k = acc - xoff - z * xsum  exactly (fp32 accumulate).
#include "common.cuh"
#include "actpack.cuh"

namespace owl {

__device__ int g_skinny_status = 0;   // first bounded-wait failure of any skinny kernel (0 = none)

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

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU_MUL = 2, EPI_F32 = 3, EPI_SILU_PACK = 4 };
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
};

constexpr int SK_WARPS = 8;    // warps per CTA = K slices of the record layout
constexpr int SK_SLOTS = 2;    // chunks in flight per warp
constexpr int SK_CHUNK_BYTES = 4352;   // bulk-copy size target (one mbarrier per chunk)

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
template <int MT, int KIND>
__global__ void __launch_bounds__(SK_WARPS * 32, 2) skinny_stream_kernel(SkinnyParams p, int epi) {
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
  // Let the next kernel's CTAs come in as SM resources free up: their own weight prefetch
  // overlaps the tail of this kernel (they still wait for this grid before reading its output).
  pdl_launch_dependents();

  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;
  bool failed = false;
  constexpr int XSTRIDE = (KIND == KIND_BF16) ? 8 : 16;   // uint4 of x per record and token
  const uint4* xbase[MT];
  const float2* xsA[MT];
  bool tok_ok[MT], okA[MT], okB[MT];
  const int KG = p.K / G;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const int tok = m * 8 + g;
    tok_ok[m] = tok < p.M;
    xbase[m] = p.x + ((size_t)tok * p.K) / 8 + (size_t)kt0 * XSTRIDE + (KIND == KIND_W8 ? t * 2 : t);
    const int tokA = m * 8 + 2 * t;
    okA[m] = tokA < p.M; okB[m] = tokA + 1 < p.M;
    xsA[m] = W4 ? p.xs + (size_t)tokA * KG + (size_t)kt0 * GPT : nullptr;
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
        const uint4* xp = xbase[m] + (size_t)kk * XSTRIDE;
        if (tok_ok[m]) {
          if (W4) {
#pragma unroll
            for (int w = 0; w < 4; ++w) xb[m][w] = __ldg(xp + w * 4);
          } else if (KIND == KIND_BF16) {
            xb[m][0] = __ldg(xp); xb[m][1] = __ldg(xp + 4);
          } else {
            xb[m][0] = __ldg(xp); xb[m][1] = __ldg(xp + 1);       // k-step 0: 16 consecutive x
            xb[m][2] = __ldg(xp + 8); xb[m][3] = __ldg(xp + 9);   // k-step 1 (+64 k)
          }
        } else {
#pragma unroll
          for (int w = 0; w < 4; ++w) xb[m][w] = make_uint4(0, 0, 0, 0);
        }
      }
      float2 sa[MT][GPT], sb[MT][GPT];
      if (W4) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int q = 0; q < GPT; ++q) {
            sa[m][q] = okA[m] ? __ldg(xsA[m] + kk * GPT + q) : make_float2(0.f, 0.f);
            sb[m][q] = okB[m] ? __ldg(xsA[m] + KG + kk * GPT + q) : make_float2(0.f, 0.f);
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
        const uint32_t ql[4] = {lo.x, lo.y, lo.z, lo.w};
        const uint32_t qh[4] = {hi.x, hi.y, hi.z, hi.w};
        const uint32_t* szr = reinterpret_cast<const uint32_t*>(rec + 64);
        uint32_t su0[GPT], su1[GPT];
#pragma unroll
        for (int q = 0; q < GPT; ++q) { su0[q] = szr[q * 16 + g]; su1[q] = szr[q * 16 + 8 + g]; }
        uint32_t fa[4][8];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          fa[w][0] = lop3_and_or(ql[w], 0x000F000Fu, 0x64006400u);
          fa[w][2] = lop3_and_or(ql[w], 0x00F000F0u, 0x64006400u);
          fa[w][1] = lop3_and_or(qh[w], 0x000F000Fu, 0x64006400u);
          fa[w][3] = lop3_and_or(qh[w], 0x00F000F0u, 0x64006400u);
          const uint32_t ql8 = ql[w] >> 8, qh8 = qh[w] >> 8;
          fa[w][4] = lop3_and_or(ql8, 0x000F000Fu, 0x64006400u);
          fa[w][6] = lop3_and_or(ql8, 0x00F000F0u, 0x64006400u);
          fa[w][5] = lop3_and_or(qh8, 0x000F000Fu, 0x64006400u);
          fa[w][7] = lop3_and_or(qh8, 0x00F000F0u, 0x64006400u);
        }
        if (G == 128) {
          // two independent chains of four MMAs (words 0,1 and words 2,3)
          float c0[MT][4], c1[MT][4];
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            mma_f16_16816_z(c0[m], fa[0][0], fa[0][1], fa[0][2], fa[0][3], xb[m][0].x, xb[m][0].y);
            mma_f16_16816_z(c1[m], fa[2][0], fa[2][1], fa[2][2], fa[2][3], xb[m][2].x, xb[m][2].y);
            mma_f16_16816(c0[m], fa[0][4], fa[0][5], fa[0][6], fa[0][7], xb[m][0].z, xb[m][0].w);
            mma_f16_16816(c1[m], fa[2][4], fa[2][5], fa[2][6], fa[2][7], xb[m][2].z, xb[m][2].w);
            mma_f16_16816(c0[m], fa[1][0], fa[1][1], fa[1][2], fa[1][3], xb[m][1].x, xb[m][1].y);
            mma_f16_16816(c1[m], fa[3][0], fa[3][1], fa[3][2], fa[3][3], xb[m][3].x, xb[m][3].y);
            mma_f16_16816(c0[m], fa[1][4], fa[1][5], fa[1][6], fa[1][7], xb[m][1].z, xb[m][1].w);
            mma_f16_16816(c1[m], fa[3][4], fa[3][5], fa[3][6], fa[3][7], xb[m][3].z, xb[m][3].w);
          }
          const __half2 h0 = *reinterpret_cast<const __half2*>(&su0[0]);
          const __half2 h1 = *reinterpret_cast<const __half2*>(&su1[0]);
          const float sc0 = __low2float(h0), z0 = __high2float(h0);
          const float sc1 = __low2float(h1), z1 = __high2float(h1);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            acc[m][0] = fmaf(sc0, (c0[m][0] + c1[m][0]) - fmaf(z0, sa[m][0].x, sa[m][0].y), acc[m][0]);
            acc[m][1] = fmaf(sc0, (c0[m][1] + c1[m][1]) - fmaf(z0, sb[m][0].x, sb[m][0].y), acc[m][1]);
            acc[m][2] = fmaf(sc1, (c0[m][2] + c1[m][2]) - fmaf(z1, sa[m][0].x, sa[m][0].y), acc[m][2]);
            acc[m][3] = fmaf(sc1, (c0[m][3] + c1[m][3]) - fmaf(z1, sb[m][0].x, sb[m][0].y), acc[m][3]);
          }
        } else {
#pragma unroll
          for (int q = 0; q < GPT; ++q) {
            const __half2 h0 = *reinterpret_cast<const __half2*>(&su0[q]);
            const __half2 h1 = *reinterpret_cast<const __half2*>(&su1[q]);
            const float sc0 = __low2float(h0), z0 = __high2float(h0);
            const float sc1 = __low2float(h1), z1 = __high2float(h1);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              float c[4];
              mma_f16_16816_z(c, fa[q][0], fa[q][1], fa[q][2], fa[q][3], xb[m][q].x, xb[m][q].y);
              mma_f16_16816(c, fa[q][4], fa[q][5], fa[q][6], fa[q][7], xb[m][q].z, xb[m][q].w);
              acc[m][0] = fmaf(sc0, c[0] - fmaf(z0, sa[m][q].x, sa[m][q].y), acc[m][0]);
              acc[m][1] = fmaf(sc0, c[1] - fmaf(z0, sb[m][q].x, sb[m][q].y), acc[m][1]);
              acc[m][2] = fmaf(sc1, c[2] - fmaf(z1, sa[m][q].x, sa[m][q].y), acc[m][2]);
              acc[m][3] = fmaf(sc1, c[3] - fmaf(z1, sb[m][q].x, sb[m][q].y), acc[m][3]);
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
            } else {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)tok * p.ldo + nt * 16 + g;
              float a = v_lo, b = v_hi;
              if (epi == EPI_RESIDUAL) {
                const __nv_bfloat16* rr = p.residual + (size_t)tok * p.ldo + nt * 16 + g;
                a += __bfloat162float(rr[0]); b += __bfloat162float(rr[8]);
              }
              o[0] = __float2bfloat16(a); o[8] = __float2bfloat16(b);
            }
          }
        }
      }
      if (epi == EPI_SILU_PACK && ((item & 15) == 15 || item == n_items - 1)) {
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
          float s_st, s_eff;
          const uint4 pk = actpack_chunk(v8, s_st, s_eff);
          actpack_group_reduce(s_st, s_eff, cpg);
          if (tok < p.M) {
            p.out_pack[((size_t)tok * I + col0) / 8 + ch] = pk;
            if ((ch % cpg) == 0)
              p.out_xs[(size_t)tok * (I / p.gout) + col0 / p.gout + ch / cpg] = make_float2(s_eff, 1024.f * s_st);
          }
        }
      }
    }
    ++item;
  }
}

template <int MT, int KIND>
static int launch_skinny(const SkinnyParams& p, int epi, int pdl, cudaStream_t st) {
  auto kernel = skinny_stream_kernel<MT, KIND>;
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
  int tpc = want > 0 ? want : (n_tiles + 295) / 296;
  if (tpc < 1) tpc = 1;
  if (epi == EPI_SILU_PACK) tpc = ((tpc + 15) / 16) * 16;
  return tpc;
}

template <int KIND>
static int dispatch_mt(const SkinnyParams& p, int epi, int pdl, cudaStream_t st) {
  const int mt = (p.M + 7) / 8;
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
  p.tiles_per_cta = pick_tiles_per_cta(p.n_tiles, epi, tiles_per_cta);
  return group == 128 ? dispatch_mt<KIND_W4_G128>(p, epi, pdl, st) : dispatch_mt<KIND_W4_G32>(p, epi, pdl, st);
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
