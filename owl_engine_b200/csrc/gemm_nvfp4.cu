// NVFP4 x NVFP4 GEMM on the block-scaled tensor-core path of sm_100a (tcgen05.mma kind::mxf4nvf4, block16).
//
//   owl_nvfp4_quant_rows : x bf16 / fp16 [T,K] -> e2m1 codes [T,K/2], e4m3 block scales in MMA atom order, one fp32 scale per row
//   owl_nvfp4_gemm       : C[T,N] = sx[t] * alpha * rs[n] * sum_k (xq[t,k] sfx[t,k/16]) (wq[n,k] sfw[n,k/16])     C bf16
//
// Both operands stay 4-bit all the way into shared memory: the codes are read as stored in the checkpoint ([rows][K/2] bytes,
// element 2i in the low nibble) by TMA with the 128-byte swizzle, 256 k per row and stage. The e4m3 block scales (one per 16
// k) are consumed by the tensor core itself; it reads them from tensor memory, where they must lie as "atoms": the scales of
// 128 rows x 4 blocks (64 k) are 512 bytes, row r / block b at byte (r % 32) * 16 + (r / 32) * 4 + b. Scale buffers are kept in
// global memory in that order, [row block of 128][k atom][512 bytes], padded with zeros to whole row blocks and to a multiple
// of 4 atoms along k (formats/nvfp4.py pack_sf_atoms for weights, owl_nvfp4_quant_rows for activations), so a stage's scales
// are one contiguous 2 KB run per operand that a bulk copy brings to shared memory and tcgen05.cp (32x128b.warpx4) moves on
// to tensor memory just ahead of the MMAs that use them.
//
// Tile 128 (tokens) x 128 (weight rows) x 256 (k). One persistent CTA per SM, 192 threads:
//   warp 0      producer: two TMA tile loads + two bulk copies of scales per stage, 5 stages of 36 KB
//   warp 1      one thread issues, per stage, 8 tcgen05.cp (scale atoms) and 4 tcgen05.mma (M128 N128 K64) into one of two
//               TMEM accumulators (2 x 128 columns; the scale atoms take 32 more columns), commit -> stage free
//   warps 2-5   epilogue of the previous tile while the next tile's MMAs run: tcgen05.ld -> scale -> bf16 -> global
// Every wait is bounded; on a timeout the CTA records an error code, the roles leave their loops, copies in flight are waited
// for (bounded) and TMEM is freed.
//
// Role in the reference: crates/kernels/cu/nvfp4/nvfp4_gemm.cu (CUTLASS block-scaled collective, 128 x 128 x 256 tile) and
// crates/kernels/cu/nvfp4/nvfp4_quant_act.cu; there the activation scale is one per tensor, here one per token row.
#include <cuda.h>
#include <cuda_fp8.h>
#include "common.cuh"
#include "actpack.cuh"

namespace owl {

__device__ int g_gemm_nvfp4_status = 0;

constexpr int NF_BM = 128, NF_BN = 128, NF_BKB = 128, NF_STAGES = 5;      // NF_BKB: code bytes per row and stage (256 k)
constexpr int NF_A_BYTES = NF_BM * NF_BKB, NF_B_BYTES = NF_BN * NF_BKB, NF_SF_BYTES = 2048;
constexpr int NF_STAGE_BYTES = NF_A_BYTES + NF_B_BYTES + 2 * NF_SF_BYTES;    // 36 KB
constexpr int NF_THREADS = 192;
constexpr int NF_SMEM = NF_STAGES * NF_STAGE_BYTES + 1024 + 256;
constexpr uint32_t NF_SFA_COL = 256, NF_SFB_COL = 272;                        // TMEM columns of the scale atoms

struct NfParams {
  __nv_bfloat16* out;
  const uint8_t* sfa;          // [m_tiles][KI][2048]
  const uint8_t* sfb;          // [n_tiles][KI][2048]
  const float* sx;             // [T] per-row activation scale
  const float* row_scale;      // [N] or null
  float alpha;
  int T, N, ldo, KI, m_tiles, n_tiles;
};
struct NfCtl {
  uint64_t full[NF_STAGES], empty[NF_STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ bool nf_wait(uint64_t* bar, uint32_t parity, NfCtl* c, int code) {
  const uint64_t t0 = global_ns();
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 15u) == 15u && wait_expired(t0)) break;
    if ((i & 255u) == 255u && c->abort_flag) return false;
  }
  c->abort_flag = 1;
  atomicCAS(&g_gemm_nvfp4_status, 0, code);
  return false;
}
// The producer's and the MMA issuer's waits: one thread each, polling with test_wait (a suspended thread's wake-up would
// add to every stage's round trip, which bounds this kernel).
__device__ __forceinline__ bool nf_spin(uint64_t* bar, uint32_t parity, NfCtl* c, int code) {
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
  atomicCAS(&g_gemm_nvfp4_status, 0, code);
  return false;
}
// plain (non-multicast) bulk copy global -> this CTA's shared memory; bytes and both addresses multiples of 16
__device__ __forceinline__ void nf_bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, the same 32 lanes repeated in all four lane quarters
__device__ __forceinline__ void nf_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void nf_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa,
                                       uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb) : "memory");
}
// Instruction descriptor of the block-scaled kinds: A and B e2m1 (code 1 of the 4-bit kind), both K-major, e4m3 scales
// (bit 23 = 0), scale ids 0, dense K = 64 (bit 31 = 0); N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __host__ constexpr uint32_t nf_idesc(int M, int N) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__global__ void __launch_bounds__(NF_THREADS, 1) gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                   const __grid_constant__ CUtensorMap tmB, NfParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  NfCtl* ctl = reinterpret_cast<NfCtl*>(base + NF_STAGES * NF_STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KI = p.KI;
  const int n_tiles_total = p.m_tiles * p.n_tiles;          // tile = m + m_tiles * n: CTAs that run together share a weight tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < NF_STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->acc_full[a], 1); mbar_init(&ctl->acc_empty[a], 4); }
    ctl->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
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
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x) {
        const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
        const uint8_t* sfa = p.sfa + (size_t)mt * KI * NF_SF_BYTES;
        const uint8_t* sfb = p.sfb + (size_t)nt * KI * NF_SF_BYTES;
        for (int k = 0; k < KI; ++k, ++it) {
          const int s = it % NF_STAGES;
          if (!nf_spin(&ctl->empty[s], (((uint32_t)(it / NF_STAGES)) & 1u) ^ 1u, ctl, OWL_ERR_WAIT_MMA)) goto prod_done;
          mbar_expect_tx(&ctl->full[s], NF_STAGE_BYTES);
          uint8_t* st = base + (size_t)s * NF_STAGE_BYTES;
          tma_load_2d(st, &tmA, &ctl->full[s], k * NF_BKB, mt * NF_BM);
          tma_load_2d(st + NF_A_BYTES, &tmB, &ctl->full[s], k * NF_BKB, nt * NF_BN);
          nf_bulk_g2s(st + NF_A_BYTES + NF_B_BYTES, sfa + (size_t)k * NF_SF_BYTES, NF_SF_BYTES, &ctl->full[s]);
          nf_bulk_g2s(st + NF_A_BYTES + NF_B_BYTES + NF_SF_BYTES, sfb + (size_t)k * NF_SF_BYTES, NF_SF_BYTES, &ctl->full[s]);
        }
      }
    prod_done:
      if (ctl->abort_flag) {
        for (int i = max(0, it - NF_STAGES); i < it; ++i)
          for (uint32_t n = 0; n < 256u; ++n)
            if (mbar_try_wait(&ctl->full[i % NF_STAGES], ((uint32_t)(i / NF_STAGES)) & 1u)) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = nf_idesc(NF_BM, NF_BN);
      int it = 0, lt = 0;
      for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++lt) {
        const int ab = lt & 1;
        if (!nf_spin(&ctl->acc_empty[ab], (((uint32_t)(lt >> 1)) & 1u) ^ 1u, ctl, OWL_ERR_WAIT_EPI)) break;
        tc_fence_after();
        const uint32_t td = tmem + ab * NF_BN;
        bool ok = true;
        for (int k = 0; k < KI; ++k, ++it) {
          const int s = it % NF_STAGES;
          if (!nf_spin(&ctl->full[s], ((uint32_t)(it / NF_STAGES)) & 1u, ctl, OWL_ERR_WAIT_TMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(base + (size_t)s * NF_STAGE_BYTES);
          const uint32_t ssfa = sa + NF_A_BYTES + NF_B_BYTES, ssfb = ssfa + NF_SF_BYTES;
#pragma unroll
          for (int a = 0; a < 4; ++a) {                      // 4 atoms (64 k each) per operand
            nf_cp_sf(tmem + NF_SFA_COL + a * 4, umma_desc_k_noswz(ssfa + a * 512, 16, 128));
            nf_cp_sf(tmem + NF_SFB_COL + a * 4, umma_desc_k_noswz(ssfb + a * 512, 16, 128));
          }
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + NF_A_BYTES);
#pragma unroll
          for (int a = 0; a < 4; ++a)                        // 64 k = 32 bytes of the 128-byte row per instruction
            nf_mma(td, da + (uint64_t)(a * 2), db + (uint64_t)(a * 2), idesc, tmem + NF_SFA_COL + a * 4, tmem + NF_SFB_COL + a * 4,
                   (k > 0 || a > 0) ? 1u : 0u);
          tc_commit(&ctl->empty[s]);
        }
        if (!ok) break;
        tc_commit(&ctl->acc_full[ab]);
      }
    }
  } else {
    const int q4 = warp & 3;                                 // TMEM lane quarter of this warp
    int lt = 0;
    for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++lt) {
      const int ab = lt & 1;
      const int m0 = (tile % p.m_tiles) * NF_BM, n0 = (tile / p.m_tiles) * NF_BN;
      if (!nf_wait(&ctl->acc_full[ab], ((uint32_t)(lt >> 1)) & 1u, ctl, OWL_ERR_WAIT_MMA)) break;
      tc_fence_after();
      const int row = m0 + q4 * 32 + lane;
      const float sr = row < p.T ? p.sx[row] * p.alpha : 0.f;
      __nv_bfloat16* obase = p.out + (size_t)row * p.ldo;
#pragma unroll 1
      for (int c = 0; c < NF_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(ab * NF_BN + c * 32), r);
        tc_wait_ld();
        if (row < p.T) {
          const int cb = n0 + c * 32;
#pragma unroll
          for (int v = 0; v < 32; ++v) {
            const float cs = p.row_scale ? (cb + v < p.N ? p.row_scale[cb + v] : 0.f) : 1.f;
            r[v] = __float_as_uint(__uint_as_float(r[v]) * sr * cs);
          }
          __nv_bfloat16* o = obase + cb;
          if (cb + 32 <= p.N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 pk;
              pk.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              pk.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              pk.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              pk.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              *reinterpret_cast<uint4*>(o + v * 8) = pk;
            }
          } else {
            for (int v = 0; v < 32; ++v)
              if (cb + v < p.N) o[v] = __float2bfloat16(__uint_as_float(r[v]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[ab]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

__device__ __forceinline__ uint32_t nf_to_e2m1(float x) {           // round to the nearest representable magnitude
  const float a = fabsf(x);
  const uint32_t mag = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
  return mag | (x < 0.f ? 8u : 0u);
}

// grid (T), 256 threads: one token row per CTA. Pass 1 finds the row's largest magnitude (row scale = amax / (6 * 448), so
// the largest block scale is representable in e4m3), pass 2 re-reads the row (L1/L2), writes codes and block scales.
__device__ __forceinline__ void nf_load16(const uint4* xp, bool f16, float* v) {
  const uint4 a = xp[0], b = xp[1];
  if (f16) {
    const __half2* h = reinterpret_cast<const __half2*>(&a);
    const __half2* g = reinterpret_cast<const __half2*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 u = __half22float2(h[i]), w = __half22float2(g[i]);
      v[2 * i] = u.x; v[2 * i + 1] = u.y; v[8 + 2 * i] = w.x; v[9 + 2 * i] = w.y;
    }
  } else {
    unpack_bf16x8(a, v);
    unpack_bf16x8(b, v + 8);
  }
}

__global__ void __launch_bounds__(256) nvfp4_quant_rows_kernel(const uint16_t* __restrict__ x, int ldx, bool f16, uint8_t* codes,
                                                               uint8_t* sf, float* sx, int K, int KI) {
  __shared__ float red[8];
  const int row = blockIdx.x, nb = K >> 4;
  const uint16_t* xr = x + (size_t)row * ldx;
  float amax = 0.f;
  for (int b = threadIdx.x; b < nb; b += 256) {
    float v[16];
    nf_load16(reinterpret_cast<const uint4*>(xr + b * 16), f16, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float gs = fmaxf(amax, 1e-12f) / (6.f * 448.f);
  if (threadIdx.x == 0) sx[row] = gs;
  uint8_t* sfrow = sf + (size_t)(row >> 7) * KI * NF_SF_BYTES + (row & 31) * 16 + ((row >> 5) & 3) * 4;
  for (int b = threadIdx.x; b < nb; b += 256) {
    float v[16];
    nf_load16(reinterpret_cast<const uint4*>(xr + b * 16), f16, v);
    float bm = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) bm = fmaxf(bm, fabsf(v[i]));
    const float bs = fminf(bm / 6.f / gs, 448.f);
    const __nv_fp8_e4m3 s8(bs);
    sfrow[(size_t)(b >> 2) * 512 + (b & 3)] = s8.__x;
    const float inv = 1.f / (fmaxf((float)s8, 0.001953125f) * gs);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo |= nf_to_e2m1(v[i] * inv) << (4 * i);
      hi |= nf_to_e2m1(v[8 + i] * inv) << (4 * i);
    }
    *reinterpret_cast<uint2*>(codes + (size_t)row * (K >> 1) + b * 8) = make_uint2(lo, hi);
  }
}

typedef CUresult (*NfEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static NfEncodeFn nf_encode() {
  static NfEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<NfEncodeFn>(p);
  }
  return fn;
}
// codes: [rows][ld bytes], K / 2 bytes valid per row; box 128 bytes x 128 rows, bytes past the row end read as zero codes
static int nf_map(CUtensorMap* m, const void* ptr, int rows, int K, int ld) {
  NfEncodeFn enc = nf_encode();
  if (!enc) return OWL_ERR_LAUNCH * 1000 - 1;
  cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {(cuuint32_t)NF_BKB, (cuuint32_t)NF_BM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OWL_OK : OWL_ERR_LAUNCH * 1000 - (int)r;
}

}  // namespace owl
using namespace owl;

// x bf16 (x_f16 = 0) or fp16 (1) [T][ldx] -> codes u8 [T][K/2], sf (ceil(T / 128) * ceil(K / 256) * 2048 bytes, zero-filled once by the caller: the k padding is
// never written), sx fp32 [T]. K multiple of 64.
OWL_API int owl_nvfp4_quant_rows(const void* x, int ldx, int x_f16, void* codes, void* sf, void* sx, int T, int K,
                                 cudaStream_t st) {
  if (T < 1 || K < 64 || (K & 63) || (ldx & 7) || !x || !codes || !sf || !sx || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(codes) & 7))
    return OWL_ERR_BAD_ARG;
  nvfp4_quant_rows_kernel<<<T, 256, 0, st>>>((const uint16_t*)x, ldx, x_f16 != 0, (uint8_t*)codes, (uint8_t*)sf, (float*)sx, K,
                                             (K + 255) / 256);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// xcodes [T][K/2], xsf atoms, sx [T]; wcodes [N][K/2], wsf atoms; out bf16 [T][ldo] = sx[t] alpha row_scale[n] (xq . wq^T).
// K multiple of 64; row_scale may be null.
OWL_API int owl_nvfp4_gemm(const void* xcodes, const void* xsf, const void* sx, const void* wcodes, const void* wsf, float alpha,
                           const void* row_scale, void* out, int T, int N, int K, int ldo, cudaStream_t st) {
  if (T < 1 || N < 1 || K < 64 || (K & 63) || (ldo & 7) || !xcodes || !xsf || !sx || !wcodes || !wsf || !out ||
      (reinterpret_cast<uintptr_t>(xcodes) & 15) || (reinterpret_cast<uintptr_t>(wcodes) & 15) ||
      (reinterpret_cast<uintptr_t>(xsf) & 15) || (reinterpret_cast<uintptr_t>(wsf) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return OWL_ERR_BAD_ARG;
  CUtensorMap a, b;
  int r = nf_map(&a, xcodes, T, K, K / 2);
  if (r) return r;
  r = nf_map(&b, wcodes, N, K, K / 2);
  if (r) return r;
  NfParams p = {};
  p.out = (__nv_bfloat16*)out; p.sfa = (const uint8_t*)xsf; p.sfb = (const uint8_t*)wsf; p.sx = (const float*)sx;
  p.row_scale = (const float*)row_scale; p.alpha = alpha; p.T = T; p.N = N; p.ldo = ldo; p.KI = (K + 255) / 256;
  p.m_tiles = (T + NF_BM - 1) / NF_BM; p.n_tiles = (N + NF_BN - 1) / NF_BN;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(gemm_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, NF_SMEM) != cudaSuccess) {
      sms = 0;
      return OWL_ERR_LAUNCH * 1000;
    }
  }
  const int tiles = p.m_tiles * p.n_tiles;
  gemm_nvfp4_kernel<<<tiles < sms ? tiles : sms, NF_THREADS, NF_SMEM, st>>>(a, b, p);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

OWL_API int owl_gemm_nvfp4_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_nvfp4_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_gemm_nvfp4_status, &zero, sizeof(int));
  return v;
}
