// tcgen05 / TMEM GEMMs for prefill-shape work (sm_100a).
//
//   owl_w4a16_gemm_tc : C[T,N] = X[T,K] . dequant(W4)[N,K]^T   X fp16, C bf16, fp32 accumulate in TMEM
//   owl_f16_gemm_tc   : C[T,N] = X[T,K] . W[N,K]^T             X, W both fp16 or both bf16 (dense)
//
// One CTA computes a 128 (tokens) x 128 (weight rows) tile; K advances in 64-element stages:
//   warp 0      TMA producer: the X tile [128 x 64] (and the dense W tile) arrives in shared memory
//               in the 128-byte-swizzled K-major layout that the MMA descriptors describe
//   warp 1      allocates TMEM, then one thread issues tcgen05.mma (M128 N128 K16 x 4 per stage) and
//               tcgen05.commit -> the stage's "empty" barrier; a last commit signals the epilogue
//   warps 2-5   W4 path: stream the int4 records of 8 row tiles, dequantise ((q - z) * s in exact
//               fp16: lop3 bias trick, one hsub2 + one hmul2 per pair) and write the swizzled
//               B tile; afterwards they are the epilogue: tcgen05.ld 32x32b -> bf16 -> global
// Two CTAs fit per SM (3 stages x 32 KB, 128 TMEM columns each) so one CTA's epilogue overlaps the
// other's main loop.
//
// Every mbarrier wait is bounded; on a timeout the CTA records an error code, all roles leave
// their loops, outstanding copies are waited for (bounded) and TMEM is freed before exit.
//
// Role in the reference: the Marlin / cuBLAS prefill GEMMs (crates/kernels/cu/marlin/*,
// crates/kernels/src/family/cublas.rs); the reference has no tcgen05 path.
#include <cuda.h>
#include "common.cuh"
#include "records.cuh"

namespace owl {

__device__ int g_gemm_status = 0;

constexpr int GT_BM = 128, GT_BN = 128, GT_BK = 64, GT_STAGES = 3;
constexpr int GT_TILE_BYTES = GT_BM * GT_BK * 2;   // 16 KB per operand per stage
constexpr int GT_THREADS = 192;
constexpr int GT_SMEM = GT_STAGES * 2 * GT_TILE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

struct GemmTcParams {
  const uint8_t* wrec;   // W4 records or nullptr for the dense path
  __nv_bfloat16* out;
  int T, N, K, ldo;
  int group;             // 32 / 128
  int layout;            // record stream layout: 0 slice-major, 1 block-major
  int fmt;               // dense path: 0 fp16, 1 bf16 operands
};

struct GemmSmem {
  uint64_t full_a[GT_STAGES], full_b[GT_STAGES], empty[GT_STAGES], acc_full;
  uint32_t tmem_base;
  volatile int abort_flag;
};

// Bounded wait that also leaves when another role aborted.
__device__ __forceinline__ bool gt_wait(uint64_t* bar, uint32_t parity, GemmSmem* sm, int code) {
  const uint64_t t0 = global_ns();
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 15u) == 15u && wait_expired(t0)) break;
    if ((i & 255u) == 255u && sm->abort_flag) return false;
  }
  sm->abort_flag = 1;
  atomicCAS(&g_gemm_status, 0, code);
  return false;
}

template <bool DEQ>
__global__ void __launch_bounds__(GT_THREADS, 2) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                const __grid_constant__ CUtensorMap tmB,
                                                                GemmTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;
  uint8_t* sB = base + GT_STAGES * GT_TILE_BYTES;
  GemmSmem* sm = reinterpret_cast<GemmSmem*>(base + GT_STAGES * 2 * GT_TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * GT_BN, m0 = blockIdx.y * GT_BM;
  const int KI = p.K / GT_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GT_STAGES; ++s) {
      mbar_init(&sm->full_a[s], 1);
      mbar_init(&sm->full_b[s], DEQ ? 4 : 1);
      mbar_init(&sm->empty[s], 1);
    }
    mbar_init(&sm->acc_full, 1);
    sm->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA);
    if (!DEQ) prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&sm->tmem_base, GT_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = sm->tmem_base;

  if (warp == 0) {
    // ------------------------------- TMA producer ---------------------------------------------
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < KI; ++it) {
        const int s = it % GT_STAGES;
        const uint32_t ph = (uint32_t)(it / GT_STAGES) & 1u;
        if (!gt_wait(&sm->empty[s], ph ^ 1u, sm, OWL_ERR_WAIT_MMA)) break;
        if (DEQ) {
          mbar_expect_tx(&sm->full_a[s], GT_TILE_BYTES);
          tma_load_2d(sA + s * GT_TILE_BYTES, &tmA, &sm->full_a[s], it * GT_BK, m0);
        } else {
          mbar_expect_tx(&sm->full_a[s], 2 * GT_TILE_BYTES);
          tma_load_2d(sA + s * GT_TILE_BYTES, &tmA, &sm->full_a[s], it * GT_BK, m0);
          tma_load_2d(sB + s * GT_TILE_BYTES, &tmB, &sm->full_a[s], it * GT_BK, n0);
        }
        issued = it + 1;
      }
      if (sm->abort_flag) {
        // wait (bounded) for copies that were issued but may never be consumed
        for (int it = max(0, issued - GT_STAGES); it < issued; ++it) {
          const int s = it % GT_STAGES;
          const uint32_t ph = (uint32_t)(it / GT_STAGES) & 1u;
          for (uint32_t i = 0; i < (1u << 20); ++i)
            if (mbar_try_wait(&sm->full_a[s], ph)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(GT_BM, GT_BN, DEQ ? 0 : p.fmt);
      bool ok = true;
      for (int it = 0; it < KI && ok; ++it) {
        const int s = it % GT_STAGES;
        const uint32_t ph = (uint32_t)(it / GT_STAGES) & 1u;
        ok = gt_wait(&sm->full_a[s], ph, sm, OWL_ERR_WAIT_TMA);
        if (ok && DEQ) ok = gt_wait(&sm->full_b[s], ph, sm, OWL_ERR_WAIT_EPI);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = umma_desc_k128(smem_u32(sA + s * GT_TILE_BYTES));
        const uint64_t db = umma_desc_k128(smem_u32(sB + s * GT_TILE_BYTES));
#pragma unroll
        for (int k4 = 0; k4 < GT_BK / 16; ++k4)
          tc_mma_f16(tmem_d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (it > 0 || k4 > 0) ? 1u : 0u);
        tc_commit(&sm->empty[s]);
      }
      if (ok) tc_commit(&sm->acc_full);
    }
  } else {
    // ------------------------------- dequant producers, then epilogue -------------------------
    const int wq = warp - 2;                 // 0..3
    bool ok = true;
    if (DEQ) {
      const int g = lane >> 2, t = lane & 3;
      const int GPT = 128 / p.group;
      const int REC = 1024 + 64 * GPT;
      const int NT = p.N / 16, KT = p.K / 128;
      const __half2 k1024 = __floats2half2_rn(1024.f, 1024.f), k64 = __floats2half2_rn(64.f, 64.f);
      const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
      uint4 cur[4], nxt[4];                  // [jt*2 + half]
      uint32_t csz[4][4], nsz[4][4];         // (scale, zero) half2 per [jt*2+half][group of record]
      auto load_rec = [&](int kt, uint4* q, uint32_t (*sz)[4]) {
#pragma unroll
        for (int jt = 0; jt < 2; ++jt) {
          const int nt = n0 / 16 + wq * 2 + jt;
          if (nt < NT && kt < KT) {
            const uint8_t* rec = p.wrec + record_offset_any(p.layout, NT, KT, nt, kt) * (size_t)REC;
            q[jt * 2 + 0] = ldg_stream(reinterpret_cast<const uint4*>(rec) + lane);
            q[jt * 2 + 1] = ldg_stream(reinterpret_cast<const uint4*>(rec) + 32 + lane);
            const uint32_t* szr = reinterpret_cast<const uint32_t*>(rec + 1024);
            for (int qg = 0; qg < GPT; ++qg) {
              sz[jt * 2 + 0][qg] = __ldg(szr + qg * 16 + g);
              sz[jt * 2 + 1][qg] = __ldg(szr + qg * 16 + 8 + g);
            }
          } else {
            q[jt * 2 + 0] = q[jt * 2 + 1] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
            for (int qg = 0; qg < 4; ++qg) sz[jt * 2 + 0][qg] = sz[jt * 2 + 1][qg] = 0x48000000u;  // s = 0, z = 8
          }
        }
      };
      load_rec(0, cur, csz);
      for (int it = 0; it < KI; ++it) {
        const int s = it % GT_STAGES;
        const uint32_t ph = (uint32_t)(it / GT_STAGES) & 1u;
        const int sp = it & 1;
        if (sp == 0) load_rec(it / 2 + 1, nxt, nsz);   // prefetch the next 128-k record
        if (!gt_wait(&sm->empty[s], ph ^ 1u, sm, OWL_ERR_WAIT_MMA)) { ok = false; break; }
        uint8_t* tileB = sB + s * GT_TILE_BYTES;
#pragma unroll
        for (int jh = 0; jh < 4; ++jh) {
          const int r8 = (wq * 2 + (jh >> 1)) * 2 + (jh & 1);     // 8-row group index inside the 128-row tile
          const uint32_t qw[4] = {cur[jh].x, cur[jh].y, cur[jh].z, cur[jh].w};
#pragma unroll
          for (int wl = 0; wl < 2; ++wl) {
            const int w = sp * 2 + wl;
            const uint32_t szv = (p.group == 32) ? (sp ? (wl ? csz[jh][3] : csz[jh][2]) : (wl ? csz[jh][1] : csz[jh][0]))
                                                 : csz[jh][0];
            const __half2 szh = *reinterpret_cast<const __half2*>(&szv);
            const __half sc = __low2half(szh), z = __high2half(szh);
            const __half2 s2 = __half2half2(sc);
            const __half2 z_lo = __hadd2(k1024, __half2half2(z));       // 1024 + z
            const __half2 z_hi = __hneg2(__hadd2(k64, __half2half2(z))); // -(64 + z)
            const uint32_t q = qw[w], q8 = q >> 8;
            uint32_t t0 = (q & 0x000F000Fu) | 0x64006400u, t1 = (q & 0x00F000F0u) | 0x64006400u;
            uint32_t t2 = (q8 & 0x000F000Fu) | 0x64006400u, t3 = (q8 & 0x00F000F0u) | 0x64006400u;
            // low nibbles: (1024 + q) - (1024 + z); high nibbles: (1024 + 16 q) / 16 - (64 + z); both exact
            __half2 h0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t0), z_lo), s2);
            __half2 h1 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&t1), k16th, z_hi), s2);
            __half2 h2 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t2), z_lo), s2);
            __half2 h3 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&t3), k16th, z_hi), s2);
            const int c = wl * 4 + t;        // 16-byte chunk inside the 128-byte row
            uint4 o;
            o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
            o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(tileB + r8 * 1024 + g * 128 + ((c ^ g) << 4)) = o;
          }
        }
        fence_async_smem();                  // generic-proxy writes -> visible to the MMA (async proxy)
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->full_b[s]);
        if (sp == 1) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            cur[i] = nxt[i];
#pragma unroll
            for (int qg = 0; qg < 4; ++qg) csz[i][qg] = nsz[i][qg];
          }
        }
      }
    }
    // epilogue: warp reads its TMEM lane quarter (warp id % 4), one token row per thread
    if (ok) ok = gt_wait(&sm->acc_full, 0, sm, OWL_ERR_WAIT_MMA);
    if (ok) {
      tc_fence_after();
      const int q4 = warp & 3;
      const int row = m0 + q4 * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < GT_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_d + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(c * 32), r);
        tc_wait_ld();
        if (row < p.T) {
          __nv_bfloat16* o = p.out + (size_t)row * p.ldo + n0 + c * 32;
          if (n0 + c * 32 + 32 <= p.N) {
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
              if (n0 + c * 32 + v < p.N) o[v] = __float2bfloat16(__uint_as_float(r[v]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, GT_BN);
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}
// 2-D K-major map over a [rows][K] 16-bit matrix: box 64 x 128, 128-byte swizzle, zero fill.
static int make_map(CUtensorMap* m, const void* ptr, int rows, int K, int ld, int fmt) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return OWL_ERR_LAUNCH * 1000 - 1;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {GT_BK, GT_BM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, fmt ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OWL_OK : OWL_ERR_LAUNCH * 1000 - (int)r;
}

template <bool DEQ>
static int launch_gemm(const CUtensorMap& a, const CUtensorMap& b, const GemmTcParams& p, cudaStream_t st) {
  auto kernel = gemm_tc_kernel<DEQ>;
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM) != cudaSuccess)
      return OWL_ERR_LAUNCH * 1000;
    attr_done = true;
  }
  dim3 grid((p.N + GT_BN - 1) / GT_BN, (p.T + GT_BM - 1) / GT_BM);
  kernel<<<grid, GT_THREADS, GT_SMEM, st>>>(a, b, p);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

}  // namespace owl
using namespace owl;

// x: fp16 [T][ldx] (ldx multiple of 8, base 16-byte aligned); out: bf16 [T][ldo].
OWL_API int owl_w4a16_gemm_tc(const void* x, int ldx, const void* records, void* out, int T, int N, int K, int ldo,
                              int group, int layout, cudaStream_t st) {
  if (T < 1 || (N & 15) || (K & 127) || (ldx & 7) || (ldo & 7) || (group != 32 && group != 128) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return OWL_ERR_BAD_ARG;
  CUtensorMap a;
  int r = make_map(&a, x, T, K, ldx, 0);
  if (r) return r;
  GemmTcParams p = {};
  p.wrec = (const uint8_t*)records; p.out = (__nv_bfloat16*)out; p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.group = group; p.layout = layout;
  return launch_gemm<true>(a, a, p, st);
}

// x: [T][ldx], w: [N][ldw], both fp16 (fmt 0) or both bf16 (fmt 1); out bf16 [T][ldo].
OWL_API int owl_f16_gemm_tc(const void* x, int ldx, const void* w, int ldw, void* out, int T, int N, int K, int ldo,
                            int fmt, cudaStream_t st) {
  if (T < 1 || N < 1 || (K & 63) || (ldx & 7) || (ldw & 7) || (ldo & 7) || (fmt != 0 && fmt != 1) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return OWL_ERR_BAD_ARG;
  CUtensorMap a, b;
  int r = make_map(&a, x, T, K, ldx, fmt);
  if (r) return r;
  r = make_map(&b, w, N, K, ldw, fmt);
  if (r) return r;
  GemmTcParams p = {};
  p.out = (__nv_bfloat16*)out; p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.fmt = fmt;
  return launch_gemm<false>(a, b, p, st);
}

OWL_API int owl_gemm_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
  return v;
}
