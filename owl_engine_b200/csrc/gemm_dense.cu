// Dense 16-bit GEMM for long prefill chunks on tcgen05 (sm_100a), persistent and epilogue-overlapped.
//
//   owl_f16_gemm_persist : C[T,N] = X[T,K] . W[N,K]^T     X, W both fp16 or both bf16, C bf16, fp32 accumulate
//   owl_e4m3_gemm        : C[T,N] = (sx[t] sw[n]) Xq[T,K] . Wq[N,K]^T   both e4m3 with per-row fp32 scales (kind::f8f6f4,
//                          twice the 16-bit rate): the tensor-core arm of W4A8 -- int4 weights dequantised once to e4m3
//                          rows, activations quantised per token (owl_quant_e4m3_rows)
//
// Tile 128 (tokens) x 256 (weight rows) x 64 (k): with a 128 x 128 tile one MMA step reads as many shared-memory
// bytes per cycle as the SM can deliver, so the tensor pipe idles half of the time; 256 weight rows per tile
// halve the operand bytes per flop. One CTA per SM walks the tiles (weight-tile major, so the CTAs that run
// together share a weight tile through L2 and the weight matrix is read from HBM once):
//   warp 0      TMA producer: X tile [128 x 64] and W tile [256 x 64] per stage, 128-byte swizzle, 4 stages
//   warp 1      MMA issuer: 4 x tcgen05.mma (M128 N256 K16) per stage into one of two TMEM accumulators
//               (2 x 256 columns), commit -> stage free; after the last stage of a tile commit -> accumulator full
//   warps 2-5   epilogue of the previous tile while the next tile's MMAs run: tcgen05.ld 32 columns at a
//               time -> bf16 -> global, then accumulator free
// Tensor-parallel forms of the same kernel (one process per GPU, peer-mapped symmetric memory):
//   owl_f16_gemm_ag : column-parallel GEMM whose activation rows are produced by other ranks (all-gather by
//                     peer stores into THIS GPU's memory). The producer warp waits, per 128-row tile, for the
//                     owner rank's sequence flag before it issues the tile's first TMA load, so the GEMM
//                     starts on the rows that have arrived while the rest are still in flight.
//   owl_f16_gemm_rs : row-parallel GEMM whose epilogue is the reduce-scatter: each 128-row tile of partial
//                     sums is written from TMEM straight into the slot [source rank] of the rank that owns
//                     the tile (plain peer stores over NVLink), and the last weight-tile of a row tile
//                     publishes a sequence flag there. The owner sums the slots in rank order (comm.cu).
// Row tile j is owned by rank j % world and is its local tile j / world. TMA never reads peer memory here.
//
// Every mbarrier wait is bounded; on a timeout the CTA records an error code, the roles leave their loops,
// copies in flight are waited for (bounded) and TMEM is freed.
//
// Role in the reference: the cuBLAS GEMMs of the dequant -> GEMM prefill arm (crates/kernels/src/family/cublas.rs).
#include <cuda.h>
#include "common.cuh"

namespace owl {

__device__ int g_gemm_dense_status = 0;

constexpr int GD_BM = 128, GD_BN = 256, GD_BK = 64, GD_STAGES = 4;
constexpr int GD_A_BYTES = GD_BM * GD_BK * 2, GD_B_BYTES = GD_BN * GD_BK * 2;
constexpr int GD_STAGE_BYTES = GD_A_BYTES + GD_B_BYTES;          // 48 KB
constexpr int GD_THREADS = 192;
constexpr int GD_SMEM = GD_STAGES * GD_STAGE_BYTES + 1024 + 256;

struct GdParams {
  __nv_bfloat16* out;
  int T, N, K, ldo, fmt;
  int m_tiles, n_tiles;
  // tensor-parallel forms
  int rank, world, max_local;        // max_local: row tiles a rank can own (slot and flag table extent)
  const uint32_t* ag_flags;          // local [world][max_local]: sequence flags of arrived activation row tiles
  uint32_t ag_seq, rs_seq, spin_limit;
  __nv_bfloat16* rs_dst[8];          // each rank's slot buffer [world][max_local * 128][ldo]
  uint32_t* rs_flag[8];              // each rank's flag table [world][max_local]
  int* rs_done;                      // local [m_tiles]: weight tiles finished per row tile
  const float* a_scale;              // e4m3 form: per-token and per-weight-row scales
  const float* b_scale;
  int out_f16;                       // direct epilogue writes fp16 instead of bf16 (attention scores); never split-k
  int ksplit;                        // > 1: the k range is cut in ksplit parts, fp32 partial tiles go to `partial`
  float* partial;                    // [ksplit][T][ldp]
  int ldp;
};
struct GdCtl {
  uint64_t full[GD_STAGES], empty[GD_STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ bool gd_wait(uint64_t* bar, uint32_t parity, GdCtl* c, int code) {
  const uint64_t t0 = global_ns();
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 15u) == 15u && wait_expired(t0)) break;
    if ((i & 255u) == 255u && c->abort_flag) return false;
  }
  c->abort_flag = 1;
  atomicCAS(&g_gemm_dense_status, 0, code);
  return false;
}

// The producer's and the MMA issuer's waits: one thread each, polling with test_wait (a suspended thread's wake-up adds to
// every stage's round trip).
__device__ __forceinline__ bool gd_spin(uint64_t* bar, uint32_t parity, GdCtl* c, int code) {
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
  atomicCAS(&g_gemm_dense_status, 0, code);
  return false;
}

__device__ __forceinline__ void gd_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t gd_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <bool AG, bool RS, bool F8>
__global__ void __launch_bounds__(GD_THREADS, 1) gemm_dense_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                   const __grid_constant__ CUtensorMap tmB, GdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  GdCtl* ctl = reinterpret_cast<GdCtl*>(base + GD_STAGES * GD_STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int BKE = F8 ? 2 * GD_BK : GD_BK;           // k elements per stage (128 bytes per row either way)
  const int KI = p.K / BKE;
  const int KS = p.ksplit > 1 ? p.ksplit : 1;
  const int n_tiles_total = p.m_tiles * p.n_tiles * KS;     // tile index = (m + m_tiles * n) * KS + k part

  if (threadIdx.x == 0) {
    for (int s = 0; s < GD_STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
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
      int it = 0;                                           // stage counter across tiles
      for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x) {
        const int mn = tile / KS, ks = tile % KS;
        const int m0 = (mn % p.m_tiles) * GD_BM, n0 = (mn / p.m_tiles) * GD_BN;
        const int kb = ks * KI / KS, ke = (ks + 1) * KI / KS;
        if (AG) {
          // the rows of this tile are written by their owner rank; its flag says they have landed
          const int j = mn % p.m_tiles;
          const uint32_t* f = p.ag_flags + (j % p.world) * p.max_local + j / p.world;
          bool got = false;
          for (uint32_t i = 0; i < p.spin_limit; ++i) {
            if ((int)(gd_ld_acquire_sys(f) - p.ag_seq) >= 0) { got = true; break; }
            if (i > 16) __nanosleep(100);
            if ((i & 255u) == 255u && ctl->abort_flag) break;
          }
          if (!got) {
            ctl->abort_flag = 1;
            atomicCAS(&g_gemm_dense_status, 0, OWL_ERR_WAIT_PEER);
            goto prod_done;
          }
          asm volatile("fence.proxy.async;" ::: "memory");   // peer-written rows are read by the copy engine next
        }
        for (int k = kb; k < ke; ++k, ++it) {
          const int s = it % GD_STAGES;
          if (!gd_spin(&ctl->empty[s], (((uint32_t)(it / GD_STAGES)) & 1u) ^ 1u, ctl, OWL_ERR_WAIT_MMA)) goto prod_done;
          mbar_expect_tx(&ctl->full[s], GD_STAGE_BYTES);
          uint8_t* st = base + (size_t)s * GD_STAGE_BYTES;
          tma_load_2d(st, &tmA, &ctl->full[s], k * BKE, m0);
          tma_load_2d(st + GD_A_BYTES, &tmB, &ctl->full[s], k * BKE, n0);
        }
      }
    prod_done:
      if (ctl->abort_flag) {
        for (int i = max(0, it - GD_STAGES); i < it; ++i)
          for (uint32_t n = 0; n < 256u; ++n)
            if (mbar_try_wait(&ctl->full[i % GD_STAGES], ((uint32_t)(i / GD_STAGES)) & 1u)) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = F8 ? umma_idesc_e4m3(GD_BM, GD_BN) : umma_idesc_f16(GD_BM, GD_BN, p.fmt);
      int it = 0, lt = 0;                                   // stage counter, local tile counter
      for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++lt) {
        const int ab = lt & 1;
        if (!gd_spin(&ctl->acc_empty[ab], (((uint32_t)(lt >> 1)) & 1u) ^ 1u, ctl, OWL_ERR_WAIT_EPI)) break;
        tc_fence_after();
        const uint32_t td = tmem + ab * GD_BN;
        bool ok = true;
        const int kb = (tile % KS) * KI / KS, ke = (tile % KS + 1) * KI / KS;
        for (int k = kb; k < ke; ++k, ++it) {
          const int s = it % GD_STAGES;
          if (!gd_spin(&ctl->full[s], ((uint32_t)(it / GD_STAGES)) & 1u, ctl, OWL_ERR_WAIT_TMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(base + (size_t)s * GD_STAGE_BYTES);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + GD_A_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < GD_BK / 16; ++k4) {       // 32 bytes of k per instruction in both forms
            if (F8) tc_mma_f8(td, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (k > kb || k4 > 0) ? 1u : 0u);
            else tc_mma_f16(td, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (k > kb || k4 > 0) ? 1u : 0u);
          }
          tc_commit(&ctl->empty[s]);
        }
        if (!ok) break;
        tc_commit(&ctl->acc_full[ab]);
      }
    }
  } else {
    const int q4 = warp & 3;                                // TMEM lane quarter of this warp
    int lt = 0;
    for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++lt) {
      const int ab = lt & 1;
      const int mn = tile / KS;
      const int m0 = (mn % p.m_tiles) * GD_BM, n0 = (mn / p.m_tiles) * GD_BN;
      if (!gd_wait(&ctl->acc_full[ab], ((uint32_t)(lt >> 1)) & 1u, ctl, OWL_ERR_WAIT_MMA)) break;
      tc_fence_after();
      const int row = m0 + q4 * 32 + lane;
      __nv_bfloat16* obase = p.out + (size_t)row * p.ldo;
      const int jt = mn % p.m_tiles;
      if (RS)   // slot [this rank] of the owner of row tile jt, at the tile's local position
        obase = p.rs_dst[jt % p.world] +
                ((size_t)p.rank * p.max_local * GD_BM + (size_t)(jt / p.world) * GD_BM + q4 * 32 + lane) * p.ldo;
#pragma unroll 1
      for (int c = 0; c < GD_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(ab * GD_BN + c * 32), r);
        tc_wait_ld();
        if (F8 && row < p.T) {
          const float sa = p.a_scale[row];
#pragma unroll
          for (int v = 0; v < 32; ++v) {
            const int col = n0 + c * 32 + v;
            r[v] = __float_as_uint(__uint_as_float(r[v]) * sa * (col < p.N ? p.b_scale[col] : 0.f));
          }
        }
        if (!AG && !RS && KS > 1) {
          // k-split: fp32 partial tile (scaled already in the e4m3 form); the reduce kernel sums the parts
          if (row < p.T) {
            float* po = p.partial + ((size_t)(tile % KS) * p.T + row) * p.ldp + n0 + c * 32;
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<uint4*>(po + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
          }
        } else if (row < p.T) {
          __nv_bfloat16* o = obase + n0 + c * 32;
          if (n0 + c * 32 + 32 <= p.N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 pk;
              if (p.out_f16) {
                pk.x = pack_f16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                pk.y = pack_f16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                pk.z = pack_f16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                pk.w = pack_f16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              } else {
                pk.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                pk.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                pk.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                pk.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              }
              *reinterpret_cast<uint4*>(o + v * 8) = pk;
            }
          } else {
            for (int v = 0; v < 32; ++v)
              if (n0 + c * 32 + v < p.N) {
                if (p.out_f16) reinterpret_cast<__half*>(o)[v] = __float2half_rn(__uint_as_float(r[v]));
                else o[v] = __float2bfloat16(__uint_as_float(r[v]));
              }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[ab]);
      if (RS) {
        // each warp fences its peer stores and counts itself; the warp that completes a row tile (4 warps x
        // its weight tiles, over all CTAs) publishes the sequence number at the owner
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int old = atomicAdd(p.rs_done + jt, 1);
          if (old == p.n_tiles * 4 - 1) {
            p.rs_done[jt] = 0;
            __threadfence_system();
            gd_st_release_sys(p.rs_flag[jt % p.world] + p.rank * p.max_local + jt / p.world, p.rs_seq);
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

// out[row][col] = bf16(sum over parts): grid (ceil(N / 1024), T), 256 threads x 4 columns
__global__ void __launch_bounds__(256) gemm_ksplit_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                                                 int T, int N, int ldp, int ldo, int ks) {
  const int row = blockIdx.y, col = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (col >= N) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < ks; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(partial + ((size_t)s * T + row) * ldp + col);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  __nv_bfloat16* o = out + (size_t)row * ldo + col;
  if (col + 4 <= N) {
    *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
  } else {
    const float a[4] = {acc.x, acc.y, acc.z, acc.w};
    for (int i = 0; i < 4 && col + i < N; ++i) o[i] = __float2bfloat16(a[i]);
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn2 gd_encode() {
  static EncodeTiledFn2 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn2>(p);
  }
  return fn;
}
static int gd_map(CUtensorMap* m, const void* ptr, int rows, int K, int ld, int fmt, int box_rows) {   // fmt 2: e4m3 bytes
  EncodeTiledFn2 enc = gd_encode();
  if (!enc) return OWL_ERR_LAUNCH * 1000 - 1;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (fmt == 2 ? 1 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)(fmt == 2 ? 2 * GD_BK : GD_BK), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, fmt == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : fmt ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OWL_OK : OWL_ERR_LAUNCH * 1000 - (int)r;
}

}  // namespace owl
using namespace owl;

constexpr int GD_MAX_DEV = 64;
static float* g_ks_scratch[GD_MAX_DEV] = {nullptr};
static size_t g_ks_scratch_bytes[GD_MAX_DEV] = {0};

static int gd_launch(const void* x, int ldx, const void* w, int ldw, GdParams& p, int mode, cudaStream_t st) {
  const int kmask = p.fmt == 2 ? 127 : 63, ldmask = p.fmt == 2 ? 15 : 7;
  if (p.T < 1 || p.N < 1 || p.K <= kmask || (p.K & kmask) || (ldx & ldmask) || (ldw & ldmask) || (p.ldo & 7) || p.fmt < 0 ||
      p.fmt > 2 || (p.fmt == 2) != (mode == 3) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return OWL_ERR_BAD_ARG;
  CUtensorMap a, b;
  int r = gd_map(&a, x, p.T, p.K, ldx, p.fmt, GD_BM);
  if (r) return r;
  r = gd_map(&b, w, p.N, p.K, ldw, p.fmt, GD_BN);
  if (r) return r;
  p.m_tiles = (p.T + GD_BM - 1) / GD_BM; p.n_tiles = (p.N + GD_BN - 1) / GD_BN;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(gemm_dense_kernel<false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GD_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_dense_kernel<true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GD_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_dense_kernel<false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GD_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_dense_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GD_SMEM) != cudaSuccess) {
      sms = 0;
      return OWL_ERR_LAUNCH * 1000;
    }
  }
  int tiles = p.m_tiles * p.n_tiles;
  // few output tiles (small T and a narrow weight): cut k so that every SM streams a share of the weight; the fp32
  // partial tiles (at most 148 tiles of 128 x 256 floats = 19.4 MB) live in a scratch buffer the CALLER registers per
  // device (owl_gemm_dense_set_scratch): this launcher never allocates; without a scratch the product runs unsplit
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  float* ks_scratch = (dev_id >= 0 && dev_id < GD_MAX_DEV) ? g_ks_scratch[dev_id] : nullptr;
  const size_t KS_SCRATCH = (dev_id >= 0 && dev_id < GD_MAX_DEV) ? g_ks_scratch_bytes[dev_id] : 0;
  p.ksplit = 1;
  const int KIs = p.K / (p.fmt == 2 ? 2 * GD_BK : GD_BK);
  if ((mode == 0 || mode == 3) && !p.out_f16 && tiles * 2 <= sms && KIs >= 8) {
    int ks = sms / tiles;
    if (ks > KIs / 4) ks = KIs / 4;
    if (ks > 16) ks = 16;
    p.ldp = p.n_tiles * GD_BN;
    if (ks > 1 && (size_t)ks * p.T * p.ldp * sizeof(float) <= KS_SCRATCH) {
      if (ks_scratch) { p.ksplit = ks; p.partial = ks_scratch; tiles *= ks; }
    }
  }
  const int grid = tiles < sms ? tiles : sms;
  if (mode == 0) gemm_dense_kernel<false, false, false><<<grid, GD_THREADS, GD_SMEM, st>>>(a, b, p);
  else if (mode == 1) gemm_dense_kernel<true, false, false><<<grid, GD_THREADS, GD_SMEM, st>>>(a, b, p);
  else if (mode == 2) gemm_dense_kernel<false, true, false><<<grid, GD_THREADS, GD_SMEM, st>>>(a, b, p);
  else gemm_dense_kernel<false, false, true><<<grid, GD_THREADS, GD_SMEM, st>>>(a, b, p);
  OWL_LAUNCH_CHECK();
  if (p.ksplit > 1) {
    gemm_ksplit_reduce_kernel<<<dim3((p.N + 1023) / 1024, p.T), 256, 0, st>>>(p.partial, p.out, p.T, p.N, p.ldp, p.ldo, p.ksplit);
    OWL_LAUNCH_CHECK();
  }
  return OWL_OK;
}

// x: [T][ldx], w: [N][ldw], both fp16 (fmt 0) or both bf16 (fmt 1); out bf16 [T][ldo]. K multiple of 64.
OWL_API int owl_f16_gemm_persist(const void* x, int ldx, const void* w, int ldw, void* out, int T, int N, int K, int ldo,
                                 int fmt, cudaStream_t st) {
  if (reinterpret_cast<uintptr_t>(out) & 15) return OWL_ERR_BAD_ARG;
  GdParams p = {};
  p.out = (__nv_bfloat16*)out; p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.fmt = fmt;
  return gd_launch(x, ldx, w, ldw, p, 0, st);
}

// The same product with an fp16 result (attention scores of the GEMM-form prefill attention): 11 mantissa bits.
OWL_API int owl_f16_gemm_persist_f16out(const void* x, int ldx, const void* w, int ldw, void* out, int T, int N, int K, int ldo,
                                        int fmt, cudaStream_t st) {
  if (reinterpret_cast<uintptr_t>(out) & 15) return OWL_ERR_BAD_ARG;
  GdParams p = {};
  p.out = (__nv_bfloat16*)out; p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.fmt = fmt; p.out_f16 = 1;
  return gd_launch(x, ldx, w, ldw, p, 0, st);
}

// xq: e4m3 [T][ldx], wq: e4m3 [N][ldw] (bytes), sx fp32 [T], sw fp32 [N]; out bf16 [T][ldo] = sx[t] sw[n] (xq . wq^T).
// K multiple of 128.
OWL_API int owl_e4m3_gemm(const void* xq, int ldx, const void* sx, const void* wq, int ldw, const void* sw, void* out, int T,
                          int N, int K, int ldo, cudaStream_t st) {
  if ((reinterpret_cast<uintptr_t>(out) & 15) || !sx || !sw) return OWL_ERR_BAD_ARG;
  GdParams p = {};
  p.out = (__nv_bfloat16*)out; p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.fmt = 2;
  p.a_scale = (const float*)sx; p.b_scale = (const float*)sw;
  return gd_launch(xq, ldx, wq, ldw, p, 3, st);
}

// Column-parallel GEMM over activation rows gathered from the ranks: x is THIS rank's copy of the gathered
// rows [T][ldx]; row tile j is valid once ag_flags[(j % world) * max_local + j / world] >= seq.
OWL_API int owl_f16_gemm_ag(const void* x, int ldx, const void* w, int ldw, void* out, int T, int N, int K, int ldo, int fmt,
                            const void* ag_flags, unsigned seq, int world, int max_local, unsigned spin_limit,
                            cudaStream_t st) {
  if ((reinterpret_cast<uintptr_t>(out) & 15) || !ag_flags || world < 1 || world > 8 || max_local < 1 ||
      (T + GD_BM - 1) / GD_BM > world * max_local)
    return OWL_ERR_BAD_ARG;
  GdParams p = {};
  p.out = (__nv_bfloat16*)out; p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.fmt = fmt;
  p.world = world; p.max_local = max_local; p.ag_flags = (const uint32_t*)ag_flags; p.ag_seq = seq; p.spin_limit = spin_limit;
  return gd_launch(x, ldx, w, ldw, p, 1, st);
}

// Row-parallel GEMM + reduce-scatter: the partial sums of row tile j go to slot [rank] of rank j % world
// (dst[r] = base of rank r's slot buffer [world][max_local * 128][ldo], flag[r] = base of its flag table
// [world][max_local]); done = local int[row tiles], zero before the first call.
OWL_API int owl_f16_gemm_rs(const void* x, int ldx, const void* w, int ldw, int T, int N, int K, int ldo, int fmt,
                            void* const* dst, void* const* flag, void* done, unsigned seq, int rank, int world, int max_local,
                            cudaStream_t st) {
  if (!dst || !flag || !done || world < 1 || world > 8 || rank < 0 || rank >= world || max_local < 1 ||
      (T + GD_BM - 1) / GD_BM > world * max_local || N > ldo)
    return OWL_ERR_BAD_ARG;
  GdParams p = {};
  p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.fmt = fmt;
  p.rank = rank; p.world = world; p.max_local = max_local; p.rs_seq = seq; p.rs_done = (int*)done;
  for (int r = 0; r < world; ++r) {
    if (!dst[r] || !flag[r] || (reinterpret_cast<uintptr_t>(dst[r]) & 15)) return OWL_ERR_BAD_ARG;
    p.rs_dst[r] = (__nv_bfloat16*)dst[r];
    p.rs_flag[r] = (uint32_t*)flag[r];
  }
  return gd_launch(x, ldx, w, ldw, p, 2, st);
}

// Registers (or with a null pointer removes) the split-K scratch of the current device: caller-owned device memory of at
// least `bytes` bytes that lives as long as dense GEMMs may run. Recommended size: 160 tiles x 128 x 256 floats (21 MB).
OWL_API int owl_gemm_dense_set_scratch(void* ptr, long long bytes) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= GD_MAX_DEV || bytes < 0) return OWL_ERR_BAD_ARG;
  if (ptr && (reinterpret_cast<uintptr_t>(ptr) & 15)) return OWL_ERR_BAD_ARG;
  g_ks_scratch[dev] = (float*)ptr;
  g_ks_scratch_bytes[dev] = ptr ? (size_t)bytes : 0;
  return OWL_OK;
}

OWL_API int owl_gemm_dense_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_dense_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_gemm_dense_status, &zero, sizeof(int));
  return v;
}
