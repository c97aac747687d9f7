// Normalisation / activation / embedding / argmax kernels and the ActPack producers.
//
// Role in the reference: owl_fused_add_rmsnorm_*, owl_rmsnorm_* (crates/kernels/cu/ln/
// fused_add_rmsnorm.cu, rmsnorm.cu), owl_silu_and_mul_merged_* (cu/ln/silu_and_mul.cu),
// owl_embed_* (cu/elems/embed_f32.cu), owl_argmax_* (cu/elems/argmax_f16.cu),
// owl_sigmoid_gate_mul_f16 (cu/elems/sigmoid_gate_mul_f16.cu).
//
// "ActPack" is the activation format consumed by owl_w4a16_skinny (see gemv.cu): fp16 values
// permuted and pre-scaled inside each run of 8 consecutive k, plus (xsum, xoff) per group.
#include "common.cuh"
#include "actpack.cuh"

namespace owl {

// ---------------------------------------------------------------------------------------
// out_h      = h (+ delta)                       (bf16, optional, may alias h)
// normed     = rmsnorm(out_h) * (w or 1+w)        (bf16, optional)
// xpack/xs   = ActPack(normed)                    (optional)
// One CTA per token row.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) rmsnorm_pack_kernel(const __nv_bfloat16* __restrict__ h,
                                                            const __nv_bfloat16* __restrict__ delta,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            __nv_bfloat16* out_h, __nv_bfloat16* normed, uint4* xpack,
                                                            float2* xs, int K, int G, float eps, int one_plus_w,
                                                            int normed_f16) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int tiles = G & ACT_TILES;
  G &= ~ACT_TILES;
  const int row = blockIdx.x;
  const int nchunks = K >> 3;
  const uint4* hp = reinterpret_cast<const uint4*>(h + (size_t)row * K);
  const uint4* dp = delta ? reinterpret_cast<const uint4*>(delta + (size_t)row * K) : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
    uint4 a = hp[c];
    float v[8];
    unpack_bf16x8(a, v);
    if (dp) {
      uint4 b = dp[c];
      float u[8];
      unpack_bf16x8(b, u);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(__float2bfloat16(v[i] + u[i]));
      if (out_h) reinterpret_cast<uint4*>(out_h + (size_t)row * K)[c] = pack_bf16x8(v);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
  }
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)K + eps);
  if (!normed && !xpack) return;
  const uint4* src = (dp && out_h) ? reinterpret_cast<const uint4*>(out_h + (size_t)row * K) : hp;
  const int nround = (nchunks + 31) & ~31;
  const int cpg = G >> 3;  // chunks per group (4 or 16)
  for (int c = threadIdx.x; c < nround; c += blockDim.x) {
    float v[8];
    const bool live = c < nchunks;
    if (live) {
      uint4 a = src[c];
      unpack_bf16x8(a, v);
      if (dp && !out_h) {  // recompute the sum when the residual is not materialised
        uint4 b = dp[c];
        float u[8];
        unpack_bf16x8(b, u);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(__float2bfloat16(v[i] + u[i]));
      }
      uint4 wv = reinterpret_cast<const uint4*>(w)[c];
      float wf[8];
      unpack_bf16x8(wv, wf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float g = one_plus_w ? 1.f + wf[i] : wf[i];
        const float y = v[i] * rinv * g;
        v[i] = normed_f16 ? __half2float(__float2half_rn(clamp_h(y))) : __bfloat162float(__float2bfloat16(y));
      }
      if (normed) reinterpret_cast<uint4*>(normed + (size_t)row * K)[c] = normed_f16 ? pack_f16x8(v) : pack_bf16x8(v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    if (xpack) {
      float sx, xsum;
      const uint4 pk = actpack_emit(v, cpg, sx, xsum);
      if (live) actpack_store(xpack, xs, tiles, G, row, c, nchunks, pk, sx, xsum);
    }
  }
}

// bf16 [M][K] -> ActPack.
__global__ void __launch_bounds__(256) act_pack_kernel(const __nv_bfloat16* __restrict__ x, int ldx, uint4* xpack,
                                                       float2* xs, int K, int G) {
  pdl_launch_dependents();
  pdl_wait();
  const int tiles = G & ACT_TILES;
  G &= ~ACT_TILES;
  const int row = blockIdx.y;
  const int nchunks = K >> 3, cpg = G >> 3;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;  // grid.x covers nchunks rounded up to 32
  const bool live = c < nchunks;
  float v[8];
  if (live) {
    uint4 a = reinterpret_cast<const uint4*>(x + (size_t)row * ldx)[c];
    unpack_bf16x8(a, v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
  float sx, xsum;
  const uint4 pk = actpack_emit(v, cpg, sx, xsum);
  if (live) actpack_store(xpack, xs, tiles, G, row, c, nchunks, pk, sx, xsum);
}

// Merged gate_up output in "interleaved-8" order: columns [t*16 .. t*16+7] are gate_j and
// [t*16+8 .. t*16+15] are up_j for j = t*8 .. t*8+7. Produces silu(gate)*up as bf16 [M][I] and/or ActPack.
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* out,
                                                       uint4* xpack, float2* xs, int I, int G, int out_f16) {
  pdl_launch_dependents();
  pdl_wait();
  const int tiles = G & ACT_TILES;
  G &= ~ACT_TILES;
  const int row = blockIdx.y;
  const int nchunks = I >> 3, cpg = G >> 3;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = c < nchunks;
  float v[8];
  if (live) {
    const uint4* p = reinterpret_cast<const uint4*>(gu + (size_t)row * 2 * I) + (size_t)c * 2;
    uint4 ga = p[0], ua = p[1];
    float gf[8], uf[8];
    unpack_bf16x8(ga, gf);
    unpack_bf16x8(ua, uf);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float y = silu_f(gf[i]) * uf[i];
      v[i] = out_f16 ? __half2float(__float2half_rn(clamp_h(y))) : __bfloat162float(__float2bfloat16(y));
    }
    if (out) reinterpret_cast<uint4*>(out + (size_t)row * I)[c] = out_f16 ? pack_f16x8(v) : pack_bf16x8(v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
  if (xpack) {
    float sx, xsum;
    const uint4 pk = actpack_emit(v, cpg, sx, xsum);
    if (live) actpack_store(xpack, xs, tiles, G, row, c, nchunks, pk, sx, xsum);
  }
}

// y = attn * sigmoid(gate); attn bf16 [M][H*D] contiguous, gate read from the q_proj output
// whose per-head layout is [q_h | gate_h] (row stride ldq, head stride 2*D, gate offset D).
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(const __nv_bfloat16* __restrict__ attn,
                                                           const __nv_bfloat16* __restrict__ qraw, int ldq, int D,
                                                           __nv_bfloat16* out, uint4* xpack, float2* xs, int HD,
                                                           int G) {
  pdl_launch_dependents();
  pdl_wait();
  const int tiles = G & ACT_TILES;
  G &= ~ACT_TILES;
  const int row = blockIdx.y;
  const int nchunks = HD >> 3, cpg = G >> 3;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = c < nchunks;
  float v[8];
  if (live) {
    const int e = c * 8, head = e / D, off = e % D;
    uint4 a = reinterpret_cast<const uint4*>(attn + (size_t)row * HD)[c];
    uint4 gq = *reinterpret_cast<const uint4*>(qraw + (size_t)row * ldq + (size_t)head * 2 * D + D + off);
    float af[8], gf[8];
    unpack_bf16x8(a, af);
    unpack_bf16x8(gq, gf);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(__float2bfloat16(af[i] * sigmoid_f(gf[i])));
    if (out) reinterpret_cast<uint4*>(out + (size_t)row * HD)[c] = pack_bf16x8(v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
  if (xpack) {
    float sx, xsum;
    const uint4 pk = actpack_emit(v, cpg, sx, xsum);
    if (live) actpack_store(xpack, xs, tiles, G, row, c, nchunks, pk, sx, xsum);
  }
}

// Embedding gather: out[m][:] = table[ids[m]][:]  (bf16, H multiple of 8).
__global__ void __launch_bounds__(256) embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                                    __nv_bfloat16* out, int H, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * H);
  for (int c = threadIdx.x; c < (H >> 3); c += blockDim.x) dst[c] = src[c];
}

// Row argmax over bf16 logits in two stages (ties -> lowest index, like torch.argmax on CPU).
__global__ void __launch_bounds__(256) argmax_stage1(const __nv_bfloat16* __restrict__ logits, int V, int ld,
                                                     float* pval, int* pidx, int nparts) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y, part = blockIdx.x;
  const int per = (((V + nparts - 1) / nparts) + 7) & ~7;
  const int beg = part * per, end = min(V, beg + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  const __nv_bfloat16* lp = logits + (size_t)row * ld;
  for (int i = beg + threadIdx.x; i < end; i += blockDim.x) {
    const float v = __bfloat162float(lp[i]);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    pval[row * nparts + part] = best;
    pidx[row * nparts + part] = bi;
  }
}
__global__ void __launch_bounds__(128) argmax_stage2(const float* pval, const int* pidx, int nparts, int* out,
                                                     int vocab_offset, float* out_val = nullptr) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < nparts; i += 32) {
    const float v = pval[row * nparts + i];
    const int id = pidx[row * nparts + i];
    if (v > best || (v == best && id < bi)) { best = v; bi = id; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (threadIdx.x == 0) {
    out[row] = bi + vocab_offset;
    if (out_val) out_val[row] = best;
  }
}

// Self-feeding greedy decode: after sampling, make the sampled token the next step's input
// and advance the per-sequence position, context length and KV write slot on the device so a
// replayed graph needs no host update between steps. inp layout (int32):
//   ids[M] | pos3[3*M] | kv_slot[M] | ctx_len[B] | gdn_slot[B] | bt_row[B]   (M = B rows, T = 1)
__global__ void decode_advance_kernel(int* inp, const int* __restrict__ tok, const int* __restrict__ block_table,
                                      int max_blocks, int B) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int* ids = inp; int* pos3 = inp + B; int* kv_slot = inp + 4 * B; int* ctx = inp + 5 * B;
  const int* gslot = inp + 6 * B; const int* bt_row = inp + 7 * B;
  if (gslot[b] < 0) return;  // padding row
  ids[b] = tok[b];
  const int np = pos3[b] + 1;
  pos3[b] = np; pos3[B + b] += 1; pos3[2 * B + b] += 1;
  ctx[b] += 1;
  const int tpos = ctx[b] - 1;   // cache index of the token that will be written next step
  const int pg = tpos >> 4;
  kv_slot[b] = pg < max_blocks ? block_table[(size_t)bt_row[b] * max_blocks + pg] * 16 + (tpos & 15) : -1;
}

template <typename... Args>
static int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, int pdl, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

}  // namespace owl
using namespace owl;

OWL_API int owl_rmsnorm_pack(const void* h, const void* delta, const void* w, void* out_h, void* normed, void* xpack,
                             void* xs, int M, int K, int G, float eps, int one_plus_w, int normed_f16, int pdl,
                             cudaStream_t st) {
  if (M < 1 || (K & 127) || !actpack_group_ok(G, M)) return OWL_ERR_BAD_ARG;
  int threads = ((K / 8 + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  return launch_pdl(rmsnorm_pack_kernel, dim3(M), dim3(threads), pdl, st, (const __nv_bfloat16*)h,
                    (const __nv_bfloat16*)delta, (const __nv_bfloat16*)w, (__nv_bfloat16*)out_h,
                    (__nv_bfloat16*)normed, (uint4*)xpack, (float2*)xs, K, G, eps, one_plus_w, normed_f16);
}
OWL_API int owl_act_pack(const void* x, int ldx, void* xpack, void* xs, int M, int K, int G, int pdl, cudaStream_t st) {
  if (M < 1 || (K & 127) || (ldx & 7) || !actpack_group_ok(G, M)) return OWL_ERR_BAD_ARG;
  const int nchunks = K / 8;
  return launch_pdl(act_pack_kernel, dim3((nchunks + 255) / 256, M), dim3(256), pdl, st, (const __nv_bfloat16*)x, ldx,
                    (uint4*)xpack, (float2*)xs, K, G);
}
OWL_API int owl_silu_mul(const void* gate_up, void* out, void* xpack, void* xs, int M, int I, int G, int out_f16,
                         int pdl, cudaStream_t st) {
  if (M < 1 || (I & 127) || !actpack_group_ok(G, M)) return OWL_ERR_BAD_ARG;
  const int nchunks = I / 8;
  return launch_pdl(silu_mul_kernel, dim3((nchunks + 255) / 256, M), dim3(256), pdl, st,
                    (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, (uint4*)xpack, (float2*)xs, I, G, out_f16);
}
OWL_API int owl_sigmoid_gate(const void* attn, const void* qraw, int ldq, int D, void* out, void* xpack, void* xs,
                             int M, int HD, int G, int pdl, cudaStream_t st) {
  if (M < 1 || (HD & 127) || (D & 7) || (ldq & 7) || !actpack_group_ok(G, M)) return OWL_ERR_BAD_ARG;
  const int nchunks = HD / 8;
  return launch_pdl(sigmoid_gate_kernel, dim3((nchunks + 255) / 256, M), dim3(256), pdl, st,
                    (const __nv_bfloat16*)attn, (const __nv_bfloat16*)qraw, ldq, D, (__nv_bfloat16*)out,
                    (uint4*)xpack, (float2*)xs, HD, G);
}
OWL_API int owl_embed(const void* ids, const void* table, void* out, int M, int H, int vocab, int pdl,
                      cudaStream_t st) {
  if (M < 1 || (H & 7)) return OWL_ERR_BAD_ARG;
  return launch_pdl(embed_kernel, dim3(M), dim3(256), pdl, st, (const int*)ids, (const __nv_bfloat16*)table,
                    (__nv_bfloat16*)out, H, vocab);
}
// scratch: float[M*nparts] + int[M*nparts]; nparts <= 1024.
OWL_API int owl_argmax(const void* logits, int M, int V, int ld, void* scratch_val, void* scratch_idx, int nparts,
                       void* out_idx, int vocab_offset, void* out_val, int pdl, cudaStream_t st) {
  if (M < 1 || nparts < 1 || nparts > 1024) return OWL_ERR_BAD_ARG;
  int r = launch_pdl(argmax_stage1, dim3(nparts, M), dim3(256), pdl, st, (const __nv_bfloat16*)logits, V, ld,
                     (float*)scratch_val, (int*)scratch_idx, nparts);
  if (r) return r;
  return launch_pdl(argmax_stage2, dim3(M), dim3(32), pdl, st, (const float*)scratch_val, (const int*)scratch_idx,
                    nparts, (int*)out_idx, vocab_offset, (float*)out_val);
}

OWL_API int owl_decode_advance(void* inp, const void* tok, const void* block_table, int max_blocks, int B, int pdl,
                               cudaStream_t st) {
  if (B < 1) return OWL_ERR_BAD_ARG;
  return launch_pdl(decode_advance_kernel, dim3((B + 63) / 64), dim3(64), pdl, st, (int*)inp, (const int*)tok,
                    (const int*)block_table, max_blocks, B);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free argmax (declared and documented in owl_noalloc.h).
// ---------------------------------------------------------------------------------------------
#include "owl_noalloc.h"

namespace {
constexpr int NA_PARTS = 64;
constexpr int NA_MAX_DEV = 64;
// Partial maxima of stage 1: [rows][parts] values followed by [rows][parts] indices.
static __device__ __align__(256) unsigned char g_noalloc_scratch[OWL_NOALLOC_MAX_ROWS * NA_PARTS * 8];
// In host code the symbol above is only a handle; the device address is looked up once per device.
static void* g_noalloc_ptr[NA_MAX_DEV] = {nullptr};
}  // namespace

OWL_API int owl_argmax_noalloc(const void* logits, int rows, int V, int ld, void* out_idx, int vocab_offset,
                               cudaStream_t st) {
  if (rows < 1 || rows > OWL_NOALLOC_MAX_ROWS || V < 1 || ld < V || !logits || !out_idx) return OWL_ERR_BAD_ARG;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  if (dev < 0 || dev >= NA_MAX_DEV) return OWL_ERR_BAD_ARG;
  if (!g_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
    g_noalloc_ptr[dev] = ptr;
  }
  float* pval = reinterpret_cast<float*>(g_noalloc_ptr[dev]);
  int* pidx = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(g_noalloc_ptr[dev]) +
                                     (size_t)OWL_NOALLOC_MAX_ROWS * NA_PARTS * 4);
  int r = launch_pdl(argmax_stage1, dim3(NA_PARTS, rows), dim3(256), 0, st, (const __nv_bfloat16*)logits, V, ld, pval,
                     pidx, NA_PARTS);
  if (r) return r;
  return launch_pdl(argmax_stage2, dim3(rows), dim3(32), 0, st, (const float*)pval, (const int*)pidx, NA_PARTS,
                    (int*)out_idx, vocab_offset, (float*)nullptr);
}
