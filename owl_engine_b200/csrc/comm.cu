// Tensor-parallel collectives written as kernels over symmetric (peer-mapped) memory.
//
//   owl_ar_residual_norm : one-shot all-reduce of a row-parallel projection's partial sums
//                          fused with the residual add, the following RMSNorm and the ActPack
//                          producer:  h += sum_r partial_r ;  x = rmsnorm(h) * (1 + w)
//                          One CTA per token row; every rank reduces the same values in the same
//                          (rank) order, so all ranks hold bit-identical h. Decode / verify sizes.
//   owl_ar_inplace       : plain one-shot all-reduce (sum) of a bf16 buffer, grid-strided; used for
//                          prefill-size payloads when the GEMM-fused path is not taken.
//   owl_argmax_merge     : vocab-split lm_head: exchange each rank's (max, index) per row and pick
//                          the global winner on every rank.
//
// Protocol: every rank owns, inside its symmetric buffer, a flag table flags[slot][src_rank]
// (uint32, monotonically increasing sequence numbers kept in a device-side counter so that a
// replayed CUDA graph needs no host update). A CTA signals by storing its sequence number into
// slot[cta] of every peer with st.release.sys and then waits (ld.acquire.sys, bounded) until all
// peers' numbers arrived in its own table. Payload buffers are double-buffered by call site
// (mixer / MLP alternate), so one barrier per collective is enough. A wait that runs out records
// OWL_ERR_WAIT_PEER in the status word and the kernel finishes without hanging.
//
// Peer data is read with ld.relaxed.sys (plain NVLink P2P loads) or, when the caller passes a
// multicast address, with multimem.ld_reduce (in-switch reduction over NVLink SHARP).
// No TMA multicast is used anywhere in this file.
//
// Role in the reference: owl_comm_ar_barrier_* / owl_comm_ar_fused_* (crates/kernels/cu/comm/*.cu,
// 2 ranks over PCIe P2P) followed by a separate owl_fused_add_rmsnorm launch; the fused
// "AR + add + rmsnorm" hook the reference's charter reserves (charter.md:79-80) is what this is.
#include "common.cuh"
#include "actpack.cuh"

namespace owl {

constexpr int MAX_RANKS = 8;
__device__ int g_comm_status = 0;

struct PeerTable {
  const void* ptr[MAX_RANKS];
};
struct FlagTable {
  uint32_t* ptr[MAX_RANKS];   // base of each rank's flag table (peer-mapped)
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// In-switch reduction of 8 bf16 values over all ranks' copies (fp32 accumulation in the switch).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}

// Cross-rank barrier of one CTA slot. `counter` is this rank's private sequence counter for the
// slot. Returns false when a peer's flag did not arrive within the limit.
__device__ __forceinline__ bool rank_barrier(const FlagTable& ft, uint32_t* counters, int slot, int rank, int world,
                                             uint32_t spin_limit) {
  __shared__ uint32_t s_seq;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_seq = counters[slot] + 1;
    counters[slot] = s_seq;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t seq = s_seq;
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    // flags[slot][src = rank] in the peer's table
    st_release_sys(ft.ptr[peer] + slot * MAX_RANKS + rank, seq);
    const uint32_t* mine = ft.ptr[rank] + slot * MAX_RANKS + peer;
    bool got = false;
    for (uint32_t i = 0; i < spin_limit; ++i) {
      // sequence numbers only grow; (int) difference handles wrap-around
      if ((int)(ld_acquire_sys(mine) - seq) >= 0) { got = true; break; }
      if (i > 64) __nanosleep(64);
    }
    if (!got) {
      s_ok = 0;
      atomicCAS(&g_comm_status, 0, OWL_ERR_WAIT_PEER);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

struct ArNormParams {
  PeerTable parts;            // each rank's partial [M][H] bf16 (same offset in every symmetric buffer)
  const void* mc_part;        // multicast address of the partial buffer, or nullptr
  FlagTable flags;
  uint32_t* counters;         // [slots] private
  __nv_bfloat16* h;           // [M][H] residual stream (in/out)
  const __nv_bfloat16* w;     // norm weight [H] (nullptr: no norm, only h is updated)
  __nv_bfloat16* normed;      // optional bf16 normalised output
  uint4* xpack; float2* xs;   // optional ActPack of the normalised output
  int H, G, rank, world, slot0, one_plus_w;
  float eps;
  uint32_t spin_limit;
};

__global__ void __launch_bounds__(1024) ar_residual_norm_kernel(ArNormParams p) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  rank_barrier(p.flags, p.counters, p.slot0 + row, p.rank, p.world, p.spin_limit);
  const int nchunks = p.H >> 3;
  __nv_bfloat16* hrow = p.h + (size_t)row * p.H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
    float acc[8];
    if (p.mc_part) {
      const uint4 u = multimem_ld_reduce_bf16x8(reinterpret_cast<const uint4*>(p.mc_part) + (size_t)row * nchunks + c);
      unpack_bf16x8(u, acc);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int r = 0; r < p.world; ++r) {   // fixed rank order -> identical sums on every rank
        const uint4 u = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(p.parts.ptr[r]) + (size_t)row * nchunks + c);
        float v[8];
        unpack_bf16x8(u, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i];
      }
    }
    const uint4 hu = reinterpret_cast<const uint4*>(hrow)[c];
    float hv[8];
    unpack_bf16x8(hu, hv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      hv[i] = __bfloat162float(__float2bfloat16(hv[i] + acc[i]));
      ss += hv[i] * hv[i];
    }
    reinterpret_cast<uint4*>(hrow)[c] = pack_bf16x8(hv);
  }
  if (!p.w) return;
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)p.H + p.eps);
  const int nround = (nchunks + 31) & ~31;
  const int tiles = p.G & ACT_TILES, gq = p.G & ~ACT_TILES, cpg = gq >> 3;
  for (int c = threadIdx.x; c < nround; c += blockDim.x) {
    float v[8];
    const bool live = c < nchunks;
    if (live) {
      const uint4 a = reinterpret_cast<const uint4*>(hrow)[c];   // written by this thread above
      unpack_bf16x8(a, v);
      const uint4 wv = reinterpret_cast<const uint4*>(p.w)[c];
      float wf[8];
      unpack_bf16x8(wv, wf);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        v[i] = __bfloat162float(__float2bfloat16(v[i] * rinv * (p.one_plus_w ? 1.f + wf[i] : wf[i])));
      if (p.normed) reinterpret_cast<uint4*>(p.normed + (size_t)row * p.H)[c] = pack_bf16x8(v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    if (p.xpack) {
      float sx, xsum;
      const uint4 pk = actpack_emit(v, cpg, sx, xsum);
      if (live) actpack_store(p.xpack, p.xs, tiles, gq, row, c, nchunks, pk, sx, xsum);
    }
  }
}

// Consumer of the push protocol (gemv.cu, EPI_PUSH): every rank's GEMV has written its partial sums into slot
// [src] of THIS rank's buffer and published a sequence number; this kernel waits for the numbers (bounded), adds the
// slots in rank order (bit-identical h on every rank), then residual + RMSNorm + ActPack as above. It touches no
// peer memory at all.
struct PushNormParams {
  const __nv_bfloat16* slots;  // local [world][push_rows][H]
  const uint32_t* flags;       // local [world]: sequence numbers published by the peers' GEMVs
  uint32_t* counters;          // private per-row sequence counters [rows]
  uint32_t* seq_src;           // when set: the expected sequence number is read here (the local producer's word) instead
  const uint2* ll;             // when set (one row only): the producer was the FMA projection, whose slots are 8-byte words
                               // (two sums + the exchange's number = *seq_src + 1) [world][H / 2]; no flags are used, every
                               // thread polls the words it adds (bounded), and the CTA writes the number back to *seq_src
  __nv_bfloat16* h; const __nv_bfloat16* w; __nv_bfloat16* normed; uint4* xpack; float2* xs;
  int H, G, world, ranks, push_rows, one_plus_w;    // world: slots to add (ranks x k parts); ranks: flags to wait for
  float eps;
  uint32_t spin_limit;
};
__global__ void __launch_bounds__(1024) push_residual_norm_kernel(PushNormParams p) {
  __shared__ float red[32];
  __shared__ uint32_t s_seq;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  if (threadIdx.x == 0) {
    if (p.ll) { s_seq = *p.seq_src + 1u; }
    else if (p.seq_src) { s_seq = *p.seq_src; }
    else { s_seq = p.counters[row] + 1; p.counters[row] = s_seq; }
  }
  __syncthreads();
  if (!p.ll && threadIdx.x < p.ranks) {
    bool got = false;
    for (uint32_t i = 0; i < p.spin_limit; ++i) {
      if ((int)(ld_acquire_sys(p.flags + threadIdx.x) - s_seq) >= 0) { got = true; break; }
      if (i > 64) __nanosleep(64);
    }
    if (!got) atomicCAS(&g_comm_status, 0, OWL_ERR_WAIT_PEER);
  }
  __syncthreads();
  const int nchunks = p.H >> 3;
  __nv_bfloat16* hrow = p.h + (size_t)row * p.H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; p.ll && r < p.world; ++r) {
      const uint4* src = reinterpret_cast<const uint4*>(p.ll + (size_t)r * (p.H >> 1)) + 2 * c;
      const uint32_t want = s_seq;
      uint4 u = ld_relaxed_sys_v4(src), v = ld_relaxed_sys_v4(src + 1);
      for (uint32_t i = 0; u.y != want || u.w != want || v.y != want || v.w != want;) {
        if (++i >= p.spin_limit) { atomicCAS(&g_comm_status, 0, OWL_ERR_WAIT_PEER); break; }
        if (i > 64) __nanosleep(32);
        u = ld_relaxed_sys_v4(src); v = ld_relaxed_sys_v4(src + 1);
      }
      acc[0] += bf16_lo(u.x); acc[1] += bf16_hi(u.x); acc[2] += bf16_lo(u.z); acc[3] += bf16_hi(u.z);
      acc[4] += bf16_lo(v.x); acc[5] += bf16_hi(v.x); acc[6] += bf16_lo(v.z); acc[7] += bf16_hi(v.z);
    }
    for (int r = 0; !p.ll && r < p.world; ++r) {
      // written by peers over NVLink: read past L1 (the acquire above orders the loads after the flag)
      const uint4 u = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(p.slots + ((size_t)r * p.push_rows + row) * p.H) + c);
      float v[8];
      unpack_bf16x8(u, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
    const uint4 hu = reinterpret_cast<const uint4*>(hrow)[c];
    float hv[8];
    unpack_bf16x8(hu, hv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      hv[i] = __bfloat162float(__float2bfloat16(hv[i] + acc[i]));
      ss += hv[i] * hv[i];
    }
    reinterpret_cast<uint4*>(hrow)[c] = pack_bf16x8(hv);
  }
  if (p.ll && threadIdx.x == 0) *p.seq_src = s_seq;      // one CTA in this form: every thread took the number from shared memory
  if (!p.w) return;
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)p.H + p.eps);
  const int nround = (nchunks + 31) & ~31;
  const int tiles = p.G & ACT_TILES, gq = p.G & ~ACT_TILES, cpg = gq >> 3;
  for (int c = threadIdx.x; c < nround; c += blockDim.x) {
    float v[8];
    const bool live = c < nchunks;
    if (live) {
      const uint4 a = reinterpret_cast<const uint4*>(hrow)[c];
      unpack_bf16x8(a, v);
      const uint4 wv = reinterpret_cast<const uint4*>(p.w)[c];
      float wf[8];
      unpack_bf16x8(wv, wf);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        v[i] = __bfloat162float(__float2bfloat16(v[i] * rinv * (p.one_plus_w ? 1.f + wf[i] : wf[i])));
      if (p.normed) reinterpret_cast<uint4*>(p.normed + (size_t)row * p.H)[c] = pack_bf16x8(v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    if (p.xpack) {
      float sx, xsum;
      const uint4 pk = actpack_emit(v, cpg, sx, xsum);
      if (live) actpack_store(p.xpack, p.xs, tiles, gq, row, c, nchunks, pk, sx, xsum);
    }
  }
}

// Owner side of the prefill reduce-scatter and the all-gather that follows it, one CTA per token row.
// The row-parallel GEMMs of all ranks have written their partial sums of this rank's row tiles into
// slots[source rank] (gemm_dense.cu, owl_f16_gemm_rs). Per row: wait for the sources' flags, add the slots
// in rank order to the residual row (kept only on the owner), RMS-normalise, and store the normalised row
// into EVERY rank's gathered-activation buffer with plain peer stores; the CTA that completes a row tile
// publishes the tile's sequence number on every rank, where the next column-parallel GEMM
// (owl_f16_gemm_ag) waits for it tile by tile. n_src = 0 seeds the pipeline (no slots: the residual rows
// already hold the embeddings); w = null ends it (residual update only).
struct RsNormAgParams {
  const __nv_bfloat16* slots;  // local [world][max_local * 128][H]
  const uint32_t* rs_flags;    // local [world][max_local]
  __nv_bfloat16* h;            // local residual rows of the owned tiles [max_local * 128][H]
  const __nv_bfloat16* w;
  void* xdst[MAX_RANKS];       // each rank's gathered activations [T][H], fp16 or bf16
  uint32_t* ag_flag[MAX_RANKS];// each rank's flag table [world][max_local]
  int* rows_done;              // local [max_local]
  int T, H, rank, world, max_local, n_src, one_plus_w, out_f16;
  uint32_t rs_seq, ag_seq, spin_limit;
  float eps;
};
__global__ void __launch_bounds__(256) rs_norm_ag_kernel(RsNormAgParams p) {
  __shared__ float red[32];
  __shared__ int s_fail;
  const int lt = blockIdx.y, j = lt * p.world + p.rank;
  const int grow = j * 128 + blockIdx.x;                       // global token row
  if (grow >= p.T) return;
  const int lrow = lt * 128 + blockIdx.x;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if ((int)threadIdx.x < p.n_src) {
    bool got = false;
    const uint32_t* f = p.rs_flags + threadIdx.x * p.max_local + lt;
    for (uint32_t i = 0; i < p.spin_limit; ++i) {
      if ((int)(ld_acquire_sys(f) - p.rs_seq) >= 0) { got = true; break; }
      if (i > 16) __nanosleep(100);
    }
    if (!got) { atomicCAS(&g_comm_status, 0, OWL_ERR_WAIT_PEER); s_fail = 1; }
  }
  __syncthreads();
  if (s_fail) return;                                          // the gather flag is never published: peers time out too
  const int nchunks = p.H >> 3;
  __nv_bfloat16* hrow = p.h + (size_t)lrow * p.H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
    float hv[8];
    unpack_bf16x8(reinterpret_cast<const uint4*>(hrow)[c], hv);
    if (p.n_src) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < p.n_src; ++r) {
        const uint4 u = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(p.slots + ((size_t)r * p.max_local * 128 + lrow) * p.H) + c);
        float v[8];
        unpack_bf16x8(u, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) hv[i] = __bfloat162float(__float2bfloat16(hv[i] + acc[i]));
      reinterpret_cast<uint4*>(hrow)[c] = pack_bf16x8(hv);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += hv[i] * hv[i];
  }
  if (!p.w) return;
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)p.H + p.eps);
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
    float v[8], wf[8];
    unpack_bf16x8(reinterpret_cast<const uint4*>(hrow)[c], v);
    unpack_bf16x8(reinterpret_cast<const uint4*>(p.w)[c], wf);
    uint4 pk;
    if (p.out_f16) {
      __half2 q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        q[i] = __floats2half2_rn(v[2 * i] * rinv * (p.one_plus_w ? 1.f + wf[2 * i] : wf[2 * i]),
                                 v[2 * i + 1] * rinv * (p.one_plus_w ? 1.f + wf[2 * i + 1] : wf[2 * i + 1]));
      pk = *reinterpret_cast<uint4*>(q);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * rinv * (p.one_plus_w ? 1.f + wf[i] : wf[i]);
      pk = pack_bf16x8(v);
    }
    for (int d = 0; d < p.world; ++d)
      reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.xdst[d]) + (size_t)grow * p.H)[c] = pk;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int valid = min(128, p.T - j * 128);
    const int old = atomicAdd(p.rows_done + lt, 1);
    if (old == valid - 1) {
      p.rows_done[lt] = 0;
      __threadfence_system();
      for (int d = 0; d < p.world; ++d) st_release_sys(p.ag_flag[d] + p.rank * p.max_local + lt, p.ag_seq);
    }
  }
}

// In-place sum over ranks of buf (bf16, n8 chunks of 8), every rank ends with the full sum.
// Each CTA reduces a contiguous share and writes it back to its OWN buffer only; two barriers
// (before reading, after reading) protect the in-place update.
struct ArInplaceParams {
  PeerTable bufs; FlagTable flags; uint32_t* counters;
  __nv_bfloat16* scratch;      // local [n8*8] staging for the reduced values
  size_t n8; int rank, world, slot0;
  uint32_t spin_limit;
};
__global__ void __launch_bounds__(512) ar_inplace_kernel(ArInplaceParams p) {
  const int slot = p.slot0 + blockIdx.x;
  rank_barrier(p.flags, p.counters, slot, p.rank, p.world, p.spin_limit);
  const size_t per = (p.n8 + gridDim.x - 1) / gridDim.x;
  const size_t lo = per * blockIdx.x, hi = min(p.n8, lo + per);
  for (size_t c = lo + threadIdx.x; c < hi; c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < p.world; ++r) {
      const uint4 u = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(p.bufs.ptr[r]) + c);
      float v[8];
      unpack_bf16x8(u, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
    reinterpret_cast<uint4*>(p.scratch)[c] = pack_bf16x8(acc);
  }
  // every rank has finished reading this share before anyone overwrites it
  rank_barrier(p.flags, p.counters, slot, p.rank, p.world, p.spin_limit);
  uint4* mine = reinterpret_cast<uint4*>(const_cast<void*>(p.bufs.ptr[p.rank]));
  for (size_t c = lo + threadIdx.x; c < hi; c += blockDim.x) mine[c] = reinterpret_cast<const uint4*>(p.scratch)[c];
}

// Vocab-split argmax merge: each rank publishes (value, index) per row, then all pick the max.
struct ArgmaxMergeParams {
  PeerTable exch;              // each rank's exchange area: float2-like {value, index} [rows][MAX_RANKS]
  FlagTable flags; uint32_t* counters;
  const float* local_val; const int* local_idx;   // this rank's per-row winner (index already global)
  int* out_idx; int rows, rank, world, slot;
  uint32_t spin_limit;
};
__global__ void __launch_bounds__(64) argmax_merge_kernel(ArgmaxMergeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  // publish into every peer's exchange area (tiny: rows * 8 bytes per peer)
  for (int i = threadIdx.x; i < p.rows * p.world; i += blockDim.x) {
    const int row = i / p.world, peer = i % p.world;
    uint2 v = make_uint2(__float_as_uint(p.local_val[row]), (uint32_t)p.local_idx[row]);
    uint2* dst = reinterpret_cast<uint2*>(const_cast<void*>(p.exch.ptr[peer])) + row * MAX_RANKS + p.rank;
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(dst), "r"(v.x), "r"(v.y) : "memory");
  }
  __threadfence_system();
  __syncthreads();
  rank_barrier(p.flags, p.counters, p.slot, p.rank, p.world, p.spin_limit);
  for (int row = threadIdx.x; row < p.rows; row += blockDim.x) {
    const uint2* src = reinterpret_cast<const uint2*>(p.exch.ptr[p.rank]) + row * MAX_RANKS;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < p.world; ++r) {
      uint2 v;
      asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(src + r) : "memory");
      const float val = __uint_as_float(v.x);
      const int idx = (int)v.y;
      if (val > best || (val == best && idx < bi)) { best = val; bi = idx; }
    }
    p.out_idx[row] = bi;
  }
}

}  // namespace owl
using namespace owl;

static void fill_tables(PeerTable& pt, const void* const* ptrs, FlagTable& ft, void* const* flags, int world) {
  for (int r = 0; r < MAX_RANKS; ++r) {
    pt.ptr[r] = r < world ? ptrs[r] : nullptr;
    ft.ptr[r] = r < world ? (uint32_t*)flags[r] : nullptr;
  }
}

// part_ptrs / flag_ptrs: host arrays of `world` device pointers (peer-mapped). slot0: first flag slot
// (rows M use slots slot0 .. slot0+M-1). mc_part may be null.
OWL_API int owl_ar_residual_norm(const void* const* part_ptrs, const void* mc_part, void* const* flag_ptrs,
                                 void* counters, void* h, const void* w, void* normed, void* xpack, void* xs, int M,
                                 int H, int G, int rank, int world, int slot0, float eps, int one_plus_w,
                                 unsigned spin_limit, int pdl, cudaStream_t st) {
  if (M < 1 || (H & 127) || world < 2 || world > MAX_RANKS || rank < 0 || rank >= world || !actpack_group_ok(G, M))
    return OWL_ERR_BAD_ARG;
  ArNormParams p = {};
  fill_tables(p.parts, part_ptrs, p.flags, flag_ptrs, world);
  p.mc_part = mc_part; p.counters = (uint32_t*)counters; p.h = (__nv_bfloat16*)h; p.w = (const __nv_bfloat16*)w;
  p.normed = (__nv_bfloat16*)normed; p.xpack = (uint4*)xpack; p.xs = (float2*)xs; p.H = H; p.G = G; p.rank = rank;
  p.world = world; p.slot0 = slot0; p.one_plus_w = one_plus_w; p.eps = eps; p.spin_limit = spin_limit;
  int threads = ((H / 8 + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(M); cfg.blockDim = dim3(threads); cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, ar_residual_norm_kernel, p);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

// slots: this rank's [world][push_rows][H] bf16 buffer; flags: this rank's [world] sequence words of the call site;
// counters: private uint32 [M] (zero before the first call). ll (optional, M = 1, seq_src required): the word buffer of the
// FMA projection's exchange [world * kparts][H / 2] instead of slots and flags.
OWL_API int owl_push_residual_norm(const void* slots, const void* flags, void* counters, void* h, const void* w,
                                   void* normed, void* xpack, void* xs, int M, int H, int G, int world, int push_rows,
                                   float eps, int one_plus_w, unsigned spin_limit, void* seq_src, int kparts, const void* ll,
                                   int pdl, cudaStream_t st) {
  if (M < 1 || M > push_rows || (H & 127) || world < 1 || kparts < 1 || world * kparts > MAX_RANKS || !actpack_group_ok(G, M))
    return OWL_ERR_BAD_ARG;
  if (ll && (M != 1 || !seq_src || (reinterpret_cast<uintptr_t>(ll) & 15))) return OWL_ERR_BAD_ARG;
  PushNormParams p = {};
  p.seq_src = (uint32_t*)seq_src;
  p.ll = (const uint2*)ll;
  p.ranks = world;
  world *= kparts;          // slots [rank * kparts + part]
  p.slots = (const __nv_bfloat16*)slots; p.flags = (const uint32_t*)flags; p.counters = (uint32_t*)counters;
  p.h = (__nv_bfloat16*)h; p.w = (const __nv_bfloat16*)w; p.normed = (__nv_bfloat16*)normed; p.xpack = (uint4*)xpack;
  p.xs = (float2*)xs; p.H = H; p.G = G; p.world = world; p.push_rows = push_rows; p.one_plus_w = one_plus_w; p.eps = eps;
  p.spin_limit = spin_limit;
  int threads = ((H / 8 + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(M); cfg.blockDim = dim3(threads); cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, push_residual_norm_kernel, p);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

// slots / rs_flags / h / rows_done are this rank's own memory; xdst[r] / ag_flag[r] are every rank's gathered
// activation buffer and flag table (peer-mapped). n_src = world (after a reduce-scatter GEMM) or 0 (seed).
OWL_API int owl_rs_norm_ag(const void* slots, const void* rs_flags, void* h, const void* w, void* const* xdst,
                           void* const* ag_flag, void* rows_done, int T, int H, int rank, int world, int max_local, int n_src,
                           unsigned rs_seq, unsigned ag_seq, float eps, int one_plus_w, int out_f16, unsigned spin_limit,
                           cudaStream_t st) {
  if (T < 1 || (H & 7) || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || max_local < 1 ||
      (n_src != 0 && n_src != world) || (T + 127) / 128 > world * max_local || !h || !rows_done || (n_src && (!slots || !rs_flags)))
    return OWL_ERR_BAD_ARG;
  RsNormAgParams p = {};
  p.slots = (const __nv_bfloat16*)slots; p.rs_flags = (const uint32_t*)rs_flags; p.h = (__nv_bfloat16*)h;
  p.w = (const __nv_bfloat16*)w; p.rows_done = (int*)rows_done; p.T = T; p.H = H; p.rank = rank; p.world = world;
  p.max_local = max_local; p.n_src = n_src; p.one_plus_w = one_plus_w; p.out_f16 = out_f16; p.rs_seq = rs_seq;
  p.ag_seq = ag_seq; p.spin_limit = spin_limit; p.eps = eps;
  if (w) {
    if (!xdst || !ag_flag) return OWL_ERR_BAD_ARG;
    for (int r = 0; r < world; ++r) {
      if (!xdst[r] || !ag_flag[r] || (reinterpret_cast<uintptr_t>(xdst[r]) & 15)) return OWL_ERR_BAD_ARG;
      p.xdst[r] = xdst[r];
      p.ag_flag[r] = (uint32_t*)ag_flag[r];
    }
  }
  const int m_tiles = (T + 127) / 128;
  const int mine = rank < m_tiles ? (m_tiles - rank + world - 1) / world : 0;   // row tiles this rank owns
  if (mine == 0) return OWL_OK;
  rs_norm_ag_kernel<<<dim3(128, mine), 256, 0, st>>>(p);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

OWL_API int owl_ar_inplace(const void* const* buf_ptrs, void* const* flag_ptrs, void* counters, void* scratch,
                           long long n_elems, int rank, int world, int slot0, int ctas, unsigned spin_limit,
                           cudaStream_t st) {
  if (n_elems < 8 || (n_elems & 7) || world < 2 || world > MAX_RANKS || ctas < 1 || ctas > 64) return OWL_ERR_BAD_ARG;
  ArInplaceParams p = {};
  fill_tables(p.bufs, buf_ptrs, p.flags, flag_ptrs, world);
  p.counters = (uint32_t*)counters; p.scratch = (__nv_bfloat16*)scratch; p.n8 = (size_t)n_elems / 8; p.rank = rank;
  p.world = world; p.slot0 = slot0; p.spin_limit = spin_limit;
  ar_inplace_kernel<<<ctas, 512, 0, st>>>(p);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

OWL_API int owl_argmax_merge(const void* const* exch_ptrs, void* const* flag_ptrs, void* counters,
                             const void* local_val, const void* local_idx, void* out_idx, int rows, int rank, int world,
                             int slot, unsigned spin_limit, int pdl, cudaStream_t st) {
  if (rows < 1 || rows > 32 || world < 2 || world > MAX_RANKS) return OWL_ERR_BAD_ARG;
  ArgmaxMergeParams p = {};
  fill_tables(p.exch, exch_ptrs, p.flags, flag_ptrs, world);
  p.counters = (uint32_t*)counters; p.local_val = (const float*)local_val; p.local_idx = (const int*)local_idx;
  p.out_idx = (int*)out_idx; p.rows = rows; p.rank = rank; p.world = world; p.slot = slot; p.spin_limit = spin_limit;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1); cfg.blockDim = dim3(64); cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, argmax_merge_kernel, p);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

// A single-rank wait that nothing satisfies: used by tests of the bounded-wait path (a flag that
// nobody sets). Returns after `spin_limit` polls with OWL_ERR_WAIT_PEER in the status word.
__global__ void wait_probe_kernel(uint32_t* flag, uint32_t want, uint32_t spin_limit, int* result) {
  bool got = false;
  for (uint32_t i = 0; i < spin_limit; ++i) {
    if ((int)(ld_acquire_sys(flag) - want) >= 0) { got = true; break; }
    if (i > 64) __nanosleep(64);
  }
  if (!got) atomicCAS(&g_comm_status, 0, OWL_ERR_WAIT_PEER);
  *result = got ? 0 : OWL_ERR_WAIT_PEER;
}
OWL_API int owl_comm_wait_probe(void* flag, unsigned want, unsigned spin_limit, void* result, cudaStream_t st) {
  wait_probe_kernel<<<1, 1, 0, st>>>((uint32_t*)flag, want, spin_limit, (int*)result);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

OWL_API int owl_comm_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_comm_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_comm_status, &zero, sizeof(int));
  return v;
}
