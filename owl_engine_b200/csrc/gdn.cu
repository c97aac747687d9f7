// Gated DeltaNet (linear attention) kernels.
//
//   owl_gdn_decode   : fused decode / verify step for T <= 8 rows per sequence: causal conv1d
//                      (k=4) + SiLU on q|k|v, l2norm(q,k), g = -exp(A_log) softplus(a+dt_bias),
//                      beta = sigmoid(b), gated delta-rule update of the fp32 state, gated
//                      RMSNorm * silu(z); writes bf16 and/or ActPack for out_proj.
//   owl_gdn_conv_fwd : prefill causal conv1d + SiLU (+ l2norm for q,k heads), parallel in T.
//   owl_gdn_scan     : prefill delta-rule recurrence, serial in T, state kept in registers,
//                      fused gating + gated RMSNorm.
//
// Math (per v-head h, k-head hk = h / (nv/nk), state S in f32[kd][vd]):
//   S <- e^g S ; kv = k^T S ; delta = beta (v - kv) ; S <- S + k (x) delta ; o = (q/sqrt(kd))^T S
// evaluated in one pass over the old state:  kS = k^T S_old, qS = q^T S_old,
//   delta = beta (v - e^g kS),  o = scale (e^g qS + (q.k) delta),  S_new = e^g S_old + k (x) delta.
//
// GVA (several v-heads share one k-head): the v-head CTAs of one k-head form a thread-block
// cluster; rank 0 computes the shared q/k convolution and is the only CTA that reads or
// writes the q/k convolution state, the others fetch q,k through distributed shared memory.
//
// Role in the reference: owl_gdn_decode_step_v2_f16, owl_gdn_conv_upd_*, owl_gdn_conv_fwd_f16,
// owl_gdn_recurrence_varlen_gqa_f16, owl_gdn_gating/l2norm/norm_act (crates/kernels/cu/gdn/*.cu).
#include <cooperative_groups.h>
#include "common.cuh"
#include "actpack.cuh"

namespace cg = cooperative_groups;

namespace owl {

constexpr int GD = 128;         // head dim (k and v)
constexpr int GDN_MAX_T = 8;    // rows per sequence in the fused decode kernel

struct GdnDecodeParams {
  const __nv_bfloat16* qkvz;    // [rows][ld]: q(K) | k(K) | v(V) | z(V)
  const __nv_bfloat16* ab;      // [rows][ldab]: a(nv) | b(nv)
  const float* conv_w;          // [conv_dim][4]
  const float* a_log;           // [nv]
  const float* dt_bias;         // [nv]
  const float* gamma;           // [128] gated-norm weight
  float* conv_state;            // [slots][conv_dim][3]  (x[t-3], x[t-2], x[t-1])
  float* state;                 // [slots][nv][128][128]
  const int* slots;             // [batch]; < 0 = padding row
  const int* tlen;              // optional [batch]: rows of sequence b to consume (min with T); the rest are skipped
  __nv_bfloat16* out;           // [rows][V] (optional)
  uint4* xpack;                 // ActPack of out (optional)
  float2* xs;
  int ld, ldab, nk, nv, T, G;
  float eps;
};

__global__ void __launch_bounds__(256) gdn_decode_kernel(GdnDecodeParams p) {
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float qk_s[2][256];       // double-buffered by row parity: q[0..127], k[128..255]
  __shared__ float v_s[128];
  __shared__ float part[2][8][128];    // [kS|qS][warp][v]
  __shared__ float o_s[128];
  __shared__ float red[32];
  __shared__ float scal[4];            // e^g, beta, q.k

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y;
  const int R = p.nv / p.nk;           // cluster size along x
  const int hk = h / R;
  const unsigned rank = (R > 1) ? cluster.block_rank() : 0;
  const int K = p.nk * GD, V = p.nv * GD, conv_dim = 2 * K + V;
  // The recurrent / convolution state and the step inputs (slots) are not written by the
  // preceding kernels of the same forward pass, so they are fetched before the
  // programmatic-dependency wait and overlap the predecessor's tail.
  const int slot = p.slots[b];
  // Padding rows still take part in the cluster barriers (slot is uniform per cluster).
  const bool live = slot >= 0;

  // State: thread owns k rows warp*16..+15, v columns lane*4..+3.
  float S[16][4];
  float* sp = live ? p.state + (((size_t)slot * p.nv + h) * GD + warp * 16) * GD + lane * 4 : nullptr;
  if (live) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float4 v = *reinterpret_cast<const float4*>(sp + (size_t)i * GD);
      S[i][0] = v.x; S[i][1] = v.y; S[i][2] = v.z; S[i][3] = v.w;
    }
  }
  // Conv windows: thread tid handles (rank 0 only) q/k channel tid of k-head hk, and threads
  // < 128 additionally handle v channel tid of head h.
  float wq[3] = {0, 0, 0}, wv[3] = {0, 0, 0};
  float cwq[4] = {0, 0, 0, 0}, cwv[4] = {0, 0, 0, 0};
  const int ch_qk = (tid < 128) ? hk * GD + tid : K + hk * GD + (tid - 128);
  const int ch_v = 2 * K + h * GD + tid;
  if (live) {
    if (rank == 0) {
      const float* cs = p.conv_state + ((size_t)slot * conv_dim + ch_qk) * 3;
      wq[0] = cs[0]; wq[1] = cs[1]; wq[2] = cs[2];
      const float4 w4 = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch_qk * 4);
      cwq[0] = w4.x; cwq[1] = w4.y; cwq[2] = w4.z; cwq[3] = w4.w;
    }
    if (tid < 128) {
      const float* cs = p.conv_state + ((size_t)slot * conv_dim + ch_v) * 3;
      wv[0] = cs[0]; wv[1] = cs[1]; wv[2] = cs[2];
      const float4 w4 = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch_v * 4);
      cwv[0] = w4.x; cwv[1] = w4.y; cwv[2] = w4.z; cwv[3] = w4.w;
    }
  }
  const float a_log = p.a_log[h], dt_bias = p.dt_bias[h];
  const float scale = rsqrtf((float)GD);
  const float4 gam4 = *reinterpret_cast<const float4*>(p.gamma + lane * 4);
  const float gam[4] = {gam4.x, gam4.y, gam4.z, gam4.w};
  pdl_launch_dependents();
  pdl_wait();

  const int Tn = p.tlen ? min(p.T, max(p.tlen[b], 0)) : p.T;     // uniform in the cluster (b is)
  for (int r = 0; r < Tn; ++r) {
    const size_t row = (size_t)b * p.T + r;
    const __nv_bfloat16* xr = p.qkvz + row * p.ld;
    const int buf = r & 1;
    // ---- conv + silu (+ l2norm for q,k) ------------------------------------------------
    if (rank == 0) {
      float x = live ? __bfloat162float(xr[ch_qk]) : 0.f;
      float y = cwq[0] * wq[0] + cwq[1] * wq[1] + cwq[2] * wq[2] + cwq[3] * x;
      wq[0] = wq[1]; wq[1] = wq[2]; wq[2] = x;
      y = silu_f(y);
      // l2norm over the 128 channels of q (warps 0-3) or k (warps 4-7)
      float ss = warp_sum(y * y);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      const int base = (tid < 128) ? 0 : 4;
      const float tot = red[base] + red[base + 1] + red[base + 2] + red[base + 3];
      qk_s[buf][tid] = y * rsqrtf(tot + 1e-6f);
    }
    if (tid < 128) {
      float x = live ? __bfloat162float(xr[ch_v]) : 0.f;
      float y = cwv[0] * wv[0] + cwv[1] * wv[1] + cwv[2] * wv[2] + cwv[3] * x;
      wv[0] = wv[1]; wv[1] = wv[2]; wv[2] = x;
      v_s[tid] = silu_f(y);
    }
    if (tid == 0) {
      float a = 0.f, bb = 0.f;
      if (live) {
        a = __bfloat162float(p.ab[row * p.ldab + h]);
        bb = __bfloat162float(p.ab[row * p.ldab + p.nv + h]);
      }
      const float gl = -__expf(a_log) * softplus_f(a + dt_bias);
      scal[0] = __expf(gl);
      scal[1] = sigmoid_f(bb);
    }
    if (R > 1) {
      cluster.sync();
      if (rank != 0) {
        const float* remote = cluster.map_shared_rank(&qk_s[buf][0], 0);
        qk_s[buf][tid] = remote[tid];
      }
    }
    __syncthreads();
    // ---- one pass over the state -------------------------------------------------------
    const float* qs = &qk_s[buf][0];
    const float* ks = &qk_s[buf][128];
    float kS[4] = {0, 0, 0, 0}, qS[4] = {0, 0, 0, 0}, qk = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float kk = ks[warp * 16 + i], qq = qs[warp * 16 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { kS[j] += kk * S[i][j]; qS[j] += qq * S[i][j]; }
    }
    {
      // q.k over 128: each warp sums 4 per lane
      float pq = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) pq += qs[lane * 4 + i] * ks[lane * 4 + i];
      qk = warp_sum(pq);
    }
    *reinterpret_cast<float4*>(&part[0][warp][lane * 4]) = make_float4(kS[0], kS[1], kS[2], kS[3]);
    *reinterpret_cast<float4*>(&part[1][warp][lane * 4]) = make_float4(qS[0], qS[1], qS[2], qS[3]);
    __syncthreads();
    float ksum[4] = {0, 0, 0, 0}, qsum[4] = {0, 0, 0, 0};
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float4 a = *reinterpret_cast<const float4*>(&part[0][w][lane * 4]);
      const float4 c = *reinterpret_cast<const float4*>(&part[1][w][lane * 4]);
      ksum[0] += a.x; ksum[1] += a.y; ksum[2] += a.z; ksum[3] += a.w;
      qsum[0] += c.x; qsum[1] += c.y; qsum[2] += c.z; qsum[3] += c.w;
    }
    const float eg = scal[0], beta = scal[1];
    float delta[4], o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      delta[j] = beta * (v_s[lane * 4 + j] - eg * ksum[j]);
      o[j] = scale * (eg * qsum[j] + qk * delta[j]);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float kk = ks[warp * 16 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) S[i][j] = eg * S[i][j] + kk * delta[j];
    }
    // ---- gated RMSNorm * silu(z), by warp 0 --------------------------------------------
    if (warp == 0) {
      float ss = o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3];
      ss = warp_sum(ss);
      const float rinv = rsqrtf(ss / (float)GD + p.eps);
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int vi = lane * 4 + j;
        const float z = live ? __bfloat162float(xr[2 * K + V + h * GD + vi]) : 0.f;
        y[j] = __bfloat162float(__float2bfloat16(o[j] * rinv * gam[j] * silu_f(z)));
        o_s[vi] = y[j];
      }
      if (live && p.out) {
        uint2 pk = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
        *reinterpret_cast<uint2*>(p.out + row * V + h * GD + lane * 4) = pk;
      }
      __syncwarp();
      if (p.xpack) {
        // 16 chunks of 8; lanes 0-15 pack one chunk each (lanes 16-31 pack zeros)
        float v8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v8[i] = (lane < 16) ? o_s[lane * 8 + i] : 0.f;
        const int tiles = p.G & ACT_TILES, gq = p.G & ~ACT_TILES;
        float sx, xsum;
        const uint4 pk = actpack_emit(v8, gq >> 3, sx, xsum);
        if (live && lane < 16) actpack_store(p.xpack, p.xs, tiles, gq, row, (h * GD) / 8 + lane, V / 8, pk, sx, xsum);
      }
    }
    // qk_s is double buffered, v_s/part/scal are rewritten only after the next barrier pair.
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      *reinterpret_cast<float4*>(sp + (size_t)i * GD) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
    if (rank == 0) {
      float* cs = p.conv_state + ((size_t)slot * conv_dim + ch_qk) * 3;
      cs[0] = wq[0]; cs[1] = wq[1]; cs[2] = wq[2];
    }
    if (tid < 128) {
      float* cs = p.conv_state + ((size_t)slot * conv_dim + ch_v) * 3;
      cs[0] = wv[0]; cs[1] = wv[1]; cs[2] = wv[2];
    }
  }
  // Keep rank 0's shared memory alive until every peer finished its last remote read.
  if (R > 1) cluster.sync();
}

// ---------------------------------------------------------------------------------------
// Prefill conv: one warp per (t, 128-channel segment). Segments 0..2nk-1 are q/k heads (get
// l2norm), the rest are v heads. Reads the 3-sample history from conv_state for t < 3 and
// (blockIdx.z == last time tile) writes the new history. Output bf16 [T][conv_dim].
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gdn_conv_fwd_kernel(const __nv_bfloat16* __restrict__ x, int ld,
                                                           const float* __restrict__ conv_w, float* conv_state,
                                                           int slot, __nv_bfloat16* out, int T, int nk, int nv,
                                                           int use_state) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seg = blockIdx.x;
  const int t = blockIdx.y * 8 + warp;
  const int K = nk * GD, conv_dim = 2 * K + nv * GD;
  if (t >= T) return;
  const int ch0 = seg * GD + lane * 4;
  float acc[4];
  float xin[4][4];  // [tap][channel]
#pragma unroll
  for (int tap = 0; tap < 4; ++tap) {
    const int tt = t - 3 + tap;
    if (tt >= 0) {
      const uint2 u = *reinterpret_cast<const uint2*>(x + (size_t)tt * ld + ch0);
      xin[tap][0] = bf16_lo(u.x); xin[tap][1] = bf16_hi(u.x); xin[tap][2] = bf16_lo(u.y); xin[tap][3] = bf16_hi(u.y);
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        xin[tap][c] = use_state ? conv_state[((size_t)slot * conv_dim + ch0 + c) * 3 + (3 + tt)] : 0.f;
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const float4 w4 = *reinterpret_cast<const float4*>(conv_w + (size_t)(ch0 + c) * 4);
    acc[c] = silu_f(w4.x * xin[0][c] + w4.y * xin[1][c] + w4.z * xin[2][c] + w4.w * xin[3][c]);
  }
  if (seg < 2 * nk) {
    float ss = warp_sum(acc[0] * acc[0] + acc[1] * acc[1] + acc[2] * acc[2] + acc[3] * acc[3]);
    const float rinv = rsqrtf(ss + 1e-6f);
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[c] *= rinv;
  }
  *reinterpret_cast<uint2*>(out + (size_t)t * conv_dim + ch0) =
      make_uint2(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]));
}
// New conv history after a prefill chunk: the last 3 inputs (falling back to the old history
// when the chunk is shorter than 3). One thread per channel. Runs after gdn_conv_fwd_kernel.
__global__ void gdn_conv_state_kernel(const __nv_bfloat16* __restrict__ x, int ld, float* conv_state, int slot, int T,
                                      int conv_dim, int use_state) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= conv_dim) return;
  float* cs = conv_state + ((size_t)slot * conv_dim + ch) * 3;
  float old[3] = {cs[0], cs[1], cs[2]};
  float nw[3];
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int tt = T - 3 + i;
    nw[i] = tt >= 0 ? __bfloat162float(x[(size_t)tt * ld + ch]) : (use_state ? old[3 + tt] : 0.f);
  }
  cs[0] = nw[0]; cs[1] = nw[1]; cs[2] = nw[2];
}

// ---------------------------------------------------------------------------------------
// Prefill recurrence: one CTA per v-head, serial in T. qkv: bf16 [T][conv_dim] from the conv
// kernel (q,k already l2-normalised); z/a/b read from the projection outputs.
// ---------------------------------------------------------------------------------------
struct GdnScanParams {
  const __nv_bfloat16* qkv;     // [T][conv_dim]
  const __nv_bfloat16* z;       // [T][ldz], z column base already applied
  const __nv_bfloat16* ab;      // [T][ldab]
  const float* a_log; const float* dt_bias; const float* gamma;
  float* state;                 // [slots][nv][128][128]
  __nv_bfloat16* out;           // [T][V]
  int ldz, ldab, nk, nv, T, slot, use_state, out_f16;
  float eps;
};
__global__ void __launch_bounds__(256) gdn_scan_kernel(GdnScanParams p) {
  __shared__ float q_s[2][128], k_s[2][128], v_s[2][128];
  __shared__ float part[2][8][128];
  __shared__ float scal[2][2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, R = p.nv / p.nk, hk = h / R;
  const int K = p.nk * GD, V = p.nv * GD, conv_dim = 2 * K + V;
  float S[16][4];
  float* sp = p.state + (((size_t)p.slot * p.nv + h) * GD + warp * 16) * GD + lane * 4;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float4 v = make_float4(0, 0, 0, 0);
    if (p.use_state) v = *reinterpret_cast<const float4*>(sp + (size_t)i * GD);
    S[i][0] = v.x; S[i][1] = v.y; S[i][2] = v.z; S[i][3] = v.w;
  }
  const float a_log = p.a_log[h], dt_bias = p.dt_bias[h];
  const float scale = rsqrtf((float)GD);
  auto stage = [&](int r, int buf) {
    const __nv_bfloat16* xr = p.qkv + (size_t)r * conv_dim;
    if (tid < 128) q_s[buf][tid] = __bfloat162float(xr[hk * GD + tid]);
    else k_s[buf][tid - 128] = __bfloat162float(xr[K + hk * GD + tid - 128]);
    if (tid < 128) v_s[buf][tid] = __bfloat162float(xr[2 * K + h * GD + tid]);
    if (tid == 128) {
      const float a = __bfloat162float(p.ab[(size_t)r * p.ldab + h]);
      const float bb = __bfloat162float(p.ab[(size_t)r * p.ldab + p.nv + h]);
      scal[buf][0] = __expf(-__expf(a_log) * softplus_f(a + dt_bias));
      scal[buf][1] = sigmoid_f(bb);
    }
  };
  if (p.T > 0) stage(0, 0);
  __syncthreads();
  for (int r = 0; r < p.T; ++r) {
    const int buf = r & 1;
    if (r + 1 < p.T) stage(r + 1, buf ^ 1);
    const float* qs = q_s[buf];
    const float* ks = k_s[buf];
    float kS[4] = {0, 0, 0, 0}, qS[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float kk = ks[warp * 16 + i], qq = qs[warp * 16 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { kS[j] += kk * S[i][j]; qS[j] += qq * S[i][j]; }
    }
    float pq = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) pq += qs[lane * 4 + i] * ks[lane * 4 + i];
    const float qk = warp_sum(pq);
    *reinterpret_cast<float4*>(&part[0][warp][lane * 4]) = make_float4(kS[0], kS[1], kS[2], kS[3]);
    *reinterpret_cast<float4*>(&part[1][warp][lane * 4]) = make_float4(qS[0], qS[1], qS[2], qS[3]);
    __syncthreads();
    float ksum[4] = {0, 0, 0, 0}, qsum[4] = {0, 0, 0, 0};
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float4 a = *reinterpret_cast<const float4*>(&part[0][w][lane * 4]);
      const float4 c = *reinterpret_cast<const float4*>(&part[1][w][lane * 4]);
      ksum[0] += a.x; ksum[1] += a.y; ksum[2] += a.z; ksum[3] += a.w;
      qsum[0] += c.x; qsum[1] += c.y; qsum[2] += c.z; qsum[3] += c.w;
    }
    const float eg = scal[buf][0], beta = scal[buf][1];
    float delta[4], o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      delta[j] = beta * (v_s[buf][lane * 4 + j] - eg * ksum[j]);
      o[j] = scale * (eg * qsum[j] + qk * delta[j]);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float kk = ks[warp * 16 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) S[i][j] = eg * S[i][j] + kk * delta[j];
    }
    if (warp == (r & 7)) {  // rotate the epilogue warp so its extra work spreads out
      float ss = warp_sum(o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3]);
      const float rinv = rsqrtf(ss / (float)GD + p.eps);
      const uint2 zu = *reinterpret_cast<const uint2*>(p.z + (size_t)r * p.ldz + h * GD + lane * 4);
      const float z[4] = {bf16_lo(zu.x), bf16_hi(zu.x), bf16_lo(zu.y), bf16_hi(zu.y)};
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = o[j] * rinv * p.gamma[lane * 4 + j] * silu_f(z[j]);
      *reinterpret_cast<uint2*>(p.out + (size_t)r * V + h * GD + lane * 4) =
          p.out_f16 ? make_uint2(pack_f16(y[0], y[1]), pack_f16(y[2], y[3]))
                    : make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 16; ++i)
    *reinterpret_cast<float4*>(sp + (size_t)i * GD) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
}

// ---------------------------------------------------------------------------------------
// Column-split scan: the delta rule never mixes the columns (v dimension) of the state, so a head is
// cut into GS2_CS column slices with one CTA each (nv * GS2_CS CTAs instead of nv). Warp w owns 16 state
// rows, lane one column: 16 state registers per thread. Token inputs arrive in chunks of GS2_CH tokens
// through a three-deep cp.async ring, q.k is precomputed per chunk, and one __syncthreads per token
// separates the partial row sums from their use. Raw outputs go to a fp32 scratch; the gated RMSNorm
// over the head's 128 columns is a second, elementwise kernel.
// ---------------------------------------------------------------------------------------
constexpr int GS2_CS = 4, GS2_COLS = GD / GS2_CS, GS2_CH = 16, GS2_RING = 3;
struct GdnScan2Smem {
  __nv_bfloat16 q[GS2_RING][GS2_CH][GD];
  __nv_bfloat16 k[GS2_RING][GS2_CH][GD];
  __nv_bfloat16 v[GS2_RING][GS2_CH][GS2_COLS];
  float scal[GS2_RING][GS2_CH][4];      // e^g, beta, q.k
  float part[2][2][8][GS2_COLS];
};
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
}
__global__ void __launch_bounds__(256) gdn_scan2_kernel(GdnScanParams p, float* raw) {
  __shared__ __align__(16) GdnScan2Smem sm;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, cs = blockIdx.y, R = p.nv / p.nk, hk = h / R;
  const int K = p.nk * GD, V = p.nv * GD, conv_dim = 2 * K + V;
  const int col = cs * GS2_COLS + lane;
  float S[16];
  float* sp = p.state + (((size_t)p.slot * p.nv + h) * GD + warp * 16) * GD + col;
#pragma unroll
  for (int i = 0; i < 16; ++i) S[i] = p.use_state ? sp[(size_t)i * GD] : 0.f;
  const float a_log = p.a_log[h], dt_bias = p.dt_bias[h];
  const float scale = rsqrtf((float)GD);
  const int nchunks = (p.T + GS2_CH - 1) / GS2_CH;
  // one chunk = 16 tokens x (16 + 16 + 4) 16-byte pieces
  auto issue = [&](int c) {
    if (c < nchunks) {
      const int buf = c % GS2_RING, r0 = c * GS2_CH;
      for (int i = tid; i < GS2_CH * 36; i += 256) {
        const int t = i / 36, piece = i % 36, r = r0 + t;
        if (r < p.T) {
          const __nv_bfloat16* xr = p.qkv + (size_t)r * conv_dim;
          if (piece < 16) cp_async16(&sm.q[buf][t][piece * 8], xr + hk * GD + piece * 8);
          else if (piece < 32) cp_async16(&sm.k[buf][t][(piece - 16) * 8], xr + K + hk * GD + (piece - 16) * 8);
          else cp_async16(&sm.v[buf][t][(piece - 32) * 8], xr + 2 * K + h * GD + cs * GS2_COLS + (piece - 32) * 8);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(0);
  issue(1);
  for (int c = 0; c < nchunks; ++c) {
    const int buf = c % GS2_RING, r0 = c * GS2_CH, nt = min(GS2_CH, p.T - r0);
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();                    // chunk c landed for every thread; chunk c-1 fully consumed
    issue(c + 2);
    // per-token scalars of the chunk: warp w handles tokens 2w, 2w+1
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int t = warp * 2 + u;
      if (t < nt) {
        float pq = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) pq += __bfloat162float(sm.q[buf][t][lane * 4 + i]) * __bfloat162float(sm.k[buf][t][lane * 4 + i]);
        const float qk = warp_sum(pq);
        if (lane == 0) {
          const float a = __bfloat162float(p.ab[(size_t)(r0 + t) * p.ldab + h]);
          const float bb = __bfloat162float(p.ab[(size_t)(r0 + t) * p.ldab + p.nv + h]);
          sm.scal[buf][t][0] = __expf(-__expf(a_log) * softplus_f(a + dt_bias));
          sm.scal[buf][t][1] = sigmoid_f(bb);
          sm.scal[buf][t][2] = qk;
        }
      }
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const int pb = t & 1;
      float kk[16], kS = 0.f, qS = 0.f;
      const uint4* kp = reinterpret_cast<const uint4*>(&sm.k[buf][t][warp * 16]);
      const uint4* qp = reinterpret_cast<const uint4*>(&sm.q[buf][t][warp * 16]);
      const uint4 k0 = kp[0], k1 = kp[1], q0 = qp[0], q1 = qp[1];
      const uint32_t kw[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
      const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        kk[2 * i] = bf16_lo(kw[i]); kk[2 * i + 1] = bf16_hi(kw[i]);
        kS += kk[2 * i] * S[2 * i] + kk[2 * i + 1] * S[2 * i + 1];
        qS += bf16_lo(qw[i]) * S[2 * i] + bf16_hi(qw[i]) * S[2 * i + 1];
      }
      sm.part[pb][0][warp][lane] = kS;
      sm.part[pb][1][warp][lane] = qS;
      __syncthreads();
      float ksum = 0.f, qsum = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) { ksum += sm.part[pb][0][w][lane]; qsum += sm.part[pb][1][w][lane]; }
      const float eg = sm.scal[buf][t][0], beta = sm.scal[buf][t][1], qk = sm.scal[buf][t][2];
      const float delta = beta * (__bfloat162float(sm.v[buf][t][lane]) - eg * ksum);
#pragma unroll
      for (int i = 0; i < 16; ++i) S[i] = eg * S[i] + kk[i] * delta;
      if (warp == (t & 7)) raw[(size_t)(r0 + t) * V + h * GD + col] = scale * (eg * qsum + qk * delta);
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) sp[(size_t)i * GD] = S[i];
}

// out[r][h] = rmsnorm(raw[r][h]) * gamma * silu(z): one warp per (token, head)
__global__ void __launch_bounds__(256) gdn_norm_gate_kernel(const float* __restrict__ raw, const __nv_bfloat16* __restrict__ z,
                                                            int ldz, const float* __restrict__ gamma, __nv_bfloat16* out,
                                                            int T, int nv, float eps, int out_f16) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (wid >= (long long)T * nv) return;
  const int r = (int)(wid / nv), h = (int)(wid % nv), V = nv * GD;
  const float4 o = *reinterpret_cast<const float4*>(raw + (size_t)r * V + h * GD + lane * 4);
  const float ss = warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
  const float rinv = rsqrtf(ss / (float)GD + eps);
  const uint2 zu = *reinterpret_cast<const uint2*>(z + (size_t)r * ldz + h * GD + lane * 4);
  const float zz[4] = {bf16_lo(zu.x), bf16_hi(zu.x), bf16_lo(zu.y), bf16_hi(zu.y)};
  const float ov[4] = {o.x, o.y, o.z, o.w};
  float y[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) y[j] = ov[j] * rinv * gamma[lane * 4 + j] * silu_f(zz[j]);
  *reinterpret_cast<uint2*>(out + (size_t)r * V + h * GD + lane * 4) =
      out_f16 ? make_uint2(pack_f16(y[0], y[1]), pack_f16(y[2], y[3])) : make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
}

}  // namespace owl
using namespace owl;

OWL_API int owl_gdn_decode(const void* qkvz, int ld, const void* ab, int ldab, const void* conv_w, const void* a_log,
                           const void* dt_bias, const void* gamma, void* conv_state, void* state, const void* slots,
                           void* out, void* xpack, void* xs, int batch, int T, int nk, int nv, int G, float eps,
                           const void* tlen, int pdl, cudaStream_t st) {
  if (batch < 1 || T < 1 || T > GDN_MAX_T || nk < 1 || nv % nk || nv / nk > 8 || !actpack_group_ok(G, xpack ? batch * T : 1))
    return OWL_ERR_BAD_ARG;
  GdnDecodeParams p;
  p.qkvz = (const __nv_bfloat16*)qkvz; p.ab = (const __nv_bfloat16*)ab; p.conv_w = (const float*)conv_w;
  p.a_log = (const float*)a_log; p.dt_bias = (const float*)dt_bias; p.gamma = (const float*)gamma;
  p.conv_state = (float*)conv_state; p.state = (float*)state; p.slots = (const int*)slots; p.tlen = (const int*)tlen;
  p.out = (__nv_bfloat16*)out; p.xpack = (uint4*)xpack; p.xs = (float2*)xs;
  p.ld = ld; p.ldab = ldab; p.nk = nk; p.nv = nv; p.T = T; p.G = G; p.eps = eps;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nv, batch); cfg.blockDim = dim3(256); cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  const int R = nv / nk;
  if (R > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = R; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr; cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gdn_decode_kernel, p);
  if (e != cudaSuccess) return (int)OWL_ERR_LAUNCH * 1000 - (int)e;
  return OWL_OK;
}

// x: projection output rows [T][ld] whose first conv_dim columns are q|k|v. out: [T][conv_dim] bf16.
OWL_API int owl_gdn_conv_fwd(const void* x, int ld, const void* conv_w, void* conv_state, int slot, void* out, int T,
                             int nk, int nv, int use_state, cudaStream_t st) {
  if (T < 1 || nk < 1 || nv < 1 || (ld & 3)) return OWL_ERR_BAD_ARG;
  const int conv_dim = (2 * nk + nv) * GD;
  gdn_conv_fwd_kernel<<<dim3(2 * nk + nv, (T + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)x, ld, (const float*)conv_w,
                                                                      (float*)conv_state, slot,
                                                                      (__nv_bfloat16*)out, T, nk, nv, use_state);
  OWL_LAUNCH_CHECK();
  gdn_conv_state_kernel<<<(conv_dim + 255) / 256, 256, 0, st>>>((const __nv_bfloat16*)x, ld, (float*)conv_state, slot, T,
                                                                conv_dim, use_state);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

OWL_API int owl_gdn_scan(const void* qkv, const void* z, int ldz, const void* ab, int ldab, const void* a_log,
                         const void* dt_bias, const void* gamma, void* state, int slot, void* out, int T, int nk, int nv,
                         int use_state, float eps, int out_f16, cudaStream_t st) {
  if (T < 1 || nk < 1 || nv % nk || (ldz & 3)) return OWL_ERR_BAD_ARG;
  GdnScanParams p;
  p.qkv = (const __nv_bfloat16*)qkv; p.z = (const __nv_bfloat16*)z; p.ab = (const __nv_bfloat16*)ab;
  p.a_log = (const float*)a_log; p.dt_bias = (const float*)dt_bias; p.gamma = (const float*)gamma;
  p.state = (float*)state; p.out = (__nv_bfloat16*)out; p.ldz = ldz; p.ldab = ldab; p.nk = nk; p.nv = nv; p.T = T;
  p.slot = slot; p.use_state = use_state; p.eps = eps; p.out_f16 = out_f16;
  gdn_scan_kernel<<<nv, 256, 0, st>>>(p);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

// Same contract as owl_gdn_scan with a caller-provided fp32 scratch of T * nv * 128 floats: the column-split
// scan (4 CTAs per head) followed by the gated RMSNorm kernel. conv_dim must be a multiple of 8 elements.
// The gated RMSNorm alone: raw float [T][nv * 128] (un-normalised scan outputs) -> out[r][h] = rmsnorm(raw) * gamma * silu(z).
OWL_API int owl_gdn_norm_gate(const void* raw, const void* z, int ldz, const void* gamma, void* out, int T, int nv, float eps,
                              int out_f16, cudaStream_t st) {
  if (T < 1 || nv < 1 || (ldz & 3) || !raw || !out) return OWL_ERR_BAD_ARG;
  const long long warps = (long long)T * nv;
  gdn_norm_gate_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>((const float*)raw, (const __nv_bfloat16*)z, ldz,
                                                                   (const float*)gamma, (__nv_bfloat16*)out, T, nv, eps, out_f16);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

OWL_API int owl_gdn_scan_split(const void* qkv, const void* z, int ldz, const void* ab, int ldab, const void* a_log,
                               const void* dt_bias, const void* gamma, void* state, int slot, void* out, void* scratch,
                               int T, int nk, int nv, int use_state, float eps, int out_f16, cudaStream_t st) {
  if (T < 1 || nk < 1 || nv % nk || (ldz & 3) || !scratch) return OWL_ERR_BAD_ARG;
  GdnScanParams p;
  p.qkv = (const __nv_bfloat16*)qkv; p.z = (const __nv_bfloat16*)z; p.ab = (const __nv_bfloat16*)ab;
  p.a_log = (const float*)a_log; p.dt_bias = (const float*)dt_bias; p.gamma = (const float*)gamma;
  p.state = (float*)state; p.out = (__nv_bfloat16*)out; p.ldz = ldz; p.ldab = ldab; p.nk = nk; p.nv = nv; p.T = T;
  p.slot = slot; p.use_state = use_state; p.eps = eps; p.out_f16 = out_f16;
  gdn_scan2_kernel<<<dim3(nv, GS2_CS), 256, 0, st>>>(p, (float*)scratch);
  OWL_LAUNCH_CHECK();
  const long long warps = (long long)T * nv;
  gdn_norm_gate_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>((const float*)scratch, (const __nv_bfloat16*)z, ldz,
                                                                   (const float*)gamma, (__nv_bfloat16*)out, T, nv, eps, out_f16);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
