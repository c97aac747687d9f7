// L2 prefetch of a weight range ahead of the kernel that streams it.
//
// A decode step is a chain of weight-streaming GEMVs separated by small kernels (norms, activation packing, state updates);
// while those run, DRAM idles. This kernel is launched on a side branch of the step's CUDA graph: its few CTAs issue
// `cp.async.bulk.prefetch.L2` requests for the front of the NEXT projection's weights and exit at once; the requests drain
// through the memory system while the small kernels run, and the next GEMV finds that part of its stream in the 126 MB L2.
// Fire and forget: nothing waits on the prefetches, a dropped request only costs the hit.
#include "common.cuh"

namespace owl {

constexpr int PF_PIECE = 8192;     // bytes per prefetch request

__global__ void __launch_bounds__(128) l2_prefetch_kernel(const uint8_t* __restrict__ base, long long pieces, int tail_bytes) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += stride) {
    const uint8_t* p = base + i * PF_PIECE;
    const uint32_t bytes = (i == pieces - 1 && tail_bytes) ? (uint32_t)tail_bytes : (uint32_t)PF_PIECE;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
  }
}

}  // namespace owl
using namespace owl;

// p: 16-byte aligned device pointer; bytes is rounded down to a multiple of 16. ctas <= 0 picks 32.
OWL_API int owl_l2_prefetch(const void* p, long long bytes, int ctas, cudaStream_t st) {
  bytes &= ~15LL;
  if (!p || (reinterpret_cast<uintptr_t>(p) & 15) || bytes < 16) return OWL_ERR_BAD_ARG;
  const long long pieces = (bytes + PF_PIECE - 1) / PF_PIECE;
  const int tail = (int)(bytes - (pieces - 1) * PF_PIECE);
  if (ctas <= 0) ctas = 32;
  const long long need = (pieces + 127) / 128;
  if (need < ctas) ctas = (int)need;
  l2_prefetch_kernel<<<ctas, 128, 0, st>>>((const uint8_t*)p, pieces, tail == PF_PIECE ? 0 : tail);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}
