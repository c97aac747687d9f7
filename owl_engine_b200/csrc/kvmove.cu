// Batched KV page moves between the paged device pool and a page-major staging buffer.
//
//   owl_kv_pages_gather  : staging[i] = concatenation over the pool's tensors and layers of the slabs of page pages[i]
//   owl_kv_pages_scatter : the inverse (staging -> pool pages)
//
// The pool is layer-major ([layer][page][16][hkv][hd]), so one page is 2 x layers small slabs (32 KB each on the 27B
// model): copying pages one slab at a time costs dozens of driver copies per page, and a long-context demotion moves
// thousands of pages. These kernels pack any number of pages into one contiguous, page-major buffer (the layout of the
// pinned-host tier and of the disk files), so a demotion or a recall is one kernel plus one copy per run of consecutive
// host slots, all on the mover's side stream.
//
// Up to four tensors form a page (K, V, and for the int8 pool the K and V scales); each is described by its base pointer,
// the bytes between layers and the bytes of one page's slab (a multiple of 16).
//
// Reference counterpart: the swap-out / swap-in batch commands of the CUDA backend (crates/backends/cuda/src/swap.rs)
// and the BlockLeg move plans (crates/store/src/leg.rs).
#include "common.cuh"

namespace owl {

constexpr int KVMOVE_MAX_T = 4;

struct KvMoveParams {
  uint8_t* base[KVMOVE_MAX_T];
  long long layer_stride[KVMOVE_MAX_T];   // bytes between consecutive layers of tensor i
  int slab[KVMOVE_MAX_T];                 // bytes of one page in one layer of tensor i
  int n_tensors, n_layers;
  const int* pages;
  uint8_t* staging;
  long long page_bytes;                   // sum over tensors of n_layers * slab
};

// grid (pages, layers * tensors): one CTA copies one slab with 16-byte words.
template <bool GATHER>
__global__ void __launch_bounds__(256) kv_pages_move_kernel(KvMoveParams p) {
  const int i = blockIdx.x, lt = blockIdx.y;
  const int tsr = lt / p.n_layers, layer = lt % p.n_layers;
  const int page = p.pages[i];
  if (page < 0) return;
  long long off = 0;
  for (int q = 0; q < tsr; ++q) off += (long long)p.n_layers * p.slab[q];
  off += (long long)layer * p.slab[tsr];
  uint4* pool = reinterpret_cast<uint4*>(p.base[tsr] + (long long)layer * p.layer_stride[tsr] + (long long)page * p.slab[tsr]);
  uint4* stg = reinterpret_cast<uint4*>(p.staging + (long long)i * p.page_bytes + off);
  const int n = p.slab[tsr] >> 4;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    if (GATHER) stg[c] = pool[c];
    else pool[c] = stg[c];
  }
}

static int kv_move(bool gather, void* const* bases, const long long* layer_strides, const int* slabs, int n_tensors, int n_layers,
                   const void* pages, int n_pages, void* staging, cudaStream_t st) {
  if (n_tensors < 1 || n_tensors > KVMOVE_MAX_T || n_layers < 1 || n_pages < 0 || !pages || !staging) return OWL_ERR_BAD_ARG;
  if (n_pages == 0) return OWL_OK;
  KvMoveParams p = {};
  p.n_tensors = n_tensors; p.n_layers = n_layers; p.pages = (const int*)pages; p.staging = (uint8_t*)staging;
  for (int i = 0; i < n_tensors; ++i) {
    if (!bases[i] || (slabs[i] & 15) || slabs[i] <= 0 || (reinterpret_cast<uintptr_t>(bases[i]) & 15) || (layer_strides[i] & 15))
      return OWL_ERR_BAD_ARG;
    p.base[i] = (uint8_t*)bases[i]; p.layer_stride[i] = layer_strides[i]; p.slab[i] = slabs[i];
    p.page_bytes += (long long)n_layers * slabs[i];
  }
  if (reinterpret_cast<uintptr_t>(staging) & 15) return OWL_ERR_BAD_ARG;
  const dim3 grid(n_pages, n_layers * n_tensors);
  if (gather) kv_pages_move_kernel<true><<<grid, 256, 0, st>>>(p);
  else kv_pages_move_kernel<false><<<grid, 256, 0, st>>>(p);
  OWL_LAUNCH_CHECK();
  return OWL_OK;
}

}  // namespace owl
using namespace owl;

// bases / layer_strides / slabs: host arrays of n_tensors entries; pages: device int32 [n_pages] (a negative entry is
// skipped); staging: device bytes [n_pages][page_bytes], 16-byte aligned.
OWL_API int owl_kv_pages_gather(void* const* bases, const long long* layer_strides, const int* slabs, int n_tensors, int n_layers,
                                const void* pages, int n_pages, void* staging, cudaStream_t st) {
  return kv_move(true, bases, layer_strides, slabs, n_tensors, n_layers, pages, n_pages, staging, st);
}
OWL_API int owl_kv_pages_scatter(void* const* bases, const long long* layer_strides, const int* slabs, int n_tensors, int n_layers,
                                 const void* pages, int n_pages, const void* staging, cudaStream_t st) {
  return kv_move(false, bases, layer_strides, slabs, n_tensors, n_layers, pages, n_pages, const_cast<void*>(staging), st);
}
