/* Allocation-free entry point of the kernel library.
 *
 * This entry point has no counterpart in the reference engine. It exists for callers that must
 * not (or cannot) allocate device memory when they need a token picked: code running inside a
 * memory budget that is already fully committed (the engine declares its VRAM budget at boot and
 * ledgers every block), code on a latency path where cudaMalloc's implicit device synchronisation
 * is unacceptable, and hosts embedding the library through the C ABI that own no allocator the
 * kernels could borrow from (no torch, no pool). Such callers pass only their inputs and outputs.
 *
 * owl_argmax_noalloc is the greedy-sampling argmax (same two-stage kernels as owl_argmax) with its
 * partial-result scratch held in a fixed array inside the library image instead of caller memory.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Limits of the built-in scratch (64 partitions per row, float + int per partition = 16 KB). */
#define OWL_NOALLOC_MAX_ROWS 32

/* out_idx[row] = vocab_offset + argmax over logits[row][0..V) (bf16, row stride ld elements);
 * ties go to the lowest index.
 *
 * - Calls no cudaMalloc / cudaFree / allocating routine. Every GPU that loads the library holds
 *   the 16 KB scratch array until the process exits.
 * - The first call on a device resolves the array's device address (once per device, with that
 *   device current); make that first call outside of any stream capture.
 * - rows > OWL_NOALLOC_MAX_ROWS, rows < 1, V < 1 or ld < V are rejected with -1 and nothing is
 *   launched; a CUDA error while resolving the scratch address or launching returns <= -2000.
 * - All calls share the one scratch array (it keeps the previous call's partials; nothing in it
 *   has to start at zero because stage 1 rewrites every slot stage 2 reads). Two calls whose
 *   kernels can overlap on the GPU (different streams, no ordering) race on it: order them.
 */
int owl_argmax_noalloc(const void* logits_bf16, int rows, int V, int ld, void* out_idx_i32, int vocab_offset,
                       cudaStream_t stream);

#ifdef __cplusplus
}
#endif
