// Split decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in tamnd/fastmlx; it exists for embedders of this
// library.  fmx_attn_decode (attention_bf16.cu) needs a workspace for the per-split partial
// results and expects its caller to provide one.  Some callers cannot: code that runs
// while a stream is being captured into a CUDA graph, code that runs under a memory pool
// it must not disturb, plug-ins handed raw pointers by a host program that owns every
// allocation.  For them the library carries the workspace itself, as a fixed array in
// device memory that is part of the loaded module.
//
// What that means for the caller:
//   * The array holds FMX_ATTN_NOALLOC_MAX_FLOATS floats (4 MiB).  Every GPU on which this
//     library is loaded holds that much until the process exits, used or not.
//   * A call needs rows * nkv * splits * 16 * (head_dim + 2) floats when splits > 1 and
//     nothing when splits == 1.  A call that needs more than the array holds is refused
//     with an error text; nothing is launched.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and sets the kernels' shared-memory
//     limit.  Make that first call outside any stream capture: a first call on a capturing
//     stream is refused with an error text.  The set-up is guarded by a lock, so two
//     threads may race to be first.
//   * Any number of splits fits that the array has room for.  (fmx_attn_decode stops at 64
//     because there the last block of a row combines the splits through shared memory; this
//     entry always combines in a second kernel, which walks the splits in a loop.)
//   * The entry point calls no cudaMalloc, cudaFree or allocating library routine.
//   * All calls share the one array and it keeps whatever the last call left in it.  The
//     kernels write every partial before the combine step reads it, so nothing has to be
//     cleared between calls; but two calls that overlap on the GPU (different streams, or
//     graphs replayed concurrently) race on it.  Run them on one stream, or otherwise in
//     order.
//
// Arguments are those of fmx_attn_decode without the workspace: the caller still passes
// inputs (queries, cache, block tables, row starts, positions) and the output.
#pragma once
#include <cuda_runtime.h>

#define FMX_ATTN_NOALLOC_MAX_FLOATS (1 << 20)

extern "C" {
// Returns 0, or non-zero after leaving a message for fmx_last_error().
int fmx_attn_decode_noalloc(const void* q, long long q_stride, const void* kv, const int* block_tables, int bt_stride,
                            const int* row_start, const int* positions, void* out, int rows, int splits, int nh,
                            int nkv, int page_size, long long num_pages, float scale, int window, int* status,
                            cudaStream_t stream);
// Floats the call above needs for these sizes (0 when splits <= 1), and the most it can have.
long long fmx_attn_decode_noalloc_floats(int rows, int nkv, int splits);
long long fmx_attn_decode_noalloc_max_floats(void);
}
