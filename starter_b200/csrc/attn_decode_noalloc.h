// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference engine: it is an addition of this
// library.  Some callers of the kernels cannot call cudaMalloc (or any routine that does so
// behind their back, torch's allocator included): code that runs inside a framework's own
// memory plan, a plugin that is handed its buffers and nothing else, a process whose device
// memory is fully accounted for before it starts.  The split-key decode attention kernel
// needs scratch memory for the partial results of its splits and for one counter per
// (sequence, kv head); sb_attn_decode takes that scratch from the caller, who has to
// allocate it.  sb_attn_decode_noalloc runs the same kernel with the scratch in a fixed
// array that is part of the library's image on the device, so the caller passes only inputs
// and outputs.
//
// Limits and rules:
//  * The array holds SB_NOALLOC_MAX_COUNTERS counters and SB_NOALLOC_MAX_FLOATS floats of partial
//    results (16 MiB + 16 KiB).  Every GPU that loads the library holds that much until the
//    process exits.  A call needs n_seqs * n_kv_heads counters and, when n_splits > 8 (up to 8 splits
//    merge through shared memory and use no scratch),
//    n_seqs * n_heads * n_splits * (head_dim + 2) floats; a call that needs more is refused
//    with SB_NOALLOC_TOO_LARGE and sb_attn_decode_noalloc_error() says what was asked for.
//  * The first call on a device (with that device current) looks the array's address on that
//    device up (cudaGetSymbolAddress) and sets the kernel's shared-memory limit there; both are
//    remembered per device.  Make that first call before any stream capture begins on that device.
//  * More splits than the merge step has shared memory for (two floats per split and query head of
//    a group: 384 splits at 16 heads per kv head and head size 64) are refused with SB_NOALLOC_TOO_LARGE.
//  * All calls share the one array, and it keeps whatever the last call left in it.  The
//    entry point clears the counters on the given stream before each launch; the partial
//    results need no clearing (every value read was written by the same launch).  Two calls
//    whose kernels can overlap on the GPU (different streams, no dependency) race on the
//    array: order them.
//  * It calls no cudaMalloc, no cudaFree and no library routine that allocates.
#pragma once

#include <cuda_runtime.h>

#include "common.cuh"

#define SB_NOALLOC_MAX_COUNTERS 4096
#define SB_NOALLOC_MAX_FLOATS (4 * 1024 * 1024)
#define SB_NOALLOC_TOO_LARGE (-1)
#define SB_NOALLOC_SETUP_FAILED (-2)

extern "C" {

// Same arguments and result as sb_attn_decode, minus the scratch pointers.  Returns 0, a CUDA error
// code (> 0), or one of the negative codes above.
int sb_attn_decode_noalloc(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window,
                           int n_splits, cudaStream_t stream);

// Text of the last negative result on the calling thread ("" if there was none).
const char* sb_attn_decode_noalloc_error(void);

// For tests and debuggers: the array's address on the current device (counters first, then the partial
// results), or null before the first call there.  Not needed to use the entry point.
void* sb_attn_decode_noalloc_scratch(void);

}
