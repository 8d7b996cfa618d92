// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for this library's users.
//
// Who needs it: the engine gives nearly all free device memory to the key/value page pool when it
// starts, so a later cudaMalloc (the split-key partial results of nv_attention_decode are such a
// buffer, and torch's allocator falls back to cudaMalloc when its cache is empty) can fail or stall
// exactly when the server is busiest; and a host thread that drives the GPU from a latency-critical
// loop must not run into cudaMalloc / cudaFree, which synchronise the whole device.  Such callers
// pass only inputs and outputs; the partial results live in a fixed array inside the library.
//
//   * The array is file-scope device memory of NV_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU
//     that loads the library holds it from the load until the process exits.
//   * A call whose partial results would not fit — rows * Hq * splits * (D + 2) floats — is refused
//     with NV_ERR_NOALLOC_TOO_LARGE and launches nothing.  nv_attention_decode_noalloc_max_rows tells
//     how many rows fit for given sizes.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current) and keeps it; make that first call before any stream capture.  Later calls do
//     no set-up.  No call allocates or frees anything, on the device or through a library.
//   * All calls share the one array, and it keeps the last call's contents.  Nothing in it has to
//     start at zero: every slot a call reads was written by that call first.  Two calls that overlap
//     on the GPU (different streams, no ordering between them) race on the array; order them.
//   * The first call on a device must not run at the same time as another call on that device from
//     a second host thread (the address look-up is not guarded); once it has returned, calls may
//     come from any thread.
//   * What runs before it on the stream: like nv_attention_decode, the kernel is launched as a
//     programmatic dependent of the kernel before it and reads `positions`, `rows`, `row_entry`, the
//     block table and every page but each row's newest one before that kernel has finished.  So the
//     kernel directly before it on the stream may write nothing of these but the query rows and the
//     newest page of each row (this library's nv_rope_store over single rows is such a kernel).  If
//     the kernel before it writes older pages or the index arrays (nv_rope_store over a portion of
//     several tokens does), put any other kernel or an event between the two, or switch dependent
//     launches off with nv_set_dependent_launch(0).
//   * The status (below) stays set once a kernel has reported trouble, until the process ends.
#pragma once

#include <cuda_runtime.h>

#define NV_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define NV_ERR_NOALLOC_TOO_LARGE (-6)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as nv_attention_decode without `scratch` and the error flag (`num_pages`: pages in the
// caches, i.e. their first dimension); `splits` >= 1 as chosen by the caller
// (nv_attention_decode_splits gives the library's own choice).  Returns 0, a negative NV_ERR_* code or a
// cudaError_t.
int nv_attention_decode_noalloc(const void* qkv, int q_dt, int q_stride, const void* kc, const void* vc, int cache_dt,
                                const int* block_table, int max_blocks, const int* row_entry, const int* positions,
                                const int* rows, int R, float scale, int window, void* out, int out_dt, int Hq,
                                int Hkv, int D, int page, int num_pages, int splits, cudaStream_t stream);

// Largest number of rows one call can take for these sizes (0 if not even one fits, or if the kernel does not
// take the sizes at all: Hq or D not positive, D above 256 or no multiple of 8).
int nv_attention_decode_noalloc_max_rows(int Hq, int D, int splits);

// 0 while no kernel launched through this entry point has reported trouble on the current device (a block
// table without a page it needed, a copy that never arrived).  Reading it waits for the device; it is
// meant for tests and for diagnosis, not for the serving loop.
int nv_attention_decode_noalloc_status(void);

#ifdef __cplusplus
}
#endif
