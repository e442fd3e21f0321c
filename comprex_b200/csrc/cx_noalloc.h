// Allocation-free entry point.  It has no counterpart in the reference library;
// it exists for callers of this library that are not allowed to, or cannot,
// allocate device memory.
#pragma once
#include "cx_common.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Largest amount of scratch the entry point below can use: the size of the
 * static device array it owns.  Every GPU on which the library is loaded keeps
 * this much memory until the process exits. */
#define CX_NOALLOC_SCRATCH_BYTES 8192

/* Same operation as cx_compress() on a CUDA device (r += g, select |r| > *thr,
 * store the pairs into every target slot, zero what was sent, publish seq), for
 * callers that must not allocate: a component that lives inside another
 * runtime which has already claimed the whole GPU for its own memory pool (any
 * cudaMalloc then fails), or a step loop whose rules forbid allocation once it
 * is running.  cx_compress() wants a scratch buffer from its caller; this
 * variant uses a static array in device memory instead and calls neither
 * cudaMalloc nor cudaFree nor any routine that allocates.
 *
 * g, r, thr, the target slots and stats are the caller's, exactly as for
 * cx_compress(); the device that owns them must be the current device and
 * `stream` must belong to it.
 *
 * The first call on a device looks the array's address up (once per device) and
 * should therefore be made before any stream capture is started.
 *
 * All calls share the one array per device.  It is cleared on the stream before
 * each use, but two calls whose kernels overlap on the GPU (different streams
 * without an ordering between them, or different host threads) race on it: keep
 * calls on one device ordered.
 *
 * Returns 0, or a negative value with the reason in cx_last_error(): n outside
 * 0 .. 2^31-1, more than CX_MAX_PEERS targets, or a vector whose scratch need,
 * cx_workspace_bytes(n), is larger than CX_NOALLOC_SCRATCH_BYTES. */
int cx_compress_noalloc(int gdtype, const void* g, float* r, int64_t n, const float* thr,
                        uint32_t cap, uint64_t seq, const CxTargets* tg, CxStats* stats,
                        uint32_t src_rank, void* stream);

#ifdef __cplusplus
}
#endif
