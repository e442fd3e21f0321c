// Allocation-free entry point.  It has no counterpart in the reference library;
// it exists for callers of this library that are not allowed to, or cannot,
// allocate device memory.
#pragma once
#include "cx_common.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Size of the static device array the entry point below keeps its scratch in.
 * The array is part of the library's device code: the CUDA runtime sets it up on a
 * GPU when the entry point is first called there (see "first call" below), and
 * from then on that GPU holds these bytes until the process exits. */
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
 * The first call on a device is also the set-up: it asks the runtime for the
 * array's device address (once per device), and with lazy module loading that is
 * the moment the runtime places the array on the GPU.  Make that first call early
 * - a call with n = 0 and no targets does - before the surrounding runtime claims
 * the rest of the GPU's memory and before any stream capture is started.
 *
 * All calls share the one array per device.  It is cleared on the stream before
 * each use, but two calls whose kernels overlap on the GPU (different streams
 * without an ordering between them, or different host threads) race on it: keep
 * calls on one device ordered.
 *
 * Limits: vectors of 0 .. 2^31-1 elements, at most CX_MAX_PEERS targets.  Returns 0,
 * or a negative value with the reason in cx_last_error() when a limit is exceeded
 * (nothing is launched then). */
int cx_compress_noalloc(int gdtype, const void* g, float* r, int64_t n, const float* thr,
                        uint32_t cap, uint64_t seq, const CxTargets* tg, CxStats* stats,
                        uint32_t src_rank, void* stream);

#ifdef __cplusplus
}
#endif
