// C ABI of the native collectives (csrc/collectives.cpp): a communicator over the symmetric
// heap and the six allreduce schedules of the reference (include/allreduce.hxx:15-211), callable
// from C or C++ without Python, plus the reference's own C names (src/GPI_C.cpp:44-73,
// src/allreduce_C.cpp:12-122).
#pragma once
#include "cx_common.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CxComm CxComm;
typedef struct CxAllreduce CxAllreduce;

/* kinds, numbered like the reference's benchmark selects them (examples/allreduce_speed.cpp:17-19) */
#define CX_AR_ALLTOONE 0
#define CX_AR_COMPREX_ALLTOONE 1
#define CX_AR_RING 2
#define CX_AR_COMPREX_RING 3
#define CX_AR_BIGRING 4
#define CX_AR_COMPREX_BIGRING 5

/* flags of cx_allreduce_create */
#define CX_AR_CONSISTENT 1      /* every rank, the sender included, applies only what was transmitted */
#define CX_AR_OWNER_RESIDUAL 2  /* compressed Ring: the owner keeps what its broadcast did not carry */
#define CX_AR_ALIGNED_CHUNKS 4  /* compressed Ring: chunks are multiples of 4 elements (16-byte accesses) */

/* A communicator over a heap the caller has already mapped: bases[r] is rank r's segment in this
 * process' address space (bases[rank] is local), mc_base its multicast alias or NULL.  Collective
 * objects carve their slots out of the heap in creation order, which must be the same on every rank. */
CxComm* cx_comm_create(int dev, int device, int rank, int ranks, void* const* bases, void* mc_base,
                       int64_t bytes, uint64_t timeout_ns);
/* The ranks of one host meet through a POSIX shared-memory block named after `job`: GPU ranks
 * exchange CUDA IPC handles of their segments, host ranks map each other's shared memory. */
CxComm* cx_comm_bootstrap(const char* job, int rank, int ranks, int dev, int device, int64_t bytes,
                          uint64_t timeout_ns);
int cx_comm_barrier(CxComm* c);               /* bootstrap communicators; bounded wait */
int cx_comm_sync(CxComm* c, void* stream);    /* wait for this rank's queued work */
uint32_t cx_comm_check(CxComm* c);            /* status bits kernels left behind (CX_ST_*), cleared */
int cx_comm_rank(const CxComm* c);
int cx_comm_ranks(const CxComm* c);
void cx_comm_destroy(CxComm* c);

/* Collective.  ratio / size_factor: compressed kinds; chief: AllToOne kinds. */
CxAllreduce* cx_allreduce_create(CxComm* c, int kind, int64_t size, int dtype, float ratio, float size_factor,
                                 int chief, int flags);
int cx_allreduce_apply(CxAllreduce* ar, void* data, void* stream);   /* in place, asynchronous on `stream` */
int cx_allreduce_flush(CxAllreduce* ar, void* data, void* stream);   /* drain the residuals into data */
int cx_allreduce_reset(CxAllreduce* ar);
int cx_allreduce_set_ratio(CxAllreduce* ar, float ratio);
void cx_allreduce_set_scale(CxAllreduce* ar, float scale);           /* dense kinds: result = scale * sum */
int64_t cx_allreduce_size(const CxAllreduce* ar);
/* checkpoint: the residual (size floats, host memory) and the step counter */
int cx_allreduce_state(CxAllreduce* ar, float* residual_out, int64_t n, uint64_t* step);
int cx_allreduce_load_state(CxAllreduce* ar, const float* residual, int64_t n, uint64_t step);
int cx_allreduce_stats(CxAllreduce* ar, CxStats* out);               /* this rank's last compression */
void cx_allreduce_destroy(CxAllreduce* ar);

#ifdef __cplusplus
}
#endif
