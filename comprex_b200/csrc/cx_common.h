// Shared host/device types of the comprex_b200 native runtime.
//
// Everything that crosses the C ABI (ctypes on the Python side) is a plain C
// struct declared here.  The wire layout of a receive slot is
//
//   [CxHeader 64 B][table: nsub_max x {u32 start, u32 count}, padded to 16 B][pairs: cap x {i32 idx, f32 val}]
//
// for sparse payloads (the IndexPairs codec of the reference,
// src/compressor.hxx:539-661, plus one table entry per 1024-element sub-tile
// that says where the sub-tile's pairs sit in the pair list), and
//
//   [CxHeader 64 B][n x T]
//
// for dense payloads (GaspiEx / CompressorNone, src/gaspiEx.tpp:70-98).
// CxHeader::seq is the notification: it is written last with release
// semantics at system scope and polled with acquire semantics by the consumer.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CX_MAX_PEERS 16
#define CX_SUBTILE 1024   /* elements per table entry on the wire; one warp's unit of work */

/* device kinds */
#define CX_DEV_HOST 0
#define CX_DEV_CUDA 1

/* element types of user vectors */
#define CX_F32 0
#define CX_BF16 1
#define CX_F16 2

/* payload kinds */
#define CX_KIND_NONE 0
#define CX_KIND_PAIRS 1
#define CX_KIND_DENSE 2
#define CX_KIND_RLE 3
#define CX_KIND_ERROR 0xBAD

/* status bits (OR-ed into a status word the host reads after a sync) */
#define CX_OK 0u
#define CX_ST_TIMEOUT 1u
#define CX_ST_BAD_HEADER 2u
#define CX_ST_OVERFLOW 4u   /* soft: survivors beyond capacity stayed in the residual */
#define CX_ST_BAD_INDEX 8u

/* apply ops */
#define CX_OP_ADD 0       /* out += scale * sum(payloads)                         */
#define CX_OP_SET 1       /* out  = scale * sum(payloads), zero elsewhere          */
#define CX_OP_SGD 2       /* w = (1-wd)*w - scale*sum                              */
#define CX_OP_MOMENTUM 3  /* mom = mu*mom + lr*scale*sum ; w = (1-wd)*w - mom      */
#define CX_OP_ADAMW 4     /* g = scale*sum ; decoupled-weight-decay Adam           */

typedef struct CxHeader {
  uint64_t seq;        /* notification, written last                      */
  uint64_t bytes;      /* payload bytes in the reference's sense           */
  uint32_t n;          /* dense length of the vector                        */
  uint32_t nnz;        /* pairs stored (<= capacity)                        */
  uint32_t nnz_found;  /* survivors found (> nnz when capacity was hit)     */
  uint32_t kind;
  float threshold;
  uint32_t nsub;
  uint32_t src_rank;
  uint32_t dtype;
  uint32_t pad[4];
} CxHeader;

typedef struct CxPair {
  int32_t idx;
  uint32_t val;  /* bit pattern of the f32 (or i32) value */
} CxPair;

typedef struct CxEndpoint {
  CxHeader* hdr;
  uint32_t* table;  /* 2 words per sub-tile: start, count */
  CxPair* pairs;  /* for dense slots: start of the n x T data region */
} CxEndpoint;

/* CxTargets::pad flag: ep[count] is the multicast alias of the targets' slots (the same block on
 * every rank, mapped through an NVSwitch multicast object).  Kernels then store payload data
 * once with multimem.st instead of once per target; headers and notifications stay per target.
 * CUDA only; needs count < CX_MAX_PEERS. */
#define CX_TG_MULTICAST 1

typedef struct CxTargets {
  int32_t count;
  int32_t pad;   /* flags: CX_TG_MULTICAST */
  CxEndpoint ep[CX_MAX_PEERS];
} CxTargets;

typedef struct CxSources {
  int32_t count;
  int32_t pad;   /* dense reduce: position of the own vector among the operands (0 = first) */
  CxEndpoint ep[CX_MAX_PEERS];
  uint64_t seq[CX_MAX_PEERS];  /* wait until hdr->seq >= seq[j] */
  uint32_t cap[CX_MAX_PEERS];  /* pair capacity of slot j: no table entry may point beyond it */
} CxSources;

/* scratch of one sender: zero-initialised, reset by the kernel that used it */
#define CX_MAX_REGIONS 32
typedef struct CxWorkCounters {
  uint32_t done;                        /* CTAs that finished                          */
  uint32_t pad[31];
  uint32_t region[CX_MAX_REGIONS][32];  /* pairs reserved per region, one 128-byte line each */
} CxWorkCounters;

/* per-call statistics a kernel leaves behind (device or pinned memory) */
typedef struct CxStats {
  uint32_t n;
  uint32_t nnz;
  uint32_t nnz_found;
  uint32_t status;
  float threshold;
  uint32_t pad[3];
} CxStats;

typedef struct CxApplyArgs {
  int32_t op;
  int32_t out_dtype;   /* CX_F32 / CX_BF16 / CX_F16 for ADD and SET */
  void* out;           /* destination or f32 master weights            */
  void* shadow;        /* optional low-precision copy of the weights   */
  int32_t shadow_dtype;
  int32_t pad;
  float* m;
  float* v;
  float scale;
  float lr;
  float beta1;
  float beta2;
  float eps;
  float wd;
  float bc1;           /* 1 - beta1^t */
  float bc2;           /* 1 - beta2^t */
  float momentum;
  float pad2;
} CxApplyArgs;

/* ---- exported C ABI ------------------------------------------------- */

const char* cx_last_error(void);
uint64_t cx_launch_count(void);
void cx_reset_launch_count(void);
int cx_version(void);

/* bytes of scratch a compressor over n elements needs */
int64_t cx_workspace_bytes(int64_t n);

/* ThresholdTopK (src/threshold.hxx:127-242): writes |x|-threshold of the
 * strided sample of (r + g) (either may be NULL) to *thr_out (device memory
 * on CUDA). */
int cx_threshold_topk(int dev, int gdtype, const void* g, const float* r,
                      int64_t n, float ratio, int default_subsamples,
                      float subsample_factor, float* thr_out, void* stream);

/* The same with scratch (cx_threshold_workspace_bytes, zeroed once, left zeroed): when sampling
 * is switched off (every element is a sample, e.g. default_subsamples = 2^31 - 128) the CUDA
 * back end then selects over the whole vector with grid-wide radix passes instead of one CTA. */
int64_t cx_threshold_workspace_bytes(void);
int cx_threshold_select(int dev, int gdtype, const void* g, const float* r, int64_t n, float ratio,
                        int default_subsamples, float subsample_factor, float* thr_out, void* workspace,
                        int64_t ws_bytes, void* stream);

/* IndexPairs compress_add_update / compress_update / compress
 * (src/compressor.hxx:556-611) fused with the transfer: survivors are
 * stored into every target slot, the residual is updated in the same pass,
 * the notification is published by the last CTA. */
int cx_compress(int dev, int gdtype, const void* g, float* r, int64_t n,
                const float* thr, uint32_t cap, uint64_t seq,
                const CxTargets* tg, void* workspace, int64_t ws_bytes,
                CxStats* stats, uint32_t src_rank, void* stream);

/* IndexPairs decompress / add (src/compressor.hxx:613-658) fused with the
 * wait, the averaging and the parameter update. */
int cx_apply(int dev, const CxSources* src, int64_t n, const CxApplyArgs* a,
             uint32_t* status, uint64_t timeout_ns, void* stream);

/* The same update rules on a dense averaged gradient g (fp32): what follows a dense allreduce,
 * and the whole step of a single rank (keras/comprex_optimizer.py:150-163).  a->scale
 * multiplies g; a->op is CX_OP_SGD, CX_OP_MOMENTUM or CX_OP_ADAMW. */
int cx_update_dense(int dev, const float* g, int64_t n, const CxApplyArgs* a, void* stream);

/* copy a received sparse slot verbatim into other slots (forward_buffer /
 * readRemote_forward, src/comprEx.tpp:248-301); counters: one zeroed
 * CxWorkCounters in device memory */
int cx_forward(int dev, const CxEndpoint* from, uint64_t expect_seq,
               const CxTargets* tg, uint64_t seq, uint32_t cap, void* counters,
               uint32_t* status, uint64_t timeout_ns, void* stream);

/* dense p2p (src/gaspiEx.tpp:70-119; CompressorNone src/compressor.hxx:84-151).
 * With starts/lens, target k receives g[starts[k] .. starts[k]+lens[k]). */
int cx_dense_send(int dev, int dtype, const void* g, float* r, int64_t n,
                  uint64_t seq, const CxTargets* tg, const int64_t* starts,
                  const int64_t* lens, void* counters, uint32_t src_rank,
                  void* stream);
/* out = scale * (own? + sum over sources, in source order); optional push of
 * the result into further slots (chief broadcast / two-shot second phase).
 * With starts/lens (gather mode) source j is copied to out[starts[j]..). */
int cx_dense_reduce(int dev, int dtype, void* out, const void* own, int64_t n,
                    const CxSources* src, float scale, const CxTargets* push,
                    uint64_t push_seq, const int64_t* starts,
                    const int64_t* lens, void* counters, uint32_t src_rank,
                    uint32_t* status, uint64_t timeout_ns, void* stream);

/* Barrier over the symmetric heap (src/gaspiEnvironment.tpp:33-35): rank `rank` stores `seq` into
 * its cell of every rank's flag block (flag_ptrs[r]: CX_MAX_PEERS x 8 bytes, zeroed once, the same
 * heap offset on every rank) and waits, bounded, for all cells of its own block.  `seq` must grow
 * from call to call.  On CUDA one small kernel on `stream`; a wait that runs out sets CX_ST_TIMEOUT. */
int cx_barrier(int dev, int rank, int ranks, void* const* flag_ptrs, uint64_t seq, uint32_t* status,
               uint64_t timeout_ns, void* stream);

/* Dense allreduce through the switch (multimem.ld_reduce + multimem.st), one kernel per rank;
 * CUDA only.  `stage` is this rank's block of the symmetric heap and `stage_mc` its multicast
 * alias; with in == NULL the vector (n elements, a multiple of 16 bytes) lives in the block
 * itself and nothing is copied, otherwise `in` is copied in and the sum written to `out`.
 * one_shot: every rank pulls the whole sum itself (small vectors); the block then holds two
 * copies `stage_stride` bytes apart, used alternately.  slab_bytes: pipeline granularity
 * (<= 0: one slab).  flag_ptrs[r]: rank r's flag block (cx_mm_flag_bytes, zeroed once, same
 * offset of the symmetric heap on every rank); counters: local scratch (cx_mm_counter_bytes,
 * zeroed once).  The result is `scale` times the sum, identical bits on every rank. */
int64_t cx_mm_flag_bytes(void);
int64_t cx_mm_counter_bytes(void);
int cx_mm_allreduce(int dtype, void* out, const void* in, void* stage, void* stage_mc,
                    int64_t stage_stride, int64_t n, int rank, int ranks, float scale, int one_shot,
                    int64_t slab_bytes, uint64_t seq, void* const* flag_ptrs, void* counters,
                    uint32_t* status, uint64_t timeout_ns, void* stream);

/* Optimizer fold (keras/comprex_optimizer.py:101-115): per-tensor L2 clip to `clip`
 * (<= 0: off) and u = mu*u + lr*coef*g, read straight from the gradient tensors
 * (seg_ptr, one pointer per tensor) into the flat fp32 vector u.  The item arrays
 * describe the tensors in pieces of at most 65536 elements; all arrays live on `dev`. */
int cx_fold(int dev, int gdtype, const void* const* seg_ptr, const int64_t* item_off,
            const int64_t* item_rel, const int32_t* item_len, const int32_t* item_seg,
            const int32_t* seg_first, int nitems, float* u, float* partial, float clip,
            float mu, float lr, void* stream);

/* small elementwise helpers of the engines and the optimizer */
int cx_axpy(int dev, int ydtype, void* y, int xdtype, const void* x, float a,
            int64_t n, void* stream); /* y += a*x */
int cx_fill_zero(int dev, void* p, int64_t bytes, void* stream);

/* RLE codec (corrected restatement of src/compressor.hxx:159-532), host */
int64_t cx_rle_compress_host(const float* g, float* r, int64_t n, float thr,
                             void* out, int64_t out_bytes);
int cx_rle_decode_host(const void* in, int64_t in_bytes, float* out, int64_t n,
                       int add);
/* RLE fused with the transfer: the payload (same byte layout as the host codec) is stored
 * into every target's slot and released with `seq`; the receiver waits (bounded), checks the
 * runs and expands.  thr points to device memory on CUDA.  slot_bytes is the payload room of
 * a slot (>= cx_rle_slot_bytes(n)); the workspace (>= cx_rle_workspace_bytes(n), zeroed once)
 * is rank-local scratch.  A payload that fails a check sets CX_ST_BAD_HEADER and leaves `out`
 * as it was. */
int64_t cx_rle_slot_bytes(int64_t n);
int64_t cx_rle_workspace_bytes(int64_t n);
int cx_rle_send(int dev, int gdtype, const void* g, float* r, int64_t n, const float* thr,
                int64_t slot_bytes, uint64_t seq, const CxTargets* tg, void* workspace,
                int64_t ws_bytes, uint32_t src_rank, void* stream);
int cx_rle_recv(int dev, const CxEndpoint* src, uint64_t expect_seq, float* out, int64_t n,
                int add, int64_t slot_bytes, void* workspace, int64_t ws_bytes,
                uint32_t* status, uint64_t timeout_ns, void* stream);

/* ---- runtime: heaps ---------------------------------------------------- */
int cx_cuda_device_count(void);
int cx_cuda_set_device(int dev);
void* cx_cuda_malloc(int64_t bytes);
int cx_cuda_free(void* p);
int cx_cuda_ipc_get(void* p, void* handle64);            /* 64-byte handle out */
void* cx_cuda_ipc_open(const void* handle64);
int cx_cuda_ipc_close(void* p);
int cx_cuda_can_access_peer(int dev, int peer);
void* cx_pinned_alloc(int64_t bytes, void** device_ptr); /* mapped host memory */
int cx_pinned_free(void* p);
int cx_cuda_stream_sync(void* stream);
int cx_cuda_memcpy(void* dst, const void* src, int64_t bytes, int kind, void* stream);

void* cx_shm_create(const char* name, int64_t bytes);    /* host ranks */
void* cx_shm_open(const char* name, int64_t bytes);
int cx_shm_close(void* p, int64_t bytes);
int cx_shm_unlink(const char* name);
void* cx_host_alloc(int64_t bytes);
int cx_host_free(void* p);

/* ---- op lists ------------------------------------------------------------
 * A collective is a short, fixed sequence of the launches above.  The caller
 * describes it once as an array of CxOp and afterwards runs the whole
 * sequence with one call per step; only the sequence number (and, when the
 * user's buffer moved, a few pointers) change between steps. */
#define CX_OPK_THRESHOLD 1
#define CX_OPK_COMPRESS 2
#define CX_OPK_APPLY 3
#define CX_OPK_DENSE_SEND 4
#define CX_OPK_DENSE_REDUCE 5
#define CX_OPK_UPDATE 6        /* cx_update_dense: g, n, apply */
#define CX_OPK_MM_ALLREDUCE 7  /* cx_mm_allreduce: out, own (= in), g (= stage), r (= stage_mc), starts[0] = stride,
                                  starts[1] = one_shot, starts[2] = slab bytes, lens[r] = rank r's flag block,
                                  src_rank, cap (= ranks), workspace (= counters), scale, status */

typedef struct CxOp {
  int32_t kind;
  int32_t dev;
  int32_t dtype;               /* element type of g (threshold, compress) or of the dense vector */
  int32_t has_ranges;          /* dense send / gather: starts and lens are valid */
  const void* g;               /* input vector (may be NULL for compress_update) */
  float* r;                    /* residual (may be NULL) */
  int64_t n;
  float ratio;                 /* threshold */
  int32_t default_subsamples;
  float subsample_factor;
  float scale;                 /* dense reduce */
  float* thr;                  /* device cell: written by threshold, read by compress */
  uint32_t cap;
  uint32_t src_rank;
  void* workspace;             /* compress scratch / dense counters */
  int64_t ws_bytes;
  CxStats* stats;
  void* out;                   /* dense reduce destination */
  const void* own;             /* dense reduce: first operand (may be NULL) */
  uint32_t* status;
  uint64_t timeout_ns;
  int32_t has_push;
  int32_t lane;                /* 0: the caller's stream; k > 0: side stream k (see cx_run_ops) */
  int64_t starts[CX_MAX_PEERS];
  int64_t lens[CX_MAX_PEERS];
  CxTargets tg;                /* compress / dense send targets, dense reduce push targets */
  CxSources src;               /* apply / dense reduce sources; their seq is set per call */
  CxApplyArgs apply;
} CxOp;

/* Runs ops[0..count) on `stream`; every notification written or waited for uses sequence
 * number `seq`.  Stops at the first failing launch.
 * Ops with lane 0 run on `stream` in order.  Ops with lane k > 0 (CUDA only, k <= CX_MAX_LANES)
 * run on an internal side stream k, in order among themselves and concurrently with the other
 * lanes: a side stream starts behind everything queued on `stream` before its first op, and the
 * next lane-0 op (or the end of the list) waits for all side streams.  Independent small
 * launches (the per-chunk compressions of a ring) then overlap instead of queueing up. */
#define CX_MAX_LANES 16
int cx_run_ops(CxOp* ops, int count, uint64_t seq, void* stream);
/* The same sequence captured as a CUDA graph (CUDA ops only): built once, then one small copy
 * (the sequence number, into a device cell the kernels read) and one graph launch per replay.
 * The ops' pointers and parameters are frozen at build time. */
int cx_graph_build(CxOp* ops, int count, void** graph_out);
int cx_graph_launch(void* graph, uint64_t seq, void* stream);
int cx_graph_free(void* graph);
int64_t cx_sizeof(int what); /* 0 CxOp, 1 CxSources, 2 CxTargets, 3 CxApplyArgs, 4 CxWorkCounters, 5 CxHeader */

/* bounded wait on a header from the host (status in the return value) */
int cx_host_wait_seq(const CxHeader* hdr, uint64_t seq, uint64_t timeout_ns);

#ifdef __cplusplus
}
#endif
