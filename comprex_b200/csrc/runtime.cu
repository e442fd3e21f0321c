// C ABI of the native runtime: error reporting, launch accounting, the
// host/CUDA dispatch of every primitive, and the memory runtime that stands in
// for the reference's GASPI segment (include/gaspiEnvironment.hxx:9-28):
// device segments shared between processes through CUDA IPC handles, POSIX
// shared-memory segments for host ranks, and pinned mapped memory for the
// status words kernels write and the host reads without a copy.
#include <cuda_runtime.h>
#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <mutex>

#include "cx_common.h"

// ---- forward declarations of the two back ends --------------------------------
int cx_threshold_topk_cuda(int, const void*, const float*, int64_t, float, int, float, float*, void*, int64_t, void*);
int cx_threshold_topk_host(int, const void*, const float*, int64_t, float, int, float, float*);
int cx_compress_cuda(int, const void*, float*, int64_t, const float*, uint32_t, uint64_t,
                     const CxTargets*, void*, int64_t, CxStats*, uint32_t, void*);
int cx_compress_host(int, const void*, float*, int64_t, const float*, uint32_t, uint64_t,
                     const CxTargets*, CxStats*, uint32_t);
int cx_apply_cuda(const CxSources*, int64_t, const CxApplyArgs*, uint32_t*, uint64_t, void*);
int cx_apply_host(const CxSources*, int64_t, const CxApplyArgs*, uint32_t*, uint64_t);
int cx_forward_cuda(const CxEndpoint*, uint64_t, const CxTargets*, uint64_t, uint32_t, void*,
                    uint32_t*, uint64_t, void*);
int cx_forward_host(const CxEndpoint*, uint64_t, const CxTargets*, uint64_t, uint32_t, uint32_t*,
                    uint64_t);
int cx_dense_send_cuda(int, const void*, float*, int64_t, uint64_t, const CxTargets*, const int64_t*,
                       const int64_t*, void*, uint32_t, void*);
int cx_dense_send_host(int, const void*, float*, int64_t, uint64_t, const CxTargets*, const int64_t*,
                       const int64_t*, uint32_t);
int cx_dense_reduce_cuda(int, void*, const void*, int64_t, const CxSources*, float, const CxTargets*,
                         uint64_t, const int64_t*, const int64_t*, void*, uint32_t, uint32_t*,
                         uint64_t, void*);
int cx_dense_reduce_host(int, void*, const void*, int64_t, const CxSources*, float, const CxTargets*,
                         uint64_t, const int64_t*, const int64_t*, uint32_t, uint32_t*, uint64_t);
int cx_axpy_cuda(int, void*, int, const void*, float, int64_t, void*);
int cx_rle_send_cuda(int, const void*, float*, int64_t, const float*, int64_t, uint64_t, const CxTargets*,
                     void*, int64_t, uint32_t, void*);
int cx_rle_send_host(int, const void*, float*, int64_t, const float*, int64_t, uint64_t, const CxTargets*,
                     uint32_t);
int cx_rle_recv_cuda(const CxEndpoint*, uint64_t, float*, int64_t, int, int64_t, void*, int64_t, uint32_t*,
                     uint64_t, void*);
int cx_rle_recv_host(const CxEndpoint*, uint64_t, float*, int64_t, int, int64_t, uint32_t*, uint64_t);
int cx_fold_cuda(int, const void* const*, const int64_t*, const int64_t*, const int32_t*, const int32_t*,
                 const int32_t*, int, float*, float*, float, float, float, void*);
int cx_fold_host(int, const void* const*, const int64_t*, const int64_t*, const int32_t*, const int32_t*,
                 const int32_t*, int, float*, float*, float, float, float);
int cx_axpy_host(int, void*, int, const void*, float, int64_t);
int cx_barrier_cuda(int, int, void* const*, uint64_t, uint32_t*, uint64_t, void*);
int cx_barrier_host(int, int, void* const*, uint64_t, uint32_t*, uint64_t);
int cx_update_dense_cuda(const float*, int64_t, const CxApplyArgs*, void*);
int cx_mm_allreduce_cuda(int, void*, const void*, void*, void*, int64_t, int64_t, int, int, float, int, int64_t,
                         uint64_t, void* const*, void*, uint32_t*, uint64_t, void*);
int cx_update_dense_host(const float*, int64_t, const CxApplyArgs*);

// ---- errors and accounting -------------------------------------------------------
static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

int cx_set_error(const char* where, int cuda_err) {
  if (cuda_err)
    snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString((cudaError_t)cuda_err));
  else
    snprintf(g_err, sizeof(g_err), "%s", where);
  return cuda_err ? -cuda_err : -1;
}
void cx_note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
static thread_local const uint64_t* g_seq_cell = nullptr;
const uint64_t* cx_seq_cell() { return g_seq_cell; }
int cx_check_launch(const char* where) {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cx_set_error(where, (int)e);
}
bool cx_pdl_enabled() {
  static const bool on = [] { const char* e = getenv("COMPREX_PDL"); return !(e && e[0] == '0'); }();
  return on;
}
int cx_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    sms[dev] = v;
  }
  return sms[dev];
}

extern "C" {

const char* cx_last_error(void) { return g_err; }
uint64_t cx_launch_count(void) { return g_launches.load(); }
void cx_reset_launch_count(void) { g_launches.store(0); }
int cx_version(void) { return 1; }

int cx_threshold_select(int dev, int gdtype, const void* g, const float* r, int64_t n, float ratio,
                        int default_subsamples, float subsample_factor, float* thr_out, void* workspace,
                        int64_t ws_bytes, void* stream) {
  return dev == CX_DEV_CUDA
             ? cx_threshold_topk_cuda(gdtype, g, r, n, ratio, default_subsamples, subsample_factor, thr_out,
                                      workspace, ws_bytes, stream)
             : cx_threshold_topk_host(gdtype, g, r, n, ratio, default_subsamples, subsample_factor, thr_out);
}

int cx_threshold_topk(int dev, int gdtype, const void* g, const float* r, int64_t n, float ratio,
                      int default_subsamples, float subsample_factor, float* thr_out, void* stream) {
  return cx_threshold_select(dev, gdtype, g, r, n, ratio, default_subsamples, subsample_factor, thr_out, nullptr, 0,
                             stream);
}

int cx_compress(int dev, int gdtype, const void* g, float* r, int64_t n, const float* thr,
                uint32_t cap, uint64_t seq, const CxTargets* tg, void* workspace, int64_t ws_bytes,
                CxStats* stats, uint32_t src_rank, void* stream) {
  return dev == CX_DEV_CUDA
             ? cx_compress_cuda(gdtype, g, r, n, thr, cap, seq, tg, workspace, ws_bytes, stats, src_rank, stream)
             : cx_compress_host(gdtype, g, r, n, thr, cap, seq, tg, stats, src_rank);
}

int cx_apply(int dev, const CxSources* src, int64_t n, const CxApplyArgs* a, uint32_t* status,
             uint64_t timeout_ns, void* stream) {
  return dev == CX_DEV_CUDA ? cx_apply_cuda(src, n, a, status, timeout_ns, stream)
                            : cx_apply_host(src, n, a, status, timeout_ns);
}

int cx_update_dense(int dev, const float* g, int64_t n, const CxApplyArgs* a, void* stream) {
  return dev == CX_DEV_CUDA ? cx_update_dense_cuda(g, n, a, stream) : cx_update_dense_host(g, n, a);
}

int cx_barrier(int dev, int rank, int ranks, void* const* flag_ptrs, uint64_t seq, uint32_t* status,
               uint64_t timeout_ns, void* stream) {
  return dev == CX_DEV_CUDA ? cx_barrier_cuda(rank, ranks, flag_ptrs, seq, status, timeout_ns, stream)
                            : cx_barrier_host(rank, ranks, flag_ptrs, seq, status, timeout_ns);
}

int cx_mm_allreduce(int dtype, void* out, const void* in, void* stage, void* stage_mc, int64_t stage_stride,
                    int64_t n, int rank, int ranks, float scale, int one_shot, int64_t slab_bytes, uint64_t seq,
                    void* const* flag_ptrs, void* counters, uint32_t* status, uint64_t timeout_ns, void* stream) {
  return cx_mm_allreduce_cuda(dtype, out, in, stage, stage_mc, stage_stride, n, rank, ranks, scale, one_shot,
                              slab_bytes, seq, flag_ptrs, counters, status, timeout_ns, stream);
}

int cx_forward(int dev, const CxEndpoint* from, uint64_t expect_seq, const CxTargets* tg,
               uint64_t seq, uint32_t cap, void* counters, uint32_t* status, uint64_t timeout_ns,
               void* stream) {
  return dev == CX_DEV_CUDA
             ? cx_forward_cuda(from, expect_seq, tg, seq, cap, counters, status, timeout_ns, stream)
             : cx_forward_host(from, expect_seq, tg, seq, cap, status, timeout_ns);
}

int cx_dense_send(int dev, int dtype, const void* g, float* r, int64_t n, uint64_t seq,
                  const CxTargets* tg, const int64_t* starts, const int64_t* lens, void* counters,
                  uint32_t src_rank, void* stream) {
  return dev == CX_DEV_CUDA
             ? cx_dense_send_cuda(dtype, g, r, n, seq, tg, starts, lens, counters, src_rank, stream)
             : cx_dense_send_host(dtype, g, r, n, seq, tg, starts, lens, src_rank);
}

int cx_dense_reduce(int dev, int dtype, void* out, const void* own, int64_t n, const CxSources* src,
                    float scale, const CxTargets* push, uint64_t push_seq, const int64_t* starts,
                    const int64_t* lens, void* counters, uint32_t src_rank, uint32_t* status,
                    uint64_t timeout_ns, void* stream) {
  return dev == CX_DEV_CUDA
             ? cx_dense_reduce_cuda(dtype, out, own, n, src, scale, push, push_seq, starts, lens,
                                    counters, src_rank, status, timeout_ns, stream)
             : cx_dense_reduce_host(dtype, out, own, n, src, scale, push, push_seq, starts, lens,
                                    src_rank, status, timeout_ns);
}

int cx_axpy(int dev, int ydtype, void* y, int xdtype, const void* x, float a, int64_t n, void* stream) {
  return dev == CX_DEV_CUDA ? cx_axpy_cuda(ydtype, y, xdtype, x, a, n, stream)
                            : cx_axpy_host(ydtype, y, xdtype, x, a, n);
}

int cx_fold(int dev, int gdtype, const void* const* seg_ptr, const int64_t* item_off,
            const int64_t* item_rel, const int32_t* item_len, const int32_t* item_seg,
            const int32_t* seg_first, int nitems, float* u, float* partial, float clip, float mu,
            float lr, void* stream) {
  return dev == CX_DEV_CUDA
             ? cx_fold_cuda(gdtype, seg_ptr, item_off, item_rel, item_len, item_seg, seg_first, nitems, u,
                            partial, clip, mu, lr, stream)
             : cx_fold_host(gdtype, seg_ptr, item_off, item_rel, item_len, item_seg, seg_first, nitems, u,
                            partial, clip, mu, lr);
}

int cx_rle_send(int dev, int gdtype, const void* g, float* r, int64_t n, const float* thr,
                int64_t slot_bytes, uint64_t seq, const CxTargets* tg, void* workspace,
                int64_t ws_bytes, uint32_t src_rank, void* stream) {
  return dev == CX_DEV_CUDA
             ? cx_rle_send_cuda(gdtype, g, r, n, thr, slot_bytes, seq, tg, workspace, ws_bytes, src_rank, stream)
             : cx_rle_send_host(gdtype, g, r, n, thr, slot_bytes, seq, tg, src_rank);
}

int cx_rle_recv(int dev, const CxEndpoint* src, uint64_t expect_seq, float* out, int64_t n, int add,
                int64_t slot_bytes, void* workspace, int64_t ws_bytes, uint32_t* status,
                uint64_t timeout_ns, void* stream) {
  return dev == CX_DEV_CUDA
             ? cx_rle_recv_cuda(src, expect_seq, out, n, add, slot_bytes, workspace, ws_bytes, status,
                                timeout_ns, stream)
             : cx_rle_recv_host(src, expect_seq, out, n, add, slot_bytes, status, timeout_ns);
}

/* struct sizes, so that the binding can verify its mirror of the layouts at load time */
int64_t cx_sizeof(int what) {
  switch (what) {
    case 0: return (int64_t)sizeof(CxOp);
    case 1: return (int64_t)sizeof(CxSources);
    case 2: return (int64_t)sizeof(CxTargets);
    case 3: return (int64_t)sizeof(CxApplyArgs);
    case 4: return (int64_t)sizeof(CxWorkCounters);
    case 5: return (int64_t)sizeof(CxHeader);
    default: return -1;
  }
}

// ---- launch sequences -------------------------------------------------------------------
namespace {

int run_one(CxOp& o, uint64_t seq, void* stream) {
  switch (o.kind) {
    case CX_OPK_THRESHOLD:
      return cx_threshold_select(o.dev, o.dtype, o.g, o.r, o.n, o.ratio, o.default_subsamples,
                                 o.subsample_factor, o.thr, o.workspace, o.ws_bytes, stream);
    case CX_OPK_COMPRESS:
      return cx_compress(o.dev, o.dtype, o.g, o.r, o.n, o.thr, o.cap, seq, &o.tg, o.workspace,
                         o.ws_bytes, o.stats, o.src_rank, stream);
    case CX_OPK_APPLY:
      for (int j = 0; j < o.src.count; ++j) o.src.seq[j] = seq;
      return cx_apply(o.dev, &o.src, o.n, &o.apply, o.status, o.timeout_ns, stream);
    case CX_OPK_DENSE_SEND:
      return cx_dense_send(o.dev, o.dtype, o.g, o.r, o.n, seq, &o.tg, o.has_ranges ? o.starts : nullptr,
                           o.has_ranges ? o.lens : nullptr, o.workspace, o.src_rank, stream);
    case CX_OPK_DENSE_REDUCE:
      for (int j = 0; j < o.src.count; ++j) o.src.seq[j] = seq;
      return cx_dense_reduce(o.dev, o.dtype, o.out, o.own, o.n, &o.src, o.scale,
                             o.has_push ? &o.tg : nullptr, seq, o.has_ranges ? o.starts : nullptr,
                             o.has_ranges ? o.lens : nullptr, o.workspace, o.src_rank, o.status,
                             o.timeout_ns, stream);
    case CX_OPK_MM_ALLREDUCE: {
      void* flags[CX_MAX_PEERS];
      for (int r = 0; r < CX_MAX_PEERS; ++r) flags[r] = reinterpret_cast<void*>(o.lens[r]);
      return cx_mm_allreduce(o.dtype, o.out, o.own, const_cast<void*>(o.g), o.r, o.starts[0], o.n, (int)o.src_rank,
                             (int)o.cap, o.scale, (int)o.starts[1], o.starts[2], seq, flags, o.workspace, o.status,
                             o.timeout_ns, stream);
    }
    case CX_OPK_UPDATE:
      return cx_update_dense(o.dev, reinterpret_cast<const float*>(o.g), o.n, &o.apply, stream);
    default:
      return cx_set_error("cx_run_ops: unknown op kind", 0);
  }
}

// side streams and their events, one set per device, created on first use
struct Lanes {
  cudaStream_t stream[CX_MAX_LANES + 1];
  cudaEvent_t done[CX_MAX_LANES + 1];
  cudaEvent_t fork;
  bool ready;
};
Lanes g_lanes[64];
std::mutex g_lanes_mutex;
std::mutex g_lanes_in_use[64];   // one sequence at a time per device uses the side streams

Lanes* lanes_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_lanes_mutex);
  Lanes& l = g_lanes[dev];
  if (!l.ready) {
    if (cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int k = 1; k <= CX_MAX_LANES; ++k) {
      if (cudaStreamCreateWithFlags(&l.stream[k], cudaStreamNonBlocking) != cudaSuccess) return nullptr;
      if (cudaEventCreateWithFlags(&l.done[k], cudaEventDisableTiming) != cudaSuccess) return nullptr;
    }
    l.ready = true;
  }
  return &l;
}

}  // namespace

int cx_run_ops(CxOp* ops, int count, uint64_t seq, void* stream) {
  cudaStream_t main_stream = reinterpret_cast<cudaStream_t>(stream);
  Lanes* lanes = nullptr;
  std::unique_lock<std::mutex> lanes_held;   // taken with the first side-stream op, released on return
  uint32_t open_mask = 0;      // side lanes with work that `stream` has not waited for yet
  bool forked = false;         // the fork event of the current region is recorded
  auto join = [&]() -> int {
    for (int k = 1; k <= CX_MAX_LANES; ++k) {
      if (!((open_mask >> k) & 1u)) continue;
      if (cudaEventRecord(lanes->done[k], lanes->stream[k]) != cudaSuccess ||
          cudaStreamWaitEvent(main_stream, lanes->done[k], 0) != cudaSuccess)
        return cx_set_error("cx_run_ops: joining a side stream", (int)cudaGetLastError());
    }
    open_mask = 0;
    forked = false;
    return 0;
  };
  for (int i = 0; i < count; ++i) {
    CxOp& o = ops[i];
    int rc;
    if (o.lane > 0 && o.dev == CX_DEV_CUDA) {
      if (o.lane > CX_MAX_LANES) return cx_set_error("cx_run_ops: lane out of range", 0);
      if (!lanes) {
        if (!(lanes = lanes_for_current_device()))
          return cx_set_error("cx_run_ops: side streams", (int)cudaGetLastError());
        int dev = 0;
        cudaGetDevice(&dev);
        lanes_held = std::unique_lock<std::mutex>(g_lanes_in_use[dev]);
      }
      if (!forked) {
        if (cudaEventRecord(lanes->fork, main_stream) != cudaSuccess)
          return cx_set_error("cx_run_ops: fork event", (int)cudaGetLastError());
        forked = true;
      }
      if (!((open_mask >> o.lane) & 1u)) {
        if (cudaStreamWaitEvent(lanes->stream[o.lane], lanes->fork, 0) != cudaSuccess)
          return cx_set_error("cx_run_ops: forking a side stream", (int)cudaGetLastError());
        open_mask |= 1u << o.lane;
      }
      rc = run_one(o, seq, lanes->stream[o.lane]);
    } else {
      if (open_mask && (rc = join())) return rc;
      rc = run_one(o, seq, stream);
    }
    if (rc) { if (open_mask) join(); return rc; }
  }
  if (open_mask) return join();
  return 0;
}

// ---- a launch sequence as a CUDA graph -------------------------------------------------
// The sequence is captured once (side-stream lanes become branches of the graph) with every
// kernel reading its sequence number from a device cell; a replay is one 8-byte copy into the
// cell plus one graph launch, instead of one runtime call per kernel.
struct CxGraph {
  cudaGraph_t graph;
  cudaGraphExec_t exec;
  uint64_t* cell;      // device memory
  int kernels;         // launches per replay (for the launch counter)
  int device;
};

int cx_graph_build(CxOp* ops, int count, void** out) {
  *out = nullptr;
  if (count <= 0) return cx_set_error("cx_graph_build: empty sequence", 0);
  for (int i = 0; i < count; ++i)
    if (ops[i].dev != CX_DEV_CUDA) return cx_set_error("cx_graph_build: host ops cannot be captured", 0);
  CxGraph* g = new CxGraph();
  g->graph = nullptr; g->exec = nullptr; g->cell = nullptr; g->kernels = 0; g->device = 0;
  cudaStream_t cap = nullptr;
  cudaError_t e = cudaGetDevice(&g->device);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&g->cell), sizeof(uint64_t));
  if (e == cudaSuccess) e = cudaMemset(g->cell, 0, sizeof(uint64_t));
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking);
  if (e != cudaSuccess || !lanes_for_current_device()) {   // side streams exist before the capture starts
    if (g->cell) cudaFree(g->cell);
    if (cap) cudaStreamDestroy(cap);
    delete g;
    return cx_set_error("cx_graph_build: set-up", (int)e);
  }
  const uint64_t before = g_launches.load();
  e = cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal);
  int rc = 0;
  if (e == cudaSuccess) {
    g_seq_cell = g->cell;
    rc = cx_run_ops(ops, count, 0, cap);
    g_seq_cell = nullptr;
    const cudaError_t e2 = cudaStreamEndCapture(cap, &g->graph);   // always ends the capture
    if (rc == 0 && e2 != cudaSuccess) e = e2;
  }
  g->kernels = (int)(g_launches.load() - before);
  g_launches.store(before);                                        // nothing ran yet
  if (e == cudaSuccess && rc == 0) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
  cudaStreamDestroy(cap);
  if (e != cudaSuccess || rc != 0) {
    if (g->graph) cudaGraphDestroy(g->graph);
    cudaFree(g->cell);
    delete g;
    cudaGetLastError();
    return rc ? rc : cx_set_error("cx_graph_build: capture", (int)e);
  }
  *out = g;
  return 0;
}

int cx_graph_launch(void* graph, uint64_t seq, void* stream) {
  CxGraph* g = reinterpret_cast<CxGraph*>(graph);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // pageable source: the runtime stages the 8 bytes before it returns, so `seq` may go away
  cudaError_t e = cudaMemcpyAsync(g->cell, &seq, sizeof(seq), cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaGraphLaunch(g->exec, s);
  if (e != cudaSuccess) return cx_set_error("cx_graph_launch", (int)e);
  g_launches.fetch_add((uint64_t)g->kernels, std::memory_order_relaxed);
  return 0;
}

int cx_graph_free(void* graph) {
  CxGraph* g = reinterpret_cast<CxGraph*>(graph);
  if (!g) return 0;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  if (g->cell) cudaFree(g->cell);
  delete g;
  return 0;
}

int cx_fill_zero(int dev, void* p, int64_t bytes, void* stream) {
  if (dev == CX_DEV_CUDA) {
    const cudaError_t e = cudaMemsetAsync(p, 0, (size_t)bytes, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : cx_set_error("cx_fill_zero", (int)e);
  }
  memset(p, 0, (size_t)bytes);
  return 0;
}

// ---- CUDA memory runtime -----------------------------------------------------------
int cx_cuda_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}
int cx_cuda_set_device(int dev) {
  const cudaError_t e = cudaSetDevice(dev);
  return e == cudaSuccess ? 0 : cx_set_error("cudaSetDevice", (int)e);
}
void* cx_cuda_malloc(int64_t bytes) {
  void* p = nullptr;
  const cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) { cx_set_error("cudaMalloc", (int)e); return nullptr; }
  const cudaError_t e2 = cudaMemset(p, 0, (size_t)bytes);
  if (e2 != cudaSuccess) { cx_set_error("cudaMemset", (int)e2); cudaFree(p); return nullptr; }
  return p;
}
int cx_cuda_free(void* p) {
  const cudaError_t e = cudaFree(p);
  return e == cudaSuccess ? 0 : cx_set_error("cudaFree", (int)e);
}
int cx_cuda_ipc_get(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  static_assert(sizeof(h) == 64, "IPC handle size");
  const cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return cx_set_error("cudaIpcGetMemHandle", (int)e);
  memcpy(handle64, &h, 64);
  return 0;
}
void* cx_cuda_ipc_open(const void* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { cx_set_error("cudaIpcOpenMemHandle", (int)e); return nullptr; }
  return p;
}
int cx_cuda_ipc_close(void* p) {
  const cudaError_t e = cudaIpcCloseMemHandle(p);
  return e == cudaSuccess ? 0 : cx_set_error("cudaIpcCloseMemHandle", (int)e);
}
int cx_cuda_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) { cudaGetLastError(); return 0; }
  return ok;
}
void* cx_pinned_alloc(int64_t bytes, void** device_ptr) {
  void* p = nullptr;
  cudaError_t e = cudaHostAlloc(&p, (size_t)bytes, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) { cx_set_error("cudaHostAlloc", (int)e); return nullptr; }
  memset(p, 0, (size_t)bytes);
  void* d = nullptr;
  e = cudaHostGetDevicePointer(&d, p, 0);
  if (e != cudaSuccess) { cx_set_error("cudaHostGetDevicePointer", (int)e); cudaFreeHost(p); return nullptr; }
  if (device_ptr) *device_ptr = d;
  return p;
}
int cx_pinned_free(void* p) {
  const cudaError_t e = cudaFreeHost(p);
  return e == cudaSuccess ? 0 : cx_set_error("cudaFreeHost", (int)e);
}
int cx_cuda_stream_sync(void* stream) {
  const cudaError_t e = cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cx_set_error("cudaStreamSynchronize", (int)e);
}
int cx_cuda_memcpy(void* dst, const void* src, int64_t bytes, int kind, void* stream) {
  const cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, (cudaMemcpyKind)kind,
                                        reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cx_set_error("cudaMemcpyAsync", (int)e);
}

// ---- host segments -------------------------------------------------------------------
static void* shm_map(const char* name, int64_t bytes, int create) {
  const int fd = shm_open(name, create ? (O_CREAT | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) { snprintf(g_err, sizeof(g_err), "shm_open(%s): %s", name, strerror(errno)); return nullptr; }
  if (create && ftruncate(fd, (off_t)bytes) != 0) {
    snprintf(g_err, sizeof(g_err), "ftruncate(%s): %s", name, strerror(errno));
    close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, (size_t)bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) { snprintf(g_err, sizeof(g_err), "mmap(%s): %s", name, strerror(errno)); return nullptr; }
  return p;
}
void* cx_shm_create(const char* name, int64_t bytes) { return shm_map(name, bytes, 1); }
void* cx_shm_open(const char* name, int64_t bytes) { return shm_map(name, bytes, 0); }
int cx_shm_close(void* p, int64_t bytes) { return munmap(p, (size_t)bytes); }
int cx_shm_unlink(const char* name) { return shm_unlink(name); }
void* cx_host_alloc(int64_t bytes) {
  void* p = nullptr;
  if (posix_memalign(&p, 256, (size_t)(bytes > 0 ? bytes : 1)) != 0) return nullptr;
  memset(p, 0, (size_t)bytes);
  return p;
}
int cx_host_free(void* p) { free(p); return 0; }

}  // extern "C"
