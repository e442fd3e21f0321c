// cx_compress_noalloc: the compress kernel with its scratch in a static device
// array, for callers that cannot allocate (see cx_noalloc.h).
#include <cuda_runtime.h>

#include <mutex>

#include "cx_noalloc.h"

int cx_set_error(const char* where, int cuda_err);
int cx_compress_cuda(int gdtype, const void* g, float* r, int64_t n, const float* thr, uint32_t cap,
                     uint64_t seq, const CxTargets* tg, void* workspace, int64_t ws_bytes,
                     CxStats* stats, uint32_t src_rank, void* stream);

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime,
// not an address a kernel could use: the device address is asked for below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CX_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the array on the current device; looked up once per device.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cx_set_error("cx_compress_noalloc: cudaGetDevice", (int)e);
  if (dev < 0 || dev >= kMaxDevices) return cx_set_error("cx_compress_noalloc: device index out of range", 0);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return cx_set_error("cx_compress_noalloc: cudaGetSymbolAddress", (int)e);
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int cx_compress_noalloc(int gdtype, const void* g, float* r, int64_t n, const float* thr,
                                   uint32_t cap, uint64_t seq, const CxTargets* tg, CxStats* stats,
                                   uint32_t src_rank, void* stream) {
  if (n < 0 || n > 0x7fffffffLL)
    return cx_set_error("cx_compress_noalloc: n must be between 0 and 2^31-1 elements", 0);
  if (!tg || tg->count < 0 || tg->count > CX_MAX_PEERS)
    return cx_set_error("cx_compress_noalloc: between 0 and CX_MAX_PEERS targets are supported", 0);
  // The kernel's scratch is a fixed block of counters today, well inside the array, so this
  // guard cannot fire; it stays so that a kernel whose need grows with n is refused here
  // instead of running past the array.
  const int64_t need = cx_workspace_bytes(n);
  if (need > CX_NOALLOC_SCRATCH_BYTES)
    return cx_set_error("cx_compress_noalloc: this vector needs more scratch than the static "
                        "CX_NOALLOC_SCRATCH_BYTES array holds; use cx_compress with a caller-provided buffer", 0);
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  if (n == 0 && tg->count == 0) return 0;   // the warm-up call: set-up only, nothing to send
  // the counters must start at zero; whatever an earlier call left behind is wiped on the stream
  const cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)need, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cx_set_error("cx_compress_noalloc: cudaMemsetAsync", (int)e);
  return cx_compress_cuda(gdtype, g, r, n, thr, cap, seq, tg, scratch, need, stats, src_rank, stream);
}
