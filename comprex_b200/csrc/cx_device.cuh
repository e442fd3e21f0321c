// Device-side helpers: system-scope acquire/release, bounded waits, typed loads.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cx_common.h"

namespace cx {

__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_gpu(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_gpu(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Spin until *seq_ptr >= want or the time budget runs out.  Never traps, never
// loops without bound: the caller turns `false` into a status word.
__device__ __forceinline__ bool wait_seq(const uint64_t* seq_ptr, uint64_t want,
                                         uint64_t timeout_ns) {
  if (ld_acquire_sys(seq_ptr) >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  unsigned backoff = 32;
  // the iteration cap bounds the loop even if the timer misbehaves
  for (uint64_t it = 0; it < (1ull << 34); ++it) {
    if (ld_acquire_sys(seq_ptr) >= want) return true;
    if ((it & 15) == 15 && globaltimer_ns() - t0 > timeout_ns) return false;
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
  }
  return false;
}

// Stores through the multicast mapping of a block: the switch writes the same offset in every
// GPU that is bound to the multicast object (multimem.st), one store instead of one per peer.
__device__ __forceinline__ void mm_st_v4(void* mc, const uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void mm_st_b64(void* mc, const uint2 v) {
  const uint64_t w = ((uint64_t)v.y << 32) | v.x;
  asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(mc), "l"(w) : "memory");
}
__device__ __forceinline__ void mm_st_b32(void* mc, const uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};

// load 4 consecutive elements as floats (pointer must be aligned to 4*sizeof(T))
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(a); v[1] = __high2float(a);
  v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void load4(const __half* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __half2 a = *reinterpret_cast<const __half2*>(&t.x);
  const __half2 b = *reinterpret_cast<const __half2*>(&t.y);
  v[0] = __low2float(a); v[1] = __high2float(a);
  v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
  __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}
__device__ __forceinline__ void store4(__half* p, const float (&v)[4]) {
  __half2 a = __floats2half2_rn(v[0], v[1]);
  __half2 b = __floats2half2_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

}  // namespace cx

// A launch that is part of a captured graph takes its sequence number from a device cell
// (written in stream order before every graph launch) instead of from its parameters.
namespace cx {
__device__ __forceinline__ uint64_t seq_of(const uint64_t* cell, uint64_t by_value) {
  return cell ? *reinterpret_cast<const volatile uint64_t*>(cell) : by_value;
}
}  // namespace cx
// the cell for launches issued by this thread right now (NULL outside a graph capture)
const uint64_t* cx_seq_cell();

// ---- programmatic dependent launch ------------------------------------------------------------
// Completion of a group of CTAs whose stores another GPU (or a later kernel) will read.  All
// threads of the CTA have issued their stores; after the block barrier ONE thread fences and counts
// the CTA in (the fence is cumulative over everything the barrier ordered before it: the pattern
// of a grid-wide barrier).  Returns true, uniformly, in the CTA that arrived last.
//
// The fences around the counter are GPU scope: they order this CTA's stores before the count and
// the count before what the last CTA does next, among the threads of this GPU.  The step that a
// peer synchronises with is the st.release.sys of the notification, issued by the last CTA after
// this call; causality is transitive across scopes (each link needs only a scope that holds its
// two ends), so that release covers every store of the whole group and needs no further fence.
// Measured with %globaltimer stamps at the end of a 296-CTA compress kernel on 2^24 elements:
// every thread fencing at system scope 11.5 us from the last sub-tile to the end of the kernel,
// one thread per CTA at system scope 9.8 us, one thread per CTA at GPU scope 3.7 us (1.3 us for
// the arrival, 1.9 us for the release of the headers).
namespace cx {
__device__ __forceinline__ bool cta_arrive(uint32_t* counter, uint32_t group, uint32_t* s_last) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    *s_last = (atomicAdd(counter, 1u) == group - 1u) ? 1u : 0u;
    __threadfence();
  }
  __syncthreads();
  return *s_last != 0u;
}
}  // namespace cx

// ---- bulk copies (the SM's copy engine) and the mbarriers that count their bytes ------------------
// cp.async.bulk wants both addresses 16-byte aligned and a size that is a multiple of 16 bytes.
// Every wait on an mbarrier is bounded.
namespace cx {
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst_smem)), "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// shared memory -> global memory by the copy engine; completion is tracked per bulk group of the
// issuing thread (commit, then wait until the groups have read their source / are complete)
__device__ __forceinline__ void bulk_store(void* dst, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(__cvta_generic_to_global(dst)), "r"(smem_u32(src_smem)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// orders accesses of the generic proxy (ordinary loads, stores, acquires, releases) with those of
// the async proxy (bulk copies) issued by this thread, in both directions
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// at most ~0.25 s: a copy that has not landed by then will not land
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) __nanosleep(64);
  }
  return false;
}
}  // namespace cx

// A kernel launched with cx_launch_pdl may become resident while the kernel in front of it on the
// stream is still finishing (as soon as all of that kernel's CTAs have called cx::pdl_trigger or
// exited).  The late kernel synchronises itself: cx::pdl_wait blocks until the earlier grid has
// completed and its writes are visible.  Used for threshold -> compress (the compress grid is
// resident and its first loads are on their way when the threshold lands) and for
// compress -> apply / send -> reduce (the receive kernel is already polling its flags when the
// sender publishes).  Inside a graph capture, and with COMPREX_PDL=0, launches are plain.
namespace cx {
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
}  // namespace cx

bool cx_pdl_enabled();   // COMPREX_PDL != 0 (read once)

template <typename K, typename P>
void cx_launch_pdl(K kernel, int grid, int threads, size_t smem, cudaStream_t s, const P& params, bool capturing) {
  if (!capturing && cx_pdl_enabled()) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, params) == cudaSuccess) return;
    cudaGetLastError();                        // e.g. a driver without the feature: plain launch
  }
  kernel<<<grid, threads, smem, s>>>(params);
}

// host-side launch bookkeeping shared by the .cu files
void cx_note_launch();
int cx_set_error(const char* where, int cuda_err);
int cx_check_launch(const char* where);
int cx_sm_count();
