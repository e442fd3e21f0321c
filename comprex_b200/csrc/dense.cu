// Dense exchange kernels over peer-mapped memory.
//
// These replace the GaspiEx engine of the reference (memcpy into a registered
// source buffer + RDMA write + notify, src/gaspiEx.tpp:70-119) and the dense
// allreduce schedules built on it (src/allreduce.tpp:73-118, 319-351,
// 571-601): the sending kernel reads the user's vector and stores it directly
// into the receive slots of its targets (no staging copy), the last CTA
// publishes the notification; the receiving kernel waits with a time budget,
// sums its sources in a fixed order in fp32 and can push the result on to
// further slots in the same pass (chief broadcast, second phase of the
// two-shot allreduce).  CompressorNone's "out = data + rests; rests = 0"
// (src/compressor.hxx:93-105) is the HAS_R variant of the send kernel.
#include "cx_device.cuh"

namespace {

constexpr int kThreads = 256;

struct Ranges {
  int64_t start[CX_MAX_PEERS];
  int64_t len[CX_MAX_PEERS];
};

struct SendParams {
  const void* g;
  float* r;
  int64_t n;
  uint64_t seq;
  const uint64_t* seq_cell;  // non-NULL inside a captured graph
  CxTargets tg;
  Ranges rg;
  int32_t has_ranges;
  uint32_t src_rank;
  uint32_t dtype;
  CxWorkCounters* ctr;
};

// Grid-stride copy of nbytes with 16-byte accesses and four loads in flight per thread.
// Both pointers must be 16-byte aligned.  VOLATILE_SRC: the source was written by a
// peer GPU during this kernel's lifetime, read it through L2.
template <bool VOLATILE_SRC>
__device__ __forceinline__ void copy_bytes16(char* dst, const char* src, int64_t nbytes, int64_t gtid,
                                             int64_t gsz) {
  const int64_t nv = nbytes / 16;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  int64_t q = gtid;
  for (; q + 3 * gsz < nv; q += 4 * gsz) {
    uint4 a, b, c, e;
    if (VOLATILE_SRC) { a = __ldcg(s + q); b = __ldcg(s + q + gsz); c = __ldcg(s + q + 2 * gsz); e = __ldcg(s + q + 3 * gsz); }
    else { a = s[q]; b = s[q + gsz]; c = s[q + 2 * gsz]; e = s[q + 3 * gsz]; }
    d[q] = a; d[q + gsz] = b; d[q + 2 * gsz] = c; d[q + 3 * gsz] = e;
  }
  for (; q < nv; q += gsz) d[q] = VOLATILE_SRC ? __ldcg(s + q) : s[q];
  for (int64_t b = nv * 16 + gtid; b < nbytes; b += gsz)
    dst[b] = VOLATILE_SRC ? __ldcg(src + b) : src[b];
}

template <typename T>
__device__ __forceinline__ void publish_dense(const CxTargets& tg, int k, int64_t n, uint64_t seq,
                                              uint32_t src_rank, uint32_t dtype) {
  CxHeader* h = tg.ep[k].hdr;
  h->bytes = (uint64_t)n * sizeof(T);
  h->n = (uint32_t)n; h->nnz = (uint32_t)n; h->nnz_found = (uint32_t)n;
  h->kind = CX_KIND_DENSE; h->threshold = 0.f; h->nsub = 0; h->src_rank = src_rank;
  h->dtype = dtype;
  cx::st_release_sys(&h->seq, seq);   // releases this thread's header stores and all that cta_arrive ordered before
}

// four elements through the multicast mapping (16 bytes of fp32, 8 bytes of a 16-bit type)
__device__ __forceinline__ void mc_store4(float* mc, const float (&v)[4]) {
  cx::mm_st_v4(mc, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
}
__device__ __forceinline__ void mc_store4(__nv_bfloat16* mc, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
  __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
  cx::mm_st_b64(mc, make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b)));
}
__device__ __forceinline__ void mc_store4(__half* mc, const float (&v)[4]) {
  __half2 a = __floats2half2_rn(v[0], v[1]);
  __half2 b = __floats2half2_rn(v[2], v[3]);
  cx::mm_st_b64(mc, make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b)));
}

template <typename T, bool HAS_R>
__global__ void __launch_bounds__(kThreads) dense_send_kernel(const SendParams p) {
  __shared__ uint32_t s_last;
  const T* __restrict__ g = reinterpret_cast<const T*>(p.g);
  const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t gsz = (int64_t)gridDim.x * kThreads;
  if (!p.has_ranges) {
    // same vector to every target, 4 elements per thread and step
    const bool vec = (reinterpret_cast<uintptr_t>(g) & (4 * sizeof(T) - 1)) == 0 &&
                     (!HAS_R || (reinterpret_cast<uintptr_t>(p.r) & 15) == 0);
    // with a multicast endpoint the aligned body goes out once for all targets
    const bool mc = (p.tg.pad & CX_TG_MULTICAST) != 0;
    const int64_t nv = (p.n + 3) / 4;
    for (int64_t q = gtid; q < nv; q += gsz) {
      const int64_t i = q * 4;
      float x[4];
      if (vec && i + 3 < p.n) {
        cx::load4(g + i, x);
        if (HAS_R) {
          float rr[4];
          cx::load4(p.r + i, rr);
          const float z[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int e = 0; e < 4; ++e) x[e] += rr[e];
          cx::store4(p.r + i, z);
        }
        if (mc) {
          mc_store4(reinterpret_cast<T*>(p.tg.ep[p.tg.count].pairs) + i, x);
        } else {
          for (int k = 0; k < p.tg.count; ++k)
            cx::store4(reinterpret_cast<T*>(p.tg.ep[k].pairs) + i, x);
        }
      } else {
        for (int e = 0; e < 4 && i + e < p.n; ++e) {
          float xe = cx::Elem<T>::to_f(g[i + e]);
          if (HAS_R) { xe += p.r[i + e]; p.r[i + e] = 0.f; }
          for (int k = 0; k < p.tg.count; ++k)
            reinterpret_cast<T*>(p.tg.ep[k].pairs)[i + e] = cx::Elem<T>::from_f(xe);
        }
      }
    }
  } else {
    // target k receives elements [start_k, start_k + len_k).  The CTAs are dealt out to the
    // targets (CTA b serves target b mod count) so that all destinations are written at the
    // same time: when every rank runs this kernel, a loop "target 0 first" would aim all of
    // them at the same receiver, whose NVLink ingress then serialises the whole phase.
    const int cnt = p.tg.count;
    const bool dealt = cnt > 0 && (int)gridDim.x >= cnt;
    const int k0 = dealt ? (int)(blockIdx.x % cnt) : 0;
    const int k1 = dealt ? k0 + 1 : cnt;
    const int64_t my_ctas = dealt ? ((int64_t)gridDim.x - k0 + cnt - 1) / cnt : gridDim.x;
    const int64_t tid_k = dealt ? (int64_t)(blockIdx.x / cnt) * kThreads + threadIdx.x : gtid;
    const int64_t sz_k = my_ctas * kThreads;
    for (int k = k0; k < k1; ++k) {
      const int64_t gtid = tid_k, gsz = sz_k;   // this target's share of the grid
      const T* src = g + p.rg.start[k];
      T* dst = reinterpret_cast<T*>(p.tg.ep[k].pairs);
      const int64_t len = p.rg.len[k];
      if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        copy_bytes16<false>(reinterpret_cast<char*>(dst), reinterpret_cast<const char*>(src),
                            len * (int64_t)sizeof(T), gtid, gsz);
        continue;
      }
      const bool vec = (reinterpret_cast<uintptr_t>(src) & (4 * sizeof(T) - 1)) == 0;
      const int64_t nv = (len + 3) / 4;
      for (int64_t q = gtid; q < nv; q += gsz) {
        const int64_t i = q * 4;
        if (vec && i + 3 < len) {
          float x[4];
          cx::load4(src + i, x);
          cx::store4(dst + i, x);
        } else {
          for (int e = 0; e < 4 && i + e < len; ++e) dst[i + e] = src[i + e];
        }
      }
    }
  }
  cx::pdl_trigger();   // the reducing kernel queued behind this one may become resident and poll
  if (!cx::cta_arrive(&p.ctr->done, gridDim.x, &s_last)) return;
  if ((int)threadIdx.x < p.tg.count)
    publish_dense<T>(p.tg, threadIdx.x, p.has_ranges ? p.rg.len[threadIdx.x] : p.n, cx::seq_of(p.seq_cell, p.seq),
                     p.src_rank, p.dtype);
  if (threadIdx.x == 0) p.ctr->done = 0;
}

struct ReduceParams {
  void* out;
  const void* own;
  int64_t n;
  CxSources src;
  float scale;
  int32_t has_push;
  CxTargets push;
  uint64_t push_seq;
  const uint64_t* seq_cell;  // non-NULL inside a captured graph: waits and the push use its value
  uint32_t src_rank;
  uint32_t dtype;
  CxWorkCounters* ctr;
  uint32_t* status;
  uint64_t timeout_ns;
  Ranges rg;           // gather mode: source j lands at out[start_j .. start_j+len_j)
  int32_t gather;
};

__device__ __forceinline__ bool wait_dense(const CxSources& src, uint64_t timeout_ns,
                                           uint32_t* status, uint32_t dtype, const uint64_t* seq_cell) {
  __shared__ uint32_t s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  if ((int)threadIdx.x < src.count) {
    const CxHeader* h = src.ep[threadIdx.x].hdr;
    uint32_t bad = 0;
    if (!cx::wait_seq(&h->seq, cx::seq_of(seq_cell, src.seq[threadIdx.x]), timeout_ns)) bad = CX_ST_TIMEOUT;
    else if (*reinterpret_cast<const volatile uint32_t*>(&h->kind) != CX_KIND_DENSE ||
             *reinterpret_cast<const volatile uint32_t*>(&h->dtype) != dtype)
      bad = CX_ST_BAD_HEADER;
    if (bad) atomicOr(&s_bad, bad);
  }
  __syncthreads();
  const uint32_t bad = s_bad;
  if (bad && threadIdx.x == 0 && status) atomicOr(status, bad);
  return bad == 0;
}

template <typename T>
__device__ __forceinline__ void ldcg4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void ldcg4<float>(const float* p, float (&v)[4]) {
  const float4 t = __ldcg(reinterpret_cast<const float4*>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void ldcg4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = __ldcg(reinterpret_cast<const uint2*>(p));
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
template <>
__device__ __forceinline__ void ldcg4<__half>(const __half* p, float (&v)[4]) {
  const uint2 t = __ldcg(reinterpret_cast<const uint2*>(p));
  const __half2 a = *reinterpret_cast<const __half2*>(&t.x);
  const __half2 b = *reinterpret_cast<const __half2*>(&t.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
template <typename T>
__device__ __forceinline__ float ldcg1(const T* p);
template <>
__device__ __forceinline__ float ldcg1<float>(const float* p) { return __ldcg(p); }
template <>
__device__ __forceinline__ float ldcg1<__nv_bfloat16>(const __nv_bfloat16* p) {
  const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __uint_as_float((uint32_t)u << 16);
}
template <>
__device__ __forceinline__ float ldcg1<__half>(const __half* p) {
  const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __half2float(__ushort_as_half(u));
}

// The arrival counter of a pushing reduce is pad[2] of the counter block, not `done`: the kernel
// may be resident while the sending kernel in front of it (which counts in `done`, often in the
// same block) has not finished its own count yet.  pad[0] is the failure mark.
template <typename T>
__device__ __forceinline__ void dense_reduce_body(const ReduceParams& p) {
  __shared__ uint32_t s_last;
  if (!wait_dense(p.src, p.timeout_ns, p.status, p.dtype, p.seq_cell)) {
    // The decision is per CTA, the bookkeeping is per grid: a CTA that gave up still arrives at
    // the completion counter of a pushing launch and marks the launch as failed, so that the
    // CTA arriving last publishes nothing and hands clean counters to the next launch.
    if (!p.has_push) return;
    if (threadIdx.x == 0) {
      atomicOr(&p.ctr->pad[0], 1u);
      __threadfence();
      s_last = (atomicAdd(&p.ctr->pad[2], 1u) == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) { p.ctr->pad[0] = 0; p.ctr->pad[2] = 0; }
    return;
  }
  T* out = reinterpret_cast<T*>(p.out);
  const T* own = reinterpret_cast<const T*>(p.own);
  const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t gsz = (int64_t)gridDim.x * kThreads;
  if (p.gather) {
    for (int j = 0; j < p.src.count; ++j) {
      const T* slot = reinterpret_cast<const T*>(p.src.ep[j].pairs);
      T* dst = out + p.rg.start[j];
      const int64_t len = p.rg.len[j];
      if (p.scale == 1.f && ((reinterpret_cast<uintptr_t>(slot) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        copy_bytes16<true>(reinterpret_cast<char*>(dst), reinterpret_cast<const char*>(slot),
                           len * (int64_t)sizeof(T), gtid, gsz);
        continue;
      }
      const bool vec = (reinterpret_cast<uintptr_t>(dst) & (4 * sizeof(T) - 1)) == 0;
      const int64_t nv = (len + 3) / 4;
      for (int64_t q = gtid; q < nv; q += gsz) {
        const int64_t i = q * 4;
        if (vec && i + 3 < len) {
          float x[4];
          ldcg4<T>(slot + i, x);
          if (p.scale != 1.f)
            for (int e = 0; e < 4; ++e) x[e] *= p.scale;
          cx::store4(dst + i, x);
        } else {
          for (int e = 0; e < 4 && i + e < len; ++e) {
            float x = ldcg1<T>(slot + i + e);
            if (p.scale != 1.f) x *= p.scale;
            dst[i + e] = cx::Elem<T>::from_f(x);
          }
        }
      }
    }
    return;
  }
  const bool vec = (reinterpret_cast<uintptr_t>(out) & (4 * sizeof(T) - 1)) == 0 &&
                   (!own || (reinterpret_cast<uintptr_t>(own) & (4 * sizeof(T) - 1)) == 0);
  // where the own vector enters the sum (CxSources::pad; 0 = first, the reference's order):
  // with the sources in rank order and own_pos = this rank, every rank adds in the same order
  const int own_pos = min(max(p.src.pad, 0), p.src.count);
  const int64_t nv = (p.n + 3) / 4;
  for (int64_t q = gtid; q < nv; q += gsz) {
    const int64_t i = q * 4;
    if (vec && i + 3 < p.n) {
      // start from the first operand instead of zero: a plain copy stays bit-exact
      // operands in order: sources [0, own_pos), the own vector, sources [own_pos, count)
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const int nops = p.src.count + (own ? 1 : 0);
      for (int k = 0; k < nops; ++k) {
        float x[4];
        if (own && k == own_pos) cx::load4(own + i, x);
        else ldcg4<T>(reinterpret_cast<const T*>(p.src.ep[(own && k > own_pos) ? k - 1 : k].pairs) + i, x);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = k == 0 ? x[e] : acc[e] + x[e];
      }
      if (p.scale != 1.f)
        for (int e = 0; e < 4; ++e) acc[e] *= p.scale;
      cx::store4(out + i, acc);
      if (p.has_push) {
        if (p.push.pad & CX_TG_MULTICAST) {
          mc_store4(reinterpret_cast<T*>(p.push.ep[p.push.count].pairs) + i, acc);
        } else {
          for (int k = 0; k < p.push.count; ++k)
            cx::store4(reinterpret_cast<T*>(p.push.ep[k].pairs) + i, acc);
        }
      }
    } else {
      for (int e = 0; e < 4 && i + e < p.n; ++e) {
        float acc = 0.f;
        const int nops = p.src.count + (own ? 1 : 0);
        for (int k = 0; k < nops; ++k) {
          const float x = (own && k == own_pos) ? cx::Elem<T>::to_f(own[i + e])
                                                : ldcg1<T>(reinterpret_cast<const T*>(p.src.ep[(own && k > own_pos) ? k - 1 : k].pairs) + i + e);
          acc = k == 0 ? x : acc + x;
        }
        if (p.scale != 1.f) acc *= p.scale;
        const T o = cx::Elem<T>::from_f(acc);
        out[i + e] = o;
        if (p.has_push)
          for (int k = 0; k < p.push.count; ++k) reinterpret_cast<T*>(p.push.ep[k].pairs)[i + e] = o;
      }
    }
  }
  if (!p.has_push) return;
  if (!cx::cta_arrive(&p.ctr->pad[2], gridDim.x, &s_last)) return;
  const uint32_t failed = *reinterpret_cast<volatile uint32_t*>(&p.ctr->pad[0]);
  if (!failed && (int)threadIdx.x < p.push.count)
    publish_dense<T>(p.push, threadIdx.x, p.n, cx::seq_of(p.seq_cell, p.push_seq), p.src_rank, p.dtype);
  __syncthreads();
  if (threadIdx.x == 0) { p.ctr->pad[0] = 0; p.ctr->pad[2] = 0; }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) dense_reduce_kernel(const ReduceParams p) {
  dense_reduce_body<T>(p);
  cx::pdl_wait();   // launched early behind the sending kernel: do not complete before that grid has
}

// ---- elementwise helpers ----------------------------------------------------

template <typename TY, typename TX>
__global__ void axpy_kernel(TY* y, const TX* x, float a, int64_t n) {
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gsz)
    y[i] = cx::Elem<TY>::from_f(cx::Elem<TY>::to_f(y[i]) + a * cx::Elem<TX>::to_f(x[i]));
}

int grid_for(int64_t work_items, int per_sm) {
  int64_t g = (work_items + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)cx_sm_count() * per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

template <typename TY>
int axpy_x(int xdtype, void* y, const void* x, float a, int64_t n, cudaStream_t s) {
  const int grid = grid_for(n, 8);
  switch (xdtype) {
    case CX_F32: axpy_kernel<TY, float><<<grid, kThreads, 0, s>>>((TY*)y, (const float*)x, a, n); break;
    case CX_BF16: axpy_kernel<TY, __nv_bfloat16><<<grid, kThreads, 0, s>>>((TY*)y, (const __nv_bfloat16*)x, a, n); break;
    case CX_F16: axpy_kernel<TY, __half><<<grid, kThreads, 0, s>>>((TY*)y, (const __half*)x, a, n); break;
    default: return cx_set_error("cx_axpy: unsupported x dtype", 0);
  }
  return 0;
}

}  // namespace

int cx_dense_send_cuda(int dtype, const void* g, float* r, int64_t n, uint64_t seq,
                       const CxTargets* tg, const int64_t* starts, const int64_t* lens,
                       void* counters, uint32_t src_rank, void* stream) {
  if (tg->count < 0 || tg->count > CX_MAX_PEERS) return cx_set_error("cx_dense_send: bad target count", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_dense_send: n out of range", 0);
  SendParams p;
  p.g = g; p.r = r; p.n = n; p.seq = seq; p.seq_cell = cx_seq_cell(); p.tg = *tg; p.src_rank = src_rank; p.dtype = dtype;
  p.ctr = reinterpret_cast<CxWorkCounters*>(counters);
  p.has_ranges = starts != nullptr;
  int64_t work = (n + 3) / 4;
  if (starts) {
    if (r) return cx_set_error("cx_dense_send: ranges and a residual cannot be combined", 0);
    work = 0;
    for (int k = 0; k < tg->count; ++k) {
      p.rg.start[k] = starts[k]; p.rg.len[k] = lens[k];
      if (starts[k] < 0 || lens[k] < 0 || starts[k] + lens[k] > n)
        return cx_set_error("cx_dense_send: range outside the vector", 0);
      if ((lens[k] + 3) / 4 > work) work = (lens[k] + 3) / 4;
    }
  }
  const int grid = grid_for(work, 8);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case CX_F32:
      if (r) dense_send_kernel<float, true><<<grid, kThreads, 0, s>>>(p);
      else dense_send_kernel<float, false><<<grid, kThreads, 0, s>>>(p);
      break;
    case CX_BF16:
      if (r) dense_send_kernel<__nv_bfloat16, true><<<grid, kThreads, 0, s>>>(p);
      else dense_send_kernel<__nv_bfloat16, false><<<grid, kThreads, 0, s>>>(p);
      break;
    case CX_F16:
      if (r) dense_send_kernel<__half, true><<<grid, kThreads, 0, s>>>(p);
      else dense_send_kernel<__half, false><<<grid, kThreads, 0, s>>>(p);
      break;
    default: return cx_set_error("cx_dense_send: unsupported dtype on CUDA", 0);
  }
  cx_note_launch();
  return cx_check_launch("dense_send_kernel");
}

int cx_dense_reduce_cuda(int dtype, void* out, const void* own, int64_t n, const CxSources* src,
                         float scale, const CxTargets* push, uint64_t push_seq,
                         const int64_t* starts, const int64_t* lens, void* counters,
                         uint32_t src_rank, uint32_t* status, uint64_t timeout_ns, void* stream) {
  if (src->count < 0 || src->count > CX_MAX_PEERS) return cx_set_error("cx_dense_reduce: bad source count", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_dense_reduce: n out of range", 0);
  ReduceParams p;
  p.out = out; p.own = own; p.n = n; p.src = *src; p.scale = scale;
  p.has_push = push && push->count > 0;
  if (p.has_push) p.push = *push; else p.push.count = 0;
  p.push_seq = push_seq; p.seq_cell = cx_seq_cell(); p.src_rank = src_rank; p.dtype = dtype;
  p.ctr = reinterpret_cast<CxWorkCounters*>(counters);
  p.status = status; p.timeout_ns = timeout_ns;
  p.gather = starts != nullptr;
  int64_t work = (n + 3) / 4;
  if (starts) {
    if (p.has_push || own) return cx_set_error("cx_dense_reduce: gather mode takes no own/push", 0);
    work = 0;
    for (int j = 0; j < src->count; ++j) {
      p.rg.start[j] = starts[j]; p.rg.len[j] = lens[j];
      if (starts[j] < 0 || lens[j] < 0 || starts[j] + lens[j] > n)
        return cx_set_error("cx_dense_reduce: range outside the vector", 0);
      if ((lens[j] + 3) / 4 > work) work = (lens[j] + 3) / 4;
    }
  }
  // every CTA waits on the notifications first: stay within one co-resident wave
  // (40 registers x 256 threads: six CTAs per SM)
  const int grid = grid_for(work, 6);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case CX_F32: cx_launch_pdl(dense_reduce_kernel<float>, grid, kThreads, 0, s, p, p.seq_cell != nullptr); break;
    case CX_BF16: cx_launch_pdl(dense_reduce_kernel<__nv_bfloat16>, grid, kThreads, 0, s, p, p.seq_cell != nullptr); break;
    case CX_F16: cx_launch_pdl(dense_reduce_kernel<__half>, grid, kThreads, 0, s, p, p.seq_cell != nullptr); break;
    default: return cx_set_error("cx_dense_reduce: unsupported dtype on CUDA", 0);
  }
  cx_note_launch();
  return cx_check_launch("dense_reduce_kernel");
}

int cx_axpy_cuda(int ydtype, void* y, int xdtype, const void* x, float a, int64_t n, void* stream) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  switch (ydtype) {
    case CX_F32: rc = axpy_x<float>(xdtype, y, x, a, n, s); break;
    case CX_BF16: rc = axpy_x<__nv_bfloat16>(xdtype, y, x, a, n, s); break;
    case CX_F16: rc = axpy_x<__half>(xdtype, y, x, a, n, s); break;
    default: return cx_set_error("cx_axpy: unsupported y dtype", 0);
  }
  if (rc) return rc;
  cx_note_launch();
  return cx_check_launch("axpy_kernel");
}
