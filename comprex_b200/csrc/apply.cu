// Receive side: wait for the notifications, then decode the sparse payloads
// of all sources in a fixed source order, fused with averaging and the
// parameter update (reference: CompressorIndexPairs::decompress / add,
// src/compressor.hxx:613-658, called after TargetBuffer::waitForCompletion in
// src/comprEx.tpp:224-246; optimizer math keras/comprex_optimizer.py:150-163).
//
// Ownership instead of atomics: every payload carries, per 1024-element
// sub-tile of the vector, a table entry {start, count} that says where that
// sub-tile's pairs sit in the pair list.  A warp owns one sub-tile at a time,
// looks the ranges of all sources up directly and applies them source after
// source.  Indices are
// unique inside one payload and a sub-tile has a single owner, so no atomic
// is needed and the floating-point sum order is the same on every rank, which
// keeps data-parallel replicas bit-identical.
//
//  * sparse ops (ADD; SGD without weight decay) touch only the addressed
//    elements in global memory;
//  * dense ops (SET, SGD with decay, momentum, AdamW) accumulate the sub-tile
//    in shared memory and then walk it once with 16-byte accesses, so the
//    averaged gradient never exists in global memory.
//
// A wait that runs out of its time budget sets CX_ST_TIMEOUT in the status
// word and the kernel returns without touching the output.
#include "cx_device.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

struct ApplyParams {
  CxSources src;
  CxApplyArgs a;
  int64_t n;
  uint32_t nsub;
  uint32_t vec;  // every dense pointer is 16-byte aligned
  uint32_t* status;
  uint64_t timeout_ns;
};

__device__ __forceinline__ CxPair ld_pair(const CxPair* p) {
  const uint2 t = __ldcg(reinterpret_cast<const uint2*>(p));
  CxPair r;
  r.idx = (int32_t)t.x;
  r.val = t.y;
  return r;
}

// Waits for all sources and validates their headers.  Returns false (uniformly
// for the CTA) when the kernel must not touch the output.
__device__ __forceinline__ bool wait_sources(const ApplyParams& p, uint32_t* s_nnz) {
  __shared__ uint32_t s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  if ((int)threadIdx.x < p.src.count) {
    const int j = threadIdx.x;
    const CxHeader* h = p.src.ep[j].hdr;
    uint32_t bad = 0;
    if (!cx::wait_seq(&h->seq, p.src.seq[j], p.timeout_ns)) {
      bad = CX_ST_TIMEOUT;
    } else {
      const uint32_t kind = *reinterpret_cast<const volatile uint32_t*>(&h->kind);
      const uint32_t hn = *reinterpret_cast<const volatile uint32_t*>(&h->n);
      if (kind != CX_KIND_PAIRS || hn != (uint32_t)p.n) bad = CX_ST_BAD_HEADER;
      s_nnz[j] = *reinterpret_cast<const volatile uint32_t*>(&h->nnz);
    }
    if (bad) atomicOr(&s_bad, bad);
  }
  __syncthreads();
  const uint32_t bad = s_bad;
  if (bad && threadIdx.x == 0 && p.status) *p.status = *p.status | bad;
  return bad == 0;
}

template <typename TO>
__global__ void __launch_bounds__(kThreads) apply_sparse_kernel(const ApplyParams p) {
  __shared__ uint32_t s_nnz[CX_MAX_PEERS];
  if (!wait_sources(p, s_nnz)) return;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t nwarps = gridDim.x * kWarps;
  const float scale = p.a.op == CX_OP_SGD ? -p.a.scale : p.a.scale;
  uint32_t bad = 0;
  for (uint32_t sub = blockIdx.x * kWarps + warp; sub < p.nsub; sub += nwarps) {
    const uint32_t lo = sub * CX_SUBTILE;
    uint32_t a = 0, b = 0;
    if (lane < p.src.count) {
      const uint2 entry = __ldcg(reinterpret_cast<const uint2*>(p.src.ep[lane].table) + sub);
      a = entry.x;
      b = min(entry.x + min(entry.y, (uint32_t)CX_SUBTILE), p.src.cap[lane]);  // never beyond the slot
      a = min(a, b);
    }
    for (int j = 0; j < p.src.count; ++j) {
      const uint32_t aj = __shfl_sync(0xffffffffu, a, j);
      const uint32_t bj = __shfl_sync(0xffffffffu, b, j);
      const CxPair* pairs = p.src.ep[j].pairs;
      for (uint32_t i = aj + lane; i < bj; i += 32) {
        const CxPair pr = ld_pair(pairs + i);
        const uint32_t d = (uint32_t)pr.idx - lo;
        if (d < CX_SUBTILE && (int64_t)pr.idx < p.n) {
          const float val = scale * __uint_as_float(pr.val);
          if (p.a.op == CX_OP_SGD) {
            float* w = reinterpret_cast<float*>(p.a.out);
            const float nw = w[pr.idx] + val;
            w[pr.idx] = nw;
            if (p.a.shadow) reinterpret_cast<TO*>(p.a.shadow)[pr.idx] = cx::Elem<TO>::from_f(nw);
          } else {
            TO* o = reinterpret_cast<TO*>(p.a.out);
            o[pr.idx] = cx::Elem<TO>::from_f(cx::Elem<TO>::to_f(o[pr.idx]) + val);
          }
        } else {
          bad = CX_ST_BAD_INDEX;
        }
      }
      __syncwarp();  // the next source may address the same elements from other lanes
    }
  }
  if (bad && p.status) *p.status = *p.status | bad;
}

template <int OP, typename TO>
__device__ __forceinline__ void update4(const ApplyParams& p, int64_t i, const float (&acc)[4],
                                        bool vec) {
  const CxApplyArgs& a = p.a;
  if (OP == CX_OP_SET) {
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = a.scale * acc[e];
    TO* out = reinterpret_cast<TO*>(a.out);
    if (vec) cx::store4(out + i, o);
    else
      for (int e = 0; e < 4; ++e) if (i + e < p.n) out[i + e] = cx::Elem<TO>::from_f(o[e]);
    return;
  }
  float* w = reinterpret_cast<float*>(a.out);
  float wv[4], mv[4], vv[4];
  if (vec) {
    cx::load4(w + i, wv);
    if (OP != CX_OP_SGD) cx::load4(a.m + i, mv);
    if (OP == CX_OP_ADAMW) cx::load4(a.v + i, vv);
  } else {
    for (int e = 0; e < 4; ++e) {
      const bool in = i + e < p.n;
      wv[e] = in ? w[i + e] : 0.f;
      mv[e] = (in && OP != CX_OP_SGD) ? a.m[i + e] : 0.f;
      vv[e] = (in && OP == CX_OP_ADAMW) ? a.v[i + e] : 0.f;
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float g = a.scale * acc[e];
    if (OP == CX_OP_SGD) {
      wv[e] = (1.f - a.wd) * wv[e] - g;
    } else if (OP == CX_OP_MOMENTUM) {
      mv[e] = a.momentum * mv[e] + a.lr * g;
      wv[e] = (1.f - a.wd) * wv[e] - mv[e];
    } else {  // AdamW
      mv[e] = a.beta1 * mv[e] + (1.f - a.beta1) * g;
      vv[e] = a.beta2 * vv[e] + (1.f - a.beta2) * g * g;
      // reciprocals instead of divisions: one correctly rounded 1/x per element, the
      // bias corrections' reciprocals are loop invariants; same arithmetic as the host twin
      const float mh = mv[e] * __frcp_rn(a.bc1);
      const float vh = vv[e] * __frcp_rn(a.bc2);
      wv[e] = wv[e] * (1.f - a.lr * a.wd) - a.lr * mh * __frcp_rn(sqrtf(vh) + a.eps);
    }
  }
  if (vec) {
    cx::store4(w + i, wv);
    if (OP != CX_OP_SGD) cx::store4(a.m + i, mv);
    if (OP == CX_OP_ADAMW) cx::store4(a.v + i, vv);
    if (a.shadow) cx::store4(reinterpret_cast<TO*>(a.shadow) + i, wv);
  } else {
    for (int e = 0; e < 4; ++e) {
      if (i + e >= p.n) continue;
      w[i + e] = wv[e];
      if (OP != CX_OP_SGD) a.m[i + e] = mv[e];
      if (OP == CX_OP_ADAMW) a.v[i + e] = vv[e];
      if (a.shadow) reinterpret_cast<TO*>(a.shadow)[i + e] = cx::Elem<TO>::from_f(wv[e]);
    }
  }
}

template <int OP, typename TO>
__global__ void __launch_bounds__(kThreads) apply_dense_kernel(const ApplyParams p) {
  __shared__ uint32_t s_nnz[CX_MAX_PEERS];
  __shared__ __align__(16) float s_acc[kWarps][CX_SUBTILE];
  if (!wait_sources(p, s_nnz)) return;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t nwarps = gridDim.x * kWarps;
  float* acc = s_acc[warp];
  uint32_t bad = 0;
  for (uint32_t sub = blockIdx.x * kWarps + warp; sub < p.nsub; sub += nwarps) {
    const uint32_t lo = sub * CX_SUBTILE;
    uint32_t a = 0, b = 0;
    if (lane < p.src.count) {
      const uint2 entry = __ldcg(reinterpret_cast<const uint2*>(p.src.ep[lane].table) + sub);
      a = entry.x;
      b = min(entry.x + min(entry.y, (uint32_t)CX_SUBTILE), p.src.cap[lane]);  // never beyond the slot
      a = min(a, b);
    }
#pragma unroll
    for (int q = 0; q < CX_SUBTILE / 128; ++q)
      *reinterpret_cast<float4*>(acc + q * 128 + lane * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    __syncwarp();
    for (int j = 0; j < p.src.count; ++j) {
      const uint32_t aj = __shfl_sync(0xffffffffu, a, j);
      const uint32_t bj = __shfl_sync(0xffffffffu, b, j);
      const CxPair* pairs = p.src.ep[j].pairs;
      for (uint32_t i = aj + lane; i < bj; i += 32) {
        const CxPair pr = ld_pair(pairs + i);
        const uint32_t d = (uint32_t)pr.idx - lo;
        if (d < CX_SUBTILE && (int64_t)pr.idx < p.n) acc[d] += __uint_as_float(pr.val);
        else bad = CX_ST_BAD_INDEX;
      }
      __syncwarp();
    }
#pragma unroll
    for (int q = 0; q < CX_SUBTILE / 128; ++q) {
      const int e0 = q * 128 + lane * 4;
      const int64_t i = (int64_t)lo + e0;
      if (i >= p.n) continue;
      const float4 t = *reinterpret_cast<const float4*>(acc + e0);
      const float av[4] = {t.x, t.y, t.z, t.w};
      update4<OP, TO>(p, i, av, p.vec && i + 3 < p.n);
    }
    __syncwarp();
  }
  if (bad && p.status) *p.status = *p.status | bad;
}

// ---- verbatim forwarding of a received slot (ring allgather hop) ----------

struct ForwardParams {
  CxEndpoint from;
  uint64_t expect;
  CxTargets tg;
  uint64_t seq;
  uint32_t cap;
  CxWorkCounters* ctr;
  uint32_t* status;
  uint64_t timeout_ns;
};

__global__ void __launch_bounds__(kThreads) forward_kernel(const ForwardParams p) {
  __shared__ uint32_t s_ok, s_last;
  if (threadIdx.x == 0) s_ok = cx::wait_seq(&p.from.hdr->seq, p.expect, p.timeout_ns) ? 1u : 0u;
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && p.status) *p.status = *p.status | CX_ST_TIMEOUT;
    return;
  }
  CxHeader hv;
  {
    const uint4* hp = reinterpret_cast<const uint4*>(p.from.hdr);
    uint4* dp = reinterpret_cast<uint4*>(&hv);
#pragma unroll
    for (int q = 0; q < 4; ++q) dp[q] = __ldcg(hp + q);
  }
  const CxHeader* h = &hv;
  const uint32_t nnz = min(h->nnz, p.cap);
  const uint32_t nsub = h->nsub;
  // a warp per sub-tile: its table entry and its pairs keep their positions
  const int lane = threadIdx.x & 31;
  const uint32_t nwarps = gridDim.x * kWarps;
  for (uint32_t sub = blockIdx.x * kWarps + (threadIdx.x >> 5); sub < nsub; sub += nwarps) {
    uint2 v = __ldcg(reinterpret_cast<const uint2*>(p.from.table) + sub);
    v.y = min(v.y, (uint32_t)CX_SUBTILE);
    if (v.x >= p.cap) v.x = v.y = 0;
    else v.y = min(v.y, p.cap - v.x);
    if (lane < p.tg.count) reinterpret_cast<uint2*>(p.tg.ep[lane].table)[sub] = v;
    for (uint32_t i = lane; i < v.y; i += 32) {
      const uint2 pr = __ldcg(reinterpret_cast<const uint2*>(p.from.pairs + v.x + i));
      for (int k = 0; k < p.tg.count; ++k) *reinterpret_cast<uint2*>(p.tg.ep[k].pairs + v.x + i) = pr;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&p.ctr->done, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if ((int)threadIdx.x < p.tg.count) {
    CxHeader* o = p.tg.ep[threadIdx.x].hdr;
    o->bytes = 8ull + 8ull * nnz; o->n = h->n; o->nnz = nnz; o->nnz_found = h->nnz_found;
    o->kind = h->kind; o->threshold = h->threshold; o->nsub = nsub; o->src_rank = h->src_rank;
    o->dtype = h->dtype;
    __threadfence_system();
    cx::st_release_sys(&o->seq, p.seq);
  }
  if (threadIdx.x == 0) p.ctr->done = 0;
}

template <typename TO>
int launch_apply(const ApplyParams& p, int grid, cudaStream_t s) {
  const int op = p.a.op;
  const bool sparse = op == CX_OP_ADD || (op == CX_OP_SGD && p.a.wd == 0.f);
  if (sparse) apply_sparse_kernel<TO><<<grid, kThreads, 0, s>>>(p);
  else if (op == CX_OP_SET) apply_dense_kernel<CX_OP_SET, TO><<<grid, kThreads, 0, s>>>(p);
  else if (op == CX_OP_SGD) apply_dense_kernel<CX_OP_SGD, TO><<<grid, kThreads, 0, s>>>(p);
  else if (op == CX_OP_MOMENTUM) apply_dense_kernel<CX_OP_MOMENTUM, TO><<<grid, kThreads, 0, s>>>(p);
  else if (op == CX_OP_ADAMW) apply_dense_kernel<CX_OP_ADAMW, TO><<<grid, kThreads, 0, s>>>(p);
  else return cx_set_error("cx_apply: unknown op", 0);
  return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int cx_apply_cuda(const CxSources* src, int64_t n, const CxApplyArgs* a, uint32_t* status,
                  uint64_t timeout_ns, void* stream) {
  if (src->count < 0 || src->count > CX_MAX_PEERS) return cx_set_error("cx_apply: bad source count", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_apply: n out of range", 0);
  if (!a->out) return cx_set_error("cx_apply: out is NULL", 0);
  if (n == 0) return 0;
  ApplyParams p;
  p.src = *src; p.a = *a; p.n = n;
  p.nsub = (uint32_t)((n + CX_SUBTILE - 1) / CX_SUBTILE);
  p.status = status; p.timeout_ns = timeout_ns;
  const bool update = a->op != CX_OP_ADD && a->op != CX_OP_SET;
  if (update && a->op != CX_OP_SGD && !a->m) return cx_set_error("cx_apply: momentum buffer missing", 0);
  if (a->op == CX_OP_ADAMW && !a->v) return cx_set_error("cx_apply: second-moment buffer missing", 0);
  p.vec = aligned16(a->out) && (!a->shadow || aligned16(a->shadow)) && (!a->m || aligned16(a->m)) &&
          (!a->v || aligned16(a->v));
  const int dt = update ? (a->shadow ? a->shadow_dtype : CX_F32) : a->out_dtype;
  int grid = cx_sm_count() * 6;
  const int need = (int)((p.nsub + kWarps - 1) / kWarps);
  if (grid > need) grid = need;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  switch (dt) {
    case CX_F32: rc = launch_apply<float>(p, grid, s); break;
    case CX_BF16: rc = launch_apply<__nv_bfloat16>(p, grid, s); break;
    case CX_F16: rc = launch_apply<__half>(p, grid, s); break;
    default: return cx_set_error("cx_apply: unsupported dtype on CUDA", 0);
  }
  if (rc) return rc;
  cx_note_launch();
  return cx_check_launch("apply_kernel");
}

int cx_forward_cuda(const CxEndpoint* from, uint64_t expect_seq, const CxTargets* tg, uint64_t seq,
                    uint32_t cap, void* counters, uint32_t* status, uint64_t timeout_ns,
                    void* stream) {
  ForwardParams p;
  p.from = *from; p.expect = expect_seq; p.tg = *tg; p.seq = seq; p.cap = cap;
  p.ctr = reinterpret_cast<CxWorkCounters*>(counters);
  p.status = status; p.timeout_ns = timeout_ns;
  // every CTA waits on the same notification, so keep the grid co-resident
  const int grid = cx_sm_count() * 2;
  forward_kernel<<<grid, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  cx_note_launch();
  return cx_check_launch("forward_kernel");
}
