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
#include <stdlib.h>

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
  uint32_t batch;  // sub-tiles with few pairs take the one-round-trip path
  uint32_t* status;
  uint64_t timeout_ns;
  const uint64_t* seq_cell;  // non-NULL inside a captured graph: the waits use its value
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
    if (!cx::wait_seq(&h->seq, cx::seq_of(p.seq_cell, p.src.seq[j]), p.timeout_ns)) {
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
  if (bad && threadIdx.x == 0 && p.status) atomicOr(p.status, bad);
  return bad == 0;
}

// ---- one memory round trip for all sources of a sub-tile ------------------------------------
// Walking the sources one after the other costs one dependent load (pairs) or two (pairs, then
// the addressed elements) per source.  When the sub-tile's pairs of ALL sources fit four per
// lane, they are fetched in one go instead: the segments [a_j, b_j) are laid end to end, lane l
// takes the pairs l, l + 32, ... of that sequence, and only the cheap part (the additions, in
// shared memory) runs source after source, which keeps the order of every sum.
constexpr int kBatch = 4;                       // pairs per lane
constexpr uint32_t kBatchMax = 32 * kBatch;      // pairs per sub-tile the batched path takes

struct Gathered {
  CxPair pr[kBatch];
  int src[kBatch];   // source of the pair, -1: none
};

// a / b: lane j holds source j's segment.  total: sum of all segment lengths (<= kBatchMax).
__device__ __forceinline__ void gather_pairs(const ApplyParams& p, int lane, uint32_t a, uint32_t b,
                                             uint32_t pre, Gathered& g) {
  uint32_t off[kBatch];
#pragma unroll
  for (int k = 0; k < kBatch; ++k) { g.src[k] = -1; off[k] = 0; }
  for (int j = 0; j < p.src.count; ++j) {
    const uint32_t pj = __shfl_sync(0xffffffffu, pre, j);
    const uint32_t aj = __shfl_sync(0xffffffffu, a, j);
    const uint32_t cj = __shfl_sync(0xffffffffu, b, j) - aj;
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const uint32_t f = (uint32_t)(k * 32 + lane);
      if (f - pj < cj) { g.src[k] = j; off[k] = aj + (f - pj); }
    }
  }
#pragma unroll
  for (int k = 0; k < kBatch; ++k) {
    g.pr[k].idx = 0;
    g.pr[k].val = 0;
    if (g.src[k] >= 0) g.pr[k] = ld_pair(p.src.ep[g.src[k]].pairs + off[k]);
  }
}

__device__ __forceinline__ void segment_prefix(int lane, uint32_t a, uint32_t b, uint32_t& pre, uint32_t& total) {
  const uint32_t cnt = b - a;
  uint32_t incl = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  pre = incl - cnt;
  total = __shfl_sync(0xffffffffu, incl, 31);
}

template <typename TO>
__global__ void __launch_bounds__(kThreads) apply_sparse_kernel(const ApplyParams p) {
  __shared__ uint32_t s_nnz[CX_MAX_PEERS];
  __shared__ float s_acc[kWarps][CX_SUBTILE];
  if (!wait_sources(p, s_nnz)) { cx::pdl_wait(); return; }
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t nwarps = gridDim.x * kWarps;
  const float scale = p.a.op == CX_OP_SGD ? -p.a.scale : p.a.scale;
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
    uint32_t pre, total;
    segment_prefix(lane, a, b, pre, total);
    if (total == 0) continue;
    if (p.batch && total <= kBatchMax) {
      // all pairs in one round trip, the addressed elements in a second one; the sums are formed
      // in shared memory, source after source and rounded like the element-by-element path
      Gathered g;
      gather_pairs(p, lane, a, b, pre, g);
      uint32_t d[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        d[k] = (uint32_t)g.pr[k].idx - lo;
        if (g.src[k] >= 0 && !(d[k] < CX_SUBTILE && (int64_t)g.pr[k].idx < p.n)) { bad = CX_ST_BAD_INDEX; g.src[k] = -1; }
      }
      if (p.a.op == CX_OP_SGD) {
        const float* w = reinterpret_cast<const float*>(p.a.out);
        float cur[kBatch];
#pragma unroll
        for (int k = 0; k < kBatch; ++k) cur[k] = g.src[k] >= 0 ? w[g.pr[k].idx] : 0.f;
#pragma unroll
        for (int k = 0; k < kBatch; ++k) if (g.src[k] >= 0) acc[d[k]] = cur[k];
      } else {
        const TO* o = reinterpret_cast<const TO*>(p.a.out);
        float cur[kBatch];
#pragma unroll
        for (int k = 0; k < kBatch; ++k) cur[k] = g.src[k] >= 0 ? cx::Elem<TO>::to_f(o[g.pr[k].idx]) : 0.f;
#pragma unroll
        for (int k = 0; k < kBatch; ++k) if (g.src[k] >= 0) acc[d[k]] = cur[k];
      }
      __syncwarp();
      for (int j = 0; j < p.src.count; ++j) {
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
          if (g.src[k] == j) {
            const float nv = acc[d[k]] + scale * __uint_as_float(g.pr[k].val);
            acc[d[k]] = p.a.op == CX_OP_SGD ? nv : cx::Elem<TO>::to_f(cx::Elem<TO>::from_f(nv));
          }
        }
        __syncwarp();
      }
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        if (g.src[k] < 0) continue;
        const float nv = acc[d[k]];
        if (p.a.op == CX_OP_SGD) {
          reinterpret_cast<float*>(p.a.out)[g.pr[k].idx] = nv;
          if (p.a.shadow) reinterpret_cast<TO*>(p.a.shadow)[g.pr[k].idx] = cx::Elem<TO>::from_f(nv);
        } else {
          reinterpret_cast<TO*>(p.a.out)[g.pr[k].idx] = cx::Elem<TO>::from_f(nv);
        }
      }
      __syncwarp();
      continue;
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
  if (bad && p.status) atomicOr(p.status, bad);
  cx::pdl_wait();   // launched early behind its sender: do not complete before that grid has
}

// The update rule on four elements held in registers (g = scale * sum of the payloads).
template <int OP>
__device__ __forceinline__ void rule4(const CxApplyArgs& a, const float (&acc)[4], float (&wv)[4],
                                      float (&mv)[4], float (&vv)[4]) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float g = a.scale * acc[e];
    if (OP == CX_OP_SGD) {
      wv[e] = (1.f - a.wd) * wv[e] - g;
    } else if (OP == CX_OP_MOMENTUM) {
      mv[e] = a.momentum * mv[e] + a.lr * g;
      wv[e] = (1.f - a.wd) * wv[e] - mv[e];
    } else {  // AdamW
      // The moments use explicit fused multiply-adds (the host twin calls fmaf in the same
      // places, so m and v agree bit for bit).  The step itself takes the hardware's
      // approximate square root and reciprocal (about 1 ulp each, two instructions instead
      // of two correctly rounded software sequences of ~12 instructions): the kernel is
      // bound by instruction issue, not by memory, and a relative error of 2^-22 in a step
      // that is itself lr-sized is far below the rounding of w.  Every rank runs this same
      // kernel, so replicas stay bit-identical.
      mv[e] = __fmaf_rn(a.beta1, mv[e], (1.f - a.beta1) * g);
      vv[e] = __fmaf_rn(a.beta2, vv[e], ((1.f - a.beta2) * g) * g);
      const float mh = mv[e] * __frcp_rn(a.bc1);   // loop invariants
      const float vh = vv[e] * __frcp_rn(a.bc2);
      float root, inv;
      asm("sqrt.approx.f32 %0, %1;" : "=f"(root) : "f"(vh));
      asm("rcp.approx.f32 %0, %1;" : "=f"(inv) : "f"(root + a.eps));
      wv[e] = __fmaf_rn(-(a.lr * mh), inv, wv[e] * (1.f - a.lr * a.wd));
    }
  }
}

template <int OP, typename TO>
__device__ __forceinline__ void store_state4(const CxApplyArgs& a, int64_t i, const float (&wv)[4],
                                             const float (&mv)[4], const float (&vv)[4]) {
  cx::store4(reinterpret_cast<float*>(a.out) + i, wv);
  if (OP != CX_OP_SGD) cx::store4(a.m + i, mv);
  if (OP == CX_OP_ADAMW) cx::store4(a.v + i, vv);
  if (a.shadow) cx::store4(reinterpret_cast<TO*>(a.shadow) + i, wv);
}

template <int OP, typename TO>
__device__ __forceinline__ void update4(const CxApplyArgs& a, const int64_t n, int64_t i,
                                        const float (&acc)[4], bool vec) {
  if (OP == CX_OP_SET) {
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = a.scale * acc[e];
    TO* out = reinterpret_cast<TO*>(a.out);
    if (vec) cx::store4(out + i, o);
    else
      for (int e = 0; e < 4; ++e) if (i + e < n) out[i + e] = cx::Elem<TO>::from_f(o[e]);
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
      const bool in = i + e < n;
      wv[e] = in ? w[i + e] : 0.f;
      mv[e] = (in && OP != CX_OP_SGD) ? a.m[i + e] : 0.f;
      vv[e] = (in && OP == CX_OP_ADAMW) ? a.v[i + e] : 0.f;
    }
  }
  rule4<OP>(a, acc, wv, mv, vv);
  if (vec) {
    store_state4<OP, TO>(a, i, wv, mv, vv);
  } else {
    for (int e = 0; e < 4; ++e) {
      if (i + e >= n) continue;
      w[i + e] = wv[e];
      if (OP != CX_OP_SGD) a.m[i + e] = mv[e];
      if (OP == CX_OP_ADAMW) a.v[i + e] = vv[e];
      if (a.shadow) reinterpret_cast<TO*>(a.shadow)[i + e] = cx::Elem<TO>::from_f(wv[e]);
    }
  }
}

// Table look-up, zeroing of the accumulator and accumulation of all sources' pairs of one
// sub-tile (shared by the two dense kernels).  Returns CX_ST_BAD_INDEX or 0.
__device__ __forceinline__ uint32_t accumulate_subtile(const ApplyParams& p, uint32_t sub, int lane, float* acc) {
  const uint32_t lo = sub * CX_SUBTILE;
  uint32_t bad = 0, a = 0, b = 0;
  if (lane < p.src.count) {
    const uint2 entry = __ldcg(reinterpret_cast<const uint2*>(p.src.ep[lane].table) + sub);
    a = entry.x;
    b = min(entry.x + min(entry.y, (uint32_t)CX_SUBTILE), p.src.cap[lane]);  // never beyond the slot
    a = min(a, b);
  }
  uint32_t pre, total;
  segment_prefix(lane, a, b, pre, total);
  Gathered g;
  const bool batched = p.batch && total <= kBatchMax;
  if (batched && total) gather_pairs(p, lane, a, b, pre, g);      // the loads fly while the accumulator is cleared
#pragma unroll
  for (int q = 0; q < CX_SUBTILE / 128; ++q)
    *reinterpret_cast<float4*>(acc + q * 128 + lane * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncwarp();
  if (total == 0) return 0;
  if (batched) {
    for (int j = 0; j < p.src.count; ++j) {
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        if (g.src[k] == j) {
          const uint32_t d = (uint32_t)g.pr[k].idx - lo;
          if (d < CX_SUBTILE && (int64_t)g.pr[k].idx < p.n) acc[d] += __uint_as_float(g.pr[k].val);
          else bad = CX_ST_BAD_INDEX;
        }
      }
      __syncwarp();
    }
    return bad;
  }
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
  return bad;
}

// Variant for the kernel below, which runs few warps per SM and therefore cannot hide one
// memory latency per source: the table entries arrive from the caller (fetched one
// iteration ahead) and the first pair of every source is loaded before any is used.  The
// sums are formed in the same source order as above.
__device__ __forceinline__ uint32_t accumulate_subtile_ahead(const ApplyParams& p, uint32_t sub, int lane,
                                                             uint32_t a, uint32_t b, float* acc) {
  const uint32_t lo = sub * CX_SUBTILE;
  uint32_t bad = 0, have = 0;
  CxPair head[CX_MAX_PEERS];
#pragma unroll
  for (int j = 0; j < CX_MAX_PEERS; ++j) {
    const uint32_t aj = __shfl_sync(0xffffffffu, a, j);
    const uint32_t bj = __shfl_sync(0xffffffffu, b, j);
    head[j].idx = 0;
    head[j].val = 0;
    if (j < p.src.count && aj + lane < bj) {
      head[j] = ld_pair(p.src.ep[j].pairs + aj + lane);
      have |= 1u << j;
    }
  }
#pragma unroll
  for (int q = 0; q < CX_SUBTILE / 128; ++q)
    *reinterpret_cast<float4*>(acc + q * 128 + lane * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncwarp();
#pragma unroll
  for (int j = 0; j < CX_MAX_PEERS; ++j) {
    if (j >= p.src.count) break;
    const uint32_t aj = __shfl_sync(0xffffffffu, a, j);
    const uint32_t bj = __shfl_sync(0xffffffffu, b, j);
    if (aj == bj) continue;            // warp-uniform
    if ((have >> j) & 1u) {
      const uint32_t d = (uint32_t)head[j].idx - lo;
      if (d < CX_SUBTILE && (int64_t)head[j].idx < p.n) acc[d] += __uint_as_float(head[j].val);
      else bad = CX_ST_BAD_INDEX;
    }
    const CxPair* pairs = p.src.ep[j].pairs;
    for (uint32_t i = aj + 32 + lane; i < bj; i += 32) {
      const CxPair pr = ld_pair(pairs + i);
      const uint32_t d = (uint32_t)pr.idx - lo;
      if (d < CX_SUBTILE && (int64_t)pr.idx < p.n) acc[d] += __uint_as_float(pr.val);
      else bad = CX_ST_BAD_INDEX;
    }
    __syncwarp();
  }
  return bad;
}

__device__ __forceinline__ void table_entry(const ApplyParams& p, uint32_t sub, int lane, uint32_t& a, uint32_t& b) {
  a = 0;
  b = 0;
  if (lane < p.src.count && sub < p.nsub) {
    const uint2 entry = __ldcg(reinterpret_cast<const uint2*>(p.src.ep[lane].table) + sub);
    a = entry.x;
    b = min(entry.x + min(entry.y, (uint32_t)CX_SUBTILE), p.src.cap[lane]);  // never beyond the slot
    a = min(a, b);
  }
}

// ---- bulk-copy (TMA) pipeline for the optimizer state ---------------------------------------
// The dense update streams 12 bytes of state per element in and out (AdamW: w, m, v).  With
// plain vector loads the bytes in flight are bounded by registers.  Here lane 0 of every warp
// asks the copy engine of the SM for the warp's next sub-tile of w / m / v (cp.async.bulk into
// shared memory, completion counted in bytes on an mbarrier) before the warp starts on the
// sparse part of the sub-tile, so the state of up to STAGES sub-tiles per warp is in flight
// without holding a register.  Every wait on an mbarrier is bounded.

using cx::smem_u32;
using cx::mbar_init;
using cx::mbar_expect_tx;
using cx::bulk_load;
using cx::mbar_try_wait;
using cx::mbar_wait_bounded;

template <int OP>
struct StateArrays { static constexpr int n = OP == CX_OP_SGD ? 1 : (OP == CX_OP_MOMENTUM ? 2 : 3); };

constexpr int kBulkMaxThreads = 512;

template <int OP, typename TO, int STAGES>
__global__ void __launch_bounds__(kBulkMaxThreads, 1) apply_dense_bulk_kernel(const ApplyParams p) {
  extern __shared__ __align__(128) unsigned char s_dyn[];
  __shared__ uint32_t s_nnz[CX_MAX_PEERS];
  constexpr int NARR = StateArrays<OP>::n;
  constexpr uint32_t kTileBytes = CX_SUBTILE * sizeof(float);
  constexpr uint32_t kWarpBytes = (1 + STAGES * NARR) * kTileBytes;
  if (!wait_sources(p, s_nnz)) { cx::pdl_wait(); return; }
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t nw = blockDim.x >> 5;
  float* acc = reinterpret_cast<float*>(s_dyn + warp * kWarpBytes);
  float* stage0 = acc + CX_SUBTILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dyn + nw * kWarpBytes) + warp * STAGES;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  const uint32_t nwarps = gridDim.x * nw;
  const uint32_t nfull = (uint32_t)(p.n / CX_SUBTILE);   // these sub-tiles are copied in bulk
  const uint32_t first = blockIdx.x * nw + warp;
  const float* wsrc = reinterpret_cast<const float*>(p.a.out);
  uint32_t issued = 0, consumed = 0, bad = 0;

  auto issue = [&](uint32_t sub) {   // warp-uniform call; lane 0 talks to the copy engine
    if (lane == 0) {
      const uint32_t s = issued % STAGES;
      float* dst = stage0 + s * NARR * CX_SUBTILE;
      const size_t off = (size_t)sub * CX_SUBTILE;
      mbar_expect_tx(&bars[s], NARR * kTileBytes);
      bulk_load(dst, wsrc + off, kTileBytes, &bars[s]);
      if (NARR > 1) bulk_load(dst + CX_SUBTILE, p.a.m + off, kTileBytes, &bars[s]);
      if (NARR > 2) bulk_load(dst + 2 * CX_SUBTILE, p.a.v + off, kTileBytes, &bars[s]);
    }
    ++issued;
  };

#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) {
    const uint64_t sub = (uint64_t)first + (uint64_t)t * nwarps;
    if (sub < nfull) issue((uint32_t)sub);
  }
  uint32_t ta, tb;
  table_entry(p, first, lane, ta, tb);
  for (uint32_t sub = first; sub < p.nsub; sub += nwarps) {
    const uint64_t ahead = (uint64_t)sub + (uint64_t)(STAGES - 1) * nwarps;
    if (ahead < nfull) issue((uint32_t)ahead);
    uint32_t na, nb;                                        // the next sub-tile's table entries:
    const uint64_t nxt = (uint64_t)sub + nwarps;            // in flight while this one is summed
    table_entry(p, nxt < p.nsub ? (uint32_t)nxt : p.nsub, lane, na, nb);
    bad |= accumulate_subtile_ahead(p, sub, lane, ta, tb, acc);
    ta = na;
    tb = nb;
    const uint32_t lo = sub * CX_SUBTILE;
    if (sub < nfull) {
      const uint32_t s = consumed % STAGES;
      const uint32_t parity = (consumed / STAGES) & 1u;
      // completion seen by any lane is final: the phase cannot advance again before the next issue()
      if (!__any_sync(0xffffffffu, mbar_wait_bounded(&bars[s], parity))) {
        // give the copies that are still in flight one more bounded chance to land in this
        // CTA's shared memory, report, and leave the output of this warp's tiles untouched
        for (uint32_t c = consumed + 1; c < issued; ++c)
          mbar_wait_bounded(&bars[c % STAGES], (c / STAGES) & 1u);
        if (lane == 0 && p.status) atomicOr(p.status, (uint32_t)CX_ST_TIMEOUT);
        return;
      }
      ++consumed;
      const float* st = stage0 + s * NARR * CX_SUBTILE;
#pragma unroll
      for (int q = 0; q < CX_SUBTILE / 128; ++q) {
        const int e0 = q * 128 + lane * 4;
        float av[4], wv[4], mv[4], vv[4];
        cx::load4(acc + e0, av);
        cx::load4(st + e0, wv);
        if (NARR > 1) cx::load4(st + CX_SUBTILE + e0, mv);
        if (NARR > 2) cx::load4(st + 2 * CX_SUBTILE + e0, vv);
        rule4<OP>(p.a, av, wv, mv, vv);
        store_state4<OP, TO>(p.a, (int64_t)lo + e0, wv, mv, vv);
      }
      // this stage is handed back to the copy engine by a later issue()
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    } else {
#pragma unroll
      for (int q = 0; q < CX_SUBTILE / 128; ++q) {
        const int e0 = q * 128 + lane * 4;
        const int64_t i = (int64_t)lo + e0;
        if (i >= p.n) continue;
        float av[4];
        cx::load4(acc + e0, av);
        update4<OP, TO>(p.a, p.n, i, av, p.vec && i + 3 < p.n);
      }
    }
    __syncwarp();
  }
  if (bad && p.status) atomicOr(p.status, bad);
}

template <int OP, typename TO>
__global__ void __launch_bounds__(kThreads) apply_dense_kernel(const ApplyParams p) {
  __shared__ uint32_t s_nnz[CX_MAX_PEERS];
  __shared__ __align__(16) float s_acc[kWarps][CX_SUBTILE];
  if (!wait_sources(p, s_nnz)) { cx::pdl_wait(); return; }
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t nwarps = gridDim.x * kWarps;
  float* acc = s_acc[warp];
  uint32_t bad = 0;
  for (uint32_t sub = blockIdx.x * kWarps + warp; sub < p.nsub; sub += nwarps) {
    const uint32_t lo = sub * CX_SUBTILE;
    bad |= accumulate_subtile(p, sub, lane, acc);
#pragma unroll
    for (int q = 0; q < CX_SUBTILE / 128; ++q) {
      const int e0 = q * 128 + lane * 4;
      const int64_t i = (int64_t)lo + e0;
      if (i >= p.n) continue;
      const float4 t = *reinterpret_cast<const float4*>(acc + e0);
      const float av[4] = {t.x, t.y, t.z, t.w};
      update4<OP, TO>(p.a, p.n, i, av, p.vec && i + 3 < p.n);
    }
    __syncwarp();
  }
  if (bad && p.status) atomicOr(p.status, bad);
  cx::pdl_wait();   // launched early behind its sender: do not complete before that grid has
}

// ---- dense update: the averaged gradient is a plain vector -------------------------------
// After a dense allreduce (or on a single rank, where nothing is exchanged) the gradient is an
// ordinary fp32 vector; the same rule runs over it in one pass with 16-byte accesses.
struct UpdateParams {
  const float* g;
  CxApplyArgs a;
  int64_t n;
  uint32_t vec;
};

template <int OP, typename TO>
__global__ void __launch_bounds__(kThreads) update_dense_kernel(const UpdateParams q) {
  const int64_t gsz = (int64_t)gridDim.x * kThreads;
  const int64_t nv = (q.n + 3) / 4;
  for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nv; v += gsz) {
    const int64_t i = v * 4;
    float gv[4];
    const bool vec = q.vec && i + 3 < q.n;
    if (vec) cx::load4(q.g + i, gv);
    else
      for (int e = 0; e < 4; ++e) gv[e] = i + e < q.n ? q.g[i + e] : 0.f;
    update4<OP, TO>(q.a, q.n, i, gv, vec);
  }
}

template <typename TO>
int launch_update(const UpdateParams& q, int grid, cudaStream_t s) {
  switch (q.a.op) {
    case CX_OP_SGD: update_dense_kernel<CX_OP_SGD, TO><<<grid, kThreads, 0, s>>>(q); return 0;
    case CX_OP_MOMENTUM: update_dense_kernel<CX_OP_MOMENTUM, TO><<<grid, kThreads, 0, s>>>(q); return 0;
    case CX_OP_ADAMW: update_dense_kernel<CX_OP_ADAMW, TO><<<grid, kThreads, 0, s>>>(q); return 0;
    default: return cx_set_error("cx_update_dense: op must be an update rule", 0);
  }
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
  // A CTA whose wait ran out copies nothing but still arrives at the completion counter and
  // marks the launch as failed there: the CTA that arrives last then publishes nothing and
  // leaves the counters clean for the next launch, whatever the other CTAs saw.
  const bool ok = s_ok != 0;
  if (!ok && threadIdx.x == 0) {
    if (p.status) atomicOr(p.status, (uint32_t)CX_ST_TIMEOUT);
    atomicOr(&p.ctr->pad[0], 1u);
  }
  CxHeader hv;
  if (!ok) { hv.nnz = 0; hv.nsub = 0; hv.n = 0; hv.nnz_found = 0; hv.kind = CX_KIND_ERROR; hv.threshold = 0.f; hv.src_rank = 0; hv.dtype = 0; }
  else
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
  if (!cx::cta_arrive(&p.ctr->done, gridDim.x, &s_last)) return;
  const uint32_t failed = *reinterpret_cast<volatile uint32_t*>(&p.ctr->pad[0]);
  if (!failed && (int)threadIdx.x < p.tg.count) {
    CxHeader* o = p.tg.ep[threadIdx.x].hdr;
    o->bytes = 8ull + 8ull * nnz; o->n = h->n; o->nnz = nnz; o->nnz_found = h->nnz_found;
    o->kind = h->kind; o->threshold = h->threshold; o->nsub = nsub; o->src_rank = h->src_rank;
    o->dtype = h->dtype;
    cx::st_release_sys(&o->seq, p.seq);
  }
  __syncthreads();
  if (threadIdx.x == 0) { p.ctr->pad[0] = 0; p.ctr->done = 0; }
}

#ifndef CX_APPLY_STAGES
#define CX_APPLY_STAGES 1
#endif
#ifndef CX_APPLY_WARPS
#define CX_APPLY_WARPS 16
#endif

// COMPREX_APPLY_BULK=1 routes the dense updates through the bulk-copy kernel.  It is off by
// default: on B200 it is 3 % faster than the register kernel for AdamW at 2^28 elements and
// 1 % survivors (1336 vs 1385 us) and slower everywhere else (2^24: 179 vs 136 us; 10 %
// survivors: 2784 vs 1787 us), because its shared-memory footprint leaves 14 warps per SM to
// cover an instruction-issue-bound update.  The variable is read at every call.
bool bulk_enabled() {
  const char* e = getenv("COMPREX_APPLY_BULK");
  return e && e[0] == '1';
}

// COMPREX_APPLY_STAGES=1|2: sub-tiles of state per warp in flight (more stages, fewer warps per SM)
int bulk_stages() {
  const char* e = getenv("COMPREX_APPLY_STAGES");
  return (e && e[0] == '1') ? 1 : (e && e[0] == '2') ? 2 : CX_APPLY_STAGES;
}

template <int OP, typename TO, int STAGES>
int launch_bulk_stages(const ApplyParams& p, cudaStream_t s) {
  constexpr size_t kWarpBytes = (size_t)(1 + STAGES * StateArrays<OP>::n) * CX_SUBTILE * sizeof(float);
  constexpr size_t kBudget = 227 * 1024 - 1024;      // per SM, minus the static part and slack
  int nw = (int)(kBudget / (kWarpBytes + 8 * STAGES));
  if (nw > CX_APPLY_WARPS) nw = CX_APPLY_WARPS;
  if (nw > kBulkMaxThreads / 32) nw = kBulkMaxThreads / 32;
  const size_t smem = (size_t)nw * (kWarpBytes + 8 * STAGES);
  const int per_sm = (int)(kBudget / (smem + 1024)) > 0 ? (int)(kBudget / (smem + 1024)) : 1;
  auto kern = apply_dense_bulk_kernel<OP, TO, STAGES>;
  static bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cx_set_error("cx_apply: cudaGetDevice", 0);
  if (!configured[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cx_set_error("cx_apply: shared memory opt-in", (int)e);
    configured[dev] = true;
  }
  int grid = cx_sm_count() * per_sm;
  const int need = (int)((p.nsub + nw - 1) / nw);
  if (grid > need) grid = need;
  kern<<<grid, nw * 32, smem, s>>>(p);
  return 0;
}

template <int OP, typename TO>
int launch_bulk(const ApplyParams& p, cudaStream_t s) {
  return bulk_stages() == 1 ? launch_bulk_stages<OP, TO, 1>(p, s) : launch_bulk_stages<OP, TO, 2>(p, s);
}

template <typename TO>
int launch_apply(const ApplyParams& p, int grid, cudaStream_t s) {
  const int op = p.a.op;
  const bool sparse = op == CX_OP_ADD || (op == CX_OP_SGD && p.a.wd == 0.f);
  if (!sparse && op != CX_OP_SET && p.vec && bulk_enabled()) {
    // optimizer state through the copy engine (16-byte aligned state, full sub-tiles in bulk)
    if (op == CX_OP_SGD) return launch_bulk<CX_OP_SGD, TO>(p, s);
    if (op == CX_OP_MOMENTUM) return launch_bulk<CX_OP_MOMENTUM, TO>(p, s);
    if (op == CX_OP_ADAMW) return launch_bulk<CX_OP_ADAMW, TO>(p, s);
  }
  const bool cap = p.seq_cell != nullptr;
  if (sparse) cx_launch_pdl(apply_sparse_kernel<TO>, grid, kThreads, 0, s, p, cap);
  else if (op == CX_OP_SET) cx_launch_pdl(apply_dense_kernel<CX_OP_SET, TO>, grid, kThreads, 0, s, p, cap);
  else if (op == CX_OP_SGD) cx_launch_pdl(apply_dense_kernel<CX_OP_SGD, TO>, grid, kThreads, 0, s, p, cap);
  else if (op == CX_OP_MOMENTUM) cx_launch_pdl(apply_dense_kernel<CX_OP_MOMENTUM, TO>, grid, kThreads, 0, s, p, cap);
  else if (op == CX_OP_ADAMW) cx_launch_pdl(apply_dense_kernel<CX_OP_ADAMW, TO>, grid, kThreads, 0, s, p, cap);
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
  p.status = status; p.timeout_ns = timeout_ns; p.seq_cell = cx_seq_cell();
  {
    const char* e = getenv("COMPREX_APPLY_BATCH");       // 0: always walk the sources one by one
    p.batch = (e && e[0] == '0') ? 0u : 1u;
  }
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

int cx_update_dense_cuda(const float* g, int64_t n, const CxApplyArgs* a, void* stream) {
  if (!a->out || !g) return cx_set_error("cx_update_dense: NULL vector", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_update_dense: n out of range", 0);
  if (a->op != CX_OP_SGD && a->op != CX_OP_MOMENTUM && a->op != CX_OP_ADAMW)
    return cx_set_error("cx_update_dense: op must be an update rule", 0);
  if (a->op != CX_OP_SGD && !a->m) return cx_set_error("cx_update_dense: momentum buffer missing", 0);
  if (a->op == CX_OP_ADAMW && !a->v) return cx_set_error("cx_update_dense: second-moment buffer missing", 0);
  if (n == 0) return 0;
  UpdateParams q;
  q.g = g; q.a = *a; q.n = n;
  q.vec = aligned16(g) && aligned16(a->out) && (!a->shadow || aligned16(a->shadow)) && (!a->m || aligned16(a->m)) &&
          (!a->v || aligned16(a->v));
  int grid = cx_sm_count() * 8;
  const int need = (int)(((n + 3) / 4 + kThreads - 1) / kThreads);
  if (grid > need) grid = need;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  switch (a->shadow ? a->shadow_dtype : CX_F32) {
    case CX_F32: rc = launch_update<float>(q, grid, s); break;
    case CX_BF16: rc = launch_update<__nv_bfloat16>(q, grid, s); break;
    case CX_F16: rc = launch_update<__half>(q, grid, s); break;
    default: return cx_set_error("cx_update_dense: unsupported dtype on CUDA", 0);
  }
  if (rc) return rc;
  cx_note_launch();
  return cx_check_launch("update_dense_kernel");
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
