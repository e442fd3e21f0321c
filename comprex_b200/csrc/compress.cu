// Fused residual-add / threshold-select / compaction / peer store.
//
// One pass over the vector does what the reference does in
// ThresholdFunction + CompressorIndexPairs::compress_add_update followed by
// SourceBuffer::initTransferPart (src/compressor.hxx:556-611,
// src/comprEx.tpp:176-191):
//
//     r += g ; if |r| > thr { emit (i, r) ; r = 0 }
//
// Work is warp-granular and free of block-wide barriers: a warp owns one
// 1024-element sub-tile at a time, loads it with 16-byte accesses (32
// elements per lane, all loads in flight together), ranks the survivors with one warp scan, reserves room
// for them in the pair list with ONE atomicAdd on a counter in this GPU's
// memory, and stores them through a small shared staging buffer as coalesced
// 8-byte (index, value) pairs straight into the receive
// slots of up to CX_MAX_PEERS targets (peer GPUs' memory mapped over NVLink,
// or local slots), or once through the switch's multicast mapping.  No warp
// ever waits for another one, so the kernel has no spin loop at all.
//
// The pairs of one sub-tile are contiguous in the list; sub-tiles land in the
// list in the order of their reservations.  Next to the pairs every target
// receives one table entry per sub-tile, {start, count}: receivers use it to
// find, without searching or sorting, the pairs that fall into the part of
// the vector they own, and to apply them in a fixed order.  (The reference's
// wire format lists the pairs in ascending index order; nothing on the
// receiving side depends on that order, each index occurs once per payload.)
//
// Survivors that do not fit into the slot are not emitted and stay in the
// residual, which error feedback makes safe; the count is reported.  The CTA
// that finishes last writes the header and publishes the notification
// (st.release.sys) after every CTA's stores were fenced at system scope.
#include <stdlib.h>
#include <string.h>

#include "cx_device.cuh"

namespace {

// Two CTAs (16 warps) per SM: each lane keeps a whole sub-tile share of 32 values in registers
// with all its loads in flight, which needs ~100 registers; squeezing the kernel into three or
// more CTAs per SM makes it spill and measured slower at every size (2^24 elements, 1 %: 55 us
// with two, 69 us with three), and so did an L2 prefetch of the warp's next sub-tile.
#ifndef CX_COMPRESS_MIN_BLOCKS
#define CX_COMPRESS_MIN_BLOCKS 2
#endif
#ifndef CX_COMPRESS_PREFETCH
#define CX_COMPRESS_PREFETCH 0
#endif
#ifndef CX_COMPRESS_BULK_DEFAULT
#define CX_COMPRESS_BULK_DEFAULT 0
#endif

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kChunks = CX_SUBTILE / 128;  // 128 elements = 32 lanes x 4
constexpr int kStage = 128;                // pairs staged per warp and pass

// -DCX_COMPRESS_TRACE: thread 0 of every CTA stamps %globaltimer at up to eight points of
// compress_kernel (entry, before the loop, after the loop, after the arrival, and in the CTA that
// arrives last: regions summed, headers published, end) into a device array that
// cx_compress_trace copies out; a development aid for the fixed part of the kernel's time, not compiled by default.
#ifdef CX_COMPRESS_TRACE
__device__ unsigned long long g_cx_trace[8 * 2048];
#define CX_TRACE(slot)                                                   \
  do {                                                                   \
    if (threadIdx.x == 0 && blockIdx.x < 2048) {                         \
      unsigned long long t_;                                             \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));             \
      g_cx_trace[blockIdx.x * 8 + (slot)] = t_;                          \
    }                                                                    \
  } while (0)
#else
#define CX_TRACE(slot) do { } while (0)
#endif

struct CompressParams {
  const void* g;
  float* r;
  int64_t n;
  const float* thr;
  uint32_t cap;
  uint32_t nsub;
  uint32_t nregions;     // power of two; sub-tile s reserves in region s % nregions
  uint32_t region_size;  // cap / nregions pairs each
  uint32_t vec;          // g and r are aligned for 16-byte (8-byte for 16-bit g) accesses
  uint64_t seq;
  const uint64_t* seq_cell;  // non-NULL inside a captured graph: the sequence number lives there
  CxWorkCounters* ctr;
  CxStats* stats;
  uint32_t src_rank;
  CxTargets tg;
};

// One aligned, complete sub-tile, one warp, one pass: lane L holds elements {c*128 + 4L + e} in
// registers from the loads to the write-back of the residual.
// gl / rl: where this sub-tile's gradient and residual are read (global memory, or the copy of the
// sub-tile that the copy engine put into shared memory); rs: the residual's sub-tile in global
// memory, where the new residual goes.
template <typename T, bool HAS_G, bool HAS_R, bool MC>
__device__ __forceinline__ void compress_subtile_regs(const CompressParams& p, const uint32_t sub,
                                                 const int lane, const float thr,
                                                 const T* __restrict__ gl, const float* __restrict__ rl,
                                                 float* __restrict__ rs, CxPair* stage) {
  constexpr bool FULL = true;
  const int64_t sub_base = (int64_t)sub * CX_SUBTILE;
  const T* gp = gl + lane * 4;
  const float* rp = rl + lane * 4;
  float* wp = rs + lane * 4;
  const int left = (int)min((int64_t)CX_SUBTILE, p.n - sub_base) - lane * 4;  // my elements e < left - c*128

  // ---- load, add -------------------------------------------------------------
  float v[kChunks][4];
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
#pragma unroll
    for (int e = 0; e < 4; ++e) v[c][e] = 0.f;
    if (HAS_R) {
      if (FULL) {
        cx::load4(rp + c * 128, v[c]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c * 128 + e < left) v[c][e] = rp[c * 128 + e];
      }
    }
  }
  if (HAS_G) {
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      float b[4] = {0.f, 0.f, 0.f, 0.f};
      if (FULL) {
        cx::load4(gp + c * 128, b);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c * 128 + e < left) b[e] = cx::Elem<T>::to_f(gp[c * 128 + e]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) v[c][e] = v[c][e] + b[e];
    }
  }

  // ---- classify: bit c*4+e of mask, strict '>' like the reference --------------
  uint32_t mask = 0;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const bool sel = fabsf(v[c][e]) > thr && (FULL || c * 128 + e < left);
      mask |= (sel ? 1u : 0u) << (4 * c + e);
    }
  }

  // ---- rank: lanes in order, each lane's survivors consecutive --------------------
  const uint32_t mine = __popc(mask);
  uint32_t incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  const uint32_t count = __shfl_sync(0xffffffffu, incl, 31);
  const uint32_t first = incl - mine;  // position of my first survivor inside the sub-tile

  // ---- reserve room in the pair list ----------------------------------------------
  // The list is cut into nregions equal regions with one counter each, neighbouring
  // sub-tiles use different regions: atomics on one address are serialised by the L2.
  const uint32_t region = sub & (p.nregions - 1);
  uint32_t base = 0;
  if (count) {
    if (lane == 0) base = atomicAdd(&p.ctr->region[region][0], count);
    base = __shfl_sync(0xffffffffu, base, 0);
  }
  const uint32_t emit = base >= p.region_size ? 0u : min(count, p.region_size - base);  // pairs that fit
  base += region * p.region_size;
  {
    uint2 entry;
    entry.x = emit ? base : 0u;
    entry.y = emit;
    if (MC) {
      if (lane == 0) cx::mm_st_b64(reinterpret_cast<uint2*>(p.tg.ep[p.tg.count].table) + sub, entry);
    } else if (lane < p.tg.count) {
      reinterpret_cast<uint2*>(p.tg.ep[lane].table)[sub] = entry;
    }
  }

  // ---- stage in shared memory, store coalesced to every target ------------------------
  const int32_t idx0 = (int32_t)sub_base + lane * 4;
  for (uint32_t w0 = 0; w0 < emit; w0 += kStage) {   // one pass unless the sub-tile is dense
    uint32_t pos = first - w0;                        // wraps below the window: fails the test
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (mask & (1u << (4 * c + e))) {
          if (pos < (uint32_t)kStage) {
            CxPair pr;
            pr.idx = idx0 + c * 128 + e;
            pr.val = __float_as_uint(v[c][e]);
            stage[pos] = pr;
          }
          ++pos;
        }
      }
    }
    __syncwarp();
    const uint32_t lim = min((uint32_t)kStage, emit - w0);
    if (MC) {
      // one store per pair into the multicast mapping: the switch writes every target's slot
      CxPair* mc = p.tg.ep[p.tg.count].pairs + base + w0;
      for (uint32_t i = lane; i < lim; i += 32) {
        const CxPair pr = stage[i];
        cx::mm_st_b64(mc + i, make_uint2((uint32_t)pr.idx, pr.val));
      }
    } else {
      for (uint32_t i = lane; i < lim; i += 32) {
        const CxPair pr = stage[i];
        for (int k = 0; k < p.tg.count; ++k) p.tg.ep[k].pairs[base + w0 + i] = pr;
      }
    }
    __syncwarp();
  }

  // ---- residual: zero what was emitted, keep the rest ---------------------------------------
  if (HAS_R) {
    if (emit < count) {  // the slot is full: survivors from position emit on stay in the residual
      uint32_t pos = first;
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (mask & (1u << (4 * c + e))) {
            if (pos >= emit) mask &= ~(1u << (4 * c + e));
            ++pos;
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const uint32_t m = (mask >> (4 * c)) & 0xfu;
      if (!HAS_G && m == 0) continue;  // nothing changed in this vector
      float out[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) out[e] = (m & (1u << e)) ? 0.f : v[c][e];
      if (FULL) {
        cx::store4(wp + c * 128, out);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c * 128 + e < left) wp[c * 128 + e] = out[e];
      }
    }
  }
}

// Sub-tiles that are partial or not aligned for 16-byte accesses (the last one of a vector, views
// at odd offsets): one element per lane and step, survivors found with warp ballots.  Two passes
// like above (sum into the residual and count; then read back, emit, zero), a handful of
// registers, and no assumption about alignment or length.
template <typename T, bool HAS_G, bool HAS_R, bool MC>
__device__ __forceinline__ void compress_subtile_edge(const CompressParams& p, const uint32_t sub,
                                                      const int lane, const float thr,
                                                      const T* __restrict__ g, float* __restrict__ r) {
  const int64_t sub_base = (int64_t)sub * CX_SUBTILE;
  const int len = (int)min((int64_t)CX_SUBTILE, p.n - sub_base);
  uint32_t count = 0;
  for (int c = 0; c < len; c += 32) {
    const int i = c + lane;
    float v = 0.f;
    if (i < len) {
      if (HAS_R) v = r[sub_base + i];
      if (HAS_G) v = v + cx::Elem<T>::to_f(g[sub_base + i]);
      if (HAS_R && HAS_G) r[sub_base + i] = v;
    }
    count += __popc(__ballot_sync(0xffffffffu, i < len && fabsf(v) > thr));
  }
  const uint32_t region = sub & (p.nregions - 1);
  uint32_t base = 0;
  if (count) {
    if (lane == 0) base = atomicAdd(&p.ctr->region[region][0], count);
    base = __shfl_sync(0xffffffffu, base, 0);
  }
  const uint32_t emit = base >= p.region_size ? 0u : min(count, p.region_size - base);
  base += region * p.region_size;
  {
    uint2 entry;
    entry.x = emit ? base : 0u;
    entry.y = emit;
    if (MC) {
      if (lane == 0) cx::mm_st_b64(reinterpret_cast<uint2*>(p.tg.ep[p.tg.count].table) + sub, entry);
    } else if (lane < p.tg.count) {
      reinterpret_cast<uint2*>(p.tg.ep[lane].table)[sub] = entry;
    }
  }
  if (emit == 0) return;
  uint32_t seen = 0;                       // survivors in the chunks before this one
  for (int c = 0; c < len && seen < emit; c += 32) {
    const int i = c + lane;
    float v = 0.f;
    if (i < len) v = HAS_R ? r[sub_base + i] : cx::Elem<T>::to_f(g[sub_base + i]);
    const bool sel = i < len && fabsf(v) > thr;
    const uint32_t bal = __ballot_sync(0xffffffffu, sel);
    const uint32_t pos = seen + __popc(bal & ((1u << lane) - 1u));
    if (sel && pos < emit) {
      CxPair pr;
      pr.idx = (int32_t)(sub_base + i);
      pr.val = __float_as_uint(v);
      if (MC) {
        cx::mm_st_b64(p.tg.ep[p.tg.count].pairs + base + pos, make_uint2((uint32_t)pr.idx, pr.val));
      } else {
        for (int k = 0; k < p.tg.count; ++k) p.tg.ep[k].pairs[base + pos] = pr;
      }
      if (HAS_R) r[sub_base + i] = 0.f;
    }
    seen += __popc(bal);
  }
}

// Completion: the CTA that arrives last adds up the regions, writes the headers and publishes the
// notification.  `failed` (CTA-uniform or not): this CTA could not process all its sub-tiles; the
// payload is then not published (the receivers' bounded waits run out) and the status says why.
__device__ __forceinline__ void compress_finish(const CompressParams& p, const int tid, const float thr,
                                                const bool failed, uint32_t& s_last, uint32_t& s_found,
                                                uint32_t& s_nnz) {
  // the receive kernel queued behind this one may become resident now: it polls its flags
  cx::pdl_trigger();
  // ---- completion: the CTA that arrives last publishes -------------------------------
  if (failed) atomicOr(&p.ctr->pad[4], 1u);
  if (tid == 0) {
    s_found = 0;
    s_nnz = 0;
  }
  const bool last = cx::cta_arrive(&p.ctr->done, gridDim.x, &s_last);
  CX_TRACE(3);
  if (!last) return;
  const uint32_t any_failed = *reinterpret_cast<volatile uint32_t*>(&p.ctr->pad[4]);
  if ((uint32_t)tid < p.nregions) {
    const uint32_t f = *reinterpret_cast<volatile uint32_t*>(&p.ctr->region[tid][0]);
    atomicAdd(&s_found, f);
    atomicAdd(&s_nnz, min(f, p.region_size));
    p.ctr->region[tid][0] = 0;
  }
  __syncthreads();
  CX_TRACE(4);
  const uint32_t found = s_found;  // survivors
  const uint32_t nnz = s_nnz;      // pairs stored
  if (tid < p.tg.count && !any_failed) {
    CxHeader* h = p.tg.ep[tid].hdr;
    h->bytes = 8ull + 8ull * nnz;
    h->n = (uint32_t)p.n;
    h->nnz = nnz;
    h->nnz_found = found;
    h->kind = CX_KIND_PAIRS;
    h->threshold = thr;
    h->nsub = p.nsub;
    h->src_rank = p.src_rank;
    h->dtype = CX_F32;
    cx::st_release_sys(&h->seq, cx::seq_of(p.seq_cell, p.seq));
  }
  CX_TRACE(5);
  if (tid == 0) {
    if (p.stats) {
      p.stats->n = (uint32_t)p.n;
      p.stats->nnz = nnz;
      p.stats->nnz_found = found;
      p.stats->status = (found > nnz ? CX_ST_OVERFLOW : 0u) | (any_failed ? CX_ST_TIMEOUT : 0u);
      p.stats->threshold = thr;
    }
    p.ctr->done = 0;
    p.ctr->pad[4] = 0;
  }
  CX_TRACE(6);
}

// T: element type of g.  HAS_G / HAS_R select compress_add_update (both),
// compress_update (r only) and compress (g only).  MC: table and pairs go out once through
// the multicast endpoint tg.ep[tg.count] (multimem.st) instead of once per target; headers and
// notifications are still written target by target.
template <typename T, bool HAS_G, bool HAS_R, bool MC>
__global__ void __launch_bounds__(kThreads, CX_COMPRESS_MIN_BLOCKS)
compress_kernel(const __grid_constant__ CompressParams p) {
  __shared__ CxPair s_stage[kWarps][kStage];
  __shared__ uint32_t s_last;
  __shared__ uint32_t s_found, s_nnz;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const T* __restrict__ g = reinterpret_cast<const T*>(p.g);
  float* __restrict__ r = p.r;
  CX_TRACE(0);
  // Launched with programmatic stream serialization, this grid may be resident while the
  // threshold kernel in front of it still runs: pull the warp's first sub-tile towards L2, then
  // wait for that kernel to finish before reading its result or touching the residual.
  {
    const uint32_t sub0 = blockIdx.x * kWarps + (tid >> 5);
    if (sub0 < p.nsub && (tid & 31) < 2 * kChunks) {
      const int c = (tid & 31) >> 1;
      const int64_t e0 = (int64_t)sub0 * CX_SUBTILE + c * 128;
      if (e0 < p.n) {
        const void* a = (tid & 1) ? (HAS_R ? (const void*)(r + e0) : nullptr) : (HAS_G ? (const void*)(g + e0) : nullptr);
        if (a) asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
      }
    }
  }
  cx::pdl_wait();
  const float thr = *p.thr;
  CX_TRACE(1);
  CxPair* stage = s_stage[warp];
  const uint32_t nwarps = gridDim.x * kWarps;
  const uint32_t nfull = p.vec ? (uint32_t)(p.n / CX_SUBTILE) : 0u;  // sub-tiles on the fast path

  for (uint32_t sub = blockIdx.x * kWarps + warp; sub < p.nsub; sub += nwarps) {
#if CX_COMPRESS_PREFETCH
    // the warp's next sub-tile starts its way from DRAM to L2 now (one 128-byte line per lane
    // and vector): its loads then find it there, without holding a register in the meantime
    if ((uint64_t)sub + nwarps < nfull) {
      const int64_t e0 = ((int64_t)sub + nwarps) * CX_SUBTILE;
      if (HAS_R) asm volatile("prefetch.global.L2 [%0];" ::"l"(r + e0 + lane * 32));
      if (HAS_G && lane * (128 / (int)sizeof(T)) < CX_SUBTILE)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(g + e0 + lane * (128 / (int)sizeof(T))));
    }
#endif
    if (sub < nfull) {
      const int64_t off = (int64_t)sub * CX_SUBTILE;
      compress_subtile_regs<T, HAS_G, HAS_R, MC>(p, sub, lane, thr, g + off, r + off, r + off, stage);
    }
    else compress_subtile_edge<T, HAS_G, HAS_R, MC>(p, sub, lane, thr, g, r);
  }

#ifdef CX_COMPRESS_TRACE
  __syncthreads();   // the stamp marks the CTA's last warp leaving the loop
#endif
  CX_TRACE(2);
  compress_finish(p, tid, thr, false, s_last, s_found, s_nnz);
}

// ---- the same sub-tile routine fed by the SM's copy engine ------------------------------------
// In compress_kernel a warp has loads in flight only between issuing them and using them; while it
// ranks, reserves and stores, nothing of its next sub-tile is on its way.  Here lane 0 of every
// warp asks the copy engine for the warp's next sub-tiles of r and g (cp.async.bulk into the
// warp's own stages in shared memory, completion counted in bytes on an mbarrier per stage)
// before the warp starts on the current one, so STAGES - 1 sub-tiles per warp are in flight all
// the time without holding a register.  One CTA per SM; the number of warps follows from the
// shared memory a warp needs.  Needs r and g 16-byte aligned; the last, partial sub-tile takes
// the edge path.  Every wait on an mbarrier is bounded; a warp whose copy does not arrive marks
// the call as failed, waits (bounded) for its other copies and joins the completion protocol,
// which then publishes nothing.
#ifndef CX_COMPRESS_BULK_STAGES
#define CX_COMPRESS_BULK_STAGES 2
#endif
constexpr int kBulkMaxWarps = 16;

template <typename T, bool HAS_G, bool HAS_R, bool MC, int STAGES>
__global__ void __launch_bounds__(kBulkMaxWarps * 32, 1)
compress_bulk_kernel(const __grid_constant__ CompressParams p) {
  extern __shared__ __align__(128) unsigned char s_dyn[];
  __shared__ uint32_t s_last;
  __shared__ uint32_t s_found, s_nnz;
  constexpr uint32_t kRB = HAS_R ? (uint32_t)(CX_SUBTILE * sizeof(float)) : 0u;
  constexpr uint32_t kGB = HAS_G ? (uint32_t)(CX_SUBTILE * sizeof(T)) : 0u;
  constexpr uint32_t kStageB = kRB + kGB;
  constexpr uint32_t kWarpB = STAGES * kStageB + kStage * (uint32_t)sizeof(CxPair);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const uint32_t nw = blockDim.x >> 5;
  unsigned char* mine = s_dyn + (size_t)warp * kWarpB;
  CxPair* stage = reinterpret_cast<CxPair*>(mine + STAGES * kStageB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dyn + (size_t)nw * kWarpB) + warp * STAGES;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) cx::mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  // everything in front of this kernel on the stream is complete and visible after this
  cx::pdl_wait();
  const float thr = *p.thr;
  const T* __restrict__ g = reinterpret_cast<const T*>(p.g);
  float* __restrict__ r = p.r;
  const uint32_t nwarps = gridDim.x * nw;
  const uint32_t nfull = (uint32_t)(p.n / CX_SUBTILE);
  const uint32_t first = blockIdx.x * nw + warp;
  uint32_t issued = 0, consumed = 0;
  bool failed = false;

  auto issue = [&](uint32_t sub) {   // warp-uniform call; lane 0 talks to the copy engine
    if (lane == 0) {
      unsigned char* dst = mine + (issued % STAGES) * kStageB;
      uint64_t* bar = &bars[issued % STAGES];
      const size_t off = (size_t)sub * CX_SUBTILE;
      cx::mbar_expect_tx(bar, kStageB);
      if (HAS_R) cx::bulk_load(dst, r + off, kRB, bar);
      if (HAS_G) cx::bulk_load(dst + kRB, g + off, kGB, bar);
    }
    ++issued;
  };

#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) {
    const uint64_t sub = (uint64_t)first + (uint64_t)t * nwarps;
    if (sub < nfull) issue((uint32_t)sub);
  }
  for (uint32_t sub = first; sub < p.nsub; sub += nwarps) {
    const uint64_t ahead = (uint64_t)sub + (uint64_t)(STAGES - 1) * nwarps;
    if (ahead < nfull) issue((uint32_t)ahead);
    if (sub < nfull) {
      const uint32_t s = consumed % STAGES;
      // completion seen by any lane is final: the phase cannot advance again before the next issue()
      if (!__any_sync(0xffffffffu, cx::mbar_wait_bounded(&bars[s], (consumed / STAGES) & 1u))) {
        for (uint32_t c = consumed + 1; c < issued; ++c)
          cx::mbar_wait_bounded(&bars[c % STAGES], (c / STAGES) & 1u);
        failed = true;
        break;
      }
      ++consumed;
      const unsigned char* src = mine + s * kStageB;
      compress_subtile_regs<T, HAS_G, HAS_R, MC>(p, sub, lane, thr, reinterpret_cast<const T*>(src + kRB),
                                                 reinterpret_cast<const float*>(src),
                                                 r + (size_t)sub * CX_SUBTILE, stage);
      // this stage is handed back to the copy engine by a later issue()
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
    } else {
      compress_subtile_edge<T, HAS_G, HAS_R, MC>(p, sub, lane, thr, g, r);
    }
  }
  compress_finish(p, tid, thr, failed, s_last, s_found, s_nnz);
}

// n == 0: nothing to scan, only the (empty) header and the notification.
__global__ void compress_empty_kernel(const CompressParams p) {
  const int tid = threadIdx.x;
  if (tid < p.tg.count) {
    CxHeader* h = p.tg.ep[tid].hdr;
    h->bytes = 8; h->n = 0; h->nnz = 0; h->nnz_found = 0; h->kind = CX_KIND_PAIRS;
    h->threshold = *p.thr; h->nsub = 0; h->src_rank = p.src_rank; h->dtype = CX_F32;
    __threadfence_system();
    cx::st_release_sys(&h->seq, cx::seq_of(p.seq_cell, p.seq));
  }
  if (tid == 0 && p.stats) {
    p.stats->n = 0; p.stats->nnz = 0; p.stats->nnz_found = 0; p.stats->status = 0;
    p.stats->threshold = *p.thr;
  }
}

template <typename K>
void launch_pdl(K kernel, const CompressParams& p, int grid, cudaStream_t s) {
  cx_launch_pdl(kernel, grid, kThreads, 0, s, p, p.seq_cell != nullptr);
}

template <typename T, bool MC>
void launch_mode_mc(const CompressParams& p, int grid, cudaStream_t s) {
  if (p.g && p.r) launch_pdl(compress_kernel<T, true, true, MC>, p, grid, s);
  else if (p.r) launch_pdl(compress_kernel<T, false, true, MC>, p, grid, s);
  else launch_pdl(compress_kernel<T, true, false, MC>, p, grid, s);
}

template <typename T>
void launch_mode(const CompressParams& p, int grid, cudaStream_t s) {
  if (p.tg.pad & CX_TG_MULTICAST) launch_mode_mc<T, true>(p, grid, s);
  else launch_mode_mc<T, false>(p, grid, s);
}

// COMPREX_COMPRESS_BULK=1 (read per call): the copy-engine variant where the alignment allows it.
// Measured equal to or up to 5 % slower than compress_kernel at every size from 2^22 to 2^28
// elements with 2, 3 and 4 stages (the kernel is not bound by its loads in flight), hence opt-in.
bool bulk_wanted() {
  const char* e = getenv("COMPREX_COMPRESS_BULK");
  return e ? atoi(e) != 0 : (CX_COMPRESS_BULK_DEFAULT != 0);
}

template <typename T, bool HAS_G, bool HAS_R, bool MC>
int launch_bulk_one(const CompressParams& p, cudaStream_t s) {
  constexpr int STAGES = CX_COMPRESS_BULK_STAGES;
  constexpr size_t kStageB = (HAS_R ? CX_SUBTILE * sizeof(float) : 0) + (HAS_G ? CX_SUBTILE * sizeof(T) : 0);
  constexpr size_t kWarpB = STAGES * kStageB + kStage * sizeof(CxPair) + 8 * STAGES;
  constexpr size_t kBudget = 227 * 1024 - 1024;   // per SM, minus the static part and slack
  int nw = (int)(kBudget / kWarpB);
  if (nw > kBulkMaxWarps) nw = kBulkMaxWarps;
#ifdef CX_COMPRESS_BULK_WARPS
  if (nw > CX_COMPRESS_BULK_WARPS) nw = CX_COMPRESS_BULK_WARPS;
#endif
  if (nw >= 8) nw &= ~3;                          // the same number of warps on every scheduler
  const size_t smem = (size_t)nw * kWarpB;
  auto kern = compress_bulk_kernel<T, HAS_G, HAS_R, MC, STAGES>;
  static bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cx_set_error("cx_compress: cudaGetDevice", 0);
  if (!configured[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cx_set_error("cx_compress: shared memory opt-in", (int)e);
    configured[dev] = true;
  }
  int grid = cx_sm_count();
  const int need = (int)((p.nsub + nw - 1) / nw);
  if (grid > need) grid = need;
  cx_launch_pdl(kern, grid, nw * 32, smem, s, p, p.seq_cell != nullptr);
  return 0;
}

template <typename T, bool MC>
int launch_bulk_mc(const CompressParams& p, cudaStream_t s) {
  if (p.g && p.r) return launch_bulk_one<T, true, true, MC>(p, s);
  if (p.r) return launch_bulk_one<T, false, true, MC>(p, s);
  return launch_bulk_one<T, true, false, MC>(p, s);
}

template <typename T>
int launch_bulk(const CompressParams& p, cudaStream_t s) {
  if (p.tg.pad & CX_TG_MULTICAST) return launch_bulk_mc<T, true>(p, s);
  return launch_bulk_mc<T, false>(p, s);
}

}  // namespace

#ifdef CX_COMPRESS_TRACE
extern "C" int cx_compress_trace(unsigned long long* host, int n) {
  if (n > 8 * 2048) n = 8 * 2048;
  return (int)cudaMemcpyFromSymbol(host, g_cx_trace, sizeof(unsigned long long) * n);
}
#endif

// The only scratch a compressor needs: one zero-initialised CxWorkCounters block.
extern "C" int64_t cx_workspace_bytes(int64_t n) {
  (void)n;
  return (int64_t)sizeof(CxWorkCounters);
}

int cx_compress_cuda(int gdtype, const void* g, float* r, int64_t n, const float* thr,
                     uint32_t cap, uint64_t seq, const CxTargets* tg, void* workspace,
                     int64_t ws_bytes, CxStats* stats, uint32_t src_rank, void* stream) {
  if (!g && !r) return cx_set_error("cx_compress: g and r are both NULL", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_compress: n out of range", 0);
  if (tg->count < 0 || tg->count > CX_MAX_PEERS) return cx_set_error("cx_compress: bad target count", 0);
  if ((tg->pad & CX_TG_MULTICAST) && tg->count >= CX_MAX_PEERS)
    return cx_set_error("cx_compress: no room for the multicast endpoint", 0);
  if (ws_bytes < cx_workspace_bytes(n)) return cx_set_error("cx_compress: workspace too small", 0);
  CompressParams p;
  p.g = g; p.r = r; p.n = n; p.thr = thr; p.cap = cap;
  p.nsub = (uint32_t)((n + CX_SUBTILE - 1) / CX_SUBTILE);
  // at least 8 sub-tiles and 256 pairs per region, so that regions fill evenly
  p.nregions = 1;
  while (p.nregions < CX_MAX_REGIONS && p.nsub / (2 * p.nregions) >= 8 && cap / (2 * p.nregions) >= 256)
    p.nregions *= 2;
  p.region_size = cap / p.nregions;
  p.seq = seq;
  p.seq_cell = cx_seq_cell();
  p.ctr = reinterpret_cast<CxWorkCounters*>(workspace);
  p.stats = stats; p.src_rank = src_rank;
  p.tg = *tg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n == 0) {
    compress_empty_kernel<<<1, 32, 0, s>>>(p);
    cx_note_launch();
    return cx_check_launch("compress_empty_kernel");
  }
  const size_t esz = gdtype == CX_F32 ? 4 : 2;
  p.vec = (!r || (reinterpret_cast<uintptr_t>(r) & 15) == 0) &&
          (!g || (reinterpret_cast<uintptr_t>(g) & (4 * esz - 1)) == 0);
  const bool aligned16 = (!r || (reinterpret_cast<uintptr_t>(r) & 15) == 0) &&
                         (!g || (reinterpret_cast<uintptr_t>(g) & 15) == 0);
  if (bulk_wanted() && aligned16 && n >= CX_SUBTILE) {
    int rc = 0;
    switch (gdtype) {
      case CX_F32: rc = launch_bulk<float>(p, s); break;
      case CX_BF16: rc = launch_bulk<__nv_bfloat16>(p, s); break;
      case CX_F16: rc = launch_bulk<__half>(p, s); break;
      default: return cx_set_error("cx_compress: unsupported dtype on CUDA", 0);
    }
    if (rc) return rc;
    cx_note_launch();
    return cx_check_launch("compress_bulk_kernel");
  }
  int grid = cx_sm_count() * CX_COMPRESS_MIN_BLOCKS;
  const int need = (int)((p.nsub + kWarps - 1) / kWarps);
  if (grid > need) grid = need;
  switch (gdtype) {
    case CX_F32: launch_mode<float>(p, grid, s); break;
    case CX_BF16: launch_mode<__nv_bfloat16>(p, grid, s); break;
    case CX_F16: launch_mode<__half>(p, grid, s); break;
    default: return cx_set_error("cx_compress: unsupported dtype on CUDA", 0);
  }
  cx_note_launch();
  return cx_check_launch("compress_kernel");
}
