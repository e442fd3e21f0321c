// Dense allreduce through the NVSwitch's multicast / in-switch reduction (multimem.*).
//
// The reference's dense collectives (src/allreduce.tpp:73-118, 319-351, 571-601) move the
// vector hop by hop through registered buffers.  Behind an NVSwitch whose memory is bound to
// a multicast object, one instruction reads the same address on every GPU and returns the
// sum (multimem.ld_reduce), and one instruction stores to the same address on every GPU
// (multimem.st).  This file is the whole allreduce as ONE kernel per rank:
//
//   copy-in    the user's vector goes into this rank's symmetric staging block (skipped when
//              the vector already lives in the symmetric heap),
//   publish    the CTA that finishes last tells every peer "my slab k is ready",
//   reduce     after all peers' "ready": rank r pulls the sum of its 1/P share of the slab out
//              of the switch, scales it, and stores it to every rank's staging block at once,
//   publish    "my share of slab k is broadcast",
//   copy-out   after all peers' "done": the slab goes back into the user's vector.
//
// The vector is cut into slabs and the three stages run as three groups of CTAs of the same
// kernel, each looping over the slabs on its own and meeting the others only through the flags:
// while one group waits for the peers, the other two work, so HBM copies, the pull direction
// and the push direction of the links are busy at the same time.  Small vectors use
// the one-shot form: every rank pulls the WHOLE sum out of the switch straight into its own
// output, one exchange instead of two; staging is then double-buffered by the parity of the
// call, because a fast rank may start its next call while a slow one still reads.
//
// Every wait has a time budget.  A CTA whose wait runs out stops touching memory, still
// arrives at every completion counter (so the counters are clean for the next launch), and
// marks the launch as failed: the last CTA then publishes nothing, the peers time out in
// turn, and the host reads CX_ST_TIMEOUT from the status word.
#include <stdlib.h>

#include "cx_device.cuh"

namespace {

constexpr int kThreads = 512;
constexpr int kMaxSlabs = 1000;   // flag values are seq * 1024 + slab + 1

struct MmParams {
  void* out;                 // user's vector (may be the staging block itself)
  const void* in;
  char* stage;               // this rank's staging block (local address), parity 0
  char* stage_mc;            // the same block through the multicast mapping
  int64_t stage_stride;      // bytes between the two parities (one-shot) or 0
  int64_t n;                 // elements
  int32_t rank, ranks;
  int32_t staged;            // 1: copy-in / copy-out run; 0: the vector is the staging block
  int32_t bulk;              // 1: the copy groups move their slabs with the SM's copy engine
  int32_t one_shot;
  int64_t slab_vec;          // 16-byte vectors per slab
  int32_t nslabs;
  int32_t n_in, n_red;       // CTAs that copy in / that reduce; the rest of the grid copies out
  float scale;
  uint64_t seq;
  const uint64_t* seq_cell;  // non-NULL inside a captured graph
  uint64_t* flags;           // local: ready[CX_MAX_PEERS] then done[CX_MAX_PEERS], written by peers
  uint64_t* peer_flags[CX_MAX_PEERS];   // the same block on every rank (peer-mapped; [rank] is local)
  uint32_t* ctr;             // local, zeroed: [0] failure mark, [1 + 2 k + phase] arrivals
  uint32_t* status;
  uint64_t timeout_ns;
};

template <typename T> struct MM;
template <> struct MM<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    v.x = __float_as_uint(__uint_as_float(v.x) * s); v.y = __float_as_uint(__uint_as_float(v.y) * s);
    v.z = __float_as_uint(__uint_as_float(v.z) * s); v.w = __float_as_uint(__uint_as_float(v.w) * s);
    return v;
  }
};
template <> struct MM<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint32_t scale2(uint32_t u, float s) {
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
    h = __floats2bfloat162_rn(__low2float(h) * s, __high2float(h) * s);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    v.x = scale2(v.x, s); v.y = scale2(v.y, s); v.z = scale2(v.z, s); v.w = scale2(v.w, s);
    return v;
  }
};
template <> struct MM<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint32_t scale2(uint32_t u, float s) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    h = __floats2half2_rn(__low2float(h) * s, __high2float(h) * s);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    v.x = scale2(v.x, s); v.y = scale2(v.y, s); v.z = scale2(v.z, s); v.w = scale2(v.w, s);
    return v;
  }
};

// The stores of a group of `group` CTAs are fenced; the CTA that arrives last publishes `value` into slot
// [which * CX_MAX_PEERS + rank] of every rank's flag block (unless the launch is marked failed).
__device__ __forceinline__ void arrive_and_publish(const MmParams& p, int counter, int group, int which,
                                                   uint64_t value, uint32_t* s_last) {
  if (!cx::cta_arrive(&p.ctr[1 + counter], (uint32_t)group, s_last)) return;
  const uint32_t failed = *reinterpret_cast<volatile uint32_t*>(&p.ctr[0]);
  if (!failed && (int)threadIdx.x < p.ranks)
    cx::st_release_sys(p.peer_flags[threadIdx.x] + which * CX_MAX_PEERS + p.rank, value);
  if (threadIdx.x == 0) p.ctr[1 + counter] = 0;
  __syncthreads();
}

// Every CTA waits until all ranks published `value` in slot group `which`.  Uniform result.
__device__ __forceinline__ bool wait_all(const MmParams& p, int which, uint64_t value, uint32_t* s_bad) {
  if (threadIdx.x == 0) *s_bad = 0;
  __syncthreads();
  if ((int)threadIdx.x < p.ranks)
    if (!cx::wait_seq(p.flags + which * CX_MAX_PEERS + threadIdx.x, value, p.timeout_ns)) atomicOr(s_bad, 1u);
  __syncthreads();
  const bool ok = *s_bad == 0;
  if (!ok && threadIdx.x == 0) {
    if (p.status) atomicOr(p.status, (uint32_t)CX_ST_TIMEOUT);
    atomicOr(&p.ctr[0], 1u);
  }
  __syncthreads();
  return ok;
}

#ifndef CX_MM_COPY_SHARE
#define CX_MM_COPY_SHARE 6     // one CTA in this many copies in, one copies out (2^28 fp32, 4 GPUs: 24 CTAs 2948 us, 14 CTAs 3324 us, 8 CTAs 4003 us)
#endif
#ifndef CX_MM_COPY_UNROLL
#define CX_MM_COPY_UNROLL 16   // 16-byte loads in flight per thread of a copy group
#endif

// The copy groups are small (most CTAs reduce), so each of their threads keeps many loads in
// flight: with 4 per thread a CTA moved ~25 GB/s and the copies, not the switch, set the pace.
__device__ __forceinline__ void copy_vec(uint4* dst, const uint4* src, int64_t nv, int64_t gtid, int64_t gsz,
                                         bool through_l2) {
  int64_t q = gtid;
  for (; q + (CX_MM_COPY_UNROLL - 1) * gsz < nv; q += CX_MM_COPY_UNROLL * gsz) {
    uint4 v[CX_MM_COPY_UNROLL];
#pragma unroll
    for (int u = 0; u < CX_MM_COPY_UNROLL; ++u) v[u] = through_l2 ? __ldcg(src + q + u * gsz) : __ldcs(src + q + u * gsz);
#pragma unroll
    for (int u = 0; u < CX_MM_COPY_UNROLL; ++u) {
      if (through_l2) __stcs(dst + q + u * gsz, v[u]);
      else dst[q + u * gsz] = v[u];
    }
  }
  for (; q < nv; q += gsz) dst[q] = through_l2 ? __ldcg(src + q) : src[q];
}

#ifndef CX_MM_UNROLL
#define CX_MM_UNROLL 8    // pulls in flight per thread: a round trip through the switch takes microseconds
#endif

// Pull the sum of vectors [a, b) out of the switch, scale, broadcast.  tid / tsz: this thread's
// index and the thread count of the CTAs that share the range.
template <typename T>
__device__ __forceinline__ void reduce_broadcast(char* stage_mc, int64_t a, int64_t b, int64_t tid, int64_t tsz,
                                                 float scale) {
  int64_t q = a + tid;
  for (; q + (CX_MM_UNROLL - 1) * tsz < b; q += CX_MM_UNROLL * tsz) {
    uint4 v[CX_MM_UNROLL];
#pragma unroll
    for (int u = 0; u < CX_MM_UNROLL; ++u) v[u] = MM<T>::ld_reduce(stage_mc + (q + u * tsz) * 16);
    if (scale != 1.f) {
#pragma unroll
      for (int u = 0; u < CX_MM_UNROLL; ++u) v[u] = MM<T>::scale(v[u], scale);
    }
#pragma unroll
    for (int u = 0; u < CX_MM_UNROLL; ++u) cx::mm_st_v4(stage_mc + (q + u * tsz) * 16, v[u]);
  }
  for (; q < b; q += tsz) {
    uint4 v = MM<T>::ld_reduce(stage_mc + q * 16);
    if (scale != 1.f) v = MM<T>::scale(v, scale);
    cx::mm_st_v4(stage_mc + q * 16, v);
  }
}

// Copy the part of slab [v0, v1) (16-byte vectors of the staging block) that the user's vector
// covers, in either direction.  The ragged last vector goes element by element; on the way in its
// padding is zeroed.
template <typename T, bool IN>
__device__ __forceinline__ void copy_slab(const MmParams& p, char* stage, int64_t v0, int64_t v1, int64_t full,
                                          int64_t nvec, int64_t tid, int64_t tsz, bool user_vec,
                                          bool body_done = false) {
  constexpr int64_t kPer = 16 / (int64_t)sizeof(T);
  const int64_t vf = min(v1, full);
  T* st = reinterpret_cast<T*>(stage);
  if (body_done) {
    // the complete 16-byte vectors went through the copy engine; only the ragged end is left
  } else if (user_vec) {
    if (vf > v0) {
      if (IN) copy_vec(reinterpret_cast<uint4*>(stage) + v0, reinterpret_cast<const uint4*>(p.in) + v0, vf - v0, tid, tsz, false);
      else copy_vec(reinterpret_cast<uint4*>(p.out) + v0, reinterpret_cast<const uint4*>(stage) + v0, vf - v0, tid, tsz, true);
    }
  } else {
    const int64_t e0 = v0 * kPer, e1 = min(p.n, vf * kPer);
    if (IN) for (int64_t i = e0 + tid; i < e1; i += tsz) st[i] = reinterpret_cast<const T*>(p.in)[i];
    else for (int64_t i = e0 + tid; i < e1; i += tsz) reinterpret_cast<T*>(p.out)[i] = __ldcg(st + i);
  }
  if (v1 > full) {
    if (IN) {
      for (int64_t i = full * kPer + tid; i < nvec * kPer; i += tsz)
        st[i] = i < p.n ? reinterpret_cast<const T*>(p.in)[i] : cx::Elem<T>::from_f(0.f);
    } else {
      for (int64_t i = full * kPer + tid; i < p.n; i += tsz) reinterpret_cast<T*>(p.out)[i] = __ldcg(st + i);
    }
  }
}

// ---- staging copies by the SM's copy engine --------------------------------------------------------
// A copy group is a handful of CTAs (most of the grid reduces), and with vector loads and stores
// one SM moves 20-30 GB/s: the copies, not the switch, set the pace of the staged allreduce.  Here
// ONE thread per copy CTA drives a ring of kBulkStages chunks in shared memory: bulk load of a
// chunk (local global memory -> shared memory, counted in bytes on the stage's mbarrier), bulk
// store of the landed chunk (shared -> local global memory, one bulk group per chunk), the next
// load into a stage once the store that used it has read it.  Source and destination are this
// GPU's own memory (the user's vector and this rank's staging block), 16-byte aligned, sizes
// multiples of 16 bytes; nothing here is a multicast load.  Every mbarrier wait is bounded.
constexpr int kBulkStages = 6;
constexpr uint32_t kBulkChunk = 32 * 1024;
constexpr size_t kBulkSmem = (size_t)kBulkStages * kBulkChunk + 8 * kBulkStages;

// Chunks part, part + parts, ... of [src, src + bytes) go to dst.  `q` counts the loads this thread
// has issued since the kernel began (stage and mbarrier phase follow from it).  False: a load did
// not land in time (the copies still in flight were given a bounded chance to).
__device__ __forceinline__ bool bulk_copy_range(char* dst, const char* src, int64_t bytes, int part, int parts,
                                                unsigned char* sbuf, uint64_t* bars, uint32_t& q) {
  const int64_t nchunks = (bytes + kBulkChunk - 1) / kBulkChunk;
  const int64_t cnt = nchunks > part ? (nchunks - part + parts - 1) / parts : 0;
  auto off = [&](int64_t i) { return ((int64_t)part + i * parts) * (int64_t)kBulkChunk; };
  auto len = [&](int64_t i) { return (uint32_t)min((int64_t)kBulkChunk, bytes - off(i)); };
  auto load = [&](int64_t i) {
    const uint32_t s = (q + (uint32_t)i) % kBulkStages;
    cx::mbar_expect_tx(&bars[s], len(i));
    cx::bulk_load(sbuf + (size_t)s * kBulkChunk, src + off(i), len(i), &bars[s]);
  };
  int64_t loaded = 0;
  for (; loaded < cnt && loaded < kBulkStages - 1; ++loaded) load(loaded);
  for (int64_t i = 0; i < cnt; ++i) {
    if (loaded < cnt) {
      cx::bulk_wait_read_all();        // the store that used this stage (chunk i - 1) has read it
      load(loaded++);
    }
    const uint32_t c = q + (uint32_t)i;
    if (!cx::mbar_wait_bounded(&bars[c % kBulkStages], (c / kBulkStages) & 1u)) {
      for (int64_t j = i + 1; j < loaded; ++j) {
        const uint32_t d = q + (uint32_t)j;
        cx::mbar_wait_bounded(&bars[d % kBulkStages], (d / kBulkStages) & 1u);
      }
      cx::bulk_wait_all();
      q += (uint32_t)loaded;
      return false;
    }
    cx::bulk_store(dst + off(i), sbuf + (size_t)(c % kBulkStages) * kBulkChunk, len(i));
    cx::bulk_commit();
  }
  cx::bulk_wait_all();                  // the stores are complete: what follows may publish them
  q += (uint32_t)cnt;
  return true;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1) mm_allreduce_kernel(const MmParams p) {
  extern __shared__ __align__(128) unsigned char s_dyn[];
  __shared__ uint32_t s_last, s_bad;
  const uint64_t seq = cx::seq_of(p.seq_cell, p.seq);
  const int64_t bytes = p.n * (int64_t)sizeof(T);
  const int64_t nvec = (bytes + 15) / 16;           // 16-byte vectors, the last one may be partial
  const int64_t full = bytes / 16;                   // vectors the user's buffer holds completely
  const int64_t par_off = p.one_shot ? (int64_t)(seq & 1) * p.stage_stride : 0;
  char* stage = p.stage + par_off;
  char* stage_mc = p.stage_mc + par_off;
  const bool user_vec = ((reinterpret_cast<uintptr_t>(p.in) | reinterpret_cast<uintptr_t>(p.out)) & 15) == 0;
  bool alive = true;

  // the failure mark is cleared by whoever leaves last
  auto leave = [&]() {
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&p.ctr[1 + 2 * kMaxSlabs], 1u) == gridDim.x - 1) {
      p.ctr[1 + 2 * kMaxSlabs] = 0;
      p.ctr[0] = 0;
    }
  };

  if (p.one_shot) {
    // one exchange: everybody pulls the whole sum out of the switch into its own output
    const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const int64_t gsz = (int64_t)gridDim.x * kThreads;
    copy_slab<T, true>(p, stage, 0, nvec, full, nvec, gtid, gsz, user_vec);
    arrive_and_publish(p, 0, gridDim.x, 0, seq * 1024 + 1, &s_last);
    alive = wait_all(p, 0, seq * 1024 + 1, &s_bad);
    if (alive) {
      const bool out_vec = (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
      for (int64_t q = gtid; q < nvec; q += gsz) {
        uint4 v = MM<T>::ld_reduce(stage_mc + q * 16);
        if (p.scale != 1.f) v = MM<T>::scale(v, p.scale);
        if (out_vec && q < full) {
          reinterpret_cast<uint4*>(p.out)[q] = v;
        } else {
          const T* e = reinterpret_cast<const T*>(&v);
          const int64_t i0 = q * (16 / (int64_t)sizeof(T));
          for (int j = 0; j < (int)(16 / sizeof(T)); ++j)
            if (i0 + j < p.n) reinterpret_cast<T*>(p.out)[i0 + j] = e[j];
        }
      }
    }
    leave();
    return;
  }

  // Three roles, each a group of CTAs with its own loop over the slabs; the groups meet only
  // through the flags, so the waits of one group are covered by the work of the others:
  //   copy-in  CTAs [0, n_in)            user vector -> staging, then "slab k ready" to all ranks
  //   reduce   CTAs [n_in, n_in + n_red)  all ranks ready -> pull sum, broadcast, "slab k done"
  //   copy-out CTAs [n_in + n_red, grid)  all ranks done -> staging -> user vector
  // Without staging (the vector lives in the symmetric heap) only the reduce group exists; it
  // announces "ready" itself and does not leave before every rank's broadcast has landed.
  const int b = blockIdx.x;
  const bool bulk = p.bulk && user_vec;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dyn + (size_t)kBulkStages * kBulkChunk);
  uint32_t bulk_q = 0;
  bool bulk_ok = true;
  if (bulk && (b < p.n_in || b >= p.n_in + p.n_red)) {
    if (threadIdx.x == 0) {
      for (int s = 0; s < kBulkStages; ++s) cx::mbar_init(&bars[s], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      cx::fence_proxy_async();
    }
    __syncthreads();
  }
  // a copy that did not land: the launch is marked failed, nothing more is published
  auto bulk_failed = [&]() {
    if (p.status) atomicOr(p.status, (uint32_t)CX_ST_TIMEOUT);
    atomicOr(&p.ctr[0], 1u);
  };
  if (b < p.n_in) {
    const int64_t tid = (int64_t)b * kThreads + threadIdx.x, tsz = (int64_t)p.n_in * kThreads;
    for (int k = 0; k < p.nslabs; ++k) {
      const int64_t v0 = (int64_t)k * p.slab_vec, v1 = min(nvec, v0 + p.slab_vec);
      if (bulk) {
        const int64_t vf = min(v1, full);
        if (threadIdx.x == 0 && bulk_ok && vf > v0) {
          bulk_ok = bulk_copy_range(stage + v0 * 16, reinterpret_cast<const char*>(p.in) + v0 * 16, (vf - v0) * 16, b,
                                    p.n_in, s_dyn, bars, bulk_q);
          if (!bulk_ok) bulk_failed();
          cx::fence_proxy_async();     // the copy engine's writes, then the release of the flag
        }
      }
      copy_slab<T, true>(p, stage, v0, v1, full, nvec, tid, tsz, user_vec, bulk);
      arrive_and_publish(p, 2 * k, p.n_in, 0, seq * 1024 + (k + 1), &s_last);
    }
  } else if (b < p.n_in + p.n_red) {
    const int64_t tid = (int64_t)(b - p.n_in) * kThreads + threadIdx.x, tsz = (int64_t)p.n_red * kThreads;
    if (!p.staged) arrive_and_publish(p, 0, p.n_red, 0, seq * 1024 + 1, &s_last);
    for (int k = 0; k < p.nslabs; ++k) {
      if (alive) alive = wait_all(p, 0, seq * 1024 + (k + 1), &s_bad);
      if (alive) {
        const int64_t v0 = (int64_t)k * p.slab_vec, v1 = min(nvec, v0 + p.slab_vec);
        const int64_t per = (v1 - v0 + p.ranks - 1) / p.ranks;
        const int64_t lo = v0 + per * p.rank, hi = min(v1, lo + per);
        reduce_broadcast<T>(stage_mc, lo, hi, tid, tsz, p.scale);
      }
      arrive_and_publish(p, 2 * k + 1, p.n_red, 1, seq * 1024 + (k + 1), &s_last);
    }
    if (!p.staged && alive) alive = wait_all(p, 1, seq * 1024 + p.nslabs, &s_bad);
  } else {
    const int n_out = (int)gridDim.x - p.n_in - p.n_red;
    const int64_t tid = (int64_t)(b - p.n_in - p.n_red) * kThreads + threadIdx.x, tsz = (int64_t)n_out * kThreads;
    for (int k = 0; k < p.nslabs && alive; ++k) {
      alive = wait_all(p, 1, seq * 1024 + (k + 1), &s_bad);
      if (!alive) break;
      const int64_t v0 = (int64_t)k * p.slab_vec, v1 = min(nvec, v0 + p.slab_vec);
      if (bulk) {
        const int64_t vf = min(v1, full);
        if (threadIdx.x == 0 && bulk_ok && vf > v0) {
          cx::fence_proxy_async();     // the acquire of the flags, then the copy engine's reads
          bulk_ok = bulk_copy_range(reinterpret_cast<char*>(p.out) + v0 * 16, stage + v0 * 16, (vf - v0) * 16,
                                    b - p.n_in - p.n_red, n_out, s_dyn, bars, bulk_q);
          if (!bulk_ok) bulk_failed();
        }
      }
      copy_slab<T, false>(p, stage, v0, v1, full, nvec, tid, tsz, user_vec, bulk);
    }
  }
  leave();
}

// ---- barrier over the symmetric heap -------------------------------------------------------------
// Every rank stores the barrier's number into its cell of every peer's flag block (release, system
// scope) and waits, bounded, until all cells of its own block carry that number: the GASPI
// barrier of the reference (src/gaspiEnvironment.tpp:33-35) as one small kernel on the caller's
// stream, no library collective involved.
struct BarrierParams {
  uint64_t* flags;                       // local block, one cell per rank
  uint64_t* peer_flags[CX_MAX_PEERS];
  int32_t rank, ranks;
  uint64_t seq;
  uint32_t* status;
  uint64_t timeout_ns;
};

__global__ void barrier_kernel(const BarrierParams p) {
  const int t = threadIdx.x;
  if (t < p.ranks) {
    __threadfence_system();
    cx::st_release_sys(p.peer_flags[t] + p.rank, p.seq);
    if (!cx::wait_seq(p.flags + t, p.seq, p.timeout_ns) && p.status) atomicOr(p.status, (uint32_t)CX_ST_TIMEOUT);
  }
}

}  // namespace

int cx_barrier_cuda(int rank, int ranks, void* const* flag_ptrs, uint64_t seq, uint32_t* status,
                    uint64_t timeout_ns, void* stream) {
  if (ranks < 1 || ranks > CX_MAX_PEERS || rank < 0 || rank >= ranks) return cx_set_error("cx_barrier: bad rank", 0);
  BarrierParams p;
  p.flags = reinterpret_cast<uint64_t*>(flag_ptrs[rank]);
  for (int r = 0; r < CX_MAX_PEERS; ++r) p.peer_flags[r] = r < ranks ? reinterpret_cast<uint64_t*>(flag_ptrs[r]) : nullptr;
  p.rank = rank; p.ranks = ranks; p.seq = seq; p.status = status; p.timeout_ns = timeout_ns;
  barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  cx_note_launch();
  return cx_check_launch("barrier_kernel");
}

extern "C" int64_t cx_mm_counter_bytes(void) { return (int64_t)sizeof(uint32_t) * (2 + 2 * kMaxSlabs + 2); }
#ifndef CX_MM_BULK_DEFAULT
#define CX_MM_BULK_DEFAULT 0
#endif

namespace {
template <typename T>
int launch_mm(const MmParams& p, int grid, size_t smem, cudaStream_t s) {
  auto kern = mm_allreduce_kernel<T>;
  if (smem) {
    static bool configured[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cx_set_error("cx_mm_allreduce: cudaGetDevice", 0);
    if (!configured[dev]) {
      const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cx_set_error("cx_mm_allreduce: shared memory opt-in", (int)e);
      configured[dev] = true;
    }
  }
  kern<<<grid, kThreads, smem, s>>>(p);
  return 0;
}
}  // namespace

extern "C" int64_t cx_mm_flag_bytes(void) { return (int64_t)sizeof(uint64_t) * 2 * CX_MAX_PEERS; }

// See cx_common.h.  `stage` / `stage_mc`: this rank's block and its multicast alias (when `in`
// is NULL the vector itself lives there and nothing is copied); `flag_ptrs[r]`: rank r's flag
// block (cx_mm_flag_bytes, zeroed once); `counters`: local scratch (cx_mm_counter_bytes, zeroed
// once).  one_shot: the staging block holds two copies `stage_stride` bytes apart.
int cx_mm_allreduce_cuda(int dtype, void* out, const void* in, void* stage, void* stage_mc,
                         int64_t stage_stride, int64_t n, int rank, int ranks, float scale, int one_shot,
                         int64_t slab_bytes, uint64_t seq, void* const* flag_ptrs, void* counters,
                         uint32_t* status, uint64_t timeout_ns, void* stream) {
  if (ranks < 1 || ranks > CX_MAX_PEERS || rank < 0 || rank >= ranks) return cx_set_error("cx_mm_allreduce: bad rank", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_mm_allreduce: n out of range", 0);
  if (!stage || !stage_mc) return cx_set_error("cx_mm_allreduce: no multicast mapping", 0);
  if ((reinterpret_cast<uintptr_t>(stage) | reinterpret_cast<uintptr_t>(stage_mc)) & 15)
    return cx_set_error("cx_mm_allreduce: staging block must be 16-byte aligned", 0);
  if (n == 0) return 0;
  const int64_t esz = dtype == CX_F32 ? 4 : 2;
  MmParams p;
  p.out = out; p.in = in; p.stage = reinterpret_cast<char*>(stage); p.stage_mc = reinterpret_cast<char*>(stage_mc);
  p.stage_stride = stage_stride; p.n = n; p.rank = rank; p.ranks = ranks;
  p.staged = in != nullptr;
  p.one_shot = one_shot;
  if (!p.staged) {
    if (one_shot) return cx_set_error("cx_mm_allreduce: the one-shot form needs a staging block", 0);
    if ((n * esz) % 16) return cx_set_error("cx_mm_allreduce: in-place vectors must be a multiple of 16 bytes", 0);
    p.out = stage;
  }
  const int64_t nvec = (n * esz + 15) / 16;
  int64_t slab_vec = slab_bytes > 0 ? slab_bytes / 16 : nvec;
  if (slab_vec < 1 || one_shot) slab_vec = nvec;
  if ((nvec + slab_vec - 1) / slab_vec > kMaxSlabs) slab_vec = (nvec + kMaxSlabs - 1) / kMaxSlabs;
  p.slab_vec = slab_vec;
  p.nslabs = (int)((nvec + slab_vec - 1) / slab_vec);
  p.scale = scale; p.seq = seq; p.seq_cell = cx_seq_cell();
  p.flags = reinterpret_cast<uint64_t*>(flag_ptrs[rank]);
  for (int r = 0; r < CX_MAX_PEERS; ++r) p.peer_flags[r] = r < ranks ? reinterpret_cast<uint64_t*>(flag_ptrs[r]) : nullptr;
  p.ctr = reinterpret_cast<uint32_t*>(counters);
  p.status = status; p.timeout_ns = timeout_ns;
  // every CTA may wait for peers or for another group: one co-resident wave, one CTA per SM at most
  int grid = cx_sm_count();
  const int64_t need = (nvec + kThreads - 1) / kThreads;
  if (grid > need) grid = (int)need;
  if (grid < 1) grid = 1;
  p.n_in = 0;
  p.n_red = grid;
  if (p.staged && !one_shot) {
    // the copies run at HBM speed, the reduction at link speed: most CTAs reduce
    if (grid < 3) grid = 3;
    int copy = grid / CX_MM_COPY_SHARE;
    if (const char* e = getenv("COMPREX_MM_COPY_CTAS")) copy = atoi(e);
    if (copy < 1) copy = 1;
    if (2 * copy > grid - 1) copy = (grid - 1) / 2;
    p.n_in = copy;
    p.n_red = grid - 2 * copy;
  }
  // COMPREX_MM_BULK (read per call): the copy groups use the copy engine
  p.bulk = 0;
  if (p.staged && !one_shot) {
    const char* e = getenv("COMPREX_MM_BULK");
    p.bulk = e ? atoi(e) != 0 : (CX_MM_BULK_DEFAULT != 0);
  }
  const size_t smem = p.bulk ? kBulkSmem : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc = 0;
  switch (dtype) {
    case CX_F32: rc = launch_mm<float>(p, grid, smem, s); break;
    case CX_BF16: rc = launch_mm<__nv_bfloat16>(p, grid, smem, s); break;
    case CX_F16: rc = launch_mm<__half>(p, grid, smem, s); break;
    default: return cx_set_error("cx_mm_allreduce: unsupported dtype", 0);
  }
  if (rc) return rc;
  cx_note_launch();
  return cx_check_launch("mm_allreduce_kernel");
}
