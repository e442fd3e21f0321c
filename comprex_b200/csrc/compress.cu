// Fused residual-add / threshold-select / ordered compaction / peer store.
//
// One pass over the vector does what the reference does in
// ThresholdFunction + CompressorIndexPairs::compress_add_update followed by
// SourceBuffer::initTransferPart (src/compressor.hxx:556-611,
// src/comprEx.tpp:176-191):
//
//     r += g ; if |r| > thr { emit (i, r) ; r = 0 }
//
// The survivors leave the SM exactly once, as coalesced 8-byte (index, value)
// stores that go straight into the receive slots of up to CX_MAX_PEERS
// targets (peer GPUs' memory mapped over NVLink, or local slots).  Output is
// in ascending index order like the reference's wire format: tiles are handed
// out by an atomic counter and chained with a single-pass decoupled look-back
// scan, so no second pass over the data and no sort is needed.  As a
// by-product every 1024-element sub-tile's offset into the pair list is
// written next to the pairs; receivers use it to find, without searching, the
// pairs that fall into the part of the vector they own.
//
// Survivors that do not fit into the slot (position >= cap) are not emitted
// and stay in the residual, which error feedback makes safe; the count is
// reported.  The CTA that finishes last writes the header and publishes the
// notification (st.release.sys) after every CTA's stores were fenced at
// system scope.
#include "cx_device.cuh"

namespace {

constexpr int kThreads = 256;
constexpr uint64_t kFlagAgg = 1ull << 32;
constexpr uint64_t kFlagIncl = 2ull << 32;
constexpr uint64_t kFlagMask = 3ull << 32;

struct CompressParams {
  const void* g;
  float* r;
  int64_t n;
  const float* thr;
  uint32_t cap;
  uint32_t ntiles;
  uint32_t nsub;
  uint32_t epoch;
  uint64_t seq;
  CxWorkCounters* ctr;
  uint64_t* tile_status;
  CxStats* stats;
  uint32_t src_rank;
  uint32_t spin_limit;
  CxTargets tg;
};

__device__ __forceinline__ uint64_t shfl_up64(uint64_t v, int d) {
  return __shfl_up_sync(0xffffffffu, (unsigned long long)v, d);
}

// T: element type of g.  HAS_G / HAS_R select compress_add_update (both),
// compress_update (r only) and compress (g only).  VEC: 16-byte aligned views.
template <typename T, bool HAS_G, bool HAS_R, bool VEC>
__global__ void __launch_bounds__(kThreads, 4) compress_kernel(const CompressParams p) {
  __shared__ CxPair s_pairs[CX_TILE];
  __shared__ uint64_t s_wtot[kThreads / 32];
  __shared__ uint32_t s_tile;
  __shared__ uint32_t s_base;
  __shared__ uint32_t s_last;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const float thr = *p.thr;
  const T* __restrict__ g = reinterpret_cast<const T*>(p.g);
  float* __restrict__ r = p.r;
  const uint64_t ep_tag = (uint64_t)p.epoch << 34;

  for (;;) {
    if (tid == 0) s_tile = atomicAdd(&p.ctr->next_tile, 1u);
    __syncthreads();
    const uint32_t tile = s_tile;
    if (tile >= p.ntiles) break;
    const int64_t tile_base = (int64_t)tile * CX_TILE;

    // ---- load, add, classify ------------------------------------------
    float v[CX_SUBS_PER_TILE][4];
    uint32_t mask = 0;  // bit c*4+e
    uint64_t packed = 0;
#pragma unroll
    for (int c = 0; c < CX_SUBS_PER_TILE; ++c) {
      const int64_t i0 = tile_base + c * CX_SUBTILE + tid * 4;
      if (VEC && i0 + 3 < p.n) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
        if (HAS_R) cx::load4(r + i0, a);
        if (HAS_G) cx::load4(g + i0, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[c][e] = a[e] + b[e];
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float a = 0.f, b = 0.f;
          if (i0 + e < p.n) {
            if (HAS_R) a = r[i0 + e];
            if (HAS_G) b = cx::Elem<T>::to_f(g[i0 + e]);
          }
          v[c][e] = a + b;
        }
      }
      uint32_t m = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (fabsf(v[c][e]) > thr && i0 + e < p.n) m |= 1u << e;  // strict '>' like the reference
      mask |= m << (4 * c);
      packed |= (uint64_t)__popc(m) << (16 * c);
    }

    // ---- block exclusive scan of the four packed counters ---------------
    uint64_t incl = packed;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint64_t t = shfl_up64(incl, d);
      if (lane >= d) incl += t;
    }
    if (lane == 31) s_wtot[warp] = incl;
    __syncthreads();
    uint64_t woff = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) {
      const uint64_t t = s_wtot[w];
      if (w < warp) woff += t;
      total += t;
    }
    const uint64_t excl = incl - packed + woff;
    const uint32_t t0 = (uint32_t)(total & 0xffff), t1 = (uint32_t)((total >> 16) & 0xffff),
                   t2 = (uint32_t)((total >> 32) & 0xffff), t3 = (uint32_t)((total >> 48) & 0xffff);
    const uint32_t coff[CX_SUBS_PER_TILE] = {0u, t0, t0 + t1, t0 + t1 + t2};
    const uint32_t tile_count = t0 + t1 + t2 + t3;

    // ---- decoupled look-back: exclusive prefix over earlier tiles -------
    if (warp == 0) {
      if (lane == 0)
        cx::st_relaxed_gpu(&p.tile_status[tile],
                           ep_tag | (tile == 0 ? kFlagIncl : kFlagAgg) | tile_count);
      uint32_t exclusive = 0;
      bool failed = false;
      int64_t look = (int64_t)tile - 1;
      while (look >= 0) {
        const int64_t idx = look - lane;
        uint64_t st = kFlagIncl;  // virtual predecessor before tile 0: inclusive, value 0
        if (idx >= 0) {
          uint32_t spins = 0;
          for (;;) {
            st = cx::ld_relaxed_gpu(&p.tile_status[idx]);
            if ((st >> 34) == p.epoch && (st & kFlagMask)) break;
            if (++spins > p.spin_limit) { failed = true; st = kFlagIncl; break; }
            __nanosleep(20);
          }
        }
        const uint32_t incl_lanes = __ballot_sync(0xffffffffu, (st & kFlagMask) == kFlagIncl);
        const int first = __ffs(incl_lanes) - 1;  // nearest predecessor with an inclusive prefix
        uint32_t val = (first < 0 || lane <= first) ? (uint32_t)(st & 0xffffffffu) : 0u;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) val += __shfl_xor_sync(0xffffffffu, val, d);
        exclusive += val;
        if (first >= 0) break;
        look -= 32;
      }
      failed = __any_sync(0xffffffffu, failed);
      if (lane == 0) {
        if (failed) atomicOr(&p.ctr->error, CX_ST_LOOKBACK);
        cx::st_relaxed_gpu(&p.tile_status[tile], ep_tag | kFlagIncl | (exclusive + tile_count));
        s_base = exclusive;
      }
    }

    // ---- stage survivors in shared memory, in index order ---------------
#pragma unroll
    for (int c = 0; c < CX_SUBS_PER_TILE; ++c) {
      uint32_t pos = coff[c] + (uint32_t)((excl >> (16 * c)) & 0xffff);
      const int32_t i0 = (int32_t)(tile_base + c * CX_SUBTILE + tid * 4);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (mask & (1u << (4 * c + e))) {
          CxPair pr;
          pr.idx = i0 + e;
          pr.val = __float_as_uint(v[c][e]);
          s_pairs[pos++] = pr;
        }
      }
    }
    __syncthreads();
    const uint32_t base = s_base;

    // ---- residual: zero what was emitted, keep the rest ------------------
    if (HAS_R) {
#pragma unroll
      for (int c = 0; c < CX_SUBS_PER_TILE; ++c) {
        const uint32_t m = (mask >> (4 * c)) & 0xfu;
        if (!HAS_G && m == 0) continue;  // nothing changed in this vector
        uint32_t pos = base + coff[c] + (uint32_t)((excl >> (16 * c)) & 0xffff);
        const int64_t i0 = tile_base + c * CX_SUBTILE + tid * 4;
        float out[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const bool sel = m & (1u << e);
          out[e] = (sel && pos < p.cap) ? 0.f : v[c][e];
          pos += sel ? 1u : 0u;
        }
        if (VEC && i0 + 3 < p.n) {
          cx::store4(r + i0, out);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (i0 + e < p.n) r[i0 + e] = out[e];
        }
      }
    }

    // ---- sub-tile offsets and the pairs themselves, to every target ------
    if (tid < CX_SUBS_PER_TILE) {
      const uint32_t sub = tile * CX_SUBS_PER_TILE + tid;
      if (sub < p.nsub) {
        const uint32_t before = tid == 0 ? 0u : tid == 1 ? t0 : tid == 2 ? t0 + t1 : t0 + t1 + t2;
        const uint32_t off = min(base + before, p.cap);
        for (int k = 0; k < p.tg.count; ++k) p.tg.ep[k].prefix[sub] = off;
      }
    }
    if (tile == p.ntiles - 1 && tid == 0) {
      const uint32_t found = base + tile_count;
      for (int k = 0; k < p.tg.count; ++k) p.tg.ep[k].prefix[p.nsub] = min(found, p.cap);
      p.ctr->nnz_found = found;
    }
    for (uint32_t i = tid; i < tile_count; i += kThreads) {
      const uint32_t gpos = base + i;
      if (gpos < p.cap) {
        const CxPair pr = s_pairs[i];
        for (int k = 0; k < p.tg.count; ++k) p.tg.ep[k].pairs[gpos] = pr;
      }
    }
    __syncthreads();  // s_pairs, s_tile, s_base are reused by the next tile
  }

  // ---- completion: the CTA that arrives last publishes ---------------------
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const uint32_t prev = atomicAdd(&p.ctr->done, 1u);
    s_last = (prev == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const uint32_t found = *reinterpret_cast<volatile uint32_t*>(&p.ctr->nnz_found);
  const uint32_t err = *reinterpret_cast<volatile uint32_t*>(&p.ctr->error);
  const uint32_t nnz = err ? 0u : min(found, p.cap);
  if (tid < p.tg.count) {
    CxHeader* h = p.tg.ep[tid].hdr;
    h->bytes = 8ull + 8ull * nnz;
    h->n = (uint32_t)p.n;
    h->nnz = nnz;
    h->nnz_found = found;
    h->kind = err ? CX_KIND_ERROR : CX_KIND_PAIRS;
    h->threshold = thr;
    h->nsub = p.nsub;
    h->src_rank = p.src_rank;
    h->dtype = CX_F32;
    __threadfence_system();
    cx::st_release_sys(&h->seq, p.seq);
  }
  if (tid == 0) {
    if (p.stats) {
      p.stats->n = (uint32_t)p.n;
      p.stats->nnz = nnz;
      p.stats->nnz_found = found;
      p.stats->status = err | (found > p.cap ? CX_ST_OVERFLOW : 0u);
      p.stats->threshold = thr;
    }
    p.ctr->next_tile = 0;
    p.ctr->done = 0;
    p.ctr->nnz_found = 0;
    p.ctr->error = 0;
  }
}

// n == 0: nothing to scan, only the (empty) header and the notification.
__global__ void compress_empty_kernel(const CompressParams p) {
  const int tid = threadIdx.x;
  if (tid < p.tg.count) {
    CxHeader* h = p.tg.ep[tid].hdr;
    p.tg.ep[tid].prefix[0] = 0;
    h->bytes = 8; h->n = 0; h->nnz = 0; h->nnz_found = 0; h->kind = CX_KIND_PAIRS;
    h->threshold = *p.thr; h->nsub = 0; h->src_rank = p.src_rank; h->dtype = CX_F32;
    __threadfence_system();
    cx::st_release_sys(&h->seq, p.seq);
  }
  if (tid == 0 && p.stats) {
    p.stats->n = 0; p.stats->nnz = 0; p.stats->nnz_found = 0; p.stats->status = 0;
    p.stats->threshold = *p.thr;
  }
}

template <typename T, bool HAS_G, bool HAS_R>
int launch_typed(const CompressParams& p, bool vec, int grid, cudaStream_t s) {
  if (vec)
    compress_kernel<T, HAS_G, HAS_R, true><<<grid, kThreads, 0, s>>>(p);
  else
    compress_kernel<T, HAS_G, HAS_R, false><<<grid, kThreads, 0, s>>>(p);
  return 0;
}

template <typename T>
int launch_mode(const CompressParams& p, bool vec, int grid, cudaStream_t s) {
  if (p.g && p.r) return launch_typed<T, true, true>(p, vec, grid, s);
  if (p.r) return launch_typed<T, false, true>(p, vec, grid, s);
  return launch_typed<T, true, false>(p, vec, grid, s);
}

uint32_t next_epoch() {
  static uint32_t e = 0;
  e = (e + 1) & 0x3fffffffu;
  if (e == 0) e = 1;
  return e;
}

}  // namespace

extern "C" int64_t cx_workspace_bytes(int64_t n) {
  const int64_t ntiles = (n + CX_TILE - 1) / CX_TILE;
  return (int64_t)sizeof(CxWorkCounters) + 8 * (ntiles > 0 ? ntiles : 1);
}

int cx_compress_cuda(int gdtype, const void* g, float* r, int64_t n, const float* thr,
                     uint32_t cap, uint64_t seq, const CxTargets* tg, void* workspace,
                     int64_t ws_bytes, CxStats* stats, uint32_t src_rank, void* stream) {
  if (!g && !r) return cx_set_error("cx_compress: g and r are both NULL", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_compress: n out of range", 0);
  if (tg->count < 0 || tg->count > CX_MAX_PEERS) return cx_set_error("cx_compress: bad target count", 0);
  if (ws_bytes < cx_workspace_bytes(n)) return cx_set_error("cx_compress: workspace too small", 0);
  CompressParams p;
  p.g = g; p.r = r; p.n = n; p.thr = thr; p.cap = cap;
  p.ntiles = (uint32_t)((n + CX_TILE - 1) / CX_TILE);
  p.nsub = (uint32_t)((n + CX_SUBTILE - 1) / CX_SUBTILE);
  p.epoch = next_epoch();
  p.seq = seq;
  p.ctr = reinterpret_cast<CxWorkCounters*>(workspace);
  p.tile_status = reinterpret_cast<uint64_t*>(reinterpret_cast<char*>(workspace) + sizeof(CxWorkCounters));
  p.stats = stats; p.src_rank = src_rank;
  p.spin_limit = 1u << 22;
  p.tg = *tg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n == 0) {
    compress_empty_kernel<<<1, 32, 0, s>>>(p);
    cx_note_launch();
    return cx_check_launch("compress_empty_kernel");
  }
  const size_t esz = gdtype == CX_F32 ? 4 : 2;
  const bool vec = (!r || (reinterpret_cast<uintptr_t>(r) & 15) == 0) &&
                   (!g || (reinterpret_cast<uintptr_t>(g) & (4 * esz - 1)) == 0);
  int grid = cx_sm_count() * 4;
  if ((uint32_t)grid > p.ntiles) grid = (int)p.ntiles;
  switch (gdtype) {
    case CX_F32: launch_mode<float>(p, vec, grid, s); break;
    case CX_BF16: launch_mode<__nv_bfloat16>(p, vec, grid, s); break;
    case CX_F16: launch_mode<__half>(p, vec, grid, s); break;
    default: return cx_set_error("cx_compress: unsupported dtype on CUDA", 0);
  }
  cx_note_launch();
  return cx_check_launch("compress_kernel");
}
