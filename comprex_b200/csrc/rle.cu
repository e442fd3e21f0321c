// Run-length codec on the GPU, fused with the transfer (reference: CompressorRLE,
// src/compressor.hxx:159-532, whose packed-value indexing is wrong for thresholds
// above zero; this is the corrected format of the host codec in host_ref.cpp).
//
// Payload, written straight into the receivers' slots:
//   i32 n | i32 nnz | nnz x f32 values (index order) | i32 nRuns | i32 firstIsYes |
//   nRuns x i32 run lengths, alternating selected / not selected.
// Selection: |r + g| >= thr, except that zeros are never selected at thr == 0.
//
// Send = three launches on one stream:
//   1. rle_count:  per 2048-element tile: selected elements, run starts, position of the
//                  last run start, whether the tile's first element starts a run,
//   2. rle_scan:   one CTA turns the per-tile numbers into offsets (exclusive sums and a
//                  running maximum) and leaves the totals,
//   3. rle_emit:   every tile recomputes its mask, stores values and run lengths at their
//                  final position in every target, updates the residual; the last CTA
//                  writes the two small headers and releases the sequence number.
// Receive = two launches:
//   1. rle_decode_scan:  one CTA waits (bounded) for the sequence number, checks the
//                  headers and the run lengths and writes, per run, its end position and
//                  the offset of its first value,
//   2. rle_expand: every thread finds the run of its first element by bisection and walks.
// A payload that fails a check sets BAD_HEADER in the status word and leaves `out` untouched.
#include "cx_device.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kPer = 8;
constexpr int kTile = kThreads * kPer;   // 2048
constexpr int kScanThreads = 1024;

struct RleMeta {           // first 256 bytes of the sender's workspace
  uint32_t done;
  int32_t nnz;
  int32_t nruns;
  int32_t first_yes;
  uint32_t pad[60];
};
struct RleRxMeta {         // first 256 bytes of the receiver's workspace
  int32_t ok;
  int32_t nnz;
  int32_t nruns;
  int32_t first_yes;
  uint32_t pad[60];
};

struct SendParams {
  const void* g;
  float* r;
  int64_t n;
  const float* thr;
  uint64_t seq;
  CxTargets tg;
  RleMeta* meta;
  int32_t* t_nnz;     // [ntiles] count, then offset
  int32_t* t_starts;  // [ntiles] count, then offset
  int32_t* t_last;    // [ntiles] last start position in the tile (-1: none), then: before the tile
  int32_t* t_first;   // [ntiles] 1 if the tile's first element starts a run
  int32_t ntiles;
  uint32_t src_rank;
};

__device__ __forceinline__ bool selected(float v, float thr) {
  return fabsf(v) >= thr && !(thr == 0.f && v == 0.f);
}

template <typename T>
__device__ __forceinline__ float value_at(const SendParams& p, int64_t i) {
  float v = p.g ? cx::Elem<T>::to_f(reinterpret_cast<const T*>(p.g)[i]) : 0.f;
  if (p.r) v += p.r[i];
  return v;
}

// the thread's 8 consecutive values; returns the number of valid ones
template <typename T>
__device__ __forceinline__ int load_values(const SendParams& p, int64_t base, float (&v)[kPer]) {
  const int64_t left = p.n - base;
  const int valid = left >= kPer ? kPer : (left > 0 ? (int)left : 0);
  const T* g = reinterpret_cast<const T*>(p.g);
  const bool gvec = !g || (reinterpret_cast<uintptr_t>(g) & (4 * sizeof(T) - 1)) == 0;
  const bool rvec = !p.r || (reinterpret_cast<uintptr_t>(p.r) & 15) == 0;
  if (valid == kPer && gvec && rvec) {
    float a[4], b[4];
    if (g) { cx::load4(g + base, a); cx::load4(g + base + 4, b); }
    else { for (int e = 0; e < 4; ++e) a[e] = b[e] = 0.f; }
    if (p.r) {
      float c[4], d[4];
      cx::load4(p.r + base, c); cx::load4(p.r + base + 4, d);
#pragma unroll
      for (int e = 0; e < 4; ++e) { a[e] += c[e]; b[e] += d[e]; }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) { v[e] = a[e]; v[4 + e] = b[e]; }
  } else {
#pragma unroll
    for (int e = 0; e < kPer; ++e) v[e] = e < valid ? value_at<T>(p, base + e) : 0.f;
  }
  return valid;
}

// bits of the selected elements and of the run starts among the thread's valid elements
__device__ __forceinline__ void masks(const float (&v)[kPer], int valid, float thr, bool prev_yes,
                                      bool first_is_start, bool use_first, uint32_t& yes,
                                      uint32_t& starts) {
  yes = 0;
#pragma unroll
  for (int e = 0; e < kPer; ++e)
    if (e < valid && selected(v[e], thr)) yes |= 1u << e;
  const uint32_t vm = valid >= kPer ? 0xffu : ((1u << valid) - 1u);
  const uint32_t shifted = (yes << 1) | (prev_yes ? 1u : 0u);
  starts = (yes ^ shifted) & vm;
  if (use_first) starts = (starts & ~1u) | ((first_is_start && valid > 0) ? 1u : 0u);
}

struct Triple { int nnz, st, last; };

// exclusive block scan: sums of nnz and st, maximum of last; totals in `tot`
template <int THREADS>
__device__ __forceinline__ Triple block_scan(Triple x, Triple& tot, int (*sm)[3]) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  Triple inc = x;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, inc.nnz, d);
    const int b = __shfl_up_sync(0xffffffffu, inc.st, d);
    const int c = __shfl_up_sync(0xffffffffu, inc.last, d);
    if (lane >= d) { inc.nnz += a; inc.st += b; inc.last = max(inc.last, c); }
  }
  if (lane == 31) { sm[w][0] = inc.nnz; sm[w][1] = inc.st; sm[w][2] = inc.last; }
  __syncthreads();
  Triple pre = {0, 0, -1};
  tot = {0, 0, -1};
  for (int j = 0; j < THREADS / 32; ++j) {
    if (j == w) pre = tot;
    tot.nnz += sm[j][0]; tot.st += sm[j][1]; tot.last = max(tot.last, sm[j][2]);
  }
  __syncthreads();
  // exclusive = warp prefix + inclusive of the lanes before
  const int a = __shfl_up_sync(0xffffffffu, inc.nnz, 1);
  const int b = __shfl_up_sync(0xffffffffu, inc.st, 1);
  const int c = __shfl_up_sync(0xffffffffu, inc.last, 1);
  Triple ex = pre;
  if (lane > 0) { ex.nnz += a; ex.st += b; ex.last = max(ex.last, c); }
  return ex;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) rle_count_kernel(const SendParams p) {
  __shared__ int sm[kThreads / 32][3];
  __shared__ uint32_t s_yes[kThreads];
  const int tile = blockIdx.x;
  const int64_t base = (int64_t)tile * kTile + (int64_t)threadIdx.x * kPer;
  const float thr = *p.thr;
  float v[kPer];
  const int valid = load_values<T>(p, base, v);
  uint32_t yes = 0;
#pragma unroll
  for (int e = 0; e < kPer; ++e)
    if (e < valid && selected(v[e], thr)) yes |= 1u << e;
  s_yes[threadIdx.x] = yes;
  __syncthreads();
  bool prev_yes = false, first_start = false;
  if (threadIdx.x > 0) prev_yes = (s_yes[threadIdx.x - 1] >> (kPer - 1)) & 1u;
  else if (tile == 0) first_start = true;
  else {
    prev_yes = selected(value_at<T>(p, base - 1), thr);
    first_start = valid > 0 && prev_yes != ((yes & 1u) != 0);
  }
  uint32_t y2, starts;
  masks(v, valid, thr, prev_yes, first_start, threadIdx.x == 0, y2, starts);
  Triple x = {__popc(yes), __popc(starts), starts ? (int)(base + 31 - __clz(starts)) : -1};
  Triple tot;
  block_scan<kThreads>(x, tot, sm);
  if (threadIdx.x == 0) {
    p.t_nnz[tile] = tot.nnz;
    p.t_starts[tile] = tot.st;
    p.t_last[tile] = tot.last;
    p.t_first[tile] = (first_start && valid > 0) ? 1 : 0;
    if (tile == 0) p.meta->first_yes = (valid > 0 && (yes & 1u)) ? 1 : 0;
  }
}

__global__ void __launch_bounds__(kScanThreads) rle_scan_kernel(const SendParams p) {
  __shared__ int sm[kScanThreads / 32][3];
  Triple carry = {0, 0, -1};
  for (int b0 = 0; b0 < p.ntiles; b0 += kScanThreads) {
    const int t = b0 + threadIdx.x;
    Triple x = {0, 0, -1};
    if (t < p.ntiles) x = {p.t_nnz[t], p.t_starts[t], p.t_last[t]};
    Triple tot;
    const Triple ex = block_scan<kScanThreads>(x, tot, sm);
    if (t < p.ntiles) {
      p.t_nnz[t] = carry.nnz + ex.nnz;
      p.t_starts[t] = carry.st + ex.st;
      p.t_last[t] = max(carry.last, ex.last);
    }
    carry.nnz += tot.nnz; carry.st += tot.st; carry.last = max(carry.last, tot.last);
  }
  if (threadIdx.x == 0) { p.meta->nnz = carry.nnz; p.meta->nruns = carry.st; }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) rle_emit_kernel(const SendParams p) {
  __shared__ int sm[kThreads / 32][3];
  __shared__ uint32_t s_yes[kThreads];
  __shared__ uint32_t s_lastblock;
  const int tile = blockIdx.x;
  const int64_t base = (int64_t)tile * kTile + (int64_t)threadIdx.x * kPer;
  const float thr = *p.thr;
  const int nnz_total = p.meta->nnz, nruns = p.meta->nruns;
  float v[kPer];
  const int valid = load_values<T>(p, base, v);
  uint32_t yes = 0;
#pragma unroll
  for (int e = 0; e < kPer; ++e)
    if (e < valid && selected(v[e], thr)) yes |= 1u << e;
  s_yes[threadIdx.x] = yes;
  __syncthreads();
  const bool prev_yes = threadIdx.x > 0 && ((s_yes[threadIdx.x - 1] >> (kPer - 1)) & 1u);
  uint32_t y2, starts;
  masks(v, valid, thr, prev_yes, p.t_first[tile] != 0, threadIdx.x == 0, y2, starts);
  Triple x = {__popc(yes), __popc(starts), starts ? (int)(base + 31 - __clz(starts)) : -1};
  Triple tot;
  const Triple ex = block_scan<kThreads>(x, tot, sm);
  int k = p.t_nnz[tile] + ex.nnz;
  int q = p.t_starts[tile] + ex.st;
  int prev = max(p.t_last[tile], ex.last);
  // residual first (vector stores when possible), then the scattered payload stores
  if (p.r && valid > 0) {
    if (valid == kPer && (reinterpret_cast<uintptr_t>(p.r) & 15) == 0) {
      float a[4], b[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        a[e] = (yes >> e) & 1u ? 0.f : v[e];
        b[e] = (yes >> (4 + e)) & 1u ? 0.f : v[4 + e];
      }
      cx::store4(p.r + base, a);
      cx::store4(p.r + base + 4, b);
    } else {
      for (int e = 0; e < valid; ++e) p.r[base + e] = (yes >> e) & 1u ? 0.f : v[e];
    }
  }
  const size_t runs_off = 8 + 4 * (size_t)nnz_total + 8;
  for (int e = 0; e < valid; ++e) {
    const int i = (int)(base + e);
    if ((starts >> e) & 1u) {
      if (q > 0)
        for (int t = 0; t < p.tg.count; ++t)
          reinterpret_cast<int32_t*>(reinterpret_cast<char*>(p.tg.ep[t].pairs) + runs_off)[q - 1] = i - prev;
      prev = i;
      ++q;
    }
    if ((yes >> e) & 1u) {
      for (int t = 0; t < p.tg.count; ++t)
        reinterpret_cast<float*>(reinterpret_cast<char*>(p.tg.ep[t].pairs) + 8)[k] = v[e];
      ++k;
    }
  }
  if (valid > 0 && base + valid == p.n && q > 0)   // the thread that holds the last element closes the last run
    for (int t = 0; t < p.tg.count; ++t)
      reinterpret_cast<int32_t*>(reinterpret_cast<char*>(p.tg.ep[t].pairs) + runs_off)[q - 1] = (int)(p.n - prev);
  if (!cx::cta_arrive(&p.meta->done, gridDim.x, &s_lastblock)) return;
  if ((int)threadIdx.x < p.tg.count) {
    const CxEndpoint ep = p.tg.ep[threadIdx.x];
    int32_t* pay = reinterpret_cast<int32_t*>(ep.pairs);
    pay[0] = (int32_t)p.n;
    pay[1] = nnz_total;
    int32_t* rh = reinterpret_cast<int32_t*>(reinterpret_cast<char*>(ep.pairs) + 8 + 4 * (size_t)nnz_total);
    rh[0] = nruns;
    rh[1] = p.meta->first_yes;
    CxHeader* h = ep.hdr;
    h->bytes = 16 + 4 * (uint64_t)nnz_total + 4 * (uint64_t)nruns;
    h->n = (uint32_t)p.n; h->nnz = (uint32_t)nnz_total; h->nnz_found = (uint32_t)nnz_total;
    h->kind = CX_KIND_RLE; h->threshold = thr; h->nsub = 0; h->src_rank = p.src_rank;
    h->dtype = CX_F32;
    cx::st_release_sys(&h->seq, p.seq);
  }
  if (threadIdx.x == 0) p.meta->done = 0;
}

// ---- receive ---------------------------------------------------------------------------

struct RecvParams {
  CxEndpoint src;
  uint64_t expect_seq;
  float* out;
  int64_t n;
  int64_t slot_bytes;
  int32_t add;
  RleRxMeta* meta;
  int32_t* run_end;    // [n + 1]
  int32_t* run_val;    // [n + 1]
  uint32_t* status;
  uint64_t timeout_ns;
};

__global__ void __launch_bounds__(kScanThreads) rle_decode_scan_kernel(const RecvParams p) {
  __shared__ int s_state;
  __shared__ long long sm[kScanThreads / 32][2];
  __shared__ long long s_carry[2];
  if (threadIdx.x == 0) {
    int st = 0;
    if (!cx::wait_seq(&p.src.hdr->seq, p.expect_seq, p.timeout_ns)) st = CX_ST_TIMEOUT;
    else if (p.src.hdr->kind != CX_KIND_RLE || (int64_t)p.src.hdr->n != p.n) st = CX_ST_BAD_HEADER;
    s_state = st;
    s_carry[0] = s_carry[1] = 0;
  }
  __syncthreads();
  int st = s_state;
  const int32_t* pay = reinterpret_cast<const int32_t*>(p.src.pairs);
  int64_t nnz = 0, nruns = 0;
  int first = 0;
  if (!st) {
    nnz = pay[1];
    if ((int64_t)pay[0] != p.n || nnz < 0 || nnz > p.n || 16 + 4 * nnz > p.slot_bytes) st = CX_ST_BAD_HEADER;
  }
  const int32_t* rh = nullptr;
  if (!st) {
    rh = reinterpret_cast<const int32_t*>(reinterpret_cast<const char*>(p.src.pairs) + 8 + 4 * nnz);
    nruns = rh[0];
    first = rh[1] != 0;
    if (nruns < 0 || nruns > p.n + 1 || 16 + 4 * nnz + 4 * nruns > p.slot_bytes) st = CX_ST_BAD_HEADER;
  }
  if (st) {
    if (threadIdx.x == 0) { atomicOr(p.status, (uint32_t)st); p.meta->ok = 0; }
    return;
  }
  const int32_t* runs = rh + 2;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int bad = 0;
  for (int64_t b0 = 0; b0 < nruns; b0 += kScanThreads) {
    const int64_t q = b0 + threadIdx.x;
    long long len = 0, ylen = 0;
    if (q < nruns) {
      len = runs[q];
      if (len < 0) { bad = 1; len = 0; }
      const bool yes = ((q & 1) == 0) == (first != 0);
      ylen = yes ? len : 0;
    }
    long long il = len, iy = ylen;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const long long a = __shfl_up_sync(0xffffffffu, il, d);
      const long long b = __shfl_up_sync(0xffffffffu, iy, d);
      if (lane >= d) { il += a; iy += b; }
    }
    if (lane == 31) { sm[w][0] = il; sm[w][1] = iy; }
    __syncthreads();
    long long pl = s_carry[0], py = s_carry[1], tl = 0, ty = 0;
    for (int j = 0; j < kScanThreads / 32; ++j) {
      if (j == w) { pl += tl; py += ty; }
      tl += sm[j][0]; ty += sm[j][1];
    }
    const long long end = pl + il, voff = py + iy - ylen;
    if (q < nruns) {
      if (end > p.n || voff + ylen > nnz) bad = 1;
      p.run_end[q] = (int32_t)(end > p.n ? p.n : end);
      p.run_val[q] = (int32_t)(voff > nnz ? nnz : voff);
    }
    __syncthreads();
    if (threadIdx.x == 0) { s_carry[0] += tl; s_carry[1] += ty; }
    __syncthreads();
  }
  bad = __syncthreads_or(bad);
  if (threadIdx.x == 0) {
    if (s_carry[0] != p.n || s_carry[1] != nnz) bad = 1;
    if (bad) atomicOr(p.status, (uint32_t)CX_ST_BAD_HEADER);
    p.meta->ok = bad ? 0 : 1;
    p.meta->nnz = (int32_t)nnz;
    p.meta->nruns = (int32_t)nruns;
    p.meta->first_yes = first;
  }
}

__global__ void __launch_bounds__(kThreads) rle_expand_kernel(const RecvParams p) {
  if (!p.meta->ok) return;
  const int nruns = p.meta->nruns, first = p.meta->first_yes;
  const float* vals = reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.src.pairs) + 8);
  const int64_t groups = (p.n + 3) / 4;
  for (int64_t gidx = (int64_t)blockIdx.x * kThreads + threadIdx.x; gidx < groups;
       gidx += (int64_t)gridDim.x * kThreads) {
    const int64_t i0 = gidx * 4;
    // first run whose end lies beyond i0 (zero-length runs are skipped by construction)
    int lo = 0, hi = nruns - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (p.run_end[mid] > i0) hi = mid; else lo = mid + 1;
    }
    int q = lo;
    int end = p.run_end[q];
    for (int e = 0; e < 4 && i0 + e < p.n; ++e) {
      const int64_t i = i0 + e;
      while (end <= i && q + 1 < nruns) { ++q; end = p.run_end[q]; }
      const bool yes = ((q & 1) == 0) == (first != 0);
      if (yes) {
        const int start = q ? p.run_end[q - 1] : 0;
        const float x = vals[p.run_val[q] + (int)(i - start)];
        p.out[i] = p.add ? p.out[i] + x : x;
      } else if (!p.add) {
        p.out[i] = 0.f;
      }
    }
  }
}

}  // namespace

int64_t cx_rle_slot_bytes(int64_t n) { return (16 + 8 * n + 15) / 16 * 16; }

int64_t cx_rle_workspace_bytes(int64_t n) {
  const int64_t ntiles = n > 0 ? (n + kTile - 1) / kTile : 1;
  const int64_t send = 256 + 16 * ntiles;
  const int64_t recv = 256 + 8 * (n + 1);
  return ((send > recv ? send : recv) + 255) / 256 * 256;
}

int cx_rle_send_cuda(int gdtype, const void* g, float* r, int64_t n, const float* thr,
                     int64_t slot_bytes, uint64_t seq, const CxTargets* tg, void* workspace,
                     int64_t ws_bytes, uint32_t src_rank, void* stream) {
  if (!g && !r) return cx_set_error("cx_rle_send: g and r are both NULL", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_rle_send: n out of range", 0);
  if (tg->count < 0 || tg->count > CX_MAX_PEERS) return cx_set_error("cx_rle_send: bad target count", 0);
  if (slot_bytes < 16 + 8 * n) return cx_set_error("cx_rle_send: slot smaller than the worst case", 0);
  if (ws_bytes < cx_rle_workspace_bytes(n)) return cx_set_error("cx_rle_send: workspace too small", 0);
  SendParams p;
  p.g = g; p.r = r; p.n = n; p.thr = thr; p.seq = seq; p.tg = *tg; p.src_rank = src_rank;
  p.ntiles = (int)(n > 0 ? (n + kTile - 1) / kTile : 1);
  char* ws = reinterpret_cast<char*>(workspace);
  p.meta = reinterpret_cast<RleMeta*>(ws);
  p.t_nnz = reinterpret_cast<int32_t*>(ws + 256);
  p.t_starts = p.t_nnz + p.ntiles;
  p.t_last = p.t_starts + p.ntiles;
  p.t_first = p.t_last + p.ntiles;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (gdtype) {
    case CX_F32: rle_count_kernel<float><<<p.ntiles, kThreads, 0, s>>>(p); break;
    case CX_BF16: rle_count_kernel<__nv_bfloat16><<<p.ntiles, kThreads, 0, s>>>(p); break;
    case CX_F16: rle_count_kernel<__half><<<p.ntiles, kThreads, 0, s>>>(p); break;
    default: return cx_set_error("cx_rle_send: unsupported dtype on CUDA", 0);
  }
  cx_note_launch();
  rle_scan_kernel<<<1, kScanThreads, 0, s>>>(p);
  cx_note_launch();
  switch (gdtype) {
    case CX_F32: rle_emit_kernel<float><<<p.ntiles, kThreads, 0, s>>>(p); break;
    case CX_BF16: rle_emit_kernel<__nv_bfloat16><<<p.ntiles, kThreads, 0, s>>>(p); break;
    default: rle_emit_kernel<__half><<<p.ntiles, kThreads, 0, s>>>(p); break;
  }
  cx_note_launch();
  return cx_check_launch("rle send kernels");
}

int cx_rle_recv_cuda(const CxEndpoint* src, uint64_t expect_seq, float* out, int64_t n, int add,
                     int64_t slot_bytes, void* workspace, int64_t ws_bytes, uint32_t* status,
                     uint64_t timeout_ns, void* stream) {
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_rle_recv: n out of range", 0);
  if (ws_bytes < cx_rle_workspace_bytes(n)) return cx_set_error("cx_rle_recv: workspace too small", 0);
  RecvParams p;
  p.src = *src; p.expect_seq = expect_seq; p.out = out; p.n = n; p.slot_bytes = slot_bytes;
  p.add = add; p.status = status; p.timeout_ns = timeout_ns;
  char* ws = reinterpret_cast<char*>(workspace);
  p.meta = reinterpret_cast<RleRxMeta*>(ws);
  p.run_end = reinterpret_cast<int32_t*>(ws + 256);
  p.run_val = p.run_end + (n + 1);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  rle_decode_scan_kernel<<<1, kScanThreads, 0, s>>>(p);
  cx_note_launch();
  if (n > 0) {
    const int64_t groups = (n + 3) / 4;
    int64_t blocks = (groups + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)cx_sm_count() * 8;
    if (blocks > cap) blocks = cap;
    rle_expand_kernel<<<(int)blocks, kThreads, 0, s>>>(p);
    cx_note_launch();
  }
  return cx_check_launch("rle receive kernels");
}
