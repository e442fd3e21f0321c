// ThresholdTopK on the device (reference: src/threshold.hxx:127-242).
//
// The reference estimates the magnitude cut from a strided sample of
// (rests + input): position (int)(i * (float)n / samples), samples =
// max(default_subsamples, subsample_factor / topK) (or every element when the
// vector is shorter), and takes the element of rank ceil(samples*topK)-1 in
// descending |x| order; when that rank is <= 0 the threshold is max|x| + 1
// so that nothing is sent.  This kernel reproduces that rule bit for bit: the
// sample keys are the bit patterns of |x| (monotonic for non-negative floats)
// and a 4-pass 8-bit radix select over one CTA finds the element of that rank.
// The result stays in device memory, where the compress kernel reads it, so
// no host round trip sits between the two.
//
// Gathering the sample is the expensive part for small top-k fractions (10 000
// strided elements at 0.1 %: 20 000 separate 32-byte sectors, more than one SM's
// load path moves in the time the rest of the kernel takes).  Above 2048 samples the
// kernel therefore runs as a thread-block cluster of 8 CTAs: every CTA gathers one
// eighth of the sample and stores the keys through distributed shared memory into
// the first CTA, which then selects alone.
#include <cooperative_groups.h>
#include <math.h>
#include <string.h>

#include "cx_device.cuh"

namespace {

constexpr int kThreads = 1024;
constexpr int kSmemKeys = 11264;  // 44 KB of cached sample keys

struct ThreshParams {
  const void* g;
  const float* r;
  int64_t n;
  int32_t samples;   // number of sampled elements
  int32_t use_all;   // sample == the whole vector
  float stepsize;
  int32_t topk_pos;  // rank in descending order; <= 0 selects the sentinel
  float* thr_out;
};

template <typename T>
__device__ __forceinline__ uint32_t sample_key(const ThreshParams& p, int i) {
  int64_t pos;
  if (p.use_all) {
    pos = i;
  } else {
    pos = (int64_t)(int)__fmul_rn((float)i, p.stepsize);
    if (pos > p.n - 1) pos = p.n - 1;
  }
  float x = 0.f;
  if (p.r) x = p.r[pos];
  if (p.g) x = x + cx::Elem<T>::to_f(reinterpret_cast<const T*>(p.g)[pos]);
  return __float_as_uint(fabsf(x));
}

constexpr int kGather = 4;  // loads of one thread that are in flight together

template <typename T>
__global__ void __launch_bounds__(kThreads) threshold_kernel(const ThreshParams p) {
  namespace cg = cooperative_groups;
  // the compress kernel queued behind this one may start its prologue now; it waits (for this
  // grid to finish) before it reads the threshold or writes the residual
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ uint32_t s_keys[kSmemKeys];
  __shared__ uint32_t s_hist[256];
  __shared__ uint32_t s_sel[2];  // chosen digit, remaining rank
  __shared__ uint32_t s_red[kThreads / 32];
  __shared__ uint32_t s_cmax[8];  // per-CTA maxima of a cluster launch (first CTA's copy is used)
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int s = p.samples;
  const bool cached = s <= kSmemKeys;
  const int s_round = (s + kThreads - 1) / kThreads * kThreads;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned ncta = cluster.num_blocks();      // 1 unless launched as a cluster (only when cached)
  const unsigned crank = cluster.block_rank();
  uint32_t* keys0 = ncta > 1 ? cluster.map_shared_rank(s_keys, 0) : s_keys;

  // pass 0: gather the sample (and its maximum, for the sentinel case); CTA c of a cluster
  // takes the samples [c, c+1) * s / ncta
  const int lo = (int)((int64_t)s * crank / ncta), hi = (int)((int64_t)s * (crank + 1) / ncta);
  uint32_t mx = 0;
  for (int i0 = lo + tid; i0 < hi; i0 += kGather * kThreads) {
    uint32_t k[kGather];
#pragma unroll
    for (int u = 0; u < kGather; ++u) {
      const int i = i0 + u * kThreads;
      k[u] = i < hi ? sample_key<T>(p, i) : 0u;
    }
#pragma unroll
    for (int u = 0; u < kGather; ++u) {
      const int i = i0 + u * kThreads;
      if (i < hi) {
        if (cached) keys0[i] = k[u];
        mx = max(mx, k[u]);
      }
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  if (lane == 0) s_red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    uint32_t m = 0;
    for (int w = 0; w < kThreads / 32; ++w) m = max(m, s_red[w]);
    (ncta > 1 ? cluster.map_shared_rank(s_cmax, 0) : s_cmax)[crank] = m;
  }
  if (ncta > 1) {
    cluster.sync();              // keys and maxima of all CTAs are in the first CTA's shared memory
    if (crank != 0) return;      // (no CTA touches another CTA's shared memory after this point)
  } else {
    __syncthreads();
  }
  if (p.topk_pos <= 0) {
    if (tid == 0) {
      uint32_t m = 0;
      for (unsigned c = 0; c < ncta; ++c) m = max(m, s_cmax[c]);
      *p.thr_out = __uint_as_float(m) + 1.0f;
    }
    return;
  }

  uint32_t prefix = 0, prefmask = 0;
  uint32_t rank = (uint32_t)p.topk_pos;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) s_hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < s_round; i += kThreads) {
      uint32_t digit = 0xffffffffu;
      if (i < s) {
        const uint32_t k = cached ? s_keys[i] : sample_key<T>(p, i);
        if ((k & prefmask) == prefix) digit = (k >> shift) & 255u;
      }
      const uint32_t peers = __match_any_sync(0xffffffffu, digit);
      if (digit != 0xffffffffu && lane == __ffs(peers) - 1) atomicAdd(&s_hist[digit], __popc(peers));
    }
    __syncthreads();
    if (tid < 32) {
      // lane L owns the 8 bins 255-8L .. 248-8L, walked from the top
      uint32_t h[8], gsum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { h[j] = s_hist[255 - 8 * lane - j]; gsum += h[j]; }
      uint32_t incl = gsum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += t;
      }
      const uint32_t before = incl - gsum;
      if (rank >= before && rank < incl) {  // exactly one lane
        uint32_t cum = before;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (rank >= cum && rank < cum + h[j]) { s_sel[0] = 255 - 8 * lane - j; s_sel[1] = rank - cum; }
          cum += h[j];
        }
      }
    }
    __syncthreads();
    prefix |= s_sel[0] << shift;
    prefmask |= 255u << shift;
    rank = s_sel[1];
    __syncthreads();
  }
  if (tid == 0) *p.thr_out = __uint_as_float(prefix);
}

// ---- exact selection over the whole vector, grid-wide ----------------------------------------
// With sampling switched off (every element is a sample) the single CTA above would walk the
// vector four times on its own.  Here every radix pass is a grid-wide histogram instead: each
// CTA replays the digits chosen so far from the global histograms of the earlier passes (256
// counters each), counts the next digit of the keys that still match into shared memory and
// adds its counts to the global histogram of this pass.  Four such launches and a one-warp
// finish read the vector four times at full bandwidth.  The result is the key of rank topk_pos
// in descending order, the same value the single CTA finds.
constexpr int kExactThreads = 256;

struct ExactParams {
  const void* g;
  const float* r;
  int64_t n;
  uint32_t topk_pos;
  int pass;            // 0..3: digit at shift 24 - 8 * pass; 4: finish
  uint32_t* hist;      // [4][256], zero before the first pass; the finish zeroes it again
  float* thr_out;
  uint32_t vec;        // 16-byte accesses are possible
};

// One warp: the digit of `hist` (256 bins, walked from the top) that holds rank `rank`, and the
// rank inside that bin.  All lanes return the same values.
__device__ __forceinline__ uint32_t pick_digit(const uint32_t* hist, uint32_t& rank, int lane) {
  uint32_t h[8], gsum = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) { h[j] = hist[255 - 8 * lane - j]; gsum += h[j]; }
  uint32_t incl = gsum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  const uint32_t before = incl - gsum;
  uint32_t digit = 0, left = 0;
  const bool mine = rank >= before && rank < incl;   // exactly one lane (rank < number of keys)
  if (mine) {
    uint32_t cum = before;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (rank >= cum && rank < cum + h[j]) { digit = 255 - 8 * lane - j; left = rank - cum; }
      cum += h[j];
    }
  }
  const uint32_t who = __ffs(__ballot_sync(0xffffffffu, mine)) - 1;
  digit = __shfl_sync(0xffffffffu, digit, who & 31);
  rank = __shfl_sync(0xffffffffu, left, who & 31);
  return digit;
}

template <typename T>
__global__ void __launch_bounds__(kExactThreads) exact_select_kernel(const ExactParams p) {
  __shared__ uint32_t s_hist[256];
  __shared__ uint32_t s_prefix;
  const int tid = threadIdx.x, lane = tid & 31;
  s_hist[tid] = 0;
  if (tid < 32) {      // the decisions of the earlier passes
    uint32_t prefix = 0, rank = p.topk_pos;
    for (int q = 0; q < p.pass && q < 4; ++q) prefix |= pick_digit(p.hist + 256 * q, rank, lane) << (24 - 8 * q);
    if (tid == 0) s_prefix = prefix;
  }
  __syncthreads();
  const uint32_t prefix = s_prefix;
  if (p.pass >= 4) {   // finish: the key of that rank is the threshold; leave the scratch clean
    if (blockIdx.x == 0) {
      if (tid == 0) *p.thr_out = __uint_as_float(prefix);
      for (int i = tid; i < 4 * 256; i += kExactThreads) p.hist[i] = 0;
    }
    return;
  }
  const int shift = 24 - 8 * p.pass;
  const uint32_t prefmask = p.pass == 0 ? 0u : (0xffffffffu << (shift + 8));
  const T* g = reinterpret_cast<const T*>(p.g);
  auto count = [&](float x, bool valid) {
    const uint32_t k = __float_as_uint(fabsf(x));
    const uint32_t digit = (valid && (k & prefmask) == prefix) ? ((k >> shift) & 255u) : 0xffffffffu;
    const uint32_t peers = __match_any_sync(0xffffffffu, digit);
    if (digit != 0xffffffffu && lane == __ffs(peers) - 1) atomicAdd(&s_hist[digit], __popc(peers));
  };
  const int64_t gsz = (int64_t)gridDim.x * kExactThreads;
  const int64_t nv = (p.n + 3) / 4;
  const int64_t rounds = (nv + gsz - 1) / gsz;      // every lane runs every round: the counting is warp-wide
  for (int64_t it = 0; it < rounds; ++it) {
    const int64_t i = (it * gsz + (int64_t)blockIdx.x * kExactThreads + tid) * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.vec && i + 3 < p.n) {
      if (p.r) cx::load4(p.r + i, v);
      if (g) {
        float b[4];
        cx::load4(g + i, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = v[e] + b[e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (i + e < p.n) {
          if (p.r) v[e] = p.r[i + e];
          if (g) v[e] = v[e] + cx::Elem<T>::to_f(g[i + e]);
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) count(v[e], i + e < p.n);
  }
  __syncthreads();
  if (s_hist[tid]) atomicAdd(&p.hist[256 * p.pass + tid], s_hist[tid]);
}

template <typename T>
int launch_exact(const ExactParams& base, cudaStream_t s) {
  int grid = cx_sm_count() * 6;
  const int64_t need = ((base.n + 3) / 4 + kExactThreads - 1) / kExactThreads;
  if (grid > need) grid = (int)need;
  for (int pass = 0; pass <= 4; ++pass) {
    ExactParams p = base;
    p.pass = pass;
    exact_select_kernel<T><<<pass < 4 ? grid : 1, kExactThreads, 0, s>>>(p);
    cx_note_launch();
  }
  return cx_check_launch("exact_select_kernel");
}

}  // namespace

extern "C" int64_t cx_threshold_workspace_bytes(void) { return 4 * 256 * (int64_t)sizeof(uint32_t); }

// Host-side part of the rule, in the reference's float arithmetic.
// sample count, stride and rank of the estimate (defined with the host back end)
extern "C" void cx_threshold_plan(int64_t n, float ratio, int default_subsamples,
                                  float subsample_factor, int32_t* samples, int32_t* use_all,
                                  float* stepsize, int32_t* topk_pos);

int cx_threshold_topk_cuda(int gdtype, const void* g, const float* r, int64_t n, float ratio,
                           int default_subsamples, float subsample_factor, float* thr_out,
                           void* workspace, int64_t ws_bytes, void* stream) {
  if (!g && !r) return cx_set_error("cx_threshold_topk: g and r are both NULL", 0);
  ThreshParams p;
  p.g = g; p.r = r; p.n = n; p.thr_out = thr_out;
  cx_threshold_plan(n, ratio, default_subsamples, subsample_factor, &p.samples, &p.use_all,
                    &p.stepsize, &p.topk_pos);
  if (n <= 0) { p.samples = 0; p.topk_pos = 0; }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (p.use_all && p.topk_pos > 0 && n > kSmemKeys && workspace && ws_bytes >= cx_threshold_workspace_bytes()) {
    // exact selection over a vector that does not fit one CTA's shared memory: grid-wide passes
    ExactParams e;
    e.g = g; e.r = r; e.n = n; e.topk_pos = (uint32_t)p.topk_pos; e.pass = 0;
    e.hist = reinterpret_cast<uint32_t*>(workspace); e.thr_out = thr_out;
    const size_t esz = gdtype == CX_F32 ? 4 : 2;
    e.vec = (!r || (reinterpret_cast<uintptr_t>(r) & 15) == 0) && (!g || (reinterpret_cast<uintptr_t>(g) & (4 * esz - 1)) == 0);
    switch (gdtype) {
      case CX_F32: return launch_exact<float>(e, s);
      case CX_BF16: return launch_exact<__nv_bfloat16>(e, s);
      case CX_F16: return launch_exact<__half>(e, s);
      default: return cx_set_error("cx_threshold_topk: unsupported dtype on CUDA", 0);
    }
  }
  // a cluster of 8 CTAs gathers large samples (their keys must fit the first CTA's shared memory)
  const unsigned ncta = (p.samples > 2048 && p.samples <= kSmemKeys) ? 8u : 1u;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(ncta, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ncta;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  switch (gdtype) {
    case CX_F32: e = cudaLaunchKernelEx(&cfg, threshold_kernel<float>, p); break;
    case CX_BF16: e = cudaLaunchKernelEx(&cfg, threshold_kernel<__nv_bfloat16>, p); break;
    case CX_F16: e = cudaLaunchKernelEx(&cfg, threshold_kernel<__half>, p); break;
    default: return cx_set_error("cx_threshold_topk: unsupported dtype on CUDA", 0);
  }
  if (e != cudaSuccess) return cx_set_error("threshold_kernel launch", (int)e);
  cx_note_launch();
  return cx_check_launch("threshold_kernel");
}
