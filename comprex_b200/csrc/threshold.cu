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

}  // namespace

// Host-side part of the rule, in the reference's float arithmetic.
// sample count, stride and rank of the estimate (defined with the host back end)
extern "C" void cx_threshold_plan(int64_t n, float ratio, int default_subsamples,
                                  float subsample_factor, int32_t* samples, int32_t* use_all,
                                  float* stepsize, int32_t* topk_pos);

int cx_threshold_topk_cuda(int gdtype, const void* g, const float* r, int64_t n, float ratio,
                           int default_subsamples, float subsample_factor, float* thr_out,
                           void* stream) {
  if (!g && !r) return cx_set_error("cx_threshold_topk: g and r are both NULL", 0);
  ThreshParams p;
  p.g = g; p.r = r; p.n = n; p.thr_out = thr_out;
  cx_threshold_plan(n, ratio, default_subsamples, subsample_factor, &p.samples, &p.use_all,
                    &p.stepsize, &p.topk_pos);
  if (n <= 0) { p.samples = 0; p.topk_pos = 0; }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
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
