// Gradient fold of the compressed optimizer: per-tensor L2 clipping and the local
// momentum update, straight from the gradient tensors autograd produced into the flat
// fp32 vector that is exchanged (reference: keras/comprex_optimizer.py:101-115 —
// tf.clip_by_norm per tensor, mom = m*mom + lr*g, concat into one blob).
//
// The tensors of a bucket are described once by a static item list (flat offset,
// length, tensor index, offset inside the tensor; tensors larger than 65536
// elements are cut into several items for load balance).  Per step only the table
// of gradient pointers changes.  Two launches:
//   1. fold_sumsq:  partial[item] = sum of squares of the item (fixed order: the
//      result does not depend on scheduling),
//   2. fold_apply:  coef = clip / max(||g_tensor||, clip) from the tensor's partials,
//                   u[off + i] = mu * u[off + i] + lr * coef * g[i].
// With mu = 0, lr = 1 this is the clipped gradient itself in fp32 (AdamW rule).
#include "cx_device.cuh"

namespace {

constexpr int kThreads = 256;

struct FoldParams {
  const void* const* seg_ptr;   // [nseg] gradient base pointers (device memory)
  const int64_t* item_off;      // [nitems] offset in the flat vector
  const int64_t* item_rel;      // [nitems] offset inside the tensor
  const int32_t* item_len;      // [nitems]
  const int32_t* item_seg;      // [nitems]
  const int32_t* seg_first;     // [nseg + 1] first item of every tensor
  float* u;
  float* partial;               // [nitems]
  float clip;                   // <= 0: no clipping
  float mu;
  float lr;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) fold_sumsq_kernel(const FoldParams p) {
  __shared__ float s_w[kThreads / 32];
  const int item = blockIdx.x;
  const int len = p.item_len[item];
  const T* g = reinterpret_cast<const T*>(p.seg_ptr[p.item_seg[item]]) + p.item_rel[item];
  float acc = 0.f;
  if ((reinterpret_cast<uintptr_t>(g) & (4 * sizeof(T) - 1)) == 0) {
    const int nv = len / 4;
    for (int q = threadIdx.x; q < nv; q += kThreads) {
      float x[4];
      cx::load4(g + 4 * q, x);
      acc += x[0] * x[0];
      acc += x[1] * x[1];
      acc += x[2] * x[2];
      acc += x[3] * x[3];
    }
    for (int i = nv * 4 + threadIdx.x; i < len; i += kThreads) {
      const float x = cx::Elem<T>::to_f(g[i]);
      acc += x * x;
    }
  } else {
    for (int i = threadIdx.x; i < len; i += kThreads) {
      const float x = cx::Elem<T>::to_f(g[i]);
      acc += x * x;
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) t += s_w[w];
    p.partial[item] = t;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) fold_apply_kernel(const FoldParams p) {
  __shared__ float s_coef;
  const int item = blockIdx.x;
  const int seg = p.item_seg[item];
  if (threadIdx.x == 0) {
    float coef = 1.f;
    if (p.clip > 0.f) {
      float ss = 0.f;
      for (int i = p.seg_first[seg]; i < p.seg_first[seg + 1]; ++i) ss += p.partial[i];
      coef = p.clip / fmaxf(sqrtf(ss), p.clip);
    }
    s_coef = p.lr * coef;
  }
  __syncthreads();
  const float a = s_coef;
  const int len = p.item_len[item];
  const T* g = reinterpret_cast<const T*>(p.seg_ptr[seg]) + p.item_rel[item];
  float* u = p.u + p.item_off[item];
  const bool vec = (reinterpret_cast<uintptr_t>(g) & (4 * sizeof(T) - 1)) == 0 &&
                   (reinterpret_cast<uintptr_t>(u) & 15) == 0;
  const int nv = vec ? len / 4 : 0;
  for (int q = threadIdx.x; q < nv; q += kThreads) {
    float x[4], y[4] = {0.f, 0.f, 0.f, 0.f};
    cx::load4(g + 4 * q, x);
    if (p.mu != 0.f) cx::load4(u + 4 * q, y);
#pragma unroll
    for (int e = 0; e < 4; ++e) y[e] = p.mu * y[e] + a * x[e];
    cx::store4(u + 4 * q, y);
  }
  for (int i = nv * 4 + threadIdx.x; i < len; i += kThreads) {
    const float y = p.mu != 0.f ? u[i] : 0.f;
    u[i] = p.mu * y + a * cx::Elem<T>::to_f(g[i]);
  }
}

}  // namespace

int cx_fold_cuda(int gdtype, const void* const* seg_ptr, const int64_t* item_off,
                 const int64_t* item_rel, const int32_t* item_len, const int32_t* item_seg,
                 const int32_t* seg_first, int nitems, float* u, float* partial, float clip,
                 float mu, float lr, void* stream) {
  if (nitems <= 0) return 0;
  FoldParams p;
  p.seg_ptr = seg_ptr; p.item_off = item_off; p.item_rel = item_rel; p.item_len = item_len;
  p.item_seg = item_seg; p.seg_first = seg_first; p.u = u; p.partial = partial;
  p.clip = clip; p.mu = mu; p.lr = lr;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (gdtype) {
    case CX_F32:
      if (clip > 0.f) { fold_sumsq_kernel<float><<<nitems, kThreads, 0, s>>>(p); cx_note_launch(); }
      fold_apply_kernel<float><<<nitems, kThreads, 0, s>>>(p);
      break;
    case CX_BF16:
      if (clip > 0.f) { fold_sumsq_kernel<__nv_bfloat16><<<nitems, kThreads, 0, s>>>(p); cx_note_launch(); }
      fold_apply_kernel<__nv_bfloat16><<<nitems, kThreads, 0, s>>>(p);
      break;
    case CX_F16:
      if (clip > 0.f) { fold_sumsq_kernel<__half><<<nitems, kThreads, 0, s>>>(p); cx_note_launch(); }
      fold_apply_kernel<__half><<<nitems, kThreads, 0, s>>>(p);
      break;
    default:
      return cx_set_error("cx_fold: unsupported dtype on CUDA", 0);
  }
  cx_note_launch();
  return cx_check_launch("fold kernels");
}
