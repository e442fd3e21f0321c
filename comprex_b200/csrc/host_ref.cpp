// Host implementation of every exchange primitive, with the same protocol
// (slots, headers, release/acquire notification, bounded waits, status words)
// as the CUDA kernels.  It serves three purposes: CPU ranks over POSIX shared
// memory run the identical Python code path without a GPU; GPU tests compare
// the kernels against it bit for bit (the kernels are built without
// multiply-add contraction); and host-side fault injection (a rank that never
// sends) exercises the timeout path without touching a GPU.
//
// Semantics follow the reference: ThresholdTopK (src/threshold.hxx:127-242),
// CompressorIndexPairs / CompressorNone / CompressorRLE
// (src/compressor.hxx:84-661), GaspiEx (src/gaspiEx.tpp:70-119).
#include <math.h>
#include <sched.h>
#include <string.h>
#include <time.h>

#include <algorithm>
#include <chrono>
#include <thread>
#include <vector>

#include "cx_common.h"

int cx_set_error(const char* where, int cuda_err);
// The float arithmetic below is the reference's (src/threshold.hxx:182-205); both back ends
// take the sample count, the stride and the rank from it.
extern "C" void cx_threshold_plan(int64_t n, float ratio, int default_subsamples,
                                  float subsample_factor, int32_t* samples, int32_t* use_all,
                                  float* stepsize, int32_t* topk_pos) {
  int subs = default_subsamples;
  if (ratio > 0.f) {
    const float req = subsample_factor / ratio;
    if (req > (float)default_subsamples) subs = req >= 2147483520.f ? 2147483520 : (int)req;
  }
  if (subs < 1) subs = 1;
  int64_t size;
  if (n < subs) { size = n; *use_all = 1; *stepsize = 1.f; }
  else { size = subs; *use_all = 0; *stepsize = (float)n / (float)subs; }
  *samples = (int32_t)size;
  *topk_pos = (int32_t)(ceilf((float)size * ratio) - 1);
}

namespace {

inline float bf16_to_f(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}
inline float f16_to_f(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      exp = 127 - 15 + 1;
      while (!(man & 0x400u)) { man <<= 1; --exp; }
      u = sign | (exp << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
  else u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
  if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to inf
  if (x < 0x33000001u) return (uint16_t)sign;                // rounds to zero
  int exp = (int)(x >> 23) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (exp <= 0) {  // subnormal half
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t half = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return (uint16_t)(sign | half);
}

inline float load_elem(int dtype, const void* p, int64_t i) {
  switch (dtype) {
    case CX_F32: return reinterpret_cast<const float*>(p)[i];
    case CX_BF16: return bf16_to_f(reinterpret_cast<const uint16_t*>(p)[i]);
    default: return f16_to_f(reinterpret_cast<const uint16_t*>(p)[i]);
  }
}
inline void store_elem(int dtype, void* p, int64_t i, float v) {
  switch (dtype) {
    case CX_F32: reinterpret_cast<float*>(p)[i] = v; break;
    case CX_BF16: reinterpret_cast<uint16_t*>(p)[i] = f_to_bf16(v); break;
    default: reinterpret_cast<uint16_t*>(p)[i] = f_to_f16(v); break;
  }
}
inline size_t elem_size(int dtype) { return dtype == CX_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) { return dtype == CX_F32 || dtype == CX_BF16 || dtype == CX_F16; }

inline uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}
inline uint64_t load_seq(const CxHeader* h) { return __atomic_load_n(&h->seq, __ATOMIC_ACQUIRE); }
inline void publish(CxHeader* h, uint64_t seq) { __atomic_store_n(&h->seq, seq, __ATOMIC_RELEASE); }

bool wait_seq(const CxHeader* h, uint64_t want, uint64_t timeout_ns) {
  if (load_seq(h) >= want) return true;
  const uint64_t t0 = now_ns();
  for (uint64_t it = 0;; ++it) {
    if (load_seq(h) >= want) return true;
    if ((it & 63) == 63) {
      if (now_ns() - t0 > timeout_ns) return false;
      sched_yield();
    }
  }
}

uint32_t wait_all(const CxSources* src, uint64_t timeout_ns) {
  uint32_t bad = 0;
  for (int j = 0; j < src->count; ++j)
    if (!wait_seq(src->ep[j].hdr, src->seq[j], timeout_ns)) bad |= CX_ST_TIMEOUT;
  return bad;
}

}  // namespace

extern "C" int cx_host_wait_seq(const CxHeader* hdr, uint64_t seq, uint64_t timeout_ns) {
  return wait_seq(hdr, seq, timeout_ns) ? 0 : (int)CX_ST_TIMEOUT;
}

int cx_threshold_topk_host(int gdtype, const void* g, const float* r, int64_t n, float ratio,
                           int default_subsamples, float subsample_factor, float* thr_out) {
  if (!g && !r) return cx_set_error("cx_threshold_topk: g and r are both NULL", 0);
  if (g && !dtype_ok(gdtype)) return cx_set_error("cx_threshold_topk: unsupported dtype", 0);
  int32_t samples, use_all, topk_pos;
  float stepsize;
  cx_threshold_plan(n, ratio, default_subsamples, subsample_factor, &samples, &use_all, &stepsize,
                    &topk_pos);
  if (n <= 0) { *thr_out = 1.0f; return 0; }
  std::vector<float> key(samples);
  for (int i = 0; i < samples; ++i) {
    int64_t pos = use_all ? i : (int64_t)(int)((float)i * stepsize);
    if (pos > n - 1) pos = n - 1;
    float x = 0.f;
    if (r) x = r[pos];
    if (g) x = x + load_elem(gdtype, g, pos);
    key[i] = fabsf(x);
  }
  if (topk_pos <= 0) {
    *thr_out = *std::max_element(key.begin(), key.end()) + 1.0f;
  } else {
    std::nth_element(key.begin(), key.begin() + topk_pos, key.end(),
                     [](float a, float b) { return a > b; });
    *thr_out = key[topk_pos];
  }
  return 0;
}

int cx_compress_host(int gdtype, const void* g, float* r, int64_t n, const float* thr_p,
                     uint32_t cap, uint64_t seq, const CxTargets* tg, CxStats* stats,
                     uint32_t src_rank) {
  if (!g && !r) return cx_set_error("cx_compress: g and r are both NULL", 0);
  if (g && !dtype_ok(gdtype)) return cx_set_error("cx_compress: unsupported dtype", 0);
  if (n < 0 || n > 0x7fffffffLL) return cx_set_error("cx_compress: n out of range", 0);
  if (tg->count < 0 || tg->count > CX_MAX_PEERS) return cx_set_error("cx_compress: bad target count", 0);
  const float thr = *thr_p;
  const uint32_t nsub = (uint32_t)((n + CX_SUBTILE - 1) / CX_SUBTILE);
  uint32_t found = 0;
  for (uint32_t sub = 0; sub < nsub; ++sub) {
    const int64_t lo = (int64_t)sub * CX_SUBTILE, hi = std::min<int64_t>(lo + CX_SUBTILE, n);
    const uint32_t start = found;
    uint32_t emitted_here = 0;
    for (int64_t i = lo; i < hi; ++i) {
      float a = 0.f, b = 0.f;
      if (r) a = r[i];
      if (g) b = load_elem(gdtype, g, i);
      const float v = a + b;
      bool emitted = false;
      if (fabsf(v) > thr) {
        if (found < cap) {
          CxPair pr;
          pr.idx = (int32_t)i;
          memcpy(&pr.val, &v, 4);
          for (int k = 0; k < tg->count; ++k) tg->ep[k].pairs[found] = pr;
          emitted = true;
          ++emitted_here;
        }
        ++found;
      }
      if (r && (g || emitted)) r[i] = emitted ? 0.f : v;
    }
    for (int k = 0; k < tg->count; ++k) {
      tg->ep[k].table[2 * sub] = emitted_here ? start : 0u;
      tg->ep[k].table[2 * sub + 1] = emitted_here;
    }
  }
  const uint32_t nnz = std::min(found, cap);
  for (int k = 0; k < tg->count; ++k) {
    CxHeader* h = tg->ep[k].hdr;
    h->bytes = 8ull + 8ull * nnz; h->n = (uint32_t)n; h->nnz = nnz; h->nnz_found = found;
    h->kind = CX_KIND_PAIRS; h->threshold = thr; h->nsub = nsub; h->src_rank = src_rank;
    h->dtype = CX_F32;
    publish(h, seq);
  }
  if (stats) {
    stats->n = (uint32_t)n; stats->nnz = nnz; stats->nnz_found = found;
    stats->status = found > cap ? CX_ST_OVERFLOW : 0u; stats->threshold = thr;
  }
  return 0;
}

// The parameter update of one element from its averaged gradient g (SGD, momentum, AdamW);
// shared by the sparse receive path and the dense update.
static inline void rule_host(const CxApplyArgs* a, float* w, int64_t i, float g, int sdt) {
  float wv = w[i];
  if (a->op == CX_OP_SGD) {
    wv = (1.f - a->wd) * wv - g;
  } else if (a->op == CX_OP_MOMENTUM) {
    const float mv = a->momentum * a->m[i] + a->lr * g;
    a->m[i] = mv;
    wv = (1.f - a->wd) * wv - mv;
  } else {
    // same operation order as the kernel (fused multiply-adds in the same places); the
    // kernel's square root and reciprocal are the hardware approximations, so w agrees
    // to a few ulp of the step, m and v bit for bit
    const float mv = fmaf(a->beta1, a->m[i], (1.f - a->beta1) * g);
    const float vv = fmaf(a->beta2, a->v[i], ((1.f - a->beta2) * g) * g);
    a->m[i] = mv; a->v[i] = vv;
    const float mh = mv * (1.f / a->bc1), vh = vv * (1.f / a->bc2);
    wv = fmaf(-(a->lr * mh), 1.f / (sqrtf(vh) + a->eps), wv * (1.f - a->lr * a->wd));
  }
  w[i] = wv;
  if (a->shadow) store_elem(sdt, a->shadow, i, wv);
}

int cx_apply_host(const CxSources* src, int64_t n, const CxApplyArgs* a, uint32_t* status,
                  uint64_t timeout_ns) {
  if (src->count < 0 || src->count > CX_MAX_PEERS) return cx_set_error("cx_apply: bad source count", 0);
  if (!a->out) return cx_set_error("cx_apply: out is NULL", 0);
  if (n == 0) return 0;
  uint32_t bad = wait_all(src, timeout_ns);
  if (!bad)
    for (int j = 0; j < src->count; ++j) {
      const CxHeader* h = src->ep[j].hdr;
      if (h->kind != CX_KIND_PAIRS || h->n != (uint32_t)n) bad |= CX_ST_BAD_HEADER;
    }
  if (bad) { if (status) *status |= bad; return 0; }
  const bool update = a->op != CX_OP_ADD && a->op != CX_OP_SET;
  if (update && a->op != CX_OP_SGD && !a->m) return cx_set_error("cx_apply: momentum buffer missing", 0);
  if (a->op == CX_OP_ADAMW && !a->v) return cx_set_error("cx_apply: second-moment buffer missing", 0);
  const bool sparse = a->op == CX_OP_ADD || (a->op == CX_OP_SGD && a->wd == 0.f);
  const uint32_t nsub = (uint32_t)((n + CX_SUBTILE - 1) / CX_SUBTILE);
  const int sdt = a->shadow_dtype;
  float acc[CX_SUBTILE];
  float* w = reinterpret_cast<float*>(a->out);
  for (uint32_t sub = 0; sub < nsub; ++sub) {
    const int64_t lo = (int64_t)sub * CX_SUBTILE;
    const int64_t hi = std::min<int64_t>(lo + CX_SUBTILE, n);
    if (!sparse) memset(acc, 0, sizeof(acc));
    for (int j = 0; j < src->count; ++j) {
      const uint32_t e_start = src->ep[j].table[2 * sub];
      const uint32_t e_count = std::min<uint32_t>(src->ep[j].table[2 * sub + 1], CX_SUBTILE);
      uint32_t b = std::min(e_start + e_count, src->cap[j]);  // never beyond the slot
      uint32_t s = std::min(e_start, b);
      for (uint32_t i = s; i < b; ++i) {
        const CxPair pr = src->ep[j].pairs[i];
        float val;
        memcpy(&val, &pr.val, 4);
        if (pr.idx < lo || pr.idx >= hi) { bad |= CX_ST_BAD_INDEX; continue; }
        if (!sparse) { acc[pr.idx - lo] += val; continue; }
        if (a->op == CX_OP_SGD) {
          const float nw = w[pr.idx] + (-a->scale) * val;
          w[pr.idx] = nw;
          if (a->shadow) store_elem(sdt, a->shadow, pr.idx, nw);
        } else {
          store_elem(a->out_dtype, a->out, pr.idx, load_elem(a->out_dtype, a->out, pr.idx) + a->scale * val);
        }
      }
    }
    if (sparse) continue;
    for (int64_t i = lo; i < hi; ++i) {
      const float g = a->scale * acc[i - lo];
      if (a->op == CX_OP_SET) { store_elem(a->out_dtype, a->out, i, g); continue; }
      rule_host(a, w, i, g, sdt);
    }
  }
  if (bad && status) *status |= bad;
  return 0;
}

int cx_forward_host(const CxEndpoint* from, uint64_t expect_seq, const CxTargets* tg, uint64_t seq,
                    uint32_t cap, uint32_t* status, uint64_t timeout_ns) {
  if (!wait_seq(from->hdr, expect_seq, timeout_ns)) { if (status) *status |= CX_ST_TIMEOUT; return 0; }
  const CxHeader h = *from->hdr;
  const uint32_t nnz = std::min(h.nnz, cap);
  for (int k = 0; k < tg->count; ++k) {
    for (uint32_t i = 0; i < h.nsub; ++i) {   // entries and pairs keep their positions
      uint32_t st = from->table[2 * i], ct = std::min<uint32_t>(from->table[2 * i + 1], CX_SUBTILE);
      if (st >= cap) st = ct = 0;
      else ct = std::min(ct, cap - st);
      tg->ep[k].table[2 * i] = st;
      tg->ep[k].table[2 * i + 1] = ct;
      memcpy(tg->ep[k].pairs + st, from->pairs + st, (size_t)ct * sizeof(CxPair));
    }
    CxHeader* o = tg->ep[k].hdr;
    o->bytes = 8ull + 8ull * nnz; o->n = h.n; o->nnz = nnz; o->nnz_found = h.nnz_found;
    o->kind = h.kind; o->threshold = h.threshold; o->nsub = h.nsub; o->src_rank = h.src_rank;
    o->dtype = h.dtype;
    publish(o, seq);
  }
  return 0;
}

int cx_dense_send_host(int dtype, const void* g, float* r, int64_t n, uint64_t seq,
                       const CxTargets* tg, const int64_t* starts, const int64_t* lens,
                       uint32_t src_rank) {
  if (!dtype_ok(dtype)) return cx_set_error("cx_dense_send: unsupported dtype", 0);
  if (starts && r) return cx_set_error("cx_dense_send: ranges and a residual cannot be combined", 0);
  const size_t es = elem_size(dtype);
  for (int k = 0; k < tg->count; ++k) {
    const int64_t s = starts ? starts[k] : 0, len = starts ? lens[k] : n;
    if (s < 0 || len < 0 || s + len > n) return cx_set_error("cx_dense_send: range outside the vector", 0);
    char* dst = reinterpret_cast<char*>(tg->ep[k].pairs);
    if (!r) memcpy(dst, reinterpret_cast<const char*>(g) + s * es, (size_t)len * es);
    else
      for (int64_t i = 0; i < n; ++i) store_elem(dtype, dst, i, load_elem(dtype, g, i) + r[i]);
  }
  if (r) memset(r, 0, (size_t)n * sizeof(float));
  for (int k = 0; k < tg->count; ++k) {
    const int64_t len = starts ? lens[k] : n;
    CxHeader* h = tg->ep[k].hdr;
    h->bytes = (uint64_t)len * es; h->n = (uint32_t)len; h->nnz = (uint32_t)len;
    h->nnz_found = (uint32_t)len; h->kind = CX_KIND_DENSE; h->threshold = 0.f; h->nsub = 0;
    h->src_rank = src_rank; h->dtype = (uint32_t)dtype;
    publish(h, seq);
  }
  return 0;
}

int cx_dense_reduce_host(int dtype, void* out, const void* own, int64_t n, const CxSources* src,
                         float scale, const CxTargets* push, uint64_t push_seq,
                         const int64_t* starts, const int64_t* lens, uint32_t src_rank,
                         uint32_t* status, uint64_t timeout_ns) {
  if (!dtype_ok(dtype)) return cx_set_error("cx_dense_reduce: unsupported dtype", 0);
  uint32_t bad = wait_all(src, timeout_ns);
  if (!bad)
    for (int j = 0; j < src->count; ++j)
      if (src->ep[j].hdr->kind != CX_KIND_DENSE || src->ep[j].hdr->dtype != (uint32_t)dtype)
        bad |= CX_ST_BAD_HEADER;
  if (bad) { if (status) *status |= bad; return 0; }
  const bool has_push = push && push->count > 0;
  if (starts) {
    if (has_push || own) return cx_set_error("cx_dense_reduce: gather mode takes no own/push", 0);
    for (int j = 0; j < src->count; ++j) {
      if (starts[j] < 0 || lens[j] < 0 || starts[j] + lens[j] > n)
        return cx_set_error("cx_dense_reduce: range outside the vector", 0);
      for (int64_t i = 0; i < lens[j]; ++i)
      {
        float x = load_elem(dtype, src->ep[j].pairs, i);
        if (scale != 1.f) x *= scale;
        store_elem(dtype, out, starts[j] + i, x);
      }
    }
    return 0;
  }
  for (int64_t i = 0; i < n; ++i) {
    float acc = 0.f;
    const int own_pos = std::min(std::max(src->pad, 0), src->count);   // where the own vector enters the sum
    const int nops = src->count + (own ? 1 : 0);
    for (int k = 0; k < nops; ++k) {
      const float x = (own && k == own_pos) ? load_elem(dtype, own, i)
                                            : load_elem(dtype, src->ep[(own && k > own_pos) ? k - 1 : k].pairs, i);
      acc = k == 0 ? x : acc + x;
    }
    if (scale != 1.f) acc *= scale;
    store_elem(dtype, out, i, acc);
    if (has_push)
      for (int k = 0; k < push->count; ++k) store_elem(dtype, push->ep[k].pairs, i, acc);
  }
  if (has_push)
    for (int k = 0; k < push->count; ++k) {
      CxHeader* h = push->ep[k].hdr;
      h->bytes = (uint64_t)n * elem_size(dtype); h->n = (uint32_t)n; h->nnz = (uint32_t)n;
      h->nnz_found = (uint32_t)n; h->kind = CX_KIND_DENSE; h->threshold = 0.f; h->nsub = 0;
      h->src_rank = src_rank; h->dtype = (uint32_t)dtype;
      publish(h, push_seq);
    }
  return 0;
}

int cx_axpy_host(int ydtype, void* y, int xdtype, const void* x, float a, int64_t n) {
  if (!dtype_ok(ydtype) || !dtype_ok(xdtype)) return cx_set_error("cx_axpy: unsupported dtype", 0);
  for (int64_t i = 0; i < n; ++i)
    store_elem(ydtype, y, i, load_elem(ydtype, y, i) + a * load_elem(xdtype, x, i));
  return 0;
}

// ---- RLE codec ----------------------------------------------------------------
// Layout: i32 n | i32 nnz | nnz x f32 values (packed, in index order) | i32 nRuns |
// i32 firstIsYes | nRuns x i32 run lengths, alternating selected / not selected.
// Selection is |x| >= thr like the reference's RLE, but the packed values are
// written at the packed position, which the reference gets wrong for thr > 0
// (src/compressor.hxx:238,277,316).  With a residual the codec fuses
// "r += g; emit and zero the selected; keep the rest" like the other codecs.

extern "C" int64_t cx_rle_compress_host(const float* g, float* r, int64_t n, float thr, void* out,
                                        int64_t out_bytes) {
  if (!g && !r) { cx_set_error("cx_rle_compress: g and r are both NULL", 0); return -1; }
  std::vector<float> vals;
  std::vector<int32_t> runs;
  int first_yes = 0;
  bool cur = false;
  int32_t len = 0;
  for (int64_t i = 0; i < n; ++i) {
    const float v = (r ? r[i] : 0.f) + (g ? g[i] : 0.f);
    const bool yes = fabsf(v) >= thr && !(thr == 0.f && v == 0.f);
    if (i == 0) { first_yes = yes; cur = yes; }
    if (yes != cur) { runs.push_back(len); len = 0; cur = yes; }
    ++len;
    if (yes) vals.push_back(v);
    if (r) r[i] = yes ? 0.f : v;
  }
  if (n > 0) runs.push_back(len);
  const int64_t need = 8 + 4 * (int64_t)vals.size() + 8 + 4 * (int64_t)runs.size();
  if (need > out_bytes) { cx_set_error("cx_rle_compress: output buffer too small", 0); return -1; }
  char* p = reinterpret_cast<char*>(out);
  const int32_t hdr[2] = {(int32_t)n, (int32_t)vals.size()};
  memcpy(p, hdr, 8); p += 8;
  if (!vals.empty()) memcpy(p, vals.data(), 4 * vals.size());
  p += 4 * vals.size();
  const int32_t rh[2] = {(int32_t)runs.size(), first_yes};
  memcpy(p, rh, 8); p += 8;
  if (!runs.empty()) memcpy(p, runs.data(), 4 * runs.size());
  return need;
}

extern "C" int cx_rle_decode_host(const void* in, int64_t in_bytes, float* out, int64_t n, int add) {
  const char* p = reinterpret_cast<const char*>(in);
  if (in_bytes < 16) return cx_set_error("cx_rle_decode: truncated payload", 0);
  int32_t hdr[2];
  memcpy(hdr, p, 8);
  if (hdr[0] != n) return cx_set_error("cx_rle_decode: length mismatch", 0);
  const int64_t nnz = hdr[1];
  if (nnz < 0 || 16 + 4 * nnz > in_bytes) return cx_set_error("cx_rle_decode: truncated payload", 0);
  const float* vals = reinterpret_cast<const float*>(p + 8);
  int32_t rh[2];
  memcpy(rh, p + 8 + 4 * nnz, 8);
  if (rh[0] < 0 || 16 + 4 * nnz + 4 * (int64_t)rh[0] > in_bytes)
    return cx_set_error("cx_rle_decode: truncated payload", 0);
  const int32_t* runs = reinterpret_cast<const int32_t*>(p + 16 + 4 * nnz);
  int64_t i = 0, k = 0;
  bool yes = rh[1] != 0;
  for (int32_t q = 0; q < rh[0]; ++q) {
    const int32_t len = runs[q];
    if (len < 0 || i + len > n || (yes && k + len > nnz)) return cx_set_error("cx_rle_decode: corrupt runs", 0);
    for (int32_t t = 0; t < len; ++t, ++i) {
      if (yes) out[i] = add ? out[i] + vals[k++] : vals[k++];
      else if (!add) out[i] = 0.f;
    }
    yes = !yes;
  }
  if (i != n) return cx_set_error("cx_rle_decode: runs do not cover the vector", 0);
  return 0;
}

// RLE through a slot: the sender encodes and stores into every target, the receiver waits,
// checks and decodes from its own slot (same protocol as the kernels in rle.cu).
int cx_rle_send_host(int gdtype, const void* g, float* r, int64_t n, const float* thr,
                     int64_t slot_bytes, uint64_t seq, const CxTargets* tg, uint32_t src_rank) {
  if (!g && !r) return cx_set_error("cx_rle_send: g and r are both NULL", 0);
  if (g && !dtype_ok(gdtype)) return cx_set_error("cx_rle_send: unsupported dtype", 0);
  if (slot_bytes < 16 + 8 * n) return cx_set_error("cx_rle_send: slot smaller than the worst case", 0);
  std::vector<float> gf;
  const float* gp = reinterpret_cast<const float*>(g);
  if (g && gdtype != CX_F32) {
    gf.resize((size_t)n);
    for (int64_t i = 0; i < n; ++i) gf[(size_t)i] = load_elem(gdtype, g, i);
    gp = gf.data();
  }
  std::vector<char> buf((size_t)(16 + 8 * n));
  const int64_t used = cx_rle_compress_host(gp, r, n, *thr, buf.data(), (int64_t)buf.size());
  if (used < 0) return 1;
  int32_t nnz;
  memcpy(&nnz, buf.data() + 4, 4);
  for (int k = 0; k < tg->count; ++k) {
    memcpy(tg->ep[k].pairs, buf.data(), (size_t)used);
    CxHeader* h = tg->ep[k].hdr;
    h->bytes = (uint64_t)used; h->n = (uint32_t)n; h->nnz = (uint32_t)nnz; h->nnz_found = (uint32_t)nnz;
    h->kind = CX_KIND_RLE; h->threshold = *thr; h->nsub = 0; h->src_rank = src_rank; h->dtype = CX_F32;
    publish(h, seq);
  }
  return 0;
}

int cx_rle_recv_host(const CxEndpoint* src, uint64_t expect_seq, float* out, int64_t n, int add,
                     int64_t slot_bytes, uint32_t* status, uint64_t timeout_ns) {
  uint32_t bad = 0;
  if (!wait_seq(src->hdr, expect_seq, timeout_ns)) bad = CX_ST_TIMEOUT;
  else if (src->hdr->kind != CX_KIND_RLE || (int64_t)src->hdr->n != n ||
           (int64_t)src->hdr->bytes > slot_bytes || src->hdr->bytes < 16) bad = CX_ST_BAD_HEADER;
  if (!bad) {
    // check the runs before anything is written: a corrupt payload leaves `out` untouched
    const char* p = reinterpret_cast<const char*>(src->pairs);
    const int64_t bytes = (int64_t)src->hdr->bytes;
    int32_t hdr[2], rh[2] = {0, 0};
    memcpy(hdr, p, 8);
    const int64_t nnz = hdr[1];
    bool ok = hdr[0] == n && nnz >= 0 && 16 + 4 * nnz <= bytes;
    if (ok) {
      memcpy(rh, p + 8 + 4 * nnz, 8);
      ok = rh[0] >= 0 && 16 + 4 * nnz + 4 * (int64_t)rh[0] <= bytes;
    }
    if (ok) {
      const int32_t* runs = reinterpret_cast<const int32_t*>(p + 16 + 4 * nnz);
      int64_t total = 0, ytotal = 0;
      bool yes = rh[1] != 0;
      for (int32_t q = 0; q < rh[0] && ok; ++q, yes = !yes) {
        if (runs[q] < 0) ok = false;
        total += runs[q];
        if (yes) ytotal += runs[q];
        if (total > n) ok = false;
      }
      ok = ok && total == n && ytotal == nnz;
    }
    if (!ok) bad = CX_ST_BAD_HEADER;
    else if (cx_rle_decode_host(p, bytes, out, n, add)) bad = CX_ST_BAD_HEADER;
  }
  if (bad && status) *status |= bad;
  return 0;
}

// ---- gradient fold (see fold.cu) -------------------------------------------------------
int cx_fold_host(int gdtype, const void* const* seg_ptr, const int64_t* item_off,
                 const int64_t* item_rel, const int32_t* item_len, const int32_t* item_seg,
                 const int32_t* seg_first, int nitems, float* u, float* partial, float clip,
                 float mu, float lr) {
  if (!dtype_ok(gdtype)) return cx_set_error("cx_fold: unsupported dtype", 0);
  if (clip > 0.f)
    for (int it = 0; it < nitems; ++it) {
      float acc = 0.f;
      for (int i = 0; i < item_len[it]; ++i) {
        const float x = load_elem(gdtype, seg_ptr[item_seg[it]], item_rel[it] + i);
        acc += x * x;
      }
      partial[it] = acc;
    }
  for (int it = 0; it < nitems; ++it) {
    const int seg = item_seg[it];
    float coef = 1.f;
    if (clip > 0.f) {
      float ss = 0.f;
      for (int i = seg_first[seg]; i < seg_first[seg + 1]; ++i) ss += partial[i];
      coef = clip / fmaxf(sqrtf(ss), clip);
    }
    const float a = lr * coef;
    float* dst = u + item_off[it];
    for (int i = 0; i < item_len[it]; ++i) {
      const float y = mu != 0.f ? dst[i] : 0.f;
      dst[i] = mu * y + a * load_elem(gdtype, seg_ptr[seg], item_rel[it] + i);
    }
  }
  return 0;
}

// Dense form of the update: the averaged gradient is a plain fp32 vector (a dense allreduce's
// result, or this rank's own vector when it is alone), keras/comprex_optimizer.py:150-163.
int cx_update_dense_host(const float* g, int64_t n, const CxApplyArgs* a) {
  if (!a->out || !g) return cx_set_error("cx_update_dense: NULL vector", 0);
  if (a->op != CX_OP_SGD && a->op != CX_OP_MOMENTUM && a->op != CX_OP_ADAMW)
    return cx_set_error("cx_update_dense: op must be an update rule", 0);
  if (a->op != CX_OP_SGD && !a->m) return cx_set_error("cx_update_dense: momentum buffer missing", 0);
  if (a->op == CX_OP_ADAMW && !a->v) return cx_set_error("cx_update_dense: second-moment buffer missing", 0);
  float* w = reinterpret_cast<float*>(a->out);
  for (int64_t i = 0; i < n; ++i) rule_host(a, w, i, a->scale * g[i], a->shadow_dtype);
  return 0;
}

// Barrier of host ranks over the shared-memory heap: the protocol of the CUDA barrier kernel.
int cx_barrier_host(int rank, int ranks, void* const* flag_ptrs, uint64_t seq, uint32_t* status,
                    uint64_t timeout_ns) {
  if (ranks < 1 || ranks > CX_MAX_PEERS || rank < 0 || rank >= ranks) return cx_set_error("cx_barrier: bad rank", 0);
  for (int r = 0; r < ranks; ++r)
    __atomic_store_n(reinterpret_cast<uint64_t*>(flag_ptrs[r]) + rank, seq, __ATOMIC_RELEASE);
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < ranks; ++r) {
    const uint64_t* cell = reinterpret_cast<const uint64_t*>(flag_ptrs[rank]) + r;
    while (__atomic_load_n(cell, __ATOMIC_ACQUIRE) < seq) {
      const auto dt = std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
      if ((uint64_t)dt > timeout_ns) { if (status) *status |= CX_ST_TIMEOUT; return 0; }
      std::this_thread::yield();
    }
  }
  return 0;
}
