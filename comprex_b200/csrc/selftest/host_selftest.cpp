// Self-test of the host back end, built with AddressSanitizer + UndefinedBehaviorSanitizer
// (and a second time with ThreadSanitizer) by `python -m comprex_b200.build --selftest`.
// The reference has no sanitizer builds (CMakeLists.txt:12-13 only adds -g); here the CPU
// restatement of every primitive - the oracle of the CUDA kernels - runs its edge cases
// under the sanitizers:
//   * sizes around the vector width, the sub-tile and the tile (0, 1, 31..33, 1023..1025, ...),
//     no survivor, exactly `capacity` survivors, more survivors than capacity,
//   * canary words before and after every slot region, checked after every case,
//   * the two-parity slot protocol between two threads that play two ranks
//     (send(s) -> recv(s) on both sides, slots alternating by the parity of s).
// Exit code 0 = all checks passed.
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <thread>
#include <vector>

#include "../cx_common.h"

int cx_threshold_topk_host(int, const void*, const float*, int64_t, float, int, float, float*);
int cx_compress_host(int, const void*, float*, int64_t, const float*, uint32_t, uint64_t,
                     const CxTargets*, CxStats*, uint32_t);
int cx_apply_host(const CxSources*, int64_t, const CxApplyArgs*, uint32_t*, uint64_t);
int cx_dense_send_host(int, const void*, float*, int64_t, uint64_t, const CxTargets*, const int64_t*,
                       const int64_t*, uint32_t);
int cx_dense_reduce_host(int, void*, const void*, int64_t, const CxSources*, float, const CxTargets*,
                         uint64_t, const int64_t*, const int64_t*, uint32_t, uint32_t*, uint64_t);
int cx_rle_send_host(int, const void*, float*, int64_t, const float*, int64_t, uint64_t, const CxTargets*,
                     uint32_t);
int cx_rle_recv_host(const CxEndpoint*, uint64_t, float*, int64_t, int, int64_t, uint32_t*, uint64_t);

static char g_err[256];
int cx_set_error(const char* where, int) {
  snprintf(g_err, sizeof(g_err), "%s", where);
  return -1;
}

static int g_fail = 0;
#define CHECK(cond)                                                            \
  do {                                                                         \
    if (!(cond)) {                                                             \
      fprintf(stderr, "FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);          \
      ++g_fail;                                                                \
    }                                                                          \
  } while (0)

static const uint64_t kCanary = 0xC0FFEE1234ABCDEFull;
static const uint64_t kTimeout = 5ull * 1000000000ull;

// A slot in ordinary heap memory: [canary][header][canary][table][canary][pairs][canary]
struct Slot {
  std::vector<uint64_t> mem;
  size_t hdr_at, table_at, pairs_at, table_words, pair_words;
  Slot(int64_t n, int64_t payload_bytes) {
    const size_t nsub = (size_t)((n + CX_SUBTILE - 1) / CX_SUBTILE);
    table_words = nsub ? nsub : 1;                        // 8 bytes per sub-tile
    pair_words = (size_t)((payload_bytes + 7) / 8) + 1;
    hdr_at = 1;
    table_at = hdr_at + 8 + 1;
    pairs_at = table_at + table_words + 1;
    mem.assign(pairs_at + pair_words + 1, 0);
    mem[0] = mem[hdr_at + 8] = mem[table_at + table_words] = mem[pairs_at + pair_words] = kCanary;
  }
  CxEndpoint ep() {
    CxEndpoint e;
    e.hdr = reinterpret_cast<CxHeader*>(&mem[hdr_at]);
    e.table = reinterpret_cast<uint32_t*>(&mem[table_at]);
    e.pairs = reinterpret_cast<CxPair*>(&mem[pairs_at]);
    return e;
  }
  bool intact() const {
    return mem[0] == kCanary && mem[hdr_at + 8] == kCanary && mem[table_at + table_words] == kCanary &&
           mem[pairs_at + pair_words] == kCanary;
  }
};

static uint32_t lcg(uint32_t& s) { return s = s * 1664525u + 1013904223u; }
static float rnd(uint32_t& s) { return ((lcg(s) >> 8) & 0xffff) / 32768.f - 1.f; }   // [-1, 1)

static void sparse_case(int64_t n, float thr, int64_t cap) {
  uint32_t seed = (uint32_t)(n * 7919 + cap);
  std::vector<float> g((size_t)n), r0((size_t)n), r;
  for (int64_t i = 0; i < n; ++i) { g[i] = rnd(seed); r0[i] = 0.25f * rnd(seed); }
  r = r0;
  Slot a(n, 8 * cap), b(n, 8 * cap);
  CxTargets tg;
  memset(&tg, 0, sizeof(tg));
  tg.count = 2; tg.ep[0] = a.ep(); tg.ep[1] = b.ep();
  CxStats st;
  memset(&st, 0, sizeof(st));
  CHECK(cx_compress_host(CX_F32, g.data(), r.data(), n, &thr, (uint32_t)cap, 1, &tg, &st, 3) == 0);
  CHECK(a.intact() && b.intact());
  // restatement: survivors in index order up to the capacity, the rest stays behind
  int64_t found = 0, sent = 0;
  std::vector<float> dense((size_t)n, 0.f);
  for (int64_t i = 0; i < n; ++i) {
    const float v = g[i] + r0[i];
    if (fabsf(v) > thr) {
      if (found < cap) { dense[i] = v; ++sent; CHECK(r[i] == 0.f); }
      else CHECK(r[i] == v);
      ++found;
    } else CHECK(r[i] == v);
  }
  CHECK(st.nnz == (uint32_t)sent && st.nnz_found == (uint32_t)found);
  CHECK((st.status == CX_ST_OVERFLOW) == (found > cap));
  CHECK(a.ep().hdr->nnz == (uint32_t)sent && a.ep().hdr->kind == CX_KIND_PAIRS && a.ep().hdr->src_rank == 3);
  // receive: SET from one slot, ADD from both
  CxSources src;
  memset(&src, 0, sizeof(src));
  src.count = 2; src.ep[0] = a.ep(); src.ep[1] = b.ep(); src.seq[0] = src.seq[1] = 1;
  src.cap[0] = src.cap[1] = (uint32_t)cap;
  std::vector<float> out((size_t)n + 1, 7.f);
  CxApplyArgs args;
  memset(&args, 0, sizeof(args));
  args.op = CX_OP_ADD; args.out_dtype = CX_F32; args.out = out.data(); args.scale = 1.f;
  uint32_t status = 0;
  CHECK(cx_apply_host(&src, n, &args, &status, kTimeout) == 0);
  CHECK(status == 0);
  for (int64_t i = 0; i < n; ++i) CHECK(out[i] == 7.f + dense[i] + dense[i]);
  CHECK(out[(size_t)n] == 7.f);
  src.count = 1;
  args.op = CX_OP_SET;
  CHECK(cx_apply_host(&src, n, &args, &status, kTimeout) == 0);
  for (int64_t i = 0; i < n; ++i) CHECK(out[i] == dense[i]);
  CHECK(out[(size_t)n] == 7.f && status == 0 && a.intact() && b.intact());
}

static void dense_case(int64_t n) {
  uint32_t seed = (uint32_t)n + 11;
  std::vector<float> g((size_t)n), r((size_t)n), own((size_t)n), out((size_t)n + 1, -1.f);
  for (int64_t i = 0; i < n; ++i) { g[i] = rnd(seed); r[i] = rnd(seed); own[i] = rnd(seed); }
  const std::vector<float> r0 = r;
  Slot a(0, 4 * n);
  CxTargets tg;
  memset(&tg, 0, sizeof(tg));
  tg.count = 1; tg.ep[0] = a.ep();
  CHECK(cx_dense_send_host(CX_F32, g.data(), r.data(), n, 1, &tg, nullptr, nullptr, 0) == 0);
  CxSources src;
  memset(&src, 0, sizeof(src));
  src.count = 1; src.ep[0] = a.ep(); src.seq[0] = 1;
  uint32_t status = 0;
  CHECK(cx_dense_reduce_host(CX_F32, out.data(), own.data(), n, &src, 1.f, nullptr, 0, nullptr, nullptr, 0,
                             &status, kTimeout) == 0);
  CHECK(status == 0 && a.intact() && out[(size_t)n] == -1.f);
  for (int64_t i = 0; i < n; ++i) { CHECK(out[i] == own[i] + (g[i] + r0[i])); CHECK(r[i] == 0.f); }
}

static void rle_case(int64_t n, float thr) {
  uint32_t seed = (uint32_t)n * 31 + 5;
  std::vector<float> g((size_t)n + 1), r((size_t)n + 1, 0.f), out((size_t)n + 1, 9.f);   // never empty: n = 0 too
  for (int64_t i = 0; i < n; ++i) g[i] = (lcg(seed) & 3) ? rnd(seed) : 0.f;
  const int64_t room = 16 + 8 * n;
  Slot a(0, room);
  CxTargets tg;
  memset(&tg, 0, sizeof(tg));
  tg.count = 1; tg.ep[0] = a.ep();
  CHECK(cx_rle_send_host(CX_F32, g.data(), r.data(), n, &thr, room, 1, &tg, 0) == 0);
  uint32_t status = 0;
  const CxEndpoint ep = a.ep();
  CHECK(cx_rle_recv_host(&ep, 1, out.data(), n, 0, room, &status, kTimeout) == 0);
  CHECK(status == 0 && a.intact() && out[(size_t)n] == 9.f);
  for (int64_t i = 0; i < n; ++i) {
    const bool yes = fabsf(g[i]) >= thr && !(thr == 0.f && g[i] == 0.f);
    CHECK(out[i] == (yes ? g[i] : 0.f));
    CHECK(r[i] == (yes ? 0.f : g[i]));
  }
  if (n >= 4) {   // a corrupted run length must be refused without touching the output
    int32_t nnz;
    memcpy(&nnz, reinterpret_cast<char*>(ep.pairs) + 4, 4);
    int32_t* run0 = reinterpret_cast<int32_t*>(reinterpret_cast<char*>(ep.pairs) + 16 + 4 * (int64_t)nnz);
    *run0 += 1;
    std::vector<float> keep(out);
    status = 0;
    CHECK(cx_rle_recv_host(&ep, 1, out.data(), n, 0, room, &status, kTimeout) == 0);
    CHECK(status == CX_ST_BAD_HEADER && out == keep);
  }
}

// two "ranks" exchange compressed vectors for many steps through two slots per direction
static void protocol_rank(int me, Slot* mine, Slot* theirs, int64_t n, int steps, int* failures) {
  std::vector<float> g((size_t)n), r((size_t)n, 0.f), out((size_t)n);
  const float thr = 0.5f;
  for (int s = 1; s <= steps; ++s) {
    for (int64_t i = 0; i < n; ++i) g[i] = ((i + s + me) % 3 == 0) ? 1.f + (float)me : 0.25f;
    CxTargets tg;
    memset(&tg, 0, sizeof(tg));
    tg.count = 1; tg.ep[0] = theirs[s & 1].ep();
    std::fill(r.begin(), r.end(), 0.f);
    if (cx_compress_host(CX_F32, g.data(), r.data(), n, &thr, (uint32_t)n, (uint64_t)s, &tg, nullptr, me)) ++*failures;
    CxSources src;
    memset(&src, 0, sizeof(src));
    src.count = 1; src.ep[0] = mine[s & 1].ep(); src.seq[0] = (uint64_t)s; src.cap[0] = (uint32_t)n;
    CxApplyArgs args;
    memset(&args, 0, sizeof(args));
    args.op = CX_OP_SET; args.out_dtype = CX_F32; args.out = out.data(); args.scale = 1.f;
    uint32_t status = 0;
    if (cx_apply_host(&src, n, &args, &status, kTimeout) || status) ++*failures;
    const int peer = 1 - me;
    for (int64_t i = 0; i < n; ++i) {
      const float want = ((i + s + peer) % 3 == 0) ? 1.f + (float)peer : 0.f;
      if (out[i] != want) { ++*failures; break; }
    }
  }
}

static void protocol_case() {
  const int64_t n = 5000;
  const int steps = 200;
  std::vector<Slot> s0, s1;
  for (int k = 0; k < 2; ++k) { s0.emplace_back(n, 8 * n); s1.emplace_back(n, 8 * n); }
  int f0 = 0, f1 = 0;
  std::thread t0(protocol_rank, 0, s0.data(), s1.data(), n, steps, &f0);
  std::thread t1(protocol_rank, 1, s1.data(), s0.data(), n, steps, &f1);
  t0.join();
  t1.join();
  CHECK(f0 == 0 && f1 == 0);
  for (int k = 0; k < 2; ++k) CHECK(s0[k].intact() && s1[k].intact());
  // a payload that never arrives: bounded wait, status instead of a hang
  Slot lone(n, 8 * n);
  CxSources src;
  memset(&src, 0, sizeof(src));
  src.count = 1; src.ep[0] = lone.ep(); src.seq[0] = 1; src.cap[0] = (uint32_t)n;
  std::vector<float> out((size_t)n, 3.f);
  CxApplyArgs args;
  memset(&args, 0, sizeof(args));
  args.op = CX_OP_ADD; args.out_dtype = CX_F32; args.out = out.data(); args.scale = 1.f;
  uint32_t status = 0;
  CHECK(cx_apply_host(&src, n, &args, &status, 20ull * 1000000ull) == 0);
  CHECK(status == CX_ST_TIMEOUT && out[0] == 3.f && out[(size_t)n - 1] == 3.f);
}

int main(int argc, char** argv) {
  const bool only_protocol = argc > 1 && !strcmp(argv[1], "--protocol");
  if (!only_protocol) {
    const int64_t sizes[] = {0, 1, 2, 3, 31, 32, 33, 1023, 1024, 1025, 2047, 2048, 2049, 4097, 10007};
    for (int64_t n : sizes) {
      if (n > 0) {
        sparse_case(n, 10.f, n);              // nothing survives
        sparse_case(n, 0.5f, n);              // room for everything
        sparse_case(n, 0.f, n > 3 ? n / 3 : 1);  // more survivors than capacity
        int64_t exact = 0;                    // exactly `capacity` survivors: the data depend on
        // the capacity through the seed, so look for a capacity that equals its own survivor count
        for (int64_t cap = 1; cap <= n; ++cap) {
          uint32_t s2 = (uint32_t)(n * 7919 + cap);
          int64_t c = 0;
          for (int64_t i = 0; i < n; ++i) { const float a = rnd(s2), b = 0.25f * rnd(s2); if (fabsf(a + b) > 0.5f) ++c; }
          if (c == cap) { exact = cap; break; }
          if (n > 64 && cap > 64) break;      // bounded search on the large sizes
        }
        if (exact) sparse_case(n, 0.5f, exact);
        dense_case(n);
      }
      rle_case(n, 0.f);
      rle_case(n, 0.6f);
      rle_case(n, 5.f);
    }
  }
  protocol_case();
  if (g_fail) { fprintf(stderr, "%d checks failed (%s)\n", g_fail, g_err); return 1; }
  printf("host selftest passed\n");
  return 0;
}
