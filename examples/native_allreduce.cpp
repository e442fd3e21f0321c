// The allreduce collectives from C++, without Python: the scenario of the reference's C++ tests
// (test/BigRingAllreduce.cpp, test/RingAllreduce.cpp, test/AllToOneAllreduce.cpp) as one program
// that starts its own ranks.
//
//   native_allreduce [--ranks P] [--kind K] [--size N] [--runs R] [--ratio RHO] [--host]
//
// K numbers the collectives like the reference's benchmark does (0 AllToOne, 1 Comprex_AllToOne,
// 2 Ring, 3 Comprex_Ring, 4 BigRing, 5 Comprex_BigRing; default 5).  The program forks P processes;
// each joins the job through GaspiEnvironment_new (one GPU per rank, or host memory with --host or
// when no GPU is present) and runs R allreduces of the vector values[i] = i * (1 - 2 * (i % 2)).
// Compressed kinds: one rank (for the ring: every rank, on the chunk it owns) keeps accumulating
// the results while the others start from `values` again each run; after `flush` the accumulator
// must hold exactly (R * (P - 1) + 1) * values: nothing that compression held back is lost.
// Dense kinds: every rank must hold P * values after one call.  Prints "+++ PASSED +++" or
// "--- FAILED ---" and exits with the number of ranks that failed.
//
// Build (from the repository root, after `python -m comprex_b200.build`):
//   g++ -std=c++17 -O2 examples/native_allreduce.cpp -Icomprex_b200/csrc -Lcomprex_b200/lib
//       -lcomprex_b200 -Wl,-rpath,$PWD/comprex_b200/lib -o native_allreduce
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "cx_collectives.h"

extern "C" {
// the reference's names for the runtime handle and the default collective
CxComm* GaspiEnvironment_new(int segment_size);
void GaspiEnvironment_del(CxComm* self);
int GaspiEnvironment_get_rank(CxComm* self);
int GaspiEnvironment_get_ranks(CxComm* self);
void GaspiEnvironment_barrier(CxComm* self);
struct CxRefAllreduce;
CxRefAllreduce* Comprex_BigRingAllreduce_new(CxComm* env);
void Comprex_BigRingAllreduce_del(CxRefAllreduce* self);
void Comprex_BigRingAllreduce_setupConnections(CxRefAllreduce* self, int size, int tag, float ratio, float size_factor);
void Comprex_BigRingAllreduce_apply(CxRefAllreduce* self, float* data, int size);
void Comprex_BigRingAllreduce_flush(CxRefAllreduce* self, float* data, int size);
}

namespace {

struct Options {
  int ranks = 2, kind = CX_AR_COMPREX_BIGRING, size = 1000, runs = 20;
  float ratio = 0.01f;
  bool host = false;
};

// A vector in the memory the environment lives in (device memory on a GPU rank).
struct Vector {
  bool cuda;
  int n;
  float* p;
  Vector(bool on_gpu, int size) : cuda(on_gpu), n(size) {
    p = reinterpret_cast<float*>(cuda ? cx_cuda_malloc((int64_t)n * 4) : cx_host_alloc((int64_t)n * 4));
  }
  ~Vector() { if (cuda) cx_cuda_free(p); else cx_host_free(p); }
  void put(const std::vector<float>& h, int first = 0, int count = -1) {
    if (count < 0) count = n;
    if (!count) return;
    if (cuda) { cx_cuda_memcpy(p + first, h.data() + first, (int64_t)count * 4, 1, nullptr); cx_cuda_stream_sync(nullptr); }
    else memcpy(p + first, h.data() + first, (size_t)count * 4);
  }
  std::vector<float> get() const {
    std::vector<float> h(n);
    if (cuda) { cx_cuda_memcpy(h.data(), p, (int64_t)n * 4, 2, nullptr); cx_cuda_stream_sync(nullptr); }
    else memcpy(h.data(), p, (size_t)n * 4);
    return h;
  }
};

int run_rank(const Options& o, int rank, const std::string& job) {
  setenv("CX_JOB", job.c_str(), 1);
  setenv("CX_RANK", std::to_string(rank).c_str(), 1);
  setenv("CX_RANKS", std::to_string(o.ranks).c_str(), 1);
  if (o.host) setenv("CX_HOST", "1", 1);
  CxComm* env = GaspiEnvironment_new(64 << 20);
  if (!env) return 1;
  const bool cuda = !o.host && cx_cuda_device_count() > 0;
  const int me = GaspiEnvironment_get_rank(env), nr = GaspiEnvironment_get_ranks(env);
  const int n = o.size;
  std::vector<float> values(n), gold(n);
  for (int i = 0; i < n; ++i) values[i] = (float)(i * (1 - 2 * (i % 2)));
  const bool compressed = o.kind == CX_AR_COMPREX_ALLTOONE || o.kind == CX_AR_COMPREX_RING || o.kind == CX_AR_COMPREX_BIGRING;
  const float size_factor = 3.0f;      // room for a full flush (src/comprEx.tpp:61)
  int errors = 0;
  {
    Vector data(cuda, n);
    data.put(values);
    if (!compressed) {
      CxAllreduce* ar = cx_allreduce_create(env, o.kind, n, CX_F32, 1.f, 1.f, 0, 0);
      if (!ar || cx_allreduce_apply(ar, data.p, nullptr) || cx_comm_sync(env, nullptr) || cx_comm_check(env)) {
        fprintf(stderr, "rank %d: %s\n", me, cx_last_error());
        errors = n;
      } else {
        const std::vector<float> got = data.get();
        for (int i = 0; i < n; ++i) errors += got[i] != nr * values[i];
      }
      cx_allreduce_destroy(ar);
    } else {
      // the part of the vector this rank accumulates in: everything on the accumulating rank, for
      // the ring the chunk this rank owns (chunk (rank + 1) mod P; the first size mod P chunks
      // are one element longer, src/allreduce.tpp:279-295)
      int keep_lo = 0, keep_hi = me == 0 ? n : 0;
      if (o.kind == CX_AR_COMPREX_RING) {
        const int ch = (me + 1) % nr, base = n / nr, rem = n % nr;
        keep_lo = ch * base + (ch < rem ? ch : rem);
        keep_hi = keep_lo + base + (ch < rem ? 1 : 0);
      }
      for (int i = 0; i < n; ++i) gold[i] = (float)(o.runs * (nr - 1) + 1) * values[i];
      CxRefAllreduce* ref = nullptr;
      CxAllreduce* ar = nullptr;
      if (o.kind == CX_AR_COMPREX_BIGRING) {       // through the reference's own C names
        ref = Comprex_BigRingAllreduce_new(env);
        Comprex_BigRingAllreduce_setupConnections(ref, n, 0, o.ratio, size_factor);
      } else {
        ar = cx_allreduce_create(env, o.kind, n, CX_F32, o.ratio, size_factor, 0, 0);
        if (!ar) { fprintf(stderr, "rank %d: %s\n", me, cx_last_error()); errors = n; }
      }
      for (int run = 0; run < o.runs && !errors; ++run) {
        GaspiEnvironment_barrier(env);
        data.put(values, 0, keep_lo);                       // everything outside the kept part starts over
        data.put(values, keep_hi, n - keep_hi);
        if (ref) Comprex_BigRingAllreduce_apply(ref, data.p, n);
        else if (cx_allreduce_apply(ar, data.p, nullptr) || cx_comm_sync(env, nullptr) || cx_comm_check(env)) {
          fprintf(stderr, "rank %d run %d: %s\n", me, run, cx_last_error());
          errors = n;
        }
      }
      if (!errors) {
        if (ref) Comprex_BigRingAllreduce_flush(ref, data.p, n);
        else if (cx_allreduce_flush(ar, data.p, nullptr) || cx_comm_sync(env, nullptr) || cx_comm_check(env)) errors = n;
        const std::vector<float> got = data.get();
        for (int i = keep_lo; i < keep_hi; ++i) {
          if (got[i] != gold[i]) {
            if (errors < 5) fprintf(stderr, "rank %d [%d]: result %g gold %g\n", me, i, got[i], gold[i]);
            ++errors;
          }
        }
      }
      if (ref) Comprex_BigRingAllreduce_del(ref);
      cx_allreduce_destroy(ar);
    }
    GaspiEnvironment_barrier(env);
  }
  GaspiEnvironment_del(env);
  return errors ? 1 : 0;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() { return i + 1 < argc ? argv[++i] : (char*)"0"; };
    if (a == "--ranks") o.ranks = atoi(next());
    else if (a == "--kind") o.kind = atoi(next());
    else if (a == "--size") o.size = atoi(next());
    else if (a == "--runs") o.runs = atoi(next());
    else if (a == "--ratio") o.ratio = (float)atof(next());
    else if (a == "--host") o.host = true;
    else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 2; }
  }
  if (o.ranks < 1 || o.ranks > CX_MAX_PEERS || o.kind < 0 || o.kind > 5 || o.size < 1) { fprintf(stderr, "bad arguments\n"); return 2; }
  const std::string job = "native" + std::to_string((long)getpid());
  std::vector<pid_t> kids;
  for (int r = 0; r < o.ranks; ++r) {       // fork before anything touches CUDA
    const pid_t pid = fork();
    if (pid == 0) _exit(run_rank(o, r, job));
    kids.push_back(pid);
  }
  int failed = 0;
  for (pid_t pid : kids) {
    int st = 0;
    waitpid(pid, &st, 0);
    failed += !(WIFEXITED(st) && WEXITSTATUS(st) == 0);
  }
  printf(failed ? "--- FAILED ---\n" : "+++ PASSED +++\n");
  return failed;
}
