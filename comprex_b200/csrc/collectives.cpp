// Native collectives: the six allreduce classes of the reference (include/allreduce.hxx:15-211,
// src/allreduce.tpp:20-721) and its runtime handle (include/gaspiEnvironment.hxx:9-28) behind a
// flat C ABI, usable from C or C++ without Python (src/allreduce_C.cpp:12-122 and
// src/GPI_C.cpp:44-73 export the same names for the reference's classes).
//
// A collective here is a short list of launches of this library's primitives (threshold,
// compress-and-store, wait-and-decode, dense send / reduce, the in-switch allreduce), built per
// call as an array of CxOp and run with cx_run_ops on the caller's stream.  The schedules are the
// NVSwitch forms: every rank stores straight into its peers' receive slots, nothing is forwarded
// hop by hop.
//
//   CxComm       rank, size, the symmetric heap (the same block sequence on every rank; a block's
//                address on rank r is r's base + offset), a status word, a barrier.  The heap
//                comes from the caller (cx_comm_create: bases already exchanged, e.g. by the
//                Python layer) or from cx_comm_bootstrap, which lets the ranks of one host meet in
//                a POSIX shared-memory control block and exchange CUDA IPC handles (GPU ranks) or
//                map each other's shared-memory segments (host ranks).
//   CxAllreduce  one collective object: its slots, residuals, scratch and step counter.
#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <string>
#include <vector>

#include "cx_collectives.h"

int cx_set_error(const char* where, int cuda_err);

namespace {

int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

// What the ranks of one host share while they meet.
struct Ctrl {
  std::atomic<uint32_t> barrier_count;
  uint32_t pad[15];
  std::atomic<uint32_t> posted[CX_MAX_PEERS];   // 1: this rank's handle / segment is there
  char handle[CX_MAX_PEERS][64];
};

struct Block { int64_t off; int64_t bytes; };

}  // namespace

struct CxComm {
  int dev;                 // CX_DEV_HOST / CX_DEV_CUDA
  int device;              // CUDA ordinal
  int rank, ranks;
  uint64_t timeout_ns;
  void* base[CX_MAX_PEERS];
  void* mc_base;           // multicast alias of the heap or NULL
  int64_t bytes, used;
  uint32_t* status_host;   // status word: kernels OR bits in, cx_comm_check reads and clears
  uint32_t* status_dev;
  // bootstrap only
  bool owns_heap;
  Ctrl* ctrl;
  std::string job;
  std::vector<void*> opened;   // peers' mappings to release
  std::vector<void*> scratch;  // local allocations of the collectives

  void* local_alloc(int64_t nbytes) {
    void* p = dev == CX_DEV_CUDA ? cx_cuda_malloc(std::max<int64_t>(nbytes, 64)) : cx_host_alloc(std::max<int64_t>(nbytes, 64));
    if (p) scratch.push_back(p);
    return p;
  }
  bool alloc(int64_t nbytes, Block* out) {   // collective: same sizes in the same order everywhere
    const int64_t off = round_up(used, 256);
    if (off + nbytes > bytes) return false;
    used = off + nbytes;
    out->off = off;
    out->bytes = nbytes;
    return true;
  }
  char* at(int r, int64_t off) const { return reinterpret_cast<char*>(base[r]) + off; }
};

namespace {

// ---- slots -------------------------------------------------------------------------------------
struct Slot {
  Block b;
  int64_t n;
  uint32_t cap;
  bool sparse;
};

int64_t sparse_bytes(int64_t n, uint32_t cap) {
  const int64_t nsub = std::max<int64_t>((n + CX_SUBTILE - 1) / CX_SUBTILE, 1);
  return 64 + round_up(8 * nsub, 16) + 8 * (int64_t)std::max<uint32_t>(cap, 1);
}

CxEndpoint endpoint(const CxComm* c, const Slot& s, int rank) {   // rank < 0: the multicast alias
  char* b = rank < 0 ? reinterpret_cast<char*>(c->mc_base) + s.b.off : c->at(rank, s.b.off);
  CxEndpoint e;
  e.hdr = reinterpret_cast<CxHeader*>(b);
  if (s.sparse) {
    const int64_t nsub = std::max<int64_t>((s.n + CX_SUBTILE - 1) / CX_SUBTILE, 1);
    e.table = reinterpret_cast<uint32_t*>(b + 64);
    e.pairs = reinterpret_cast<CxPair*>(b + 64 + round_up(8 * nsub, 16));
  } else {
    e.table = nullptr;
    e.pairs = reinterpret_cast<CxPair*>(b + 64);
  }
  return e;
}

uint32_t cap_for(int64_t n, float size_factor) {   // pairs in n*4*size_factor bytes (src/comprEx.tpp:61)
  const int64_t c = ((int64_t)((double)n * 4.0 * size_factor) - 8) / 8;
  return (uint32_t)std::max<int64_t>(c, 1);
}

void chunks(int64_t size, int ranks, int64_t align, std::vector<int64_t>& sizes, std::vector<int64_t>& starts) {
  sizes.assign(ranks, 0);
  starts.assign(ranks, 0);
  if (align > 1) {
    const int64_t base = (size / ranks) / align * align;
    for (int i = 0; i < ranks - 1; ++i) sizes[i] = base;
    sizes[ranks - 1] = size - base * (ranks - 1);
  } else {   // the reference's rule: the remainder goes to the first chunks (src/allreduce.tpp:279-295)
    const int64_t base = size / ranks, rem = size % ranks;
    for (int i = 0; i < ranks; ++i) sizes[i] = base + (i < rem ? 1 : 0);
  }
  for (int i = 1; i < ranks; ++i) starts[i] = starts[i - 1] + sizes[i - 1];
}

struct Compressor {   // scratch, threshold cell and statistics of one sparse sender
  void* workspace;
  int64_t ws_bytes;
  float* thr;
  void* thr_ws;        // scratch of the exact (whole-vector) threshold selection
  CxStats* stats;
};

}  // namespace

struct CxAllreduce {
  CxComm* c;
  int kind;
  int64_t size;
  int dtype;
  float ratio, size_factor;
  int chief;
  bool consistent;
  uint64_t step;
  int es;
  // sampling of the sender-side threshold (src/allreduce.tpp:401-403, 625-627; AllToOne :142)
  int subsamples;
  float sample_factor;
  uint32_t cap;
  std::vector<int64_t> seg_size, seg_start;
  std::vector<std::vector<Slot>> a, b;   // [rank][parity]: first / second exchange of the schedule
  std::vector<Slot> bc;                  // [parity]: the chief's broadcast
  float* rests;
  float* owner_rests;
  Compressor comp;
  std::vector<Compressor> chunk_comp;
  void* counters;
  // in-switch dense allreduce
  bool mm;
  Block mm_stage, mm_flags;
  int64_t mm_stride;
  bool mm_one_shot;
  void* mm_counters;
  float result_scale;
};

namespace {

bool make_compressor(CxComm* c, Compressor* k) {
  k->ws_bytes = cx_workspace_bytes(0);
  k->workspace = c->local_alloc(k->ws_bytes);
  k->thr = reinterpret_cast<float*>(c->local_alloc(64));
  k->thr_ws = c->local_alloc(cx_threshold_workspace_bytes());
  k->stats = reinterpret_cast<CxStats*>(c->local_alloc(sizeof(CxStats)));
  return k->workspace && k->thr && k->thr_ws && k->stats;
}

CxOp blank(const CxAllreduce* ar, int kind, int dtype, int64_t n, int lane) {
  CxOp o;
  memset(&o, 0, sizeof(o));
  o.kind = kind;
  o.dev = ar->c->dev;
  o.dtype = dtype;
  o.n = n;
  o.lane = lane;
  o.src_rank = (uint32_t)ar->c->rank;
  o.status = ar->c->status_dev;
  o.timeout_ns = ar->c->timeout_ns;
  return o;
}

CxOp op_threshold(const CxAllreduce* ar, const void* g, int gdtype, float* r, int64_t n, const Compressor& k,
                  int subsamples, float factor, int lane) {
  CxOp o = blank(ar, CX_OPK_THRESHOLD, gdtype, n, lane);
  o.g = g; o.r = r; o.thr = k.thr; o.ratio = ar->ratio;
  o.default_subsamples = subsamples; o.subsample_factor = factor;
  o.workspace = k.thr_ws; o.ws_bytes = cx_threshold_workspace_bytes();
  return o;
}

void set_targets(const CxAllreduce* ar, CxTargets* tg, const Slot& s, const std::vector<int>& dests) {
  tg->count = (int32_t)dests.size();
  tg->pad = 0;
  for (size_t i = 0; i < dests.size(); ++i) tg->ep[i] = endpoint(ar->c, s, dests[i]);
  if (ar->c->mc_base && dests.size() >= 2 && dests.size() < CX_MAX_PEERS) {   // one store through the switch
    tg->pad = CX_TG_MULTICAST;
    tg->ep[dests.size()] = endpoint(ar->c, s, -1);
  }
}

CxOp op_compress(const CxAllreduce* ar, const void* g, int gdtype, float* r, int64_t n, const Compressor& k,
                 const Slot& s, const std::vector<int>& dests, int lane) {
  CxOp o = blank(ar, CX_OPK_COMPRESS, gdtype, n, lane);
  o.g = g; o.r = r; o.thr = k.thr; o.cap = s.cap;
  o.workspace = k.workspace; o.ws_bytes = k.ws_bytes; o.stats = k.stats;
  set_targets(ar, &o.tg, s, dests);
  return o;
}

void set_sources(const CxAllreduce* ar, CxSources* src, const std::vector<const Slot*>& slots) {
  src->count = (int32_t)slots.size();
  for (size_t i = 0; i < slots.size(); ++i) {
    src->ep[i] = endpoint(ar->c, *slots[i], ar->c->rank);
    src->seq[i] = 0;
    src->cap[i] = slots[i]->cap;
  }
}

CxOp op_apply(const CxAllreduce* ar, const std::vector<const Slot*>& slots, int64_t n, int op, void* out,
              int out_dtype, float scale, int lane) {
  CxOp o = blank(ar, CX_OPK_APPLY, CX_F32, n, lane);
  set_sources(ar, &o.src, slots);
  o.apply.op = op; o.apply.out = out; o.apply.out_dtype = out_dtype; o.apply.scale = scale;
  return o;
}

char* elem(void* data, int64_t i, int es) { return reinterpret_cast<char*>(data) + i * es; }

int run(CxAllreduce* ar, std::vector<CxOp>& ops, void* stream) {
  if (ops.empty()) return 0;
  return cx_run_ops(ops.data(), (int)ops.size(), ar->step, stream);
}

// The compress kernel cuts the pair list into regions; sub-tile s may only use region s mod R.
int flush_rounds(int64_t n, uint32_t cap) {
  const int64_t nsub = (n + CX_SUBTILE - 1) / CX_SUBTILE;
  int64_t regions = 1;
  while (regions < CX_MAX_REGIONS && nsub / (2 * regions) >= 8 && cap / (2 * regions) >= 256) regions *= 2;
  const int64_t region_size = std::max<int64_t>(cap / regions, 1);
  const int64_t per_region = (nsub + regions - 1) / regions * CX_SUBTILE;
  return (int)std::max<int64_t>(1, (per_region + region_size - 1) / region_size);
}

int zero_cell(CxAllreduce* ar, float* cell, void* stream) { return cx_fill_zero(ar->c->dev, cell, 4, stream); }

// ---- the schedules ---------------------------------------------------------------------------------
int bigring_dense(CxAllreduce* ar, void* data, void* stream) {
  CxComm* c = ar->c;
  const int me = c->rank, nr = c->ranks;
  ar->step += 1;
  if (nr == 1) return 0;
  std::vector<CxOp> ops;
  if (ar->mm) {
    CxOp o = blank(ar, CX_OPK_MM_ALLREDUCE, ar->dtype, ar->size, 0);
    o.out = data; o.own = data;
    o.g = c->at(me, ar->mm_stage.off);
    o.r = reinterpret_cast<float*>(reinterpret_cast<char*>(c->mc_base) + ar->mm_stage.off);
    o.starts[0] = ar->mm_stride; o.starts[1] = ar->mm_one_shot ? 1 : 0; o.starts[2] = 32 << 20;
    for (int r = 0; r < nr; ++r) o.lens[r] = (int64_t)(intptr_t)c->at(r, ar->mm_flags.off);
    o.cap = (uint32_t)nr; o.workspace = ar->mm_counters; o.scale = ar->result_scale;
    ops.push_back(o);
    return run(ar, ops, stream);
  }
  const int par = (int)(ar->step & 1);
  std::vector<int> peers;
  for (int r = 0; r < nr; ++r) if (r != me) peers.push_back(r);
  CxOp s = blank(ar, CX_OPK_DENSE_SEND, ar->dtype, ar->size, 0);
  s.g = data; s.workspace = ar->counters;
  s.tg.count = (int32_t)peers.size();
  for (size_t i = 0; i < peers.size(); ++i) s.tg.ep[i] = endpoint(c, ar->a[me][par], peers[i]);
  ops.push_back(s);
  CxOp r = blank(ar, CX_OPK_DENSE_REDUCE, ar->dtype, ar->size, 0);
  r.out = data; r.own = data; r.scale = ar->result_scale;
  std::vector<const Slot*> src;
  for (int k = 1; k < nr; ++k) src.push_back(&ar->a[(me - k + nr) % nr][par]);   // ring arrival order
  set_sources(ar, &r.src, src);
  ops.push_back(r);
  return run(ar, ops, stream);
}

int ring_dense(CxAllreduce* ar, void* data, void* stream) {
  CxComm* c = ar->c;
  const int me = c->rank, nr = c->ranks;
  if (ar->mm || nr == 1) return bigring_dense(ar, data, stream);
  ar->step += 1;
  const int par = (int)(ar->step & 1), mine = (me + 1) % nr;
  std::vector<CxOp> ops;
  CxOp s = blank(ar, CX_OPK_DENSE_SEND, ar->dtype, ar->size, 0);
  s.g = data; s.workspace = ar->counters; s.has_ranges = 1;
  int k = 0;
  for (int ch = 0; ch < nr; ++ch) {
    if (ch == mine) continue;
    s.tg.ep[k] = endpoint(c, ar->a[me][par], (ch - 1 + nr) % nr);   // chunk ch belongs to rank ch-1
    s.starts[k] = ar->seg_start[ch]; s.lens[k] = ar->seg_size[ch];
    ++k;
  }
  s.tg.count = k;
  ops.push_back(s);
  std::vector<int> peers;
  for (int r = 0; r < nr; ++r) if (r != me) peers.push_back(r);
  CxOp r = blank(ar, CX_OPK_DENSE_REDUCE, ar->dtype, ar->seg_size[mine], 0);
  r.out = elem(data, ar->seg_start[mine], ar->es); r.own = r.out; r.scale = ar->result_scale;
  r.workspace = ar->counters; r.has_push = 1;
  std::vector<const Slot*> src;
  for (int j : peers) src.push_back(&ar->a[j][par]);
  set_sources(ar, &r.src, src);
  r.tg.count = (int32_t)peers.size();
  for (size_t i = 0; i < peers.size(); ++i) r.tg.ep[i] = endpoint(c, ar->b[me][par], peers[i]);
  ops.push_back(r);
  CxOp g = blank(ar, CX_OPK_DENSE_REDUCE, ar->dtype, ar->size, 0);
  g.out = data; g.scale = 1.f; g.has_ranges = 1;
  src.clear();
  k = 0;
  for (int j : peers) {
    src.push_back(&ar->b[j][par]);
    g.starts[k] = ar->seg_start[(j + 1) % nr]; g.lens[k] = ar->seg_size[(j + 1) % nr];
    ++k;
  }
  set_sources(ar, &g.src, src);
  ops.push_back(g);
  return run(ar, ops, stream);
}

int alltoone_dense(CxAllreduce* ar, void* data, void* stream) {
  CxComm* c = ar->c;
  const int me = c->rank, nr = c->ranks, chief = ar->chief;
  ar->step += 1;
  if (nr == 1) return 0;
  const int par = (int)(ar->step & 1);
  std::vector<CxOp> ops;
  std::vector<int> workers;
  for (int r = 0; r < nr; ++r) if (r != chief) workers.push_back(r);
  if (me != chief) {
    CxOp s = blank(ar, CX_OPK_DENSE_SEND, ar->dtype, ar->size, 0);
    s.g = data; s.workspace = ar->counters; s.tg.count = 1;
    s.tg.ep[0] = endpoint(c, ar->a[me][par], chief);
    ops.push_back(s);
    CxOp r = blank(ar, CX_OPK_DENSE_REDUCE, ar->dtype, ar->size, 0);
    r.out = data; r.scale = 1.f;
    set_sources(ar, &r.src, {&ar->bc[par]});
    ops.push_back(r);
  } else {
    CxOp r = blank(ar, CX_OPK_DENSE_REDUCE, ar->dtype, ar->size, 0);
    r.out = data; r.own = data; r.scale = ar->result_scale; r.workspace = ar->counters; r.has_push = 1;
    std::vector<const Slot*> src;
    for (int w : workers) src.push_back(&ar->a[w][par]);
    set_sources(ar, &r.src, src);
    set_targets(ar, &r.tg, ar->bc[par], workers);
    ops.push_back(r);
  }
  return run(ar, ops, stream);
}

// Comprex_BigRing (src/allreduce.tpp:649-721): one compression stored to all peers, one decode.
int bigring_comprex(CxAllreduce* ar, void* data, bool flush, void* stream) {
  CxComm* c = ar->c;
  const int me = c->rank, nr = c->ranks;
  const int rounds = flush ? flush_rounds(ar->size, ar->cap) : 1;
  for (int rd = 0; rd < rounds; ++rd) {
    ar->step += 1;
    if (nr == 1 && !ar->consistent) continue;
    const int par = (int)(ar->step & 1);
    std::vector<CxOp> ops;
    std::vector<int> dests;
    for (int r = 0; r < nr; ++r) if (r != me || ar->consistent) dests.push_back(r);
    if (flush) { if (int rc = zero_cell(ar, ar->comp.thr, stream)) return rc; }
    else ops.push_back(op_threshold(ar, data, ar->dtype, ar->rests, ar->size, ar->comp, ar->subsamples, ar->sample_factor, 0));
    ops.push_back(op_compress(ar, flush ? nullptr : data, ar->dtype, ar->rests, ar->size, ar->comp, ar->a[me][par], dests, 0));
    std::vector<const Slot*> src;
    if (ar->consistent) for (int j = 0; j < nr; ++j) src.push_back(&ar->a[j][par]);
    else for (int k = 1; k < nr; ++k) src.push_back(&ar->a[(me - k + nr) % nr][par]);
    if (!src.empty())
      ops.push_back(op_apply(ar, src, ar->size, (ar->consistent && rd == 0) ? CX_OP_SET : CX_OP_ADD, data, ar->dtype, 1.f, 0));
    if (int rc = run(ar, ops, stream)) return rc;
  }
  return 0;
}

// Comprex_Ring, direct form (src/allreduce.tpp:420-508): compress every foreign chunk to its owner,
// the owner adds, re-selects and stores to all, everyone decodes.
int ring_comprex(CxAllreduce* ar, void* data, bool flush, void* stream) {
  CxComm* c = ar->c;
  const int me = c->rank, nr = c->ranks, mine = (me + 1) % nr;
  int64_t nmax = 1;
  for (int64_t s : ar->seg_size) nmax = std::max(nmax, s);
  const int rounds = flush ? flush_rounds(nmax, ar->cap) : 1;
  std::vector<int> peers, everyone;
  for (int r = 0; r < nr; ++r) { everyone.push_back(r); if (r != me) peers.push_back(r); }
  for (int rd = 0; rd < rounds; ++rd) {
    ar->step += 1;
    const int par = (int)(ar->step & 1);
    const bool last = rd == rounds - 1;
    std::vector<CxOp> ops;
    for (int k = 1; k < nr; ++k) {   // start behind the own chunk: every rank addresses another owner
      const int ch = (mine + k) % nr;
      const Compressor& kc = ar->chunk_comp[ch];
      float* r = ar->rests + ar->seg_start[ch];
      const void* g = flush ? nullptr : elem(data, ar->seg_start[ch], ar->es);
      if (flush) { if (int rc = zero_cell(ar, kc.thr, stream)) return rc; }
      else ops.push_back(op_threshold(ar, g, ar->dtype, r, ar->seg_size[ch], kc, ar->subsamples, ar->sample_factor, k));
      ops.push_back(op_compress(ar, g, ar->dtype, r, ar->seg_size[ch], kc, ar->a[me][par], {(ch - 1 + nr) % nr}, k));
    }
    if (nr > 1 || ar->consistent) {
      void* mv = elem(data, ar->seg_start[mine], ar->es);
      const int64_t n = ar->seg_size[mine];
      if (!peers.empty()) {
        std::vector<const Slot*> src;
        for (int j : peers) src.push_back(&ar->a[j][par]);
        ops.push_back(op_apply(ar, src, n, CX_OP_ADD, mv, ar->dtype, 1.f, 0));
      }
      if (!flush || last) {
        if (flush) { if (int rc = zero_cell(ar, ar->comp.thr, stream)) return rc; }
        else ops.push_back(op_threshold(ar, mv, ar->dtype, ar->owner_rests, n, ar->comp, 1000, 10.f, 0));
        ops.push_back(op_compress(ar, mv, ar->dtype, ar->owner_rests, n, ar->comp, ar->b[me][par],
                                  ar->consistent ? everyone : peers, 0));
        int k = 1;
        for (int j : (ar->consistent ? everyone : peers)) {
          const int ch = (j + 1) % nr;
          ops.push_back(op_apply(ar, {&ar->b[j][par]}, ar->seg_size[ch], CX_OP_SET,
                                 elem(data, ar->seg_start[ch], ar->es), ar->dtype, 1.f, k++));
        }
      }
    }
    if (int rc = run(ar, ops, stream)) return rc;
  }
  return 0;
}

// Comprex_AllToOne (src/allreduce.tpp:171-258), both legs fresh; flush does not broadcast.
int alltoone_comprex(CxAllreduce* ar, void* data, bool flush, void* stream) {
  CxComm* c = ar->c;
  const int me = c->rank, nr = c->ranks, chief = ar->chief;
  const int rounds = flush ? flush_rounds(ar->size, ar->cap) : 1;
  std::vector<int> workers;
  for (int r = 0; r < nr; ++r) if (r != chief) workers.push_back(r);
  for (int rd = 0; rd < rounds; ++rd) {
    ar->step += 1;
    const int par = (int)(ar->step & 1);
    std::vector<CxOp> ops;
    if (me != chief) {
      if (flush) { if (int rc = zero_cell(ar, ar->comp.thr, stream)) return rc; }
      else ops.push_back(op_threshold(ar, data, ar->dtype, ar->rests, ar->size, ar->comp, ar->subsamples, ar->sample_factor, 0));
      ops.push_back(op_compress(ar, flush ? nullptr : data, ar->dtype, ar->rests, ar->size, ar->comp, ar->a[me][par], {chief}, 0));
      if (!flush) ops.push_back(op_apply(ar, {&ar->bc[par]}, ar->size, CX_OP_SET, data, ar->dtype, 1.f, 0));
    } else if (!workers.empty()) {
      std::vector<const Slot*> src;
      for (int w : workers) src.push_back(&ar->a[w][par]);
      ops.push_back(op_apply(ar, src, ar->size, CX_OP_ADD, data, ar->dtype, 1.f, 0));
      if (!flush) {
        ops.push_back(op_threshold(ar, data, ar->dtype, ar->rests, ar->size, ar->comp, ar->subsamples, ar->sample_factor, 0));
        ops.push_back(op_compress(ar, data, ar->dtype, ar->rests, ar->size, ar->comp, ar->bc[par], workers, 0));
      }
    }
    if (int rc = run(ar, ops, stream)) return rc;
  }
  return 0;
}

bool is_comprex(int kind) {
  return kind == CX_AR_COMPREX_ALLTOONE || kind == CX_AR_COMPREX_RING || kind == CX_AR_COMPREX_BIGRING;
}

}  // namespace

extern "C" {

// ---- communicator ---------------------------------------------------------------------------------
CxComm* cx_comm_create(int dev, int device, int rank, int ranks, void* const* bases, void* mc_base,
                       int64_t bytes, uint64_t timeout_ns) {
  if (ranks < 1 || ranks > CX_MAX_PEERS || rank < 0 || rank >= ranks) { cx_set_error("cx_comm_create: bad rank", 0); return nullptr; }
  if (dev == CX_DEV_CUDA && cx_cuda_set_device(device)) return nullptr;
  CxComm* c = new CxComm();
  c->dev = dev; c->device = device; c->rank = rank; c->ranks = ranks; c->timeout_ns = timeout_ns;
  for (int r = 0; r < CX_MAX_PEERS; ++r) c->base[r] = r < ranks ? bases[r] : nullptr;
  c->mc_base = mc_base; c->bytes = bytes; c->used = 0;
  c->owns_heap = false; c->ctrl = nullptr;
  if (dev == CX_DEV_CUDA) {
    void* d = nullptr;
    c->status_host = reinterpret_cast<uint32_t*>(cx_pinned_alloc(64, &d));
    c->status_dev = reinterpret_cast<uint32_t*>(d);
  } else {
    c->status_host = c->status_dev = reinterpret_cast<uint32_t*>(cx_host_alloc(64));
  }
  if (!c->status_host) { delete c; return nullptr; }
  return c;
}

CxComm* cx_comm_bootstrap(const char* job, int rank, int ranks, int dev, int device, int64_t bytes,
                          uint64_t timeout_ns) {
  if (ranks < 1 || ranks > CX_MAX_PEERS || rank < 0 || rank >= ranks || !job) { cx_set_error("cx_comm_bootstrap: bad arguments", 0); return nullptr; }
  if (dev == CX_DEV_CUDA && cx_cuda_set_device(device)) return nullptr;
  bytes = round_up(std::max<int64_t>(bytes, 1 << 16), 1 << 16);
  const std::string ctrl_name = std::string("/cxjob_") + job;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(cx_shm_create(ctrl_name.c_str(), (int64_t)sizeof(Ctrl)));   // zero-filled when new
  if (!ctrl) return nullptr;
  void* mine = nullptr;
  const std::string seg_name = ctrl_name + "_" + std::to_string(rank);
  if (dev == CX_DEV_CUDA) {
    mine = cx_cuda_malloc(bytes);
    if (!mine || cx_cuda_ipc_get(mine, ctrl->handle[rank])) return nullptr;
  } else {
    mine = cx_shm_create(seg_name.c_str(), bytes);
    if (!mine) return nullptr;
    memset(mine, 0, (size_t)bytes);
  }
  ctrl->posted[rank].store(1, std::memory_order_release);
  void* bases[CX_MAX_PEERS] = {nullptr};
  std::vector<void*> opened;
  const uint64_t t0 = now_ns();
  for (int r = 0; r < ranks; ++r) {
    if (r == rank) { bases[r] = mine; continue; }
    while (!ctrl->posted[r].load(std::memory_order_acquire)) {
      if (now_ns() - t0 > timeout_ns) { cx_set_error("cx_comm_bootstrap: a rank did not arrive in time", 0); return nullptr; }
      usleep(200);
    }
    bases[r] = dev == CX_DEV_CUDA ? cx_cuda_ipc_open(ctrl->handle[r])
                                  : cx_shm_open((ctrl_name + "_" + std::to_string(r)).c_str(), bytes);
    if (!bases[r]) return nullptr;
    opened.push_back(bases[r]);
  }
  CxComm* c = cx_comm_create(dev, device, rank, ranks, bases, nullptr, bytes, timeout_ns);
  if (!c) return nullptr;
  c->owns_heap = true; c->ctrl = ctrl; c->job = ctrl_name; c->opened = opened;
  if (cx_comm_barrier(c)) { return nullptr; }     // everybody has mapped everybody: the names can go
  if (dev != CX_DEV_CUDA) cx_shm_unlink(seg_name.c_str());
  if (rank == 0) cx_shm_unlink(ctrl_name.c_str());
  return c;
}

int cx_comm_barrier(CxComm* c) {
  if (!c->ctrl || c->ranks == 1) return 0;
  const uint32_t n = c->ctrl->barrier_count.fetch_add(1, std::memory_order_acq_rel) + 1;
  const uint32_t target = ((n - 1) / (uint32_t)c->ranks + 1) * (uint32_t)c->ranks;
  const uint64_t t0 = now_ns();
  while (c->ctrl->barrier_count.load(std::memory_order_acquire) < target) {
    if (now_ns() - t0 > c->timeout_ns) return cx_set_error("cx_comm_barrier: timed out", 0);
    usleep(50);
  }
  return 0;
}

int cx_comm_rank(const CxComm* c) { return c->rank; }
int cx_comm_ranks(const CxComm* c) { return c->ranks; }

int cx_comm_sync(CxComm* c, void* stream) {
  return c->dev == CX_DEV_CUDA ? cx_cuda_stream_sync(stream) : 0;
}

uint32_t cx_comm_check(CxComm* c) {
  const uint32_t v = *reinterpret_cast<volatile uint32_t*>(c->status_host);
  *reinterpret_cast<volatile uint32_t*>(c->status_host) = 0;
  return v & ~CX_ST_OVERFLOW;
}

void cx_comm_destroy(CxComm* c) {
  if (!c) return;
  if (c->dev == CX_DEV_CUDA) cx_cuda_stream_sync(nullptr);
  if (c->ctrl) cx_comm_barrier(c);      // nobody frees memory a peer may still be storing into
  for (void* p : c->scratch) { if (c->dev == CX_DEV_CUDA) cx_cuda_free(p); else cx_host_free(p); }
  if (c->owns_heap) {
    for (void* p : c->opened) { if (c->dev == CX_DEV_CUDA) cx_cuda_ipc_close(p); else cx_shm_close(p, c->bytes); }
    if (c->ctrl) cx_comm_barrier(c);    // every importer has unmapped before the owner frees
    if (c->dev == CX_DEV_CUDA) cx_cuda_free(c->base[c->rank]); else cx_shm_close(c->base[c->rank], c->bytes);
    if (c->ctrl) cx_shm_close(c->ctrl, (int64_t)sizeof(Ctrl));
  }
  if (c->dev == CX_DEV_CUDA) cx_pinned_free(c->status_host); else cx_host_free(c->status_host);
  delete c;
}

// ---- allreduce objects -------------------------------------------------------------------------------
CxAllreduce* cx_allreduce_create(CxComm* c, int kind, int64_t size, int dtype, float ratio, float size_factor,
                                 int chief, int flags) {
  if (kind < 0 || kind > CX_AR_COMPREX_BIGRING || size < 1 || size > 0x7fffffffLL) { cx_set_error("cx_allreduce_create: bad kind or size", 0); return nullptr; }
  if (dtype != CX_F32 && dtype != CX_BF16 && dtype != CX_F16) { cx_set_error("cx_allreduce_create: bad dtype", 0); return nullptr; }
  CxAllreduce* ar = new CxAllreduce();
  ar->c = c; ar->kind = kind; ar->size = size; ar->dtype = dtype; ar->ratio = ratio; ar->size_factor = size_factor;
  ar->chief = chief; ar->consistent = (flags & CX_AR_CONSISTENT) != 0; ar->step = 0;
  ar->es = dtype == CX_F32 ? 4 : 2;
  ar->rests = ar->owner_rests = nullptr; ar->mm = false; ar->result_scale = 1.f; ar->cap = 1;
  ar->counters = c->local_alloc(64);
  const int nr = c->ranks;
  bool ok = ar->counters != nullptr;
  auto slots = [&](std::vector<std::vector<Slot>>& v, int64_t n, uint32_t cap, bool sparse) {
    v.assign(nr, std::vector<Slot>(2));
    for (int r = 0; r < nr; ++r)
      for (int par = 0; par < 2; ++par) {
        Slot& s = v[r][par];
        s.n = n; s.cap = cap; s.sparse = sparse;
        ok = ok && c->alloc(sparse ? sparse_bytes(n, cap) : 64 + round_up(std::max<int64_t>(n * ar->es, 16), 16), &s.b);
      }
  };
  auto one = [&](std::vector<Slot>& v, int64_t n, uint32_t cap, bool sparse) {
    v.assign(2, Slot());
    for (int par = 0; par < 2; ++par) {
      v[par].n = n; v[par].cap = cap; v[par].sparse = sparse;
      ok = ok && c->alloc(sparse ? sparse_bytes(n, cap) : 64 + round_up(std::max<int64_t>(n * ar->es, 16), 16), &v[par].b);
    }
  };
  if (is_comprex(kind)) {
    ar->subsamples = 1000 / nr; ar->sample_factor = 4.f;
    ar->rests = reinterpret_cast<float*>(c->local_alloc(size * 4));
    ok = ok && ar->rests && make_compressor(c, &ar->comp);
  }
  switch (kind) {
    case CX_AR_BIGRING:
    case CX_AR_RING: {
      const int64_t nbytes = size * ar->es;
      const char* e1 = getenv("COMPREX_MM_MIN_RANKS");
      const char* e2 = getenv("COMPREX_MM_MIN_BYTES");
      if (c->mc_base && c->dev == CX_DEV_CUDA && nr >= (e1 ? atoi(e1) : 4) && nbytes >= (e2 ? atoll(e2) : (256 << 10))) {
        ar->mm = true;
        ar->mm_one_shot = round_up(nbytes, 16) <= (512 << 10);
        ar->mm_stride = round_up(round_up(nbytes, 16), 256);
        ok = ok && c->alloc(ar->mm_stride * (ar->mm_one_shot ? 2 : 1), &ar->mm_stage) && c->alloc(cx_mm_flag_bytes(), &ar->mm_flags);
        ar->mm_counters = c->local_alloc(cx_mm_counter_bytes());
        ok = ok && ar->mm_counters;
        break;
      }
      chunks(size, nr, 1, ar->seg_size, ar->seg_start);
      const char* e3 = getenv("COMPREX_TWO_SHOT_BYTES");
      const bool two_shot = kind == CX_AR_RING || (nr > 2 && nbytes > (e3 ? atoll(e3) : (1 << 20)));
      if (two_shot) {
        ar->kind = CX_AR_RING;
        int64_t nmax = 1;
        for (int64_t s : ar->seg_size) nmax = std::max(nmax, s);
        slots(ar->a, nmax, 0, false);
        slots(ar->b, nmax, 0, false);
      } else {
        slots(ar->a, size, 0, false);
      }
      break;
    }
    case CX_AR_ALLTOONE:
      slots(ar->a, size, 0, false);
      one(ar->bc, size, 0, false);
      break;
    case CX_AR_COMPREX_BIGRING:
      ar->cap = cap_for(size, size_factor);
      slots(ar->a, size, ar->cap, true);
      break;
    case CX_AR_COMPREX_RING: {
      chunks(size, nr, (flags & CX_AR_ALIGNED_CHUNKS) ? 4 : 1, ar->seg_size, ar->seg_start);
      int64_t nmax = 1;
      for (int64_t s : ar->seg_size) nmax = std::max(nmax, s);
      ar->cap = cap_for(nmax, size_factor);
      slots(ar->a, nmax, ar->cap, true);
      slots(ar->b, nmax, ar->cap, true);
      ar->chunk_comp.resize(nr);
      for (int r = 0; r < nr; ++r) ok = ok && make_compressor(c, &ar->chunk_comp[r]);
      if (ar->consistent || (flags & CX_AR_OWNER_RESIDUAL)) {
        ar->owner_rests = reinterpret_cast<float*>(c->local_alloc(nmax * 4));
        ok = ok && ar->owner_rests;
      }
      break;
    }
    case CX_AR_COMPREX_ALLTOONE:
      ar->consistent = false;
      ar->subsamples = 1000; ar->sample_factor = 10.f;   // default sampling (src/allreduce.tpp:142)
      ar->cap = cap_for(size, size_factor);
      slots(ar->a, size, ar->cap, true);
      one(ar->bc, size, ar->cap, true);
      break;
  }
  if (!ok) {
    cx_set_error("cx_allreduce_create: out of heap or device memory", 0);
    delete ar;
    return nullptr;
  }
  return ar;
}

int cx_allreduce_apply(CxAllreduce* ar, void* data, void* stream) {
  switch (ar->kind) {
    case CX_AR_ALLTOONE: return alltoone_dense(ar, data, stream);
    case CX_AR_COMPREX_ALLTOONE: return alltoone_comprex(ar, data, false, stream);
    case CX_AR_RING: return ring_dense(ar, data, stream);
    case CX_AR_COMPREX_RING: return ring_comprex(ar, data, false, stream);
    case CX_AR_BIGRING: return bigring_dense(ar, data, stream);
    default: return bigring_comprex(ar, data, false, stream);
  }
}

int cx_allreduce_reset(CxAllreduce* ar) {
  if (!is_comprex(ar->kind)) return 0;
  int rc = cx_fill_zero(ar->c->dev, ar->rests, ar->size * 4, nullptr);
  if (!rc && ar->owner_rests) {
    int64_t nmax = 1;
    for (int64_t s : ar->seg_size) nmax = std::max(nmax, s);
    rc = cx_fill_zero(ar->c->dev, ar->owner_rests, nmax * 4, nullptr);
  }
  return rc;
}

int cx_allreduce_flush(CxAllreduce* ar, void* data, void* stream) {
  int rc;
  switch (ar->kind) {
    case CX_AR_COMPREX_ALLTOONE: rc = alltoone_comprex(ar, data, true, stream); break;
    case CX_AR_COMPREX_RING: rc = ring_comprex(ar, data, true, stream); break;
    case CX_AR_COMPREX_BIGRING: return bigring_comprex(ar, data, true, stream);
    default: return 0;
  }
  if (rc) return rc;
  if ((rc = cx_comm_sync(ar->c, stream))) return rc;
  return cx_allreduce_reset(ar);     // the reference resets after these two flushes (src/allreduce.tpp:236,506)
}

int cx_allreduce_set_ratio(CxAllreduce* ar, float ratio) {
  ar->ratio = ratio;
  return 0;
}

void cx_allreduce_set_scale(CxAllreduce* ar, float scale) { ar->result_scale = scale; }

int64_t cx_allreduce_size(const CxAllreduce* ar) { return ar->size; }

int cx_allreduce_state(CxAllreduce* ar, float* residual_out, int64_t n, uint64_t* step) {
  if (step) *step = ar->step;
  if (!residual_out) return 0;
  if (!is_comprex(ar->kind) || n != ar->size) return cx_set_error("cx_allreduce_state: no residual of that size", 0);
  if (ar->c->dev != CX_DEV_CUDA) { memcpy(residual_out, ar->rests, (size_t)n * 4); return 0; }
  int rc = cx_cuda_memcpy(residual_out, ar->rests, n * 4, 2, nullptr);
  return rc ? rc : cx_cuda_stream_sync(nullptr);
}

int cx_allreduce_load_state(CxAllreduce* ar, const float* residual, int64_t n, uint64_t step) {
  ar->step = step;
  if (!residual) return 0;
  if (!is_comprex(ar->kind) || n != ar->size) return cx_set_error("cx_allreduce_load_state: no residual of that size", 0);
  if (ar->c->dev != CX_DEV_CUDA) { memcpy(ar->rests, residual, (size_t)n * 4); return 0; }
  int rc = cx_cuda_memcpy(ar->rests, residual, n * 4, 1, nullptr);
  return rc ? rc : cx_cuda_stream_sync(nullptr);
}

int cx_allreduce_stats(CxAllreduce* ar, CxStats* out) {
  if (!is_comprex(ar->kind)) return cx_set_error("cx_allreduce_stats: not a compressed allreduce", 0);
  if (ar->c->dev != CX_DEV_CUDA) { *out = *ar->comp.stats; return 0; }
  int rc = cx_cuda_memcpy(out, ar->comp.stats, sizeof(CxStats), 2, nullptr);
  return rc ? rc : cx_cuda_stream_sync(nullptr);
}

void cx_allreduce_destroy(CxAllreduce* ar) { delete ar; }   // its memory belongs to the communicator

// ---- the reference's C names (src/GPI_C.cpp:44-73, src/allreduce_C.cpp:12-122) --------------------
// GaspiEnvironment_new joins the job named by CX_JOB (default "default") as rank CX_RANK / RANK of
// CX_RANKS / WORLD_SIZE; CX_DEVICE picks the GPU (default: rank), CX_HOST=1 keeps everything in
// host memory.  data_t is float and `data` lives where the environment lives.
static void complain(int rc, const char* what) {
  if (rc) fprintf(stderr, "comprex_b200: %s failed: %s\n", what, cx_last_error());
}
static int env_int(const char* a, const char* b, int dflt) {
  const char* e = getenv(a);
  if (!e && b) e = getenv(b);
  return e ? atoi(e) : dflt;
}

CxComm* GaspiEnvironment_new(int segment_size) {
  const char* job = getenv("CX_JOB");
  const int rank = env_int("CX_RANK", "RANK", 0), ranks = env_int("CX_RANKS", "WORLD_SIZE", 1);
  const bool host = env_int("CX_HOST", nullptr, 0) != 0 || cx_cuda_device_count() == 0;
  const int ndev = host ? 1 : cx_cuda_device_count();
  CxComm* c = cx_comm_bootstrap(job ? job : "default", rank, ranks, host ? CX_DEV_HOST : CX_DEV_CUDA,
                                env_int("CX_DEVICE", nullptr, rank % ndev), segment_size,
                                (uint64_t)env_int("COMPREX_TIMEOUT_MS", nullptr, 20000) * 1000000ull);
  if (!c) complain(-1, "GaspiEnvironment_new");
  return c;
}
void GaspiEnvironment_del(CxComm* self) { cx_comm_destroy(self); }
int GaspiEnvironment_get_rank(CxComm* self) { return self->rank; }
int GaspiEnvironment_get_ranks(CxComm* self) { return self->ranks; }
void GaspiEnvironment_barrier(CxComm* self) {
  complain(cx_comm_sync(self, nullptr), "GaspiEnvironment_barrier");
  complain(cx_comm_barrier(self), "GaspiEnvironment_barrier");
}
void GaspiEnvironment_flush(CxComm* self) { complain(cx_comm_sync(self, nullptr), "GaspiEnvironment_flush"); }
void Gaspi_Printf(const char* msg) { fputs(msg, stdout); fflush(stdout); }

struct CxRefAllreduce {      // a reference-style object: created first, connected later
  CxComm* c;
  int kind;
  CxAllreduce* ar;
};
static CxRefAllreduce* ref_new(CxComm* c, int kind) { return new CxRefAllreduce{c, kind, nullptr}; }
static void ref_del(CxRefAllreduce* s) { if (s) { cx_allreduce_destroy(s->ar); delete s; } }
static void ref_setup(CxRefAllreduce* s, int size, int chief, float ratio, float size_factor) {
  s->ar = cx_allreduce_create(s->c, s->kind, size, CX_F32, ratio, size_factor, chief, 0);
  complain(s->ar ? 0 : -1, "setupConnections");
}
static void ref_apply(CxRefAllreduce* s, float* data, int size) {
  if (!s->ar || size != s->ar->size) { complain(cx_set_error("apply: size does not match setupConnections", 0), "apply"); return; }
  int rc = cx_allreduce_apply(s->ar, data, nullptr);
  if (!rc) rc = cx_comm_sync(s->c, nullptr);        // the reference's apply returns with the result in place
  complain(rc, "apply");
  if (const uint32_t st = cx_comm_check(s->c)) fprintf(stderr, "comprex_b200: apply left status bits 0x%x\n", st);
}
static void ref_flush(CxRefAllreduce* s, float* data, int size) {
  if (!s->ar || size != s->ar->size) { complain(cx_set_error("flush: size does not match setupConnections", 0), "flush"); return; }
  int rc = cx_allreduce_flush(s->ar, data, nullptr);
  if (!rc) rc = cx_comm_sync(s->c, nullptr);
  complain(rc, "flush");
  if (const uint32_t st = cx_comm_check(s->c)) fprintf(stderr, "comprex_b200: flush left status bits 0x%x\n", st);
}

#define CX_REF_DENSE(Name, KIND)                                                                      \
  CxRefAllreduce* Name##_new(CxComm* env) { return ref_new(env, KIND); }                              \
  void Name##_del(CxRefAllreduce* self) { ref_del(self); }                                            \
  void Name##_apply(CxRefAllreduce* self, float* data, int size) { ref_apply(self, data, size); }
#define CX_REF_COMPREX(Name, KIND)                                                                    \
  CX_REF_DENSE(Name, KIND)                                                                            \
  void Name##_flush(CxRefAllreduce* self, float* data, int size) { ref_flush(self, data, size); }     \
  void Name##_reset(CxRefAllreduce* self) { if (self->ar) complain(cx_allreduce_reset(self->ar), #Name "_reset"); } \
  void Name##_set_compression_ratio(CxRefAllreduce* self, float r) { if (self->ar) cx_allreduce_set_ratio(self->ar, r); }

CX_REF_DENSE(AllToOneAllreduce, CX_AR_ALLTOONE)
void AllToOneAllreduce_setupConnections(CxRefAllreduce* self, int size, int tag, int chiefRank) { (void)tag; ref_setup(self, size, chiefRank, 1.f, 1.f); }
CX_REF_COMPREX(Comprex_AllToOneAllreduce, CX_AR_COMPREX_ALLTOONE)
void Comprex_AllToOneAllreduce_setupConnections(CxRefAllreduce* self, int size, int tag, int chiefRank, float compression_ratio, float size_factor) { (void)tag; ref_setup(self, size, chiefRank, compression_ratio, size_factor); }
CX_REF_DENSE(RingAllreduce, CX_AR_RING)
void RingAllreduce_setupConnections(CxRefAllreduce* self, int size, int tag) { (void)tag; ref_setup(self, size, 0, 1.f, 1.f); }
CX_REF_COMPREX(Comprex_RingAllreduce, CX_AR_COMPREX_RING)
void Comprex_RingAllreduce_setupConnections(CxRefAllreduce* self, int size, int tag, float compression_ratio, float size_factor) { (void)tag; ref_setup(self, size, 0, compression_ratio, size_factor); }
CX_REF_DENSE(BigRingAllreduce, CX_AR_BIGRING)
void BigRingAllreduce_setupConnections(CxRefAllreduce* self, int size, int tag) { (void)tag; ref_setup(self, size, 0, 1.f, 1.f); }
CX_REF_COMPREX(Comprex_BigRingAllreduce, CX_AR_COMPREX_BIGRING)
void Comprex_BigRingAllreduce_setupConnections(CxRefAllreduce* self, int size, int tag, float compression_ratio, float size_factor) { (void)tag; ref_setup(self, size, 0, compression_ratio, size_factor); }

}  // extern "C"
