// A minimal stand-in for the part of the GaspiCxx API that the ComprEx reference uses, over
// POSIX shared memory and atomics, so that the reference's exchange and allreduce code can be
// compiled UNMODIFIED and run as P processes on one host ("reference algorithms on a shim
// transport": the algorithms and the compression are the reference's, the one-sided
// write + notify of GPI-2 is a memcpy into the peer's mapped segment plus an atomic counter).
//
// Environment of every rank (set by baseline/run_reference_on_shim.py): CXSHIM_RANK,
// CXSHIM_SIZE, CXSHIM_JOB.  The control block /cxshim_<job>_ctl is created (zero-filled) by the
// launcher; every rank creates its segment /cxshim_<job>_seg<rank> and maps its peers' on demand.
#pragma once
#include <fcntl.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace gaspi {
namespace shim {

constexpr int kMaxRanks = 64;
constexpr int kEntries = 1 << 14;

struct Entry {                       // one per (source rank, target rank, tag)
  std::atomic<uint64_t> key;         // 0 = free
  std::atomic<uint64_t> generation;  // registrations of a target buffer under this key
  std::atomic<uint64_t> offset;      // of the target buffer in the target rank's segment
  std::atomic<uint64_t> notify;      // transfers completed, ever
};

struct Control {
  std::atomic<int> barrier_count;
  std::atomic<int> barrier_sense;
  std::atomic<uint64_t> segment_bytes[kMaxRanks];   // 0 until the rank's segment exists
  Entry entries[kEntries];
};

inline int env_int(const char* name) {
  const char* v = getenv(name);
  if (!v) throw std::runtime_error(std::string("shim: environment variable missing: ") + name);
  return atoi(v);
}

inline void* map_shared(const std::string& name, size_t bytes, bool create) {
  int fd = -1;
  for (long spin = 0; spin < 600000; ++spin) {       // peers may not have created it yet (<= ~60 s)
    fd = shm_open(name.c_str(), create ? (O_CREAT | O_RDWR) : O_RDWR, 0600);
    if (fd >= 0 || create) break;
    usleep(100);
  }
  if (fd < 0) throw std::runtime_error("shim: cannot open " + name);
  if (create && ftruncate(fd, (off_t)bytes) != 0) throw std::runtime_error("shim: ftruncate " + name);
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) throw std::runtime_error("shim: mmap " + name);
  return p;
}

class World {
 public:
  static World& get() {
    static World w;
    return w;
  }
  int rank, size;
  std::string job;
  Control* ctl;

  void barrier() {
    const int sense = 1 - local_sense_;
    local_sense_ = sense;
    if (ctl->barrier_count.fetch_add(1, std::memory_order_acq_rel) == size - 1) {
      ctl->barrier_count.store(0, std::memory_order_relaxed);
      ctl->barrier_sense.store(sense, std::memory_order_release);
    } else {
      long spins = 0;
      while (ctl->barrier_sense.load(std::memory_order_acquire) != sense)
        if (++spins % 1024 == 0) sched_yield();
    }
  }

  std::string segment_name(int r) const { return "/cxshim_" + job + "_seg" + std::to_string(r); }

  // my own segment (one per process, like the reference's GaspiEnvironment)
  char* create_segment(size_t bytes) {
    if (bases_[rank]) throw std::runtime_error("shim: one segment per rank");
    bases_[rank] = static_cast<char*>(map_shared(segment_name(rank), bytes, true));
    ctl->segment_bytes[rank].store(bytes, std::memory_order_release);
    return bases_[rank];
  }
  char* base(int r) {
    if (!bases_[r]) {
      uint64_t bytes = 0;
      long spins = 0;
      while ((bytes = ctl->segment_bytes[r].load(std::memory_order_acquire)) == 0)
        if (++spins % 1024 == 0) sched_yield();
      bases_[r] = static_cast<char*>(map_shared(segment_name(r), bytes, false));
    }
    return bases_[r];
  }

  Entry& entry(int src, int dst, int tag) {
    const uint64_t key = (1ull << 63) | ((uint64_t)(uint32_t)tag << 16) | ((uint64_t)src << 8) | (uint64_t)dst;
    uint64_t h = key * 0x9E3779B97F4A7C15ull;
    for (int probe = 0; probe < kEntries; ++probe) {
      Entry& e = ctl->entries[(h >> 20) + probe & (kEntries - 1)];
      uint64_t cur = e.key.load(std::memory_order_acquire);
      if (cur == key) return e;
      if (cur == 0) {
        if (e.key.compare_exchange_strong(cur, key, std::memory_order_acq_rel)) return e;
        if (cur == key) return e;
      }
    }
    throw std::runtime_error("shim: connection table full");
  }

  // how many times this rank connected (as source / as target) under a key
  uint64_t next_use(bool as_source, int src, int dst, int tag) {
    return ++uses_[{as_source, ((uint64_t)(uint32_t)tag << 16) | ((uint64_t)src << 8) | (uint64_t)dst}];
  }

 private:
  World() : bases_(kMaxRanks, nullptr) {
    rank = env_int("CXSHIM_RANK");
    size = env_int("CXSHIM_SIZE");
    job = getenv("CXSHIM_JOB") ? getenv("CXSHIM_JOB") : "job";
    if (size < 1 || size > kMaxRanks || rank < 0 || rank >= size) throw std::runtime_error("shim: bad rank/size");
    ctl = static_cast<Control*>(map_shared("/cxshim_" + job + "_ctl", sizeof(Control), false));
  }
  int local_sense_ = 0;
  std::vector<char*> bases_;
  std::map<std::pair<bool, uint64_t>, uint64_t> uses_;
};

// first-fit allocator over the local segment (metadata stays in the process)
class Arena {
 public:
  void init(size_t bytes) { free_[0] = bytes; }
  size_t alloc(size_t bytes) {
    bytes = (bytes + 255) / 256 * 256;
    for (auto it = free_.begin(); it != free_.end(); ++it) {
      if (it->second >= bytes) {
        const size_t off = it->first, rest = it->second - bytes;
        free_.erase(it);
        if (rest) free_[off + bytes] = rest;
        used_[off] = bytes;
        return off;
      }
    }
    throw std::runtime_error("shim: segment exhausted");
  }
  void release(size_t off) {
    auto u = used_.find(off);
    if (u == used_.end()) return;
    size_t bytes = u->second;
    used_.erase(u);
    auto next = free_.find(off + bytes);
    if (next != free_.end()) { bytes += next->second; free_.erase(next); }
    auto it = free_.lower_bound(off);
    if (it != free_.begin()) {
      auto prev = std::prev(it);
      if (prev->first + prev->second == off) { prev->second += bytes; return; }
    }
    free_[off] = bytes;
  }

 private:
  std::map<size_t, size_t> free_, used_;
};

}  // namespace shim
}  // namespace gaspi
