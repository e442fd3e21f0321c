#pragma once
#include <functional>

#include "TargetBuffer.hpp"

namespace gaspi {
namespace singlesided {
namespace write {

class SourceBuffer {
 public:
  SourceBuffer(segment::Segment& seg, std::size_t bytes)
      : seg_(seg), bytes_(bytes), off_(seg.alloc(bytes)), owns_(true), local_(seg.base() + off_) {}
  // alias of memory that another SourceBuffer owns (one payload, several targets)
  SourceBuffer(void* address, segment::Segment& seg, std::size_t bytes)
      : seg_(seg), bytes_(bytes), off_(0), owns_(false), local_(static_cast<char*>(address)) {}
  ~SourceBuffer() { if (owns_) seg_.release(off_); }
  void* address() const { return local_; }

  ConnectHandle connectToRemoteTarget(const group::Group&, const group::Rank& target, int tag) {
    shim::World& w = shim::World::get();
    const int dst = target.get();
    entry_ = &w.entry(w.rank, dst, tag);
    const uint64_t want = w.next_use(true, w.rank, dst, tag);        // my k-th connection under this key
    return ConnectHandle{[this, dst, want]() {
      long spins = 0;
      while (entry_->generation.load(std::memory_order_acquire) < want)
        if (++spins % 1024 == 0) sched_yield();
      remote_ = shim::World::get().base(dst) + entry_->offset.load(std::memory_order_relaxed);
    }};
  }

  // one-sided write of [offset, offset + bytes) into the same range of the target, then notify
  void initTransferPart(Runtime&, std::size_t bytes, std::size_t offset) {
    std::memcpy(remote_, local_ + offset, bytes);
    entry_->notify.fetch_add(1, std::memory_order_release);
  }

 private:
  segment::Segment& seg_;
  std::size_t bytes_, off_;
  bool owns_;
  char* local_;
  char* remote_ = nullptr;
  shim::Entry* entry_ = nullptr;
};

}  // namespace write
}  // namespace singlesided
}  // namespace gaspi
