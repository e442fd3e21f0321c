#pragma once
#include <functional>

#include "../../Runtime.hpp"
#include "../../group/Group.hpp"
#include "../../segment/Segment.hpp"

namespace gaspi {
namespace singlesided {

struct ConnectHandle {           // connect...(...).waitForCompletion()
  std::function<void()> finish;
  void waitForCompletion() { if (finish) finish(); }
};

namespace write {

class TargetBuffer {
 public:
  TargetBuffer(segment::Segment& seg, std::size_t bytes) : seg_(seg), bytes_(bytes), off_(seg.alloc(bytes)) {}
  ~TargetBuffer() { seg_.release(off_); }
  void* address() const { return seg_.base() + off_; }

  ConnectHandle connectToRemoteSource(const group::Group&, const group::Rank& src, int tag) {
    shim::World& w = shim::World::get();
    entry_ = &w.entry(src.get(), w.rank, tag);
    w.next_use(false, src.get(), w.rank, tag);
    consumed_ = entry_->notify.load(std::memory_order_acquire);
    entry_->offset.store(off_, std::memory_order_relaxed);
    entry_->generation.fetch_add(1, std::memory_order_release);     // the source may resolve us now
    return ConnectHandle{};
  }

  void waitForCompletion() {       // blocks until the next transfer into this buffer has landed
    long spins = 0;
    while (entry_->notify.load(std::memory_order_acquire) <= consumed_)
      if (++spins % 4096 == 0) sched_yield();
    ++consumed_;
  }

 private:
  segment::Segment& seg_;
  std::size_t bytes_, off_;
  shim::Entry* entry_ = nullptr;
  uint64_t consumed_ = 0;
};

}  // namespace write
}  // namespace singlesided
}  // namespace gaspi
