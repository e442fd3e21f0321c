#pragma once
#include "../shim_core.hpp"

namespace gaspi {
namespace segment {

class Segment {
 public:
  explicit Segment(std::size_t bytes) : bytes_(bytes) {
    base_ = shim::World::get().create_segment(bytes);
    arena_.init(bytes);
  }
  char* base() { return base_; }
  std::size_t alloc(std::size_t bytes) { return arena_.alloc(bytes); }
  void release(std::size_t off) { arena_.release(off); }

 private:
  std::size_t bytes_;
  char* base_;
  shim::Arena arena_;
};

}  // namespace segment
}  // namespace gaspi
