#pragma once
namespace gaspi {
namespace group {

class Rank {
 public:
  Rank() : r_(0) {}
  explicit Rank(int r) : r_(r) {}
  int get() const { return r_; }
  bool operator==(const Rank& o) const { return r_ == o.r_; }
  bool operator!=(const Rank& o) const { return r_ != o.r_; }

 private:
  int r_;
};

}  // namespace group
}  // namespace gaspi
