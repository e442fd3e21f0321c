#pragma once
#include "../shim_core.hpp"
#include "Rank.hpp"

namespace gaspi {
namespace group {

class Group {   // the group of all ranks
 public:
  Rank rank() const { return Rank(shim::World::get().rank); }
  int size() const { return shim::World::get().size; }
};

}  // namespace group
}  // namespace gaspi
