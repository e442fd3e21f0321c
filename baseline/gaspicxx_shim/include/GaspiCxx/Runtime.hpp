#pragma once
#include "shim_core.hpp"

namespace gaspi {

class Runtime {
 public:
  void barrier() { shim::World::get().barrier(); }
  void flush() {}
  int global_rank() { return shim::World::get().rank; }
  int size() { return shim::World::get().size; }
};

inline void initGaspiCxx() { shim::World::get(); }
inline Runtime& getRuntime() {
  static Runtime rt;
  return rt;
}

}  // namespace gaspi
