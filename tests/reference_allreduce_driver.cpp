// Runs the reference's own compressed allreduce classes (include/allreduce.hxx, src/*.tpp,
// compiled unmodified against the GaspiCxx stand-in of baseline/gaspicxx_shim) on float vectors
// read from files, and writes the vector after every call.  Used by
// tests/test_reference_allreduce_parity.py when COMPREX_REFERENCE names the reference's tree.
//   argv: variant(bigring|ring|alltoone|dense_bigring|dense_ring|dense_alltoone) n ratio size_factor runs
//         in_prefix out_prefix
// Input of rank r for call k: <in_prefix>_r<r>_k<k>.bin (n floats); output likewise.  For the
// compressed variants one more vector (k = runs) goes through flush().
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include <allreduce.hxx>
#include <allreduce.tpp>
#include <gaspiEnvironment.hxx>
#include <gaspiEnvironment.tpp>

static std::vector<float> read_vec(const std::string& path, int n) {
  std::vector<float> v(n);
  FILE* f = fopen(path.c_str(), "rb");
  if (!f || fread(v.data(), 4, n, f) != (size_t)n) { fprintf(stderr, "cannot read %s\n", path.c_str()); exit(3); }
  fclose(f);
  return v;
}

static void write_vec(const std::string& path, const std::vector<float>& v) {
  FILE* f = fopen(path.c_str(), "wb");
  fwrite(v.data(), 4, v.size(), f);
  fclose(f);
}

int main(int argc, char** argv) {
  if (argc != 8) return 2;
  const std::string variant = argv[1];
  const int n = atoi(argv[2]);
  const float ratio = atof(argv[3]), size_factor = atof(argv[4]);
  const int runs = atoi(argv[5]);
  const std::string in = argv[6], out = argv[7];
  GaspiEnvironment env(static_cast<size_t>(1) << 28);
  const int me = env.get_rank();
  Allreduce_base<float>* ar = nullptr;
  if (variant == "bigring") {
    auto* a = new Comprex_BigRingAllreduce<float>(&env);
    a->setupConnections(n, 1, ratio, size_factor);
    ar = a;
  } else if (variant == "ring") {
    auto* a = new Comprex_RingAllreduce<float>(&env);
    a->setupConnections(n, 1, ratio, size_factor);
    ar = a;
  } else if (variant == "alltoone") {
    auto* a = new Comprex_AllToOneAllreduce<float>(&env);
    a->setupConnections(n, 1, 0, ratio, size_factor);
    ar = a;
  } else if (variant == "dense_bigring") {
    auto* a = new BigRingAllreduce<float>(&env);
    a->setupConnections(n, 1);
    ar = a;
  } else if (variant == "dense_ring") {
    auto* a = new RingAllreduce<float>(&env);
    a->setupConnections(n, 1);
    ar = a;
  } else {
    auto* a = new AllToOneAllreduce<float>(&env);
    a->setupConnections(n, 1, 0);
    ar = a;
  }
  for (int k = 0; k < runs; ++k) {
    const std::string tag = "_r" + std::to_string(me) + "_k" + std::to_string(k) + ".bin";
    std::vector<float> v = read_vec(in + tag, n);
    env.barrier();
    ar->apply(v.data(), n);
    write_vec(out + tag, v);
  }
  {
    const std::string tag = "_r" + std::to_string(me) + "_k" + std::to_string(runs) + ".bin";
    if (variant == "bigring" || variant == "ring" || variant == "alltoone") {
      std::vector<float> v = read_vec(in + tag, n);
      env.barrier();
      if (variant == "bigring") dynamic_cast<Comprex_BigRingAllreduce<float>*>(ar)->flush(v.data(), n);
      else if (variant == "ring") dynamic_cast<Comprex_RingAllreduce<float>*>(ar)->flush(v.data(), n);
      else dynamic_cast<Comprex_AllToOneAllreduce<float>*>(ar)->flush(v.data(), n);
      write_vec(out + tag, v);
    }
  }
  env.barrier();
  delete ar;
  return 0;
}
