// Times the reference's own header-only compression code (ThresholdTopK::prepare_with,
// CompressorIndexPairs::compress_add_update and ::add from its src/threshold.hxx and
// src/compressor.hxx, included unmodified through -I) on one CPU core, for the vector sizes
// and top-k ratios of the GPU kernel table.  Built and run by bench/reference_cpu.py.
// Output: one JSON object per line.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "compressor.hxx"

static double now_us() {
  using namespace std::chrono;
  return duration_cast<duration<double, std::micro>>(steady_clock::now().time_since_epoch()).count();
}

static double median(std::vector<double> v) {
  std::sort(v.begin(), v.end());
  return v[v.size() / 2];
}

int main(int argc, char** argv) {
  const int reps = argc > 1 ? atoi(argv[1]) : 5;
  const long sizes[] = {1L << 16, 1L << 20, 1L << 24, 1L << 26};
  const float ratios[] = {0.001f, 0.01f, 0.1f};
  for (long n : sizes) {
    std::mt19937 gen(1234);
    std::normal_distribution<float> dist(0.f, 1.f);
    std::vector<float> g(n), r0(n), r(n), out(n);
    for (long i = 0; i < n; ++i) { g[i] = dist(gen); r0[i] = 0.5f * dist(gen); }
    std::vector<char> buffer((size_t)n * 8 + 64);
    for (float ratio : ratios) {
      std::vector<double> t_thr, t_comp, t_add;
      long nnz = 0;
      for (int rep = 0; rep < reps; ++rep) {
        r = r0;
        std::fill(out.begin(), out.end(), 0.f);
        ThresholdTopK<float> thr(ratio);
        CompressorIndexPairs<float> comp;
        double t0 = now_us();
        thr.prepare_with(r.data(), (int)n, g.data(), (int)n);
        const float cut = thr.get_threshold();
        double t1 = now_us();
        comp.compress_add_update(buffer.data(), r.data(), (int)n, g.data(), (int)n, cut);
        double t2 = now_us();
        comp.add(out.data(), (int)n, buffer.data());
        double t3 = now_us();
        t_thr.push_back(t1 - t0); t_comp.push_back(t2 - t1); t_add.push_back(t3 - t2);
        nnz = reinterpret_cast<int*>(buffer.data())[1];
      }
      printf("{\"n\": %ld, \"ratio\": %g, \"nnz\": %ld, \"threshold_us\": %.1f, \"compress_add_update_us\": %.1f, "
             "\"add_us\": %.1f}\n", n, ratio, nnz, median(t_thr), median(t_comp), median(t_add));
      fflush(stdout);
    }
  }
  return 0;
}
