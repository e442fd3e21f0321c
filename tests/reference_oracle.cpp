// Oracle built from the reference's own headers (included unmodified through -I): reads
// n, top-k, g[n], r[n], base[n] from a binary file, runs ThresholdTopK::prepare_with / get_threshold,
// CompressorIndexPairs::compress_add_update, ::add (into base) and ::decompress, and writes threshold,
// payload, the new residual, base after the scatter-add and the decompressed vector.
// Used by tests/test_reference_oracle.py when COMPREX_REFERENCE points at the reference's tree.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "compressor.hxx"

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  FILE* in = fopen(argv[1], "rb");
  if (!in) return 3;
  int n = 0;
  float ratio = 0.f;
  if (fread(&n, 4, 1, in) != 1 || fread(&ratio, 4, 1, in) != 1) return 4;
  std::vector<float> g(n), r(n), base(n), dec(n, 7.f);
  if (fread(g.data(), 4, n, in) != (size_t)n || fread(r.data(), 4, n, in) != (size_t)n ||
      fread(base.data(), 4, n, in) != (size_t)n) return 5;
  fclose(in);
  // mode (argv[3], default 0): 0 compress_add_update(r, g), 1 compress_update(r), 2 compress(g),
  // 3: ThresholdTopK::apply and ::apply_split of g only (writes out, high, low)
  const int mode = argc > 3 ? atoi(argv[3]) : 0;
  if (mode == 3) {
    ThresholdTopK<float> t(ratio);
    std::vector<float> o(n), hi(n), lo(n);
    t.apply(o.data(), n, g.data(), n);
    ThresholdTopK<float> t2(ratio);
    t2.apply_split(hi.data(), n, lo.data(), n, g.data(), n);
    FILE* out = fopen(argv[2], "wb");
    if (!out) return 6;
    fwrite(o.data(), 4, n, out);
    fwrite(hi.data(), 4, n, out);
    fwrite(lo.data(), 4, n, out);
    fclose(out);
    return 0;
  }
  ThresholdTopK<float> thr(ratio);
  if (mode == 0) thr.prepare_with(r.data(), n, g.data(), n);
  else if (mode == 1) thr.prepare(r.data(), n);
  else thr.prepare(g.data(), n);
  const float cut = thr.get_threshold();
  std::vector<char> buf((size_t)n * 8 + 64);
  CompressorIndexPairs<float> comp;
  int bytes;
  if (mode == 0) bytes = comp.compress_add_update(buf.data(), r.data(), n, g.data(), n, cut);
  else if (mode == 1) bytes = comp.compress_update(buf.data(), r.data(), n, cut);
  else bytes = comp.compress(buf.data(), g.data(), n, cut);
  comp.add(base.data(), n, buf.data());
  comp.decompress(dec.data(), n, buf.data());
  FILE* out = fopen(argv[2], "wb");
  if (!out) return 6;
  fwrite(&cut, 4, 1, out);
  fwrite(&bytes, 4, 1, out);
  fwrite(buf.data(), 1, bytes, out);
  fwrite(r.data(), 4, n, out);
  fwrite(base.data(), 4, n, out);
  fwrite(dec.data(), 4, n, out);
  fclose(out);
  return 0;
}
