// Host-side dump of the CUTLASS numeric conversions the reference quantiser
// relies on (cutlass::float_e4m3_t(float), cutlass::float_e2m1_t(float);
// integrations/vllm/native/runtime.cu:76,79 of the reference).  Reads fp32
// values from stdin (binary), writes one code byte per value to stdout.
// Compiled and run only by make_golden.py; not part of the product.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>
#include "cutlass/float8.h"
#include "cutlass/float_subbyte.h"

int main(int argc, char** argv) {
  bool fp4 = argc > 1 && std::strcmp(argv[1], "e2m1") == 0;
  std::vector<float> in;
  float buf[4096];
  size_t n;
  while ((n = std::fread(buf, sizeof(float), 4096, stdin)) > 0) in.insert(in.end(), buf, buf + n);
  std::vector<uint8_t> out(in.size());
  for (size_t i = 0; i < in.size(); ++i)
    out[i] = fp4 ? uint8_t(cutlass::float_e2m1_t(in[i]).raw()) : uint8_t(cutlass::float_e4m3_t(in[i]).raw());
  std::fwrite(out.data(), 1, out.size(), stdout);
  return 0;
}
