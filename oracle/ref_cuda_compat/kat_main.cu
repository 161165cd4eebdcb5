// Runs the reference's known-answer tests registered through the gtest stand-in:
//   ref_kats [substring]      runs the tests whose "Suite.Name" contains the substring
// Exit code 0 = all passed.  Checker only; never part of the product.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

#include "gtest/gtest.h"

int main(int argc, char **argv) {
  const char *filter = argc > 1 ? argv[1] : "";
  int ran = 0, failed = 0;
  for (const kat::Case &c : kat::cases()) {
    const std::string full = std::string(c.suite) + "." + c.name;
    if (full.find(filter) == std::string::npos) continue;
    const int before = kat::failures();
    std::printf("[ RUN  ] %s\n", full.c_str());
    std::fflush(stdout);
    c.fn();
    const cudaError_t e = cudaDeviceSynchronize();
    const bool ok = kat::failures() == before && e == cudaSuccess;
    if (e != cudaSuccess) std::printf("         CUDA error after the test: %s\n", cudaGetErrorString(e));
    std::printf("[ %s ] %s\n", ok ? " OK " : "FAIL", full.c_str());
    std::fflush(stdout);
    ++ran;
    if (!ok) {
      ++failed;
      if (e != cudaSuccess) break;  // the context is gone: stop here
    }
  }
  std::printf("%d tests ran, %d failed\n", ran, failed);
  return failed == 0 && ran > 0 ? 0 : 1;
}
