// Compiled and run by tests/test_cpp_facade.py: includes the C++ face of the library with a plain
// host compiler, links the shared object and exercises the argument checks that need no GPU.
#include <cstdio>
#include <cstring>

#include "flashmoe/flashmoe.cuh"   // the include path of the reference

int main() {
  using namespace flashmoe;
  int fails = 0;
  const int emap[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int rmap[1] = {0};
  auto expect_throw = [&](const char* what, const char* needle, auto fn) {
    try {
      fn();
      std::printf("FAIL %s: no exception\n", what);
      ++fails;
    } catch (const std::runtime_error& e) {
      if (std::strstr(e.what(), needle) == nullptr) {
        std::printf("FAIL %s: message '%s' lacks '%s'\n", what, e.what(), needle);
        ++fails;
      }
    }
  };
  LayerDesc layer;
  layer.topK = 2;
  {
    MoEArgs a(2, 128, 256, 256, 128, 128, 128, 128, 64, 64, 128, 148, 0, 0, 1, 0, 8, 8, Topology::NVLINK_ONLY);
    expect_throw("arch", "sm_100a", [&] { initialize(a, layer, 900, emap, rmap, nullptr); });
    expect_throw("gate arch", "sm_100a", [&] { initializeGate(a, layer, 900, false, nullptr); });
  }
  {
    MoEArgs a(2, 128, 100, 256, 128, 128, 128, 128, 64, 64, 128, 148, 0, 0, 1, 0, 8, 8, Topology::NVLINK_ONLY);
    expect_throw("tokenDim", "token dimension", [&] { initialize(a, layer, 1000, emap, rmap, nullptr); });
  }
  {
    MoEArgs a(3, 128, 256, 256, 128, 128, 128, 128, 64, 64, 128, 148, 0, 0, 1, 0, 8, 8, Topology::NVLINK_ONLY);
    expect_throw("elementBytes", "elementBytes", [&] { initialize(a, layer, 1000, emap, rmap, nullptr); });
  }
  {
    MoEArgs a(2, 128, 256, 256, 128, 128, 128, 128, 64, 64, 128, 148, 0, 0, 1, 0, 8, 8, Topology::MIXED);
    expect_throw("topology", "NVLINK_ONLY", [&] { initialize(a, layer, 1000, emap, rmap, nullptr); });
  }
  {
    // getWorkspaceBytes needs no device: 128 tokens, H = I = 256, 8 experts on one rank, k = 2, BF16.
    // It must at least hold the landing rows, the GEMM0 output and the return rows.
    MoEArgs a(2, 128, 256, 256, 128, 128, 128, 128, 64, 64, 128, 148, 0, 0, 1, 0, 8, 8, Topology::NVLINK_ONLY);
    const size_t bytes = getWorkspaceBytes(a, layer);
    const size_t floor = static_cast<size_t>(128) * 2 * 256 * 2 * 3;
    if (bytes < floor || bytes > 64u * 1024 * 1024) {
      std::printf("FAIL getWorkspaceBytes: %zu\n", bytes);
      ++fails;
    }
    MoEArgs bad(2, 128, 100, 256, 128, 128, 128, 128, 64, 64, 128, 148, 0, 0, 1, 0, 8, 8, Topology::NVLINK_ONLY);
    expect_throw("getWorkspaceBytes tokenDim", "token dimension", [&] { getWorkspaceBytes(bad, layer); });
  }
  static_assert(sizeof(TPS) == 8, "routing-table entry is 8 bytes");
  std::printf(fails == 0 ? "FACADE_OK\n" : "FACADE_FAILED\n");
  return fails;
}
