// The reference's include path (csrc/include/flashmoe/flashmoe.cuh of hnts03-moreh/FlashMoE):
// code written against it finds the same names here.  Everything lives in flashmoe.hpp, which is
// host-only C++ over the C ABI and needs no CUDA compiler.
#pragma once
#include "flashmoe.hpp"
