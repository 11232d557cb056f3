// The router's arithmetic that must be the same, operation for operation, wherever it runs (the
// stand-alone router kernels and the routing phase inside the persistent kernel): the exponential,
// the lane fold, and softmax + top-k over one token's row of logits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace fmoe {

// 2^f on [-0.5, 0.5]: (ln 2)^k / k!, k = 0..7, rounded to fp32.
__device__ __forceinline__ float det_exp(float x) {
  float t = __fmul_rn(x, 0x1.715476p+0f);
  t = fmaxf(t, -100.0f);
  const float n = rintf(t);
  const float f = __fsub_rn(t, n);
  float p = 0x1.ffcbfcp-17f;
  p = __fadd_rn(__fmul_rn(p, f), 0x1.430912p-13f);
  p = __fadd_rn(__fmul_rn(p, f), 0x1.5d87fep-10f);
  p = __fadd_rn(__fmul_rn(p, f), 0x1.3b2ab6p-7f);
  p = __fadd_rn(__fmul_rn(p, f), 0x1.c6b08ep-5f);
  p = __fadd_rn(__fmul_rn(p, f), 0x1.ebfbep-3f);
  p = __fadd_rn(__fmul_rn(p, f), 0x1.62e43p-1f);
  p = __fadd_rn(__fmul_rn(p, f), 1.0f);
  const float scale = __int_as_float((static_cast<int>(n) + 127) << 23);
  return __fmul_rn(p, scale);
}

__device__ __forceinline__ float butterfly_sum(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

template <typename T>
struct Vec8;  // loads 8 consecutive elements as fp32

template <>
struct Vec8<__nv_bfloat16> {
  static constexpr bool kExactProducts = true;
  static constexpr bool kIsBf16 = true;
  __device__ __forceinline__ static void load(const void* p, float (&f)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <>
struct Vec8<__half> {
  static constexpr bool kExactProducts = true;
  static constexpr bool kIsBf16 = false;
  __device__ __forceinline__ static void load(const void* p, float (&f)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
};
template <>
struct Vec8<float> {
  static constexpr bool kExactProducts = false;
  static constexpr bool kIsBf16 = false;
  __device__ __forceinline__ static void load(const void* p, float (&f)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};

// Softmax over all experts, k rounds of arg-max, combine weights: one warp, one token; `r` is the
// token's row of logits in shared memory (it ends up holding the probabilities, the selected ones
// overwritten).  Lane j < k leaves with the token's j-th choice in (idx, weight).
__device__ __forceinline__ void softmax_topk_row(int E, int k, float* routing, float* r, int tok, int lane,
                                                 int& idx, float& weight) {
  float m = -INFINITY;
  for (int j = lane; j < E; j += 32) m = fmaxf(m, r[j]);
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  float d = 0.0f;
  for (int j = lane; j < E; j += 32) {
    const float ex = det_exp(__fsub_rn(r[j], m));
    r[j] = ex;
    d = __fadd_rn(d, ex);
  }
  d = butterfly_sum(d);
  for (int j = lane; j < E; j += 32) {
    const float pr = __fdiv_rn(r[j], d);
    r[j] = pr;
    if (routing) routing[static_cast<size_t>(tok) * E + j] = pr;
  }
  float wsum = 0.0f, my_p = 0.0f;
  int my_idx = 0;
  for (int round = 0; round < k; ++round) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int j = lane; j < E; j += 32) {
      const float v = r[j];
      if (v > bv) { bv = v; bi = j; }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;  // nothing left to pick (all NaN)
    if (lane == (bi & 31)) r[bi] = -INFINITY;
    wsum = __fadd_rn(wsum, bv);
    if (lane == (round & 31)) { my_p = bv; my_idx = bi; }
    __syncwarp();
  }
  idx = my_idx;
  weight = __fdiv_rn(my_p, wsum);
  __syncwarp();
}
__device__ __forceinline__ void softmax_topk_row(const RouterParams& p, float* r, int tok, int lane) {
  int idx;
  float weight;
  softmax_topk_row(p.E, p.k, p.routing, r, tok, lane, idx, weight);
  if (lane < p.k) {
    p.topk_idx[static_cast<size_t>(tok) * p.k + lane] = idx;
    p.topk_w[static_cast<size_t>(tok) * p.k + lane] = weight;
  }
}

}  // namespace fmoe
