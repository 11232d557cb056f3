// Router: logits = X * Wr^T, softmax over all experts, top-k, routing-table construction.
//
// Replaces the reference's fused gate kernel (csrc/include/flashmoe/gate.cuh:98-565) with two
// SIMT kernels whose fp32 arithmetic is fixed operation by operation, so that a CPU
// restatement performing the same operations in the same order reproduces expert ids,
// counts, slots AND probabilities bit for bit:
//
//  * dot product: H is cut into vectors of 8 elements; lane (v mod 32) consumes vector v;
//    a lane walks its vectors in ascending order and each vector in ascending element
//    order with acc = acc + x*w (one FMA for 16-bit inputs, whose products are exact in
//    fp32; a rounded multiply followed by a rounded add for fp32 inputs); the 32 lane
//    sums are folded with an xor-butterfly, offsets 16, 8, 4, 2, 1.
//  * softmax: p_j = det_exp(x_j - max) / d with IEEE division; d is summed with element j
//    on lane (j mod 32), ascending j per lane, then the same butterfly.
//  * top-k: k rounds of arg-max on the probabilities, larger value wins, equal values go
//    to the lower expert id (the reference's strict '>' ascending scan, gate.cuh:505-522);
//    combine weight = p / (sum of the selected p, added in selection order).
//  * slots: expert e's routing-table row lists the tokens that chose e in ascending token
//    order (a second kernel scans tokens in order; the reference orders by tile arrival).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "common.cuh"
#include "router_math.cuh"

namespace fmoe {

namespace {

// 8 consecutive elements as loaded (16 or 32 bytes), converted to fp32 only when they are used, so
// that a load issued several iterations ahead does not stall the warp where it is issued.
template <typename T>
struct Raw8 {
  static constexpr int kPieces = static_cast<int>(sizeof(T)) * 8 / 16;
  uint4 q[kPieces];
  __device__ __forceinline__ void fetch(const T* p) {
#pragma unroll
    for (int i = 0; i < kPieces; ++i) q[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
  }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        f[4 * i] = __uint_as_float(q[i].x); f[4 * i + 1] = __uint_as_float(q[i].y);
        f[4 * i + 2] = __uint_as_float(q[i].z); f[4 * i + 3] = __uint_as_float(q[i].w);
      }
    } else {
      const uint32_t w[4] = {q[0].x, q[0].y, q[0].z, q[0].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if constexpr (sizeof(T) == 2 && Vec8<T>::kIsBf16) {
          f[2 * i] = __uint_as_float(w[i] << 16);
          f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
          const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
          f[2 * i] = v.x;
          f[2 * i + 1] = v.y;
        }
      }
    }
  }
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T>
__device__ __forceinline__ void vec8_from_smem(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void vec8_from_smem<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void vec8_from_smem<__half>(const __half* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <>
__device__ __forceinline__ void vec8_from_smem<float>(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// One warp owns TT consecutive tokens; the CTA walks the experts in groups of EG and the H axis
// in chunks of 256 elements (one 8-element vector per lane).  The EG x 256 chunk of the router
// weight is staged in shared memory (cp.async, a ring of 2 or 4 chunks) and shared by all warps, so the
// weight matrix crosses L2 once per CTA instead of once per warp.
//
// The CTA's warps form TG token groups x ES expert parts: warp (tg, part) accumulates, for its TT
// tokens, the EG / ES experts of every group that fall in its part.  Splitting the experts over
// warps keeps the accumulators small (TT * EG / ES registers) and puts 4 * ES warps on the SM,
// which is what hides the FMA and shared-memory latencies when E is large.
template <typename T, int TT, int EG, int TG, int ES>
__global__ void __launch_bounds__(TG * ES * 32)
router_topk_kernel(const RouterParams p) {
  constexpr int WARPS = TG * ES;
  constexpr int EP = EG / ES;                        // experts of a group one warp accumulates
  static_assert(EG % ES == 0, "expert group must split evenly");
  extern __shared__ __align__(16) unsigned char s_raw[];
  float* s_row = reinterpret_cast<float*>(s_raw);  // [TG][TT][E]: logits, then exp, then probabilities
  const int H = p.H, E = p.E;
  T* wbuf = reinterpret_cast<T*>(s_raw + ((static_cast<size_t>(TG) * TT * E * sizeof(float) + 15) & ~size_t(15)));
  constexpr int kChunk = 256;                       // elements of H per step
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tg = warp % TG, part = warp / TG;
  const int t0 = (blockIdx.x * TG + tg) * TT;
  const int nvec = H >> 3;
  const int iters = (nvec + 31) >> 5;
  const T* __restrict__ X = static_cast<const T*>(p.tokens);
  const T* __restrict__ Wr = static_cast<const T*>(p.weights);
  float* rows = s_row + static_cast<size_t>(tg) * TT * E;

  // weight chunks in flight: with few experts a chunk's arithmetic is shorter than an L2 round trip
  constexpr bool kDeep = EG <= 16;
  constexpr int NSTG = kDeep ? 4 : 2;
  // chunk `it` of expert group `eg` -> ring slot it % NSTG; always commits a group (an empty one
  // past the end), so that "all but the newest NSTG - 1 groups have landed" means chunk it is in
  auto stage = [&](int eg, int it) {
    const int buf = it % NSTG;
    const int v = it * 32 + lane;
    if (it < iters && v < nvec) {
#pragma unroll
      for (int e = warp; e < EG; e += WARPS) {
        T* dst = wbuf + (static_cast<size_t>(buf) * EG + e) * kChunk + lane * 8;
        const T* src = Wr + static_cast<size_t>(eg + e) * H + v * 8;
#pragma unroll
        for (int piece = 0; piece < static_cast<int>(sizeof(T)) * 8 / 16; ++piece)
          cp_async16(reinterpret_cast<unsigned char*>(dst) + 16 * piece,
                     reinterpret_cast<const unsigned char*>(src) + 16 * piece);
      }
    }
    cp_async_commit();
  };

  for (int eg = 0; eg < E; eg += EG) {
    float acc[TT][EP];
#pragma unroll
    for (int t = 0; t < TT; ++t)
#pragma unroll
      for (int e = 0; e < EP; ++e) acc[t][e] = 0.0f;

    // One 8-element vector of each of the warp's TT tokens per iteration.  With few experts
    // (EG <= 16) there is little arithmetic per loaded byte, so the token vectors of the next PF
    // iterations are kept in flight in registers; the order of the additions into acc[][] is the
    // same either way.
    auto accumulate = [&](int it, const float (&xv)[TT][8]) {
      const T* wb = wbuf + (static_cast<size_t>(it % NSTG) * EG + part * EP) * kChunk + lane * 8;
#pragma unroll
      for (int e = 0; e < EP; ++e) {
        float wv[8];
        vec8_from_smem<T>(wb + e * kChunk, wv);
#pragma unroll
        for (int t = 0; t < TT; ++t) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if constexpr (Vec8<T>::kExactProducts) {
              acc[t][e] = __fmaf_rn(xv[t][j], wv[j], acc[t][e]);
            } else {
              acc[t][e] = __fadd_rn(acc[t][e], __fmul_rn(xv[t][j], wv[j]));
            }
          }
        }
      }
    };
    // iterations of token vectors in flight: 8 (fp32: 4) vectors of 16 (32) bytes per lane
    constexpr int PF = kDeep ? (sizeof(T) == 4 ? (TT >= 4 ? 1 : 4 / TT) : 8 / TT) : 0;
    if constexpr (PF > 0) {
      Raw8<T> xr[PF][TT];
      auto fetch = [&](int it, Raw8<T> (&slot)[TT]) {
        const int v = it * 32 + lane;
        if (it < iters && v < nvec) {
#pragma unroll
          for (int t = 0; t < TT; ++t) {
            const int tok = min(t0 + t, p.S - 1);  // ragged last group: recompute the last token
            slot[t].fetch(X + static_cast<size_t>(tok) * H + v * 8);
          }
        }
      };
#pragma unroll
      for (int j = 0; j < PF; ++j) fetch(j, xr[j]);
#pragma unroll
      for (int j = 0; j < NSTG - 1; ++j) stage(eg, j);
      for (int it0 = 0; it0 < iters; it0 += PF) {
#pragma unroll
        for (int j = 0; j < PF; ++j) {
          const int it = it0 + j;
          if (it < iters) {   // the same for every thread of the CTA
            stage(eg, it + NSTG - 1);   // into the slot that chunk it - 1 left behind the last barrier
            cp_async_wait<NSTG - 1>();
            __syncthreads();
            if (it * 32 + lane < nvec) {
              float xv[TT][8];
#pragma unroll
              for (int t = 0; t < TT; ++t) xr[j][t].unpack(xv[t]);
              accumulate(it, xv);
            }
            fetch(it + PF, xr[j]);
            __syncthreads();
          }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < NSTG - 1; ++j) stage(eg, j);
      for (int it = 0; it < iters; ++it) {
        stage(eg, it + NSTG - 1);
        cp_async_wait<NSTG - 1>();
        __syncthreads();
        const int v = it * 32 + lane;
        if (v < nvec) {
          float xv[TT][8];
#pragma unroll
          for (int t = 0; t < TT; ++t) {
            const int tok = min(t0 + t, p.S - 1);  // ragged last group: recompute the last token
            Vec8<T>::load(X + static_cast<size_t>(tok) * H + v * 8, xv[t]);
          }
          accumulate(it, xv);
        }
        __syncthreads();
      }
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
#pragma unroll
      for (int e = 0; e < EP; ++e) {
        const int ex = eg + part * EP + e;
        const float s = butterfly_sum(acc[t][e]);
        if (lane == (ex & 31)) {
          const float b = p.logit_bias ? __ldg(p.logit_bias + ex) : 0.0f;
          rows[t * E + ex] = p.logit_bias ? __fadd_rn(s, b) : s;
        }
      }
    }
  }
  __syncthreads();   // a token's logits come from all ES parts
  if (t0 >= p.S) return;

  for (int t = part; t < TT; t += ES) {   // the parts share the group's tokens for the softmax
    const int tok = t0 + t;
    if (tok >= p.S) break;
    softmax_topk_row(p, rows + t * E, tok, lane);
  }
}

// ---- many experts (E a multiple of 32, E >= 64) --------------------------------------------
// Same arithmetic, operation for operation, as router_topk_kernel; what differs is how the
// operands reach the FMA pipe.  Per 256-element chunk of H the CTA converts the 32 x 256 weight
// chunk to fp32 ONCE (not per warp and per use) and parks it in shared memory as
// [element j][expert quad][lane][4 experts], so that a lane fetches four experts' weights for its
// own 8-element vector with one conflict-free 16-byte load; the raw chunk for the next step is
// already in registers while this one is consumed.  The multiply-adds are issued two at a time
// (fma.rn.f32x2: two independent fp32 FMAs per instruction, each rounded as a scalar FMA would
// be), one pair = one token against two neighbouring experts, so every accumulator still sees its
// products in the same order and the result bits are unchanged.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
template <typename T, int TT>
__global__ void __launch_bounds__(512)
router_topk_wide_kernel(const RouterParams p) {
  constexpr int EG = 32, TG = 4, ES = 4, EP = EG / ES;   // 16 warps, 8 experts per warp
  constexpr int kStageFloats = 8 * EG * 32;                                // one chunk: 32 KB
  extern __shared__ __align__(16) unsigned char s_raw[];
  float* s_row = reinterpret_cast<float*>(s_raw);  // [TG][TT][E]: logits, then exp, then probabilities
  const int H = p.H, E = p.E;
  float4* wst = reinterpret_cast<float4*>(s_raw + ((static_cast<size_t>(TG) * TT * E * sizeof(float) + 15) & ~size_t(15)));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tg = warp % TG, part = warp / TG;
  const int t0 = (blockIdx.x * TG + tg) * TT;
  const int nvec = H >> 3;
  const int iters = (nvec + 31) >> 5;
  const T* __restrict__ X = static_cast<const T*>(p.tokens);
  const T* __restrict__ Wr = static_cast<const T*>(p.weights);
  float* rows = s_row + static_cast<size_t>(tg) * TT * E;

  // staging: warps 0..7, warp w = expert quad w of the group, lane = vector of the chunk
  const bool stager = warp < EG / 4;
  Raw8<T> wraw[4];
  auto fetch_w = [&](int eg, int it) {
    const int v = it * 32 + lane;
    if (stager && it < iters && v < nvec) {
#pragma unroll
      for (int q = 0; q < 4; ++q) wraw[q].fetch(Wr + static_cast<size_t>(eg + warp * 4 + q) * H + v * 8);
    }
  };
  auto park_w = [&](int it) {
    const int v = it * 32 + lane;
    if (stager && it < iters && v < nvec) {
      float f[4][8];
#pragma unroll
      for (int q = 0; q < 4; ++q) wraw[q].unpack(f[q]);
      float4* dst = wst + static_cast<size_t>(it & 1) * (kStageFloats / 4) + warp * 32 + lane;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j * (EG / 4) * 32] = make_float4(f[0][j], f[1][j], f[2][j], f[3][j]);
    }
  };

  for (int eg = 0; eg < E; eg += EG) {
    unsigned long long acc[TT][EP / 2];
#pragma unroll
    for (int t = 0; t < TT; ++t)
#pragma unroll
      for (int e = 0; e < EP / 2; ++e) acc[t][e] = 0ull;

    Raw8<T> xr[TT];
    auto fetch_x = [&](int it) {
      const int v = it * 32 + lane;
      if (it < iters && v < nvec) {
#pragma unroll
        for (int t = 0; t < TT; ++t) {
          const int tok = min(t0 + t, p.S - 1);  // ragged last group: recompute the last token
          xr[t].fetch(X + static_cast<size_t>(tok) * H + v * 8);
        }
      }
    };
    __syncthreads();            // the previous group's last chunk has been read by every warp
    fetch_w(eg, 0);
    fetch_x(0);
    park_w(0);
    __syncthreads();
    for (int it = 0; it < iters; ++it) {
      fetch_w(eg, it + 1);      // in flight while this chunk is consumed
      if (it * 32 + lane < nvec) {
        float xv[TT][8];
#pragma unroll
        for (int t = 0; t < TT; ++t) xr[t].unpack(xv[t]);
        fetch_x(it + 1);
        const float4* wb = wst + static_cast<size_t>(it & 1) * (kStageFloats / 4) + (part * 2) * 32 + lane;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 wa = wb[j * (EG / 4) * 32], wc = wb[j * (EG / 4) * 32 + 32];
          const unsigned long long wp[4] = {pack2(wa.x, wa.y), pack2(wa.z, wa.w), pack2(wc.x, wc.y), pack2(wc.z, wc.w)};
#pragma unroll
          for (int t = 0; t < TT; ++t) {
            const unsigned long long xx = pack2(xv[t][j], xv[t][j]);
#pragma unroll
            for (int e = 0; e < EP / 2; ++e) {
              if constexpr (Vec8<T>::kExactProducts) {
                acc[t][e] = fma2(xx, wp[e], acc[t][e]);
              } else {
                // fp32 inputs: a rounded multiply, then a rounded add, as scalar operations (the
                // paired forms did not reproduce the scalar bits on sm_100a)
                float a0, a1, w0, w1;
                unpack2(acc[t][e], a0, a1);
                unpack2(wp[e], w0, w1);
                acc[t][e] = pack2(__fadd_rn(a0, __fmul_rn(xv[t][j], w0)), __fadd_rn(a1, __fmul_rn(xv[t][j], w1)));
              }
            }
          }
        }
      } else {
        fetch_x(it + 1);
      }
      park_w(it + 1);           // into the buffer chunk it - 1 left behind the last barrier
      __syncthreads();
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
#pragma unroll
      for (int e = 0; e < EP; ++e) {
        float lo, hi;
        unpack2(acc[t][e >> 1], lo, hi);
        const int ex = eg + part * EP + e;
        const float s = butterfly_sum((e & 1) ? hi : lo);
        if (lane == (ex & 31)) {
          const float b = p.logit_bias ? __ldg(p.logit_bias + ex) : 0.0f;
          rows[t * E + ex] = p.logit_bias ? __fadd_rn(s, b) : s;
        }
      }
    }
  }
  __syncthreads();   // a token's logits come from all ES parts
  if (t0 >= p.S) return;
  for (int t = part; t < TT; t += ES) {   // the parts share the group's tokens for the softmax
    const int tok = t0 + t;
    if (tok >= p.S) break;
    softmax_topk_row(p, rows + t * E, tok, lane);
  }
}

// One CTA per expert walks the tokens in ascending order and hands out slots.
__global__ void __launch_bounds__(1024) router_slots_kernel(const RouterParams p) {
  __shared__ int warp_tot[32];
  __shared__ int base_s;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < p.S; c0 += blockDim.x) {
    const int t = c0 + threadIdx.x;
    int hit = -1;
    if (t < p.S) {
      for (int j = 0; j < p.k; ++j)
        if (p.topk_idx[static_cast<size_t>(t) * p.k + j] == e) { hit = j; break; }
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, hit >= 0);
    const int before = __popc(ballot & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int warp_base = 0, total = 0;
    for (int w = 0; w < nwarps; ++w) {
      const int c = warp_tot[w];
      if (w < warp) warp_base += c;
      total += c;
    }
    const int base = base_s;
    if (hit >= 0) {
      const int slot = base + warp_base + before;
      const float wt = p.topk_w[static_cast<size_t>(t) * p.k + hit];
      if (slot < p.EC)
        p.table[static_cast<size_t>(e) * p.round_ec + slot] = TokenSlot{static_cast<uint32_t>(t), wt};
      p.routes[static_cast<size_t>(t) * p.k + hit] = Route{e, slot, wt, 0};
    }
    __syncthreads();
    if (threadIdx.x == 0) base_s = base + total;
    __syncthreads();
  }
  if (threadIdx.x == 0) p.expert_counts[e] = base_s;
}

template <typename T, int TT, int TG, int ES>
cudaError_t launch_topk_eg(const RouterParams& p, cudaStream_t stream) {
  const int ctas = (p.S + TG * TT - 1) / (TG * TT);
  auto go = [&](auto kern, int eg) -> cudaError_t {
    const size_t rows = (static_cast<size_t>(TG) * TT * p.E * sizeof(float) + 15) & ~size_t(15);
    const size_t smem = rows + (eg <= 16 ? 4 : 2) * static_cast<size_t>(eg) * 256 * sizeof(T);
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return e;
    }
    kern<<<ctas, TG * ES * 32, smem, stream>>>(p);
    ++g_launches;
    return cudaGetLastError();
  };
  if (p.E % 32 == 0) return go(router_topk_kernel<T, TT, 32, TG, ES>, 32);
  if (p.E % 16 == 0) return go(router_topk_kernel<T, TT, 16, TG, ES>, 16);
  return go(router_topk_kernel<T, TT, 8, TG, ES>, 8);
}

// A CTA holds TG = 4 token groups x ES expert parts of warps, each warp TT tokens.  With many
// experts: ES = 4, and TT the largest that still fills the SMs with warps.  With few experts a
// warp has little arithmetic per token and the kernel lives on how many warps hide its latencies:
// two tokens per warp and the experts split over two warps measured fastest from 1 K to 8 K tokens
// (Scout shapes, 1024 tokens: 21.5 us for both router kernels, against 24-43 us for the other
// splits).
template <typename T, int TT>
cudaError_t launch_topk_wide(const RouterParams& p, cudaStream_t stream) {
  const int ctas = (p.S + 4 * TT - 1) / (4 * TT);
  const size_t rows = (static_cast<size_t>(4) * TT * p.E * sizeof(float) + 15) & ~size_t(15);
  const size_t smem = rows + 2 * static_cast<size_t>(8 * 32 * 32) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(router_topk_wide_kernel<T, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  router_topk_wide_kernel<T, TT><<<ctas, 512, smem, stream>>>(p);
  ++g_launches;
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_topk(const RouterParams& p, cudaStream_t stream) {
  // many experts and enough tokens to fill the SMs four to a warp: weights converted once per CTA,
  // paired FMAs (router_topk_wide_kernel); below that its per-CTA staging does not pay
  // (two tokens per warp and two CTAs per SM measured slower: 303 vs 262 us at Qwen3 shapes, 8192 tokens)
  if (p.E >= 64 && p.E % 32 == 0 && p.S >= 120 * 16) return launch_topk_wide<T, 4>(p, stream);
  if (p.E >= 64) {
    if (p.S >= 120 * 16) return launch_topk_eg<T, 4, 4, 4>(p, stream);
    if (p.S >= 120 * 8) return launch_topk_eg<T, 2, 4, 4>(p, stream);
    return launch_topk_eg<T, 1, 4, 4>(p, stream);
  }
  return launch_topk_eg<T, 2, 4, 2>(p, stream);
}

}  // namespace

cudaError_t launch_router(const RouterParams& p, cudaStream_t stream) {
  cudaError_t e;
  switch (p.dtype) {
    case FMOE_DT_BF16: e = launch_topk<__nv_bfloat16>(p, stream); break;
    case FMOE_DT_FP16: e = launch_topk<__half>(p, stream); break;
    case FMOE_DT_FP32: e = launch_topk<float>(p, stream); break;
    default: return cudaErrorInvalidValue;
  }
  if (e != cudaSuccess) return e;
  const int threads = p.S >= 1024 ? 1024 : (p.S >= 256 ? 256 : 64);
  router_slots_kernel<<<p.E, threads, 0, stream>>>(p);
  ++g_launches;
  return cudaGetLastError();
}

}  // namespace fmoe

// ---- routing without any allocation ---------------------------------------------------------
//
// Some hosts of this library may not allocate device memory at all when they want a routing
// decision: a serving engine that has handed the whole GPU to its own memory pool and treats any
// later cudaMalloc as a bug (it can fail, and it synchronises the device), or a plug-in that is
// called between two of the engine's own launches and must not disturb its allocator.  For them
// the router's only scratch (the per-token top-k ids and weights the first kernel hands to the
// second) lives in this fixed array instead of a per-context allocation.  Every GPU that loads
// the library carries these 1 MiB until the process exits.
constexpr int kStaticRouterMaxPairs = 1 << 17;  // tokens_per_rank * top_k this entry point accepts
static __device__ __align__(256) unsigned char g_router_scratch[kStaticRouterMaxPairs * 8];

namespace fmoe {
namespace {
std::mutex g_scratch_mu;
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};  // device address of g_router_scratch, per device
}  // namespace
}  // namespace fmoe

extern "C" int fmoe_router_forward_static(const fmoe_model_desc* model, int32_t device_id,
                                          const fmoe_router_args* a, void* token_table,
                                          int32_t round_ec, void* routes, void* stream) {
  using namespace fmoe;
  int rc = validate_model(model);
  if (rc != FMOE_OK) return rc;
  if (a == nullptr || a->tokens == nullptr || a->weights == nullptr || a->expert_counts == nullptr ||
      token_table == nullptr || routes == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "tokens, weights, expert_counts, token_table and routes are required");
  if (model->data_type == FMOE_DT_FP64)
    return set_error(FMOE_ERR_UNSUPPORTED, "the router handles BF16, FP16 and FP32");
  if ((reinterpret_cast<uintptr_t>(a->tokens) | reinterpret_cast<uintptr_t>(a->weights) |
       reinterpret_cast<uintptr_t>(routes)) & 15)
    return set_error(FMOE_ERR_INVALID_ARG, "tokens, weights and routes must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(token_table) & 7)
    return set_error(FMOE_ERR_INVALID_ARG, "token_table must be 8-byte aligned");
  if ((reinterpret_cast<uintptr_t>(a->expert_counts) | reinterpret_cast<uintptr_t>(a->routing) |
       reinterpret_cast<uintptr_t>(a->logit_bias)) & 3)
    return set_error(FMOE_ERR_INVALID_ARG, "expert_counts, routing and logit_bias must be 4-byte aligned");
  if (round_ec < model->expert_peer_capacity)
    return set_error(FMOE_ERR_INVALID_ARG, "round_ec (row stride of token_table) is smaller than expert_peer_capacity");
  const long long pairs = static_cast<long long>(model->tokens_per_rank) * model->top_k;
  if (pairs > kStaticRouterMaxPairs)
    return set_error(FMOE_ERR_UNSUPPORTED,
                     "fmoe_router_forward_static handles at most " + std::to_string(kStaticRouterMaxPairs) +
                         " (token, choice) pairs per call; this layer has " + std::to_string(pairs) +
                         ": use fmoe_router_forward with a router context instead");
  if (static_cast<size_t>(model->num_experts) * 4 * 8 * 4 > 200 * 1024)
    return set_error(FMOE_ERR_UNSUPPORTED, "num_experts too large for the router's shared-memory rows");
  if (device_id < 0 || device_id >= kMaxDevices)
    return set_error(FMOE_ERR_INVALID_ARG, "device_id out of range");
  // The calling thread's current device is put back on every way out: a plug-in running between a
  // host engine's own launches must not leave the engine on another GPU.
  struct DeviceGuard {
    int prev = -1;
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
  } guard;
  cudaError_t ce = cudaGetDevice(&guard.prev);
  if (ce != cudaSuccess) { guard.prev = -1; return set_error(FMOE_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(ce)); }
  if (guard.prev == device_id) guard.prev = -1;   // nothing to restore
  else {
    ce = cudaSetDevice(device_id);
    if (ce != cudaSuccess) return set_error(FMOE_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(ce));
  }
  void* scratch = nullptr;
  {
    // One-time set-up per device, with that device current: the array's name is only a host-side
    // stand-in for the symbol, the kernels need its device address.
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (g_scratch_addr[device_id] == nullptr) {
      void* addr = nullptr;
      ce = cudaGetSymbolAddress(&addr, g_router_scratch);
      if (ce != cudaSuccess || addr == nullptr)
        return set_error(FMOE_ERR_CUDA, std::string("cudaGetSymbolAddress(router scratch): ") +
                                            cudaGetErrorString(ce));
      g_scratch_addr[device_id] = addr;
    }
    scratch = g_scratch_addr[device_id];
  }
  RouterParams p{};
  p.S = model->tokens_per_rank; p.H = model->token_dim; p.E = model->num_experts; p.k = model->top_k;
  p.EC = model->expert_peer_capacity; p.round_ec = round_ec; p.dtype = model->data_type;
  p.tokens = a->tokens; p.weights = a->weights; p.logit_bias = a->logit_bias; p.routing = a->routing;
  // both halves are fully rewritten for [0, pairs) by the first kernel before the second reads
  // them, so nothing has to start at zero
  p.topk_idx = static_cast<int32_t*>(scratch);
  p.topk_w = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + kStaticRouterMaxPairs * 4);
  p.expert_counts = a->expert_counts;
  p.table = static_cast<TokenSlot*>(token_table);
  p.routes = static_cast<Route*>(routes);
  ce = launch_router(p, static_cast<cudaStream_t>(stream));
  if (ce != cudaSuccess) return set_error(FMOE_ERR_CUDA, std::string("router launch: ") + cudaGetErrorString(ce));
  return FMOE_OK;
}
