// The MoE-layer forward as one persistent sm_100a kernel: count exchange, dispatch, expert
// GEMMs (tcgen05 / TMEM, TMA-fed), return of the expert outputs, combine.
//
// It replaces the reference's moe::forward kernel and its in-kernel runtime
// (csrc/include/flashmoe/moe.cuh:161-247, os.cuh, scheduler.cuh, subscriber.cuh,
// dispatch.cuh, processor.cuh, combine.cuh).  What is kept is the contract: one launch per
// forward, experts sharded over the ranks of one NVLink box, tokens pushed to the expert's
// owner by in-kernel peer stores, results pushed back, readiness carried by flags and
// counters in a symmetric block, nothing cleared by the host between launches.  What is
// different, and why:
//
//  * Rows are PACKED per expert at the owner (all source ranks back to back), so M tiles are
//    full whenever an expert has >= 128 rows in total; the reference tiles per (source rank,
//    expert) and pads each to the tile height (subscriber.cuh:121-160).  Packing needs every
//    rank's per-expert counts first: each launch opens with a count exchange through the
//    symmetric block (W*E ints per rank), which doubles as the epoch handshake.
//  * No central "OS" CTA: every CTA runs the same scheduler warp, which takes tickets from one
//    global counter over a fixed task order (GEMM0 of expert i, then GEMM1 of expert i-lag)
//    and waits on the task's readiness counters itself.  Tickets are handed out in an order
//    in which a task only ever waits on tasks with smaller tickets, so the kernel cannot
//    deadlock as long as all CTAs are co-resident (grid <= SM count, one CTA per SM), which the
//    cooperative launch guarantees.
//  * Each CTA is warp-specialised: warp 0 = scheduler + TMA producer, warp 1 = UMMA issuer and
//    TMEM owner, warps 2..5 = epilogue, warps 6..7 = dispatch: this rank's routed rows go to the
//    experts' owners in chunks taken from a per-CTA queue by the dispatch warps and, between
//    epilogues, by the epilogue warps, while warps 0 and 1 already work on the first tiles whose
//    rows are in.  By default every CTA works alone on 128 x 256 output
//    tiles (tcgen05.mma.cta_group::1, M = 128, N = 256): a 4-stage TMA->UMMA ring of 48 KB stages
//    (A tile 128 x 64, B tile 256 x 64) and a double-buffered 2 x 256-column TMEM accumulator
//    overlap loads, MMA and epilogue.  A second form of the same body (opt-in) runs CTA pairs,
//    clusters of 2 on the two SMs of a TPC, on 256 x 256 tiles with tcgen05.mma.cta_group::2:
//    each CTA loads its own 128 rows of A and HALF of the B tile (6 stages of 32 KB), the leader's
//    scheduler draws the ticket, waits for readiness and passes the ticket to the follower
//    through distributed shared memory.
//  * Gate and up projections are ONE UMMA of N = 256 (gate rows | up rows in the B tile);
//    the SiLU-gate product is formed in the epilogue straight from TMEM.  The reference
//    runs its main loop twice and parks the gate tile in shared memory
//    (processor.cuh:97-136).  Rounding points are the reference's: the activated gate value
//    is rounded to Element, the product is rounded to Element, the GEMM1 output is rounded
//    to Element.
//  * Expert outputs return to the token's owner as rows indexed by (token, choice), written as
//    whole 128-byte runs of one row through a shared-memory transpose; the owner sums a
//    token's k rows in fp32 in selection order and rounds once (the reference accumulates with
//    Element-precision atomics in arrival order, combine.cuh:120-223).
//  * The last GEMM1 tiles of the task order are cut along K into parts whose fp32 partial sums
//    are added in part order by whichever part finishes last, so the kernel ends on short
//    tickets without losing run-to-run reproducibility.
//  * Every signal that crosses CTAs or GPUs is one fence followed by relaxed counter updates
//    (per batch of dispatched rows, per GEMM1 epilogue), not a release per update.
//  * Optionally the launch opens with the router itself (three grid-wide phases).
//
// Every wait is bounded; a wait that runs out records where in `status`, raises the
// kernel-wide abort word and every role leaves through the common exit (TMEM freed).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"
#include "router_math.cuh"

namespace fmoe {

unsigned long long g_launches = 0;

namespace {

using namespace ptx;

struct alignas(64) TmaMaps {
  CUtensorMap landing;  // [landing_rows, H]   box 64 x 128
  CUtensorMap y;        // [landing_rows, I]   box 64 x 128
  CUtensorMap up;       // [nLx*I, H]          box 64 x 128
  CUtensorMap up_v;     // [nLx*I, H]          box 64 x 128
  CUtensorMap down;     // [nLx*H, I]          box 64 x 128
};

enum : int { kTaskGemm0 = 0, kTaskGemm1 = 1, kTaskStop = 2 };

// What one CTA of a pair does for one ticket: its own M tile (the leader takes the even tile of
// the group, the follower the odd one) of the pair's 256 x 256 output tile.
struct Task {
  int kind, lx, mt, row0, rows, n, m_in_expert, ticket;
  // GEMM1 tiles of the closing wave are cut along K into `nparts` tickets: part `part` covers K
  // blocks [nk * part / nparts, nk * (part + 1) / nparts); `split_idx` numbers the tile among the
  // split ones (its slot in the partial-sum scratch and in the part counters).
  int part, nparts, split_idx;
};

constexpr uint32_t kRetStageBytes = 4 * 2048;

struct Control {
  uint64_t full[6], empty[6];   // ring depth: 6 in pair mode, 4 alone
  uint64_t acc_full[kAccBufs], acc_empty[kAccBufs];
  uint64_t task_full[kTaskSlots], task_empty[kTaskSlots];
  uint64_t pair_full[kTaskSlots], pair_empty[kTaskSlots];   // leader -> follower ticket ring
  uint32_t pair_ticket[kTaskSlots];
  Task tasks[kTaskSlots];
  uint32_t tmem_base;
  uint32_t ok;            // cleared when a CTA-wide wait failed
  int total_tasks, n_segs, send_rows, class0_experts, expected_ret;
  int next_chunk;          // dispatch: next chunk of this CTA's rows nobody has taken yet
  uint64_t epoch;
};

__device__ __forceinline__ void fail(const MoeParams& p, int phase, long long detail) {
  if (atomicCAS(p.abort_word, 0u, 1u) == 0u) {
    p.status->code = FMOE_ERR_DEVICE_TIMEOUT;
    p.status->phase = phase;
    p.status->rank = p.rank;
    p.status->cta = static_cast<int>(blockIdx.x);
    p.status->detail = detail;
    __threadfence_system();
  }
}

// Spin until *ctr >= want (acquire, system scope).  false = gave up.
__device__ __forceinline__ bool wait_counter_sys(const uint32_t* ctr, uint32_t want,
                                                 const WaitCtx& w) {
  if (ld_acquire_sys(ctr) >= want) return true;
  SpinGuard g;
  while (ld_acquire_sys(ctr) < want) {
    if (g.expired(w)) return ld_acquire_sys(ctr) >= want;
  }
  return true;
}
__device__ __forceinline__ bool wait_counter_gpu(const uint32_t* ctr, uint32_t want,
                                                 const WaitCtx& w) {
  if (ld_acquire_gpu(ctr) >= want) return true;
  SpinGuard g;
  while (ld_acquire_gpu(ctr) < want) {
    if (g.expired(w)) return ld_acquire_gpu(ctr) >= want;
  }
  return true;
}

template <typename T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
  static constexpr int kFormat = 1;
  __device__ __forceinline__ static float up(uint32_t bits16) { return __uint_as_float(bits16 << 16); }
  __device__ __forceinline__ static uint32_t pack(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ __forceinline__ static float round(float a) {
    return __bfloat162float(__float2bfloat16_rn(a));
  }
};
template <> struct Cvt<__half> {
  static constexpr int kFormat = 0;
  __device__ __forceinline__ static float up(uint32_t bits16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
  }
  __device__ __forceinline__ static uint32_t pack(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ __forceinline__ static float round(float a) { return __half2float(__float2half_rn(a)); }
};

// FP32 layers run on the same BF16 tensor-core pipeline: every fp32 operand is held as three BF16
// planes a = a1 + a2 + a3 (a1 = bf16(a), a2 = bf16(a - a1), a3 = bf16(a - a1 - a2), 24 mantissa
// bits in all) and a product is the six plane pairs with i + j <= 2.  The three dropped pairs are
// below 2^-24 relative.  The leading pair (a1, b1) accumulates in one TMEM accumulator and the five
// correction pairs in a second one; the epilogue adds the two in fp32.  Keeping the corrections
// apart matters: the tensor core's accumulate step is not correctly rounded, and its error scales
// with the accumulator's magnitude and with the number of MMA steps into it.
template <> struct Cvt<float> {
  static constexpr int kFormat = 1;
  __device__ __forceinline__ static float round(float a) { return a; }
};
template <typename T> struct Elem { static constexpr int kBytes = 2; static constexpr int kPlanes = 1; };
template <> struct Elem<float> { static constexpr int kBytes = 4; static constexpr int kPlanes = 3; };

__device__ __forceinline__ void split3(float a, unsigned short (&out)[3]) {
  const __nv_bfloat16 a1 = __float2bfloat16_rn(a);
  const float r1 = a - __bfloat162float(a1);
  const __nv_bfloat16 a2 = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(a2);
  const __nv_bfloat16 a3 = __float2bfloat16_rn(r2);
  out[0] = __bfloat16_as_ushort(a1); out[1] = __bfloat16_as_ushort(a2); out[2] = __bfloat16_as_ushort(a3);
}

// 32 consecutive columns of one row of a GEMM operand buffer (Y): Element for 16-bit types, three
// BF16 planes `plane_bytes` apart for fp32.  `row` points at the row's first column in plane 0.
template <typename T>
__device__ __forceinline__ void store_operand32(char* row, int col0, const float (&v)[32], size_t plane_bytes) {
  if constexpr (Elem<T>::kPlanes == 1) {
    uint4* dst = reinterpret_cast<uint4*>(row + static_cast<size_t>(col0) * 2);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      dst[q] = make_uint4(Cvt<T>::pack(v[8 * q], v[8 * q + 1]), Cvt<T>::pack(v[8 * q + 2], v[8 * q + 3]),
                          Cvt<T>::pack(v[8 * q + 4], v[8 * q + 5]), Cvt<T>::pack(v[8 * q + 6], v[8 * q + 7]));
  } else {
    uint32_t pl[3][16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      unsigned short a[3], b[3];
      split3(v[i], a);
      split3(v[i + 1], b);
#pragma unroll
      for (int q = 0; q < 3; ++q) pl[q][i >> 1] = static_cast<uint32_t>(a[q]) | (static_cast<uint32_t>(b[q]) << 16);
    }
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      uint4* dst = reinterpret_cast<uint4*>(row + q * plane_bytes + static_cast<size_t>(col0) * 2);
#pragma unroll
      for (int w = 0; w < 4; ++w) dst[w] = make_uint4(pl[q][4 * w], pl[q][4 * w + 1], pl[q][4 * w + 2], pl[q][4 * w + 3]);
    }
  }
}
template <bool kPrecise>
__device__ __forceinline__ float activate_t(float x, int act) {
  switch (act) {
    case FMOE_ACT_SILU:
      if constexpr (kPrecise) return x / (1.0f + expf(-x));
      else return __fdividef(x, 1.0f + __expf(-x));
    case FMOE_ACT_GELU: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    case FMOE_ACT_RELU: return fmaxf(x, 0.0f);
    default: return x;
  }
}

template <typename T>
__device__ __forceinline__ float bias_at(const void* bias, size_t idx) {
  if (bias == nullptr) return 0.0f;
  if constexpr (Elem<T>::kBytes == 4) {
    return __ldg(static_cast<const float*>(bias) + idx);
  } else {
    return Cvt<T>::up(static_cast<uint32_t>(__ldg(static_cast<const unsigned short*>(bias) + idx)));
  }
}

// Shared-memory tables built by every CTA from the exchanged counts.
struct Tables {
  int* n;          // [W][E] rows rank s sends to expert e (clamped to EC)
  int* dst_row0;   // [E]    landing row at e's owner where THIS rank's rows for e start
  int* ord;        // [E]    send order: position -> expert (experts their owners work on first come first)
  int* send_pref;  // [E+1]  rows this rank sends before send-order position i
  int* lx_base;    // [nLx]  landing row where local expert lx starts (multiple of 128)
  int* lx_rows;    // [nLx]  rows of local expert lx, all sources
  int* lx_mt0;     // [nLx+1] prefix of M tiles
  int* seg_first;  // [2 nLx + 1] first ticket of each segment of the task order
  int* seg_kind;   // [2 nLx]
  int* seg_lx;     // [2 nLx]
  int* seg_whole;  // [2 nLx] GEMM1 segments: leading tickets that cover a whole tile (the rest are K parts)
  int* tot;        // [E]    rows expert e receives from all sources
  int* tmp;        // [E]    scratch of the table construction
  int* owner;      // [E]    expert -> rank                      (copies of the context's maps, so
  int* lidx;       // [E]    expert -> index at its owner         that nothing after the count
  int* local_e;    // [W][nLx] -> expert                          exchange waits on global memory)
};

__host__ __device__ inline size_t tables_ints(int W, int E, int nLx) {
  return static_cast<size_t>(W) * E + E + E + (E + 1) + nLx + nLx + (nLx + 1) + (2 * nLx + 1) +
         2 * nLx + 2 * nLx + 2 * nLx + E + E + E + E + static_cast<size_t>(W) * nLx;
}

// kPair = true: CTA pairs on 256-row tile groups (experts with several M tiles; tensor-bound work).
// kPair = false: every CTA on its own 128 x 256 tile with the whole B tile (4 stages of 48 KB):
// more weight bytes in flight per SM, which is what counts when experts hold <= 128 rows and the
// layer streams weights from HBM.
template <typename T, bool kPair, typename Spec>
__device__ __forceinline__ void moe_forward_body(const MoeParams& p, const TmaMaps& maps) {
  extern __shared__ uint8_t smem_raw[];
  // the layer's shape: launch parameters in the generic build, constants in a specialised one
  const int H_ = Spec::kFixed ? Spec::kH : p.H, I_ = Spec::kFixed ? Spec::kI : p.I;
  const int K_ = Spec::kFixed ? Spec::kTopK : p.k;
  const bool gated_ = Spec::kFixed ? Spec::kGated : p.gated != 0;
  const int act_ = Spec::kFixed ? Spec::kAct : p.act;
  const int tiles_n0_ = Spec::kFixed ? (Spec::kI + (Spec::kGated ? 128 : 256) - 1) / (Spec::kGated ? 128 : 256) : p.tiles_n0;
  const int tiles_n1_ = Spec::kFixed ? (Spec::kH + 255) / 256 : p.tiles_n1;
  constexpr int NS = kPair ? 6 : 4;                                   // ring depth
  constexpr uint32_t SA = kStageABytes;                               // A tile of this CTA
  constexpr uint32_t SB = kPair ? kStageABytes : 2 * kStageABytes;    // B rows this CTA loads
  constexpr uint32_t STAGE = SA + SB;
  constexpr int kGroup = kPair ? 2 : 1;                               // M tiles per ticket
  // stage ring first, 1024-byte aligned (128-byte swizzle atoms)
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  // 2 KB per epilogue warp: expert output rows pass through here so that they leave as whole lines
  uint4* ret_stage = reinterpret_cast<uint4*>(stages + NS * STAGE);
  Control* ctl = reinterpret_cast<Control*>(stages + NS * STAGE + kRetStageBytes);
  int* tab = reinterpret_cast<int*>(ctl + 1);
  Tables tb;
  {
    int* q = tab;
    tb.n = q; q += p.W * p.E;
    tb.dst_row0 = q; q += p.E;
    tb.ord = q; q += p.E;
    tb.send_pref = q; q += p.E + 1;
    tb.lx_base = q; q += p.nLx;
    tb.lx_rows = q; q += p.nLx;
    tb.lx_mt0 = q; q += p.nLx + 1;
    tb.seg_first = q; q += 2 * p.nLx + 1;
    tb.seg_kind = q; q += 2 * p.nLx;
    tb.seg_lx = q; q += 2 * p.nLx;
    tb.seg_whole = q; q += 2 * p.nLx;
    tb.tot = q; q += p.E;
    tb.tmp = q; q += p.E;
    tb.owner = q; q += p.E;
    tb.lidx = q; q += p.E;
    tb.local_e = q;
  }
  const WaitCtx wc{p.abort_word, p.spin_limit};
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t pair_rank = 0;                         // 0 = leader of the CTA pair, 1 = follower
  if constexpr (kPair) pair_rank = cluster_ctarank();
  const bool leader = pair_rank == 0;
  const int W = p.W, E = p.E, nLx = p.nLx;
  char* const self = p.peers[p.rank];
  constexpr int EB = Elem<T>::kBytes;     // bytes per element of tokens, return rows and output
  constexpr int kPlanes = Elem<T>::kPlanes;  // BF16 planes per GEMM operand
  const size_t landing_plane = static_cast<size_t>(p.landing_rows) * H_ * 2;
  const size_t y_plane = static_cast<size_t>(p.landing_rows) * I_ * 2;

  // ---- set-up: barriers, TMEM, epoch ---------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) { mbar_init(&ctl->full[i], 1); mbar_init(&ctl->empty[i], 1); }
    // acc_empty collects the four epilogue warps of BOTH CTAs of the pair (only the leader's is
    // waited on); task_empty: this CTA's MMA thread (leader only) + its four epilogue warps
    for (int i = 0; i < kAccBufs; ++i) { mbar_init(&ctl->acc_full[i], 1); mbar_init(&ctl->acc_empty[i], kPair ? 8 : 4); }
    for (int i = 0; i < kTaskSlots; ++i) {
      mbar_init(&ctl->task_full[i], 1); mbar_init(&ctl->task_empty[i], leader ? 5 : 4);
      mbar_init(&ctl->pair_full[i], 1); mbar_init(&ctl->pair_empty[i], 1);
    }
    ctl->ok = 1;
    ctl->next_chunk = kThreads / 32 - 2;   // every dispatching warp starts on the chunk of its own number
    ctl->epoch = *p.epoch;
    mbar_fence_init();
    prefetch_tmap(&maps.landing); prefetch_tmap(&maps.y); prefetch_tmap(&maps.up);
    prefetch_tmap(&maps.up_v); prefetch_tmap(&maps.down);
  }
  if (warp == 1) {
    if constexpr (kPair) { tmem_alloc_pair(&ctl->tmem_base, 512); tmem_relinquish_pair(); }
    else { tmem_alloc(&ctl->tmem_base, 512); tmem_relinquish(); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  tc_fence_after_sync();
  // per-CTA phase stamps (%globaltimer, ns): 0 start, 1 counts of all ranks in, 2 task order built
  // (warp 0), 3 this CTA's dispatch warps done (may precede 2), 4 last ticket (stop) drawn, 5 this
  // CTA's last task finished, 6 returns all in, 7 combine done, 8 first operand stage of this CTA's
  // first task landed (the first MMA can issue), 9..11 the epilogue of the CTA's last task
  auto stamp_now = [&](int i) {   // called by one thread
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.trace[static_cast<size_t>(blockIdx.x) * kTraceSlots + i] = t;
  };
  auto stamp = [&](int i) { if (tid == 0) stamp_now(i); };
  if (tid == 0) p.trace[static_cast<size_t>(blockIdx.x) * kTraceSlots + 8] = 0;
  stamp(0);
  const uint64_t epoch = ctl->epoch;
  const uint64_t flag_val = epoch + 1;
  const int parity = static_cast<int>(epoch & 1);

  // ---- routing inside the launch (optional) ----------------------------------------------
  // The router's two steps as phases of this kernel, for callers that want one launch per
  // layer (decode-sized batches, where two extra launches cost as much as the layer): every warp
  // of the grid computes logits in the router kernels' own fp32 order (lane l of the warp owns the
  // 8-element vectors v = l mod 32 of H, ascending, one FMA per element; xor-butterfly fold), a
  // grid barrier, a warp per token runs softmax and top-k, a barrier, every CTA takes experts and
  // hands out slots in ascending token order, a third barrier.  The stage ring is idle until the
  // first ticket and lends each warp a row of E floats.
  if (p.router_w != nullptr) {
    auto grid_barrier = [&](unsigned long long target) {
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        atomicAdd(p.grid_bar, 1ull);
        SpinGuard g;
        while (ld_acquire_gpu(reinterpret_cast<const uint64_t*>(p.grid_bar)) < target) {
          if (g.expired(wc)) {
            if (ld_acquire_gpu(reinterpret_cast<const uint64_t*>(p.grid_bar)) < target) { fail(p, FMOE_PHASE_ROUTING, target); ctl->ok = 0; }
            break;
          }
        }
      }
      __syncthreads();
    };
    {
      // logits: one work item = one token against 8 experts, items dealt round-robin to the grid's
      // warps (a single token still spreads over E / 8 warps)
      const T* __restrict__ X = static_cast<const T*>(p.tokens);
      const T* __restrict__ Wr = static_cast<const T*>(p.router_w);
      const int nvec = H_ >> 3, iters = (nvec + 31) >> 5;
      const int groups = E >> 3;
      const int G = gridDim.x * (kThreads / 32);
      for (int item = blockIdx.x * (kThreads / 32) + warp; item < p.S * groups; item += G) {
        const int tok = item / groups, eg = (item - tok * groups) << 3;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
#pragma unroll 2
        for (int it = 0; it < iters; ++it) {
          const int v = it * 32 + lane;
          if (v < nvec) {
            float xv[8];
            Vec8<T>::load(X + static_cast<size_t>(tok) * H_ + v * 8, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float wv[8];
              Vec8<T>::load(Wr + static_cast<size_t>(eg + e) * H_ + v * 8, wv);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if constexpr (Vec8<T>::kExactProducts) acc[e] = __fmaf_rn(xv[j], wv[j], acc[e]);
                else acc[e] = __fadd_rn(acc[e], __fmul_rn(xv[j], wv[j]));
              }
            }
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float sum = butterfly_sum(acc[e]);
          if (lane == e) __stcg(p.route_logits + static_cast<size_t>(tok) * E + eg + e,
                                p.logit_bias ? __fadd_rn(sum, __ldg(p.logit_bias + eg + e)) : sum);
        }
      }
    }
    grid_barrier(gridDim.x);
    if (ctl->ok) {
      // softmax and top-k: one warp per token, the token's row of logits in shared memory
      float* row = reinterpret_cast<float*>(stages) + static_cast<size_t>(warp) * E;
      Route* routes = const_cast<Route*>(p.routes);
      for (int tok = blockIdx.x * (kThreads / 32) + warp; tok < p.S; tok += gridDim.x * (kThreads / 32)) {
        for (int j = lane; j < E; j += 32) row[j] = __ldcg(p.route_logits + static_cast<size_t>(tok) * E + j);
        __syncwarp();
        int idx;
        float weight;
        softmax_topk_row(E, K_, p.routing, row, tok, lane, idx, weight);
        if (lane < K_) routes[static_cast<size_t>(tok) * K_ + lane] = Route{idx, 0x7fffffff, weight, 0};
        __syncwarp();
      }
    }
    grid_barrier(2ull * gridDim.x);
    if (ctl->ok) {
      // slots: one CTA per expert (strided), tokens in ascending order, kThreads at a time
      int* warp_tot = reinterpret_cast<int*>(stages);      // [warps] + running base
      Route* routes = const_cast<Route*>(p.routes);
      TokenSlot* table = const_cast<TokenSlot*>(p.table);
      for (int e = blockIdx.x; e < E; e += gridDim.x) {
        __syncthreads();
        if (tid == 0) warp_tot[8] = 0;
        __syncthreads();
        for (int c0 = 0; c0 < p.S; c0 += kThreads) {
          const int tkn = c0 + tid;
          int hit = -1;
          if (tkn < p.S) {
            for (int j = 0; j < K_; ++j)
              if (__ldcg(&routes[static_cast<size_t>(tkn) * K_ + j].expert) == e) { hit = j; break; }
          }
          const unsigned ballot = __ballot_sync(0xffffffffu, hit >= 0);
          const int before = __popc(ballot & ((1u << lane) - 1));
          if (lane == 0) warp_tot[warp] = __popc(ballot);
          __syncthreads();
          int warp_base = 0, total = 0;
          for (int w = 0; w < kThreads / 32; ++w) {
            const int c = warp_tot[w];
            if (w < warp) warp_base += c;
            total += c;
          }
          const int base = warp_tot[8];
          if (hit >= 0) {
            const int slot = base + warp_base + before;
            Route* rt = &routes[static_cast<size_t>(tkn) * K_ + hit];
            const float wt = __ldcg(&rt->weight);
            if (slot < p.EC) table[static_cast<size_t>(e) * p.round_ec + slot] = TokenSlot{static_cast<uint32_t>(tkn), wt};
            rt->slot = slot;
          }
          __syncthreads();
          if (tid == 0) warp_tot[8] = base + total;
          __syncthreads();
        }
        if (tid == 0) p.counts_out[e] = warp_tot[8];
      }
    }
    grid_barrier(3ull * gridDim.x);
  }

  // ---- count exchange (CTA 0 publishes; everyone waits) --------------------------------
  if (blockIdx.x == 0) {
    // Counters of the previous forward are reset here: nobody can touch them before this
    // rank's counts are out, because every rank needs every rank's counts to proceed.
    for (int i = tid; i < p.max_mtiles; i += kThreads) p.gemm0_done[i] = 0;
    uint32_t* arrived = reinterpret_cast<uint32_t*>(self + p.lay.disp_arrived);
    for (int i = tid; i < W * nLx; i += kThreads) arrived[i] = 0;
    for (int i = tid; i < p.split_tiles * 4; i += kThreads) p.split_done[i] = 0;
    if (tid == 0) {
      *reinterpret_cast<uint32_t*>(self + p.lay.ret_arrived) = 0;
      *p.ticket = 0;
    }
    __syncthreads();
    for (int i = tid; i < W * E; i += kThreads) {
      const int r = i / E, e = i - r * E;
      int32_t* t = reinterpret_cast<int32_t*>(p.peers[r] + p.lay.cnt_table);
      t[(static_cast<size_t>(parity) * W + p.rank) * E + e] = p.expert_counts[e];
    }
    // the barrier orders every thread's writes above before the releases below; one release per
    // peer is the only system-wide fence of the exchange (device-wide with a single rank)
    __syncthreads();
    // (a context created with FMOE_WITHHOLD_FLAGS=1 never publishes the flags: every CTA's wait
    // below then runs out, which is how the tests exercise the bounded-wait and status path
    // without faulting anything)
    if (tid < W && !p.withhold_flags) {
      uint64_t* f = reinterpret_cast<uint64_t*>(p.peers[tid] + p.lay.cnt_flag) + parity * W + p.rank;
      if (W > 1) st_release_sys(f, flag_val); else st_release_gpu(f, flag_val);
    }
  }
  // ---- what depends on this rank's own counts only, while the other ranks' counts travel ----
  // exclusive prefix sums by one warp, 32 entries per step: emit(i, sum of values before i)
  auto warp_scan = [&](auto value_of, auto emit, int n) -> int {   // returns the total
    int carry = 0;
    for (int base = 0; base < n; base += 32) {
      const int i = base + lane;
      const int v = i < n ? value_of(i) : 0;
      int incl = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += u;
      }
      if (i < n) emit(i, carry + incl - v);
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    return carry;
  };
  // Send order: the experts that are in the first half of their owner's local list come first
  // (class 0), the others after them (class 1); inside a class ascending expert id.  Every warp
  // sends its share of class 0 before its share of class 1, so the rows the owners' first GEMM0
  // tickets wait for are on the wire first and the second half of the transfer overlaps compute.
  for (int e = tid; e < E; e += kThreads) {
    tb.owner[e] = p.owner[e]; tb.lidx[e] = p.lidx[e]; tb.local_e[e] = p.local_e[e];   // W * nLx == E
  }
  __syncthreads();
  auto first_class = [&](int e) { return 2 * tb.lidx[e] < nLx ? 1 : 0; };
  if (warp == 0) {
    const int e0 = warp_scan(first_class, [&](int e, int v) { tb.tmp[e] = v; }, E);
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
      const int before = tb.tmp[e];
      tb.ord[first_class(e) ? before : e0 + (e - before)] = e;
    }
    __syncwarp();
    const int sp = warp_scan([&](int i) { const int v = p.expert_counts[tb.ord[i]]; return v < p.EC ? (v < 0 ? 0 : v) : p.EC; },
                             [&](int i, int v) { tb.send_pref[i] = v; }, E);
    if (lane == 0) {
      tb.send_pref[E] = sp;
      ctl->send_rows = sp;
      ctl->class0_experts = e0;
      ctl->expected_ret = sp * tiles_n1_;   // one count per returned row and N1 tile
    }
  }
  __syncthreads();
  // One routed row: where it stands in the send order, which token it is and which of the token's
  // k choices.  Lane i of a dispatching warp looks up row (q + i): the dependent loads (routing
  // table, then the token's route records) are in flight before the counts of the peers are in.
  struct RowInfo { int pos, row; uint32_t token, choice; };
  // This CTA's share of the rows to send: a contiguous slice of class 0 and one of class 1, cut
  // into chunks of `chunk_rows` rows (at most 16) that the CTA's dispatching warps take from a
  // queue: warps 6 and 7 do nothing else, the epilogue warps 2..5 take chunks whenever no finished
  // accumulator is waiting for them.  Class 0 chunks come first in the queue.
  int cta_a0 = 0, cta_n0 = 0, cta_a1 = 0, cta_n1 = 0, chunk_rows = 1, chunks0 = 0, total_chunks = 0;
  {
    const long long R0 = tb.send_pref[ctl->class0_experts], R1 = ctl->send_rows - R0;
    const long long nc = gridDim.x, c = blockIdx.x;
    cta_a0 = static_cast<int>(R0 * c / nc); cta_n0 = static_cast<int>(R0 * (c + 1) / nc) - cta_a0;
    cta_a1 = static_cast<int>(R0 + R1 * c / nc); cta_n1 = static_cast<int>(R0 + R1 * (c + 1) / nc) - cta_a1;
    constexpr int kDispWarps = kThreads / 32 - 2;
    chunk_rows = min(16, max(1, (cta_n0 + cta_n1 + kDispWarps - 1) / kDispWarps));
    chunks0 = (cta_n0 + chunk_rows - 1) / chunk_rows;
    total_chunks = chunks0 + (cta_n1 + chunk_rows - 1) / chunk_rows;
  }
  auto chunk_range = [&](int ch, int& first, int& len) {
    if (ch < chunks0) { first = cta_a0 + ch * chunk_rows; len = min(chunk_rows, cta_a0 + cta_n0 - first); }
    else { first = cta_a1 + (ch - chunks0) * chunk_rows; len = min(chunk_rows, cta_a1 + cta_n1 - first); }
  };
  auto lookup = [&](int ch) -> RowInfo {      // lane i looks up row i of chunk ch
    RowInfo ri{0, 0, 0u, 0u};
    if (ch < total_chunks) {
      int first, len;
      chunk_range(ch, first, len);
      if (lane < len) {
        const int row = first + lane;
        int lo = 0, hi = E;  // largest position with send_pref[position] <= row
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (tb.send_pref[mid] <= row) lo = mid; else hi = mid;
        }
        const int e = tb.ord[lo];
        ri.pos = lo;
        ri.row = row;
        ri.token = p.table[static_cast<size_t>(e) * p.round_ec + (row - tb.send_pref[lo])].token;
        for (int c = 0; c < K_; ++c)
          if (p.routes[static_cast<size_t>(ri.token) * K_ + c].expert == e) { ri.choice = c; break; }
      }
    }
    return ri;
  };
  auto next_chunk = [&]() -> int {            // the next chunk nobody has taken (warp-uniform)
    int ch = 0;
    if (lane == 0) ch = atomicAdd(&ctl->next_chunk, 1);
    return __shfl_sync(0xffffffffu, ch, 0);
  };
  int my_chunk = warp >= 2 ? warp - 2 : total_chunks;
  RowInfo pre = lookup(my_chunk);             // in flight while the peers' counts travel

  if (tid < W) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(self + p.lay.cnt_flag) + parity * W + tid;
    auto poll = [&]() { return W > 1 ? ld_acquire_sys(f) : ld_acquire_gpu(f); };
    SpinGuard g;
    bool ok = true;
    while (poll() != flag_val) {
      if (g.expired(wc)) { ok = (poll() == flag_val); break; }
    }
    if (!ok) { fail(p, FMOE_PHASE_COUNTS, tid); ctl->ok = 0; }
  }
  __syncthreads();
  stamp(1);
  if (ctl->ok) {
    const int32_t* t = reinterpret_cast<const int32_t*>(self + p.lay.cnt_table) +
                       static_cast<size_t>(parity) * W * E;
    for (int i = tid; i < W * E; i += kThreads) {
      const int v = __ldcg(t + i);
      tb.n[i] = v < p.EC ? (v < 0 ? 0 : v) : p.EC;
    }
  }
  __syncthreads();
  if (ctl->ok) {
    // per expert: rows from all sources, and rows from sources below this rank
    for (int e = tid; e < E; e += kThreads) {
      int tot = 0, before = 0;
      for (int s = 0; s < W; ++s) {
        if (s == p.rank) before = tot;
        tot += tb.n[s * E + e];
      }
      tb.tot[e] = tot;
      tb.dst_row0[e] = before;
    }
  }
  __syncthreads();
  if (ctl->ok) {
    // landing-row base of every expert at its owner: that owner's experts in local order, each
    // rounded up to whole M tiles (one warp per owner rank)
    for (int r = warp; r < W; r += kThreads / 32) {
      warp_scan([&](int lx) { return (tb.tot[tb.local_e[r * nLx + lx]] + kTileM - 1) / kTileM * kTileM; },
                [&](int lx, int base) {
                  const int e = tb.local_e[r * nLx + lx];
                  tb.dst_row0[e] += base;
                  if (r == p.rank) { tb.lx_base[lx] = base; tb.lx_rows[lx] = tb.tot[e]; }
                }, nLx);
    }
  }
  __syncthreads();
  // From here on the warps part: what is left of the tables (M-tile prefix, task order) is read by
  // the scheduler only, so warp 0 builds it alone while the epilogue warps already send rows.
  if (ctl->ok && warp == 0) {
    const int mt = warp_scan([&](int lx) { return (tb.lx_rows[lx] + kTileM - 1) / kTileM; },
                             [&](int lx, int v) { tb.lx_mt0[lx] = v; }, nLx);
    if (lane == 0) tb.lx_mt0[nLx] = mt;
    __syncwarp();
    // task order: GEMM1 of expert i trails GEMM0 of expert i by `lag` experts, the smallest lag
    // whose GEMM0 tiles cover two tickets per CTA, so that by the time a GEMM1 ticket is drawn the
    // GEMM0 tiles it depends on are long finished: G0(0..lag-1), G0(lag), G1(0), G0(lag+1), G1(1), ...
    int lag = nLx;
    for (int t = 1 + lane; t < nLx; t += 32)
      if (tb.lx_mt0[t] * tiles_n0_ >= 2 * static_cast<int>(gridDim.x)) { lag = t; break; }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) lag = min(lag, __shfl_xor_sync(0xffffffffu, lag, off));
    // A ticket is a group of kGroup M tiles (one per CTA of a pair) times one N tile.  Step s of the
    // order emits G0(s) (s < nLx) and then G1(s - lag) (s >= lag); sizes go to seg_first and are
    // turned into first-ticket numbers by the scan below.
    for (int i = lane; i < nLx; i += 32) {
      const int groups = (tb.lx_mt0[i + 1] - tb.lx_mt0[i] + kGroup - 1) / kGroup;
      const int i0 = i + max(0, i - lag);                                   // G0(i)
      const int s1 = i + lag;
      const int i1 = min(s1, nLx) + i + (s1 < nLx ? 1 : 0);                 // G1(i)
      tb.seg_first[i0] = groups * tiles_n0_; tb.seg_kind[i0] = kTaskGemm0; tb.seg_lx[i0] = i;
      tb.seg_whole[i0] = groups * tiles_n0_;
      // The last `split_tiles` GEMM1 tiles of the task order (about one wave of CTAs) are cut along
      // K into `split_parts` tickets each, so that the kernel ends on short tickets: `after` tiles
      // follow this segment, so its last (split_tiles - after) tiles are cut.  Never in pair mode.
      const int tiles = groups * tiles_n1_;
      const int after = (tb.lx_mt0[nLx] - tb.lx_mt0[i + 1]) * tiles_n1_;   // kGroup == 1 when splitting
      const int cut = (kPair || p.split_parts <= 1) ? 0 : max(0, min(tiles, p.split_tiles - after));
      tb.seg_first[i1] = (tiles - cut) + cut * p.split_parts;
      tb.seg_whole[i1] = tiles - cut;
      tb.seg_kind[i1] = kTaskGemm1; tb.seg_lx[i1] = i;
    }
    __syncwarp();
    const int total = warp_scan([&](int i) { return tb.seg_first[i]; },
                                [&](int i, int v) { tb.seg_first[i] = v; }, 2 * nLx);
    if (lane == 0) {
      tb.seg_first[2 * nLx] = total;
      ctl->n_segs = 2 * nLx;
      ctl->total_tasks = total;
    }
    __syncwarp();
    stamp(2);
  }

  // ---- dispatch: push this rank's routed rows to the experts' owners --------------------
  // Done by warps 6 and 7 of every CTA and, between epilogues, by the epilogue warps; warps 0 and 1
  // are already drawing tickets and loading weights.  A GEMM0 ticket waits for the rows of its own
  // M tile only (per source, on disp_arrived) and the dispatch depends on no ticket, so the order
  // stays deadlock-free.
  // Sends the rows [a, b) of a chunk; `ri` holds the chunk's look-ups (lane i = row i of the chunk).
  auto send_rows = [&](const int a, const int b, const RowInfo ri) {
    const int vecs = H_ * EB / 16;
    const uint4* tok_base = static_cast<const uint4*>(p.tokens);
    for (int i = a; i < b; ++i) {
      const int pos = __shfl_sync(0xffffffffu, ri.pos, i);
      const int row = __shfl_sync(0xffffffffu, ri.row, i);
      const uint32_t token = __shfl_sync(0xffffffffu, ri.token, i);
      const uint32_t choice = __shfl_sync(0xffffffffu, ri.choice, i);
      const int e = tb.ord[pos];
      char* peer = p.peers[tb.owner[e]];
      const int drow = tb.dst_row0[e] + (row - tb.send_pref[pos]);
      const uint4* src = tok_base + static_cast<size_t>(token) * vecs;
      if constexpr (kPlanes == 1) {
        uint4* dst = reinterpret_cast<uint4*>(peer + p.lay.landing) + static_cast<size_t>(drow) * vecs;
        // A warp owns only a row or two, so its time is a chain of load -> store round trips:
        // twenty 16-byte loads in flight per lane make a 5120-element row one trip instead of five.
        constexpr int kDepth = 20;
        for (int w0 = lane; w0 < vecs; w0 += 32 * kDepth) {
          uint4 x[kDepth];
#pragma unroll
          for (int u = 0; u < kDepth; ++u) if (w0 + 32 * u < vecs) x[u] = __ldg(src + w0 + 32 * u);
#pragma unroll
          for (int u = 0; u < kDepth; ++u) if (w0 + 32 * u < vecs) dst[w0 + 32 * u] = x[u];
        }
      } else {
        // fp32 row -> three BF16 planes at the owner (4 floats in, 3 x 8 bytes out)
        for (int w = lane; w < vecs; w += 32) {
          const uint4 raw = __ldg(src + w);
          const float f[4] = {__uint_as_float(raw.x), __uint_as_float(raw.y), __uint_as_float(raw.z),
                              __uint_as_float(raw.w)};
          unsigned short h[4][3];
#pragma unroll
          for (int z = 0; z < 4; ++z) split3(f[z], h[z]);
#pragma unroll
          for (int pl = 0; pl < 3; ++pl) {
            uint2* dst = reinterpret_cast<uint2*>(peer + p.lay.landing + pl * landing_plane) +
                         static_cast<size_t>(drow) * vecs + w;
            *dst = make_uint2(static_cast<uint32_t>(h[0][pl]) | (static_cast<uint32_t>(h[1][pl]) << 16),
                              static_cast<uint32_t>(h[2][pl]) | (static_cast<uint32_t>(h[3][pl]) << 16));
          }
        }
      }
      if (lane == 0)
        reinterpret_cast<uint32_t*>(peer + p.lay.landing_meta)[drow] =
            (static_cast<uint32_t>(p.rank) << kMetaSrcShift) | (token * K_ + choice);
    }
    // Count the rows in at their owners, one update per expert.  Every lane's stores happen before
    // the barrier, the barrier before lane 0's fence, and that ONE fence orders them before all the
    // updates lane 0 makes after it (a fence per update would cost a trip over the link each).
    __syncwarp();
    if (lane == 0) { if (W > 1) fence_acq_rel_sys(); else fence_acq_rel_gpu(); }
    const int prev = __shfl_up_sync(0xffffffffu, ri.pos, 1);
    unsigned heads = __ballot_sync(0xffffffffu, lane >= a && lane < b && (lane == a || prev != ri.pos));
    while (heads != 0) {
      const int h = __ffs(heads) - 1;
      heads &= heads - 1;
      const int end = heads != 0 ? __ffs(heads) - 1 : b;      // the next run's first entry
      const int pos = __shfl_sync(0xffffffffu, ri.pos, h);
      if (lane == 0) {
        const int e = tb.ord[pos];
        red_add_relaxed_sys(reinterpret_cast<uint32_t*>(p.peers[tb.owner[e]] + p.lay.disp_arrived) + p.rank * nLx + tb.lidx[e],
                            static_cast<uint32_t>(end - h));
      }
    }
  };

  // ---- expert GEMMs ---------------------------------------------------------------------
  // Lone form: this CTA's 128 x 256 output tile, whole B tile per stage.  Pair form: two CTAs (a
  // cluster of 2, on the two SMs of one TPC) work on one 256 x 256 output tile: each loads its own
  // 128 rows of A and its own half of the B tile, the leader issues tcgen05.mma.cta_group::2, each
  // keeps its 128 rows of the accumulator in its own TMEM.
  const int nk0 = H_ / kTileK, nk1 = I_ / kTileK;
  // plane pairs (A plane, B plane) per K block, smallest contributions first
  constexpr int kPairs = kPlanes == 1 ? 1 : 6;
  constexpr int kBufs = kPlanes == 1 ? kAccBufs : 1;   // fp32 layers use both TMEM halves per task
  constexpr int kPairA[6] = {0, 2, 1, 0, 1, 0};
  constexpr int kPairB[6] = {2, 0, 1, 1, 0, 0};
  // ticket -> this CTA's task
  auto decode = [&](int ticket) -> Task {
    Task t{};
    t.ticket = ticket;
    if (ticket >= ctl->total_tasks) { t.kind = kTaskStop; return t; }
    int lo = 0, hi = ctl->n_segs;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tb.seg_first[mid] <= ticket) lo = mid; else hi = mid;
    }
    const int lx = tb.seg_lx[lo];
    int idx = ticket - tb.seg_first[lo];     // tile of the segment, N-major
    const int mts = tb.lx_mt0[lx + 1] - tb.lx_mt0[lx];
    const int groups = (mts + kGroup - 1) / kGroup;
    t.kind = tb.seg_kind[lo];
    t.lx = lx;
    t.nparts = 1;
    const int whole = tb.seg_whole[lo];
    if (idx >= whole) {                      // a K part of one of the segment's last tiles
      const int j = idx - whole;
      idx = whole + j / p.split_parts;
      t.part = j - (idx - whole) * p.split_parts;
      t.nparts = p.split_parts;
      const int after = (tb.lx_mt0[nLx] - tb.lx_mt0[lx + 1]) * tiles_n1_;
      t.split_idx = after + (groups * tiles_n1_ - 1 - idx);
    }
    const int n2 = idx / groups;
    t.n = n2;
    t.m_in_expert = kGroup * (idx - n2 * groups) + static_cast<int>(pair_rank);
    t.mt = tb.lx_mt0[lx] + t.m_in_expert;
    t.row0 = tb.lx_base[lx] + t.m_in_expert * kTileM;
    t.rows = max(0, min(kTileM, tb.lx_rows[lx] - t.m_in_expert * kTileM));   // 0: no such M tile
    return t;
  };

  if (ctl->ok && warp == 0) {
    if (lane == 0) {
      // scheduler (leader: draws tickets and waits for readiness) + TMA producer (both CTAs)
      uint32_t fill = 0;  // stage fills issued so far
      uint32_t tslot = 0;
      bool ok = true;
      int next_ticket = -1;   // drawn a few K blocks before the current task's loads end
      for (uint32_t it = 0; ok; ++it, tslot = (tslot + 1) % kTaskSlots) {
        const uint32_t ring_par = (it / kTaskSlots) & 1;
        int ticket;
        if (leader) {
          ticket = next_ticket >= 0 ? next_ticket : static_cast<int>(atomicAdd(p.ticket, 1u));
          next_ticket = -1;
        } else {
          if (!mbar_wait_cluster(&ctl->pair_full[tslot], ring_par, wc)) {
            fail(p, FMOE_PHASE_TASK, -3); ok = false; break;
          }
          ticket = static_cast<int>(ctl->pair_ticket[tslot]);
          if constexpr (kPair) mbar_arrive_cluster(map_to_cta(&ctl->pair_empty[tslot], 0));
        }
        const Task t = decode(ticket);
        if (leader) {
          // readiness of BOTH M tiles of the group, then hand the ticket to the follower
          if (t.kind == kTaskGemm0) {
            const int e = tb.local_e[p.rank * nLx + t.lx];
            const uint32_t* arrived = reinterpret_cast<const uint32_t*>(self + p.lay.disp_arrived);
            const int lo_row = t.m_in_expert * kTileM, hi_row = lo_row + kGroup * kTileM;
            int off = 0;
            for (int s = 0; s < W && ok; ++s) {
              const int ns = tb.n[s * E + e];
              if (ns > 0 && off < hi_row && off + ns > lo_row) {
                const bool in = W > 1 ? wait_counter_sys(arrived + s * nLx + t.lx, static_cast<uint32_t>(ns), wc)
                                      : wait_counter_gpu(arrived + s * nLx + t.lx, static_cast<uint32_t>(ns), wc);
                if (!in) {
                  fail(p, FMOE_PHASE_DISPATCH_ARRIVAL, s); ok = false;
                }
              }
              off += ns;
            }
          } else if (t.kind == kTaskGemm1) {
            const int mts = tb.lx_mt0[t.lx + 1] - tb.lx_mt0[t.lx];
            for (int q = 0; q < kGroup && ok; ++q) {
              if (t.m_in_expert + q >= mts) break;
              if (!wait_counter_gpu(p.gemm0_done + t.mt + q, static_cast<uint32_t>(4 * tiles_n0_), wc)) {
                fail(p, FMOE_PHASE_GEMM0_DONE, t.mt + q); ok = false;
              }
            }
          }
          if (!ok) break;
          if constexpr (kPair) {
            if (!mbar_wait_cluster(&ctl->pair_empty[tslot], ring_par ^ 1, wc)) {
              fail(p, FMOE_PHASE_TASK, -4); ok = false; break;
            }
            st_cluster_u32(map_to_cta(&ctl->pair_ticket[tslot], 1), static_cast<uint32_t>(ticket));
            mbar_arrive_cluster(map_to_cta(&ctl->pair_full[tslot], 1));
          }
        }
        if (!mbar_wait(&ctl->task_empty[tslot], ring_par ^ 1, wc)) {
          fail(p, FMOE_PHASE_TASK, ticket); ok = false; break;
        }
        ctl->tasks[tslot] = t;
        mbar_arrive(&ctl->task_full[tslot]);
        if (t.kind == kTaskStop) { stamp(4); break; }
        fence_proxy_async();

        const bool g0 = t.kind == kTaskGemm0;
        const int nk = g0 ? nk0 : nk1;
        const CUtensorMap* map_a = g0 ? &maps.landing : &maps.y;
        // the B tile as two halves of 128 rows: GEMM0 gated = gate rows | up rows.  In a pair the
        // leader loads the first half and the follower the second; alone, a CTA loads both.
        const CUtensorMap* map_b0 = g0 ? &maps.up : &maps.down;
        const CUtensorMap* map_b1 = g0 ? (gated_ ? &maps.up_v : &maps.up) : &maps.down;
        int brow0, brow1;
        if (g0) {
          if (gated_) { brow0 = t.lx * I_ + t.n * 128; brow1 = brow0; }
          else { brow0 = t.lx * I_ + t.n * 256; brow1 = brow0 + 128; }
        } else {
          brow0 = t.lx * H_ + t.n * kUmmaN; brow1 = brow0 + 128;
        }
        const CUtensorMap* map_b = leader ? map_b0 : map_b1;
        const int brow = leader ? brow0 : brow1;
        const int b_plane_rows = g0 ? nLx * I_ : nLx * H_;   // rows of one BF16 plane of the weights
        const int kb_begin = nk * t.part / t.nparts, kb_end = nk * (t.part + 1) / t.nparts;
        for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
          // the next ticket is drawn while the last stages of this task are still being consumed,
          // so the atomic's round trip is off the path between two tasks (not earlier: a CTA
          // holding a spare ticket for long would unbalance the closing wave)
          if (leader && kb == max(kb_begin, kb_end - 6)) next_ticket = static_cast<int>(atomicAdd(p.ticket, 1u));
          for (int pp = 0; pp < kPairs; ++pp, ++fill) {
            const int pa = kPlanes == 1 ? 0 : kPairA[pp], pb = kPlanes == 1 ? 0 : kPairB[pp];
            const uint32_t s = fill % NS;
            if (!mbar_wait_cluster(&ctl->empty[s], ((fill / NS) & 1) ^ 1, wc)) {
              fail(p, FMOE_PHASE_PIPE_EMPTY, ticket); ok = false; break;
            }
            uint8_t* sa = stages + s * STAGE;
            uint8_t* sb = sa + SA;
            if constexpr (kPair) {
              // the leader's barrier counts the bytes of both CTAs
              if (leader) mbar_expect_tx(&ctl->full[s], 2 * STAGE);
              tma_load_2d_pair(sa, map_a, &ctl->full[s], kb * kTileK, t.row0 + pa * p.landing_rows);
              tma_load_2d_pair(sb, map_b, &ctl->full[s], kb * kTileK, brow + pb * b_plane_rows);
            } else {
              mbar_expect_tx(&ctl->full[s], STAGE);
              tma_load_2d(sa, map_a, &ctl->full[s], kb * kTileK, t.row0 + pa * p.landing_rows);
              tma_load_2d(sb, map_b0, &ctl->full[s], kb * kTileK, brow0 + pb * b_plane_rows);
              tma_load_2d(sb + SB / 2, map_b1, &ctl->full[s], kb * kTileK, brow1 + pb * b_plane_rows);
            }
          }
        }
      }
      if (!ok) {
        // let the copies already in flight land before this CTA's shared memory goes away: the
        // leader can watch its barriers (bounded), the follower allows the same time to pass
        const long long t_start = clock_now();
        if (leader) {
          const uint32_t first = fill > NS ? fill - NS : 0;
          for (uint32_t f = first; f < fill; ++f)
            while (!mbar_try_wait_cluster(&ctl->full[f % NS], (f / NS) & 1) &&
                   clock_now() - t_start < 2000000LL) {}
        } else {
          while (clock_now() - t_start < 2000000LL) {}
        }
      }
    }
  } else if (ctl->ok && warp == 1) {
    if (lane == 0 && leader) {
      const uint32_t idesc = umma_idesc_f16(Cvt<T>::kFormat, kGroup * kTileM, kUmmaN);
      uint32_t fill = 0, tslot = 0, acc_it = 0;
      for (uint32_t it = 0;; ++it, tslot = (tslot + 1) % kTaskSlots) {
        if (!mbar_wait(&ctl->task_full[tslot], (it / kTaskSlots) & 1, wc)) {
          fail(p, FMOE_PHASE_TASK, -1); break;
        }
        const Task t = ctl->tasks[tslot];
        mbar_arrive(&ctl->task_empty[tslot]);
        if (t.kind == kTaskStop) break;
        const int nkb = t.kind == kTaskGemm0 ? nk0 : nk1;   // this ticket's K blocks: the task's, or one part of them
        const int nk = (nkb * (t.part + 1) / t.nparts - nkb * t.part / t.nparts) * kPairs;
        const uint32_t buf = acc_it % kBufs;
        if (!mbar_wait_cluster(&ctl->acc_empty[buf], ((acc_it / kBufs) & 1) ^ 1, wc)) {
          fail(p, FMOE_PHASE_TMEM_EMPTY, t.mt); break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = ctl->tmem_base + buf * kUmmaN;
        const uint32_t d_corr = ctl->tmem_base + kUmmaN;   // fp32 layers only (single-buffered there)
        bool ok = true;
        for (int kb = 0; kb < nk; ++kb, ++fill) {
          const uint32_t s = fill % NS;
          if (!mbar_wait_cluster(&ctl->full[s], (fill / NS) & 1, wc)) {
            fail(p, FMOE_PHASE_PIPE_FULL, t.mt); ok = false; break;
          }
          tc_fence_after_sync();
          if (fill == 0) stamp_now(8);
          const uint32_t a_addr = smem_u32(stages + s * STAGE);
          const uint32_t b_addr = a_addr + SA;
          // fp32 layers: the last pair of every K block is the leading one (planes 0 x 0)
          const bool lead = kPlanes == 1 || (kb % kPairs) == kPairs - 1;
          const uint32_t d = lead ? d_tmem : d_corr;
          const bool first = lead ? (kb < kPairs) : (kb == 0);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) {
            const uint64_t da = umma_desc_sw128(a_addr + k * 32), db = umma_desc_sw128(b_addr + k * 32);
            if constexpr (kPair) umma_f16_pair(d, da, db, idesc, (!first || k > 0) ? 1u : 0u);
            else umma_f16(d, da, db, idesc, (!first || k > 0) ? 1u : 0u);
          }
          if constexpr (kPair) umma_commit_pair(&ctl->empty[s], 3);    // frees the stage in both CTAs
          else umma_commit(&ctl->empty[s]);
        }
        if (!ok) break;
        // this CTA's (both CTAs') epilogue warps may read their rows of the accumulator
        if constexpr (kPair) umma_commit_pair(&ctl->acc_full[buf], 3);
        else umma_commit(&ctl->acc_full[buf]);
        ++acc_it;
      }
    }
  } else if (ctl->ok && warp >= 6) {
    // dispatch warps: chunks of this CTA's rows until the queue is empty
    RowInfo cur = pre;
    while (my_chunk < total_chunks) {
      int first, len;
      chunk_range(my_chunk, first, len);
      send_rows(0, len, cur);
      my_chunk = next_chunk();
      cur = lookup(my_chunk);
    }
    if (warp == 6 && lane == 0) stamp_now(3);
  } else if (ctl->ok) {
    // epilogue warps: TMEM lane quadrant = warp id mod 4; this CTA's 128 rows of the pair's tile.
    // They help with the dispatch for as long as no finished accumulator is waiting for them, so
    // the first rows leave on six warps per CTA and a long dispatch (many routed rows per CTA)
    // never keeps the MMA warp waiting for a free TMEM buffer.
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    uint32_t acc_empty_leader = 0;
    if constexpr (kPair) acc_empty_leader = map_to_cta(&ctl->acc_empty[0], 0);
    uint32_t tslot = 0, acc_it = 0;
    RowInfo cur = pre;               // look-ups of the chunk this warp holds (my_chunk)
    for (uint32_t it = 0;; ++it, tslot = (tslot + 1) % kTaskSlots) {
      while (my_chunk < total_chunks) {
        // lane 0 looks: is the next task known, and (unless it is the stop task) its accumulator full?
        int ready = 0;
        if (lane == 0 && mbar_try_wait(&ctl->task_full[tslot], (it / kTaskSlots) & 1)) {
          const uint32_t b = acc_it % kBufs;
          ready = ctl->tasks[tslot].kind != kTaskStop &&
                  mbar_try_wait_cluster(&ctl->acc_full[b], (acc_it / kBufs) & 1);
        }
        if (__shfl_sync(0xffffffffu, ready, 0)) break;
        int first, len;
        chunk_range(my_chunk, first, len);
        send_rows(0, len, cur);
        my_chunk = next_chunk();
        cur = lookup(my_chunk);
      }
      if (!mbar_wait(&ctl->task_full[tslot], (it / kTaskSlots) & 1, wc)) {
        fail(p, FMOE_PHASE_TASK, -2); break;
      }
      const Task t = ctl->tasks[tslot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->task_empty[tslot]);
      if (t.kind == kTaskStop) break;
      const uint32_t buf = acc_it % kBufs;
      if (!mbar_wait_cluster(&ctl->acc_full[buf], (acc_it / kBufs) & 1, wc)) {
        fail(p, FMOE_PHASE_TMEM_FULL, t.mt); break;
      }
      tc_fence_after_sync();
      if (warp == 2 && lane == 0) stamp_now(9);
      const uint32_t taddr = ctl->tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * kUmmaN;
      const bool valid = row_in_tile < t.rows;
      const int row = t.row0 + row_in_tile;
      // hands this warp's quarter of the accumulator back to the leader's MMA thread; called right
      // after the last TMEM load of the task, before the remaining math and stores
      auto release_acc = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) mbar_arrive_cluster(acc_empty_leader + buf * static_cast<uint32_t>(sizeof(uint64_t)));
          else mbar_arrive(&ctl->acc_empty[buf]);
        }
      };

      if (t.kind == kTaskGemm0) {
        char* yrow = static_cast<char*>(p.y) + static_cast<size_t>(row) * I_ * 2;
        if (gated_) {
          const int col_base = t.n * 128;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t g[32], u[32];
            __syncwarp();
            tmem_ld_32x32(taddr + c * 32, g);
            tmem_ld_32x32(taddr + 128 + c * 32, u);
            tmem_ld_wait();
            if constexpr (kPlanes == 3) {
              uint32_t cg[32], cu[32];
              tmem_ld_32x32(taddr + kUmmaN + c * 32, cg);
              tmem_ld_32x32(taddr + kUmmaN + 128 + c * 32, cu);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                g[i] = __float_as_uint(__uint_as_float(g[i]) + __uint_as_float(cg[i]));
                u[i] = __float_as_uint(__uint_as_float(u[i]) + __uint_as_float(cu[i]));
              }
            }
            if (c == 3) release_acc();
            const int col0 = col_base + c * 32;
            if (valid && col0 < I_) {
              float y[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const size_t bi = static_cast<size_t>(t.lx) * I_ + col0 + i;
                const float gate = (__uint_as_float(g[i]) + bias_at<T>(p.bias_up, bi)) * p.beta;
                const float tt = Cvt<T>::round(p.alpha * activate_t<EB == 4>(gate, act_));
                const float v = __uint_as_float(u[i]) + bias_at<T>(p.bias_up_v, bi);
                y[i] = v * tt;
              }
              store_operand32<T>(yrow, col0, y, y_plane);
            }
          }
        } else {
          const int col_base = t.n * 256;
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t a[32];
            __syncwarp();
            tmem_ld_32x32(taddr + c * 32, a);
            tmem_ld_wait();
            if constexpr (kPlanes == 3) {
              uint32_t ca[32];
              tmem_ld_32x32(taddr + kUmmaN + c * 32, ca);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) + __uint_as_float(ca[i]));
            }
            if (c == 7) release_acc();
            const int col0 = col_base + c * 32;
            if (valid && col0 < I_) {
              float y[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const size_t bi = static_cast<size_t>(t.lx) * I_ + col0 + i;
                y[i] = activate_t<EB == 4>(__uint_as_float(a[i]) + bias_at<T>(p.bias_up, bi), act_);
              }
              store_operand32<T>(yrow, col0, y, y_plane);
            }
          }
        }
        // every lane's stores happen before the barrier, the barrier before lane 0's release
        __syncwarp();
        if (lane == 0 && t.rows > 0) red_add_release_gpu(p.gemm0_done + t.mt, 1u);
      } else {
        // GEMM1.  A tile of the closing wave arrives as `nparts` tickets, one per K range: every
        // part parks its fp32 partial sums (column quad j of chunk c, row r at float4 index
        // (8 c + j) * 128 + r, so that a warp moves whole 512-byte lines) and counts itself in; the
        // part that counts in last adds all of them up in part order, whichever it is, and
        // finishes the tile.  Nobody waits for anybody, and the sum does not depend on who was last.
        const bool split = t.nparts > 1;
        constexpr int kTileFloats = kTileM * kUmmaN;
        bool finish = true;
        if (split) {
          float4* mine = reinterpret_cast<float4*>(
                             p.split_scratch + (static_cast<size_t>(t.split_idx) * p.split_parts + t.part) * kTileFloats) +
                         row_in_tile;
#pragma unroll 1
          for (int c = 0; c < kUmmaN / 32; ++c) {
            uint32_t a[32];
            __syncwarp();
            tmem_ld_32x32(taddr + c * 32, a);
            tmem_ld_wait();
            if constexpr (kPlanes == 3) {
              uint32_t ca[32];
              tmem_ld_32x32(taddr + kUmmaN + c * 32, ca);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) + __uint_as_float(ca[i]));
            }
            if (c == kUmmaN / 32 - 1) release_acc();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              __stcg(mine + (c * 8 + j) * kTileM,
                     make_float4(__uint_as_float(a[4 * j]), __uint_as_float(a[4 * j + 1]),
                                 __uint_as_float(a[4 * j + 2]), __uint_as_float(a[4 * j + 3])));
          }
          // every lane's stores happen before the barrier, the barrier before lane 0's release;
          // lane 0's acquire before the second barrier, that barrier before every lane's loads
          __syncwarp();
          uint32_t before = 0;
          if (lane == 0) before = atom_add_acq_rel_gpu(p.split_done + t.split_idx * 4 + quad, 1u);
          before = __shfl_sync(0xffffffffu, before, 0);
          __syncwarp();
          finish = before == static_cast<uint32_t>(t.nparts - 1);
        }
        if (finish) {
          uint32_t meta = 0;
          if (valid) meta = __ldcg(reinterpret_cast<const uint32_t*>(self + p.lay.landing_meta) + row);
          const int src = static_cast<int>(meta >> kMetaSrcShift);
          const uint32_t ret_row = meta & ((1u << kMetaSrcShift) - 1);
          char* orow = p.peers[valid ? src : p.rank] + p.lay.ret + static_cast<size_t>(ret_row) * H_ * EB;
          const int col_base = t.n * kUmmaN;
          const float4* parts = reinterpret_cast<const float4*>(
                                    p.split_scratch + static_cast<size_t>(t.split_idx) * p.split_parts * kTileFloats) +
                                row_in_tile;
          // Bias, rounding, and the row's 32 columns on their way to the token's owner.  A lane holds
          // 32 columns of ITS row, so a warp-wide store straight from registers would be 32 pieces of
          // 16 bytes in 32 different rows, which is the worst shape for a write that may cross
          // NVLink.  128 bytes of every row (two chunks of a 16-bit type, one of fp32) are transposed
          // through 2 KB of shared memory instead (16-byte pieces, xor-swizzled against bank
          // conflicts) and leave as 128-byte runs of one row each, four rows per instruction.
          uint4* stage_w = ret_stage + (warp - 2) * 128;
          const uint32_t orow_lo = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(orow));
          const uint32_t orow_hi = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(orow) >> 32);
          auto row_ptr = [&](int r) -> char* {      // row r's destination, from the lane that owns it
            const uint32_t lo = __shfl_sync(0xffffffffu, orow_lo, r), hi = __shfl_sync(0xffffffffu, orow_hi, r);
            return reinterpret_cast<char*>((static_cast<uintptr_t>(hi) << 32) | lo);
          };
          // 128 bytes of every row of the warp (32 words per lane) out through the 2 KB stage, 16
          // rows at a time: every store instruction writes four whole 128-byte runs.
          auto stage_out = [&](const uint32_t (&w)[32], size_t byte_off) {
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
              if ((lane >> 4) == pass) {
                const int r16 = lane & 15;
                uint4* mine = stage_w + r16 * 8;
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  mine[q ^ (r16 & 7)] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
              }
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int r16 = 4 * i + (lane >> 3), piece = lane & 7, r = pass * 16 + r16;
                const uint4 v = stage_w[r16 * 8 + (piece ^ (r16 & 7))];
                char* dst = row_ptr(r);
                const bool ok = __shfl_sync(0xffffffffu, valid ? 1 : 0, r) != 0;
                if (ok) *reinterpret_cast<uint4*>(dst + byte_off + piece * 16) = v;
              }
              __syncwarp();
            }
          };
          uint32_t held[16];   // 16-bit types: the even chunk of a pair waits here for the odd one
          auto finish_chunk = [&](int c, float (&o)[32]) {   // every lane of the warp calls this, c ascending
            const int col0 = col_base + c * 32;
            if (col0 >= H_) return;                            // H is a multiple of 64: whole pairs
            if (valid) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                o[i] += bias_at<T>(p.bias_down, static_cast<size_t>(t.lx) * H_ + col0 + i);
            }
            if constexpr (EB == 2) {
              if ((c & 1) == 0) {
#pragma unroll
                for (int i = 0; i < 16; ++i) held[i] = Cvt<T>::pack(o[2 * i], o[2 * i + 1]);
              } else {
                uint32_t w[32];
#pragma unroll
                for (int i = 0; i < 16; ++i) { w[i] = held[i]; w[16 + i] = Cvt<T>::pack(o[2 * i], o[2 * i + 1]); }
                stage_out(w, static_cast<size_t>(col0 - 32) * 2);
              }
            } else {
              uint32_t w[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(o[i]);
              stage_out(w, static_cast<size_t>(col0) * 4);
            }
          };
          if (!split) {
#pragma unroll 1
            for (int c = 0; c < kUmmaN / 32; ++c) {
              uint32_t a[32];
              __syncwarp();
              tmem_ld_32x32(taddr + c * 32, a);
              tmem_ld_wait();
              if constexpr (kPlanes == 3) {
                uint32_t ca[32];
                tmem_ld_32x32(taddr + kUmmaN + c * 32, ca);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) + __uint_as_float(ca[i]));
              }
              if (c == kUmmaN / 32 - 1) release_acc();
              float o[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(a[i]);
              finish_chunk(c, o);
            }
          } else {
            // two chunks per step: the parked sums of both are in flight before either is added up
            // (rows past the tile's end read parked garbage that is never stored)
#pragma unroll 1
            for (int c = 0; c < kUmmaN / 32; c += 2) {
              float o[2][32];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float4 v = __ldcg(parts + ((c + h) * 8 + j) * kTileM);
                  o[h][4 * j] = v.x; o[h][4 * j + 1] = v.y; o[h][4 * j + 2] = v.z; o[h][4 * j + 3] = v.w;
                }
              }
              for (int pp = 1; pp < t.nparts; ++pp) {
                const float4* q = parts + static_cast<size_t>(pp) * (kTileFloats / 4);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const float4 v = __ldcg(q + ((c + h) * 8 + j) * kTileM);
                    o[h][4 * j] = __fadd_rn(o[h][4 * j], v.x); o[h][4 * j + 1] = __fadd_rn(o[h][4 * j + 1], v.y);
                    o[h][4 * j + 2] = __fadd_rn(o[h][4 * j + 2], v.z); o[h][4 * j + 3] = __fadd_rn(o[h][4 * j + 3], v.w);
                  }
                }
              }
              finish_chunk(c, o[0]);
              finish_chunk(c + 1, o[1]);
            }
          }
          if (warp == 2 && lane == 0) stamp_now(10);
          // Tell every owner how many of its rows this warp just delivered: every lane's stores
          // happen before the barrier, the barrier before lane 0's fence, and ONE fence orders them
          // before all the counter updates that follow (a release per update would pay the
          // system-wide fence once per source rank).
          __syncwarp();
          if (lane == 0) { if (W > 1) fence_acq_rel_sys(); else fence_acq_rel_gpu(); }
          for (int s = 0; s < W; ++s) {
            const unsigned b = __ballot_sync(0xffffffffu, valid && src == s);
            if (lane == 0 && b != 0)
              red_add_relaxed_sys(reinterpret_cast<uint32_t*>(p.peers[s] + p.lay.ret_arrived),
                                  static_cast<uint32_t>(__popc(b)));
          }
        }
      }
      if (warp == 2 && lane == 0) stamp_now(11);
      ++acc_it;
    }
  }

  // ---- combine: this rank's tokens, fp32 sum over the k returned rows -------------------
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  stamp(5);
  if (tid == 0 && ctl->ok && *reinterpret_cast<volatile uint32_t*>(p.abort_word) == 0) {
    const uint32_t* ra = reinterpret_cast<const uint32_t*>(self + p.lay.ret_arrived);
    const bool in = W > 1 ? wait_counter_sys(ra, static_cast<uint32_t>(ctl->expected_ret), wc)
                          : wait_counter_gpu(ra, static_cast<uint32_t>(ctl->expected_ret), wc);
    if (!in) {
      fail(p, FMOE_PHASE_RETURN_ARRIVAL, ctl->expected_ret);
      ctl->ok = 0;
    }
  }
  __syncthreads();
  stamp(6);
  if (ctl->ok && *reinterpret_cast<volatile uint32_t*>(p.abort_word) == 0) {
    const int G = gridDim.x * (kThreads / 32);
    const int vecs = H_ * EB / 16;
    const uint4* ret = reinterpret_cast<const uint4*>(self + p.lay.ret);
    uint4* out = static_cast<uint4*>(p.out);
    constexpr int kPer = 16 / EB;   // elements per 16-byte vector
    for (int tkn = blockIdx.x * (kThreads / 32) + warp; tkn < p.S; tkn += G) {
      // lane j holds the token's j-th route; a dropped pair gets weight-slot -1
      Route mine{0, p.EC, 0.0f, 0};
      if (lane < K_) mine = p.routes[static_cast<size_t>(tkn) * K_ + lane];
      const unsigned live = __ballot_sync(0xffffffffu, lane < K_ && mine.slot < p.EC);
      if (K_ == 1) {
        if (live & 1u) {
          const uint4* src = ret + static_cast<size_t>(tkn) * vecs;
          uint4* dst = out + static_cast<size_t>(tkn) * vecs;
          for (int v0 = lane; v0 < vecs; v0 += 128) {   // four loads in flight per lane
            uint4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) if (v0 + 32 * u < vecs) x[u] = __ldcg(src + v0 + 32 * u);
#pragma unroll
            for (int u = 0; u < 4; ++u) if (v0 + 32 * u < vecs) dst[v0 + 32 * u] = x[u];
          }
        }
      } else {
        for (int v0 = lane; v0 < vecs; v0 += 64) {      // two vectors x k rows in flight per lane
          float acc[2][kPer];
#pragma unroll
          for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int i = 0; i < kPer; ++i) acc[u][i] = 0.0f;
          // rows of four choices are fetched together (eight loads in flight per lane), then
          // accumulated in choice order.  (No warp shuffle in here: with H < 256 only some lanes
          // run this loop.)
          for (int j0 = 0; j0 < K_; j0 += 4) {
            uint4 x[4][2];
            float wj[4];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const int j = j0 + jj;
              wj[jj] = 0.0f;
              if (j < K_ && ((live >> j) & 1u)) {
                wj[jj] = p.routes[static_cast<size_t>(tkn) * K_ + j].weight;
                const uint4* src = ret + (static_cast<size_t>(tkn) * K_ + j) * vecs;
#pragma unroll
                for (int u = 0; u < 2; ++u) if (v0 + 32 * u < vecs) x[jj][u] = __ldcg(src + v0 + 32 * u);
              }
            }
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const int j = j0 + jj;
              if (!(j < K_ && ((live >> j) & 1u))) continue;
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const uint32_t w4[4] = {x[jj][u].x, x[jj][u].y, x[jj][u].z, x[jj][u].w};
                if constexpr (EB == 2) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    acc[u][2 * i] = __fadd_rn(acc[u][2 * i], __fmul_rn(Cvt<T>::up(w4[i] & 0xffffu), wj[jj]));
                    acc[u][2 * i + 1] = __fadd_rn(acc[u][2 * i + 1], __fmul_rn(Cvt<T>::up(w4[i] >> 16), wj[jj]));
                  }
                } else {
#pragma unroll
                  for (int i = 0; i < 4; ++i)
                    acc[u][i] = __fadd_rn(acc[u][i], __fmul_rn(__uint_as_float(w4[i]), wj[jj]));
                }
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            if (v0 + 32 * u >= vecs) continue;
            uint4 o;
            if constexpr (EB == 2) {
              o = make_uint4(Cvt<T>::pack(acc[u][0], acc[u][1]), Cvt<T>::pack(acc[u][2], acc[u][3]),
                             Cvt<T>::pack(acc[u][4], acc[u][5]), Cvt<T>::pack(acc[u][6], acc[u][7]));
            } else {
              o = make_uint4(__float_as_uint(acc[u][0]), __float_as_uint(acc[u][1]), __float_as_uint(acc[u][2]),
                             __float_as_uint(acc[u][3]));
            }
            out[static_cast<size_t>(tkn) * vecs + v0 + 32 * u] = o;
          }
        }
      }
    }
  }

  // ---- leave ------------------------------------------------------------------------------
  stamp(7);
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();   // the peer no longer touches this CTA's barriers, tiles or TMEM
  tc_fence_after_sync();
  if (warp == 1) {
    if constexpr (kPair) tmem_dealloc_pair(ctl->tmem_base, 512);
    else tmem_dealloc(ctl->tmem_base, 512);
  }
  if (tid == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(p.done_ctas, 1u);
    if (prev == gridDim.x - 1) {
      *p.done_ctas = 0;
      *p.grid_bar = 0ull;
      *p.epoch = epoch + 1;
      p.status->epoch = epoch + 1;
    }
  }
}

// The generic build reads the layer's shape from the launch parameters.  A specialised build
// (-DFMOE_SPEC, one per model description, the counterpart of the reference's per-model JIT
// module, flashmoe/bindings.py:34-46) fixes H, I, top-k, the MLP type and the activation at compile
// time: loop bounds and the epilogue's branches fold away.
struct GenericSpec {
  static constexpr bool kFixed = false;
  static constexpr int kH = 0, kI = 0, kTopK = 0, kAct = 0;
  static constexpr bool kGated = false;
};
#ifdef FMOE_SPEC
struct FixedSpec {
  static constexpr bool kFixed = true;
  static constexpr int kH = FMOE_SPEC_H, kI = FMOE_SPEC_I, kTopK = FMOE_SPEC_K, kAct = FMOE_SPEC_ACT;
  static constexpr bool kGated = FMOE_SPEC_GATED != 0;
};
using KernelSpec = FixedSpec;
#else
using KernelSpec = GenericSpec;
#endif

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
moe_forward_kernel_pair(const __grid_constant__ MoeParams p, const __grid_constant__ TmaMaps maps) {
  moe_forward_body<T, true, KernelSpec>(p, maps);
}
template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
moe_forward_kernel(const __grid_constant__ MoeParams p, const __grid_constant__ TmaMaps maps) {
  moe_forward_body<T, false, KernelSpec>(p, maps);
}

}  // namespace

size_t moe_smem_bytes(int W, int E, int nLx) {
  return 1024 + static_cast<size_t>(4) * 3 * kStageABytes + kRetStageBytes + sizeof(Control) +
         tables_ints(W, E, nLx) * sizeof(int) + 64;
}

#ifdef FMOE_SPEC
// a specialised build holds exactly one kernel: its element type and its form (alone / pairs)
#if FMOE_SPEC_DT == 2
using SpecElement = float;
#elif FMOE_SPEC_DT == 1
using SpecElement = __half;
#else
using SpecElement = __nv_bfloat16;
#endif
#if FMOE_SPEC_PAIR
#define FMOE_SPEC_KERNEL moe_forward_kernel_pair<SpecElement>
#else
#define FMOE_SPEC_KERNEL moe_forward_kernel<SpecElement>
#endif
#endif

cudaError_t moe_prepare_kernel(size_t smem) {
  const int n = static_cast<int>(smem);
  cudaError_t e = cudaSuccess;
  auto set = [&](auto kern) { if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, n); };
#ifdef FMOE_SPEC
  set(FMOE_SPEC_KERNEL);
#else
  set(moe_forward_kernel<__nv_bfloat16>); set(moe_forward_kernel<__half>); set(moe_forward_kernel<float>);
  set(moe_forward_kernel_pair<__nv_bfloat16>); set(moe_forward_kernel_pair<__half>); set(moe_forward_kernel_pair<float>);
#endif
  return e;
}

namespace {
// fp32 [n] -> three BF16 planes [3][n] (see Cvt<float>)
__global__ void split_planes_kernel(const float* __restrict__ in, unsigned short* __restrict__ out, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    unsigned short q[3];
    split3(__ldg(in + i), q);
    out[i] = q[0]; out[n + i] = q[1]; out[2 * n + i] = q[2];
  }
}
}  // namespace

long long spin_limit_cycles(double ms, int device) {
  int khz = 0;
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device) != cudaSuccess || khz <= 0) khz = 2000000;
  return static_cast<long long>(ms * static_cast<double>(khz));
}

cudaError_t launch_split_planes(const float* in, void* out, size_t n, cudaStream_t stream) {
  const int threads = 256;
  const size_t want = (n + threads - 1) / threads;
  const int blocks = static_cast<int>(want < 148 * 16 ? (want ? want : 1) : 148 * 16);
  split_planes_kernel<<<blocks, threads, 0, stream>>>(in, static_cast<unsigned short*>(out), n);
  ++g_launches;
  return cudaGetLastError();
}

// The kernel's CTAs wait on one another (count flags, arrival counters, tickets), so all of them
// must be resident at once.  A cooperative launch makes that a guarantee: the grid starts only
// when every CTA has an SM, whatever else the device is running, and a grid that could never fit
// is refused at launch instead of timing out in its first wait.
cudaError_t launch_moe(const MoeParams& p, const CUtensorMap* maps, int grid, size_t smem,
                       cudaStream_t stream) {
  TmaMaps m;
  m.landing = maps[0]; m.y = maps[1]; m.up = maps[2]; m.up_v = maps[3]; m.down = maps[4];
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
#ifdef FMOE_SPEC
  e = cudaLaunchKernelEx(&cfg, FMOE_SPEC_KERNEL, p, m);
#else
  if (p.pair) {
    if (p.elem_bytes == 4) e = cudaLaunchKernelEx(&cfg, moe_forward_kernel_pair<float>, p, m);
    else if (p.ab_format == 1) e = cudaLaunchKernelEx(&cfg, moe_forward_kernel_pair<__nv_bfloat16>, p, m);
    else e = cudaLaunchKernelEx(&cfg, moe_forward_kernel_pair<__half>, p, m);
  } else {
    if (p.elem_bytes == 4) e = cudaLaunchKernelEx(&cfg, moe_forward_kernel<float>, p, m);
    else if (p.ab_format == 1) e = cudaLaunchKernelEx(&cfg, moe_forward_kernel<__nv_bfloat16>, p, m);
    else e = cudaLaunchKernelEx(&cfg, moe_forward_kernel<__half>, p, m);
  }
#endif
  return e;
}

}  // namespace fmoe

#ifdef FMOE_SPEC
// What a specialised library exports (loaded by fmoe_ctx_load_specialised): its constants, so the
// host can check them against the context, and the two calls that replace the generic ones.
extern "C" {
int fmoe_spec_info(int32_t* out8) {
  out8[0] = FMOE_SPEC_H; out8[1] = FMOE_SPEC_I; out8[2] = FMOE_SPEC_K; out8[3] = FMOE_SPEC_GATED;
  out8[4] = FMOE_SPEC_ACT; out8[5] = FMOE_SPEC_DT; out8[6] = FMOE_SPEC_PAIR;
  out8[7] = static_cast<int32_t>(sizeof(fmoe::MoeParams));
  return 0;
}
int fmoe_spec_prepare(size_t smem) { return static_cast<int>(fmoe::moe_prepare_kernel(smem)); }
int fmoe_spec_launch(const void* params, const void* maps, int grid, size_t smem, void* stream) {
  return static_cast<int>(fmoe::launch_moe(*static_cast<const fmoe::MoeParams*>(params),
                                           static_cast<const CUtensorMap*>(maps), grid, smem,
                                           static_cast<cudaStream_t>(stream)));
}
}
#endif
