// Structures shared by the host code and the kernels.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/flashmoe_b200.h"

namespace fmoe {

// One routing-table entry, the reference's TPS (csrc/include/flashmoe/infra/packed.cuh:8-11).
struct __align__(8) TokenSlot {
  uint32_t token;
  float weight;
};

// Per (token, choice) record the router leaves for the combine step: which expert, which slot
// of that expert's routing-table row (slot >= EC means the pair was dropped), which weight.
struct __align__(16) Route {
  int32_t expert;
  int32_t slot;
  float weight;
  int32_t pad;
};

constexpr int kTileM = 128;      // rows of an expert's batch per CTA (a CTA pair covers 256)
constexpr int kTileK = 64;       // 64 x 16-bit = one 128-byte swizzle span
constexpr int kUmmaN = 256;      // UMMA N: gate|up halves for GEMM0, 256 output columns for GEMM1
// TMA -> UMMA ring: 6 stages of 32 KB per CTA in pair mode, 4 stages of 48 KB alone (192 KB both)
constexpr int kAccBufs = 2;      // TMEM accumulator double buffer (2 x 256 columns)
constexpr int kTaskSlots = 4;    // task ring between the scheduler warp and its consumers
constexpr int kThreads = 256;    // warp 0 scheduler + TMA, warp 1 UMMA, warps 2..5 epilogue (+ dispatch), warps 6..7 dispatch
constexpr uint32_t kStageABytes = kTileM * kTileK * 2;        // 128 rows x 64 columns of 16-bit: 16 KB

constexpr int kTraceSlots = 16;   // phase stamps per CTA
constexpr uint32_t kMetaSrcShift = 26;  // landing meta = (source rank << 26) | return row

// Offsets inside a rank's symmetric block (identical on every rank).
struct SymmLayout {
  size_t cnt_table;     // int32  [2][W][E]   counts every rank published, by epoch parity
  size_t cnt_flag;      // uint64 [2][W]      epoch number that table holds
  size_t disp_arrived;  // uint32 [W][nLx]    rows landed from (source rank, local expert)
  size_t ret_arrived;   // uint32 [1]         (rows x N1 tiles) returned to this rank
  size_t landing;       // Element [landing_rows][H]  dispatched rows, packed per local expert
  size_t landing_meta;  // uint32 [landing_rows]
  size_t ret;           // Element [S*k][H]   expert outputs for this rank's (token, choice) pairs
  size_t total;
};

// Everything the persistent kernel needs; passed by value as a __grid_constant__.
struct MoeParams {
  int S, H, I, E, k, EC, round_ec;
  int W, rank, nLx;
  int gated, act, ab_format;  // ab_format: 0 fp16, 1 bf16 (fp32 layers run as BF16 planes)
  int elem_bytes;             // 2, or 4 for fp32 layers
  int pair;                   // 1: CTA pairs (cta_group::2), 0: every CTA alone
  int withhold_flags;         // 1: never publish the count flags, so that the first wait runs out (a test of the bounded waits)
  int split_parts;            // K parts per GEMM1 tile of the closing wave (1 = no tile is cut)
  int split_tiles;            // how many GEMM1 tiles, counted from the end of the task order, are cut
  long long spin_limit;       // SM clock ticks after which a device-side wait gives up
  int tiles_n0, tiles_n1;
  int landing_rows;
  int max_mtiles;
  float alpha, beta;

  const int32_t* owner;    // [E] expert -> ep rank
  const int32_t* lidx;     // [E] expert -> index among its owner's experts
  const int32_t* local_e;  // [W][nLx] -> global expert id

  char* peers[FMOE_MAX_WORLD];  // symmetric block of every rank (peers[rank] = own)
  SymmLayout lay;

  // private workspace
  void* y;                 // Element [landing_rows][I]  GEMM0 output
  uint32_t* gemm0_done;    // [max_mtiles] finished N0 tiles per M tile
  float* split_scratch;    // [split_tiles][split_parts][128 x 256] fp32 partial sums of the cut tiles
  uint32_t* split_done;    // [split_tiles][4] parts parked, per tile and epilogue warp
  uint32_t* ticket;        // next task
  uint32_t* done_ctas;
  uint64_t* epoch;         // forward number, bumped by the last CTA to leave
  uint32_t* abort_word;
  fmoe_status* status;
  unsigned long long* trace;  // [grid][kTraceSlots] %globaltimer stamps of the last forward, per CTA

  const TokenSlot* table;  // [E][round_ec]
  const Route* routes;     // [S][k]

  // Routing inside this launch (fmoe_forward_routed): non-null router_w makes the kernel open with
  // the router itself (logits, softmax, top-k, slots; same arithmetic as the router kernels) and
  // write expert_counts, the routing table and the route records before it exchanges counts.
  const void* router_w;     // [E, H] Element, or null: the router ran as launches of its own
  const float* logit_bias;  // [E] or null
  float* routing;           // [S, E] probabilities out, or null
  int32_t* counts_out;      // [E] (the same array as expert_counts)
  float* route_logits;      // [S, E] workspace of the routing phase
  unsigned long long* grid_bar;   // arrivals at the routing phase's grid barriers (zero between launches)

  // per forward
  const void* tokens;
  const int32_t* expert_counts;
  const void* bias_up;
  const void* bias_up_v;
  const void* bias_down;
  void* out;
};

struct RouterParams {
  int S, H, E, k, EC, round_ec;
  int dtype;                // FMOE_DT_*
  const void* tokens;
  const void* weights;
  const float* logit_bias;
  float* routing;           // [S, E] or null
  int32_t* topk_idx;        // [S, k] scratch
  float* topk_w;            // [S, k] scratch
  int32_t* expert_counts;   // [E]
  TokenSlot* table;         // [E][round_ec]
  Route* routes;            // [S][k]
};

cudaError_t launch_router(const RouterParams& p, cudaStream_t stream);
size_t moe_smem_bytes(int W, int E, int nLx);
cudaError_t moe_prepare_kernel(size_t smem);
long long spin_limit_cycles(double ms, int device);   // a wait limit in SM clock ticks
cudaError_t launch_split_planes(const float* in, void* out, size_t n, cudaStream_t stream);
cudaError_t launch_moe(const MoeParams& p, const CUtensorMap* maps, int grid, size_t smem,
                       cudaStream_t stream);

extern unsigned long long g_launches;

// host-side helpers shared by the translation units that export C entry points
int set_error(int code, const std::string& msg);   // records the thread's last error text
int validate_model(const fmoe_model_desc* m);

}  // namespace fmoe
