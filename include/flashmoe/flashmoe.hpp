// C++ face of libflashmoe_b200.so for code written against the reference's headers
// (csrc/include/flashmoe/flashmoe.cuh of hnts03-moreh/FlashMoE): the same namespace, type and
// function names -- flashmoe::MoEArgs, Context, GateContext, initialize, finalize,
// moe::KernelArgs, moe::forwardHost, initializeGate, gate::forward, finalizeGate -- as a
// header-only layer over the C ABI in flashmoe_b200.h.  Host code only: no CUDA, CuTe or cuBLASDx
// headers are needed to include it, and nothing here launches a kernel itself.
//
// What differs from the reference, and why:
//  * The reference fixes data type, MLP type, activation and top-k as template parameters of
//    moe::MoEConfig / forwardHost<Config, topo, act> (moe.cuh:21-44, 255-260).  One ahead-of-time
//    library takes them at run time, so they travel in LayerDesc, next to MoEArgs.
//  * MoEArgs keeps its constructor (bootstrap.cuh:50-82); the tile, thread, CTA and shared-memory
//    fields are accepted and ignored (the library chooses its own geometry).
//  * Peers are mapped through CUDA IPC instead of NVSHMEM: exportSymmetric / importSymmetric /
//    commit between initialize and the first forward (a single rank needs none of them).
//  * Errors are std::runtime_error carrying the library's message; nothing exits or traps.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "../flashmoe_b200.h"

namespace flashmoe {

using Stream = void*;  // a cudaStream_t

enum class Topology : int { NVLINK_ONLY = FMOE_TOPO_NVLINK_ONLY, MIXED = FMOE_TOPO_MIXED };
enum class MLPMatmulType : int { gated = FMOE_MLP_GATED, vanilla = FMOE_MLP_VANILLA };
enum class Activation : int { identity = FMOE_ACT_IDENTITY, silu = FMOE_ACT_SILU, gelu = FMOE_ACT_GELU,
                              relu = FMOE_ACT_RELU };
enum class ElementType : int { bf16 = FMOE_DT_BF16, fp16 = FMOE_DT_FP16, fp32 = FMOE_DT_FP32,
                               fp64 = FMOE_DT_FP64 };

// One routing-table entry (infra/packed.cuh:8-11).
struct alignas(8) TPS {
  uint32_t tokenIdx;
  float probability;
};

inline void check(int code, const char* what) {
  if (code != FMOE_OK) {
    const char* msg = fmoe_last_error();
    throw std::runtime_error(std::string(what) + ": " + ((msg && *msg) ? msg : fmoe_strerror(code)));
  }
}

// Same fields and constructor as the reference's MoEArgs (bootstrap.cuh:50-82).
struct MoEArgs {
  const size_t elementBytes;
  const unsigned sequenceLength;
  const size_t EC;
  const unsigned tokenDim, ffnIntermediateSize;
  const unsigned bM, bN0, bN1, bK0, bK1, threads, blocks, smemSize;  // ignored
  const uint16_t epRank, epWorld, myPE;
  const size_t numExperts;
  const uint16_t numLocalExperts;
  const Topology topo;
  MoEArgs(size_t eb, unsigned S, unsigned H, unsigned I, size_t ec, unsigned bm, unsigned bn0, unsigned bn1,
          unsigned bk0, unsigned bk1, unsigned threads_, unsigned ctas, unsigned sharedSize, uint16_t ep_rank,
          uint16_t ep_world, uint16_t mype, uint16_t experts, uint16_t nlx, Topology topo_)
      : elementBytes(eb), sequenceLength(S), EC(ec), tokenDim(H), ffnIntermediateSize(I), bM(bm), bN0(bn0),
        bN1(bn1), bK0(bk0), bK1(bk1), threads(threads_), blocks(ctas), smemSize(sharedSize), epRank(ep_rank),
        epWorld(ep_world), myPE(mype), numExperts(experts), numLocalExperts(nlx), topo(topo_) {}
};

// Run-time form of the reference's compile-time MoEConfig parameters (moe.cuh:21-44).
struct LayerDesc {
  ElementType element = ElementType::bf16;
  MLPMatmulType mlp = MLPMatmulType::gated;
  Activation act = Activation::silu;
  int topK = 1;
  int deviceId = 0;
};

// What the reference returns by value from initialize (context.cuh:16-52); here a handle plus the
// fields callers read.
struct Context {
  fmoe_ctx* handle = nullptr;
  TPS* tokenIndices = nullptr;  // [E, roundEC]
  unsigned S = 0, H = 0, I = 0, EC = 0;
  uint16_t nLx = 0, E = 0, world = 0, epRank = 0, myPE = 0;
  Topology topo = Topology::NVLINK_ONLY;
};

struct GateContext {
  fmoe_router* handle = nullptr;
};

inline fmoe_model_desc modelDesc(const MoEArgs& a, const LayerDesc& l, int arch) {
  if (a.elementBytes != 2 && a.elementBytes != 4 && a.elementBytes != 8)
    throw std::runtime_error("elementBytes not supported");
  fmoe_model_desc m{};
  m.tokens_per_rank = static_cast<int32_t>(a.sequenceLength);
  m.token_dim = static_cast<int32_t>(a.tokenDim);
  m.ffn_size = static_cast<int32_t>(a.ffnIntermediateSize);
  m.num_experts = static_cast<int32_t>(a.numExperts);
  m.top_k = l.topK;
  m.expert_peer_capacity = static_cast<int32_t>(a.EC);
  m.data_type = static_cast<int32_t>(l.element);
  m.mlp_type = static_cast<int32_t>(l.mlp);
  m.act_type = static_cast<int32_t>(l.act);
  m.gpu_arch = arch;
  return m;
}

// flashmoe::initialize (bootstrap.cuh:197).
inline Context initialize(const MoEArgs& args, const LayerDesc& layer, int arch, const int* expertToEpRank,
                          const int* epRankToGlobalRank, Stream stream) {
  const fmoe_model_desc m = modelDesc(args, layer, arch);
  fmoe_ep_desc ep{};
  ep.ep_world = args.epWorld; ep.ep_rank = args.epRank; ep.my_pe = args.myPE; ep.device_id = layer.deviceId;
  ep.num_local_experts = args.numLocalExperts; ep.topology = static_cast<int32_t>(args.topo);
  ep.expert_map = expertToEpRank; ep.rank_map = epRankToGlobalRank;
  Context c;
  check(fmoe_ctx_create(&m, &ep, stream, &c.handle), "flashmoe::initialize");
  void* table = nullptr;
  check(fmoe_token_indices(c.handle, &table), "flashmoe::initialize");
  c.tokenIndices = static_cast<TPS*>(table);
  c.S = args.sequenceLength; c.H = args.tokenDim; c.I = args.ffnIntermediateSize;
  c.EC = static_cast<unsigned>(args.EC); c.nLx = args.numLocalExperts;
  c.E = static_cast<uint16_t>(args.numExperts); c.world = args.epWorld; c.epRank = args.epRank;
  c.myPE = args.myPE; c.topo = args.topo;
  if (args.epWorld == 1) check(fmoe_ctx_commit(c.handle), "flashmoe::initialize");
  return c;
}
// flashmoe::getWorkspaceBytes (bootstrap.cuh:377-410): device bytes initialize would allocate on
// this rank (symmetric block + private workspace), computed on the host.
inline size_t getWorkspaceBytes(const MoEArgs& args, const LayerDesc& layer = LayerDesc{}, int arch = 1000) {
  const fmoe_model_desc m = modelDesc(args, layer, arch);
  fmoe_ep_desc ep{};
  ep.ep_world = args.epWorld; ep.ep_rank = args.epRank; ep.my_pe = args.myPE; ep.device_id = layer.deviceId;
  ep.num_local_experts = args.numLocalExperts; ep.topology = static_cast<int32_t>(args.topo);
  int64_t symm = 0, work = 0;
  check(fmoe_workspace_bytes(&m, &ep, &symm, &work), "flashmoe::getWorkspaceBytes");
  return static_cast<size_t>(symm + work);
}
// Peer mapping for epWorld > 1 (replaces nvshmem_malloc / nvshmem_ptr, bootstrap.cuh:141-151).
inline std::vector<unsigned char> exportSymmetric(Context& c) {
  std::vector<unsigned char> h(FMOE_IPC_HANDLE_BYTES);
  check(fmoe_symm_export(c.handle, h.data()), "flashmoe::exportSymmetric");
  return h;
}
inline void importSymmetric(Context& c, int peerEpRank, const std::vector<unsigned char>& handle) {
  check(fmoe_symm_import(c.handle, peerEpRank, handle.data()), "flashmoe::importSymmetric");
}
inline void commit(Context& c) { check(fmoe_ctx_commit(c.handle), "flashmoe::commit"); }

// flashmoe::finalize (bootstrap.cuh:450).
inline void finalize(Context& c, Stream stream) {
  check(fmoe_ctx_destroy(c.handle, stream), "flashmoe::finalize");
  c.handle = nullptr;
}

// initializeGate / finalizeGate (bootstrap.cuh:413-447).
inline GateContext initializeGate(const MoEArgs& args, const LayerDesc& layer, int arch, bool returnLogits,
                                  Stream stream) {
  const fmoe_model_desc m = modelDesc(args, layer, arch);
  GateContext g;
  check(fmoe_router_create(&m, layer.deviceId, returnLogits ? 1 : 0, stream, &g.handle), "flashmoe::initializeGate");
  return g;
}
inline void finalizeGate(GateContext& g, Stream stream) {
  check(fmoe_router_destroy(g.handle, stream), "flashmoe::finalizeGate");
  g.handle = nullptr;
}

namespace gate {
// Stands for the launch of gate::forwardKernel (gate.cuh:588-608): tokens [S,H], weights [E,H],
// routing [S,E] fp32 or null, expertCounts [E]; the routing table goes into `moeCtx`.
inline void forward(GateContext& g, Context& moeCtx, const void* tokens, const void* weights, float* routing,
                    int* expertCounts, Stream stream, const float* logitBias = nullptr) {
  fmoe_router_args a{tokens, weights, routing, expertCounts, logitBias};
  check(fmoe_router_forward(g.handle, moeCtx.handle, &a, stream), "flashmoe::gate::forward");
}
}  // namespace gate

namespace moe {
// Same members as the reference's KernelArgs (moe.cuh:100-159); shapes live in the context.
struct KernelArgs {
  const void* tokens;              // [S, H]
  const void* expertUpWeights;     // [nLx, I, H]
  const void* expertUpVWeights;    // [nLx, I, H] or null
  const void* biasUp;              // [nLx, I] or null
  const void* biasUpV;             // [nLx, I] or null
  const void* expertDownWeights;   // [nLx, H, I]
  const void* biasDown;            // [nLx, H] or null
  const int* expertCounts;         // [E]
  void* moeOut;                    // [S, H]
  float swishAlpha = 1.f;
  float swishBeta = 1.f;
};
// moe::forwardHost (moe.cuh:255-260): one launch on `stream`.
inline void forwardHost(const Context& ctx, const KernelArgs& k, Stream stream) {
  fmoe_forward_args a{k.tokens, k.expertCounts, k.expertUpWeights, k.expertUpVWeights, k.biasUp, k.biasUpV,
                      k.expertDownWeights, k.biasDown, k.moeOut, k.swishAlpha, k.swishBeta};
  check(fmoe_forward(ctx.handle, &a, stream), "flashmoe::moe::forwardHost");
}
}  // namespace moe

}  // namespace flashmoe
