// Host side of the C ABI declared in include/flashmoe_b200.h: validation, allocation of the
// symmetric block and the private workspace, CUDA-IPC peer mapping, TMA descriptor
// construction and the launches.  It plays the role of the reference's bootstrap
// (csrc/include/flashmoe/bootstrap.cuh:197-474) and of its pybind glue
// (flashmoe/bindings.py:68-185, 238-315), with CUDA IPC in place of the NVSHMEM heap.
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace fmoe {

thread_local std::string t_error;

int set_error(int code, const std::string& msg) {
  t_error = msg;
  return code;
}

namespace {

#define FMOE_CUDA(expr)                                                                      \
  do {                                                                                       \
    cudaError_t err__ = (expr);                                                              \
    if (err__ != cudaSuccess) {                                                              \
      return set_error(FMOE_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorName(err__) +  \
                                          " (" + cudaGetErrorString(err__) + ")");           \
    }                                                                                        \
  } while (0)

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Makes `device` current for the rest of the scope and puts the calling thread's device back on
// every way out: a library called between a host engine's own launches must not leave the engine
// on another GPU.
struct ScopedDevice {
  int prev = -1;
  cudaError_t err = cudaSuccess;
  explicit ScopedDevice(int device) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) cur = -1;
    err = cudaSetDevice(device);
    if (err == cudaSuccess && cur >= 0 && cur != device) prev = cur;
  }
  ~ScopedDevice() { if (prev >= 0) cudaSetDevice(prev); }
  ScopedDevice(const ScopedDevice&) = delete;
  ScopedDevice& operator=(const ScopedDevice&) = delete;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  }
  return fn;
}

// 2-D row-major [rows, cols] 16-bit tensor, box = 64 columns x 128 rows, 128-byte swizzle.
int make_map(CUtensorMap* out, int ab_format, const void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return set_error(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kTileK), 128};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(out, ab_format == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return set_error(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(r) +
                                        " (base must be 16-byte aligned, row pitch a multiple of 16 bytes)");
  }
  return FMOE_OK;
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

struct fmoe_ctx {
  fmoe_model_desc model{};
  int W = 1, rank = 0, nLx = 0, device = 0;
  std::vector<int32_t> owner, lidx, local_e;
  fmoe_geometry geo{};
  SymmLayout lay{};
  char* symm = nullptr;                 // this rank's block
  char* peers[FMOE_MAX_WORLD] = {};     // mapped blocks (peers[rank] == symm)
  bool imported[FMOE_MAX_WORLD] = {};   // opened through IPC (must be closed)
  bool committed = false;
  bool owns_memory = true;              // false: symmetric block and workspace belong to the caller
  bool poisoned = false;                // a forward of this context ran out of a device-side wait
  char* work = nullptr;                 // private workspace, one allocation
  size_t work_bytes = 0;
  MoeParams params{};                   // everything but the per-forward pointers
  CUtensorMap maps[5];
  // TMA descriptors of the weight sets seen so far (one per layer served by this context),
  // oldest replaced first once FMOE_LAYER_CACHE are held
  struct WeightMaps {
    const void* src[3] = {nullptr, nullptr, nullptr};  // up, up_v, down
    CUtensorMap m[3];
  };
  std::vector<WeightMaps> layer_maps;
  size_t layer_next = 0;
  void* stage_tokens = nullptr;         // host-buffer entry point staging
  void* stage_out = nullptr;
  // pipelined host-buffer entry point: two slots, a copy-in and a copy-out stream, events per slot
  struct Pipe {
    bool ready = false;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    void* tokens[2] = {nullptr, nullptr};
    void* out[2] = {nullptr, nullptr};
    cudaEvent_t in_done[2] = {}, compute_done[2] = {}, out_done[2] = {};
    unsigned long long submitted = 0;
  } pipe;
  int eb = 2;                           // bytes per Element (4 for fp32 layers)
  int planes = 1;                       // BF16 planes per GEMM operand (3 for fp32 layers)
  char* wsplit = nullptr;               // fp32 layers: BF16 planes of up | up_v | down
  size_t wsplit_up = 0, wsplit_up_v = 0, wsplit_down = 0;
  const void* wsplit_src[3] = {nullptr, nullptr, nullptr};   // the weight set those planes were made from
  // a library built for exactly this layer's description (fmoe_ctx_load_specialised), or none
  void* spec_handle = nullptr;
  int (*spec_launch)(const void*, const void*, int, size_t, void*) = nullptr;
};

struct fmoe_router {
  fmoe_model_desc model{};
  int device = 0;
  int return_logits = 0;
  int32_t* topk_idx = nullptr;
  float* topk_w = nullptr;
};

namespace fmoe {

int validate_model(const fmoe_model_desc* m) {
  if (m == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "model description is null");
  if (m->gpu_arch != 1000 && m->gpu_arch != 1030)
    return set_error(FMOE_ERR_UNSUPPORTED, "gpu_arch " + std::to_string(m->gpu_arch) +
                                               " is not supported: this library is built for sm_100a only "
                                               "(pass 1000)");
  if (m->tokens_per_rank < 1 || m->token_dim < 1 || m->ffn_size < 1 || m->num_experts < 1 || m->top_k < 1)
    return set_error(FMOE_ERR_INVALID_ARG, "S, H, I, E and k must be positive");
  if (m->top_k > m->num_experts || m->top_k > 32)
    return set_error(FMOE_ERR_INVALID_ARG, "top_k must not exceed num_experts (or 32)");
  if (m->expert_peer_capacity < 1)
    return set_error(FMOE_ERR_INVALID_ARG, "expert_peer_capacity must be positive");
  if (m->num_experts % 8 != 0)
    return set_error(FMOE_ERR_INVALID_ARG, "num_experts must be a multiple of 8");
  if (m->token_dim % kTileK != 0)
    return set_error(FMOE_ERR_INVALID_ARG, "token dimension should be multiples of tile dimensions (64)");
  if (m->ffn_size % kTileK != 0)
    return set_error(FMOE_ERR_INVALID_ARG, "Intermediate size should be multiples of tile dimensions (64)");
  if (m->mlp_type != FMOE_MLP_GATED && m->mlp_type != FMOE_MLP_VANILLA)
    return set_error(FMOE_ERR_INVALID_ARG, "unknown mlp_type");
  if (m->act_type < FMOE_ACT_IDENTITY || m->act_type > FMOE_ACT_RELU)
    return set_error(FMOE_ERR_INVALID_ARG, "unknown act_type");
  if (m->data_type < FMOE_DT_BF16 || m->data_type > FMOE_DT_FP64)
    return set_error(FMOE_ERR_INVALID_ARG, "elementBytes not supported");
  if (static_cast<long long>(m->tokens_per_rank) * m->top_k >= (1LL << kMetaSrcShift))
    return set_error(FMOE_ERR_UNSUPPORTED, "tokens_per_rank * top_k must stay below 2^26");
  return FMOE_OK;
}

}  // namespace fmoe

namespace {

// Sizes and offsets of everything a context allocates, from the layer's description alone (no
// device call): the symmetric block (mapped by every peer) and the private workspace.
struct Plan {
  int round_ec = 0, landing_rows = 0, max_mtiles = 0;
  SymmLayout lay{};
  size_t w_y = 0, w_logits = 0, w_split = 0, w_done = 0, w_split_done = 0, w_ctl = 0, w_status = 0, w_trace = 0, w_table = 0,
         w_routes = 0, w_owner = 0, w_lidx = 0, w_local = 0, work_bytes = 0;
  int split_parts = 1, split_tiles = 0;
  size_t weight_plane_bytes = 0;   // fp32 layers: the BF16 planes of up, up_v and down
};

// GEMM1 tiles of the closing wave are cut along K into this many tickets (FMOE_SPLIT_PARTS
// overrides; 1 = never).  The count of cut tiles is one wave of the largest grid (one CTA per SM).
constexpr int kSplitPartsDefault = 2;
constexpr int kSplitTilesMax = 160;

int split_parts_for(const fmoe_model_desc& m) {
  int parts = kSplitPartsDefault;
  if (const char* e = std::getenv("FMOE_SPLIT_PARTS")) parts = std::atoi(e);
  if (const char* e = std::getenv("FMOE_PAIR")) if (std::atoi(e)) parts = 1;   // the CTA-pair form never cuts
  const int nk1 = m.ffn_size / kTileK;
  if (parts > 8) parts = 8;
  if (parts < 2 || nk1 < 4 * parts) parts = 1;   // at least four K blocks per part
  return parts;
}

Plan plan_sizes(const fmoe_model_desc& m, int W, int nLx) {
  Plan pl;
  const int S = m.tokens_per_rank, H = m.token_dim, I = m.ffn_size, k = m.top_k, E = m.num_experts;
  const int EC = m.expert_peer_capacity;
  const int eb = m.data_type == FMOE_DT_FP32 ? 4 : 2, planes = m.data_type == FMOE_DT_FP32 ? 3 : 1;
  pl.round_ec = static_cast<int>(align_up(EC, kTileM));
  const long long cap_a = static_cast<long long>(nLx) * align_up(static_cast<size_t>(W) * EC, kTileM);
  const long long cap_b = static_cast<long long>(align_up(static_cast<size_t>(W) * S * k, kTileM)) +
                          static_cast<long long>(nLx) * kTileM;
  pl.landing_rows = static_cast<int>(cap_a < cap_b ? cap_a : cap_b);
  pl.max_mtiles = pl.landing_rows / kTileM;
  // symmetric block layout (same arithmetic on every rank)
  SymmLayout& L = pl.lay;
  size_t off = 0;
  L.cnt_table = off; off = align_up(off + sizeof(int32_t) * 2 * W * E, 256);
  L.cnt_flag = off; off = align_up(off + sizeof(uint64_t) * 2 * W, 256);
  L.disp_arrived = off; off = align_up(off + sizeof(uint32_t) * W * nLx, 256);
  L.ret_arrived = off; off = align_up(off + sizeof(uint32_t), 256);
  L.landing_meta = off; off = align_up(off + sizeof(uint32_t) * pl.landing_rows, 1024);
  L.landing = off; off = align_up(off + static_cast<size_t>(planes) * pl.landing_rows * H * 2, 1024);
  L.ret = off; off = align_up(off + static_cast<size_t>(S) * k * H * eb, 1024);
  L.total = off;
  // private workspace
  size_t w = 0;
  pl.w_y = w; w = align_up(w + static_cast<size_t>(planes) * pl.landing_rows * I * 2, 1024);
  pl.split_parts = split_parts_for(m);
  pl.split_tiles = pl.split_parts > 1 ? kSplitTilesMax : 0;
  pl.w_split = w; w = align_up(w + static_cast<size_t>(pl.split_tiles) * pl.split_parts * kTileM * kUmmaN * sizeof(float), 1024);
  pl.w_logits = w; w = align_up(w + sizeof(float) * S * E, 1024);
  pl.w_done = w; w = align_up(w + sizeof(uint32_t) * pl.max_mtiles, 256);
  pl.w_split_done = w; w = align_up(w + sizeof(uint32_t) * 4 * (pl.split_tiles + 1), 256);
  pl.w_ctl = w; w = align_up(w + 256, 256);   // ticket, done_ctas, abort, epoch
  pl.w_status = w; w = align_up(w + sizeof(fmoe_status), 256);
  pl.w_trace = w; w = align_up(w + sizeof(unsigned long long) * kTraceSlots * 256, 256);
  pl.w_table = w; w = align_up(w + sizeof(TokenSlot) * E * pl.round_ec, 256);
  pl.w_routes = w; w = align_up(w + sizeof(Route) * S * k, 256);
  pl.w_owner = w; w = align_up(w + sizeof(int32_t) * E, 256);
  pl.w_lidx = w; w = align_up(w + sizeof(int32_t) * E, 256);
  pl.w_local = w; w = align_up(w + sizeof(int32_t) * W * nLx, 256);
  pl.work_bytes = align_up(w, 1024);   // what follows it (the BF16 weight planes of fp32 layers) stays aligned
  if (planes == 3)
    pl.weight_plane_bytes = static_cast<size_t>(nLx) * I * H * 2 * 3 * (m.mlp_type == FMOE_MLP_GATED ? 3 : 2);
  return pl;
}

// The argument checks of fmoe_ctx_create that need no device.
int check_layer(const fmoe_model_desc* model, const fmoe_ep_desc* ep) {
  int rc = validate_model(model);
  if (rc != FMOE_OK) return rc;
  if (ep == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "ep description is null");
  if (model->data_type == FMOE_DT_FP64)
    return set_error(FMOE_ERR_UNSUPPORTED, "the expert kernels handle BF16, FP16 and FP32; FP64 is not built");
  if (ep->topology != FMOE_TOPO_NVLINK_ONLY)
    return set_error(FMOE_ERR_UNSUPPORTED, "only Topology.NVLINK_ONLY (one NVLink box) is implemented");
  const int W = ep->ep_world, E = model->num_experts;
  if (W < 1 || W > FMOE_MAX_WORLD)
    return set_error(FMOE_ERR_UNSUPPORTED, "ep_world must be between 1 and " + std::to_string(FMOE_MAX_WORLD));
  if (ep->ep_rank < 0 || ep->ep_rank >= W) return set_error(FMOE_ERR_INVALID_ARG, "ep_rank out of range");
  if (ep->num_local_experts < 1 || ep->num_local_experts * W != E)
    return set_error(FMOE_ERR_INVALID_ARG, "every rank must hold num_experts / ep_world experts");
  if (static_cast<long long>(W) * E > 4096)
    return set_error(FMOE_ERR_UNSUPPORTED, "ep_world * num_experts must not exceed 4096");
  return FMOE_OK;
}

void free_ctx(fmoe_ctx* c) {
  if (c == nullptr) return;
  for (int r = 0; r < FMOE_MAX_WORLD; ++r)
    if (c->imported[r] && c->peers[r] != nullptr) cudaIpcCloseMemHandle(c->peers[r]);
  if (c->owns_memory) {
    if (c->symm) cudaFree(c->symm);
    if (c->work) cudaFree(c->work);
    if (c->wsplit) cudaFree(c->wsplit);
  }
  if (c->stage_tokens) cudaFree(c->stage_tokens);
  if (c->stage_out) cudaFree(c->stage_out);
  if (c->spec_handle) dlclose(c->spec_handle);
  if (c->pipe.ready) {
    for (int i = 0; i < 2; ++i) {
      cudaFree(c->pipe.tokens[i]); cudaFree(c->pipe.out[i]);
      cudaEventDestroy(c->pipe.in_done[i]); cudaEventDestroy(c->pipe.compute_done[i]);
      cudaEventDestroy(c->pipe.out_done[i]);
    }
    cudaStreamDestroy(c->pipe.s_in); cudaStreamDestroy(c->pipe.s_out);
  }
  delete c;
}

}  // namespace

extern "C" {

const char* fmoe_strerror(int code) {
  switch (code) {
    case FMOE_OK: return "success";
    case FMOE_ERR_INVALID_ARG: return "invalid argument";
    case FMOE_ERR_UNSUPPORTED: return "unsupported configuration";
    case FMOE_ERR_CUDA: return "CUDA call failed";
    case FMOE_ERR_NOT_READY: return "context not ready (peers missing or not committed)";
    case FMOE_ERR_DEVICE_TIMEOUT: return "a device-side wait ran out";
    case FMOE_ERR_NO_MEMORY: return "out of memory";
    default: return "unknown status";
  }
}

const char* fmoe_last_error(void) { return t_error.c_str(); }

uint64_t fmoe_launch_count(void) { return g_launches; }

int fmoe_workspace_bytes(const fmoe_model_desc* model, const fmoe_ep_desc* ep, int64_t* symm_bytes_out,
                         int64_t* workspace_bytes_out) {
  const int rc = check_layer(model, ep);
  if (rc != FMOE_OK) return rc;
  const Plan pl = plan_sizes(*model, ep->ep_world, ep->num_local_experts);
  if (symm_bytes_out) *symm_bytes_out = static_cast<int64_t>(pl.lay.total);
  if (workspace_bytes_out) *workspace_bytes_out = static_cast<int64_t>(align_up(pl.work_bytes, 1024) + pl.weight_plane_bytes);
  return FMOE_OK;
}

static int ctx_create_impl(const fmoe_model_desc* model, const fmoe_ep_desc* ep, void* stream, void* symm_mem,
                           size_t symm_bytes, void* work_mem, size_t work_bytes, bool caller_memory, fmoe_ctx** out);

int fmoe_ctx_create(const fmoe_model_desc* model, const fmoe_ep_desc* ep, void* stream, fmoe_ctx** out) {
  return ctx_create_impl(model, ep, stream, nullptr, 0, nullptr, 0, false, out);
}

int fmoe_ctx_create_in(const fmoe_model_desc* model, const fmoe_ep_desc* ep, void* stream, void* symm_mem,
                       size_t symm_bytes, void* work_mem, size_t work_bytes, fmoe_ctx** out) {
  if (symm_mem == nullptr || work_mem == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "symmetric block and workspace are required");
  if ((reinterpret_cast<uintptr_t>(symm_mem) | reinterpret_cast<uintptr_t>(work_mem)) & 1023)
    return set_error(FMOE_ERR_INVALID_ARG, "symmetric block and workspace must be 1024-byte aligned");
  return ctx_create_impl(model, ep, stream, symm_mem, symm_bytes, work_mem, work_bytes, true, out);
}

static int ctx_create_impl(const fmoe_model_desc* model, const fmoe_ep_desc* ep, void* stream, void* symm_mem,
                           size_t symm_bytes, void* work_mem, size_t work_bytes, bool caller_memory, fmoe_ctx** out) {
  if (out == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "out is null");
  *out = nullptr;
  int rc = check_layer(model, ep);
  if (rc != FMOE_OK) return rc;
  if (ep->expert_map == nullptr || ep->rank_map == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "expert_map and rank_map are required");
  const int W = ep->ep_world, E = model->num_experts;
  const int nLx = ep->num_local_experts;

  fmoe_ctx* c = new (std::nothrow) fmoe_ctx();
  if (c == nullptr) return set_error(FMOE_ERR_NO_MEMORY, "host allocation failed");
  c->model = *model;
  c->W = W; c->rank = ep->ep_rank; c->nLx = nLx; c->device = ep->device_id;
  c->eb = model->data_type == FMOE_DT_FP32 ? 4 : 2;
  c->planes = model->data_type == FMOE_DT_FP32 ? 3 : 1;
  c->owner.assign(ep->expert_map, ep->expert_map + E);
  c->lidx.assign(E, 0);
  c->local_e.assign(static_cast<size_t>(W) * nLx, -1);
  std::vector<int> fill(W, 0);
  for (int e = 0; e < E; ++e) {
    const int r = c->owner[e];
    if (r < 0 || r >= W || fill[r] >= nLx) {
      free_ctx(c);
      return set_error(FMOE_ERR_INVALID_ARG, "expert_map must give every rank exactly num_local_experts experts");
    }
    c->lidx[e] = fill[r];
    c->local_e[static_cast<size_t>(r) * nLx + fill[r]] = e;
    ++fill[r];
  }

  ScopedDevice on_device(c->device);
  cudaError_t ce = on_device.err;
  if (ce != cudaSuccess) { free_ctx(c); return set_error(FMOE_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(ce)); }
  int sms = 0, cc_major = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
  cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, c->device);
  if (cc_major != 10) { free_ctx(c); return set_error(FMOE_ERR_UNSUPPORTED, "device is not compute capability 10.x"); }

  const int S = model->tokens_per_rank, H = model->token_dim, I = model->ffn_size, k = model->top_k;
  const int EC = model->expert_peer_capacity;
  const bool gated = model->mlp_type == FMOE_MLP_GATED;
  fmoe_geometry& g = c->geo;
  g.tile_m = kTileM; g.tile_k = kTileK;
  g.tile_n0 = gated ? 128 : 256; g.tile_n1 = 256;
  const Plan pl = plan_sizes(*model, W, nLx);
  g.round_ec = pl.round_ec;
  g.landing_rows = pl.landing_rows;
  g.grid = sms & ~1; g.threads = kThreads;   // CTA pairs: an even number of CTAs, one per SM
  g.smem_bytes = static_cast<int>(moe_smem_bytes(W, E, nLx));
  if (g.smem_bytes > 227 * 1024) { free_ctx(c); return set_error(FMOE_ERR_UNSUPPORTED, "tables do not fit in shared memory"); }

  // symmetric block layout (same arithmetic on every rank)
  SymmLayout& L = c->lay;
  L = pl.lay;
  g.symm_bytes = static_cast<int64_t>(L.total);

  c->owns_memory = !caller_memory;
  if (caller_memory) {
    const size_t need_work = align_up(pl.work_bytes, 1024) + pl.weight_plane_bytes;
    if (symm_bytes < L.total || work_bytes < need_work) {
      free_ctx(c);
      return set_error(FMOE_ERR_INVALID_ARG, "caller's memory is too small: this layer needs " + std::to_string(L.total) +
                                                 " bytes of symmetric block and " + std::to_string(need_work) +
                                                 " bytes of workspace (see fmoe_workspace_bytes)");
    }
    c->symm = static_cast<char*>(symm_mem);
    ce = cudaSuccess;
  } else {
    ce = cudaMalloc(&c->symm, L.total);
  }
  if (ce != cudaSuccess) { free_ctx(c); return set_error(FMOE_ERR_NO_MEMORY, std::string("symmetric block: ") + cudaGetErrorString(ce)); }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // control words must start at zero; the data areas need no initial value
  ce = cudaMemsetAsync(c->symm, 0, L.landing, st);
  if (ce != cudaSuccess) { free_ctx(c); return set_error(FMOE_ERR_CUDA, cudaGetErrorString(ce)); }
  c->peers[c->rank] = c->symm;

  // private workspace
  const int max_mtiles = pl.max_mtiles;
  const size_t w_y = pl.w_y, w_done = pl.w_done, w_ctl = pl.w_ctl, w_status = pl.w_status, w_trace = pl.w_trace,
               w_table = pl.w_table, w_routes = pl.w_routes, w_owner = pl.w_owner, w_lidx = pl.w_lidx,
               w_local = pl.w_local, w = pl.work_bytes;
  c->work_bytes = w;
  g.workspace_bytes = static_cast<int64_t>(w);
  if (caller_memory) c->work = static_cast<char*>(work_mem);
  else ce = cudaMalloc(&c->work, w);
  if (ce != cudaSuccess) { free_ctx(c); return set_error(FMOE_ERR_NO_MEMORY, std::string("workspace: ") + cudaGetErrorString(ce)); }
  ce = cudaMemsetAsync(c->work + w_done, 0, w - w_done, st);
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(c->work + w_owner, c->owner.data(), sizeof(int32_t) * E, cudaMemcpyHostToDevice, st);
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(c->work + w_lidx, c->lidx.data(), sizeof(int32_t) * E, cudaMemcpyHostToDevice, st);
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(c->work + w_local, c->local_e.data(), sizeof(int32_t) * W * nLx, cudaMemcpyHostToDevice, st);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
  if (ce == cudaSuccess) ce = moe_prepare_kernel(g.smem_bytes);
  if (ce != cudaSuccess) { free_ctx(c); return set_error(FMOE_ERR_CUDA, std::string("workspace set-up: ") + cudaGetErrorString(ce)); }

  MoeParams& p = c->params;
  p.S = S; p.H = H; p.I = I; p.E = E; p.k = k; p.EC = EC; p.round_ec = g.round_ec;
  p.W = W; p.rank = c->rank; p.nLx = nLx;
  p.gated = gated ? 1 : 0; p.act = model->act_type; p.ab_format = model->data_type == FMOE_DT_FP16 ? 0 : 1;
  p.elem_bytes = c->eb;
  {
    // every device-side wait of this context gives up after this long (default 2 s)
    const char* lim = std::getenv("FMOE_SPIN_LIMIT_MS");
    p.spin_limit = spin_limit_cycles(lim ? std::atof(lim) : 2000.0, c->device);
    const char* wh = std::getenv("FMOE_WITHHOLD_FLAGS");   // test hook: see MoeParams::withhold_flags
    p.withhold_flags = (wh && std::atoi(wh)) ? 1 : 0;
  }
  // Two forms of the GEMM loop exist: every CTA alone on a 128 x 256 tile (default), or CTA pairs
  // on 256 x 256 tiles with tcgen05.mma.cta_group::2 (FMOE_PAIR=1).  Measured on one B200 the pair
  // form gains 3-6 % per unit of MMA work on experts with many M tiles and loses more than that
  // to its coarser 256-row granularity and to the fewer weight bytes it keeps in flight when
  // experts hold about one tile, so it is opt-in.
  {
    p.pair = 0;
    const char* force = std::getenv("FMOE_PAIR");
    if (force) p.pair = std::atoi(force) ? 1 : 0;
    g.cta_pairs = p.pair; g.stages = p.pair ? 6 : 4;
    p.split_parts = pl.split_parts;
    p.split_tiles = pl.split_parts > 1 ? (g.grid < kSplitTilesMax ? g.grid : kSplitTilesMax) : 0;
    g.split_parts = p.split_parts;
  }
  p.tiles_n0 = (I + g.tile_n0 - 1) / g.tile_n0;
  p.tiles_n1 = (H + g.tile_n1 - 1) / g.tile_n1;
  if (static_cast<long long>(S) * k * p.tiles_n1 >= (1LL << 31)) {
    free_ctx(c);
    return set_error(FMOE_ERR_UNSUPPORTED, "tokens_per_rank * top_k * ceil(H / 256) is too large for the 32-bit arrival counters");
  }
  p.landing_rows = g.landing_rows; p.max_mtiles = max_mtiles;
  p.owner = reinterpret_cast<const int32_t*>(c->work + w_owner);
  p.lidx = reinterpret_cast<const int32_t*>(c->work + w_lidx);
  p.local_e = reinterpret_cast<const int32_t*>(c->work + w_local);
  p.lay = L;
  p.y = c->work + w_y;
  p.gemm0_done = reinterpret_cast<uint32_t*>(c->work + w_done);
  p.split_scratch = reinterpret_cast<float*>(c->work + pl.w_split);
  p.split_done = reinterpret_cast<uint32_t*>(c->work + pl.w_split_done);
  p.route_logits = reinterpret_cast<float*>(c->work + pl.w_logits);
  p.ticket = reinterpret_cast<uint32_t*>(c->work + w_ctl);
  p.done_ctas = reinterpret_cast<uint32_t*>(c->work + w_ctl + 64);
  p.abort_word = reinterpret_cast<uint32_t*>(c->work + w_ctl + 128);
  p.epoch = reinterpret_cast<uint64_t*>(c->work + w_ctl + 192);
  p.grid_bar = reinterpret_cast<unsigned long long*>(c->work + w_ctl + 208);
  p.status = reinterpret_cast<fmoe_status*>(c->work + w_status);
  p.trace = reinterpret_cast<unsigned long long*>(c->work + w_trace);
  p.table = reinterpret_cast<const TokenSlot*>(c->work + w_table);
  p.routes = reinterpret_cast<const Route*>(c->work + w_routes);

  const uint64_t prow = static_cast<uint64_t>(c->planes) * g.landing_rows;
  rc = make_map(&c->maps[0], p.ab_format, c->symm + L.landing, prow, H);
  if (rc == FMOE_OK) rc = make_map(&c->maps[1], p.ab_format, p.y, prow, I);
  if (rc == FMOE_OK && c->planes == 3) {
    // fp32 layers: the weights are re-split into BF16 planes on every forward, into buffers the
    // context owns, so their tensor maps are built once here
    const size_t mat = static_cast<size_t>(nLx) * I * H * 2 * 3;
    c->wsplit_up = 0; c->wsplit_up_v = gated ? mat : 0; c->wsplit_down = gated ? 2 * mat : mat;
    if (caller_memory) c->wsplit = c->work + align_up(pl.work_bytes, 1024);   // behind the workspace proper
    else ce = cudaMalloc(&c->wsplit, c->wsplit_down + mat);
    if (ce != cudaSuccess) { free_ctx(c); return set_error(FMOE_ERR_NO_MEMORY, std::string("weight planes: ") + cudaGetErrorString(ce)); }
    g.workspace_bytes += static_cast<int64_t>(c->wsplit_down + mat);
    rc = make_map(&c->maps[2], 1, c->wsplit + c->wsplit_up, 3ull * nLx * I, H);
    if (rc == FMOE_OK) rc = make_map(&c->maps[3], 1, c->wsplit + c->wsplit_up_v, 3ull * nLx * I, H);
    if (rc == FMOE_OK) rc = make_map(&c->maps[4], 1, c->wsplit + c->wsplit_down, 3ull * nLx * H, I);
  }
  if (rc != FMOE_OK) { free_ctx(c); return rc; }
  c->committed = (W == 1);
  if (W == 1) c->params.peers[0] = c->symm;
  *out = c;
  return FMOE_OK;
}

int fmoe_symm_bytes(const fmoe_ctx* ctx, size_t* bytes) {
  if (ctx == nullptr || bytes == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  *bytes = ctx->lay.total;
  return FMOE_OK;
}

int fmoe_symm_export(fmoe_ctx* ctx, void* handle_out) {
  if (ctx == nullptr || handle_out == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == FMOE_IPC_HANDLE_BYTES, "IPC handle size");
  ScopedDevice on_device(ctx->device);
  FMOE_CUDA(on_device.err);
  if (!ctx->owns_memory) {
    // CUDA IPC shares whole allocations: a peer that opens the handle gets the allocation's first
    // byte, so a caller's block that starts anywhere else would be mapped at the wrong address.
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess && sym != nullptr) {
      CUdeviceptr base = 0;
      size_t size = 0;
      if (reinterpret_cast<RangeFn>(sym)(&base, &size, reinterpret_cast<CUdeviceptr>(ctx->symm)) == CUDA_SUCCESS &&
          base != reinterpret_cast<CUdeviceptr>(ctx->symm))
        return set_error(FMOE_ERR_INVALID_ARG,
                         "the caller's symmetric block starts " +
                             std::to_string(reinterpret_cast<CUdeviceptr>(ctx->symm) - base) +
                             " bytes into its device allocation; to be shared through CUDA IPC it must be an "
                             "allocation of its own (or map the peers yourself and use fmoe_symm_set_peer)");
    }
  }
  cudaIpcMemHandle_t h;
  FMOE_CUDA(cudaIpcGetMemHandle(&h, ctx->symm));
  std::memcpy(handle_out, &h, sizeof(h));
  return FMOE_OK;
}

int fmoe_symm_import(fmoe_ctx* ctx, int32_t peer, const void* handle) {
  if (ctx == nullptr || handle == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  if (peer < 0 || peer >= ctx->W) return set_error(FMOE_ERR_INVALID_ARG, "peer rank out of range");
  if (peer == ctx->rank) return FMOE_OK;
  ScopedDevice on_device(ctx->device);
  FMOE_CUDA(on_device.err);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* base = nullptr;
  FMOE_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  ctx->peers[peer] = static_cast<char*>(base);
  ctx->imported[peer] = true;
  return FMOE_OK;
}

int fmoe_symm_base(fmoe_ctx* ctx, void** base_out) {
  if (ctx == nullptr || base_out == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  *base_out = ctx->symm;
  return FMOE_OK;
}

int fmoe_symm_set_peer(fmoe_ctx* ctx, int32_t peer, void* peer_base) {
  if (ctx == nullptr || peer_base == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  if (peer < 0 || peer >= ctx->W) return set_error(FMOE_ERR_INVALID_ARG, "peer rank out of range");
  if (peer != ctx->rank) ctx->peers[peer] = static_cast<char*>(peer_base);
  return FMOE_OK;
}

int fmoe_ctx_commit(fmoe_ctx* ctx) {
  if (ctx == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null context");
  for (int r = 0; r < ctx->W; ++r) {
    if (ctx->peers[r] == nullptr)
      return set_error(FMOE_ERR_NOT_READY, "symmetric block of ep rank " + std::to_string(r) + " has not been imported");
    ctx->params.peers[r] = ctx->peers[r];
  }
  ctx->committed = true;
  return FMOE_OK;
}

int fmoe_token_indices(fmoe_ctx* ctx, void** table_out) {
  if (ctx == nullptr || table_out == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  *table_out = const_cast<TokenSlot*>(ctx->params.table);
  return FMOE_OK;
}

int fmoe_get_geometry(const fmoe_ctx* ctx, fmoe_geometry* out) {
  if (ctx == nullptr || out == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  *out = ctx->geo;
  return FMOE_OK;
}

int fmoe_debug_buffer(fmoe_ctx* ctx, int32_t which, void** ptr_out, size_t* bytes_out) {
  if (ctx == nullptr || ptr_out == nullptr || bytes_out == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  const MoeParams& p = ctx->params;
  switch (which) {
    case 0: *ptr_out = ctx->symm + ctx->lay.landing; *bytes_out = static_cast<size_t>(ctx->planes) * p.landing_rows * p.H * 2; break;
    case 1: *ptr_out = ctx->symm + ctx->lay.landing_meta; *bytes_out = sizeof(uint32_t) * p.landing_rows; break;
    case 2: *ptr_out = p.y; *bytes_out = static_cast<size_t>(ctx->planes) * p.landing_rows * p.I * 2; break;
    case 3: *ptr_out = ctx->symm + ctx->lay.ret; *bytes_out = static_cast<size_t>(p.S) * p.k * p.H * ctx->eb; break;
    case 4: *ptr_out = const_cast<Route*>(p.routes); *bytes_out = sizeof(Route) * p.S * p.k; break;
    case 5: *ptr_out = p.trace; *bytes_out = sizeof(unsigned long long) * kTraceSlots * ctx->geo.grid; break;
    default: return set_error(FMOE_ERR_INVALID_ARG, "unknown buffer id");
  }
  return FMOE_OK;
}

int fmoe_ctx_destroy(fmoe_ctx* ctx, void* stream) {
  if (ctx == nullptr) return FMOE_OK;
  ScopedDevice on_device(ctx->device);
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  free_ctx(ctx);
  return FMOE_OK;
}

static int forward_impl(fmoe_ctx* ctx, const fmoe_forward_args* a, const fmoe_router_args* ra, void* stream);

int fmoe_forward(fmoe_ctx* ctx, const fmoe_forward_args* a, void* stream) {
  return forward_impl(ctx, a, nullptr, stream);
}

int fmoe_forward_routed(fmoe_ctx* ctx, const fmoe_router_args* ra, const fmoe_forward_args* a, void* stream) {
  if (ra == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  if (ra->weights == nullptr || ra->expert_counts == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "weights and expert_counts are required");
  if (reinterpret_cast<uintptr_t>(ra->weights) & 15)
    return set_error(FMOE_ERR_INVALID_ARG, "the router weights must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(ra->expert_counts) | reinterpret_cast<uintptr_t>(ra->routing) |
       reinterpret_cast<uintptr_t>(ra->logit_bias)) & 3)
    return set_error(FMOE_ERR_INVALID_ARG, "expert_counts, routing and logit_bias must be 4-byte aligned");
  return forward_impl(ctx, a, ra, stream);
}

static int forward_impl(fmoe_ctx* ctx, const fmoe_forward_args* a, const fmoe_router_args* ra, void* stream) {
  if (ctx == nullptr || a == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  if (!ctx->committed) return set_error(FMOE_ERR_NOT_READY, "call fmoe_ctx_commit after importing every peer");
  if (ctx->poisoned)
    return set_error(FMOE_ERR_DEVICE_TIMEOUT, "an earlier forward of this context ran out of a device-side wait "
                                              "(see fmoe_last_status); destroy the context and create a new one");
  const bool gated = ctx->params.gated != 0;
  if (a->tokens == nullptr || (ra == nullptr && a->expert_counts == nullptr) || a->local_expert_up == nullptr ||
      a->local_expert_down == nullptr || a->moe_out == nullptr || (gated && a->local_expert_up_v == nullptr))
    return set_error(FMOE_ERR_INVALID_ARG, "a required device pointer is null");
  if ((reinterpret_cast<uintptr_t>(a->tokens) | reinterpret_cast<uintptr_t>(a->moe_out) |
       reinterpret_cast<uintptr_t>(a->local_expert_up) | reinterpret_cast<uintptr_t>(a->local_expert_up_v) |
       reinterpret_cast<uintptr_t>(a->local_expert_down)) & 15)
    return set_error(FMOE_ERR_INVALID_ARG, "tokens, moe_out and the expert weights must be 16-byte aligned");
  MoeParams p = ctx->params;
  const void* up_v = gated ? a->local_expert_up_v : a->local_expert_up;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ctx->planes == 3) {
    // fp32 weights run as three BF16 planes.  The planes of the weight set seen last are kept, so a
    // layer whose weights stay where they are pays for the split once, not per forward (a caller
    // that rewrites weights in place calls fmoe_weights_changed).
    if (ctx->wsplit_src[0] != a->local_expert_up || ctx->wsplit_src[1] != up_v ||
        ctx->wsplit_src[2] != a->local_expert_down) {
      const size_t n = static_cast<size_t>(p.nLx) * p.I * p.H;
      FMOE_CUDA(launch_split_planes(static_cast<const float*>(a->local_expert_up), ctx->wsplit + ctx->wsplit_up, n, st));
      if (gated)
        FMOE_CUDA(launch_split_planes(static_cast<const float*>(a->local_expert_up_v), ctx->wsplit + ctx->wsplit_up_v, n, st));
      FMOE_CUDA(launch_split_planes(static_cast<const float*>(a->local_expert_down), ctx->wsplit + ctx->wsplit_down, n, st));
      ctx->wsplit_src[0] = a->local_expert_up; ctx->wsplit_src[1] = up_v; ctx->wsplit_src[2] = a->local_expert_down;
    }
  } else {
    const fmoe_ctx::WeightMaps* hit = nullptr;
    for (const auto& wm : ctx->layer_maps)
      if (wm.src[0] == a->local_expert_up && wm.src[1] == up_v && wm.src[2] == a->local_expert_down) { hit = &wm; break; }
    if (hit == nullptr) {
      fmoe_ctx::WeightMaps wm;
      int rc = make_map(&wm.m[0], p.ab_format, a->local_expert_up, static_cast<uint64_t>(p.nLx) * p.I, p.H);
      if (rc == FMOE_OK) rc = make_map(&wm.m[1], p.ab_format, up_v, static_cast<uint64_t>(p.nLx) * p.I, p.H);
      if (rc == FMOE_OK) rc = make_map(&wm.m[2], p.ab_format, a->local_expert_down, static_cast<uint64_t>(p.nLx) * p.H, p.I);
      if (rc != FMOE_OK) return rc;
      wm.src[0] = a->local_expert_up; wm.src[1] = up_v; wm.src[2] = a->local_expert_down;
      if (ctx->layer_maps.size() < FMOE_LAYER_CACHE) {
        ctx->layer_maps.push_back(wm);
        hit = &ctx->layer_maps.back();
      } else {
        ctx->layer_maps[ctx->layer_next] = wm;
        hit = &ctx->layer_maps[ctx->layer_next];
        ctx->layer_next = (ctx->layer_next + 1) % FMOE_LAYER_CACHE;
      }
    }
    ctx->maps[2] = hit->m[0]; ctx->maps[3] = hit->m[1]; ctx->maps[4] = hit->m[2];
  }
  p.tokens = a->tokens; p.expert_counts = a->expert_counts;
  if (ra != nullptr) {   // the router runs as the first phase of this launch
    p.router_w = ra->weights; p.logit_bias = ra->logit_bias; p.routing = ra->routing;
    p.counts_out = ra->expert_counts; p.expert_counts = ra->expert_counts;
  }
  p.bias_up = a->local_bias_up; p.bias_up_v = a->local_bias_up_v; p.bias_down = a->local_bias_down;
  p.out = a->moe_out; p.alpha = a->swish_alpha; p.beta = a->swish_beta;
  if (ctx->spec_launch != nullptr) {
    const cudaError_t e = static_cast<cudaError_t>(ctx->spec_launch(&p, ctx->maps, ctx->geo.grid,
                                                                     static_cast<size_t>(ctx->geo.smem_bytes), st));
    ++g_launches;
    if (e != cudaSuccess)
      return set_error(FMOE_ERR_CUDA, std::string("specialised launch: ") + cudaGetErrorName(e) + " (" +
                                          cudaGetErrorString(e) + ")");
  } else {
    const cudaError_t e = launch_moe(p, ctx->maps, ctx->geo.grid, ctx->geo.smem_bytes, st);
    ++g_launches;
    if (e != cudaSuccess)
      return set_error(FMOE_ERR_CUDA, std::string("launch: ") + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
  }
  return FMOE_OK;
}

int fmoe_ctx_load_specialised(fmoe_ctx* ctx, const char* path) {
  if (ctx == nullptr || path == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (h == nullptr) return set_error(FMOE_ERR_INVALID_ARG, std::string("cannot load ") + path + ": " + dlerror());
  auto info = reinterpret_cast<int (*)(int32_t*)>(dlsym(h, "fmoe_spec_info"));
  auto prepare = reinterpret_cast<int (*)(size_t)>(dlsym(h, "fmoe_spec_prepare"));
  auto launch = reinterpret_cast<int (*)(const void*, const void*, int, size_t, void*)>(dlsym(h, "fmoe_spec_launch"));
  if (info == nullptr || prepare == nullptr || launch == nullptr) {
    dlclose(h);
    return set_error(FMOE_ERR_INVALID_ARG, std::string(path) + " is not a specialised flashmoe_b200 kernel library");
  }
  int32_t v[8] = {};
  info(v);
  const fmoe_model_desc& m = ctx->model;
  const bool same = v[0] == m.token_dim && v[1] == m.ffn_size && v[2] == m.top_k &&
                    v[3] == (m.mlp_type == FMOE_MLP_GATED ? 1 : 0) && v[4] == m.act_type && v[5] == m.data_type &&
                    v[6] == ctx->params.pair && v[7] == static_cast<int32_t>(sizeof(MoeParams));
  if (!same) {
    dlclose(h);
    return set_error(FMOE_ERR_INVALID_ARG, std::string(path) + " was built for another layer description (or another "
                                           "version of the library)");
  }
  ScopedDevice on_device(ctx->device);
  cudaError_t ce = on_device.err;
  if (ce == cudaSuccess) ce = static_cast<cudaError_t>(prepare(static_cast<size_t>(ctx->geo.smem_bytes)));
  if (ce != cudaSuccess) {
    dlclose(h);
    return set_error(FMOE_ERR_CUDA, std::string("specialised kernel set-up: ") + cudaGetErrorString(ce));
  }
  if (ctx->spec_handle != nullptr) dlclose(ctx->spec_handle);
  ctx->spec_handle = h;
  ctx->spec_launch = launch;
  ctx->geo.specialised = 1;
  return FMOE_OK;
}

int fmoe_last_status(fmoe_ctx* ctx, void* stream, fmoe_status* out) {
  if (ctx == nullptr || out == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  FMOE_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  FMOE_CUDA(cudaMemcpy(out, ctx->params.status, sizeof(fmoe_status), cudaMemcpyDeviceToHost));
  if (out->code != FMOE_OK) ctx->poisoned = true;
  return out->code;
}

int fmoe_weights_changed(fmoe_ctx* ctx) {
  if (ctx == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null context");
  ctx->wsplit_src[0] = ctx->wsplit_src[1] = ctx->wsplit_src[2] = nullptr;
  return FMOE_OK;
}

int fmoe_router_create(const fmoe_model_desc* model, int32_t device_id, int32_t return_logits, void* stream,
                       fmoe_router** out) {
  if (out == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "out is null");
  *out = nullptr;
  int rc = validate_model(model);
  if (rc != FMOE_OK) return rc;
  if (model->data_type == FMOE_DT_FP64) return set_error(FMOE_ERR_UNSUPPORTED, "the router handles BF16, FP16 and FP32");
  if (model->token_dim % 8 != 0) return set_error(FMOE_ERR_INVALID_ARG, "token_dim must be a multiple of 8");
  if (static_cast<size_t>(model->num_experts) * 4 * 8 * 4 > 200 * 1024)
    return set_error(FMOE_ERR_UNSUPPORTED, "num_experts too large for the router's shared-memory rows");
  fmoe_router* r = new (std::nothrow) fmoe_router();
  if (r == nullptr) return set_error(FMOE_ERR_NO_MEMORY, "host allocation failed");
  r->model = *model; r->device = device_id; r->return_logits = return_logits;
  ScopedDevice on_device(device_id);
  cudaError_t ce = on_device.err;
  const size_t n = static_cast<size_t>(model->tokens_per_rank) * model->top_k;
  if (ce == cudaSuccess) ce = cudaMalloc(&r->topk_idx, n * sizeof(int32_t));
  if (ce == cudaSuccess) ce = cudaMalloc(&r->topk_w, n * sizeof(float));
  if (ce != cudaSuccess) {
    if (r->topk_idx) cudaFree(r->topk_idx);
    delete r;
    return set_error(FMOE_ERR_CUDA, std::string("router scratch: ") + cudaGetErrorString(ce));
  }
  (void)stream;
  *out = r;
  return FMOE_OK;
}

int fmoe_router_forward(fmoe_router* router, fmoe_ctx* moe, const fmoe_router_args* a, void* stream) {
  if (router == nullptr || moe == nullptr || a == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  if (moe->poisoned)
    return set_error(FMOE_ERR_DEVICE_TIMEOUT, "an earlier forward of this context ran out of a device-side wait "
                                              "(see fmoe_last_status); destroy the context and create a new one");
  if (a->tokens == nullptr || a->weights == nullptr || a->expert_counts == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "tokens, weights and expert_counts are required");
  if (router->return_logits && a->routing == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "this router was created with return_logits: routing is required");
  if ((reinterpret_cast<uintptr_t>(a->tokens) | reinterpret_cast<uintptr_t>(a->weights)) & 15)
    return set_error(FMOE_ERR_INVALID_ARG, "tokens and weights must be 16-byte aligned");
  const fmoe_model_desc& m = router->model;
  const fmoe_model_desc& mm = moe->model;
  if (m.tokens_per_rank != mm.tokens_per_rank || m.num_experts != mm.num_experts || m.top_k != mm.top_k ||
      m.expert_peer_capacity != mm.expert_peer_capacity || m.token_dim != mm.token_dim)
    return set_error(FMOE_ERR_INVALID_ARG, "router and MoE context describe different layers");
  RouterParams p{};
  p.S = m.tokens_per_rank; p.H = m.token_dim; p.E = m.num_experts; p.k = m.top_k;
  p.EC = m.expert_peer_capacity; p.round_ec = moe->geo.round_ec; p.dtype = m.data_type;
  p.tokens = a->tokens; p.weights = a->weights; p.logit_bias = a->logit_bias;
  p.routing = router->return_logits ? a->routing : nullptr;
  p.topk_idx = router->topk_idx; p.topk_w = router->topk_w;
  p.expert_counts = a->expert_counts;
  p.table = const_cast<TokenSlot*>(moe->params.table);
  p.routes = const_cast<Route*>(moe->params.routes);
  FMOE_CUDA(launch_router(p, static_cast<cudaStream_t>(stream)));
  return FMOE_OK;
}

int fmoe_router_destroy(fmoe_router* router, void* stream) {
  if (router == nullptr) return FMOE_OK;
  ScopedDevice on_device(router->device);
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  cudaFree(router->topk_idx);
  cudaFree(router->topk_w);
  delete router;
  return FMOE_OK;
}

int fmoe_forward_host(fmoe_ctx* ctx, fmoe_router* router, const void* tokens_host, void* out_host,
                      const fmoe_router_args* rargs, const fmoe_forward_args* args, void* stream) {
  if (ctx == nullptr || router == nullptr || tokens_host == nullptr || out_host == nullptr ||
      rargs == nullptr || args == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  const size_t bytes = static_cast<size_t>(ctx->params.S) * ctx->params.H * ctx->eb;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ctx->stage_tokens == nullptr) {
    ScopedDevice on_device(ctx->device);
    FMOE_CUDA(on_device.err);
    FMOE_CUDA(cudaMalloc(&ctx->stage_tokens, bytes));
    FMOE_CUDA(cudaMalloc(&ctx->stage_out, bytes));
  }
  FMOE_CUDA(cudaMemcpyAsync(ctx->stage_tokens, tokens_host, bytes, cudaMemcpyHostToDevice, st));
  fmoe_router_args ra = *rargs;
  ra.tokens = ctx->stage_tokens;
  int rc = fmoe_router_forward(router, ctx, &ra, stream);
  if (rc != FMOE_OK) return rc;
  fmoe_forward_args fa = *args;
  fa.tokens = ctx->stage_tokens;
  fa.moe_out = ctx->stage_out;
  rc = fmoe_forward(ctx, &fa, stream);
  if (rc != FMOE_OK) return rc;
  FMOE_CUDA(cudaMemcpyAsync(out_host, ctx->stage_out, bytes, cudaMemcpyDeviceToHost, st));
  FMOE_CUDA(cudaStreamSynchronize(st));
  return FMOE_OK;
}

int fmoe_forward_host_async(fmoe_ctx* ctx, fmoe_router* router, const void* tokens_host, void* out_host,
                            const fmoe_router_args* rargs, const fmoe_forward_args* args, void* stream) {
  if (ctx == nullptr || router == nullptr || tokens_host == nullptr || out_host == nullptr ||
      rargs == nullptr || args == nullptr)
    return set_error(FMOE_ERR_INVALID_ARG, "null argument");
  const size_t bytes = static_cast<size_t>(ctx->params.S) * ctx->params.H * ctx->eb;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  fmoe_ctx::Pipe& pp = ctx->pipe;
  if (!pp.ready) {
    ScopedDevice on_device(ctx->device);
    FMOE_CUDA(on_device.err);
    FMOE_CUDA(cudaStreamCreateWithFlags(&pp.s_in, cudaStreamNonBlocking));
    FMOE_CUDA(cudaStreamCreateWithFlags(&pp.s_out, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      FMOE_CUDA(cudaMalloc(&pp.tokens[i], bytes));
      FMOE_CUDA(cudaMalloc(&pp.out[i], bytes));
      FMOE_CUDA(cudaEventCreateWithFlags(&pp.in_done[i], cudaEventDisableTiming));
      FMOE_CUDA(cudaEventCreateWithFlags(&pp.compute_done[i], cudaEventDisableTiming));
      FMOE_CUDA(cudaEventCreateWithFlags(&pp.out_done[i], cudaEventDisableTiming));
    }
    pp.ready = true;
  }
  const int slot = static_cast<int>(pp.submitted & 1);
  const bool reused = pp.submitted >= 2;   // the slot's previous user is step n - 2
  // copy-in: the slot's token buffer is free once the kernels of step n - 2 are done
  if (reused) FMOE_CUDA(cudaStreamWaitEvent(pp.s_in, pp.compute_done[slot], 0));
  FMOE_CUDA(cudaMemcpyAsync(pp.tokens[slot], tokens_host, bytes, cudaMemcpyHostToDevice, pp.s_in));
  FMOE_CUDA(cudaEventRecord(pp.in_done[slot], pp.s_in));
  // kernels: after this step's tokens are in and step n - 2's result has left the slot
  FMOE_CUDA(cudaStreamWaitEvent(st, pp.in_done[slot], 0));
  if (reused) FMOE_CUDA(cudaStreamWaitEvent(st, pp.out_done[slot], 0));
  fmoe_router_args ra = *rargs;
  ra.tokens = pp.tokens[slot];
  int rc = fmoe_router_forward(router, ctx, &ra, stream);
  if (rc != FMOE_OK) return rc;
  fmoe_forward_args fa = *args;
  fa.tokens = pp.tokens[slot];
  fa.moe_out = pp.out[slot];
  rc = fmoe_forward(ctx, &fa, stream);
  if (rc != FMOE_OK) return rc;
  FMOE_CUDA(cudaEventRecord(pp.compute_done[slot], st));
  // copy-out
  FMOE_CUDA(cudaStreamWaitEvent(pp.s_out, pp.compute_done[slot], 0));
  FMOE_CUDA(cudaMemcpyAsync(out_host, pp.out[slot], bytes, cudaMemcpyDeviceToHost, pp.s_out));
  FMOE_CUDA(cudaEventRecord(pp.out_done[slot], pp.s_out));
  ++pp.submitted;
  return FMOE_OK;
}

int fmoe_forward_host_wait(fmoe_ctx* ctx, void* stream) {
  if (ctx == nullptr) return set_error(FMOE_ERR_INVALID_ARG, "null context");
  FMOE_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (ctx->pipe.ready) {
    FMOE_CUDA(cudaStreamSynchronize(ctx->pipe.s_in));
    FMOE_CUDA(cudaStreamSynchronize(ctx->pipe.s_out));
  }
  return FMOE_OK;
}

}  // extern "C"
