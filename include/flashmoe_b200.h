/*
 * flashmoe_b200 -- C ABI of the B200-native MoE-layer forward.
 *
 * One shared library (libflashmoe_b200.so) exports exactly these entry points.  Every
 * pointer argument that is documented as "device" is a plain device address; nothing in
 * this interface carries a framework type.  Every function returns an fmoe_status_code
 * (0 = success); no entry point throws, exits or terminates the process.
 *
 * Each declaration names the reference interface it replaces (paths inside the
 * hnts03-moreh/FlashMoE project).  In the reference those are the functions a JIT-built
 * pybind11 module exports per model description (flashmoe/bindings.py:154-185, 300-315)
 * on top of the C++ host API (csrc/include/flashmoe/bootstrap.cuh, moe.cuh).
 */
#ifndef FLASHMOE_B200_H
#define FLASHMOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FMOE_MAX_WORLD 8          /* ranks of one NVSwitch box */
#define FMOE_IPC_HANDLE_BYTES 64  /* sizeof(cudaIpcMemHandle_t) */

typedef struct fmoe_ctx fmoe_ctx;       /* replaces flashmoe::Context (context.cuh:16-52) */
typedef struct fmoe_router fmoe_router; /* replaces flashmoe::GateContext (context.cuh:54-59) */

typedef enum fmoe_status_code {
  FMOE_OK = 0,
  FMOE_ERR_INVALID_ARG = 1,    /* reference: std::invalid_argument / std::runtime_error */
  FMOE_ERR_UNSUPPORTED = 2,    /* shape, dtype, arch or topology this build does not handle */
  FMOE_ERR_CUDA = 3,           /* a CUDA runtime or driver call failed (reference: exit(1)) */
  FMOE_ERR_NOT_READY = 4,      /* peers not imported / context not committed */
  FMOE_ERR_DEVICE_TIMEOUT = 5, /* a bounded device-side wait ran out (reference: spins forever) */
  FMOE_ERR_NO_MEMORY = 6
} fmoe_status_code;

/* enum values of flashmoe/jit.py:22-40 */
enum { FMOE_TOPO_NVLINK_ONLY = 0, FMOE_TOPO_MIXED = 1 };
enum { FMOE_MLP_GATED = 0, FMOE_MLP_VANILLA = 1 };
enum { FMOE_DT_BF16 = 0, FMOE_DT_FP16 = 1, FMOE_DT_FP32 = 2, FMOE_DT_FP64 = 3 };
enum { FMOE_ACT_IDENTITY = 0, FMOE_ACT_SILU = 1, FMOE_ACT_GELU = 2, FMOE_ACT_RELU = 3 };

/* The compile-time constants of a reference module (flashmoe/bindings.py:34-46), at run time. */
typedef struct fmoe_model_desc {
  int32_t tokens_per_rank;      /* S */
  int32_t token_dim;            /* H */
  int32_t ffn_size;             /* I */
  int32_t num_experts;          /* E */
  int32_t top_k;                /* k */
  int32_t expert_peer_capacity; /* EC: rows one rank may send to one expert */
  int32_t data_type;            /* FMOE_DT_* */
  int32_t mlp_type;             /* FMOE_MLP_* */
  int32_t act_type;             /* FMOE_ACT_* */
  int32_t gpu_arch;             /* compute capability * 100; only 1000 and 1030 accepted */
} fmoe_model_desc;

/* Arguments of moe_initialize (flashmoe/bindings.py:68-110). */
typedef struct fmoe_ep_desc {
  int32_t ep_world;
  int32_t ep_rank;
  int32_t my_pe;
  int32_t device_id;
  int32_t num_local_experts;
  int32_t topology;           /* FMOE_TOPO_*; only NVLINK_ONLY is implemented */
  const int32_t* expert_map;  /* host, [num_experts]: expert -> ep rank */
  const int32_t* rank_map;    /* host, [ep_world]: ep rank -> global rank */
} fmoe_ep_desc;

/* Arguments of moe_forward (flashmoe/bindings.py:112-140); all pointers device. */
typedef struct fmoe_forward_args {
  const void* tokens;            /* [S, H] Element */
  const int32_t* expert_counts;  /* [E], written by the router */
  const void* local_expert_up;   /* [nLx, I, H] activated branch */
  const void* local_expert_up_v; /* [nLx, I, H] linear branch; null for a plain MLP */
  const void* local_bias_up;     /* [nLx, I]; null = zero bias */
  const void* local_bias_up_v;   /* [nLx, I]; null = zero bias */
  const void* local_expert_down; /* [nLx, H, I] */
  const void* local_bias_down;   /* [nLx, H]; null = zero bias */
  void* moe_out;                 /* [S, H] Element */
  float swish_alpha;
  float swish_beta;
} fmoe_forward_args;

/* Arguments of gate_forward (flashmoe/bindings.py:266-290); all pointers device. */
typedef struct fmoe_router_args {
  const void* tokens;      /* [S, H] Element */
  const void* weights;     /* [E, H] Element */
  float* routing;          /* [S, E] fp32 softmax probabilities, or null */
  int32_t* expert_counts;  /* [E] out: tokens that chose each expert (not clamped) */
  const float* logit_bias; /* [E] fp32 added to the logits, or null (not in the reference) */
} fmoe_router_args;

/* What a device-side wait recorded when it gave up (no counterpart: the reference traps). */
typedef struct fmoe_status {
  int32_t code;   /* fmoe_status_code */
  int32_t phase;  /* which wait: see FMOE_PHASE_* */
  int32_t rank;
  int32_t cta;
  int64_t detail; /* wait-specific: tile id, peer rank, ... */
  uint64_t epoch; /* forward number on this context */
} fmoe_status;
enum {
  FMOE_PHASE_NONE = 0, FMOE_PHASE_COUNTS = 1, FMOE_PHASE_DISPATCH_ARRIVAL = 2,
  FMOE_PHASE_GEMM0_DONE = 3, FMOE_PHASE_RETURN_ARRIVAL = 4, FMOE_PHASE_PIPE_FULL = 5,
  FMOE_PHASE_PIPE_EMPTY = 6, FMOE_PHASE_TMEM_FULL = 7, FMOE_PHASE_TMEM_EMPTY = 8,
  FMOE_PHASE_TASK = 9, FMOE_PHASE_ROUTING = 10
};

/* --- context life cycle -------------------------------------------------------------- */

/* Replaces flashmoe::initialize (bootstrap.cuh:197-374) minus the peer exchange: validates
 * the description, allocates this rank's symmetric block (token landing area, return area,
 * count tables, arrival counters) and its private workspace.  `stream` is a cudaStream_t. */
int fmoe_ctx_create(const fmoe_model_desc* model, const fmoe_ep_desc* ep, void* stream,
                    fmoe_ctx** out);

/* Replaces flashmoe::getWorkspaceBytes (bootstrap.cuh:377-410): what fmoe_ctx_create would
 * allocate for this description on this rank, without allocating or touching a device:
 * the symmetric block and the private workspace (for FP32 layers including the BF16 planes of
 * the expert weights).  Same argument checks as fmoe_ctx_create; expert_map / rank_map may be
 * null.  Either output may be null. */
int fmoe_workspace_bytes(const fmoe_model_desc* model, const fmoe_ep_desc* ep,
                         int64_t* symm_bytes_out, int64_t* workspace_bytes_out);

/* The same with memory the CALLER owns, sized by fmoe_workspace_bytes (the reference's
 * getWorkspaceBytes exists so that a serving engine can budget, bootstrap.cuh:377-410; here it can
 * also place): `symm_mem` (>= symm bytes) becomes the symmetric block, `work_mem` (>= workspace
 * bytes) the private workspace; both 1024-byte aligned device memory, and `symm_mem` the start of
 * an allocation of its own when other ranks are to map it (CUDA IPC shares whole allocations).
 * Nothing is allocated on the device by this call or by fmoe_forward / fmoe_router_forward on the
 * context, and fmoe_ctx_destroy leaves the two blocks to the caller.  (The host-buffer entry
 * points fmoe_forward_host* still allocate their staging buffers on first use.) */
int fmoe_ctx_create_in(const fmoe_model_desc* model, const fmoe_ep_desc* ep, void* stream, void* symm_mem,
                       size_t symm_bytes, void* work_mem, size_t work_bytes, fmoe_ctx** out);

/* Replaces nvshmem_malloc + nvshmem_ptr (bootstrap.cuh:141-151, 239-249): the symmetric
 * block is an ordinary device allocation shared through CUDA IPC.  Export this rank's
 * handle, gather the handles by any host-side means, import every peer's, then commit.
 * With ep_world == 1 only fmoe_ctx_commit is needed. */
int fmoe_symm_bytes(const fmoe_ctx* ctx, size_t* bytes);
int fmoe_symm_export(fmoe_ctx* ctx, void* handle_out /* FMOE_IPC_HANDLE_BYTES */);
int fmoe_symm_import(fmoe_ctx* ctx, int32_t peer_ep_rank, const void* handle);
/* Peers living in the same process (tests): hand over the peer's base address directly. */
int fmoe_symm_base(fmoe_ctx* ctx, void** base_out);
int fmoe_symm_set_peer(fmoe_ctx* ctx, int32_t peer_ep_rank, void* peer_base);
int fmoe_ctx_commit(fmoe_ctx* ctx);

/* Replaces get_tIdx (flashmoe/bindings.py:142-144): device address of the routing table
 * [E, roundEC] of {uint32 token, float weight} the router fills. */
int fmoe_token_indices(fmoe_ctx* ctx, void** table_out);

/* Replaces flashmoe::finalize (bootstrap.cuh:450-474). */
int fmoe_ctx_destroy(fmoe_ctx* ctx, void* stream);

/* --- the hot path -------------------------------------------------------------------- */

/* Replaces moe::forwardHost / moe_forward (moe.cuh:255-260; flashmoe/bindings.py:112-140):
 * one launch of the persistent kernel (dispatch, expert GEMMs, combine) on `stream`.
 * Every rank of the group must call it the same number of times.  `stream` belongs to the
 * context's device, and that device is the calling thread's current one, as for any launch
 * (the calls that create, map or destroy things make the device current themselves and put the
 * caller's back before they return).
 * One context serves every layer of a model that shares this description: forwards on a
 * stream are ordered, the epoch protocol needs nothing cleared between them, and the TMA
 * descriptors of up to FMOE_LAYER_CACHE distinct (up, up_v, down) weight sets are kept, so
 * alternating between layers costs no descriptor encoding (the reference builds one Context
 * per layer, each with its own symmetric heap). */
#define FMOE_LAYER_CACHE 128
int fmoe_forward(fmoe_ctx* ctx, const fmoe_forward_args* args, void* stream);

/* The reference's fused gate is a launch of its own and leaves "emit the top-k indices ... and fuse
 * with the consumer" as a note (gate.cuh:554).  Here the consumer can take the router in: ONE launch
 * that opens with the router (logits, softmax, top-k, slots, routing table: the arithmetic of
 * fmoe_router_forward, bit for bit, run by the persistent kernel's own warps with two grid
 * barriers) and goes on with dispatch, experts and combine.  `rargs->tokens` is ignored
 * (`args->tokens` are routed); `rargs->expert_counts` is written and `args->expert_counts` ignored;
 * `rargs->routing` ([S, E] probabilities) is written when non-null.  Meant for decode-sized
 * batches, where two extra launches cost as much as the layer; for large batches the router
 * kernels, which fill the SMs with many more warps, are faster. */
int fmoe_forward_routed(fmoe_ctx* ctx, const fmoe_router_args* rargs, const fmoe_forward_args* args,
                        void* stream);

/* Replaces the per-model JIT module of the reference (flashmoe/jit.py:188-296, bindings.py:34-46:
 * shapes as constexpr): `path` is a shared library built from the same kernel source with the
 * layer's H, I, top-k, MLP type, activation, element type and tile form fixed at compile time
 * (flashmoe_b200.jit builds and caches them).  The library is checked against this context's
 * description and refused if it differs; on success fmoe_forward launches the specialised kernel
 * instead of the generic one.  Results are bit-identical either way. */
int fmoe_ctx_load_specialised(fmoe_ctx* ctx, const char* path);

/* No counterpart in the reference (its FP32 kernels read fp32 weights directly).  An FP32 context
 * runs the expert GEMMs on BF16 tensor cores with every weight held as three BF16 planes; it keeps
 * the planes of the weight set it saw last, keyed by the three weight addresses, so the split is
 * paid once per weight set and not per forward.  Call this after rewriting weights IN PLACE (same
 * addresses); the next forward splits them again.  A no-op for BF16 / FP16 contexts. */
int fmoe_weights_changed(fmoe_ctx* ctx);

/* Replaces initializeGate / gate_initialize (bootstrap.cuh:413-447; bindings.py:238-264). */
int fmoe_router_create(const fmoe_model_desc* model, int32_t device_id, int32_t return_logits,
                       void* stream, fmoe_router** out);
/* Replaces gate::forwardKernel launch / gate_forward (gate.cuh:588-608; bindings.py:266-290).
 * Writes expert_counts, the routing table of `moe` and `moe`'s per-token route records. */
int fmoe_router_forward(fmoe_router* router, fmoe_ctx* moe, const fmoe_router_args* args,
                        void* stream);
/* Replaces finalizeGate / gate_finalize (bootstrap.cuh:434-447). */
int fmoe_router_destroy(fmoe_router* router, void* stream);

/* No counterpart in the reference.  The router for callers that must not allocate device memory
 * (an engine whose memory pool owns the whole GPU, a plug-in running between the engine's own
 * launches): same kernels and same results as fmoe_router_forward, but no router context and no
 * cudaMalloc/cudaFree anywhere on the path.  The two scratch arrays the router needs live in a
 * fixed device array inside the library (1 MiB per GPU that loads it, held until exit), which
 * limits a call to tokens_per_rank * top_k <= 131072; larger layers get FMOE_ERR_UNSUPPORTED.
 * The caller passes every input and output: `a->routing` is written when non-null, `token_table`
 * is the [num_experts, round_ec] table of {uint32 token, float weight} (round_ec >=
 * expert_peer_capacity), `routes` the [tokens_per_rank, top_k] records of {int32 expert, int32
 * slot, float weight, int32 pad}, 16-byte aligned.  The first call on a device looks up the
 * array's device address, once.  All calls on a device
 * share the one array: it keeps the last call's contents (nothing in it has to start at zero), and
 * two calls whose kernels overlap on the GPU (different streams, no ordering between them) race on
 * it, so order them. */
int fmoe_router_forward_static(const fmoe_model_desc* model, int32_t device_id,
                               const fmoe_router_args* a, void* token_table, int32_t round_ec,
                               void* routes, void* stream);

/* The call sequence of quickstart.py:150-153 with HOST buffers: copies `tokens_host`
 * (pinned or pageable, [S, H] Element) to the device, runs router + forward, copies the
 * [S, H] result to `out_host` and synchronises `stream`.  `args->tokens`, `args->moe_out`
 * and `rargs->tokens` are ignored (internal staging buffers are used). */
int fmoe_forward_host(fmoe_ctx* ctx, fmoe_router* router, const void* tokens_host,
                      void* out_host, const fmoe_router_args* rargs,
                      const fmoe_forward_args* args, void* stream);

/* The same step without waiting for it: the copy-in of step n runs on a stream of its own and
 * overlaps the kernels of step n - 1, the copy-out overlaps the kernels of step n + 1 (two
 * staging slots; `tokens_host` may be reused once the call returns only if it is not rewritten
 * before the copy-in ran, so alternate two host buffers; `out_host` holds step n's result after
 * fmoe_forward_host_wait, or once two later steps have been submitted and waited for).
 * The kernels run on `stream`; every rank must submit the same number of steps. */
int fmoe_forward_host_async(fmoe_ctx* ctx, fmoe_router* router, const void* tokens_host,
                            void* out_host, const fmoe_router_args* rargs,
                            const fmoe_forward_args* args, void* stream);
/* Blocks until every submitted step, its copies included, is done. */
int fmoe_forward_host_wait(fmoe_ctx* ctx, void* stream);

/* --- diagnostics --------------------------------------------------------------------- */

/* Reads the record the last forward left (synchronises `stream` first).  A record with a non-zero
 * code marks the context as poisoned: from then on fmoe_forward and fmoe_router_forward on it
 * return FMOE_ERR_DEVICE_TIMEOUT without launching; destroy it and create a new one (on every
 * rank of the group). */
int fmoe_last_status(fmoe_ctx* ctx, void* stream, fmoe_status* out);
const char* fmoe_strerror(int code);
/* Last host-side error message of the calling thread (empty string if none). */
const char* fmoe_last_error(void);
/* Number of kernels this library has launched in this process (all contexts). */
uint64_t fmoe_launch_count(void);

/* Geometry chosen at create time, for tests and benchmarks. */
typedef struct fmoe_geometry {
  int32_t tile_m, tile_n0, tile_n1, tile_k, stages;
  int32_t round_ec;        /* row stride of the routing table */
  int32_t landing_rows;    /* rows of the token landing area */
  int32_t grid, threads;   /* launch shape of the persistent kernel */
  int32_t smem_bytes;
  int32_t cta_pairs;       /* 1: tiles are worked by CTA pairs (cta_group::2), 0: by single CTAs */
  int32_t split_parts;     /* K parts per GEMM1 tile of the closing wave (1: no tile is cut) */
  int64_t symm_bytes, workspace_bytes;
  int32_t specialised;     /* 1: forwards run a kernel compiled for this layer's description */
  int32_t reserved;
} fmoe_geometry;
int fmoe_get_geometry(const fmoe_ctx* ctx, fmoe_geometry* out);

/* Device addresses of internal buffers, for stage-by-stage parity tests.
 * which: 0 landing rows [landing_rows, H], 1 landing meta [landing_rows] u32,
 *        2 GEMM0 output [landing_rows, I], 3 return rows [S*k, H],
 *        4 route records [S, k] of {int32 expert, int32 slot, float weight},
 *        5 phase stamps of the last forward: uint64 [grid][16] %globaltimer nanoseconds per CTA
 *          (0 start, 1 all ranks' counts in, 2 task order built (warp 0), 3 this CTA's dispatch
 *           warps done (may precede 2), 4 last ticket drawn, 5 this CTA's last task finished, 6 all returns in,
 *           7 combine done, 8 first operand tiles of the CTA's first task landed (0: it had none),
 *           9, 10, 11 the epilogue of the CTA's last task: accumulator ready, rows stored, owners
 *           told; 12..15 unused) */
int fmoe_debug_buffer(fmoe_ctx* ctx, int32_t which, void** ptr_out, size_t* bytes_out);

#ifdef __cplusplus
}
#endif
#endif /* FLASHMOE_B200_H */
