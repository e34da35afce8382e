/*
 * infmoe_c.h -- C ABI of the B200-native MoE layer (libinfmoe_b200.so).
 *
 * Everything the TensorRT-facing plugin classes (MoELayerPlugin /
 * MoELayerPluginCreator) and the Python binding need is reached through the
 * entry points below: plain pointers and sizes, no C++ or framework types.
 * Each declaration names the reference interface it replaces (paths are
 * relative to the InfMoE repository root).
 *
 * Conventions
 *   - every function returns an infmoe_status (0 = ok) and never exits or
 *     throws; infmoe_last_error() gives a thread-local message;
 *   - pointers named d_* are device pointers on the current CUDA device,
 *     h_* are host pointers; `stream` is a cudaStream_t passed as void*;
 *   - all tensors are FP32, row-major, indices are int32;
 *   - work is ordered on `stream`; unless a function says so it does not
 *     block the host.
 */
#ifndef INFMOE_C_H
#define INFMOE_C_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define INFMOE_API __attribute__((visibility("default")))

typedef enum infmoe_status {
    INFMOE_OK = 0,
    INFMOE_ERR_INVALID_ARGUMENT = 1, /* reference: assert(false) after a message on stderr */
    INFMOE_ERR_CUDA = 2,             /* reference: CUDA_SAFE_CALL -> exit(-1), plugin/utility.h:15-21 */
    INFMOE_ERR_NAN = 3,              /* a token selected no expert; reference: device assert, plugin/cuda/moe.cu:70 */
    INFMOE_ERR_IO = 4,               /* weight file missing / unreadable */
    INFMOE_ERR_FORMAT = 5,           /* npz / serialised blob malformed, wrong shapes or dtypes */
    INFMOE_ERR_UNSUPPORTED = 6,
    INFMOE_ERR_DEVICE_TIMEOUT = 7,   /* a bounded device-side wait ran out */
    INFMOE_ERR_STATE = 8             /* call order violated (e.g. enqueue before initialize) */
} infmoe_status;

/* Thread-local description of the last non-zero status returned on this thread. */
INFMOE_API const char* infmoe_last_error(void);

/* ------------------------------------------------------------------------ */
/* Layer object = what MoELayerPlugin holds (plugin/MoELayerPlugin.h:45-80)  */
/* ------------------------------------------------------------------------ */
typedef struct infmoe_layer infmoe_layer;

/* The nine plugin attributes, plugin/MoELayerPluginCreator.cc:15-47 (parsed at :75-115). */
typedef struct infmoe_layer_config {
    int32_t expert_count;
    int32_t embedding_size;            /* d_model */
    int32_t hidden_size;               /* d_ff */
    int32_t max_concurrency;           /* number of device weight slots when experts are streamed; default 2 */
    const float* expert_centroids;     /* host, [expert_count][embedding_size] row-major (MoELayerPlugin.cc:334-336) */
    const float* layernorm_weight;     /* host, [embedding_size]; required iff moe_variant == "cpm_2" */
    const char* expert_weight_file;    /* npz path; may be NULL if weights are given with infmoe_layer_set_expert */
    const char* expert_sublayer_type;  /* "T5_FF" or "Identity" */
    const char* moe_variant;           /* "cpm_2", "base_layer" or "default" */
} infmoe_layer_config;

/* MoELayerPluginCreator::createPlugin + MoELayerPlugin main constructor
 * (plugin/MoELayerPluginCreator.cc:58-148, plugin/MoELayerPlugin.cc:60-81).
 * Copies the arrays and strings.  No device work. */
INFMOE_API int infmoe_layer_create(const infmoe_layer_config* cfg, infmoe_layer** out);

/* MoELayerPlugin::clone (plugin/MoELayerPlugin.cc:83-102,465-468): deep-copies
 * centroids / layernorm weight, shares the expert weights. */
INFMOE_API int infmoe_layer_clone(const infmoe_layer* src, infmoe_layer** out);

/* MoELayerPlugin::initialize -> T5FFLayer::initialize (plugin/sublayers/T5FFLayer.cc:143-147):
 * reads the whole npz into pinned host memory.  Keys "{n}/layer_norm_weight",
 * "{n}/wi_0_weight", "{n}/wi_1_weight", "{n}/wo_weight" (T5FFLayer.cc:55-88). */
INFMOE_API int infmoe_layer_initialize(infmoe_layer* layer);

/* Gives one expert's weights by pointer instead of through the npz (host or
 * device pointers; they are copied).  ln_w [D], wi0/wi1 [F][D], wo [D][F].
 * With on_device != 0 the data is taken from device memory straight into the
 * resident device store (no host copy is kept).  No reference counterpart: the
 * reference only reads npz files. */
INFMOE_API int infmoe_layer_set_expert(infmoe_layer* layer, int32_t expert, const float* ln_w, const float* wi0,
                                       const float* wi1, const float* wo, int on_device);

/* For a layer that holds a contiguous share of a larger layer's experts (one rank of an expert-parallel layer):
 * expert n of this layer is expert first_expert + n of the weight file; infmoe_layer_initialize then reads only
 * those.  No reference counterpart (single GPU). */
INFMOE_API int infmoe_layer_set_file_expert_offset(infmoe_layer* layer, int32_t first_expert);

/* Residency of expert weights.  mode 0: stream every used expert from pinned
 * host memory on every call through max_concurrency slots, like the reference
 * (plugin/MoELayerPlugin.cc:360-394); mode 1: keep all experts in device
 * memory owned by the layer; mode -1: choose 1 when they fit. */
INFMOE_API int infmoe_layer_set_residency(infmoe_layer* layer, int mode);

/* Expert cache of the streamed mode; no counterpart in the reference, whose max_concurrency slots forget their
 * expert after every call (plugin/MoELayerPlugin.cc:360-402 copies every used expert on every enqueue) and which
 * leaves smarter scheduling as a TODO.  slots > 0: the layer keeps that many experts (at least max_concurrency) in
 * device memory of its own across enqueue calls, replacing the least recently used one on a miss, so a decode
 * loop that keeps hitting the same experts stops paying for the host->device copies; slots = 0 (default): off.
 * Device memory: slots x 12 * d_model * d_ff bytes, allocated at the next streamed enqueue. */
INFMOE_API int infmoe_layer_set_expert_cache(infmoe_layer* layer, int32_t slots);
/* Diagnostic, no counterpart in the reference: launches one warp that waits on a barrier nothing completes,
 * through the bounded wait every role of the expert GEMM uses, with a limit of limit_ms (1..2000) instead of the
 * GEMM's 4 s.  timed_out = 1 when the wait gave up and raised the status bit that infmoe_layer_sync_status
 * reports as INFMOE_ERR_DEVICE_TIMEOUT; waited_ms = how long the warp waited.  The context stays usable. */
INFMOE_API int infmoe_wait_timeout_probe(uint32_t limit_ms, int32_t* timed_out, float* waited_ms);

/* Host-only companion of the expert cache (no GPU needed, no counterpart in the reference): replays `calls`
 * enqueue calls against a cache of `slots` slots with the layer's own replacement policy and reports how many
 * experts each call would have to copy.  experts: the active expert ids of all calls back to back, ascending
 * inside a call; call_sizes[c]: how many of them belong to call c.  For sizing the cache from a routing trace. */
INFMOE_API int infmoe_expert_cache_simulate(int32_t slots, int32_t expert_count, const int32_t* experts,
                                            const int32_t* call_sizes, int32_t calls, int32_t* loads_per_call);
/* Expert weight bytes enqueue has copied host -> device for this layer object so far (streamed mode). */
INFMOE_API int infmoe_layer_weight_h2d_bytes(const infmoe_layer* layer, uint64_t* bytes);

/* MoELayerPlugin::getWorkspaceSize (plugin/MoELayerPlugin.cc:253-273) for token_num = B * S. */
INFMOE_API int infmoe_layer_workspace_bytes(const infmoe_layer* layer, int64_t token_num, size_t* bytes);

/* MoELayerPlugin::enqueue (plugin/MoELayerPlugin.cc:279-416).  d_input and
 * d_output are [token_num][embedding_size] and must not alias.  The status of
 * device-side checks (NaN routing, bounded waits) of this call is returned by
 * the next infmoe_layer_sync_status. */
INFMOE_API int infmoe_layer_enqueue(infmoe_layer* layer, const float* d_input, float* d_output, void* d_workspace,
                                    size_t workspace_bytes, int64_t token_num, void* stream);

/* The experts alone, for rows whose expert is already known: d_y[i,:] = expert d_expert_of_row[i] applied to
 * d_rows[i,:] (T5FFLayer::run, plugin/sublayers/T5FFLayer.cc:90-141, grouped over all experts of this layer).
 * Rows may come in any order; results come back in the same order; no routing and no score mix.  This is what an
 * expert-parallel rank runs on the rows it received from the other ranks (the reference has no multi-GPU path).
 * Workspace as for infmoe_layer_enqueue with token_num = rows. */
INFMOE_API int infmoe_layer_expert_forward(infmoe_layer* layer, const float* d_rows, const int32_t* d_expert_of_row,
                                           float* d_y, void* d_workspace, size_t workspace_bytes, int64_t rows,
                                           void* stream);

/* infmoe_layer_expert_forward with the combine step of the expert-parallel path folded in: the result of row i is
 * written to the address d_row_dst[i] (embedding_size floats), which may lie in another GPU's memory that this
 * process has mapped (peer access / CUDA IPC) -- the owner of the experts stores each row straight into the output
 * buffer of the rank the token came from, instead of returning rows for a second all-to-all.  d_row_score (or NULL):
 * the routing scores of the rows; passing them asks for the base_layer output mix
 * out = sigmoid(score) * expert(row) + (1 - sigmoid(score)) * row (plugin/cuda/moe.cu:115-127), whatever the
 * variant this layer object was created with.  No counterpart in the reference (single GPU). */
INFMOE_API int infmoe_layer_expert_forward_scatter(infmoe_layer* layer, const float* d_rows,
                                                   const int32_t* d_expert_of_row, const float* d_row_score,
                                                   const uint64_t* d_row_dst, void* d_workspace,
                                                   size_t workspace_bytes, int64_t rows, void* stream);

/* Blocks until `stream` is idle and returns the device-side status of the calls enqueued so far. */
INFMOE_API int infmoe_layer_sync_status(infmoe_layer* layer, void* stream);

/* Host-buffer convenience: copies h_input to the device, runs enqueue with an
 * internally owned workspace, copies the result to h_output and waits.  This
 * is the end-to-end call the benchmark times. */
INFMOE_API int infmoe_layer_forward_host(infmoe_layer* layer, const float* h_input, float* h_output,
                                         int64_t token_num);
/* The same without waiting (no reference counterpart): the step's upload, pass and result transfer are enqueued and
 * the call returns; infmoe_layer_wait_host blocks until the OLDEST submitted step's result is in its h_output and
 * returns that step's status.  At most two steps may be in flight: the upload of one then runs behind the pass of
 * the one before.  Buffers should be page-locked (the result is then written into h_output by the last kernel of the
 * pass itself) and must stay untouched until the step has been waited for.  infmoe_layer_forward_host refuses to
 * run while steps are in flight.  With streamed experts a pass waits for its weight copies on the host: submit then
 * takes as long as the pass, and a token without an expert is reported by submit itself (the step is not in flight
 * afterwards). */
INFMOE_API int infmoe_layer_submit_host(infmoe_layer* layer, const float* h_input, float* h_output, int64_t token_num);
INFMOE_API int infmoe_layer_wait_host(infmoe_layer* layer);

/* Routing/dispatch results of the last enqueue (device pointers inside the
 * workspace of that call; valid until the next enqueue).  Any out pointer may be NULL. */
INFMOE_API int infmoe_layer_last_routing(const infmoe_layer* layer, const int32_t** d_gate, const float** d_score,
                                         const int32_t** d_pos, const int32_t** d_count, const int32_t** d_offset);

/* Per-stage device timing.  When enabled, enqueue records CUDA events on the
 * caller's stream around its stages (a ring of the last 64 calls).
 * infmoe_layer_stage_ms waits for those calls and returns the average
 * milliseconds of: routing, dispatch, scatter, expert GEMM 1 (wi_0/wi_1 + gelu),
 * expert GEMM 2 (wo + residual), combine -- ms[6] -- then restarts the ring.
 * With streamed experts the two GEMM entries are reported together in ms[3]. */
INFMOE_API int infmoe_layer_set_profiling(infmoe_layer* layer, int enable);
INFMOE_API int infmoe_layer_stage_ms(infmoe_layer* layer, float* ms, int32_t* calls);

/* Number of kernels this library launched on behalf of `layer` so far. */
INFMOE_API int64_t infmoe_layer_kernel_launches(const infmoe_layer* layer);

/* MoELayerPlugin::terminate + destructor (plugin/MoELayerPlugin.cc:203-237). */
INFMOE_API int infmoe_layer_destroy(infmoe_layer* layer);

/* MoELayerPlugin::getSerializationSize / serialize / deserialising constructor
 * (plugin/MoELayerPlugin.cc:418-458, :104-143).  Same fields in the same order,
 * in a self-consistent versioned blob. */
INFMOE_API int infmoe_layer_serialization_size(const infmoe_layer* layer, size_t* bytes);
INFMOE_API int infmoe_layer_serialize(const infmoe_layer* layer, void* h_buffer, size_t bytes);
INFMOE_API int infmoe_layer_deserialize(const void* h_buffer, size_t bytes, infmoe_layer** out);

/* Walks an expert weight file exactly like infmoe_layer_initialize (same reader,
 * same key and size checks as plugin/sublayers/T5FFLayer.cc:55-88) without
 * keeping the data or touching CUDA.  h_sums (may be NULL) receives, per expert,
 * the double-precision sums of its four tensors in the order layer_norm, wi_0,
 * wi_1, wo: [expert_count][4]. */
INFMOE_API int infmoe_weight_file_check(const char* path, int32_t expert_count, int32_t embedding_size,
                                        int32_t hidden_size, double* h_sums);

/* Custom expert sublayers: the C form of deriving from MoESubLayer (plugin/sublayers/SubLayer.h:18-48) and adding
 * a case to MoELayerPlugin::createSublayer (plugin/MoELayerPlugin.cc:28-41; README "custom sublayer").  A type
 * registered here can be named in expert_sublayer_type.  The layer then routes, dispatches and scatters as for
 * the built-in types, and for every expert that has rows calls copy_weights into one of max_concurrency device
 * slots (on a copy stream, while the expert before it runs) and run on the caller's stream; the combine step
 * follows.  One host synchronisation per call (the token counts), like the streamed built-in experts.  The copy
 * stream handed to copy_weights belongs to the layer and is destroyed with it: a callback must not leave anything
 * behind that refers to it later (an allocator that remembers which streams used a buffer, for instance). */
typedef struct infmoe_sublayer_vtable {
    void* user;                                    /* passed back to every callback */
    /* MoESubLayer::initialize (SubLayer.h:44): read weights etc.; called by infmoe_layer_initialize.  May be NULL. */
    int (*initialize)(void* user, int32_t expert_count, int32_t embedding_size, int32_t hidden_size,
                      const char* weight_file);
    /* MoESubLayer::weightSize (:36): bytes of one expert's weights in a device slot; NULL or 0 = no slots. */
    size_t (*weight_size)(void* user);
    /* MoESubLayer::workspaceSize (:37): scratch bytes run needs for token_count rows.  May be NULL. */
    size_t (*workspace_size)(void* user, int32_t token_count);
    /* MoESubLayer::copyWeights (:39): enqueue the copy of expert `expert`'s weights to d_dst on `stream`. */
    int (*copy_weights)(void* user, void* d_dst, int32_t expert, void* stream);
    /* MoESubLayer::run (:40-41): d_output[token_count][embedding_size] = the expert applied to d_input, enqueued on
     * `stream` (it need not, and should not, synchronise); 0 = ok.  Required. */
    int (*run)(void* user, int32_t expert, int32_t token_count, const void* d_weights, const float* d_input,
               float* d_output, void* d_workspace, void* stream);
} infmoe_sublayer_vtable;

/* Registers (or replaces) a sublayer type for this process.  The callbacks must stay valid while layers of the
 * type exist; layers created before a re-registration keep the callbacks they were created with. */
INFMOE_API int infmoe_register_sublayer(const char* type_name, const infmoe_sublayer_vtable* vt);

/* Read-back of the attributes (for the plugin classes and the Python binding). */
INFMOE_API int infmoe_layer_get_config(const infmoe_layer* layer, infmoe_layer_config* out);

/* ------------------------------------------------------------------------ */
/* Expert parallelism over the GPUs of one node (one process per GPU)         */
/* ------------------------------------------------------------------------ */
/* No counterpart in the reference, which runs on device 0 only
 * (plugin/MoELayerPlugin.cc:319).  An infmoe_ep object is one rank's share of a
 * MoE layer whose expert_count experts are sharded over `world` ranks in
 * contiguous blocks: it routes this rank's tokens over all experts, stores every
 * row into the receive buffer of the rank that owns its expert (peer stores over
 * NVLink), runs its own experts on what it received and stores the results into
 * the output buffers of the ranks the tokens came from.  The only cross-GPU
 * synchronisation is a two-word NCCL all-reduce before and after the experts.
 * NCCL (libnccl.so.2) is loaded at run time, only when world > 1. */
typedef struct infmoe_ep infmoe_ep;
#define INFMOE_EP_ID_BYTES 128

typedef struct infmoe_ep_config {
    int32_t rank, world;
    const void* unique_id;             /* INFMOE_EP_ID_BYTES from infmoe_ep_unique_id on one rank, the same on all */
    int32_t expert_count;              /* experts of the whole layer; divisible by world */
    int32_t embedding_size, hidden_size;
    int64_t max_tokens;                /* most tokens any rank passes to one call (sizes the receive regions) */
    const float* expert_centroids;     /* host, all experts: [expert_count][embedding_size] */
    const float* layernorm_weight;     /* host [embedding_size]; required iff moe_variant == "cpm_2" */
    const char* moe_variant;           /* of the whole layer: "cpm_2", "base_layer" or "default" */
    infmoe_layer* local_experts;       /* a layer object holding this rank's expert_count / world experts (rank r:
                                          experts r * E/world ...), any variant; borrowed, must outlive the ep object */
} infmoe_ep_config;

/* ncclGetUniqueId: call on one rank, hand the bytes to all ranks by any host-side channel. */
INFMOE_API int infmoe_ep_unique_id(void* h_id);
/* Collective over all ranks: creates the communicator, allocates the buffers and maps the peers' with CUDA IPC
 * (peer access between the GPUs is required).  Uses the current device. */
INFMOE_API int infmoe_ep_create(const infmoe_ep_config* cfg, infmoe_ep** out);
/* The same from the configuration of the WHOLE layer (what the plugin creator holds): creates this rank's layer
 * object (experts rank * E/world ..., read from the same weight file), initializes it, and wraps it.  *local_out
 * is owned by the caller and must outlive *ep_out. */
INFMOE_API int infmoe_ep_create_sharded(const infmoe_layer_config* whole_layer, int32_t rank, int32_t world,
                                        const void* unique_id, int64_t max_tokens, infmoe_layer** local_out,
                                        infmoe_ep** ep_out);
/* One layer pass for this rank's `tokens` rows (collective, stream ordered, does not block the host).
 * d_out may be the pointer infmoe_ep_output returns (or NULL): then the result is left in that buffer and no copy
 * is made.  Device-side findings are returned by infmoe_ep_sync_status. */
INFMOE_API int infmoe_ep_forward(infmoe_ep* ep, const float* d_x, float* d_out, int64_t tokens, void* stream);
/* The buffer the other ranks store this rank's results into: [max_tokens][embedding_size], token order; valid
 * after infmoe_ep_forward until the next one. */
INFMOE_API int infmoe_ep_output(const infmoe_ep* ep, float** d_out);
/* Host buffers in and out, copies inside; blocks until the result is there and returns the status. */
INFMOE_API int infmoe_ep_forward_host(infmoe_ep* ep, const float* h_x, float* h_out, int64_t tokens);
/* The same without waiting (collective; every rank submits the same sequence): the step's upload, pass and
 * download are enqueued and the call returns; infmoe_ep_wait_host blocks until the OLDEST submitted step's result is
 * in its h_out and returns that step's status.  At most two steps may be in flight: the upload of one then runs
 * behind the experts of the one before, its download under the one after.  h_x and h_out must be page-locked for
 * the copies to overlap, and must stay untouched until the step has been waited for.  infmoe_ep_forward and
 * infmoe_ep_forward_host refuse to run while steps are in flight. */
INFMOE_API int infmoe_ep_submit_host(infmoe_ep* ep, const float* h_x, float* h_out, int64_t tokens);
INFMOE_API int infmoe_ep_wait_host(infmoe_ep* ep);
/* Blocks until `stream` is idle; non-zero when this rank (or, for routing, any rank) raised a device-side status. */
INFMOE_API int infmoe_ep_sync_status(infmoe_ep* ep, void* stream);
/* Routing results of this rank's tokens in the last pass (as infmoe_layer_last_routing, expert indices global). */
INFMOE_API int infmoe_ep_last_routing(const infmoe_ep* ep, const int32_t** d_gate, const float** d_score,
                                      const int32_t** d_pos, const int32_t** d_count, const int32_t** d_offset);
/* What this rank received in the last pass: filled slots per source rank [world], and per slot (region s starts at
 * s * region_size) the local expert index and the token index at the source. */
INFMOE_API int infmoe_ep_received(const infmoe_ep* ep, const int32_t** d_region_count, const int32_t** d_expert_of_slot,
                                  const int32_t** d_home_of_slot, int64_t* region_size);
/* Per-phase device timing (CUDA events on the caller's stream): ms[5] = routing + dispatch + sending rows,
 * waiting for all ranks' rows, experts (incl. storing results), waiting for all ranks' results, copy-out. */
INFMOE_API int infmoe_ep_set_profiling(infmoe_ep* ep, int enable);
INFMOE_API int infmoe_ep_phase_ms(infmoe_ep* ep, float* ms, int32_t* calls);
INFMOE_API int infmoe_ep_destroy(infmoe_ep* ep);

/* All `world` ranks inside this process on the current device, for tests and single-GPU emulation: the peers'
 * buffers are each other's allocations and one stream orders what the barriers order between processes.  The caller
 * drives the phases itself: infmoe_ep_forward_begin on every rank, then infmoe_ep_forward_experts on every rank,
 * then infmoe_ep_forward_end on every rank, all on one stream.  unique_id is ignored. */
INFMOE_API int infmoe_ep_create_loopback(const infmoe_ep_config* cfgs, int32_t world, infmoe_ep** outs);
INFMOE_API int infmoe_ep_forward_begin(infmoe_ep* ep, const float* d_x, int64_t tokens, void* stream);
INFMOE_API int infmoe_ep_forward_experts(infmoe_ep* ep, void* stream);
INFMOE_API int infmoe_ep_forward_end(infmoe_ep* ep, float* d_out, void* stream);

/* ------------------------------------------------------------------------ */
/* Stage entry points = the free functions of plugin/cuda/moe.h and ops.h     */
/* ------------------------------------------------------------------------ */

/* Fused routing: [cpm_2 LayerNorm, plugin/MoELayerPlugin.cc:315-327] + gating
 * scores [cublasSgemm_v2, :334-336] + top-1 [moe_expert_select, plugin/cuda/moe.cu:147-159].
 * d_ln_w == NULL skips the LayerNorm.  d_status (int32, may be NULL) gets bit 0
 * set when a token selects no expert. */
INFMOE_API int infmoe_route(const float* d_x, const float* d_centroids, const float* d_ln_w, int64_t token_num,
                            int32_t embedding_size, int32_t expert_count, int32_t* d_gate, float* d_score,
                            int32_t* d_status, void* stream);

/* moe_expert_select (plugin/cuda/moe.cu:147-159): top-1 over a given score matrix [T][E]. */
INFMOE_API int infmoe_expert_select(int64_t token_num, int32_t expert_count, const float* d_aff, int32_t* d_gate,
                                    float* d_weight, int32_t* d_status, void* stream);

/* moe_expert_count (plugin/cuda/moe.cu:161-212), on the device: d_count[E],
 * d_offset[E+1] (offset[E] = T, plugin/MoELayerPlugin.cc:351), d_pos[T] in the
 * reference's stable order.  A gate outside [0, E) (the reference asserts,
 * moe.cu:184) sets bit 1 of d_status; such tokens are listed, in ascending order,
 * behind the tokens of the last expert, and d_offset[E] is the number of tokens
 * that do have an expert, so d_pos is always a permutation of 0..T-1. */
INFMOE_API int infmoe_expert_count(int64_t token_num, int32_t expert_count, const int32_t* d_gate, int32_t* d_pos,
                                   int32_t* d_count, int32_t* d_offset, int32_t* d_status, void* stream);

/* moe_expert_scatter (plugin/cuda/moe.cu:214-228). d_coeff / d_routed_coeff may be NULL. */
INFMOE_API int infmoe_expert_scatter(int64_t token_num, int32_t token_len, const float* d_input,
                                     const float* d_coeff, const int32_t* d_pos, float* d_routed,
                                     float* d_routed_coeff, void* stream);

/* moe_expert_gather (plugin/cuda/moe.cu:230-240). */
INFMOE_API int infmoe_expert_gather(int64_t token_num, int32_t token_len, const float* d_routed,
                                    const int32_t* d_pos, float* d_output, void* stream);

/* moe_expert_base_layer_fused_mix_and_gather (plugin/cuda/moe.cu:242-258). */
INFMOE_API int infmoe_expert_mix_gather(int64_t token_num, int32_t token_len, const int32_t* d_pos,
                                        const float* d_routed, const float* d_post, const float* d_coeff,
                                        float* d_output, void* stream);

/* layernorm_gpu<float,float> with gamma, no beta, eps 1e-6 (plugin/cuda/ops/layernorm.cu:179-188). */
INFMOE_API int infmoe_layernorm(float* d_out, const float* d_in, int64_t rows, int32_t cols, const float* d_gamma,
                                void* stream);

/* fused_gelu_dot_gpu<float> (plugin/cuda/ops/gelu.cu:18-25): B = gelu(A) * B. */
INFMOE_API int infmoe_gelu_dot(const float* d_a, float* d_b, size_t len, void* stream);

/* T5FFLayer::run for one expert (plugin/sublayers/T5FFLayer.cc:90-141) on
 * `rows` rows: d_y = d_x + (gelu(LN(x) wi0^T) * (LN(x) wi1^T)) wo^T.  Weights are
 * plain FP32 device arrays.  d_workspace must hold infmoe_t5ff_workspace_bytes.
 * Blocks the host until the result is there (like the reference's run, which ends
 * in a stream synchronisation) and returns the device-side status. */
INFMOE_API int infmoe_t5ff_workspace_bytes(int64_t rows, int32_t embedding_size, int32_t hidden_size, size_t* bytes);
INFMOE_API int infmoe_t5ff_run(int64_t rows, int32_t embedding_size, int32_t hidden_size, const float* d_ln_w,
                               const float* d_wi0, const float* d_wi1, const float* d_wo, const float* d_x,
                               float* d_y, void* d_workspace, size_t workspace_bytes, void* stream);

/* The same expert FFN for callers that cannot allocate device memory at the
 * moment they need it: a TensorRT plugin inside enqueue(), whose engine fixed its
 * memory plan when it was built, and a serving loop that may not risk the
 * device-wide synchronisation a cudaMalloc can cause.  It has no counterpart in
 * the reference: it is infmoe_t5ff_run without the workspace argument.  All
 * scratch lives in an array that is part of the library image (32 MiB, held by
 * every GPU that loads the library until the process exits); the call performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.  Like
 * infmoe_t5ff_run it blocks the host until the result is there.
 *   - Sizes whose scratch need (infmoe_t5ff_workspace_bytes) exceeds the array are
 *     rejected with INFMOE_ERR_UNSUPPORTED; infmoe_t5ff_static_limit reports both
 *     numbers.  Examples that fit: d_model 512, d_ff 1024, 256 rows; d_model 1024,
 *     d_ff 1024, 64 rows.
 *   - The first call on each device looks up the array's device address (with
 *     that device current).  Make that first call before any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents;
 *     the function rewrites everything it reads and clears its status word, so
 *     back-to-back calls on one stream are fine, but two calls that overlap on
 *     the GPU (different streams, or different host threads) race on it. */
INFMOE_API int infmoe_t5ff_static_limit(int64_t rows, int32_t embedding_size, int32_t hidden_size, size_t* needed,
                                        size_t* available);
INFMOE_API int infmoe_t5ff_run_static(int64_t rows, int32_t embedding_size, int32_t hidden_size,
                                      const float* d_ln_w, const float* d_wi0, const float* d_wi1,
                                      const float* d_wo, const float* d_x, float* d_y, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INFMOE_C_H */
