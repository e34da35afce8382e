// Host side of the B200 MoE layer: the layer object behind the C ABI
// (include/infmoe_c.h), its expert-weight store, the max_concurrency weight
// streaming scheduler and the stream-ordered forward pass.
//
// Reference counterparts:
//   MoELayerPlugin ctor / clone / terminate   plugin/MoELayerPlugin.cc:60-102,203-237
//   MoELayerPlugin::getWorkspaceSize          plugin/MoELayerPlugin.cc:253-273
//   MoELayerPlugin::enqueue                   plugin/MoELayerPlugin.cc:279-416
//   T5FFLayer::initialize / copyWeights       plugin/sublayers/T5FFLayer.cc:143-147,55-88
//   serialize / deserialising ctor            plugin/MoELayerPlugin.cc:418-458,104-143
//
// Differences by design: the forward pass never blocks the host when the
// experts are resident (the reference synchronises after every stage); when
// experts are streamed from pinned host memory there is exactly one host
// synchronisation per call (the per-expert token counts), after which copies
// and GEMMs are chained with events only.
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <sys/mman.h>
#include <sys/stat.h>

#include "common.cuh"
#include "kernels.h"
#include "layer_internal.h"
#include "npz.h"

namespace infmoe {

long long g_kernel_launches = 0;

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

namespace {

constexpr size_t ALIGN = 256;
inline size_t align_up(size_t x) { return (x + ALIGN - 1) / ALIGN * ALIGN; }

// Behaviour flags of the three variants (plugin/MoELayerPlugin.h:36-42, parseFlags MoELayerPlugin.cc:44-58).
struct Flags {
    bool layernorm_before_score = false;  // cpm_2
    bool base_layer_mix = false;          // base_layer
};

// Expert weights, shared by a layer and its clones like the reference's
// shared_ptr<MoESubLayer> (plugin/MoELayerPlugin.cc:83-102).
struct ExpertStore {
    int E = 0, D = 0, F = 0;
    std::mutex mu;
    // pinned host copies of the raw FP32 weights (streaming mode source); nullptr if absent.  A weight file is
    // loaded into ONE page-locked arena (a single cudaHostAlloc instead of four per expert); weights given by
    // pointer get allocations of their own.
    std::vector<float*> h_ln, h_wi0, h_wi1, h_wo;
    char* h_arena = nullptr;
    size_t arena_bytes = 0;
    bool arena_registered = false;   // the arena is an anonymous mapping page-locked with cudaHostRegister
    bool in_arena(const void* p) const { return h_arena && (const char*)p >= h_arena && (const char*)p < h_arena + arena_bytes; }
    std::vector<char> on_host;
    // device: LayerNorm weights of all experts [E][D] (always resident, 4*E*D bytes)
    float* d_ln = nullptr;
    std::vector<char> ln_on_device;
    // device-resident raw FP32 weights in the GEMM's tile-contiguous layout (launch_retile):
    //   [0] w01 [E] x tiled(2F x D)  (row 2f = wi_0[f], row 2f+1 = wi_1[f])
    //   [1] wo  [E] x tiled(D x F)
    float* d_plane[2] = {nullptr, nullptr};
    float* d_staging = nullptr;   // 3*D*F floats: landing area of host weights before they are retiled
    std::vector<char> on_device;
    std::vector<unsigned> version;   // bumped whenever an expert's host weights are replaced (expert caches compare it)
    bool fortran_warning = false;
    // Recorded behind the copies and retile kernels of the last upload_resident, on the stream that ran them.
    // Clones share this store and enqueue on streams of their own: each of them waits for the event before its
    // GEMMs read the planes, and the next upload waits for it before it reuses d_staging.
    cudaEvent_t ev_uploaded = nullptr;
    bool upload_recorded = false;

    size_t matrix_elems() const { return (size_t)D * (size_t)F; }
    size_t plane_elems(int p) const { return p == 0 ? tiled_elems(2 * F, D) : tiled_elems(D, F); }   // per expert
    size_t resident_bytes() const { return (plane_elems(0) + plane_elems(1)) * (size_t)E * sizeof(float); }

    ~ExpertStore() {
        for (auto& v : {&h_ln, &h_wi0, &h_wi1, &h_wo})
            for (float* p : *v)
                if (p && !in_arena(p)) cudaFreeHost(p);
        if (h_arena) {
            if (arena_registered) cudaHostUnregister(h_arena);
            munmap(h_arena, arena_bytes);
        }
        if (d_ln) cudaFree(d_ln);
        for (float* p : d_plane)
            if (p) cudaFree(p);
        if (d_staging) cudaFree(d_staging);
        if (ev_uploaded) cudaEventDestroy(ev_uploaded);
    }
};

struct WsLayout {
    size_t gate, pos, count, offset, slot_map, score, rscore, routed, post, h_hi, h_lo, g_hi, g_lo, slots, custom_slots,
        custom_ws, total;
};

// Sublayer types registered through infmoe_register_sublayer (the reference's extension point is deriving from
// MoESubLayer and adding a case to createSublayer, plugin/MoELayerPlugin.cc:28-41).
std::mutex g_sublayer_mu;
std::map<std::string, infmoe_sublayer_vtable>& sublayer_registry() {
    static std::map<std::string, infmoe_sublayer_vtable> r;
    return r;
}

}  // namespace
}  // namespace infmoe

using namespace infmoe;

struct infmoe_layer {
    int E = 0, D = 0, F = 0, mc = 2;
    std::vector<float> centroids, gating_ln;
    std::string weight_file, sublayer_type, variant;
    Flags flags;
    int file_expert_offset = 0;          // expert n of this layer is expert file_expert_offset + n of the weight file
    bool identity = false;
    bool custom = false;                 // a registered sublayer type; `sub` holds its callbacks
    infmoe_sublayer_vtable sub{};
    bool sub_initialized = false;
    std::shared_ptr<ExpertStore> store;
    int residency = -1;          // -1 auto, 0 streamed, 1 resident
    bool residency_resolved = false;
    bool resident = false;
    bool initialized = false;
    int ffn_path = 0;            // 0 tensor cores when the shape allows, 1 exact CUDA-core kernels

    // device state, created at the first enqueue (reference: ensureCUDAContext / ensureGPUWeights,
    // plugin/MoELayerPlugin.cc:182-195,14-26)
    bool device_ready = false;
    int device = -1, num_sms = 0;
    float* d_centroids = nullptr;
    float* d_gating_ln = nullptr;
    int* d_status = nullptr;
    int* h_status = nullptr;     // pinned
    int* h_count = nullptr;      // pinned [E]
    int* h_slot_map = nullptr;   // pinned [E]
    std::vector<cudaStream_t> copy_streams;
    std::vector<cudaEvent_t> ev_ready, ev_freed;
    cudaEvent_t ev_fork = nullptr;

    // results of the last enqueue
    const int* last_gate = nullptr;
    const float* last_score = nullptr;
    const int* last_pos = nullptr;
    const int* last_count = nullptr;
    const int* last_offset = nullptr;

    // buffers owned for infmoe_layer_forward_host
    float* own_in = nullptr;
    float* own_out = nullptr;
    void* own_ws = nullptr;
    size_t own_io_bytes = 0, own_ws_bytes = 0;
    // two host-buffer steps in flight (infmoe_layer_submit_host / _wait_host)
    float* pipe_in[2] = {nullptr, nullptr};
    float* pipe_out[2] = {nullptr, nullptr};
    size_t pipe_io_bytes = 0;
    cudaStream_t pipe_in_stream = nullptr, pipe_out_stream = nullptr;
    cudaEvent_t pipe_ev_in[2] = {nullptr, nullptr}, pipe_ev_pass[2] = {nullptr, nullptr}, pipe_ev_out[2] = {nullptr, nullptr};
    bool pipe_used[2] = {false, false};
    int* pipe_h_status = nullptr;        // pinned [2]
    long long pipe_submitted = 0, pipe_waited = 0;
    cudaStream_t own_stream = nullptr;

    // Optional expert cache of the streamed mode (no counterpart in the reference, whose slots forget their
    // expert after every call): layer-owned slots that keep their expert across enqueue calls; a missing
    // expert replaces the least recently used slot.
    int cache_slots = 0;
    float* d_cache[2] = {nullptr, nullptr};     // [cache_slots] x tiled plane
    float* d_cache_staging = nullptr;           // [mc] raw landing areas (3 D F floats each)
    std::vector<int> cache_expert;              // slot -> expert, -1 = empty
    std::vector<unsigned> cache_version;        // slot -> version of the expert's weights it holds
    std::vector<int> cache_slot_of;             // expert -> slot, -1 = not cached
    std::vector<long long> cache_used;          // slot -> tick of the last use
    long long cache_tick = 0;
    std::vector<cudaEvent_t> ev_stage;          // landing area k has been retiled and may be overwritten
    unsigned long long weight_h2d_bytes = 0;    // expert weight bytes copied host -> device by enqueue so far

    long long launches_at_create = 0;

    // optional per-stage timing: a ring of CUDA events recorded on the caller's stream
    bool profiling = false;
    std::vector<cudaEvent_t> prof_events;   // [PROF_CALLS][PROF_MARKS]
    int prof_calls = 0;
};

namespace {

int parse_flags(const char* variant, Flags* f) {
    *f = Flags();
    if (!variant) {
        set_error("moe_variant is missing");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (strcmp(variant, "base_layer") == 0) f->base_layer_mix = true;
    else if (strcmp(variant, "cpm_2") == 0) f->layernorm_before_score = true;
    else if (strcmp(variant, "default") == 0) {}
    else {
        set_error("unsupported moe variant: %s", variant);  // plugin/MoELayerPlugin.cc:54-55
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    return INFMOE_OK;
}

bool uses_umma(const infmoe_layer* L) { return L->ffn_path == 0 && ffn_umma_supported(L->D, L->F, L->E); }

WsLayout ws_layout(const infmoe_layer* L, long long T, bool streamed) {
    WsLayout w{};
    size_t o = 0;
    auto take = [&](size_t bytes) {
        const size_t at = o;
        o += align_up(bytes);
        return at;
    };
    const size_t t = (size_t)T, D = (size_t)L->D, F = (size_t)L->F, E = (size_t)L->E;
    w.gate = take(4 * t);
    w.pos = take(4 * t);
    w.count = take(4 * E);
    w.offset = take(4 * (E + 1));
    w.slot_map = take(4 * E);
    w.score = take(4 * t);
    w.rscore = take(4 * t);
    // The tensor-core GEMM reads its residual from the input through pos[] and writes the layer output from its
    // epilogue; only the CUDA-core path and the Identity sublayer keep routed rows and expert-ordered results.
    const bool row_planes = L->identity || L->custom || !uses_umma(L);
    w.routed = take(row_planes ? 4 * t * D : 0);
    w.post = take(row_planes ? 4 * t * D : 0);
    w.h_hi = take(4 * t * D);
    w.h_lo = take(second_plane_bytes((long long)t, L->D));
    w.g_hi = take(4 * t * F);
    w.g_lo = take(second_plane_bytes((long long)t, L->F));
    w.slots = take(streamed && !L->identity && !L->custom
                       ? 4 * (size_t)L->mc * (tiled_elems(2 * L->F, L->D) + tiled_elems(L->D, L->F) + 3 * D * F)
                       : 0);
    // registered sublayer: max_concurrency weight slots (MoESubLayer::weightSize each) and its own scratch
    const size_t sub_weight = L->custom && L->sub.weight_size ? align_up(L->sub.weight_size(L->sub.user)) : 0;
    w.custom_slots = take(sub_weight * (size_t)L->mc);
    w.custom_ws = take(L->custom && L->sub.workspace_size ? L->sub.workspace_size(L->sub.user, (int32_t)T) : 0);
    w.total = o;
    return w;
}

int ensure_store_device_ln(ExpertStore* s) {
    if (!s->d_ln) {
        INFMOE_CUDA_TRY(cudaMalloc(&s->d_ln, sizeof(float) * (size_t)s->E * s->D));
        // experts never given weights keep gamma = 1 so that stray rows stay finite
        std::vector<float> ones((size_t)s->E * s->D, 1.0f);
        INFMOE_CUDA_TRY(cudaMemcpy(s->d_ln, ones.data(), sizeof(float) * ones.size(), cudaMemcpyHostToDevice));
    }
    for (int e = 0; e < s->E; ++e) {
        if (!s->ln_on_device[e] && s->on_host[e]) {
            INFMOE_CUDA_TRY(cudaMemcpy(s->d_ln + (size_t)e * s->D, s->h_ln[e], sizeof(float) * s->D,
                                       cudaMemcpyHostToDevice));
            s->ln_on_device[e] = 1;
        }
    }
    return INFMOE_OK;
}

int ensure_resident_planes(ExpertStore* s) {
    for (int p = 0; p < 2; ++p)
        if (!s->d_plane[p]) INFMOE_CUDA_TRY(cudaMalloc(&s->d_plane[p], sizeof(float) * s->plane_elems(p) * s->E));
    return INFMOE_OK;
}

// Puts one expert's matrices into its two planes (tile-contiguous, wi_0 / wi_1 rows interleaved).  Host
// sources first land in `staging` (device, 3*D*F floats); the weights stay raw FP32 (the GEMM kernel splits
// them into TF32 head and tail on the fly).
int load_expert_planes(int D, int F, const float* wi0, const float* wi1, const float* wo, float* w01, float* wo_dst,
                       bool src_on_host, float* staging, cudaStream_t stream) {
    const size_t n = (size_t)D * F;
    if (src_on_host) {
        if (!staging) {
            set_error("load_expert_planes: no staging buffer for host weights");
            return INFMOE_ERR_STATE;
        }
        INFMOE_CUDA_TRY(cudaMemcpyAsync(staging, wi0, sizeof(float) * n, cudaMemcpyHostToDevice, stream));
        INFMOE_CUDA_TRY(cudaMemcpyAsync(staging + n, wi1, sizeof(float) * n, cudaMemcpyHostToDevice, stream));
        INFMOE_CUDA_TRY(cudaMemcpyAsync(staging + 2 * n, wo, sizeof(float) * n, cudaMemcpyHostToDevice, stream));
        wi0 = staging;
        wi1 = staging + n;
        wo = staging + 2 * n;
    }
    INFMOE_TRY(launch_retile(wi0, wi1, 2 * F, D, w01, stream));
    INFMOE_TRY(launch_retile(wo, nullptr, D, F, wo_dst, stream));
    return INFMOE_OK;
}

// Uploads every expert that is on the host but not yet on the device.
// Called with the store's lock held.  Whatever stream the caller works on, it leaves this function ordered behind
// every upload queued so far (by itself or by a clone on another stream).
int upload_resident(ExpertStore* s, cudaStream_t stream) {
    INFMOE_TRY(ensure_resident_planes(s));
    if (!s->ev_uploaded) INFMOE_CUDA_TRY(cudaEventCreateWithFlags(&s->ev_uploaded, cudaEventDisableTiming));
    if (s->upload_recorded) INFMOE_CUDA_TRY(cudaStreamWaitEvent(stream, s->ev_uploaded, 0));
    bool queued = false;
    for (int e = 0; e < s->E; ++e) {
        if (s->on_device[e] || !s->on_host[e]) continue;
        if (!s->d_staging) INFMOE_CUDA_TRY(cudaMalloc(&s->d_staging, sizeof(float) * 3 * s->matrix_elems()));
        INFMOE_TRY(load_expert_planes(s->D, s->F, s->h_wi0[e], s->h_wi1[e], s->h_wo[e],
                                      s->d_plane[0] + s->plane_elems(0) * e, s->d_plane[1] + s->plane_elems(1) * e,
                                      true, s->d_staging, stream));
        s->on_device[e] = 1;
        queued = true;
    }
    if (queued) {
        INFMOE_CUDA_TRY(cudaEventRecord(s->ev_uploaded, stream));
        s->upload_recorded = true;
    }
    return INFMOE_OK;
}

int ensure_device(infmoe_layer* L) {
    if (L->device_ready) return INFMOE_OK;
    INFMOE_CUDA_TRY(cudaGetDevice(&L->device));
    cudaDeviceProp prop;
    INFMOE_CUDA_TRY(cudaGetDeviceProperties(&prop, L->device));
    if (prop.major != 10) {
        set_error("this library is built for sm_100a (B200); device %d is sm_%d%d", L->device, prop.major, prop.minor);
        return INFMOE_ERR_UNSUPPORTED;
    }
    L->num_sms = prop.multiProcessorCount;
    const size_t cbytes = sizeof(float) * (size_t)L->E * L->D;
    INFMOE_CUDA_TRY(cudaMalloc(&L->d_centroids, cbytes));
    INFMOE_CUDA_TRY(cudaMemcpy(L->d_centroids, L->centroids.data(), cbytes, cudaMemcpyHostToDevice));
    if (!L->gating_ln.empty()) {
        INFMOE_CUDA_TRY(cudaMalloc(&L->d_gating_ln, sizeof(float) * L->D));
        INFMOE_CUDA_TRY(cudaMemcpy(L->d_gating_ln, L->gating_ln.data(), sizeof(float) * L->D, cudaMemcpyHostToDevice));
    }
    INFMOE_CUDA_TRY(cudaMalloc(&L->d_status, sizeof(int)));
    INFMOE_CUDA_TRY(cudaMemset(L->d_status, 0, sizeof(int)));
    INFMOE_CUDA_TRY(cudaHostAlloc(&L->h_status, sizeof(int), cudaHostAllocDefault));
    *L->h_status = 0;
    INFMOE_CUDA_TRY(cudaHostAlloc(&L->h_count, sizeof(int) * (L->E + 1), cudaHostAllocDefault));
    INFMOE_CUDA_TRY(cudaHostAlloc(&L->h_slot_map, sizeof(int) * L->E, cudaHostAllocDefault));
    const int ncopy = L->mc < 2 ? 1 : 2;
    L->copy_streams.resize(ncopy);
    for (auto& s : L->copy_streams) INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    L->ev_ready.resize(L->mc);
    L->ev_freed.resize(L->mc);
    for (int i = 0; i < L->mc; ++i) {
        INFMOE_CUDA_TRY(cudaEventCreateWithFlags(&L->ev_ready[i], cudaEventDisableTiming));
        INFMOE_CUDA_TRY(cudaEventCreateWithFlags(&L->ev_freed[i], cudaEventDisableTiming));
    }
    INFMOE_CUDA_TRY(cudaEventCreateWithFlags(&L->ev_fork, cudaEventDisableTiming));
    L->device_ready = true;
    return INFMOE_OK;
}

int resolve_residency(infmoe_layer* L) {
    if (L->residency_resolved) return INFMOE_OK;
    int mode = L->residency;
    if (mode < 0) {
        const char* env = getenv("INFMOE_RESIDENT");
        if (env && *env) mode = atoi(env) ? 1 : 0;
    }
    ExpertStore* s = L->store.get();
    bool any_host_only = false, any_device = false;
    for (int e = 0; e < s->E; ++e) {
        if (s->on_device[e]) any_device = true;
        else if (s->on_host[e]) any_host_only = true;
    }
    if (L->identity) {
        L->resident = true;
    } else if (any_device) {
        L->resident = true;  // weights were handed over on the device: nothing to stream from
    } else if (mode < 0) {
        size_t free_b = 0, total_b = 0;
        INFMOE_CUDA_TRY(cudaMemGetInfo(&free_b, &total_b));
        L->resident = s->resident_bytes() < free_b / 10 * 7;
    } else {
        L->resident = mode == 1;
    }
    (void)any_host_only;
    L->residency_resolved = true;
    return INFMOE_OK;
}

int status_to_rc(int status) {
    if (status & STATUS_WAIT_TIMEOUT) {
        set_error("a bounded device-side wait ran out inside the expert GEMM (status 0x%x)", status);
        return INFMOE_ERR_DEVICE_TIMEOUT;
    }
    if (status & (STATUS_NO_EXPERT | STATUS_BAD_GATE)) {
        set_error("routing selected no expert for at least one token (NaN in input, centroids or weights)");
        return INFMOE_ERR_NAN;
    }
    if (status) {
        set_error("device status 0x%x", status);
        return INFMOE_ERR_CUDA;
    }
    return INFMOE_OK;
}

// Where the experts' result goes: `post` in expert order (a combine kernel follows), or, on the tensor-core path,
// straight into the layer output in token order (`out` with the row map `pos`, optionally the base_layer mix).
struct FfnOutput {
    float* post;
    float* out = nullptr;
    const int* pos = nullptr;
    const float* mix_score = nullptr;
    const unsigned long long* row_ptr = nullptr;   // address of output row i instead of out + i * D
};

int run_ffn(infmoe_layer* L, long long T, int e_begin, int e_end, const int* d_offset, const int* d_slot_map,
            int slots, float* const planes[2], const float* h_hi, const float* h_lo, const float* routed, float* g_hi,
            float* g_lo, const FfnOutput& o, cudaStream_t stream, cudaEvent_t mid = nullptr) {
    if (uses_umma(L))
        return launch_ffn_umma(T, L->D, L->F, L->E, e_begin, e_end, d_offset, d_slot_map, slots, h_hi, h_lo, planes[0],
                               planes[1], routed, g_hi, g_lo, o.out ? o.out : o.post, L->d_status, L->num_sms, stream,
                               mid, o.out ? o.pos : nullptr, o.out ? o.mix_score : nullptr, o.out ? o.row_ptr : nullptr);
    float* post = o.post;
    return launch_ffn_simt(T, L->D, L->F, e_begin, e_end, d_offset, d_slot_map, h_hi, h_lo, planes[0], planes[1],
                           routed, g_hi, g_lo, post, stream);
}

void free_device_state(infmoe_layer* L) {
    if (L->d_centroids) cudaFree(L->d_centroids);
    if (L->d_gating_ln) cudaFree(L->d_gating_ln);
    if (L->d_status) cudaFree(L->d_status);
    if (L->h_status) cudaFreeHost(L->h_status);
    if (L->h_count) cudaFreeHost(L->h_count);
    if (L->h_slot_map) cudaFreeHost(L->h_slot_map);
    for (auto s : L->copy_streams) cudaStreamDestroy(s);
    for (auto e : L->ev_ready) cudaEventDestroy(e);
    for (auto e : L->ev_freed) cudaEventDestroy(e);
    if (L->ev_fork) cudaEventDestroy(L->ev_fork);
    for (auto e : L->prof_events) cudaEventDestroy(e);
    for (auto e : L->ev_stage) cudaEventDestroy(e);
    for (float* p : L->d_cache)
        if (p) cudaFree(p);
    if (L->d_cache_staging) cudaFree(L->d_cache_staging);
    if (L->own_in) cudaFree(L->own_in);
    if (L->own_out) cudaFree(L->own_out);
    if (L->own_ws) cudaFree(L->own_ws);
    for (int i = 0; i < 2; ++i) {
        if (L->pipe_in[i]) cudaFree(L->pipe_in[i]);
        if (L->pipe_out[i]) cudaFree(L->pipe_out[i]);
        for (cudaEvent_t e : {L->pipe_ev_in[i], L->pipe_ev_pass[i], L->pipe_ev_out[i]})
            if (e) cudaEventDestroy(e);
        L->pipe_in[i] = L->pipe_out[i] = nullptr;
        L->pipe_ev_in[i] = L->pipe_ev_pass[i] = L->pipe_ev_out[i] = nullptr;
        L->pipe_used[i] = false;
    }
    L->pipe_io_bytes = 0;
    if (L->pipe_h_status) cudaFreeHost(L->pipe_h_status);
    L->pipe_h_status = nullptr;
    if (L->pipe_in_stream) cudaStreamDestroy(L->pipe_in_stream);
    if (L->pipe_out_stream) cudaStreamDestroy(L->pipe_out_stream);
    L->pipe_in_stream = L->pipe_out_stream = nullptr;
    if (L->own_stream) cudaStreamDestroy(L->own_stream);
}

std::shared_ptr<ExpertStore> make_store(int E, int D, int F) {
    auto s = std::make_shared<ExpertStore>();
    s->E = E;
    s->D = D;
    s->F = F;
    s->h_ln.assign(E, nullptr);
    s->h_wi0.assign(E, nullptr);
    s->h_wi1.assign(E, nullptr);
    s->h_wo.assign(E, nullptr);
    s->on_host.assign(E, 0);
    s->on_device.assign(E, 0);
    s->ln_on_device.assign(E, 0);
    s->version.assign(E, 0);
    return s;
}

int pinned_alloc(float** p, size_t elems) {
    if (*p) return INFMOE_OK;
    INFMOE_CUDA_TRY(cudaHostAlloc((void**)p, sizeof(float) * elems, cudaHostAllocDefault));
    return INFMOE_OK;
}

constexpr int PROF_CALLS = 64;   // calls kept in the timing ring
constexpr int PROF_MARKS = 7;    // start, route, dispatch, scatter, ffn gemm 1, ffn gemm 2, combine

int prof_mark(infmoe_layer* L, int mark, cudaStream_t stream) {
    if (!L->profiling) return INFMOE_OK;
    if (L->prof_events.empty()) {
        L->prof_events.resize((size_t)PROF_CALLS * PROF_MARKS);
        for (auto& e : L->prof_events) INFMOE_CUDA_TRY(cudaEventCreate(&e));
    }
    INFMOE_CUDA_TRY(cudaEventRecord(L->prof_events[(size_t)(L->prof_calls % PROF_CALLS) * PROF_MARKS + mark], stream));
    return INFMOE_OK;
}

constexpr uint32_t BLOB_MAGIC = 0x454F4D49u;  // "IMOE"
constexpr uint32_t BLOB_VERSION = 1;

}  // namespace

// =================================================================================================
// C ABI
// =================================================================================================
extern "C" {

const char* infmoe_last_error(void) { return t_error; }

int infmoe_layer_create(const infmoe_layer_config* cfg, infmoe_layer** out) {
    if (!cfg || !out) {
        set_error("layer_create: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    *out = nullptr;
    if (cfg->expert_count <= 0 || cfg->embedding_size <= 0 || cfg->hidden_size <= 0) {
        set_error("layer_create: expert_count, embedding_size and hidden_size must be positive");
        return INFMOE_ERR_INVALID_ARGUMENT;  // plugin/MoELayerPluginCreator.cc:118-128
    }
    if (cfg->max_concurrency <= 0) {
        set_error("layer_create: max_concurrency must be positive");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (!cfg->expert_centroids) {
        set_error("layer_create: expert_centroids is required");
        return INFMOE_ERR_INVALID_ARGUMENT;  // plugin/MoELayerPlugin.cc:75
    }
    Flags flags;
    INFMOE_TRY(parse_flags(cfg->moe_variant, &flags));
    if (flags.layernorm_before_score && !cfg->layernorm_weight) {
        set_error("layer_create: layernorm_weight is required for moe_variant cpm_2");
        return INFMOE_ERR_INVALID_ARGUMENT;  // plugin/MoELayerPlugin.cc:76-79
    }
    const char* type = cfg->expert_sublayer_type ? cfg->expert_sublayer_type : "T5_FF";
    const bool identity = strcmp(type, "Identity") == 0;
    bool custom = false;
    infmoe_sublayer_vtable sub{};
    if (!identity && strcmp(type, "T5_FF") != 0) {
        std::lock_guard<std::mutex> lock(g_sublayer_mu);
        auto it = sublayer_registry().find(type);
        if (it == sublayer_registry().end()) {
            set_error("unsupported sublayer type: %s", type);  // plugin/MoELayerPlugin.cc:37-39
            return INFMOE_ERR_INVALID_ARGUMENT;
        }
        custom = true;
        sub = it->second;
    }
    if (cfg->expert_weight_file && *cfg->expert_weight_file) {
        struct stat st;
        if (stat(cfg->expert_weight_file, &st) != 0 || !S_ISREG(st.st_mode)) {
            set_error("expert weight file %s is not a regular file", cfg->expert_weight_file);
            return INFMOE_ERR_IO;  // plugin/MoELayerPluginCreator.cc:132-140
        }
    }
    auto* L = new infmoe_layer();
    L->E = cfg->expert_count;
    L->D = cfg->embedding_size;
    L->F = cfg->hidden_size;
    L->mc = cfg->max_concurrency;
    L->centroids.assign(cfg->expert_centroids, cfg->expert_centroids + (size_t)L->E * L->D);
    if (cfg->layernorm_weight) L->gating_ln.assign(cfg->layernorm_weight, cfg->layernorm_weight + L->D);
    L->weight_file = cfg->expert_weight_file ? cfg->expert_weight_file : "";
    L->sublayer_type = type;
    L->variant = cfg->moe_variant;
    L->flags = flags;
    L->identity = identity;
    L->custom = custom;
    L->sub = sub;
    L->store = make_store(L->E, L->D, L->F);
    L->launches_at_create = g_kernel_launches;
    // decided here, not at the first enqueue: the workspace size depends on it
    const char* path = getenv("INFMOE_FFN");
    if (path && strcmp(path, "simt") == 0) L->ffn_path = 1;
    *out = L;
    return INFMOE_OK;
}

int infmoe_layer_clone(const infmoe_layer* src, infmoe_layer** out) {
    if (!src || !out) {
        set_error("layer_clone: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    auto* L = new infmoe_layer();
    L->E = src->E;
    L->D = src->D;
    L->F = src->F;
    L->mc = src->mc;
    L->centroids = src->centroids;
    L->gating_ln = src->gating_ln;
    L->weight_file = src->weight_file;
    L->sublayer_type = src->sublayer_type;
    L->variant = src->variant;
    L->flags = src->flags;
    L->file_expert_offset = src->file_expert_offset;
    L->identity = src->identity;
    L->custom = src->custom;
    L->sub = src->sub;
    L->sub_initialized = src->sub_initialized;
    L->store = src->store;  // shared, like the reference's sublayer
    L->residency = src->residency;
    L->initialized = src->initialized;
    L->ffn_path = src->ffn_path;
    L->launches_at_create = g_kernel_launches;
    *out = L;
    return INFMOE_OK;
}

int infmoe_layer_initialize(infmoe_layer* L) {
    if (!L) {
        set_error("layer_initialize: null layer");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (L->custom) {   // MoESubLayer::initialize (sublayers/SubLayer.h:44)
        if (!L->sub_initialized && L->sub.initialize) {
            const int rc = L->sub.initialize(L->sub.user, L->E, L->D, L->F, L->weight_file.c_str());
            if (rc != 0) {
                set_error("sublayer %s: initialize failed with %d", L->sublayer_type.c_str(), rc);
                return INFMOE_ERR_STATE;
            }
        }
        L->sub_initialized = true;
        L->initialized = true;
        return INFMOE_OK;
    }
    if (L->identity || L->weight_file.empty()) {
        L->initialized = true;
        return INFMOE_OK;
    }
    ExpertStore* s = L->store.get();
    std::lock_guard<std::mutex> lock(s->mu);
    bool all = true;
    for (int e = 0; e < s->E; ++e) all = all && (s->on_host[e] || s->on_device[e]);
    if (all) {  // already loaded through a clone (reference: mSavedWeights != nullptr, T5FFLayer.cc:145)
        L->initialized = true;
        return INFMOE_OK;
    }
    std::vector<int> seen((size_t)s->E, 0);
    const int D = s->D, F = s->F, E = s->E;
    // one page-locked arena for the whole file: per expert [ln | wi_0 | wi_1 | wo], every tensor 256-byte aligned
    const size_t ln_bytes = align_up(sizeof(float) * (size_t)D), mat_bytes = align_up(sizeof(float) * (size_t)D * F);
    const size_t per_expert = ln_bytes + 3 * mat_bytes;
    // The arena is an anonymous mapping that the reader threads fill (and thereby populate) in parallel; it is
    // page-locked afterwards in one cudaHostRegister call.  Pinning memory that is already resident is several
    // times faster than cudaHostAlloc followed by single-threaded first touches.
    if (!s->h_arena) {
        void* m = mmap(nullptr, per_expert * (size_t)E, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
        if (m == MAP_FAILED) {
            set_error("cannot map %zu bytes of host memory for the expert weights", per_expert * (size_t)E);
            return INFMOE_ERR_IO;
        }
        s->h_arena = (char*)m;
        s->arena_bytes = per_expert * (size_t)E;
    }
    auto arena_slot = [&](long e, int k) -> float* {   // k: 0 ln, 1 wi_0, 2 wi_1, 3 wo
        return (float*)(s->h_arena + per_expert * (size_t)e + (k == 0 ? 0 : ln_bytes + (size_t)(k - 1) * mat_bytes));
    };
    auto alloc = [&](const std::string& name, const std::vector<int64_t>& shape, float** dst) -> int {
        *dst = nullptr;
        const size_t slash = name.find('/');
        if (slash == std::string::npos) return INFMOE_OK;  // not an expert tensor: ignored like the reference
        char* endp = nullptr;
        const long e_file = strtol(name.c_str(), &endp, 10);
        const long e = e_file - L->file_expert_offset;   // experts outside this layer's share are skipped
        if (endp != name.c_str() + slash || e < 0 || e >= E) return INFMOE_OK;
        const std::string key = name.substr(slash + 1);
        size_t count = 1;
        for (int64_t d : shape) count *= (size_t)d;
        float** slot = nullptr;
        size_t want = 0;
        int bit = 0;
        int kind = 0;
        if (key == "layer_norm_weight") { slot = &s->h_ln[e]; want = (size_t)D; bit = 1; kind = 0; }
        else if (key == "wi_0_weight") { slot = &s->h_wi0[e]; want = (size_t)D * F; bit = 2; kind = 1; }
        else if (key == "wi_1_weight") { slot = &s->h_wi1[e]; want = (size_t)D * F; bit = 4; kind = 2; }
        else if (key == "wo_weight") { slot = &s->h_wo[e]; want = (size_t)D * F; bit = 8; kind = 3; }
        else return INFMOE_OK;
        if (count != want) {  // reference: assert on num_bytes(), T5FFLayer.cc:61,68,75,82
            set_error("%s: %s has %zu elements, expected %zu", L->weight_file.c_str(), name.c_str(), count, want);
            return INFMOE_ERR_FORMAT;
        }
        if (*slot && !s->in_arena(*slot)) cudaFreeHost(*slot);   // an expert given by pointer before: the file wins
        *slot = arena_slot(e, kind);
        *dst = *slot;
        seen[e] |= bit;
        return INFMOE_OK;
    };
    bool fortran = false;
    // the members are independent ranges of the file: read (and inflate) them with a few threads at once
    static const int threads = [] {
        const char* v = getenv("INFMOE_LOAD_THREADS");
        const int n = v ? atoi(v) : 8;
        return n < 1 ? 1 : (n > 64 ? 64 : n);
    }();
    INFMOE_TRY(npz_read(L->weight_file.c_str(), alloc, &fortran, threads));
    s->fortran_warning = fortran;
    if (!s->arena_registered) {
        INFMOE_CUDA_TRY(cudaHostRegister(s->h_arena, s->arena_bytes, cudaHostRegisterPortable));
        s->arena_registered = true;
    }
    for (int e = 0; e < E; ++e) {
        if (seen[e] != 15) {
            set_error("%s: expert %d is missing tensors (mask 0x%x of 0xf)", L->weight_file.c_str(), e, seen[e]);
            return INFMOE_ERR_FORMAT;
        }
        s->on_host[e] = 1;
        s->on_device[e] = 0;
        s->ln_on_device[e] = 0;
        ++s->version[e];
    }
    L->initialized = true;
    return INFMOE_OK;
}

int infmoe_layer_set_expert(infmoe_layer* L, int32_t e, const float* ln_w, const float* wi0, const float* wi1,
                            const float* wo, int on_device) {
    if (!L || !ln_w || !wi0 || !wi1 || !wo || e < 0 || e >= L->E) {
        set_error("layer_set_expert: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    ExpertStore* s = L->store.get();
    std::lock_guard<std::mutex> lock(s->mu);
    const size_t n = s->matrix_elems();
    if (on_device) {
        if (!s->d_ln) INFMOE_TRY(ensure_store_device_ln(s));
        INFMOE_TRY(ensure_resident_planes(s));
        INFMOE_CUDA_TRY(cudaMemcpy(s->d_ln + (size_t)e * s->D, ln_w, sizeof(float) * s->D, cudaMemcpyDeviceToDevice));
        s->ln_on_device[e] = 1;
        INFMOE_TRY(load_expert_planes(s->D, s->F, wi0, wi1, wo, s->d_plane[0] + s->plane_elems(0) * e,
                                      s->d_plane[1] + s->plane_elems(1) * e, false, nullptr, 0));
        INFMOE_CUDA_TRY(cudaStreamSynchronize(0));
        s->on_device[e] = 1;
    } else {
        INFMOE_TRY(pinned_alloc(&s->h_ln[e], (size_t)s->D));
        INFMOE_TRY(pinned_alloc(&s->h_wi0[e], n));
        INFMOE_TRY(pinned_alloc(&s->h_wi1[e], n));
        INFMOE_TRY(pinned_alloc(&s->h_wo[e], n));
        memcpy(s->h_ln[e], ln_w, sizeof(float) * s->D);
        memcpy(s->h_wi0[e], wi0, sizeof(float) * n);
        memcpy(s->h_wi1[e], wi1, sizeof(float) * n);
        memcpy(s->h_wo[e], wo, sizeof(float) * n);
        ++s->version[e];
        s->on_host[e] = 1;
        s->on_device[e] = 0;
        s->ln_on_device[e] = 0;
    }
    L->initialized = true;
    return INFMOE_OK;
}

int infmoe_layer_set_file_expert_offset(infmoe_layer* L, int32_t first_expert) {
    if (!L || first_expert < 0) {
        set_error("layer_set_file_expert_offset: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    L->file_expert_offset = first_expert;
    return INFMOE_OK;
}

int infmoe_layer_set_residency(infmoe_layer* L, int mode) {
    if (!L || mode < -1 || mode > 1) {
        set_error("layer_set_residency: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    L->residency = mode;
    L->residency_resolved = false;
    return INFMOE_OK;
}

int infmoe_layer_set_expert_cache(infmoe_layer* L, int32_t slots) {
    if (!L || slots < 0) {
        set_error("layer_set_expert_cache: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (L->d_cache[0]) {   // resizing drops what is cached; the slots may still be read by work in flight
        INFMOE_CUDA_TRY(cudaDeviceSynchronize());
        for (float*& p : L->d_cache) {
            cudaFree(p);
            p = nullptr;
        }
        cudaFree(L->d_cache_staging);
        L->d_cache_staging = nullptr;
    }
    L->cache_slots = slots == 0 ? 0 : std::max(slots, L->mc);
    L->cache_expert.clear();
    return INFMOE_OK;
}

int infmoe_layer_weight_h2d_bytes(const infmoe_layer* L, uint64_t* bytes) {
    if (!L || !bytes) {
        set_error("layer_weight_h2d_bytes: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    *bytes = L->weight_h2d_bytes;
    return INFMOE_OK;
}

namespace {

// Device memory and bookkeeping of the expert cache, created at the first streamed enqueue that uses it.
int ensure_cache(infmoe_layer* L) {
    const ExpertStore* s = L->store.get();
    const int S = L->cache_slots;
    if (!L->d_cache[0]) {
        for (int p = 0; p < 2; ++p)
            INFMOE_CUDA_TRY(cudaMalloc(&L->d_cache[p], sizeof(float) * s->plane_elems(p) * (size_t)S));
        INFMOE_CUDA_TRY(cudaMalloc(&L->d_cache_staging, sizeof(float) * 3 * s->matrix_elems() * (size_t)L->mc));
    }
    if ((int)L->cache_expert.size() != S) {
        L->cache_expert.assign(S, -1);
        L->cache_version.assign(S, 0);
        L->cache_used.assign(S, 0);
        L->cache_slot_of.assign(L->E, -1);
    }
    while ((int)L->ev_ready.size() < S) {
        cudaEvent_t a, b;
        INFMOE_CUDA_TRY(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        INFMOE_CUDA_TRY(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        L->ev_ready.push_back(a);
        L->ev_freed.push_back(b);
    }
    while ((int)L->ev_stage.size() < L->mc) {
        cudaEvent_t a;
        INFMOE_CUDA_TRY(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        L->ev_stage.push_back(a);
    }
    return INFMOE_OK;
}

struct CachePlan {
    int slot;
    bool load;
};

// Chooses a slot for every active expert, in execution order.  Experts already cached (with current weights)
// keep their slot; a missing expert takes the least recently used slot that no later expert of this call is
// waiting for; if every slot is spoken for, the expert needed last gives its slot up and is loaded again later.
std::vector<CachePlan> plan_cache(infmoe_layer* L, const std::vector<int>& active) {
    const ExpertStore* s = L->store.get();
    const int S = L->cache_slots;
    std::vector<CachePlan> plan(active.size(), CachePlan{-1, true});
    std::vector<int> reserved_by(S, -1);   // slot -> position in `active` of the cached expert that will use it
    for (size_t j = 0; j < active.size(); ++j) {
        const int e = active[j], sl = L->cache_slot_of[e];
        if (sl >= 0 && L->cache_expert[sl] == e && L->cache_version[sl] == s->version[e]) {
            plan[j] = CachePlan{sl, false};
            reserved_by[sl] = (int)j;
        }
    }
    for (size_t j = 0; j < active.size(); ++j) {
        const int e = active[j];
        int sl = plan[j].slot;
        if (plan[j].load) {
            int victim = -1;
            for (int v = 0; v < S; ++v)
                if (reserved_by[v] < 0 && (victim < 0 || L->cache_used[v] < L->cache_used[victim])) victim = v;
            if (victim < 0) {   // all slots reserved by later hits: take the one needed last
                for (int v = 0; v < S; ++v)
                    if (victim < 0 || reserved_by[v] > reserved_by[victim]) victim = v;
                plan[(size_t)reserved_by[victim]] = CachePlan{-1, true};
            }
            sl = victim;
            if (L->cache_expert[sl] >= 0) L->cache_slot_of[L->cache_expert[sl]] = -1;
            L->cache_expert[sl] = e;
            L->cache_version[sl] = s->version[e];
            L->cache_slot_of[e] = sl;
            plan[j].slot = sl;
        }
        reserved_by[sl] = -1;              // once its GEMMs are queued the slot may be handed on (behind an event)
        L->cache_used[sl] = ++L->cache_tick;
    }
    return plan;
}

}  // namespace

int infmoe_wait_timeout_probe(uint32_t limit_ms, int32_t* timed_out, float* waited_ms) {
    if (limit_ms == 0 || limit_ms > 2000 || !timed_out) {
        set_error("wait_timeout_probe: the limit must be 1..2000 ms");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    int* d_status = nullptr;
    unsigned long long* d_ns = nullptr;
    INFMOE_CUDA_TRY(cudaMalloc(&d_status, sizeof(int)));
    INFMOE_CUDA_TRY(cudaMalloc(&d_ns, sizeof(unsigned long long)));
    int rc = INFMOE_OK, h_status = 0;
    unsigned long long h_ns = 0;
    if (cudaMemset(d_status, 0, sizeof(int)) != cudaSuccess) rc = INFMOE_ERR_CUDA;
    if (rc == INFMOE_OK) rc = launch_wait_probe((unsigned long long)limit_ms * 1000000ull, d_status, d_ns, 0);
    if (rc == INFMOE_OK && (cudaMemcpy(&h_status, d_status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess ||
                            cudaMemcpy(&h_ns, d_ns, sizeof(h_ns), cudaMemcpyDeviceToHost) != cudaSuccess)) {
        set_error("wait_timeout_probe: %s", cudaGetErrorString(cudaGetLastError()));
        rc = INFMOE_ERR_CUDA;
    }
    cudaFree(d_status);
    cudaFree(d_ns);
    if (rc != INFMOE_OK) return rc;
    *timed_out = (h_status & STATUS_WAIT_TIMEOUT) ? 1 : 0;
    if (waited_ms) *waited_ms = (float)(h_ns * 1e-6);
    // the same translation enqueue's callers see
    return *timed_out ? INFMOE_OK : status_to_rc(h_status);
}

int infmoe_expert_cache_simulate(int32_t slots, int32_t expert_count, const int32_t* experts, const int32_t* call_sizes,
                                 int32_t calls, int32_t* loads_per_call) {
    if (slots <= 0 || expert_count <= 0 || calls < 0 || (calls > 0 && (!experts || !call_sizes || !loads_per_call))) {
        set_error("expert_cache_simulate: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    // the layer's own planning code on a layer object without device state
    infmoe_layer L;
    L.E = expert_count;
    L.store = make_store(expert_count, 1, 1);
    L.cache_slots = slots;
    L.cache_expert.assign(slots, -1);
    L.cache_version.assign(slots, 0);
    L.cache_used.assign(slots, 0);
    L.cache_slot_of.assign(expert_count, -1);
    const int32_t* p = experts;
    for (int32_t c = 0; c < calls; ++c) {
        std::vector<int> active;
        for (int32_t i = 0; i < call_sizes[c]; ++i, ++p) {
            if (*p < 0 || *p >= expert_count || (!active.empty() && *p <= active.back())) {
                set_error("expert_cache_simulate: call %d: expert ids must be ascending and inside [0, %d)", c, expert_count);
                return INFMOE_ERR_INVALID_ARGUMENT;
            }
            active.push_back(*p);
        }
        int loads = 0;
        for (const CachePlan& pl : plan_cache(&L, active)) loads += pl.load ? 1 : 0;
        loads_per_call[c] = loads;
    }
    return INFMOE_OK;
}

int infmoe_layer_workspace_bytes(const infmoe_layer* L, int64_t T, size_t* bytes) {
    if (!L || !bytes || T < 0) {
        set_error("layer_workspace_bytes: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    // Sized for the streamed case so that the answer does not depend on a decision taken later.
    *bytes = ws_layout(L, T, true).total + ALIGN;
    return INFMOE_OK;
}

// The forward pass.  With given_gate == nullptr this is the whole layer (routing included).  With a
// caller-provided expert index per row it runs dispatch + experts only and returns every row's expert
// output in the caller's row order (no score mix): the building block of the expert-parallel path, where
// routing happened on the rank that owns the token.
// region_count / region_size (expert-parallel receive buffer): the T rows are slots in regions of region_size, of
// which only the first region_count[s] of region s hold a row.
static int layer_run(infmoe_layer* L, const float* d_in, float* d_out, void* d_ws, size_t ws_bytes, int64_t T,
                     void* stream_v, const int* given_gate, const float* row_score = nullptr,
                     const unsigned long long* row_dst = nullptr, const int* region_count = nullptr,
                     int region_size = 0) {
    if (!L || T < 0 || (T > 0 && (!d_in || (!d_out && !row_dst) || !d_ws))) {
        set_error("layer_enqueue: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (T == 0) return INFMOE_OK;
    if (d_in == d_out) {
        set_error("layer_enqueue: input and output must not alias");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (T > 0x7fffffffLL / (L->D > L->F ? L->D : L->F)) {
        set_error("layer_enqueue: token_num %lld is too large for 32-bit row offsets", (long long)T);
        return INFMOE_ERR_UNSUPPORTED;
    }
    cudaStream_t stream = (cudaStream_t)stream_v;
    ExpertStore* s = L->store.get();
    INFMOE_TRY(ensure_device(L));
    if (L->custom) {
        if (!L->sub_initialized) {
            set_error("layer_enqueue: sublayer %s is not initialized (call infmoe_layer_initialize first)",
                      L->sublayer_type.c_str());
            return INFMOE_ERR_STATE;
        }
        L->resident = false;
    } else if (!L->identity) {
        std::lock_guard<std::mutex> lock(s->mu);
        for (int e = 0; e < s->E; ++e) {
            if (!s->on_host[e] && !s->on_device[e]) {
                set_error("layer_enqueue: expert %d has no weights (call infmoe_layer_initialize first)", e);
                return INFMOE_ERR_STATE;
            }
        }
        INFMOE_TRY(ensure_store_device_ln(s));
        INFMOE_TRY(resolve_residency(L));
        if (L->resident) INFMOE_TRY(upload_resident(s, stream));
    } else {
        L->resident = true;
    }
    const bool streamed = !L->resident && !L->custom;
    const WsLayout w = ws_layout(L, T, streamed);
    char* base = (char*)(((uintptr_t)d_ws + ALIGN - 1) / ALIGN * ALIGN);
    if ((size_t)(base - (char*)d_ws) + w.total > ws_bytes) {
        set_error("layer_enqueue: workspace of %zu bytes is too small, %zu needed", ws_bytes, w.total + ALIGN);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    int* gate = (int*)(base + w.gate);
    int* pos = (int*)(base + w.pos);
    int* count = (int*)(base + w.count);
    int* offset = (int*)(base + w.offset);
    int* slot_map = (int*)(base + w.slot_map);
    float* score = (float*)(base + w.score);
    float* rscore = (float*)(base + w.rscore);
    float* routed = (float*)(base + w.routed);
    float* post = (float*)(base + w.post);
    float* h_hi = (float*)(base + w.h_hi);
    float* h_lo = (float*)(base + w.h_lo);
    float* g_hi = (float*)(base + w.g_hi);
    float* g_lo = (float*)(base + w.g_lo);
    const int* gate_in = given_gate ? given_gate : gate;
    if (given_gate) score = const_cast<float*>(row_score);   // scores of the caller's rows, or none
    L->last_gate = gate_in;
    L->last_score = score;
    L->last_pos = pos;
    L->last_count = count;
    L->last_offset = offset;

    INFMOE_TRY(prof_mark(L, 0, stream));
    // 1. routing (plugin/MoELayerPlugin.cc:312-345)
    if (!given_gate)
        INFMOE_TRY(launch_route(d_in, L->d_centroids, L->flags.layernorm_before_score ? L->d_gating_ln : nullptr, T,
                                L->D, L->E, gate, score, L->d_status, stream));
    INFMOE_TRY(prof_mark(L, 1, stream));
    // 2. dispatch metadata (:350-352)
    INFMOE_TRY(launch_dispatch(gate_in, T, L->E, pos, count, offset, L->d_status, stream, region_count, region_size));
    const int* valid_rows = offset + L->E;   // rows past it have no expert (or are empty slots): nobody touches them
    INFMOE_TRY(prof_mark(L, 2, stream));
    // whole layer: the variant decides; experts alone: the caller asks for the mix by passing the scores
    const bool mix = given_gate ? row_score != nullptr : L->flags.base_layer_mix;
    // the tensor-core GEMM writes the layer output itself (combine fused into its epilogue)
    const bool fused_combine = !L->identity && !L->custom && uses_umma(L);
    FfnOutput ffn_out;
    ffn_out.post = post;
    if (fused_combine) {
        ffn_out.out = row_dst ? post : d_out;   // with per-row addresses `out` only switches the fused path on
        ffn_out.pos = pos;
        ffn_out.mix_score = mix ? rscore : nullptr;
        ffn_out.row_ptr = row_dst;
    }
    if (L->identity) {
        // Identity expert (plugin/sublayers/IdentityLayer.hh): post = routed
        INFMOE_TRY(launch_scatter(T, L->D, d_in, score, pos, routed, rscore, stream));
        INFMOE_CUDA_TRY(cudaMemcpyAsync(post, routed, sizeof(float) * (size_t)T * L->D, cudaMemcpyDeviceToDevice, stream));
    } else if (L->custom) {
        // A registered sublayer, driven the way the reference drives any MoESubLayer (plugin/MoELayerPlugin.cc:
        // 360-402): for every expert that has rows, its weights go into slot j % max_concurrency on a copy stream
        // while the expert before it runs, then run() on the caller's stream.  One host synchronisation (the
        // token counts), everything after it chained by events.
        INFMOE_TRY(launch_scatter(T, L->D, d_in, score, pos, routed, rscore, stream));
        INFMOE_CUDA_TRY(cudaMemcpyAsync(L->h_count, count, sizeof(int) * L->E, cudaMemcpyDeviceToHost, stream));
        INFMOE_CUDA_TRY(cudaMemcpyAsync(L->h_status, L->d_status, sizeof(int), cudaMemcpyDeviceToHost, stream));
        INFMOE_CUDA_TRY(cudaStreamSynchronize(stream));
        if (*L->h_status) {
            const int st = *L->h_status;
            cudaMemsetAsync(L->d_status, 0, sizeof(int), stream);
            *L->h_status = 0;
            return status_to_rc(st);
        }
        const size_t slot_bytes = L->sub.weight_size ? align_up(L->sub.weight_size(L->sub.user)) : 0;
        char* slots = base + w.custom_slots;
        void* sub_ws = base + w.custom_ws;
        INFMOE_CUDA_TRY(cudaEventRecord(L->ev_fork, stream));
        for (auto cs : L->copy_streams) INFMOE_CUDA_TRY(cudaStreamWaitEvent(cs, L->ev_fork, 0));
        long long row0 = 0;
        size_t j = 0;
        for (int e = 0; e < L->E; ++e) {
            const int n = L->h_count[e];
            if (n == 0) continue;
            const int slot = (int)(j % (size_t)L->mc);
            void* weights = slot_bytes ? slots + slot_bytes * (size_t)slot : nullptr;
            if (slot_bytes && L->sub.copy_weights) {
                cudaStream_t cs = L->copy_streams[j % L->copy_streams.size()];
                if (j >= (size_t)L->mc) INFMOE_CUDA_TRY(cudaStreamWaitEvent(cs, L->ev_freed[slot], 0));
                if (L->sub.copy_weights(L->sub.user, weights, e, cs) != 0) {
                    set_error("sublayer %s: copy_weights failed for expert %d", L->sublayer_type.c_str(), e);
                    return INFMOE_ERR_STATE;
                }
                INFMOE_CUDA_TRY(cudaEventRecord(L->ev_ready[slot], cs));
                INFMOE_CUDA_TRY(cudaStreamWaitEvent(stream, L->ev_ready[slot], 0));
            }
            if (L->sub.run(L->sub.user, e, n, weights, routed + row0 * L->D, post + row0 * L->D, sub_ws, stream) != 0) {
                set_error("sublayer %s: run failed for expert %d", L->sublayer_type.c_str(), e);
                return INFMOE_ERR_STATE;
            }
            INFMOE_CUDA_TRY(cudaEventRecord(L->ev_freed[slot], stream));
            row0 += n;
            ++j;
        }
    } else {
        // 3. scatter fused with the experts' LayerNorm and the TF32 split (:354-355, T5FFLayer.cc:99-103)
        const bool pack = uses_umma(L);   // the GEMM run_ffn picks
        // tensor-core path: no routed copy, the second GEMM's epilogue reads its residual from d_in through pos[]
        if (pack) routed = nullptr;
        INFMOE_TRY(launch_scatter_ln_split(T, L->D, d_in, score, pos, gate_in, s->d_ln, valid_rows, routed, rscore,
                                           h_hi, h_lo, pack, stream));
        if (pack) routed = const_cast<float*>(d_in);   // run_ffn's residual operand
        INFMOE_TRY(prof_mark(L, 3, stream));
        // 4. experts (:360-402)
        if (!streamed) {
            cudaEvent_t mid = nullptr;
            if (L->profiling) mid = L->prof_events[(size_t)(L->prof_calls % PROF_CALLS) * PROF_MARKS + 4];
            INFMOE_TRY(run_ffn(L, T, 0, L->E, offset, nullptr, L->E, s->d_plane, h_hi, h_lo, routed, g_hi, g_lo,
                               ffn_out, stream, mid));
        } else {
            const size_t n = s->matrix_elems();
            // slot planes: w01 [mc] x tiled(2F x D), wo [mc] x tiled(D x F), then one raw landing area per slot
            const size_t n0 = s->plane_elems(0), n1 = s->plane_elems(1);
            float* planes[2];
            planes[0] = (float*)(base + w.slots);
            planes[1] = planes[0] + n0 * L->mc;
            float* staging = planes[1] + n1 * L->mc;
            // the one host synchronisation of the streamed path: which experts have rows?
            INFMOE_CUDA_TRY(cudaMemcpyAsync(L->h_count, count, sizeof(int) * L->E, cudaMemcpyDeviceToHost, stream));
            INFMOE_CUDA_TRY(cudaMemcpyAsync(L->h_status, L->d_status, sizeof(int), cudaMemcpyDeviceToHost, stream));
            INFMOE_CUDA_TRY(cudaStreamSynchronize(stream));
            if (*L->h_status) {
                const int st = *L->h_status;
                cudaMemsetAsync(L->d_status, 0, sizeof(int), stream);
                *L->h_status = 0;
                return status_to_rc(st);
            }
            std::vector<int> active;
            for (int e = 0; e < L->E; ++e)
                if (L->h_count[e] > 0) active.push_back(e);
            // slot of every active expert: round robin over the max_concurrency workspace slots (the reference's
            // scheme, MoELayerPlugin.cc:360-402), or the layer's expert cache when one is configured
            const bool cached = L->cache_slots > 0;
            std::vector<CachePlan> plan(active.size());
            int nslots = L->mc;
            if (cached) {
                INFMOE_TRY(ensure_cache(L));
                plan = plan_cache(L, active);
                planes[0] = L->d_cache[0];
                planes[1] = L->d_cache[1];
                staging = L->d_cache_staging;
                nslots = L->cache_slots;
            } else {
                for (size_t j = 0; j < active.size(); ++j) plan[j] = CachePlan{(int)(j % (size_t)L->mc), true};
            }
            for (int e = 0; e < L->E; ++e) L->h_slot_map[e] = 0;
            for (size_t j = 0; j < active.size(); ++j) L->h_slot_map[active[j]] = plan[j].slot;
            INFMOE_CUDA_TRY(cudaMemcpyAsync(slot_map, L->h_slot_map, sizeof(int) * L->E, cudaMemcpyHostToDevice, stream));
            // copy streams may touch the workspace slots only after everything queued so far on `stream`
            INFMOE_CUDA_TRY(cudaEventRecord(L->ev_fork, stream));
            for (auto cs : L->copy_streams) INFMOE_CUDA_TRY(cudaStreamWaitEvent(cs, L->ev_fork, 0));
            size_t loads = 0;
            bool all_cached = cached && !active.empty();
            for (const CachePlan& pl : plan) all_cached = all_cached && !pl.load;
            if (all_cached) {
                // nothing to copy: one grouped launch over all experts, as in resident mode
                for (const CachePlan& pl : plan) INFMOE_CUDA_TRY(cudaStreamWaitEvent(stream, L->ev_ready[pl.slot], 0));
                INFMOE_TRY(run_ffn(L, T, 0, L->E, offset, slot_map, nslots, planes, h_hi, h_lo, routed, g_hi, g_lo,
                                   ffn_out, stream));
                for (const CachePlan& pl : plan) INFMOE_CUDA_TRY(cudaEventRecord(L->ev_freed[pl.slot], stream));
            }
            for (size_t j = 0; j < active.size() && !all_cached; ++j) {
                const int e = active[j];
                const int slot = plan[j].slot;
                if (plan[j].load) {
                    cudaStream_t cs = L->copy_streams[loads % L->copy_streams.size()];
                    // the slot is free once the expert that used it last has run (an event that was never
                    // recorded does not block)
                    if (cached || j >= (size_t)L->mc) INFMOE_CUDA_TRY(cudaStreamWaitEvent(cs, L->ev_freed[slot], 0));
                    // landing area of the raw matrices: one per workspace slot, or max_concurrency of them in
                    // rotation for the cache, each reusable once its retile kernels are done
                    const int area = cached ? (int)(loads % (size_t)L->mc) : slot;
                    if (cached) INFMOE_CUDA_TRY(cudaStreamWaitEvent(cs, L->ev_stage[area], 0));
                    INFMOE_TRY(load_expert_planes(L->D, L->F, s->h_wi0[e], s->h_wi1[e], s->h_wo[e],
                                                  planes[0] + n0 * slot, planes[1] + n1 * slot, true,
                                                  staging + 3 * n * area, cs));
                    if (cached) INFMOE_CUDA_TRY(cudaEventRecord(L->ev_stage[area], cs));
                    INFMOE_CUDA_TRY(cudaEventRecord(L->ev_ready[slot], cs));
                    L->weight_h2d_bytes += 3ull * n * sizeof(float);
                    ++loads;
                }
                INFMOE_CUDA_TRY(cudaStreamWaitEvent(stream, L->ev_ready[slot], 0));
                INFMOE_TRY(run_ffn(L, T, e, e + 1, offset, slot_map, nslots, planes, h_hi, h_lo, routed, g_hi, g_lo,
                                   ffn_out, stream));
                INFMOE_CUDA_TRY(cudaEventRecord(L->ev_freed[slot], stream));
            }
            INFMOE_TRY(prof_mark(L, 4, stream));   // streamed: copies and both GEMMs are timed together
        }
    }
    INFMOE_TRY(prof_mark(L, 5, stream));
    // 5. combine (:407-412; the gather reads the expert output), unless the GEMM epilogue has done it
    if (fused_combine) {
    } else {
        // with per-row addresses the rows are first combined in the caller's row order (g_hi is free by now:
        // T x d_ff floats), then copied out
        float* ordered = row_dst ? g_hi : d_out;
        if (mix)
            INFMOE_TRY(launch_mix_gather(T, L->D, pos, routed, post, rscore, ordered, stream, valid_rows));
        else
            INFMOE_TRY(launch_gather(T, L->D, post, pos, ordered, stream, valid_rows));
        if (row_dst) INFMOE_TRY(launch_rows_to_ptrs(T, L->D, ordered, row_dst, stream));
    }
    INFMOE_TRY(prof_mark(L, 6, stream));
    if (L->profiling) L->prof_calls++;
    return INFMOE_OK;
}

int infmoe_layer_enqueue(infmoe_layer* L, const float* d_in, float* d_out, void* d_ws, size_t ws_bytes, int64_t T,
                         void* stream_v) {
    return layer_run(L, d_in, d_out, d_ws, ws_bytes, T, stream_v, nullptr);
}

int infmoe_layer_expert_forward(infmoe_layer* L, const float* d_rows, const int32_t* d_expert_of_row, float* d_out,
                                void* d_ws, size_t ws_bytes, int64_t rows, void* stream_v) {
    if (rows > 0 && !d_expert_of_row) {
        set_error("layer_expert_forward: expert index array is required");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0) return INFMOE_OK;
    return layer_run(L, d_rows, d_out, d_ws, ws_bytes, rows, stream_v, d_expert_of_row);
}

int infmoe_layer_expert_forward_scatter(infmoe_layer* L, const float* d_rows, const int32_t* d_expert_of_row,
                                        const float* d_row_score, const uint64_t* d_row_dst, void* d_ws,
                                        size_t ws_bytes, int64_t rows, void* stream_v) {
    if (rows > 0 && (!d_expert_of_row || !d_row_dst)) {
        set_error("layer_expert_forward_scatter: expert index and destination arrays are required");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0) return INFMOE_OK;
    if (L && L->F < L->D) {
        set_error("layer_expert_forward_scatter: needs d_ff >= d_model");   // the ordered rows borrow a d_ff-wide plane
        return INFMOE_ERR_UNSUPPORTED;
    }
    return layer_run(L, d_rows, nullptr, d_ws, ws_bytes, rows, stream_v, d_expert_of_row, d_row_score,
                     reinterpret_cast<const unsigned long long*>(d_row_dst));
}

}  // extern "C"

namespace infmoe {
int layer_run_slots(infmoe_layer* L, const float* d_rows, const int32_t* d_expert_of_slot, const float* d_slot_score,
                    const unsigned long long* d_slot_dst, void* d_ws, size_t ws_bytes, int64_t slots,
                    const int32_t* d_region_count, int32_t region_size, cudaStream_t stream) {
    if (slots > 0 && (!d_expert_of_slot || !d_slot_dst || !d_region_count || region_size <= 0)) {
        set_error("layer_run_slots: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (slots == 0) return INFMOE_OK;
    if (L && L->F < L->D) {
        set_error("layer_run_slots: needs d_ff >= d_model");
        return INFMOE_ERR_UNSUPPORTED;
    }
    return layer_run(L, d_rows, nullptr, d_ws, ws_bytes, slots, (void*)stream, d_expert_of_slot, d_slot_score,
                     d_slot_dst, d_region_count, region_size);
}
}  // namespace infmoe

namespace infmoe {

int layer_snapshot_status(infmoe_layer* L, int* h_word, cudaStream_t stream) {
    if (!L || !h_word) {
        set_error("layer_snapshot_status: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (!L->device_ready) {
        *h_word = 0;
        return INFMOE_OK;
    }
    INFMOE_CUDA_TRY(cudaMemcpyAsync(h_word, L->d_status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    INFMOE_CUDA_TRY(cudaMemsetAsync(L->d_status, 0, sizeof(int), stream));
    return INFMOE_OK;
}

int layer_status_code(int word) { return status_to_rc(word); }

}  // namespace infmoe

extern "C" {

int infmoe_layer_sync_status(infmoe_layer* L, void* stream_v) {
    if (!L) {
        set_error("layer_sync_status: null layer");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (!L->device_ready) return INFMOE_OK;
    cudaStream_t stream = (cudaStream_t)stream_v;
    INFMOE_CUDA_TRY(cudaMemcpyAsync(L->h_status, L->d_status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    INFMOE_CUDA_TRY(cudaMemsetAsync(L->d_status, 0, sizeof(int), stream));
    INFMOE_CUDA_TRY(cudaStreamSynchronize(stream));
    const int st = *L->h_status;
    *L->h_status = 0;
    return status_to_rc(st);
}

int infmoe_layer_forward_host(infmoe_layer* L, const float* h_in, float* h_out, int64_t T) {
    if (!L || T < 0 || (T > 0 && (!h_in || !h_out))) {
        set_error("layer_forward_host: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (L->pipe_submitted != L->pipe_waited) {
        set_error("layer_forward_host: steps submitted with infmoe_layer_submit_host are still in flight");
        return INFMOE_ERR_STATE;
    }
    if (T == 0) return INFMOE_OK;
    if (!L->own_stream) INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&L->own_stream, cudaStreamNonBlocking));
    const size_t io = sizeof(float) * (size_t)T * L->D;
    if (io > L->own_io_bytes) {
        if (L->own_in) cudaFree(L->own_in);
        if (L->own_out) cudaFree(L->own_out);
        L->own_in = L->own_out = nullptr;
        L->own_io_bytes = 0;
        INFMOE_CUDA_TRY(cudaMalloc(&L->own_in, io));
        INFMOE_CUDA_TRY(cudaMalloc(&L->own_out, io));
        L->own_io_bytes = io;
    }
    size_t need = 0;
    INFMOE_TRY(infmoe_layer_workspace_bytes(L, T, &need));
    if (need > L->own_ws_bytes) {
        if (L->own_ws) cudaFree(L->own_ws);
        L->own_ws = nullptr;
        L->own_ws_bytes = 0;
        INFMOE_CUDA_TRY(cudaMalloc(&L->own_ws, need));
        L->own_ws_bytes = need;
    }
    INFMOE_CUDA_TRY(cudaMemcpyAsync(L->own_in, h_in, io, cudaMemcpyHostToDevice, L->own_stream));
    // Page-locked output buffers are written by the last kernel of the layer itself (with the combine fused into
    // the second GEMM the rows cross PCIe while the GEMM is still running); pageable ones get a copy afterwards.
    float* direct = nullptr;
    static const bool allow_direct = [] {
        const char* v = getenv("INFMOE_DIRECT_HOST_OUTPUT");
        return !(v && atoi(v) == 0);
    }();
    if (allow_direct && !L->identity && uses_umma(L)) {
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, h_out) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer)
            direct = (float*)attr.devicePointer;
        else
            (void)cudaGetLastError();
    }
    INFMOE_TRY(infmoe_layer_enqueue(L, L->own_in, direct ? direct : L->own_out, L->own_ws, L->own_ws_bytes, T,
                                    L->own_stream));
    if (!direct) INFMOE_CUDA_TRY(cudaMemcpyAsync(h_out, L->own_out, io, cudaMemcpyDeviceToHost, L->own_stream));
    return infmoe_layer_sync_status(L, L->own_stream);
}

// Host buffers in and out without waiting: at most two steps in flight.  The upload of a step runs on a copy stream
// behind the pass of the step before; the result goes straight into a page-locked h_out from the last kernel of the
// pass, or through a device buffer and a copy on a third stream into a pageable one.
int infmoe_layer_submit_host(infmoe_layer* L, const float* h_in, float* h_out, int64_t T) {
    if (!L || T <= 0 || !h_in || !h_out) {
        set_error("layer_submit_host: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (L->pipe_submitted - L->pipe_waited >= 2) {
        set_error("layer_submit_host: two steps are in flight already; call infmoe_layer_wait_host first");
        return INFMOE_ERR_STATE;
    }
    const size_t io = sizeof(float) * (size_t)T * L->D;
    if (!L->own_stream) INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&L->own_stream, cudaStreamNonBlocking));
    if (!L->pipe_in_stream) {
        INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&L->pipe_in_stream, cudaStreamNonBlocking));
        INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&L->pipe_out_stream, cudaStreamNonBlocking));
        INFMOE_CUDA_TRY(cudaHostAlloc(&L->pipe_h_status, 2 * sizeof(int), cudaHostAllocDefault));
        L->pipe_h_status[0] = L->pipe_h_status[1] = 0;
        for (int i = 0; i < 2; ++i)
            for (cudaEvent_t* e : {&L->pipe_ev_in[i], &L->pipe_ev_pass[i], &L->pipe_ev_out[i]})
                INFMOE_CUDA_TRY(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
    }
    if (io > L->pipe_io_bytes) {
        if (L->pipe_submitted != L->pipe_waited) {
            set_error("layer_submit_host: a larger step cannot be submitted while a smaller one is in flight");
            return INFMOE_ERR_STATE;
        }
        for (int i = 0; i < 2; ++i) {
            if (L->pipe_in[i]) cudaFree(L->pipe_in[i]);
            if (L->pipe_out[i]) cudaFree(L->pipe_out[i]);
            L->pipe_in[i] = L->pipe_out[i] = nullptr;
            L->pipe_used[i] = false;
        }
        L->pipe_io_bytes = 0;
        for (int i = 0; i < 2; ++i) {
            INFMOE_CUDA_TRY(cudaMalloc(&L->pipe_in[i], io));
            INFMOE_CUDA_TRY(cudaMalloc(&L->pipe_out[i], io));
        }
        L->pipe_io_bytes = io;
    }
    size_t need = 0;
    INFMOE_TRY(infmoe_layer_workspace_bytes(L, T, &need));
    if (need > L->own_ws_bytes) {
        INFMOE_CUDA_TRY(cudaStreamSynchronize(L->own_stream));   // a pass in flight may still use the old block
        if (L->own_ws) cudaFree(L->own_ws);
        L->own_ws = nullptr;
        L->own_ws_bytes = 0;
        INFMOE_CUDA_TRY(cudaMalloc(&L->own_ws, need));
        L->own_ws_bytes = need;
    }
    const int s = (int)(L->pipe_submitted & 1);
    cudaStream_t main = L->own_stream;
    // upload: the staging buffer is free once the pass that read it last is done (the second GEMM reads its
    // residual from the input)
    if (L->pipe_used[s]) INFMOE_CUDA_TRY(cudaStreamWaitEvent(L->pipe_in_stream, L->pipe_ev_pass[s], 0));
    INFMOE_CUDA_TRY(cudaMemcpyAsync(L->pipe_in[s], h_in, io, cudaMemcpyHostToDevice, L->pipe_in_stream));
    INFMOE_CUDA_TRY(cudaEventRecord(L->pipe_ev_in[s], L->pipe_in_stream));
    INFMOE_CUDA_TRY(cudaStreamWaitEvent(main, L->pipe_ev_in[s], 0));
    float* direct = nullptr;
    static const bool allow_direct = [] {
        const char* v = getenv("INFMOE_DIRECT_HOST_OUTPUT");
        return !(v && atoi(v) == 0);
    }();
    if (allow_direct && !L->identity && uses_umma(L)) {
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, h_out) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer)
            direct = (float*)attr.devicePointer;
        else
            (void)cudaGetLastError();
    }
    // the device output buffer of this slot has been copied out
    if (!direct && L->pipe_used[s]) INFMOE_CUDA_TRY(cudaStreamWaitEvent(main, L->pipe_ev_out[s], 0));
    INFMOE_TRY(infmoe_layer_enqueue(L, L->pipe_in[s], direct ? direct : L->pipe_out[s], L->own_ws, L->own_ws_bytes, T, main));
    INFMOE_TRY(layer_snapshot_status(L, L->pipe_h_status + s, main));
    INFMOE_CUDA_TRY(cudaEventRecord(L->pipe_ev_pass[s], main));
    if (direct) {
        INFMOE_CUDA_TRY(cudaEventRecord(L->pipe_ev_out[s], main));
    } else {
        INFMOE_CUDA_TRY(cudaStreamWaitEvent(L->pipe_out_stream, L->pipe_ev_pass[s], 0));
        INFMOE_CUDA_TRY(cudaMemcpyAsync(h_out, L->pipe_out[s], io, cudaMemcpyDeviceToHost, L->pipe_out_stream));
        INFMOE_CUDA_TRY(cudaEventRecord(L->pipe_ev_out[s], L->pipe_out_stream));
    }
    L->pipe_used[s] = true;
    L->pipe_submitted++;
    return INFMOE_OK;
}

int infmoe_layer_wait_host(infmoe_layer* L) {
    if (!L) {
        set_error("layer_wait_host: null layer");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (L->pipe_waited == L->pipe_submitted) {
        set_error("layer_wait_host: nothing in flight");
        return INFMOE_ERR_STATE;
    }
    const int s = (int)(L->pipe_waited & 1);
    INFMOE_CUDA_TRY(cudaEventSynchronize(L->pipe_ev_out[s]));
    L->pipe_waited++;
    const int st = L->pipe_h_status[s];
    L->pipe_h_status[s] = 0;
    return status_to_rc(st);
}

int infmoe_layer_last_routing(const infmoe_layer* L, const int32_t** gate, const float** score, const int32_t** pos,
                              const int32_t** count, const int32_t** offset) {
    if (!L) {
        set_error("layer_last_routing: null layer");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (!L->last_gate) {
        set_error("layer_last_routing: no enqueue has run yet");
        return INFMOE_ERR_STATE;
    }
    if (gate) *gate = L->last_gate;
    if (score) *score = L->last_score;
    if (pos) *pos = L->last_pos;
    if (count) *count = L->last_count;
    if (offset) *offset = L->last_offset;
    return INFMOE_OK;
}

int infmoe_layer_set_profiling(infmoe_layer* L, int enable) {
    if (!L) {
        set_error("layer_set_profiling: null layer");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    L->profiling = enable != 0;
    L->prof_calls = 0;
    return INFMOE_OK;
}

int infmoe_layer_stage_ms(infmoe_layer* L, float* ms, int32_t* calls) {
    if (!L || !ms) {
        set_error("layer_stage_ms: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    for (int i = 0; i < PROF_MARKS - 1; ++i) ms[i] = 0.f;
    const int n = L->prof_calls < PROF_CALLS ? L->prof_calls : PROF_CALLS;
    if (calls) *calls = n;
    if (n == 0) return INFMOE_OK;
    for (int c = 0; c < n; ++c) {
        const cudaEvent_t* ev = &L->prof_events[(size_t)c * PROF_MARKS];
        INFMOE_CUDA_TRY(cudaEventSynchronize(ev[PROF_MARKS - 1]));
        for (int i = 0; i < PROF_MARKS - 1; ++i) {
            float t = 0.f;
            // when the experts are streamed the GEMMs are not split by a middle mark
            if (cudaEventElapsedTime(&t, ev[i], ev[i + 1]) != cudaSuccess) {
                cudaGetLastError();
                t = 0.f;
            }
            ms[i] += t / (float)n;
        }
    }
    L->prof_calls = 0;
    return INFMOE_OK;
}

int64_t infmoe_layer_kernel_launches(const infmoe_layer* L) {
    return L ? (int64_t)(g_kernel_launches - L->launches_at_create) : (int64_t)g_kernel_launches;
}

int infmoe_register_sublayer(const char* type_name, const infmoe_sublayer_vtable* vt) {
    if (!type_name || !*type_name || !vt || !vt->run) {
        set_error("register_sublayer: a type name and a run callback are required");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (strcmp(type_name, "T5_FF") == 0 || strcmp(type_name, "Identity") == 0) {
        set_error("register_sublayer: %s is a built-in sublayer type", type_name);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    std::lock_guard<std::mutex> lock(g_sublayer_mu);
    sublayer_registry()[type_name] = *vt;
    return INFMOE_OK;
}

int infmoe_layer_destroy(infmoe_layer* L) {
    if (!L) return INFMOE_OK;
    if (L->device_ready || L->own_stream) {
        cudaDeviceSynchronize();
        free_device_state(L);
    }
    delete L;
    return INFMOE_OK;
}

int infmoe_layer_serialization_size(const infmoe_layer* L, size_t* bytes) {
    if (!L || !bytes) {
        set_error("layer_serialization_size: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    size_t n = 8 + 6 * 4 + 4;                                              // magic, version, 6 ints, flags
    n += L->weight_file.size() + 1 + L->sublayer_type.size() + 1;          // two NUL-terminated strings
    n = (n + 7) / 8 * 8;                                                   // floats start 8-byte aligned
    n += sizeof(float) * L->centroids.size() + sizeof(float) * L->gating_ln.size();
    *bytes = n;
    return INFMOE_OK;
}

int infmoe_layer_serialize(const infmoe_layer* L, void* buffer, size_t bytes) {
    size_t need = 0;
    INFMOE_TRY(infmoe_layer_serialization_size(L, &need));
    if (!buffer || bytes < need) {
        set_error("layer_serialize: buffer of %zu bytes is too small, %zu needed", bytes, need);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    uint8_t* p = (uint8_t*)buffer;
    memset(p, 0, need);
    auto put32 = [&](uint32_t v) {
        memcpy(p, &v, 4);
        p += 4;
    };
    put32(BLOB_MAGIC);
    put32(BLOB_VERSION);
    put32((uint32_t)L->E);                        // field order of plugin/MoELayerPlugin.cc:429-436
    put32((uint32_t)L->D);
    put32((uint32_t)L->F);
    put32((uint32_t)L->mc);
    put32((uint32_t)L->weight_file.size());
    put32((uint32_t)L->sublayer_type.size());
    *p++ = L->flags.layernorm_before_score ? 1 : 0;  // MoEFlags, plugin/MoELayerPlugin.h:36-42
    *p++ = L->flags.base_layer_mix ? 1 : 0;
    p += 2;
    memcpy(p, L->weight_file.c_str(), L->weight_file.size() + 1);
    p += L->weight_file.size() + 1;
    memcpy(p, L->sublayer_type.c_str(), L->sublayer_type.size() + 1);
    p += L->sublayer_type.size() + 1;
    p = (uint8_t*)buffer + ((size_t)(p - (uint8_t*)buffer) + 7) / 8 * 8;
    memcpy(p, L->centroids.data(), sizeof(float) * L->centroids.size());
    p += sizeof(float) * L->centroids.size();
    memcpy(p, L->gating_ln.data(), sizeof(float) * L->gating_ln.size());
    return INFMOE_OK;
}

int infmoe_layer_deserialize(const void* buffer, size_t bytes, infmoe_layer** out) {
    if (!buffer || !out || bytes < 36) {
        set_error("layer_deserialize: blob too short");
        return INFMOE_ERR_FORMAT;
    }
    const uint8_t* p = (const uint8_t*)buffer;
    const uint8_t* end = p + bytes;
    uint32_t v[8];
    memcpy(v, p, 32);
    p += 32;
    if (v[0] != BLOB_MAGIC || v[1] != BLOB_VERSION) {
        set_error("layer_deserialize: bad magic or version");
        return INFMOE_ERR_FORMAT;
    }
    const int E = (int)v[2], D = (int)v[3], F = (int)v[4], mc = (int)v[5];
    const size_t flen = v[6], tlen = v[7];
    const bool ln = p[0] != 0, mix = p[1] != 0;
    p += 4;
    if (E <= 0 || D <= 0 || F <= 0 || mc <= 0 || (size_t)(end - p) < flen + tlen + 2) {
        set_error("layer_deserialize: corrupt header");
        return INFMOE_ERR_FORMAT;
    }
    if (p[flen] != 0 || p[flen + 1 + tlen] != 0) {
        set_error("layer_deserialize: strings are not terminated");
        return INFMOE_ERR_FORMAT;
    }
    const std::string file((const char*)p, flen), type((const char*)p + flen + 1, tlen);
    p += flen + tlen + 2;
    p = (const uint8_t*)buffer + ((size_t)(p - (const uint8_t*)buffer) + 7) / 8 * 8;
    const size_t nfloat = (size_t)E * D + (ln ? (size_t)D : 0);
    if (p > end || (size_t)(end - p) < nfloat * sizeof(float)) {
        set_error("layer_deserialize: blob of %zu bytes is truncated", bytes);
        return INFMOE_ERR_FORMAT;
    }
    std::vector<float> cent((size_t)E * D), gl(ln ? (size_t)D : 0);
    memcpy(cent.data(), p, sizeof(float) * cent.size());
    if (ln) memcpy(gl.data(), p + sizeof(float) * cent.size(), sizeof(float) * gl.size());
    infmoe_layer_config cfg{};
    cfg.expert_count = E;
    cfg.embedding_size = D;
    cfg.hidden_size = F;
    cfg.max_concurrency = mc;
    cfg.expert_centroids = cent.data();
    cfg.layernorm_weight = ln ? gl.data() : nullptr;
    cfg.expert_weight_file = file.c_str();
    cfg.expert_sublayer_type = type.c_str();
    cfg.moe_variant = mix ? "base_layer" : (ln ? "cpm_2" : "default");
    return infmoe_layer_create(&cfg, out);
}

int infmoe_weight_file_check(const char* path, int32_t E, int32_t D, int32_t F, double* h_sums) {
    if (!path || E <= 0 || D <= 0 || F <= 0) {
        set_error("weight_file_check: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    std::vector<int> seen((size_t)E, 0);
    std::vector<float> buf;
    struct Pending { int e, k; size_t n; } pend{-1, 0, 0};
    auto flush = [&]() {
        if (pend.e >= 0 && h_sums) {
            double acc = 0;
            for (size_t i = 0; i < pend.n; ++i) acc += buf[i];
            h_sums[(size_t)pend.e * 4 + pend.k] = acc;
        }
        pend.e = -1;
    };
    auto alloc = [&](const std::string& name, const std::vector<int64_t>& shape, float** dst) -> int {
        flush();
        *dst = nullptr;
        const size_t slash = name.find('/');
        if (slash == std::string::npos) return INFMOE_OK;
        char* endp = nullptr;
        const long e = strtol(name.c_str(), &endp, 10);
        if (endp != name.c_str() + slash || e < 0 || e >= E) return INFMOE_OK;
        const std::string key = name.substr(slash + 1);
        size_t count = 1;
        for (int64_t d : shape) count *= (size_t)d;
        int k = -1;
        size_t want = (size_t)D * F;
        if (key == "layer_norm_weight") { k = 0; want = (size_t)D; }
        else if (key == "wi_0_weight") k = 1;
        else if (key == "wi_1_weight") k = 2;
        else if (key == "wo_weight") k = 3;
        else return INFMOE_OK;
        if (count != want) {
            set_error("%s: %s has %zu elements, expected %zu", path, name.c_str(), count, want);
            return INFMOE_ERR_FORMAT;
        }
        buf.resize(want);
        *dst = buf.data();
        seen[e] |= 1 << k;
        pend = {(int)e, k, want};
        return INFMOE_OK;
    };
    bool fortran = false;
    INFMOE_TRY(npz_read(path, alloc, &fortran));
    flush();
    for (int e = 0; e < E; ++e) {
        if (seen[e] != 15) {
            set_error("%s: expert %d is missing tensors (mask 0x%x of 0xf)", path, e, seen[e]);
            return INFMOE_ERR_FORMAT;
        }
    }
    return INFMOE_OK;
}

int infmoe_layer_get_config(const infmoe_layer* L, infmoe_layer_config* out) {
    if (!L || !out) {
        set_error("layer_get_config: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    out->expert_count = L->E;
    out->embedding_size = L->D;
    out->hidden_size = L->F;
    out->max_concurrency = L->mc;
    out->expert_centroids = L->centroids.data();
    out->layernorm_weight = L->gating_ln.empty() ? nullptr : L->gating_ln.data();
    out->expert_weight_file = L->weight_file.c_str();
    out->expert_sublayer_type = L->sublayer_type.c_str();
    out->moe_variant = L->variant.c_str();
    return INFMOE_OK;
}

// ---- stage entry points -------------------------------------------------------------------------

int infmoe_route(const float* x, const float* centroids, const float* ln_w, int64_t T, int32_t D, int32_t E,
                 int32_t* gate, float* score, int32_t* status, void* stream) {
    return launch_route(x, centroids, ln_w, T, D, E, gate, score, status, (cudaStream_t)stream);
}

int infmoe_expert_select(int64_t T, int32_t E, const float* aff, int32_t* gate, float* weight, int32_t* status,
                         void* stream) {
    return launch_select_top1(T, E, aff, gate, weight, status, (cudaStream_t)stream);
}

int infmoe_expert_count(int64_t T, int32_t E, const int32_t* gate, int32_t* pos, int32_t* count, int32_t* offset,
                        int32_t* status, void* stream) {
    return launch_dispatch(gate, T, E, pos, count, offset, status, (cudaStream_t)stream);
}

int infmoe_expert_scatter(int64_t T, int32_t D, const float* in, const float* coeff, const int32_t* pos,
                          float* routed, float* routed_coeff, void* stream) {
    return launch_scatter(T, D, in, coeff, pos, routed, routed_coeff, (cudaStream_t)stream);
}

int infmoe_expert_gather(int64_t T, int32_t D, const float* routed, const int32_t* pos, float* out, void* stream) {
    return launch_gather(T, D, routed, pos, out, (cudaStream_t)stream);
}

int infmoe_expert_mix_gather(int64_t T, int32_t D, const int32_t* pos, const float* routed, const float* post,
                             const float* coeff, float* out, void* stream) {
    return launch_mix_gather(T, D, pos, routed, post, coeff, out, (cudaStream_t)stream);
}

int infmoe_layernorm(float* out, const float* in, int64_t rows, int32_t cols, const float* gamma, void* stream) {
    return launch_layernorm(out, in, rows, cols, gamma, (cudaStream_t)stream);
}

int infmoe_gelu_dot(const float* a, float* b, size_t len, void* stream) {
    return launch_gelu_dot(a, b, len, (cudaStream_t)stream);
}

}  // extern "C"

namespace {

// One expert's FFN with all scratch carved from `base` (256-byte aligned, infmoe_t5ff_workspace_bytes long):
// the body shared by infmoe_t5ff_run (caller's workspace) and infmoe_t5ff_run_static (the library's own array).
// Everything it reads from the scratch it writes first (offsets, activation planes, weight planes), and it
// clears its status word, so leftovers of an earlier call do not matter.  Blocks until the stream is idle and
// returns the device-side status.
int t5ff_run_in(char* base, int64_t rows, int32_t D, int32_t F, const float* ln_w, const float* wi0, const float* wi1,
                const float* wo, const float* x, float* y, cudaStream_t stream) {
    const size_t r = (size_t)rows, d = (size_t)D, f = (size_t)F;
    char* p = base;
    auto take = [&](size_t bytes) {
        char* at = p;
        p += align_up(bytes);
        return at;
    };
    float* h_hi = (float*)take(4 * r * d);
    float* h_lo = (float*)take(second_plane_bytes(rows, D));
    float* g_hi = (float*)take(4 * r * f);
    float* g_lo = (float*)take(second_plane_bytes(rows, F));
    float* planes[2];
    planes[0] = (float*)take(4 * tiled_elems(2 * F, D));
    planes[1] = (float*)take(4 * tiled_elems(D, F));
    int* offset = (int*)take(8);
    int* status = (int*)take(4);
    // offset[] = {0, rows}: the row count travels as a kernel parameter, so no host buffer has to outlive the call
    INFMOE_CUDA_TRY(cudaMemsetAsync(offset, 0, 4, stream));
    INFMOE_TRY(launch_fill_int(offset + 1, (int)rows, stream));
    INFMOE_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), stream));
    const char* path = getenv("INFMOE_FFN");
    const bool simt = (path && strcmp(path, "simt") == 0) || !ffn_umma_supported(D, F, 1);
    INFMOE_TRY(launch_ln_split(rows, D, x, ln_w, h_hi, h_lo, !simt, stream));
    INFMOE_TRY(load_expert_planes(D, F, wi0, wi1, wo, planes[0], planes[1], false, nullptr, stream));
    int dev = 0, sms = 0;
    INFMOE_CUDA_TRY(cudaGetDevice(&dev));
    INFMOE_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (simt)
        INFMOE_TRY(launch_ffn_simt(rows, D, F, 0, 1, offset, nullptr, h_hi, h_lo, planes[0], planes[1], x, g_hi, g_lo,
                                   y, stream));
    else
        INFMOE_TRY(launch_ffn_umma(rows, D, F, 1, 0, 1, offset, nullptr, 1, h_hi, h_lo, planes[0], planes[1], x, g_hi,
                                   g_lo, y, status, sms, stream));
    int h_status = 0;
    INFMOE_CUDA_TRY(cudaMemcpyAsync(&h_status, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    INFMOE_CUDA_TRY(cudaStreamSynchronize(stream));
    return status_to_rc(h_status);
}

}  // namespace

extern "C" {

int infmoe_t5ff_workspace_bytes(int64_t rows, int32_t D, int32_t F, size_t* bytes) {
    if (!bytes || rows < 0 || D <= 0 || F <= 0) {
        set_error("t5ff_workspace_bytes: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    const size_t r = (size_t)rows, d = (size_t)D, f = (size_t)F;
    *bytes = align_up(4 * r * d) + align_up(second_plane_bytes(rows, D)) + align_up(4 * r * f) +
             align_up(second_plane_bytes(rows, F)) + align_up(4 * tiled_elems(2 * F, D)) +
             align_up(4 * tiled_elems(D, F)) + 2 * ALIGN + ALIGN;
    return INFMOE_OK;
}

int infmoe_t5ff_run(int64_t rows, int32_t D, int32_t F, const float* ln_w, const float* wi0, const float* wi1,
                    const float* wo, const float* x, float* y, void* ws, size_t ws_bytes, void* stream_v) {
    if (rows < 0 || D <= 0 || F <= 0 || !ln_w || !wi0 || !wi1 || !wo || (rows > 0 && (!x || !y || !ws))) {
        set_error("t5ff_run: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0) return INFMOE_OK;
    size_t need = 0;
    INFMOE_TRY(infmoe_t5ff_workspace_bytes(rows, D, F, &need));
    if (ws_bytes < need) {
        set_error("t5ff_run: workspace of %zu bytes is too small, %zu needed", ws_bytes, need);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    char* base = (char*)(((uintptr_t)ws + ALIGN - 1) / ALIGN * ALIGN);
    return t5ff_run_in(base, rows, D, F, ln_w, wi0, wi1, wo, x, y, (cudaStream_t)stream_v);
}

}  // extern "C"

// =================================================================================================
// Expert FFN for callers that must not allocate
// =================================================================================================
// Two kinds of caller may not call cudaMalloc at the moment they need an expert FFN: a TensorRT
// plugin inside enqueue(), whose engine fixed its memory plan when it was built, and a serving loop
// with a hard latency budget, for which the device-wide synchronisation an allocation can cause is
// not acceptable.  infmoe_t5ff_run needs a caller-provided workspace, which such a caller has to
// have planned for in advance.  infmoe_t5ff_run_static needs none: its scratch (LayerNorm output,
// gate activations, the row-interleaved copy of the weight matrices) lives in the array
// below, which is part of the library image.  Every GPU that loads the library keeps these
// INFMOE_STATIC_SCRATCH_BYTES resident until the process exits, so the size is deliberately modest;
// larger problems are rejected and belong to infmoe_t5ff_run.  Like infmoe_t5ff_run the call
// blocks the host until the result is there.
#define INFMOE_STATIC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[INFMOE_STATIC_SCRATCH_BYTES];

namespace {

constexpr int MAX_DEVICES = 64;
std::mutex g_static_mu;
unsigned char* g_static_ptr[MAX_DEVICES] = {};   // device address of g_static_scratch, per device

// In host code `g_static_scratch` is only a handle for the symbol, not an address a kernel can
// use; the device address has to be asked for, once per device, with that device current.
int static_scratch_address(unsigned char** out) {
    int dev = -1;
    INFMOE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) {
        set_error("t5ff_run_static: device index %d out of range", dev);
        return INFMOE_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        INFMOE_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) {
            set_error("t5ff_run_static: cudaGetSymbolAddress returned a null address");
            return INFMOE_ERR_CUDA;
        }
        g_static_ptr[dev] = (unsigned char*)p;
    }
    *out = g_static_ptr[dev];
    return INFMOE_OK;
}

}  // namespace

extern "C" {

int infmoe_t5ff_static_limit(int64_t rows, int32_t D, int32_t F, size_t* needed, size_t* available) {
    size_t need = 0;
    INFMOE_TRY(infmoe_t5ff_workspace_bytes(rows, D, F, &need));
    if (needed) *needed = need;
    if (available) *available = (size_t)INFMOE_STATIC_SCRATCH_BYTES;
    return INFMOE_OK;
}

int infmoe_t5ff_run_static(int64_t rows, int32_t D, int32_t F, const float* ln_w, const float* wi0, const float* wi1,
                           const float* wo, const float* x, float* y, void* stream_v) {
    if (rows < 0 || D <= 0 || F <= 0 || !ln_w || !wi0 || !wi1 || !wo || (rows > 0 && (!x || !y))) {
        set_error("t5ff_run_static: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0) return INFMOE_OK;
    size_t need = 0;
    INFMOE_TRY(infmoe_t5ff_workspace_bytes(rows, D, F, &need));
    if (need > (size_t)INFMOE_STATIC_SCRATCH_BYTES) {
        set_error("t5ff_run_static: rows=%lld d_model=%d d_ff=%d needs %zu bytes of scratch but the built-in array "
                  "holds %u; use infmoe_t5ff_run with a workspace of your own", (long long)rows, D, F, need,
                  INFMOE_STATIC_SCRATCH_BYTES);
        return INFMOE_ERR_UNSUPPORTED;
    }
    unsigned char* scratch = nullptr;
    INFMOE_TRY(static_scratch_address(&scratch));
    // the array is 256-byte aligned already
    return t5ff_run_in((char*)scratch, rows, D, F, ln_w, wi0, wi1, wo, x, y, (cudaStream_t)stream_v);
}

}  // extern "C"
