// Expert parallelism behind the C ABI: one MoE layer whose experts are sharded
// over the GPUs of one node, one process per GPU.
//
// The reference is single-GPU (device 0 is hard-wired, plugin/MoELayerPlugin.cc:319);
// this file adds the sharding its path allows.  Tokens are data-parallel (every
// rank brings its own rows), experts are sharded in contiguous blocks of E / R.
// One pass, all of it ordered on the caller's stream with no host synchronisation:
//
//   1. routing over all E centroids and dispatch metadata, locally        (route.cu, dispatch.cu)
//   2. ep_send_kernel: every routed row is stored straight into the receive
//      buffer of the rank that owns its expert -- plain peer stores over
//      NVLink from the kernel that gathers the rows, together with the row's
//      local expert index, its token index at home and its routing score.
//      Rank s fills region s of every receive buffer (max_tokens slots), in
//      its own dispatch order, and writes how many slots it filled.
//   3. barrier (a two-word NCCL all-reduce, which also spreads the status word)
//   4. the owner runs its experts over the filled slots (layer_run_slots:
//      dispatch by local expert, LayerNorm + split, the two grouped GEMMs);
//      the second GEMM's epilogue stores every result row into the output
//      buffer of the rank the token came from, at the token's own row
//   5. barrier; the output buffer now holds this rank's tokens in token order
//
// Buffers that other ranks write (receive regions, output) live in one
// cudaMalloc allocation per rank that the others map with CUDA IPC.  No kernel
// waits for another GPU: the only cross-GPU synchronisation is NCCL's.  No TMA
// and no library kernel ever touches peer memory, and nothing uses multicast.
//
// NCCL is loaded at run time (libnccl.so.2, whichever copy the process already
// has), so single-GPU users of the library do not need it.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#if __has_include(<nccl.h>)
#include <nccl.h>
#define INFMOE_HAVE_NCCL 1
#else
#define INFMOE_HAVE_NCCL 0
#endif

#include "common.cuh"
#include "kernels.h"
#include "layer_internal.h"

namespace infmoe {
namespace {

constexpr int EP_MAX_WORLD = 16;
constexpr size_t EP_ALIGN = 256;
inline size_t ep_align(size_t x) { return (x + EP_ALIGN - 1) / EP_ALIGN * EP_ALIGN; }

// The remotely written buffers of every rank as seen from this process.
struct EpPeers {
    float* rows[EP_MAX_WORLD];     // [world * cap][D]  received rows, region s filled by rank s
    int* expert[EP_MAX_WORLD];     // [world * cap]     local expert index of the slot's row
    int* home[EP_MAX_WORLD];       // [world * cap]     token index of the row on the rank it came from
    float* score[EP_MAX_WORLD];    // [world * cap]     routing score of the row
    int* count[EP_MAX_WORLD];      // [world]           filled slots of each region
    float* out[EP_MAX_WORLD];      // [cap][D]          the rank's output rows, token order
};

struct SymLayout {
    size_t rows, expert, home, score, count, out, total;
};

SymLayout sym_layout(int world, long long cap, int D) {
    SymLayout l{};
    size_t o = 0;
    auto take = [&](size_t bytes) {
        const size_t at = o;
        o += ep_align(bytes);
        return at;
    };
    const size_t slots = (size_t)world * (size_t)cap;
    l.rows = take(slots * (size_t)D * 4);
    l.expert = take(slots * 4);
    l.home = take(slots * 4);
    l.score = take(slots * 4);
    l.count = take((size_t)EP_MAX_WORLD * 4);
    l.out = take(2 * (size_t)cap * (size_t)D * 4);   // two output buffers: see infmoe_ep_submit_host
    l.total = o;
    return l;
}

constexpr int SEND_WARPS = 8;

// Step 2 of the pass.  One warp per routed row j (dispatch order): token p = pos[j], expert e = gate[p], owner
// r = e / per; the row is the (j - offset[r * per])-th row this rank sends to r.
__global__ void __launch_bounds__(SEND_WARPS * 32)
ep_send_kernel(long long T, int D, int vec, const float* __restrict__ X, const int* __restrict__ gate,
               const float* __restrict__ score, const int* __restrict__ pos, const int* __restrict__ offset, int E,
               int per, int world, int me, long long cap, EpPeers peers) {
    if (blockIdx.x == 0 && threadIdx.x < world)
        peers.count[threadIdx.x][me] = offset[(threadIdx.x + 1) * per] - offset[threadIdx.x * per];
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * SEND_WARPS + (threadIdx.x >> 5);
    if (j < T && j < offset[E]) {   // rows past offset[E] have no expert
        const int p = pos[j];
        const int e = gate[p];
        const int r = e / per;
        const long long slot = (long long)me * cap + (j - offset[r * per]);
        const float* src = X + (long long)p * D;
        float* dst = peers.rows[r] + slot * D;
        if (vec) {
            const float4* s4 = reinterpret_cast<const float4*>(src);
            float4* d4 = reinterpret_cast<float4*>(dst);
            for (int i = lane; i < D / 4; i += 32) d4[i] = s4[i];
        } else {
            for (int i = lane; i < D; i += 32) dst[i] = src[i];
        }
        if (lane == 0) {
            peers.expert[r][slot] = e - r * per;
            peers.home[r][slot] = p;
            peers.score[r][slot] = score[p];
        }
    }
    __threadfence_system();   // the stores are performed at the peer before the kernel counts as finished
}

// Where the result of every filled slot goes: row home[slot] of the output buffer of the rank owning region slot / cap.
__global__ void ep_prepare_kernel(long long slots, long long cap, int D, const int* __restrict__ count,
                                  const int* __restrict__ home, EpPeers peers, long long out_off,
                                  unsigned long long* __restrict__ dst) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x; s < slots; s += stride) {
        const int src = (int)(s / cap);
        if ((int)(s - (long long)src * cap) < count[src])
            dst[s] = (unsigned long long)(peers.out[src] + out_off + (long long)home[s] * D);
    }
}

__global__ void ep_status_kernel(const int* __restrict__ a, const int* __restrict__ b, int* __restrict__ sync_words) {
    sync_words[0] = (a ? *a : 0) | (b ? *b : 0);
    sync_words[1] = 0;
}

#if INFMOE_HAVE_NCCL
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        const char* override_path = getenv("INFMOE_NCCL_LIB");
        const char* names[] = {override_path, "libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            if (!n || !*n) continue;
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (api.handle) {
            api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
            api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
            api.AllReduce = (decltype(api.AllReduce))dlsym(api.handle, "ncclAllReduce");
            api.AllGather = (decltype(api.AllGather))dlsym(api.handle, "ncclAllGather");
            api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
            if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce || !api.AllGather ||
                !api.GetErrorString) {
                dlclose(api.handle);
                api.handle = nullptr;
            }
        }
    }
    return api.handle ? &api : nullptr;
}

#define INFMOE_NCCL_TRY(api, call)                                                                   \
    do {                                                                                             \
        ncclResult_t r__ = (call);                                                                   \
        if (r__ != ncclSuccess) {                                                                    \
            set_error("NCCL error %d (%s) at %s:%d", (int)r__, (api)->GetErrorString(r__), __FILE__, __LINE__); \
            return INFMOE_ERR_CUDA;                                                                  \
        }                                                                                            \
    } while (0)
#endif

constexpr int EP_MARKS = 6;   // start, sent, barrier 1, experts, barrier 2, copied out
constexpr int EP_PROF_CALLS = 64;

}  // namespace
}  // namespace infmoe

using namespace infmoe;

struct infmoe_ep {
    int rank = 0, world = 1, E = 0, D = 0, F = 0, per = 0;
    long long cap = 0;
    bool mix = false, use_ln = false, loopback = false;
    infmoe_layer* local = nullptr;       // borrowed
    // remotely written buffers
    unsigned char* sym = nullptr;
    SymLayout lay{};
    EpPeers peers{};
    std::vector<void*> opened;           // peer mappings to close
    // private device state
    float* d_centroids = nullptr;
    float* d_gating_ln = nullptr;
    int* d_gate = nullptr;
    float* d_score = nullptr;
    int* d_pos = nullptr;
    int* d_count = nullptr;
    int* d_offset = nullptr;
    unsigned long long* d_slot_dst = nullptr;
    int* d_status = nullptr;
    int* d_sync = nullptr;               // [2] all-reduced words: status of any rank, spare
    int* h_words = nullptr;              // pinned [4]
    void* d_ws = nullptr;
    size_t ws_bytes = 0;
    float* d_x = nullptr;                // input staging of forward_host
    cudaStream_t own_stream = nullptr;
    long long tokens = 0;                // of the pass in flight
    int out_sel = 0;                     // which of the two output buffers the pass in flight fills (same on all ranks)
    // pipelined host path (infmoe_ep_submit_host / _wait_host): two steps in flight
    float* d_xp[2] = {nullptr, nullptr};
    cudaStream_t in_stream = nullptr, out_stream = nullptr;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_sent[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr},
                ev_out[2] = {nullptr, nullptr};
    bool sent_once[2] = {false, false}, out_once[2] = {false, false};
    int* h_step = nullptr;               // pinned [2][4]: status words of the two steps
    long long submitted = 0, waited = 0;
#if INFMOE_HAVE_NCCL
    ncclComm_t comm = nullptr;
#endif
    bool profiling = false;
    std::vector<cudaEvent_t> prof;
    int prof_calls = 0;
};

namespace {

long long ep_out_off(const infmoe_ep* ep) { return (long long)ep->out_sel * ep->cap * ep->D; }

int ep_mark(infmoe_ep* ep, int mark, cudaStream_t stream) {
    if (!ep->profiling) return INFMOE_OK;
    if (ep->prof.empty()) {
        ep->prof.resize((size_t)EP_PROF_CALLS * EP_MARKS);
        for (auto& e : ep->prof) INFMOE_CUDA_TRY(cudaEventCreate(&e));
    }
    INFMOE_CUDA_TRY(cudaEventRecord(ep->prof[(size_t)(ep->prof_calls % EP_PROF_CALLS) * EP_MARKS + mark], stream));
    return INFMOE_OK;
}

void ep_set_peer(infmoe_ep* ep, int r, unsigned char* base) {
    ep->peers.rows[r] = (float*)(base + ep->lay.rows);
    ep->peers.expert[r] = (int*)(base + ep->lay.expert);
    ep->peers.home[r] = (int*)(base + ep->lay.home);
    ep->peers.score[r] = (float*)(base + ep->lay.score);
    ep->peers.count[r] = (int*)(base + ep->lay.count);
    ep->peers.out[r] = (float*)(base + ep->lay.out);
}

int ep_check_config(const infmoe_ep_config* c) {
    if (!c || c->world <= 0 || c->world > EP_MAX_WORLD || c->rank < 0 || c->rank >= c->world || c->expert_count <= 0 ||
        c->expert_count % c->world != 0 || c->embedding_size <= 0 || c->hidden_size <= 0 || c->max_tokens <= 0 ||
        !c->expert_centroids || !c->local_experts || !c->moe_variant) {
        set_error("ep_create: bad configuration (world 1..%d, expert_count divisible by world, max_tokens > 0)",
                  EP_MAX_WORLD);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    infmoe_layer_config lc{};
    INFMOE_TRY(infmoe_layer_get_config(c->local_experts, &lc));
    if (lc.expert_count != c->expert_count / c->world || lc.embedding_size != c->embedding_size ||
        lc.hidden_size != c->hidden_size) {
        set_error("ep_create: the local layer must hold expert_count / world = %d experts of the same sizes",
                  c->expert_count / c->world);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (strcmp(c->moe_variant, "cpm_2") == 0 && !c->layernorm_weight) {
        set_error("ep_create: layernorm_weight is required for moe_variant cpm_2");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (strcmp(c->moe_variant, "cpm_2") != 0 && strcmp(c->moe_variant, "base_layer") != 0 &&
        strcmp(c->moe_variant, "default") != 0) {
        set_error("unsupported moe variant: %s", c->moe_variant);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if ((long long)c->world * c->max_tokens > 0x7fffffffLL / (c->embedding_size > c->hidden_size ? c->embedding_size
                                                                                             : c->hidden_size)) {
        set_error("ep_create: world * max_tokens is too large for 32-bit row offsets");
        return INFMOE_ERR_UNSUPPORTED;
    }
    return INFMOE_OK;
}

// Everything except the peer table and the communicator.
int ep_alloc(const infmoe_ep_config* c, infmoe_ep* ep) {
    ep->rank = c->rank;
    ep->world = c->world;
    ep->E = c->expert_count;
    ep->D = c->embedding_size;
    ep->F = c->hidden_size;
    ep->per = ep->E / ep->world;
    ep->cap = c->max_tokens;
    ep->mix = strcmp(c->moe_variant, "base_layer") == 0;
    ep->use_ln = strcmp(c->moe_variant, "cpm_2") == 0;
    ep->local = c->local_experts;
    ep->lay = sym_layout(ep->world, ep->cap, ep->D);
    INFMOE_CUDA_TRY(cudaMalloc(&ep->sym, ep->lay.total));
    INFMOE_CUDA_TRY(cudaMemset(ep->sym + ep->lay.count, 0, EP_MAX_WORLD * 4));
    const size_t cb = sizeof(float) * (size_t)ep->E * ep->D;
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_centroids, cb));
    INFMOE_CUDA_TRY(cudaMemcpy(ep->d_centroids, c->expert_centroids, cb, cudaMemcpyHostToDevice));
    if (ep->use_ln) {
        INFMOE_CUDA_TRY(cudaMalloc(&ep->d_gating_ln, sizeof(float) * ep->D));
        INFMOE_CUDA_TRY(cudaMemcpy(ep->d_gating_ln, c->layernorm_weight, sizeof(float) * ep->D, cudaMemcpyHostToDevice));
    }
    const size_t cap = (size_t)ep->cap, slots = cap * ep->world;
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_gate, 4 * cap));
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_score, 4 * cap));
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_pos, 4 * cap));
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_count, 4 * (size_t)ep->E));
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_offset, 4 * (size_t)(ep->E + 1)));
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_slot_dst, 8 * slots));
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_status, 4));
    INFMOE_CUDA_TRY(cudaMemset(ep->d_status, 0, 4));
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_sync, 8));
    INFMOE_CUDA_TRY(cudaMemset(ep->d_sync, 0, 8));
    INFMOE_CUDA_TRY(cudaHostAlloc(&ep->h_words, 16, cudaHostAllocDefault));
    memset(ep->h_words, 0, 16);
    INFMOE_TRY(infmoe_layer_workspace_bytes(ep->local, (int64_t)slots, &ep->ws_bytes));
    INFMOE_CUDA_TRY(cudaMalloc(&ep->d_ws, ep->ws_bytes));
    return INFMOE_OK;
}

void ep_free(infmoe_ep* ep) {
    for (void* p : ep->opened) cudaIpcCloseMemHandle(p);
#if INFMOE_HAVE_NCCL
    if (ep->comm) {
        NcclApi* api = nccl_api();
        if (api) api->CommDestroy(ep->comm);
    }
#endif
    void* bufs[] = {ep->sym, ep->d_centroids, ep->d_gating_ln, ep->d_gate, ep->d_score, ep->d_pos, ep->d_count,
                    ep->d_offset, ep->d_slot_dst, ep->d_status, ep->d_sync, ep->d_ws, ep->d_x};
    for (void* p : bufs)
        if (p) cudaFree(p);
    for (int i = 0; i < 2; ++i) {
        if (ep->d_xp[i]) cudaFree(ep->d_xp[i]);
        for (cudaEvent_t e : {ep->ev_in[i], ep->ev_sent[i], ep->ev_done[i], ep->ev_out[i]})
            if (e) cudaEventDestroy(e);
    }
    if (ep->h_step) cudaFreeHost(ep->h_step);
    if (ep->in_stream) cudaStreamDestroy(ep->in_stream);
    if (ep->out_stream) cudaStreamDestroy(ep->out_stream);
    if (ep->h_words) cudaFreeHost(ep->h_words);
    if (ep->own_stream) cudaStreamDestroy(ep->own_stream);
    for (auto e : ep->prof) cudaEventDestroy(e);
    delete ep;
}

int ep_barrier(infmoe_ep* ep, cudaStream_t stream) {
    if (ep->loopback || ep->world == 1) return INFMOE_OK;   // one stream orders everything
#if INFMOE_HAVE_NCCL
    NcclApi* api = nccl_api();
    INFMOE_NCCL_TRY(api, api->AllReduce(ep->d_sync, ep->d_sync, 2, ncclInt32, ncclMax, ep->comm, stream));
    return INFMOE_OK;
#else
    set_error("this build has no NCCL support");
    return INFMOE_ERR_UNSUPPORTED;
#endif
}

int ep_begin(infmoe_ep* ep, const float* d_x, int64_t T, cudaStream_t stream) {
    if (!ep || T < 0 || T > ep->cap || (T > 0 && !d_x)) {
        set_error("ep_forward: bad argument (tokens %lld, max_tokens %lld)", (long long)T, ep ? ep->cap : 0);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    ep->tokens = T;
    INFMOE_TRY(ep_mark(ep, 0, stream));
    if (T > 0) {
        INFMOE_TRY(launch_route(d_x, ep->d_centroids, ep->use_ln ? ep->d_gating_ln : nullptr, T, ep->D, ep->E, ep->d_gate,
                                ep->d_score, ep->d_status, stream));
    }
    // with no tokens the dispatch kernel still writes count[] = 0 and offset[] = 0, and the send kernel the zero counts
    INFMOE_TRY(launch_dispatch(ep->d_gate, T, ep->E, ep->d_pos, ep->d_count, ep->d_offset, ep->d_status, stream));
    const int vec = (ep->D % 4 == 0) && (((uintptr_t)d_x) % 16 == 0);
    const long long grid = T > 0 ? (T + SEND_WARPS - 1) / SEND_WARPS : 1;
    ep_send_kernel<<<(unsigned)grid, SEND_WARPS * 32, 0, stream>>>(T, ep->D, vec, d_x, ep->d_gate, ep->d_score, ep->d_pos,
                                                                  ep->d_offset, ep->E, ep->per, ep->world, ep->rank,
                                                                  ep->cap, ep->peers);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    INFMOE_TRY(ep_mark(ep, 1, stream));
    return INFMOE_OK;
}

int ep_experts(infmoe_ep* ep, cudaStream_t stream) {
    const long long slots = (long long)ep->world * ep->cap;
    const unsigned grid = (unsigned)((slots + 255) / 256 < 1024 ? (slots + 255) / 256 : 1024);
    ep_prepare_kernel<<<grid, 256, 0, stream>>>(slots, ep->cap, ep->D, ep->peers.count[ep->rank], ep->peers.home[ep->rank],
                                                ep->peers, ep_out_off(ep), ep->d_slot_dst);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    INFMOE_TRY(layer_run_slots(ep->local, ep->peers.rows[ep->rank], ep->peers.expert[ep->rank],
                               ep->mix ? ep->peers.score[ep->rank] : nullptr, ep->d_slot_dst, ep->d_ws, ep->ws_bytes, slots,
                               ep->peers.count[ep->rank], (int32_t)ep->cap, stream));
    INFMOE_TRY(ep_mark(ep, 3, stream));
    return INFMOE_OK;
}

int ep_end(infmoe_ep* ep, float* d_out, cudaStream_t stream) {
    float* mine = ep->peers.out[ep->rank] + ep_out_off(ep);
    if (d_out && d_out != mine && ep->tokens > 0)
        INFMOE_CUDA_TRY(cudaMemcpyAsync(d_out, mine, sizeof(float) * (size_t)ep->tokens * ep->D, cudaMemcpyDeviceToDevice,
                                        stream));
    INFMOE_TRY(ep_mark(ep, 5, stream));
    if (ep->profiling) ep->prof_calls++;
    return INFMOE_OK;
}

// One whole pass on `stream`; after_send (or NULL) is recorded once the rows have left (the input is free again).
int ep_pass(infmoe_ep* ep, const float* d_x, float* d_out, int64_t tokens, cudaStream_t stream, cudaEvent_t after_send) {
    INFMOE_TRY(ep_begin(ep, d_x, tokens, stream));
    if (after_send) INFMOE_CUDA_TRY(cudaEventRecord(after_send, stream));
    // the status of routing and dispatch travels with the first barrier
    ep_status_kernel<<<1, 1, 0, stream>>>(ep->d_status, nullptr, ep->d_sync);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    INFMOE_TRY(ep_barrier(ep, stream));       // every rank's rows have arrived
    INFMOE_TRY(ep_mark(ep, 2, stream));
    INFMOE_TRY(ep_experts(ep, stream));
    INFMOE_TRY(ep_barrier(ep, stream));       // every rank's results have been stored
    INFMOE_TRY(ep_mark(ep, 4, stream));
    return ep_end(ep, d_out, stream);
}

}  // namespace

extern "C" {

int infmoe_ep_unique_id(void* h_id) {
#if INFMOE_HAVE_NCCL
    static_assert(INFMOE_EP_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "the id is NCCL's");
    NcclApi* api = nccl_api();
    if (!h_id || !api) {
        set_error(api ? "ep_unique_id: null argument" : "libnccl.so.2 could not be loaded");
        return api ? INFMOE_ERR_INVALID_ARGUMENT : INFMOE_ERR_UNSUPPORTED;
    }
    ncclUniqueId id;
    INFMOE_NCCL_TRY(api, api->GetUniqueId(&id));
    memcpy(h_id, &id, sizeof(id));
    return INFMOE_OK;
#else
    (void)h_id;
    set_error("this build has no NCCL support");
    return INFMOE_ERR_UNSUPPORTED;
#endif
}

int infmoe_ep_create(const infmoe_ep_config* c, infmoe_ep** out) {
    if (!out) {
        set_error("ep_create: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    *out = nullptr;
    INFMOE_TRY(ep_check_config(c));
    if (c->world > 1 && !c->unique_id) {
        set_error("ep_create: unique_id is required when world > 1");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    auto* ep = new infmoe_ep();
    int rc = ep_alloc(c, ep);
    if (rc != INFMOE_OK) {
        ep_free(ep);
        return rc;
    }
    ep_set_peer(ep, ep->rank, ep->sym);
    if (ep->world > 1) {
#if INFMOE_HAVE_NCCL
        NcclApi* api = nccl_api();
        if (!api) {
            set_error("libnccl.so.2 could not be loaded");
            ep_free(ep);
            return INFMOE_ERR_UNSUPPORTED;
        }
        auto fail = [&](int code) {
            ep_free(ep);
            return code;
        };
        ncclUniqueId id;
        memcpy(&id, c->unique_id, sizeof(id));
        ncclResult_t nr = api->CommInitRank(&ep->comm, ep->world, id, ep->rank);
        if (nr != ncclSuccess) {
            set_error("ncclCommInitRank failed: %s", api->GetErrorString(nr));
            ep->comm = nullptr;
            return fail(INFMOE_ERR_CUDA);
        }
        // exchange the IPC handles of the remotely written allocation through the communicator itself
        cudaIpcMemHandle_t mine;
        if (cudaIpcGetMemHandle(&mine, ep->sym) != cudaSuccess) {
            set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(cudaGetLastError()));
            return fail(INFMOE_ERR_CUDA);
        }
        unsigned char* d_handles = nullptr;
        const size_t hb = sizeof(cudaIpcMemHandle_t);
        if (cudaMalloc(&d_handles, hb * (ep->world + 1)) != cudaSuccess) return fail(INFMOE_ERR_CUDA);
        std::vector<cudaIpcMemHandle_t> all((size_t)ep->world);
        bool ok = cudaMemcpy(d_handles + hb * ep->world, &mine, hb, cudaMemcpyHostToDevice) == cudaSuccess;
        ok = ok && api->AllGather(d_handles + hb * ep->world, d_handles, hb, ncclInt8, ep->comm, 0) == ncclSuccess;
        ok = ok && cudaStreamSynchronize(0) == cudaSuccess;
        ok = ok && cudaMemcpy(all.data(), d_handles, hb * ep->world, cudaMemcpyDeviceToHost) == cudaSuccess;
        cudaFree(d_handles);
        if (!ok) {
            set_error("ep_create: exchanging the IPC handles failed");
            return fail(INFMOE_ERR_CUDA);
        }
        for (int r = 0; r < ep->world; ++r) {
            if (r == ep->rank) continue;
            void* p = nullptr;
            if (cudaIpcOpenMemHandle(&p, all[(size_t)r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                set_error("cudaIpcOpenMemHandle for rank %d failed: %s (peer access between the GPUs is required)", r,
                          cudaGetErrorString(cudaGetLastError()));
                return fail(INFMOE_ERR_CUDA);
            }
            ep->opened.push_back(p);
            ep_set_peer(ep, r, (unsigned char*)p);
        }
#else
        ep_free(ep);
        set_error("this build has no NCCL support");
        return INFMOE_ERR_UNSUPPORTED;
#endif
    }
    *out = ep;
    return INFMOE_OK;
}

int infmoe_ep_create_sharded(const infmoe_layer_config* whole, int32_t rank, int32_t world, const void* unique_id,
                             int64_t max_tokens, infmoe_layer** local_out, infmoe_ep** ep_out) {
    if (!whole || !local_out || !ep_out || world <= 0 || rank < 0 || rank >= world || whole->expert_count <= 0 ||
        whole->expert_count % world != 0 || !whole->expert_centroids) {
        set_error("ep_create_sharded: bad argument (expert_count must be divisible by world)");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    *local_out = nullptr;
    *ep_out = nullptr;
    const int per = whole->expert_count / world, lo = rank * per;
    infmoe_layer_config lc = *whole;
    lc.expert_count = per;
    lc.expert_centroids = whole->expert_centroids + (size_t)lo * whole->embedding_size;   // unused by the experts
    lc.layernorm_weight = nullptr;
    lc.moe_variant = "default";   // routing and the output mix are the wrapper's; the local layer only runs experts
    infmoe_layer* local = nullptr;
    INFMOE_TRY(infmoe_layer_create(&lc, &local));
    int rc = infmoe_layer_set_file_expert_offset(local, lo);
    if (rc == INFMOE_OK) rc = infmoe_layer_initialize(local);
    if (rc == INFMOE_OK) rc = infmoe_layer_set_residency(local, 1);
    infmoe_ep_config ec{};
    ec.rank = rank;
    ec.world = world;
    ec.unique_id = unique_id;
    ec.expert_count = whole->expert_count;
    ec.embedding_size = whole->embedding_size;
    ec.hidden_size = whole->hidden_size;
    ec.max_tokens = max_tokens;
    ec.expert_centroids = whole->expert_centroids;
    ec.layernorm_weight = whole->layernorm_weight;
    ec.moe_variant = whole->moe_variant;
    ec.local_experts = local;
    infmoe_ep* ep = nullptr;
    if (rc == INFMOE_OK) rc = infmoe_ep_create(&ec, &ep);
    if (rc != INFMOE_OK) {
        infmoe_layer_destroy(local);
        return rc;
    }
    *local_out = local;
    *ep_out = ep;
    return INFMOE_OK;
}

int infmoe_ep_create_loopback(const infmoe_ep_config* configs, int32_t world, infmoe_ep** outs) {
    if (!configs || !outs || world <= 0 || world > EP_MAX_WORLD) {
        set_error("ep_create_loopback: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    std::vector<infmoe_ep*> made;
    auto undo = [&](int code) {
        for (infmoe_ep* e : made) ep_free(e);
        return code;
    };
    for (int r = 0; r < world; ++r) {
        outs[r] = nullptr;
        if (configs[r].world != world || configs[r].rank != r) {
            set_error("ep_create_loopback: configs[%d] must have rank %d of world %d", r, r, world);
            return undo(INFMOE_ERR_INVALID_ARGUMENT);
        }
        int rc = ep_check_config(&configs[r]);
        if (rc != INFMOE_OK) return undo(rc);
        auto* ep = new infmoe_ep();
        made.push_back(ep);
        ep->loopback = true;
        rc = ep_alloc(&configs[r], ep);
        if (rc != INFMOE_OK) return undo(rc);
        if (ep->cap != made[0]->cap || ep->D != made[0]->D || ep->E != made[0]->E) {
            set_error("ep_create_loopback: all ranks must agree on max_tokens and the layer's sizes");
            return undo(INFMOE_ERR_INVALID_ARGUMENT);
        }
    }
    for (int r = 0; r < world; ++r)
        for (int q = 0; q < world; ++q) ep_set_peer(made[(size_t)r], q, made[(size_t)q]->sym);
    for (int r = 0; r < world; ++r) outs[r] = made[(size_t)r];
    return INFMOE_OK;
}

int infmoe_ep_forward_begin(infmoe_ep* ep, const float* d_x, int64_t tokens, void* stream) {
    return ep_begin(ep, d_x, tokens, (cudaStream_t)stream);
}

int infmoe_ep_forward_experts(infmoe_ep* ep, void* stream) {
    if (!ep) {
        set_error("ep_forward_experts: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    return ep_experts(ep, (cudaStream_t)stream);
}

int infmoe_ep_forward_end(infmoe_ep* ep, float* d_out, void* stream) {
    if (!ep) {
        set_error("ep_forward_end: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    return ep_end(ep, d_out, (cudaStream_t)stream);
}

int infmoe_ep_forward(infmoe_ep* ep, const float* d_x, float* d_out, int64_t tokens, void* stream_v) {
    if (!ep) {
        set_error("ep_forward: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (ep->loopback && ep->world > 1) {
        set_error("ep_forward: loopback ranks are driven phase by phase (forward_begin / _experts / _end)");
        return INFMOE_ERR_STATE;
    }
    if (ep->submitted != ep->waited) {
        set_error("ep_forward: steps submitted with infmoe_ep_submit_host are still in flight");
        return INFMOE_ERR_STATE;
    }
    ep->out_sel = 0;
    return ep_pass(ep, d_x, d_out, tokens, (cudaStream_t)stream_v, nullptr);
}

int infmoe_ep_output(const infmoe_ep* ep, float** d_out) {
    if (!ep || !d_out) {
        set_error("ep_output: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    *d_out = ep->peers.out[ep->rank] + (long long)ep->out_sel * ep->cap * ep->D;
    return INFMOE_OK;
}

int infmoe_ep_sync_status(infmoe_ep* ep, void* stream_v) {
    if (!ep) {
        set_error("ep_sync_status: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    cudaStream_t stream = (cudaStream_t)stream_v;
    INFMOE_CUDA_TRY(cudaMemcpyAsync(ep->h_words, ep->d_status, 4, cudaMemcpyDeviceToHost, stream));
    INFMOE_CUDA_TRY(cudaMemcpyAsync(ep->h_words + 1, ep->d_sync, 4, cudaMemcpyDeviceToHost, stream));
    INFMOE_CUDA_TRY(cudaMemsetAsync(ep->d_status, 0, 4, stream));
    INFMOE_CUDA_TRY(cudaMemsetAsync(ep->d_sync, 0, 8, stream));
    const int rc_local = infmoe_layer_sync_status(ep->local, stream_v);   // synchronises the stream
    INFMOE_CUDA_TRY(cudaStreamSynchronize(stream));
    const int mine = ep->h_words[0], anyone = ep->h_words[1];
    ep->h_words[0] = ep->h_words[1] = 0;
    if (rc_local != INFMOE_OK) return rc_local;
    if (mine & (STATUS_NO_EXPERT | STATUS_BAD_GATE)) {
        set_error("routing selected no expert for at least one token of this rank (NaN in input or centroids)");
        return INFMOE_ERR_NAN;
    }
    if (anyone) {
        set_error("another rank reported device status 0x%x during routing", anyone);
        return INFMOE_ERR_NAN;
    }
    return INFMOE_OK;
}

int infmoe_ep_forward_host(infmoe_ep* ep, const float* h_x, float* h_out, int64_t tokens) {
    if (!ep || tokens < 0 || tokens > (ep ? ep->cap : 0) || (tokens > 0 && (!h_x || !h_out))) {
        set_error("ep_forward_host: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (ep->submitted != ep->waited) {
        set_error("ep_forward_host: steps submitted with infmoe_ep_submit_host are still in flight");
        return INFMOE_ERR_STATE;
    }
    if (!ep->own_stream) INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&ep->own_stream, cudaStreamNonBlocking));
    if (!ep->d_x) INFMOE_CUDA_TRY(cudaMalloc(&ep->d_x, sizeof(float) * (size_t)ep->cap * ep->D));
    const size_t io = sizeof(float) * (size_t)tokens * ep->D;
    if (tokens > 0) INFMOE_CUDA_TRY(cudaMemcpyAsync(ep->d_x, h_x, io, cudaMemcpyHostToDevice, ep->own_stream));
    INFMOE_TRY(infmoe_ep_forward(ep, ep->d_x, nullptr, tokens, ep->own_stream));
    if (tokens > 0)
        INFMOE_CUDA_TRY(cudaMemcpyAsync(h_out, ep->peers.out[ep->rank], io, cudaMemcpyDeviceToHost, ep->own_stream));
    return infmoe_ep_sync_status(ep, ep->own_stream);
}

// Up to two steps in flight: the upload of a step runs on a copy stream behind the previous step's experts, its
// download on another one under the next step's; two input stagings and the two output buffers of the symmetric
// allocation make that safe.  Before a rank joins the first barrier of a step it has finished copying out the output
// buffer the step is going to fill, so after that barrier every rank may store into it.
int infmoe_ep_submit_host(infmoe_ep* ep, const float* h_x, float* h_out, int64_t tokens) {
    if (!ep || tokens < 0 || tokens > (ep ? ep->cap : 0) || (tokens > 0 && (!h_x || !h_out))) {
        set_error("ep_submit_host: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (ep->loopback && ep->world > 1) {
        set_error("ep_submit_host: loopback ranks are driven phase by phase");
        return INFMOE_ERR_STATE;
    }
    if (ep->submitted - ep->waited >= 2) {
        set_error("ep_submit_host: two steps are in flight already; call infmoe_ep_wait_host first");
        return INFMOE_ERR_STATE;
    }
    if (!ep->own_stream) INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&ep->own_stream, cudaStreamNonBlocking));
    if (!ep->in_stream) {
        INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&ep->in_stream, cudaStreamNonBlocking));
        INFMOE_CUDA_TRY(cudaStreamCreateWithFlags(&ep->out_stream, cudaStreamNonBlocking));
        INFMOE_CUDA_TRY(cudaHostAlloc(&ep->h_step, 32, cudaHostAllocDefault));
        memset(ep->h_step, 0, 32);
        for (int i = 0; i < 2; ++i) {
            INFMOE_CUDA_TRY(cudaMalloc(&ep->d_xp[i], sizeof(float) * (size_t)ep->cap * ep->D));
            for (cudaEvent_t* e : {&ep->ev_in[i], &ep->ev_sent[i], &ep->ev_done[i], &ep->ev_out[i]})
                INFMOE_CUDA_TRY(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        }
    }
    const int s = (int)(ep->submitted & 1);
    const size_t io = sizeof(float) * (size_t)tokens * ep->D;
    cudaStream_t main = ep->own_stream;
    // upload: the staging buffer is free once the step that used it last has sent its rows
    if (ep->sent_once[s]) INFMOE_CUDA_TRY(cudaStreamWaitEvent(ep->in_stream, ep->ev_sent[s], 0));
    if (tokens > 0) INFMOE_CUDA_TRY(cudaMemcpyAsync(ep->d_xp[s], h_x, io, cudaMemcpyHostToDevice, ep->in_stream));
    INFMOE_CUDA_TRY(cudaEventRecord(ep->ev_in[s], ep->in_stream));
    INFMOE_CUDA_TRY(cudaStreamWaitEvent(main, ep->ev_in[s], 0));
    // the output buffer this step fills has been copied out (by this rank; the barrier of the pass tells the others)
    if (ep->out_once[s]) INFMOE_CUDA_TRY(cudaStreamWaitEvent(main, ep->ev_out[s], 0));
    ep->out_sel = s;
    INFMOE_TRY(ep_pass(ep, ep->d_xp[s], nullptr, tokens, main, ep->ev_sent[s]));
    ep->sent_once[s] = true;
    // the step's status words, for infmoe_ep_wait_host
    int* hs = ep->h_step + 4 * s;
    INFMOE_CUDA_TRY(cudaMemcpyAsync(hs, ep->d_status, 4, cudaMemcpyDeviceToHost, main));
    INFMOE_CUDA_TRY(cudaMemcpyAsync(hs + 1, ep->d_sync, 4, cudaMemcpyDeviceToHost, main));
    INFMOE_CUDA_TRY(cudaMemsetAsync(ep->d_status, 0, 4, main));
    INFMOE_CUDA_TRY(cudaMemsetAsync(ep->d_sync, 0, 8, main));
    INFMOE_TRY(layer_snapshot_status(ep->local, hs + 2, main));
    INFMOE_CUDA_TRY(cudaEventRecord(ep->ev_done[s], main));
    // download
    INFMOE_CUDA_TRY(cudaStreamWaitEvent(ep->out_stream, ep->ev_done[s], 0));
    if (tokens > 0)
        INFMOE_CUDA_TRY(cudaMemcpyAsync(h_out, ep->peers.out[ep->rank] + ep_out_off(ep), io, cudaMemcpyDeviceToHost,
                                        ep->out_stream));
    INFMOE_CUDA_TRY(cudaEventRecord(ep->ev_out[s], ep->out_stream));
    ep->out_once[s] = true;
    ep->submitted++;
    return INFMOE_OK;
}

int infmoe_ep_wait_host(infmoe_ep* ep) {
    if (!ep) {
        set_error("ep_wait_host: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (ep->waited == ep->submitted) {
        set_error("ep_wait_host: nothing in flight");
        return INFMOE_ERR_STATE;
    }
    const int s = (int)(ep->waited & 1);
    INFMOE_CUDA_TRY(cudaEventSynchronize(ep->ev_out[s]));
    ep->waited++;
    int* hs = ep->h_step + 4 * s;
    const int mine = hs[0], anyone = hs[1], local = hs[2];
    hs[0] = hs[1] = hs[2] = 0;
    const int rc_local = layer_status_code(local);
    if (rc_local != INFMOE_OK) return rc_local;
    if (mine & (STATUS_NO_EXPERT | STATUS_BAD_GATE)) {
        set_error("routing selected no expert for at least one token of this rank (NaN in input or centroids)");
        return INFMOE_ERR_NAN;
    }
    if (anyone) {
        set_error("another rank reported device status 0x%x during routing", anyone);
        return INFMOE_ERR_NAN;
    }
    return INFMOE_OK;
}

int infmoe_ep_last_routing(const infmoe_ep* ep, const int32_t** gate, const float** score, const int32_t** pos,
                           const int32_t** count, const int32_t** offset) {
    if (!ep) {
        set_error("ep_last_routing: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (gate) *gate = ep->d_gate;
    if (score) *score = ep->d_score;
    if (pos) *pos = ep->d_pos;
    if (count) *count = ep->d_count;
    if (offset) *offset = ep->d_offset;
    return INFMOE_OK;
}

int infmoe_ep_received(const infmoe_ep* ep, const int32_t** d_region_count, const int32_t** d_expert_of_slot,
                       const int32_t** d_home_of_slot, int64_t* region_size) {
    if (!ep) {
        set_error("ep_received: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (d_region_count) *d_region_count = ep->peers.count[ep->rank];
    if (d_expert_of_slot) *d_expert_of_slot = ep->peers.expert[ep->rank];
    if (d_home_of_slot) *d_home_of_slot = ep->peers.home[ep->rank];
    if (region_size) *region_size = ep->cap;
    return INFMOE_OK;
}

int infmoe_ep_set_profiling(infmoe_ep* ep, int enable) {
    if (!ep) {
        set_error("ep_set_profiling: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    ep->profiling = enable != 0;
    ep->prof_calls = 0;
    return INFMOE_OK;
}

int infmoe_ep_phase_ms(infmoe_ep* ep, float* ms, int32_t* calls) {
    if (!ep || !ms) {
        set_error("ep_phase_ms: null argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    for (int i = 0; i < EP_MARKS - 1; ++i) ms[i] = 0.f;
    const int n = ep->prof_calls < EP_PROF_CALLS ? ep->prof_calls : EP_PROF_CALLS;
    if (calls) *calls = n;
    for (int c = 0; c < n; ++c) {
        const cudaEvent_t* ev = &ep->prof[(size_t)c * EP_MARKS];
        INFMOE_CUDA_TRY(cudaEventSynchronize(ev[EP_MARKS - 1]));
        for (int i = 0; i < EP_MARKS - 1; ++i) {
            float t = 0.f;
            if (cudaEventElapsedTime(&t, ev[i], ev[i + 1]) != cudaSuccess) {
                cudaGetLastError();
                t = 0.f;
            }
            ms[i] += t / (float)n;
        }
    }
    ep->prof_calls = 0;
    return INFMOE_OK;
}

int infmoe_ep_destroy(infmoe_ep* ep) {
    if (!ep) return INFMOE_OK;
    cudaDeviceSynchronize();
#if INFMOE_HAVE_NCCL
    if (!ep->loopback && ep->world > 1 && ep->comm) {
        // nobody may unmap or free while another rank can still store into this rank's buffers
        NcclApi* api = nccl_api();
        if (api && api->AllReduce(ep->d_sync, ep->d_sync, 2, ncclInt32, ncclMax, ep->comm, 0) == ncclSuccess)
            cudaStreamSynchronize(0);
    }
#endif
    ep_free(ep);
    return INFMOE_OK;
}

}  // extern "C"
