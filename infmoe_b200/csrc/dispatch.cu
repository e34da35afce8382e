// Expert dispatch metadata on the device: histogram, exclusive scan and the
// stable counting sort that the reference runs on the host
// (moe_expert_count, plugin/cuda/moe.cu:161-212: D2H copy of gate[], three CPU
// loops, H2D copy of pos[], two stream synchronisations).
//
// One CTA of 1024 threads does the whole job in shared memory with warp
// match/ballot primitives, so there is no inter-CTA wait anywhere:
//   pass 1  histogram of gate[] (shared-memory atomics) -> count[E]
//   scan    exclusive prefix -> offset[E+1], offset[E] = T (plugin/MoELayerPlugin.cc:351)
//   pass 2  chunks of 1024 tokens in ascending token order; inside a chunk the
//           rank of a token among equal experts is (tokens of earlier warps,
//           from a 32 x E table) + (earlier lanes of its own warp, from
//           __match_any_sync); a running per-expert cursor carries the order
//           across chunks.  pos[offset[e] + rank] = t, i.e. tokens of one expert
//           keep ascending token order exactly like moe.cu:198-200.
// Traffic: gate[] is read twice (8 T bytes, the second read hits L2), pos[] is
// written once.
#include "common.cuh"

namespace infmoe {

namespace {

constexpr int DISPATCH_THREADS = 1024;
constexpr int DISPATCH_WARPS = DISPATCH_THREADS / 32;

__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_kernel(const int* __restrict__ gate, long long T, int E, int* __restrict__ pos, int* __restrict__ count,
                int* __restrict__ offset, int* __restrict__ status) {
    extern __shared__ int smem[];
    int* s_count = smem;                 // [E]
    int* s_cursor = s_count + E;         // [E] next free slot of each expert
    int* s_warp = s_cursor + E;          // [DISPATCH_WARPS][E]
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    for (int e = tid; e < E; e += DISPATCH_THREADS) s_count[e] = 0;
    __syncthreads();
    bool bad = false;
    for (long long t = tid; t < T; t += DISPATCH_THREADS) {
        const int e = gate[t];
        if (e < 0 || e >= E) bad = true;  // reference: host assert, plugin/cuda/moe.cu:184
        else atomicAdd(&s_count[e], 1);
    }
    if (bad && status) atomicOr(status, STATUS_BAD_GATE);
    __syncthreads();

    // exclusive scan over experts by warp 0, 32 at a time
    if (warp == 0) {
        int carry = 0;
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < E ? s_count[e] : 0;
            int incl = c;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += n;
            }
            if (e < E) {
                const int excl = carry + incl - c;
                s_cursor[e] = excl;
                offset[e] = excl;
                count[e] = c;
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) offset[E] = (int)T;
    }
    __syncthreads();

    for (long long c0 = 0; c0 < T; c0 += DISPATCH_THREADS) {
        for (int i = tid; i < DISPATCH_WARPS * E; i += DISPATCH_THREADS) s_warp[i] = 0;
        __syncthreads();
        const long long t = c0 + tid;
        int e = -1;
        if (t < T) {
            e = gate[t];
            if (e < 0 || e >= E) e = -1;
        }
        // rank among equal experts inside the warp, in lane (= token) order
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        if (e >= 0 && rank_in_warp == 0) s_warp[warp * E + e] = __popc(peers);
        __syncthreads();
        // per expert: exclusive prefix over the 32 warps, then advance the cursor
        for (int x = tid; x < E; x += DISPATCH_THREADS) {
            int run = s_cursor[x];
#pragma unroll 4
            for (int w = 0; w < DISPATCH_WARPS; ++w) {
                const int n = s_warp[w * E + x];
                s_warp[w * E + x] = run;
                run += n;
            }
            s_cursor[x] = run;
        }
        __syncthreads();
        if (e >= 0) pos[s_warp[warp * E + e] + rank_in_warp] = (int)t;
        __syncthreads();
    }
}

}  // namespace

size_t dispatch_smem_bytes(int E) { return sizeof(int) * (size_t)(2 + DISPATCH_WARPS) * (size_t)E; }

int launch_dispatch(const int* gate, long long T, int E, int* pos, int* count, int* offset, int* status,
                    cudaStream_t stream) {
    if (T < 0 || T > 0x7fffffffLL || E <= 0 || (T > 0 && (!gate || !pos)) || !count || !offset) {
        set_error("expert_count: bad argument (T=%lld E=%d)", T, E);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    const size_t smem = dispatch_smem_bytes(E);
    if (smem > 200 * 1024) {
        set_error("expert_count: expert_count %d exceeds the single-CTA dispatch limit", E);
        return INFMOE_ERR_UNSUPPORTED;
    }
    if (smem > 48 * 1024)
        INFMOE_CUDA_TRY(cudaFuncSetAttribute(dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    dispatch_kernel<<<1, DISPATCH_THREADS, smem, stream>>>(gate, T, E, pos, count, offset, status);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

}  // namespace infmoe
