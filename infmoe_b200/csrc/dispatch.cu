// Expert dispatch metadata on the device: histogram, exclusive scan and the
// stable counting sort that the reference runs on the host
// (moe_expert_count, plugin/cuda/moe.cu:161-212: D2H copy of gate[], three CPU
// loops, H2D copy of pos[], two stream synchronisations).
//
// One thread-block cluster of 1..8 CTAs (1024 threads each) does the whole job
// in shared memory; the CTAs exchange their per-chunk histograms through
// distributed shared memory and meet at the cluster's hardware barrier, so no
// CTA ever polls memory and no scratch buffer is needed:
//   pass 1  every CTA counts the tokens of its chunks (shared-memory atomics);
//           the cluster-wide totals give count[E] and, after an exclusive scan,
//           offset[E+1]
//   pass 2  super-chunks of C x 1024 tokens in ascending token order, CTA r
//           taking chunk r.  Inside a chunk the rank of a token among equal
//           experts is (tokens of earlier warps, from a 32 x B table) + (earlier
//           lanes of its own warp, from __match_any_sync); across the chunks of a
//           super-chunk it is the sum of the earlier CTAs' chunk histograms; a
//           running per-expert cursor, kept identically by every CTA, carries the
//           order across super-chunks.  pos[offset[e] + rank] = t, i.e. tokens of
//           one expert keep ascending token order exactly like moe.cu:198-200.
//
// Tokens without a usable expert (gate outside [0, E): the routing kernel writes
// -1 when every score is NaN) are counted in an extra bucket behind the last
// expert.  They raise STATUS_BAD_GATE, their indices fill the tail of pos[] in
// ascending order, and offset[E] is the number of VALID tokens -- equal to T, the
// value the reference stores (plugin/MoELayerPlugin.cc:351), whenever every token
// has an expert.  Everything handed on is therefore defined: pos[] is a
// permutation of 0..T-1 and no later stage tiles the rows past offset[E].
//
// Slots of a partly filled receive buffer (expert-parallel path): with
// region_count != NULL the T slots are regions of region_size slots each and only
// the first region_count[s] slots of region s hold rows; the others go to the
// tail bucket silently.
//
// Traffic: gate[] is read twice (8 T bytes, the second read hits L2), pos[] is
// written once.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace infmoe {

namespace {

constexpr int DISPATCH_THREADS = 1024;
constexpr int DISPATCH_WARPS = DISPATCH_THREADS / 32;
constexpr int DISPATCH_MAX_CLUSTER = 8;   // portable cluster size
// per bucket: histogram, cursor, two chunk histograms, chunk base, one row per warp
constexpr int DISPATCH_TABLES = 5 + DISPATCH_WARPS;

__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_kernel(const int* __restrict__ gate, long long T, int E, const int* __restrict__ region_count,
                int region_size, int* __restrict__ pos, int* __restrict__ count, int* __restrict__ offset,
                int* __restrict__ status) {
    cg::cluster_group cluster = cg::this_cluster();
    const int C = (int)cluster.num_blocks(), r = (int)cluster.block_rank();
    extern __shared__ int smem[];
    const int B = E + 1;                  // buckets: experts, then the tail bucket
    int* s_count = smem;                  // [B] tokens of this CTA's chunks per bucket
    int* s_cursor = s_count + B;          // [B] next free slot of each bucket (same in every CTA)
    int* s_chunk = s_cursor + B;          // [2][B] this CTA's histogram of the current chunk, double buffered
    int* s_base = s_chunk + 2 * B;        // [B] first slot of this CTA's chunk
    int* s_warp = s_base + B;             // [DISPATCH_WARPS][B]
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    // bucket of token t; `bad` is raised for a gate outside [0, E) in a slot that holds a row
    auto bucket_of = [&](long long t, bool& bad) -> int {
        if (region_count) {
            const long long s = t / region_size;
            if ((int)(t - s * region_size) >= region_count[s]) return E;   // empty slot
        }
        const int e = gate[t];
        if (e < 0 || e >= E) {   // reference: host assert, plugin/cuda/moe.cu:184
            bad = true;
            return E;
        }
        return e;
    };

    for (int e = tid; e < B; e += DISPATCH_THREADS) s_count[e] = 0;
    __syncthreads();
    bool bad = false;
    const long long super = (long long)C * DISPATCH_THREADS;
    for (long long t = (long long)r * DISPATCH_THREADS + tid; t < T; t += super)
        atomicAdd(&s_count[bucket_of(t, bad)], 1);
    if (bad && status) atomicOr(status, STATUS_BAD_GATE);
    cluster.sync();

    // cluster-wide totals, then their exclusive scan by warp 0, 32 buckets at a time
    for (int e = tid; e < B; e += DISPATCH_THREADS) {
        int total = 0;
        for (int q = 0; q < C; ++q) total += cluster.map_shared_rank(s_count, q)[e];
        s_base[e] = total;
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int e0 = 0; e0 < B; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < B ? s_base[e] : 0;
            int incl = c;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += n;
            }
            if (e < B) {
                const int excl = carry + incl - c;
                s_cursor[e] = excl;
                if (r == 0) {
                    offset[e] = excl;            // offset[E] = number of tokens that have an expert
                    if (e < E) count[e] = c;
                }
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();

    const long long rounds = (T + super - 1) / super;
    for (long long i = 0; i < rounds; ++i) {
        int* chunk = s_chunk + (int)(i & 1) * B;
        for (int x = tid; x < DISPATCH_WARPS * B; x += DISPATCH_THREADS) s_warp[x] = 0;
        __syncthreads();
        const long long t = (i * C + r) * DISPATCH_THREADS + tid;
        bool ignored = false;
        const int e = t < T ? bucket_of(t, ignored) : -1;
        // rank among equal buckets inside the warp, in lane (= token) order
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        if (e >= 0 && rank_in_warp == 0) s_warp[warp * B + e] = __popc(peers);
        __syncthreads();
        // per bucket: exclusive prefix over the 32 warps; the total is this chunk's histogram
        for (int x = tid; x < B; x += DISPATCH_THREADS) {
            int run = 0;
#pragma unroll 4
            for (int w = 0; w < DISPATCH_WARPS; ++w) {
                const int n = s_warp[w * B + x];
                s_warp[w * B + x] = run;
                run += n;
            }
            chunk[x] = run;
        }
        cluster.sync();   // every CTA's chunk histogram is complete
        for (int x = tid; x < B; x += DISPATCH_THREADS) {
            int before = 0, all = 0;
            for (int q = 0; q < C; ++q) {
                const int n = q == r ? chunk[x] : cluster.map_shared_rank(chunk, q)[x];
                if (q < r) before += n;
                all += n;
            }
            s_base[x] = s_cursor[x] + before;
            s_cursor[x] += all;
        }
        __syncthreads();
        if (e >= 0) pos[s_base[e] + s_warp[warp * B + e] + rank_in_warp] = (int)t;
        // The other buffer of s_chunk is written next; this one is overwritten two rounds from now, after
        // the cluster barrier of the next round, which no CTA passes before every CTA has read it.
        __syncthreads();
    }
    cluster.sync();   // no CTA may exit while its shared memory can still be read by another one
}

}  // namespace

size_t dispatch_smem_bytes(int E) { return sizeof(int) * (size_t)DISPATCH_TABLES * (size_t)(E + 1); }

int launch_dispatch(const int* gate, long long T, int E, int* pos, int* count, int* offset, int* status,
                    cudaStream_t stream, const int* region_count, int region_size) {
    if (T < 0 || T > 0x7fffffffLL || E <= 0 || (T > 0 && (!gate || !pos)) || !count || !offset ||
        (region_count && region_size <= 0)) {
        set_error("expert_count: bad argument (T=%lld E=%d)", T, E);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    const size_t smem = dispatch_smem_bytes(E);
    if (smem > 200 * 1024) {
        set_error("expert_count: expert_count %d exceeds the dispatch kernel's shared-memory limit", E);
        return INFMOE_ERR_UNSUPPORTED;
    }
    if (smem > 48 * 1024)
        INFMOE_CUDA_TRY(cudaFuncSetAttribute(dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    // one CTA per 1024-token chunk up to the portable cluster size, rounded to a power of two
    const long long chunks = (T + DISPATCH_THREADS - 1) / DISPATCH_THREADS;
    int cluster = 1;
    while (cluster < DISPATCH_MAX_CLUSTER && cluster < chunks) cluster *= 2;
    static const int forced = [] {
        const char* v = getenv("INFMOE_DISPATCH_CLUSTER");
        return v ? atoi(v) : 0;
    }();
    if (forced == 1 || forced == 2 || forced == 4 || forced == 8) cluster = forced;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster);
    cfg.blockDim = dim3(DISPATCH_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    INFMOE_CUDA_TRY(cudaLaunchKernelEx(&cfg, dispatch_kernel, gate, T, E, region_count, region_size, pos, count, offset,
                                       status));
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

}  // namespace infmoe
