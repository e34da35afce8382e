// Fused routing for the MoE layer: optional pre-gating LayerNorm, centroid
// scores and top-1 selection in one kernel.
//
// Replaces three reference launches and two host synchronisations:
//   layernorm_gpu        plugin/MoELayerPlugin.cc:324  (kernel plugin/cuda/ops/layernorm.cu:136-174)
//   cublasSgemm_v2       plugin/MoELayerPlugin.cc:334-336  (aff = Xs * C^T)
//   moe_expert_select    plugin/cuda/moe.cu:147-159     (strict '>' scan, first maximum wins)
//
// Layout: X [T][D], centroids [E][D], both row-major FP32.  A CTA owns 4 * TW tokens (TPW = 4 per
// warp; TW token warps, picked per launch so that the CTAs fill whole waves of the SMs).  With more
// than one group of EG experts the CTA has two such sets of warps ("halves"): both work on the same
// tokens, half h takes the expert groups h, h + 2, ..., and their winners are merged at the end, which
// doubles the warps that hide each other's latencies.  The rows of X are read from global memory one 128-float step
// ahead of their use.  Centroids are streamed through shared memory in
// tiles of EG experts x KT floats with double-buffered cp.async, so every
// centroid byte is fetched from L2 once per CTA and every LDS.128 feeds
// 4 * TPW fused multiply-adds; a warp keeps TPW * EG per-lane partial sums in
// registers.  The per-(token, expert) summation order does not depend on the
// blocking, so the result is the canonical order of common.cuh bit for bit.
// All arithmetic is explicit round-to-nearest FP32 (no tensor cores).
#include "common.cuh"

namespace infmoe {

namespace {


__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Fills one shared-memory tile: experts [e0, e0+EG) x floats [k0, k0+KT) of the centroids, zero padded.
template <int EG, int KT, int ROUTE_THREADS>
__device__ __forceinline__ void load_centroid_tile(float* __restrict__ tile, const float* __restrict__ C, int E, int D,
                                                   int e0, int k0, bool vec, int tid) {
    if (vec) {
        for (int idx = tid; idx < EG * (KT / 4); idx += ROUTE_THREADS) {
            const int j = idx / (KT / 4), k = (idx % (KT / 4)) * 4;
            float* dst = tile + j * KT + k;
            if (e0 + j < E && k0 + k < D) cp_async16(dst, C + (long long)(e0 + j) * D + k0 + k);
            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
        for (int idx = tid; idx < EG * KT; idx += ROUTE_THREADS) {
            const int j = idx / KT, k = idx % KT;
            tile[idx] = (e0 + j < E && k0 + k < D) ? C[(long long)(e0 + j) * D + k0 + k] : 0.f;
        }
    }
}

template <int TPW, int EG, int KT, int TW, int HALVES>
__global__ void __launch_bounds__(TW * HALVES * 32)
route_kernel(const float* __restrict__ X, const float* __restrict__ C, const float* __restrict__ gamma,
             long long T, int D, int E, int vec, int* __restrict__ gate, float* __restrict__ score,
             int* __restrict__ status) {
    constexpr int HALF_THREADS = TW * 32;
    extern __shared__ __align__(16) float s_all_tiles[];   // [HALVES][2][EG][KT]
    __shared__ float s_merge_score[TW][TPW];
    __shared__ int s_merge_e[TW][TPW];
    const int lane = threadIdx.x & 31;
    const int half = (threadIdx.x >> 5) / TW;          // which set of expert groups this warp works on
    const int warp = (threadIdx.x >> 5) % TW;          // which tokens
    const int tid = threadIdx.x - half * HALF_THREADS; // thread index inside the half (tile loads)
    float* const s_tiles = s_all_tiles + half * 2 * EG * KT;
    const long long t0 = ((long long)blockIdx.x * TW + warp) * TPW;
    const bool warp_live = t0 < T;   // whole warps past the end still help loading tiles

    const float* rows[TPW];
    float mean[TPW], rstd[TPW];
    bool live[TPW];
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
        live[i] = t0 + i < T;
        rows[i] = X + (live[i] ? (t0 + i) : (warp_live ? t0 : 0)) * (long long)D;  // dead slots alias a valid row
        mean[i] = 0.f;
        rstd[i] = 1.f;
    }
    const bool use_ln = gamma != nullptr;
    if (use_ln) {
        // row statistics once per token: half 0 computes them, the other half reads them from shared memory
        if (warp_live && half == 0) {
#pragma unroll
            for (int i = 0; i < TPW; ++i) warp_row_stats(rows[i], D, vec != 0, mean[i], rstd[i]);
        }
        if (HALVES > 1) {
            __shared__ float s_mean[TW][TPW], s_rstd[TW][TPW];
            if (half == 0 && lane == 0) {
#pragma unroll
                for (int i = 0; i < TPW; ++i) {
                    s_mean[warp][i] = mean[i];
                    s_rstd[warp][i] = rstd[i];
                }
            }
            __syncthreads();
            if (half != 0) {
#pragma unroll
                for (int i = 0; i < TPW; ++i) {
                    mean[i] = s_mean[warp][i];
                    rstd[i] = s_rstd[warp][i];
                }
            }
        }
    }

    float best[TPW];
    int best_e[TPW];
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
        best[i] = -FLT_MAX;   // reference plugin/cuda/moe.cu:26-27
        best_e[i] = -1;
    }

    const int ntiles = (D + KT - 1) / KT;
    // The row values of step s (floats [128 s, 128 s + 128) of the row; lane l owns 4 of them) are fetched while
    // step s - 1 is computed; after the last step of an expert group the first step of the next one follows.
    float4 v_next[TPW], g_next = make_float4(1.f, 1.f, 1.f, 1.f);
    auto fetch = [&](int base) {
        if (base < D && warp_live) {
#pragma unroll
            for (int i = 0; i < TPW; ++i) v_next[i] = load_row4(rows[i], base, D, vec != 0);
            if (use_ln) g_next = load_row4(gamma, base, D, vec != 0);
        }
    };
    fetch(4 * lane);
    // both halves run the same number of group passes (they share the CTA-wide barriers); a pass past the last
    // group loads zero tiles and selects nothing
    const int groups = (E + EG - 1) / EG, passes = (groups + HALVES - 1) / HALVES;
    for (int pass = 0; pass < passes; ++pass) {
        const int e0 = (pass * HALVES + half) * EG;
        float acc[TPW][EG];
#pragma unroll
        for (int i = 0; i < TPW; ++i)
#pragma unroll
            for (int j = 0; j < EG; ++j) acc[i][j] = 0.f;

        load_centroid_tile<EG, KT, HALF_THREADS>(s_tiles, C, E, D, e0, 0, vec != 0, tid);
        cp_async_commit();
        for (int kt = 0; kt < ntiles; ++kt) {
            const float* tile = s_tiles + (kt & 1) * EG * KT;
            if (kt + 1 < ntiles)
                load_centroid_tile<EG, KT, HALF_THREADS>(s_tiles + ((kt + 1) & 1) * EG * KT, C, E, D, e0, (kt + 1) * KT,
                                                         vec != 0, tid);
            cp_async_commit();
            cp_async_wait<1>();   // tile kt has landed (the group of tile kt+1 may still be in flight)
            __syncthreads();
            if (warp_live && e0 < E) {
#pragma unroll 1   // one step is 256 FMAs per lane; unrolling further only thrashes the instruction cache
                for (int it = 0; it < KT / 128; ++it) {
                    const int kl = it * 128 + 4 * lane;       // offset inside the tile
                    const int base = kt * KT + kl;            // offset inside the row
                    // this step's values (normalised if asked for) leave v_next before the next fetch overwrites it
                    float xs[TPW][4];
#pragma unroll
                    for (int i = 0; i < TPW; ++i) {
                        const float4 v = v_next[i];
                        if (use_ln) {
                            xs[i][0] = ln_apply(v.x, mean[i], rstd[i], g_next.x);
                            xs[i][1] = ln_apply(v.y, mean[i], rstd[i], g_next.y);
                            xs[i][2] = ln_apply(v.z, mean[i], rstd[i], g_next.z);
                            xs[i][3] = ln_apply(v.w, mean[i], rstd[i], g_next.w);
                        } else {
                            xs[i][0] = v.x; xs[i][1] = v.y; xs[i][2] = v.z; xs[i][3] = v.w;
                        }
                    }
                    fetch(base + 128 < ntiles * KT ? base + 128 : 4 * lane);
                    if (base < D) {
                        // Positions past the end of a row (D not a multiple of 4) hold zeros in the centroid tile and
                        // a zero gamma or zero x: their products are exact zeros and leave the partial sums'
                        // bits unchanged, so they need no predicate.
#pragma unroll
                        for (int j = 0; j < EG; ++j) {
                            const float4 c = *reinterpret_cast<const float4*>(tile + j * KT + kl);
                            const float cc[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
#pragma unroll
                                for (int i = 0; i < TPW; ++i) acc[i][j] = __fmaf_rn(xs[i][k], cc[k], acc[i][j]);
                            }
                        }
                    }
                }
            }
            __syncthreads();   // everyone is done with tile kt before it is overwritten
        }
#pragma unroll
        for (int j = 0; j < EG; ++j) {
            if (e0 + j < E) {
#pragma unroll
                for (int i = 0; i < TPW; ++i) {
                    const float s = warp_xor_sum(acc[i][j]);
                    if (s > best[i]) {  // strict '>': the first maximum wins (plugin/cuda/moe.cu:62-67)
                        best[i] = s;
                        best_e[i] = e0 + j;
                    }
                }
            }
        }
    }
    if (HALVES > 1) {
        // merge the halves' winners: highest score, lowest expert index among equal scores -- the expert the
        // reference's sequential strict '>' scan would have kept
        if (half == 1 && lane == 0) {
#pragma unroll
            for (int i = 0; i < TPW; ++i) {
                s_merge_score[warp][i] = best[i];
                s_merge_e[warp][i] = best_e[i];
            }
        }
        __syncthreads();
        if (half == 0) {
#pragma unroll
            for (int i = 0; i < TPW; ++i) {
                const float so = s_merge_score[warp][i];
                const int eo = s_merge_e[warp][i];
                if (eo >= 0 && (best_e[i] < 0 || so > best[i] || (so == best[i] && eo < best_e[i]))) {
                    best[i] = so;
                    best_e[i] = eo;
                }
            }
        }
    }
    if (lane == 0 && warp_live && half == 0) {
#pragma unroll
        for (int i = 0; i < TPW; ++i) {
            if (!live[i]) continue;
            gate[t0 + i] = best_e[i];
            if (score) score[t0 + i] = best[i];
            if (best_e[i] < 0 && status) atomicOr(status, STATUS_NO_EXPERT);
        }
    }
}

// Top-1 over a materialised score matrix (one warp per token; lanes scan
// strided expert indices and the lowest index wins ties, which equals the
// reference's sequential strict '>' scan).
__global__ void select_top1_kernel(long long T, int E, const float* __restrict__ aff, int* __restrict__ gate,
                                   float* __restrict__ weight, int* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (t >= T) return;
    const float* row = aff + t * E;
    float best = -FLT_MAX;
    int best_e = -1;
    for (int e = lane; e < E; e += 32) {
        const float s = row[e];
        if (s > best) {
            best = s;
            best_e = e;
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
        const bool take = (oe >= 0) && (best_e < 0 || ob > best || (ob == best && oe < best_e));
        if (take) {
            best = ob;
            best_e = oe;
        }
    }
    if (lane == 0) {
        gate[t] = best_e;
        if (weight) weight[t] = best;
        if (best_e < 0 && status) atomicOr(status, STATUS_NO_EXPERT);
    }
}

}  // namespace

int launch_route(const float* X, const float* C, const float* gamma, long long T, int D, int E, int* gate,
                 float* score, int* status, cudaStream_t stream) {
    if (T < 0 || D <= 0 || E <= 0 || !X || !C || !gate) {
        set_error("route: bad argument (T=%lld D=%d E=%d)", T, D, E);
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (T == 0) return INFMOE_OK;
    const bool vec = (D % 4 == 0) && (((uintptr_t)X | (uintptr_t)C | (uintptr_t)gamma) % 16 == 0);
    constexpr int TPW = 4, EG = 16, KT = 512;
    constexpr int SMEM = 2 * EG * KT * (int)sizeof(float);
    // The kernel is bound by FP32 FMAs, so a CTA's time grows with its warps and the launch takes
    // waves x warps: pick the warp count (5..8) that wastes the least of the last wave.
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        INFMOE_CUDA_TRY(cudaGetDevice(&dev));
        INFMOE_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    const int halves = E > EG / 2 ? 2 : 1;
    int warps = 7;
    long long best_cost = -1;
    for (int w = (halves == 2 ? 7 : 8); w >= 5; --w) {
        const long long ctas = (T + (long long)w * TPW - 1) / ((long long)w * TPW);
        const long long cost = ((ctas + sms - 1) / sms) * w;
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            warps = w;
        }
    }
    const long long grid = (T + (long long)warps * TPW - 1) / ((long long)warps * TPW);
#define INFMOE_ROUTE_LAUNCH(W, H)                                                                                  \
    do {                                                                                                           \
        /* two halves: 8 experts per group and half, so that the accumulators of 448 threads fit the register file */ \
        auto kern = route_kernel<TPW, EG / H, KT, W, H>;                                                           \
        INFMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));            \
        kern<<<(unsigned)grid, W * H * 32, SMEM, stream>>>(X, C, gamma, T, D, E, vec ? 1 : 0, gate, score, status); \
    } while (0)
    switch (warps * 10 + halves) {
        case 51: INFMOE_ROUTE_LAUNCH(5, 1); break;
        case 61: INFMOE_ROUTE_LAUNCH(6, 1); break;
        case 71: INFMOE_ROUTE_LAUNCH(7, 1); break;
        case 81: INFMOE_ROUTE_LAUNCH(8, 1); break;
        case 52: INFMOE_ROUTE_LAUNCH(5, 2); break;
        case 62: INFMOE_ROUTE_LAUNCH(6, 2); break;
        default: INFMOE_ROUTE_LAUNCH(7, 2); break;
    }
#undef INFMOE_ROUTE_LAUNCH
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_select_top1(long long T, int E, const float* aff, int* gate, float* weight, int* status,
                       cudaStream_t stream) {
    if (T < 0 || E <= 0 || !aff || !gate) {
        set_error("expert_select: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (T == 0) return INFMOE_OK;
    const int threads = 256;
    const long long grid = (T * 32 + threads - 1) / threads;
    select_top1_kernel<<<(unsigned)grid, threads, 0, stream>>>(T, E, aff, gate, weight, status);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

}  // namespace infmoe
