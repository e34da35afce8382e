// Fused routing for the MoE layer: optional pre-gating LayerNorm, centroid
// scores and top-1 selection in one kernel.
//
// Replaces three reference launches and two host synchronisations:
//   layernorm_gpu        plugin/MoELayerPlugin.cc:324  (kernel plugin/cuda/ops/layernorm.cu:136-174)
//   cublasSgemm_v2       plugin/MoELayerPlugin.cc:334-336  (aff = Xs * C^T)
//   moe_expert_select    plugin/cuda/moe.cu:147-159     (strict '>' scan, first maximum wins)
//
// Layout: X [T][D], centroids [E][D], both row-major FP32.  All arithmetic is explicit
// round-to-nearest FP32 (no tensor cores), in the canonical order of common.cuh: the score of
// (token, expert) is the butterfly sum of 32 partial sums, partial l running over the elements
// k = 128 i + 4 l + c (i ascending, c = 0..3) with fused multiply-adds.
//
// The 32 partial sums are 32 independent small matrix products, and the kernel is blocked like
// one.  A CTA of 16 warps owns 32 tokens and walks over the experts 32 at a time.  Half a warp
// works on one partial index l (lanes 0-15: l = warp, lanes 16-31: l = warp + 16); its 16 threads
// tile the 32 tokens x 32 experts as 4 x 4 threads with 8 x 8 accumulators each.  Per 128-float
// step of the row a thread reads 8 token values and 8 centroid values (one 128-bit shared-memory
// load each, every load shared by four lanes) for 256 fused multiply-adds, so neither the
// shared-memory pipe nor the instruction issue limits the FP32 pipe.  Rows and centroids are
// staged through shared memory with cp.async, 256 floats per row and stage, double buffered; the
// LayerNorm is applied once per staged value, in place, by the thread that fetched it.  After the
// last stage the partial sums of l and l + 16 are combined by a shuffle (the butterfly's first
// step), the other 16 go through shared memory, and a warp per token finishes the butterfly and
// the argmax.
//
// Shared-memory tiles: [stage][step][row][slot] of 16-byte chunks, slot = l ^ (row & 3) ^ (4 if
// l >= 16): consecutive l of one row fill one 512-byte line (conflict-free staging), and the eight
// chunks a warp reads at once (4 rows x 2 values of l) fall into eight different bank groups.
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

constexpr int RT_TOKENS = 32;       // tokens per CTA
constexpr int RT_EXPERTS = 32;      // experts per pass
constexpr int RT_THREADS = 512;
constexpr int RT_STEPS = 2;         // 128-float steps per stage
constexpr int RT_STAGE_FLOATS = RT_STEPS * 128;
constexpr int RT_STAGES = 2;
constexpr int RT_TILE_CHUNKS = RT_STEPS * 32 * 32;             // 16-byte chunks of one tile (tokens or experts) of one stage
constexpr int RT_SMEM = RT_STAGES * 2 * RT_TILE_CHUNKS * 16;   // token and centroid tiles
constexpr int RT_RED_PITCH = 36;    // floats per token row of the partial-sum buffer (32 experts + padding)
static_assert(16 * RT_TOKENS * RT_RED_PITCH * 4 <= RT_SMEM, "the partial sums reuse the tile memory");

__device__ __forceinline__ int rt_slot(int l, int row) { return l ^ (row & 3) ^ ((l >> 4) << 2); }

// LayerNorm statistics of two rows at once, each in the order of warp_row_stats (same bits); interleaving the two
// keeps twice as many loads in flight, which is what bounds this phase.
template <bool VEC>
__device__ __forceinline__ void warp_two_row_stats(const float* __restrict__ r0, const float* __restrict__ r1, int D,
                                                   float (&mean)[2], float (&rstd)[2]) {
    const int lane = threadIdx.x & 31;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
    for (int base = 4 * lane; base < D; base += 128) {
        const float4 a = load_row4(r0, base, D, VEC), b = load_row4(r1, base, D, VEC);
        s0 = __fadd_rn(s0, a.x);
        s1 = __fadd_rn(s1, b.x);
        if (VEC || base + 1 < D) { s0 = __fadd_rn(s0, a.y); s1 = __fadd_rn(s1, b.y); }
        if (VEC || base + 2 < D) { s0 = __fadd_rn(s0, a.z); s1 = __fadd_rn(s1, b.z); }
        if (VEC || base + 3 < D) { s0 = __fadd_rn(s0, a.w); s1 = __fadd_rn(s1, b.w); }
    }
    mean[0] = __fdiv_rn(warp_xor_sum(s0), (float)D);
    mean[1] = __fdiv_rn(warp_xor_sum(s1), (float)D);
    float q0 = 0.f, q1 = 0.f;
#pragma unroll 8
    for (int base = 4 * lane; base < D; base += 128) {
        const float4 a = load_row4(r0, base, D, VEC), b = load_row4(r1, base, D, VEC);
        float d = __fsub_rn(a.x, mean[0]);
        q0 = __fmaf_rn(d, d, q0);
        d = __fsub_rn(b.x, mean[1]);
        q1 = __fmaf_rn(d, d, q1);
        if (VEC || base + 1 < D) {
            d = __fsub_rn(a.y, mean[0]); q0 = __fmaf_rn(d, d, q0);
            d = __fsub_rn(b.y, mean[1]); q1 = __fmaf_rn(d, d, q1);
        }
        if (VEC || base + 2 < D) {
            d = __fsub_rn(a.z, mean[0]); q0 = __fmaf_rn(d, d, q0);
            d = __fsub_rn(b.z, mean[1]); q1 = __fmaf_rn(d, d, q1);
        }
        if (VEC || base + 3 < D) {
            d = __fsub_rn(a.w, mean[0]); q0 = __fmaf_rn(d, d, q0);
            d = __fsub_rn(b.w, mean[1]); q1 = __fmaf_rn(d, d, q1);
        }
    }
    rstd[0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(warp_xor_sum(q0), (float)D), 1e-6f)));
    rstd[1] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(warp_xor_sum(q1), (float)D), 1e-6f)));
}

template <bool VEC>
__global__ void __launch_bounds__(RT_THREADS, 1)
route_kernel(const float* __restrict__ X, const float* __restrict__ C, const float* __restrict__ gamma,
             long long T, int D, int E, int* __restrict__ gate, float* __restrict__ score,
             int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char rt_smem[];
    float4* const xs = reinterpret_cast<float4*>(rt_smem);          // [stage][step][token][slot]
    float4* const cs = xs + RT_STAGES * RT_TILE_CHUNKS;             // [stage][step][expert][slot]
    float* const red = reinterpret_cast<float*>(rt_smem);           // [16][token][RT_RED_PITCH], after the last stage
    __shared__ float s_mean[RT_TOKENS], s_rstd[RT_TOKENS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long t0 = (long long)blockIdx.x * RT_TOKENS;
    const bool use_ln = gamma != nullptr;

    // row statistics, two tokens per warp (rows past the end alias the tile's first row)
    if (use_ln) {
        float mean[2], rstd[2];
        warp_two_row_stats<VEC>(X + (t0 + (t0 + warp < T ? warp : 0)) * (long long)D,
                                X + (t0 + (t0 + warp + 16 < T ? warp + 16 : 0)) * (long long)D, D, mean, rstd);
        if (lane == 0) {
            s_mean[warp] = mean[0];
            s_rstd[warp] = rstd[0];
            s_mean[warp + 16] = mean[1];
            s_rstd[warp + 16] = rstd[1];
        }
    }
    __syncthreads();

    // compute role: partial index l, 8 tokens tt + 4 j, 8 experts te + 4 jj
    const int l = warp + 16 * (lane >> 4);
    const int tt = (lane >> 2) & 3, te = lane & 3;
    // staging role: chunk (step, l) of rows rg + 8 r, r = 0..3
    const int st_step = (tid & 63) >> 5, st_l = tid & 31, rg = tid >> 6;
    const int st_k = st_step * 128 + st_l * 4;   // first float of my chunk inside a stage

    // stages of one pass over the row; tiles past the end of a row (or of the tokens / experts) are zero
    const int nstages = (D + RT_STAGE_FLOATS - 1) / RT_STAGE_FLOATS;
    auto issue = [&](int stage, int e0) {
        const int buf = stage & 1;
        const int k = stage * RT_STAGE_FLOATS + st_k;
        float4* xt = xs + (buf * RT_STEPS + st_step) * 1024;
        float4* ct = cs + (buf * RT_STEPS + st_step) * 1024;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = rg + 8 * r;
            float4* xd = xt + row * 32 + rt_slot(st_l, row);
            float4* cd = ct + row * 32 + rt_slot(st_l, row);
            const bool x_ok = t0 + row < T && k < D, c_ok = e0 + row < E && k < D;
            const float* xsrc = X + (t0 + row) * (long long)D + k;
            const float* csrc = C + (long long)(e0 + row) * D + k;
            if (VEC) {
                if (x_ok) cp_async16(xd, xsrc); else *xd = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c_ok) cp_async16(cd, csrc); else *cd = make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                *xd = x_ok ? load_row4(xsrc, 0, D - k, false) : make_float4(0.f, 0.f, 0.f, 0.f);
                *cd = c_ok ? load_row4(csrc, 0, D - k, false) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    };
    // LayerNorm of the token chunks this thread staged, in place; elements past the row stay zero
    auto load_gamma = [&](int stage) -> float4 {
        const int k = stage * RT_STAGE_FLOATS + st_k;
        return (use_ln && k < D) ? load_row4(gamma, k, D, VEC) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto normalise = [&](int stage, const float4& g) {
        const int buf = stage & 1;
        const int k = stage * RT_STAGE_FLOATS + st_k;
        if (k >= D) return;
        float4* xt = xs + (buf * RT_STEPS + st_step) * 1024;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = rg + 8 * r;
            if (t0 + row >= T) continue;
            float4* xd = xt + row * 32 + rt_slot(st_l, row);
            float4 v = *xd;
            const float mean = s_mean[row], rstd = s_rstd[row];
            v.x = ln_apply(v.x, mean, rstd, g.x);
            v.y = k + 1 < D ? ln_apply(v.y, mean, rstd, g.y) : 0.f;
            v.z = k + 2 < D ? ln_apply(v.z, mean, rstd, g.z) : 0.f;
            v.w = k + 3 < D ? ln_apply(v.w, mean, rstd, g.w) : 0.f;
            *xd = v;
        }
    };

    float best[2] = {-FLT_MAX, -FLT_MAX};   // reference plugin/cuda/moe.cu:26-27; tokens warp and warp + 16
    int best_e[2] = {-1, -1};

    for (int e0 = 0; e0 < E; e0 += RT_EXPERTS) {
        float acc[8][8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) acc[j][jj] = 0.f;

        issue(0, e0);
        cp_async_commit();
        for (int stage = 0; stage < nstages; ++stage) {
            const float4 g = load_gamma(stage);   // in flight while the copies below are issued and awaited
            if (stage + 1 < nstages) issue(stage + 1, e0);
            cp_async_commit();
            cp_async_wait<1>();          // this thread's copies of `stage` have landed
            if (use_ln) normalise(stage, g);
            __syncthreads();             // ... and everybody else's
            const int buf = stage & 1;
#pragma unroll
            for (int step = 0; step < RT_STEPS; ++step) {
                if (stage * RT_STAGE_FLOATS + step * 128 >= D) break;
                const float4* xt = xs + (buf * RT_STEPS + step) * 1024;
                const float4* ct = cs + (buf * RT_STEPS + step) * 1024;
                float4 c[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    const int row = te + 4 * jj;
                    c[jj] = ct[row * 32 + rt_slot(l, row)];
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int row = tt + 4 * j;
                    const float4 x = xt[row * 32 + rt_slot(l, row)];
                    // Elements past the end of a row are zero in both tiles: their products are exact zeros and
                    // leave the partial sums' bits unchanged, so they need no predicate.
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) acc[j][jj] = __fmaf_rn(x.x, c[jj].x, acc[j][jj]);
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) acc[j][jj] = __fmaf_rn(x.y, c[jj].y, acc[j][jj]);
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) acc[j][jj] = __fmaf_rn(x.z, c[jj].z, acc[j][jj]);
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) acc[j][jj] = __fmaf_rn(x.w, c[jj].w, acc[j][jj]);
                }
            }
            __syncthreads();             // everyone is done with this stage's tiles before they are refilled
        }

        // butterfly, first step (xor 16 over l): the two halves of the warp hold l and l + 16 of the same pairs
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int jj = 0; jj < 8; ++jj)
                acc[j][jj] = __fadd_rn(acc[j][jj], __shfl_xor_sync(0xffffffffu, acc[j][jj], 16));
        if (lane < 16) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int jj = 0; jj < 8; ++jj)
                    red[(warp * RT_TOKENS + tt + 4 * j) * RT_RED_PITCH + te + 4 * jj] = acc[j][jj];
        }
        __syncthreads();
        // steps xor 8, 4, 2, 1 and the argmax: warp -> tokens warp and warp + 16, lane -> expert e0 + lane
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int t = warp + 16 * q;
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = red[(i * RT_TOKENS + t) * RT_RED_PITCH + lane];
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1)
#pragma unroll
                for (int i = 0; i < off; ++i) v[i] = __fadd_rn(v[i], v[i + off]);
            // Candidates of this pass have higher indices than the running winner, so they replace it only when
            // strictly greater; among themselves the lowest index wins a tie.  That is the expert the reference's
            // sequential strict '>' scan keeps (plugin/cuda/moe.cu:62-67).  A NaN score is never greater.
            float cand = v[0];
            int cand_e = (e0 + lane < E && cand > best[q]) ? e0 + lane : -1;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                const float os = __shfl_xor_sync(0xffffffffu, cand, off);
                const int oe = __shfl_xor_sync(0xffffffffu, cand_e, off);
                if (oe >= 0 && (cand_e < 0 || os > cand || (os == cand && oe < cand_e))) {
                    cand = os;
                    cand_e = oe;
                }
            }
            if (cand_e >= 0) {
                best[q] = cand;
                best_e[q] = cand_e;
            }
        }
        __syncthreads();   // the partial sums have been read before the next pass refills the tiles
    }
    if (lane == 0) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const long long t = t0 + warp + 16 * q;
            if (t >= T) continue;
            gate[t] = best_e[q];
            if (score) score[t] = best[q];
            if (best_e[q] < 0 && status) atomicOr(status, STATUS_NO_EXPERT);
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
    const long long grid = (T + RT_TOKENS - 1) / RT_TOKENS;
    if (vec) {
        INFMOE_CUDA_TRY(cudaFuncSetAttribute(route_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM));
        route_kernel<true><<<(unsigned)grid, RT_THREADS, RT_SMEM, stream>>>(X, C, gamma, T, D, E, gate, score, status);
    } else {
        INFMOE_CUDA_TRY(cudaFuncSetAttribute(route_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM));
        route_kernel<false><<<(unsigned)grid, RT_THREADS, RT_SMEM, stream>>>(X, C, gamma, T, D, E, gate, score, status);
    }
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
