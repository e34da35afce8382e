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
// staged through shared memory with cp.async, 256 floats per row and stage, three buffers; the
// LayerNorm is applied once per staged value, in place, by the thread that fetched it.  After the
// last stage the partial sums of l and l + 16 are combined by a shuffle (the butterfly's first
// step), the other 16 go through shared memory, and a warp per token finishes the butterfly and
// the argmax.
//
// Shared-memory tiles: [stage][step][row][slot] of 16-byte chunks, slot = l ^ (row & 3) ^ (4 if
// l >= 16): consecutive l of one row fill one 512-byte line (conflict-free staging), and the eight
// chunks a warp reads at once (4 rows x 2 values of l) fall into eight different bank groups.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

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
constexpr int RT_THREADS = 256;
constexpr int RT_STEPS = 2;         // 128-float steps per stage
constexpr int RT_STAGE_FLOATS = RT_STEPS * 128;
constexpr int RT_STAGES = 3;
constexpr int RT_TILE_CHUNKS = RT_STEPS * 32 * 32;             // 16-byte chunks of one tile (tokens or experts) of one stage
constexpr int RT_SMEM = RT_STAGES * 2 * RT_TILE_CHUNKS * 16;   // token and centroid tiles
constexpr int RT_RED_PITCH = 36;    // floats per token row of the partial-sum buffer (32 experts + padding)
static_assert(8 * RT_TOKENS * RT_RED_PITCH * 4 <= RT_SMEM, "the partial sums reuse the tile memory");

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

// The same for four aligned rows at once: the statistics phase waits for HBM, and what it gets is what it has in
// flight (16 KB per warp here against 8 KB with two rows).
__device__ __forceinline__ void warp_four_row_stats(const float* const (&r)[4], int D, float (&mean)[4], float (&rstd)[4]) {
    const int lane = threadIdx.x & 31;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int base = 4 * lane; base < D; base += 128) {
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = *reinterpret_cast<const float4*>(r[i] + base);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s[i] = __fadd_rn(s[i], v[i].x);
            s[i] = __fadd_rn(s[i], v[i].y);
            s[i] = __fadd_rn(s[i], v[i].z);
            s[i] = __fadd_rn(s[i], v[i].w);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) mean[i] = __fdiv_rn(warp_xor_sum(s[i]), (float)D);
    float q[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int base = 4 * lane; base < D; base += 128) {
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = *reinterpret_cast<const float4*>(r[i] + base);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float d = __fsub_rn(v[i].x, mean[i]);
            q[i] = __fmaf_rn(d, d, q[i]);
            d = __fsub_rn(v[i].y, mean[i]);
            q[i] = __fmaf_rn(d, d, q[i]);
            d = __fsub_rn(v[i].z, mean[i]);
            q[i] = __fmaf_rn(d, d, q[i]);
            d = __fsub_rn(v[i].w, mean[i]);
            q[i] = __fmaf_rn(d, d, q[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
        rstd[i] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(warp_xor_sum(q[i]), (float)D), 1e-6f)));
}

template <bool VEC>
__global__ void __launch_bounds__(RT_THREADS, 1)
route_kernel(const float* __restrict__ X, const float* __restrict__ C, const float* __restrict__ gamma,
             long long T, int D, int E, int* __restrict__ gate, float* __restrict__ score,
             int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char rt_smem[];
    float4* const xs = reinterpret_cast<float4*>(rt_smem);          // [stage][step][token][slot]
    float4* const cs = xs + RT_STAGES * RT_TILE_CHUNKS;             // [stage][step][expert][slot]
    float* const red = reinterpret_cast<float*>(rt_smem);           // [8][token][RT_RED_PITCH], after the last stage
    __shared__ float s_mean[RT_TOKENS], s_rstd[RT_TOKENS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long t0 = (long long)blockIdx.x * RT_TOKENS;
    const bool use_ln = gamma != nullptr;
    // row statistics, four tokens per warp, two at a time (rows past the end alias the tile's first row)
    if (use_ln) {
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const int ra = warp + 16 * p, rb = ra + 8;
            float mean[2], rstd[2];
            warp_two_row_stats<VEC>(X + (t0 + (t0 + ra < T ? ra : 0)) * (long long)D,
                                    X + (t0 + (t0 + rb < T ? rb : 0)) * (long long)D, D, mean, rstd);
            if (lane == 0) {
                s_mean[ra] = mean[0];
                s_rstd[ra] = rstd[0];
                s_mean[rb] = mean[1];
                s_rstd[rb] = rstd[1];
            }
        }
    }
    __syncthreads();

    // compute role: partial index l = 8 (lane / 8) + warp, 16 tokens tt + 2 j, 8 experts te + 4 jj
    const int l = 8 * (lane >> 3) + warp;
    const int tt = (lane >> 2) & 1, te = lane & 3;
    const int xslot0 = rt_slot(l, tt), xslot1 = rt_slot(l, tt + 2);   // rows tt + 2 j: j even / odd
    const int cslot = rt_slot(l, te);
    // staging role: chunk (step, l) of rows rg + 4 r, r = 0..7
    const int st_step = (tid >> 5) & 1, st_l = tid & 31, rg = tid >> 6;
    const int st_k = st_step * 128 + st_l * 4;   // first float of my chunk inside a stage

    // stages of one pass over the row; tiles past the end of a row (or of the tokens / experts) are zero
    const int nstages = (D + RT_STAGE_FLOATS - 1) / RT_STAGE_FLOATS;
    auto issue = [&](int stage, int buf, int e0) {
        const int k = stage * RT_STAGE_FLOATS + st_k;
        float4* xt = xs + (buf * RT_STEPS + st_step) * 1024;
        float4* ct = cs + (buf * RT_STEPS + st_step) * 1024;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int row = rg + 4 * r;
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
    auto normalise = [&](int stage, int buf, const float4& g) {
        const int k = stage * RT_STAGE_FLOATS + st_k;
        if (k >= D) return;
        float4* xt = xs + (buf * RT_STEPS + st_step) * 1024;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int row = rg + 4 * r;
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

    float best[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};   // reference plugin/cuda/moe.cu:26-27; tokens warp + 8 q
    int best_e[4] = {-1, -1, -1, -1};

    for (int e0 = 0; e0 < E; e0 += RT_EXPERTS) {
        float acc[16][8];
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) acc[j][jj] = 0.f;

        // Three buffers.  While the warps of a CTA multiply stage s, each of them, when it is done, waits for its own
        // copies of stage s + 1 and normalises them, so that this work overlaps the other warps' multiply-adds
        // instead of standing between two barriers; the copies of stage s + 2 go out before the multiply-adds.
        issue(0, 0, e0);
        cp_async_commit();
        if (nstages > 1) issue(1, 1, e0);
        cp_async_commit();
        float4 g = load_gamma(0);
        cp_async_wait<1>();              // this thread's copies of stage 0 have landed
        if (use_ln) normalise(0, 0, g);
        g = load_gamma(1);
        __syncthreads();
        for (int stage = 0, buf = 0; stage < nstages; ++stage, buf = buf == RT_STAGES - 1 ? 0 : buf + 1) {
            const int next = buf == RT_STAGES - 1 ? 0 : buf + 1, after = next == RT_STAGES - 1 ? 0 : next + 1;
            // buffer `after` was read in stage - 1, which every thread left before the barrier that ended it
            if (stage + 2 < nstages) issue(stage + 2, after, e0);
            cp_async_commit();
#pragma unroll
            for (int step = 0; step < RT_STEPS; ++step) {
                if (stage * RT_STAGE_FLOATS + step * 128 >= D) break;
                const float4* xt = xs + (buf * RT_STEPS + step) * 1024;
                const float4* ct = cs + (buf * RT_STEPS + step) * 1024;
                float4 c[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) c[jj] = ct[(te + 4 * jj) * 32 + cslot];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float4 x = xt[(tt + 2 * j) * 32 + ((j & 1) ? xslot1 : xslot0)];
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
            if (stage + 1 < nstages) {
                cp_async_wait<1>();      // this thread's copies of stage + 1 have landed
                if (use_ln) normalise(stage + 1, next, g);
                g = load_gamma(stage + 2);
            }
            __syncthreads();             // stage + 1 is complete for everybody; everybody is done with `stage`
        }
        // butterfly, first two steps (xor 16 and xor 8 over l): the four quarters of the warp hold l, l + 8, l + 16
        // and l + 24 of the same (token, expert) pairs
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                acc[j][jj] = __fadd_rn(acc[j][jj], __shfl_xor_sync(0xffffffffu, acc[j][jj], 16));
                acc[j][jj] = __fadd_rn(acc[j][jj], __shfl_xor_sync(0xffffffffu, acc[j][jj], 8));
            }
        if (lane < 8) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
#pragma unroll
                for (int jj = 0; jj < 8; ++jj)
                    red[(warp * RT_TOKENS + tt + 2 * j) * RT_RED_PITCH + te + 4 * jj] = acc[j][jj];
        }
        __syncthreads();
        // steps xor 4, 2, 1 and the argmax: warp -> tokens warp + 8 q, lane -> expert e0 + lane
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int t = warp + 8 * q;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = red[(i * RT_TOKENS + t) * RT_RED_PITCH + lane];
#pragma unroll
            for (int off = 4; off >= 1; off >>= 1)
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
        for (int q = 0; q < 4; ++q) {
            const long long t = t0 + warp + 8 * q;
            if (t >= T) continue;
            gate[t] = best_e[q];
            if (score) score[t] = best[q];
            if (best_e[q] < 0 && status) atomicOr(status, STATUS_NO_EXPERT);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same kernel with the tiles fetched by TMA.  Issuing 4096 16-byte cp.async copies per stage costs the CTA about
// 1500 cycles of its load/store pipe, as much as half of the multiply-adds of the stage; one thread issuing 16
// tensor copies (boxes of 32 floats x 32 rows, eight per tile) costs nothing.  Rows past the tokens, the experts or
// the end of a row are zero-filled by the copy.  The 128-byte swizzle of the copy takes the place of rt_slot: 16-byte
// chunk c of row r of a box sits at chunk c ^ (r & 7), which keeps both the normalising and the multiplying reads
// (rows r, r + 1 or r .. r + 3 within a quarter warp) free of bank conflicts.  The partial sums of all 32 values of
// l go through shared memory (the three stage buffers leave room for them), which replaces 256 shuffles per thread.
// Needs 16-byte aligned rows (D % 4 == 0); other shapes take route_kernel.
__device__ __forceinline__ uint32_t rt_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long rt_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool rt_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up (and tells the other threads to) two seconds after it started.
__device__ __forceinline__ bool rt_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (rt_mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = rt_global_ns();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (rt_mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (rt_global_ns() - t0 > 2000000000ull) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void rt_tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

constexpr int RT_RED_L = 1153;      // floats between the partial sums of l and l + 1 (odd: conflict-free stores)
static_assert(32 * RT_RED_L * 4 <= RT_SMEM, "the partial sums reuse the tile memory");
// float4 index of chunk l of row `row` in the tile of one stage (boxes: [step][l / 8][row][8 chunks])
__device__ __forceinline__ int rt_box_idx(int step, int l, int row) {
    return ((step * 4 + (l >> 3)) * 32 + row) * 8 + ((l & 7) ^ (row & 7));
}

__global__ void __launch_bounds__(RT_THREADS, 1)
route_tma_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_c,
                 const float* __restrict__ X, const float* __restrict__ gamma, long long T, int D, int E,
                 int* __restrict__ gate, float* __restrict__ score, int* __restrict__ status) {
    extern __shared__ unsigned char rt_smem_raw[];
    unsigned char* const rt_smem = rt_smem_raw + ((1024u - (rt_smem_u32(rt_smem_raw) & 1023u)) & 1023u);
    float4* const xs = reinterpret_cast<float4*>(rt_smem);          // [buffer][step][box][token][chunk]
    float4* const cs = xs + RT_STAGES * RT_TILE_CHUNKS;             // [buffer][step][box][expert][chunk]
    float* const red = reinterpret_cast<float*>(rt_smem);           // [l][token][RT_RED_PITCH] at pitch RT_RED_L
    __shared__ float s_mean[RT_TOKENS], s_rstd[RT_TOKENS];
    __shared__ __align__(8) uint64_t s_full[RT_STAGES];
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long t0 = (long long)blockIdx.x * RT_TOKENS;
    const bool use_ln = gamma != nullptr;
    volatile int* abort_flag = &s_abort;

    const int nstages = (D + RT_STAGE_FLOATS - 1) / RT_STAGE_FLOATS;
    const uint32_t xs_addr = rt_smem_u32(xs), cs_addr = rt_smem_u32(cs);
    // one thread: the 16 copies of a stage (gs counts the stages of all passes; buffer and barrier gs % RT_STAGES)
    auto issue = [&](uint32_t gs, int stage, int e0) {
        const uint32_t buf = gs % RT_STAGES, bar = rt_smem_u32(&s_full[buf]);
        // the buffer was last touched by ordinary loads and stores; order them before the copies' writes
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2u * RT_TILE_CHUNKS * 16u)
                     : "memory");
#pragma unroll
        for (int b = 0; b < RT_STEPS * 4; ++b) {
            const int k0 = stage * RT_STAGE_FLOATS + b * 32;
            rt_tma_load_2d(xs_addr + (buf * RT_TILE_CHUNKS + b * 256) * 16, &map_x, bar, k0, (int)t0);
            rt_tma_load_2d(cs_addr + (buf * RT_TILE_CHUNKS + b * 256) * 16, &map_c, bar, k0, e0);
        }
    };
    if (tid == 0) {
        for (int i = 0; i < RT_STAGES; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(rt_smem_u32(&s_full[i])), "r"(1u) : "memory");
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the first two stages of the first pass are fetched while the warps compute the row statistics
        issue(0, 0, 0);
        if (nstages > 1) issue(1, 1, 0);
    }
    if (use_ln) {   // rows warp + 8 i of the tile; rows past the end alias the tile's first row
        const float* rows[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) rows[i] = X + (t0 + (t0 + warp + 8 * i < T ? warp + 8 * i : 0)) * (long long)D;
        float mean[4], rstd[4];
        warp_four_row_stats(rows, D, mean, rstd);
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                s_mean[warp + 8 * i] = mean[i];
                s_rstd[warp + 8 * i] = rstd[i];
            }
        }
    }
    __syncthreads();

    // compute role: partial index l = 8 (lane / 8) + warp, 16 tokens tt + 2 j, 8 experts te + 4 jj
    const int l = 8 * (lane >> 3) + warp;
    const int tt = (lane >> 2) & 1, te = lane & 3;
    // normalising role: chunk (step, l) of rows rg + 4 r, r = 0..7
    const int st_step = (tid >> 5) & 1, st_l = tid & 31, rg = tid >> 6;
    const int st_k = st_step * 128 + st_l * 4;

    auto load_gamma = [&](int stage) -> float4 {
        const int k = stage * RT_STAGE_FLOATS + st_k;
        return (use_ln && k < D) ? load_row4(gamma, k, D, true) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    // LayerNorm of the token chunks of this thread, in place; chunks past the row (zero-filled) stay zero
    auto normalise = [&](int stage, uint32_t buf, const float4& g) {
        const int k = stage * RT_STAGE_FLOATS + st_k;
        if (k >= D) return;
        float4* xt = xs + buf * RT_TILE_CHUNKS;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int row = rg + 4 * r;
            if (t0 + row >= T) continue;
            float4* xd = xt + rt_box_idx(st_step, st_l, row);
            float4 v = *xd;
            const float mean = s_mean[row], rstd = s_rstd[row];
            v.x = ln_apply(v.x, mean, rstd, g.x);
            v.y = ln_apply(v.y, mean, rstd, g.y);
            v.z = ln_apply(v.z, mean, rstd, g.z);
            v.w = ln_apply(v.w, mean, rstd, g.w);
            *xd = v;
        }
    };

    float best[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};   // reference plugin/cuda/moe.cu:26-27; tokens warp + 8 q
    int best_e[4] = {-1, -1, -1, -1};
    uint32_t gs = 0;
    bool failed = false;

    for (int e0 = 0; e0 < E && !failed; e0 += RT_EXPERTS) {
        float acc[16][8];
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) acc[j][jj] = 0.f;

        if (tid == 0 && e0 > 0) {      // (the first pass's were issued before the statistics)
            issue(gs, 0, e0);
            if (nstages > 1) issue(gs + 1, 1, e0);
        }
        float4 g = load_gamma(0);
        bool ok = rt_mbar_wait(rt_smem_u32(&s_full[gs % RT_STAGES]), (gs / RT_STAGES) & 1, abort_flag);
        if (ok && use_ln) normalise(0, gs % RT_STAGES, g);
        g = load_gamma(1);
        if (__syncthreads_or(!ok)) { failed = true; break; }
        for (int stage = 0; stage < nstages; ++stage) {
            const uint32_t buf = (gs + stage) % RT_STAGES, next = (gs + stage + 1) % RT_STAGES;
            // the buffer of stage + 2 was read in stage - 1, which every thread left before the last barrier
            if (tid == 0 && stage + 2 < nstages) issue(gs + stage + 2, stage + 2, e0);
            const float4* xt = xs + buf * RT_TILE_CHUNKS;
            const float4* ct = cs + buf * RT_TILE_CHUNKS;
#pragma unroll
            for (int step = 0; step < RT_STEPS; ++step) {
                if (stage * RT_STAGE_FLOATS + step * 128 >= D) break;
                float4 c[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) c[jj] = ct[rt_box_idx(step, l, te + 4 * jj)];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float4 x = xt[rt_box_idx(step, l, tt + 2 * j)];
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
            ok = true;
            if (stage + 1 < nstages) {
                const uint32_t gn = gs + stage + 1;
                ok = rt_mbar_wait(rt_smem_u32(&s_full[next]), (gn / RT_STAGES) & 1, abort_flag);
                if (ok && use_ln) normalise(stage + 1, next, g);
                g = load_gamma(stage + 2);
            }
            // stage + 1 is complete for everybody; everybody is done with `stage`
            if (__syncthreads_or(!ok)) { failed = true; break; }
        }
        if (failed) break;
        gs += (uint32_t)nstages;

        // the 32 partial sums of every (token, expert) pair, through shared memory
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int jj = 0; jj < 8; ++jj)
                red[l * RT_RED_L + (tt + 2 * j) * RT_RED_PITCH + te + 4 * jj] = acc[j][jj];
        __syncthreads();
        // the butterfly (xor 16, 8, 4, 2, 1 over l) and the argmax: warp -> tokens warp + 8 q, lane -> expert e0 + lane
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int t = warp + 8 * q;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = red[i * RT_RED_L + t * RT_RED_PITCH + lane];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1)
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
    if (failed) {
        // a copy never arrived: report it, give copies in flight time to land before the shared memory goes away
        if (tid == 0 && status) atomicOr(status, STATUS_WAIT_TIMEOUT);
        const unsigned long long w0 = rt_global_ns();
        while (rt_global_ns() - w0 < 200000ull) __nanosleep(1000);
        return;
    }
    if (lane == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const long long t = t0 + warp + 8 * q;
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

namespace {
// Tensor maps of the token rows and the centroids (boxes of 32 floats x 32 rows); the last few are kept per host
// thread, because the same buffers come back call after call.
int route_maps(CUtensorMap* mx, CUtensorMap* mc, const float* X, const float* C, long long T, int D, int E) {
    struct Entry {
        const float* base = nullptr;
        long long rows = 0;
        int D = 0;
        CUtensorMap map;
    };
    static thread_local Entry cache[8];
    static thread_local int next = 0;
    auto get = [&](const float* base, long long rows, CUtensorMap* out) -> int {
        for (const Entry& e : cache)
            if (e.base == base && e.rows == rows && e.D == D) {
                *out = e.map;
                return INFMOE_OK;
            }
        Entry& e = cache[next];
        next = (next + 1) % 8;
        e.base = nullptr;
        INFMOE_TRY(make_f32_row_map(&e.map, base, D, rows, 32));
        e.base = base;
        e.rows = rows;
        e.D = D;
        *out = e.map;
        return INFMOE_OK;
    };
    INFMOE_TRY(get(X, T, mx));
    return get(C, E, mc);
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
    static const bool no_tma = [] { const char* v = getenv("INFMOE_ROUTE"); return v && !strcmp(v, "cp_async"); }();
    CUtensorMap map_x, map_c;
    if (vec && !no_tma && T < (1ll << 31) && route_maps(&map_x, &map_c, X, C, T, D, E) == INFMOE_OK) {
        INFMOE_CUDA_TRY(cudaFuncSetAttribute(route_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM + 1024));
        route_tma_kernel<<<(unsigned)grid, RT_THREADS, RT_SMEM + 1024, stream>>>(map_x, map_c, X, gamma, T, D, E, gate,
                                                                               score, status);
    } else if (vec) {
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
