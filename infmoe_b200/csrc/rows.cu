// Row-wise kernels of the MoE layer: scatter into expert-contiguous order,
// gather / mix back to token order, LayerNorm, gelu-dot and the TF32 head/tail
// split that feeds the tensor-core GEMMs.  All of them are pure HBM streaming:
// one warp per row, 128-bit loads and stores, rows of one warp contiguous.
//
// Reference counterparts (all scalar 4-byte copies, one CTA of 256 threads per row):
//   batch_scatter_feature_and_weight_kernel  plugin/cuda/moe.cu:98-113
//   batch_gather_kernel                      plugin/cuda/moe.cu:89-96
//   fused_batch_mix_and_gather_kernel        plugin/cuda/moe.cu:115-127
//   cuApplyLayerNorm                         plugin/cuda/ops/layernorm.cu:136-174
//   gelu_dot functor via thrust::transform   plugin/cuda/ops/gelu.cu:6-25
#include "common.cuh"

namespace infmoe {

namespace {

constexpr int ROW_WARPS = 8;

__device__ __forceinline__ void copy_row(const float* __restrict__ src, float* __restrict__ dst, int D, bool vec,
                                         int lane) {
    if (vec) {
        const float4* s4 = reinterpret_cast<const float4*>(src);
        float4* d4 = reinterpret_cast<float4*>(dst);
        for (int i = lane; i < D / 4; i += 32) d4[i] = s4[i];
    } else {
        for (int i = lane; i < D; i += 32) dst[i] = src[i];
    }
}

// routed[j,:] = X[pos[j],:]; rcoeff[j] = coeff[pos[j]]
__global__ void __launch_bounds__(ROW_WARPS * 32)
scatter_kernel(long long T, int D, int vec, const float* __restrict__ X, const float* __restrict__ coeff,
               const int* __restrict__ pos, float* __restrict__ routed, float* __restrict__ rcoeff) {
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (j >= T) return;
    const int p = pos[j];
    copy_row(X + (long long)p * D, routed + j * D, D, vec != 0, lane);
    if (lane == 0 && coeff && rcoeff) rcoeff[j] = coeff[p];
}

// The layer's fused scatter: one read of X[pos[j],:] produces its per-expert
// LayerNorm h = LN(x; gamma_e) (T5FFLayer.cc:99-103) already split for the
// grouped GEMM, the routed score and, when `routed` is given, the routed row
// itself (the tensor-core GEMM reads its residual from X through pos[] and needs
// no such copy).  gamma is [E][D]; the expert of row j is gate[pos[j]].  Rows at or
// past *valid_rows (tokens without an expert, empty receive slots) are skipped.
// PACK = false: TF32 head and FP32 tail planes h_hi / h_lo [T][D] (exact split,
// CUDA-core GEMM); PACK = true: head plane h_hi and the packed BF16 plane (see
// store_pack4) in h_lo (tensor-core GEMM).
template <bool PACK>
__global__ void __launch_bounds__(ROW_WARPS * 32)
scatter_ln_split_kernel(long long T, int D, int vec, const float* __restrict__ X, const float* __restrict__ score,
                        const int* __restrict__ pos, const int* __restrict__ gate,
                        const float* __restrict__ gamma_all, const int* __restrict__ valid_rows,
                        float* __restrict__ routed, float* __restrict__ rscore, float* __restrict__ h_hi,
                        float* __restrict__ h_lo) {
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (j >= T || (valid_rows && j >= *valid_rows)) return;
    const int p = pos[j];
    const int e = gate[p];
    const float* src = X + (long long)p * D;
    const float* gamma = gamma_all + (long long)e * D;
    float mean, rstd;
    warp_row_stats(src, D, vec != 0, mean, rstd);
    uint16_t* pack_row = PACK ? reinterpret_cast<uint16_t*>(h_lo) + j * (long long)pack_pitch(D) : nullptr;
    const int k_end = PACK ? ((D + 31) & ~31) : D;   // the packed plane is zero padded to whole groups
    for (int base = 4 * lane; base < k_end; base += 128) {
        float hh[4] = {0.f, 0.f, 0.f, 0.f}, ll[4] = {0.f, 0.f, 0.f, 0.f};
        if (base < D) {
            const float4 v = load_row4(src, base, D, vec != 0);
            const float4 g = load_row4(gamma, base, D, vec != 0);
            const float vv[4] = {v.x, v.y, v.z, v.w}, gg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (base + k < D) split_tf32(ln_apply(vv[k], mean, rstd, gg[k]), hh[k], ll[k]);
            const long long o = j * D + base;
            if (vec) {
                if (routed) *reinterpret_cast<float4*>(routed + o) = v;
                *reinterpret_cast<float4*>(h_hi + o) = make_float4(hh[0], hh[1], hh[2], hh[3]);
                if (!PACK) *reinterpret_cast<float4*>(h_lo + o) = make_float4(ll[0], ll[1], ll[2], ll[3]);
            } else {
                for (int k = 0; k < 4 && base + k < D; ++k) {
                    if (routed) routed[o + k] = vv[k];
                    h_hi[o + k] = hh[k];
                    if (!PACK) h_lo[o + k] = ll[k];
                }
            }
        }
        if (PACK) store_pack4(pack_row, base, hh, ll);
    }
    if (lane == 0 && rscore && score) rscore[j] = score[p];
}

// The same for aligned rows of up to 128 * NV floats, with more bytes in flight per warp: the whole row is
// fetched into registers by back-to-back 128-bit loads (NV per lane) before any of it is used, so it crosses HBM
// once in one burst and both statistics passes and the split run from registers.  The additions happen in the
// order of warp_row_stats, so the results are the same bits.  Few rows per SM (4096 rows on 148 SMs) would
// otherwise leave the memory system half idle.  The expert's LayerNorm weights are fetched into shared memory by
// cp.async while the row is on its way, so the output loop never waits for L2.
template <bool PACK, int NV>
__global__ void __launch_bounds__(128)
scatter_ln_split_reg_kernel(long long T, int D, const float* __restrict__ X, const float* __restrict__ score,
                            const int* __restrict__ pos, const int* __restrict__ gate,
                            const float* __restrict__ gamma_all, const int* __restrict__ valid_rows,
                            float* __restrict__ routed, float* __restrict__ rscore, float* __restrict__ h_hi,
                            float* __restrict__ h_lo) {
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (j >= T || (valid_rows && j >= *valid_rows)) return;
    extern __shared__ __align__(16) float4 s_gamma_all[];     // [4 warps][NV * 32]
    float4* s_gamma = s_gamma_all + (threadIdx.x >> 5) * (NV * 32);
    const int p = pos[j];
    const int e = gate[p];
    const float4* src = reinterpret_cast<const float4*>(X + (long long)p * D);
    const float4* gamma = reinterpret_cast<const float4*>(gamma_all + (long long)e * D);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int base = 4 * lane + 128 * i;
        v[i] = base < D ? src[base >> 2] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int base = 4 * lane + 128 * i;
        if (base < D) {
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(s_gamma + (base >> 2));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gamma + (base >> 2)) : "memory");
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (4 * lane + 128 * i < D) s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, v[i].x), v[i].y), v[i].z), v[i].w);
    const float mean = __fdiv_rn(warp_xor_sum(s), (float)D);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (4 * lane + 128 * i < D) {
            float d = __fsub_rn(v[i].x, mean);
            q = __fmaf_rn(d, d, q);
            d = __fsub_rn(v[i].y, mean);
            q = __fmaf_rn(d, d, q);
            d = __fsub_rn(v[i].z, mean);
            q = __fmaf_rn(d, d, q);
            d = __fsub_rn(v[i].w, mean);
            q = __fmaf_rn(d, d, q);
        }
    const float var = __fdiv_rn(warp_xor_sum(q), (float)D);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, 1e-6f)));
    uint16_t* pack_row = PACK ? reinterpret_cast<uint16_t*>(h_lo) + j * (long long)pack_pitch(D) : nullptr;
    const int k_end = PACK ? ((D + 31) & ~31) : D;
    asm volatile("cp.async.wait_group 0;" ::: "memory");   // every lane reads back only what it fetched itself
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int base = 4 * lane + 128 * i;
        if (base >= k_end) continue;
        float hh[4] = {0.f, 0.f, 0.f, 0.f}, ll[4] = {0.f, 0.f, 0.f, 0.f};
        if (base < D) {
            const float4 g = s_gamma[base >> 2];
            split_tf32(ln_apply(v[i].x, mean, rstd, g.x), hh[0], ll[0]);
            split_tf32(ln_apply(v[i].y, mean, rstd, g.y), hh[1], ll[1]);
            split_tf32(ln_apply(v[i].z, mean, rstd, g.z), hh[2], ll[2]);
            split_tf32(ln_apply(v[i].w, mean, rstd, g.w), hh[3], ll[3]);
            const long long o = j * D + base;
            if (routed) *reinterpret_cast<float4*>(routed + o) = v[i];
            *reinterpret_cast<float4*>(h_hi + o) = make_float4(hh[0], hh[1], hh[2], hh[3]);
            if (!PACK) *reinterpret_cast<float4*>(h_lo + o) = make_float4(ll[0], ll[1], ll[2], ll[3]);
        }
        if (PACK) store_pack4(pack_row, base, hh, ll);
    }
    if (lane == 0 && rscore && score) rscore[j] = score[p];
}

// out[pos[j],:] = in[j,:] for the rows below *valid_rows (all rows when valid_rows is NULL)
__global__ void __launch_bounds__(ROW_WARPS * 32)
gather_kernel(long long T, int D, int vec, const float* __restrict__ in, const int* __restrict__ pos,
              const int* __restrict__ valid_rows, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (j >= T || (valid_rows && j >= *valid_rows)) return;
    copy_row(in + j * D, out + (long long)pos[j] * D, D, vec != 0, lane);
}

// alpha = 1 / (1 + exp(-coeff[j])); out[pos[j],:] = alpha * post[j,:] + (1 - alpha) * routed[j,:]
// (sigmoid: plugin/cuda/common.cuh:24-27)
__global__ void __launch_bounds__(ROW_WARPS * 32)
mix_gather_kernel(long long T, int D, int vec, const int* __restrict__ pos, const float* __restrict__ routed,
                  const float* __restrict__ post, const float* __restrict__ coeff,
                  const int* __restrict__ valid_rows, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (j >= T || (valid_rows && j >= *valid_rows)) return;
    const float alpha = mix_alpha(coeff[j]);
    const float beta = 1.0f - alpha;
    const float* a = post + j * D;
    const float* b = routed + j * D;
    float* o = out + (long long)pos[j] * D;
    if (vec) {
        for (int i = lane; i < D / 4; i += 32) {
            const float4 x = reinterpret_cast<const float4*>(a)[i];
            const float4 y = reinterpret_cast<const float4*>(b)[i];
            float4 r;
            r.x = mix_value(alpha, beta, x.x, y.x);
            r.y = mix_value(alpha, beta, x.y, y.y);
            r.z = mix_value(alpha, beta, x.z, y.z);
            r.w = mix_value(alpha, beta, x.w, y.w);
            reinterpret_cast<float4*>(o)[i] = r;
        }
    } else {
        for (int i = lane; i < D; i += 32) o[i] = mix_value(alpha, beta, a[i], b[i]);
    }
}

__global__ void __launch_bounds__(ROW_WARPS * 32)
layernorm_kernel(long long n, int D, int vec, const float* __restrict__ in, const float* __restrict__ gamma,
                 float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (j >= n) return;
    const float* src = in + j * D;
    float mean, rstd;
    warp_row_stats(src, D, vec != 0, mean, rstd);
    for (int base = 4 * lane; base < D; base += 128) {
        const float4 v = load_row4(src, base, D, vec != 0);
        const float4 g = load_row4(gamma, base, D, vec != 0);
        const float r[4] = {ln_apply(v.x, mean, rstd, g.x), ln_apply(v.y, mean, rstd, g.y),
                            ln_apply(v.z, mean, rstd, g.z), ln_apply(v.w, mean, rstd, g.w)};
        if (vec) {
            *reinterpret_cast<float4*>(out + j * D + base) = make_float4(r[0], r[1], r[2], r[3]);
        } else {
            for (int k = 0; k < 4 && base + k < D; ++k) out[j * D + base + k] = r[k];
        }
    }
}

// h = LN(x; gamma) split for the grouped GEMM (rows already in place); planes as in scatter_ln_split_kernel.
template <bool PACK>
__global__ void __launch_bounds__(ROW_WARPS * 32)
ln_split_kernel(long long n, int D, int vec, const float* __restrict__ in, const float* __restrict__ gamma,
                float* __restrict__ h_hi, float* __restrict__ h_lo) {
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (j >= n) return;
    const float* src = in + j * D;
    float mean, rstd;
    warp_row_stats(src, D, vec != 0, mean, rstd);
    uint16_t* pack_row = PACK ? reinterpret_cast<uint16_t*>(h_lo) + j * (long long)pack_pitch(D) : nullptr;
    const int k_end = PACK ? ((D + 31) & ~31) : D;
    for (int base = 4 * lane; base < k_end; base += 128) {
        float hh[4] = {0.f, 0.f, 0.f, 0.f}, ll[4] = {0.f, 0.f, 0.f, 0.f};
        if (base < D) {
            const float4 v = load_row4(src, base, D, vec != 0);
            const float4 g = load_row4(gamma, base, D, vec != 0);
            const float vv[4] = {v.x, v.y, v.z, v.w}, gg[4] = {g.x, g.y, g.z, g.w};
            for (int k = 0; k < 4 && base + k < D; ++k) {
                split_tf32(ln_apply(vv[k], mean, rstd, gg[k]), hh[k], ll[k]);
                h_hi[j * D + base + k] = hh[k];
                if (!PACK) h_lo[j * D + base + k] = ll[k];
            }
        }
        if (PACK) store_pack4(pack_row, base, hh, ll);
    }
}

__global__ void gelu_dot_kernel(const float* __restrict__ a, float* __restrict__ b, size_t len) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) b[i] = gelu_dot(a[i], b[i]);
}

// hi/lo planes of a raw FP32 array (weights at load time).
__global__ void split_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo,
                             size_t len4, size_t len) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len4; i += stride) {
        const float4 v = reinterpret_cast<const float4*>(src)[i];
        float4 h, l;
        split_tf32(v.x, h.x, l.x);
        split_tf32(v.y, h.y, l.y);
        split_tf32(v.z, h.z, l.z);
        split_tf32(v.w, h.w, l.w);
        reinterpret_cast<float4*>(hi)[i] = h;
        reinterpret_cast<float4*>(lo)[i] = l;
    }
    for (size_t i = len4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride)
        split_tf32(src[i], hi[i], lo[i]);
}

// Weight matrix -> tile-contiguous layout for the tensor-core GEMM: tiles of 128 rows x 32 floats (16 KB),
// tile (mb, kb) at ((mb * KB + kb) * 128 rows; rows and columns past the matrix are zero.  With two sources
// the rows are interleaved: row 2f = src0[f], row 2f+1 = src1[f] (wi_0 / wi_1).  One warp moves one 128-byte
// row segment, so both the read and the write are coalesced.
__global__ void __launch_bounds__(256)
retile_kernel(const float* __restrict__ src0, const float* __restrict__ src1, int M, int K, int MB, int KB,
              float* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const long long seg = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);   // (mb, kb, r) flattened
    const long long total = (long long)MB * KB * 128;
    if (seg >= total) return;
    const int r = (int)(seg % 128);
    const long long tile = seg / 128;
    const int kb = (int)(tile % KB), mb = (int)(tile / KB);
    const int m = mb * 128 + r, k = kb * 32 + lane;
    float v = 0.f;
    if (m < M && k < K) {
        if (src1) v = (m & 1) ? src1[(size_t)(m >> 1) * K + k] : src0[(size_t)(m >> 1) * K + k];
        else v = src0[(size_t)m * K + k];
    }
    dst[seg * 32 + lane] = v;
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
inline unsigned row_grid(long long rows) { return (unsigned)((rows + ROW_WARPS - 1) / ROW_WARPS); }

}  // namespace

int launch_scatter(long long T, int D, const float* X, const float* coeff, const int* pos, float* routed,
                   float* rcoeff, cudaStream_t stream) {
    if (T < 0 || D <= 0 || !X || !pos || !routed) {
        set_error("expert_scatter: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (T == 0) return INFMOE_OK;
    const int vec = (D % 4 == 0) && aligned16(X) && aligned16(routed);
    scatter_kernel<<<row_grid(T), ROW_WARPS * 32, 0, stream>>>(T, D, vec, X, coeff, pos, routed, rcoeff);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_scatter_ln_split(long long T, int D, const float* X, const float* score, const int* pos, const int* gate,
                            const float* gamma_all, const int* valid_rows, float* routed, float* rscore, float* h_hi,
                            float* h_lo, bool pack, cudaStream_t stream) {
    if (T == 0) return INFMOE_OK;
    const int vec = (D % 4 == 0) && aligned16(X) && aligned16(routed) && aligned16(h_hi) && aligned16(h_lo) &&
                    aligned16(gamma_all);
    if (vec && D <= 4096) {
        const unsigned grid = (unsigned)((T + 3) / 4);
#define INFMOE_SCATTER_REG(PACK, NV)                                                                               \
    do {                                                                                                           \
        auto kern = scatter_ln_split_reg_kernel<PACK, NV>;                                                         \
        constexpr int smem = 4 * NV * 32 * 16;                                                                     \
        if (smem > 48 * 1024)                                                                                      \
            INFMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));        \
        kern<<<grid, 128, smem, stream>>>(T, D, X, score, pos, gate, gamma_all, valid_rows, routed, rscore, h_hi,  \
                                          h_lo);                                                                   \
    } while (0)
        if (pack) {
            if (D <= 1024) INFMOE_SCATTER_REG(true, 8);
            else if (D <= 2048) INFMOE_SCATTER_REG(true, 16);
            else INFMOE_SCATTER_REG(true, 32);
        } else {
            if (D <= 1024) INFMOE_SCATTER_REG(false, 8);
            else if (D <= 2048) INFMOE_SCATTER_REG(false, 16);
            else INFMOE_SCATTER_REG(false, 32);
        }
#undef INFMOE_SCATTER_REG
    } else if (pack)
        scatter_ln_split_kernel<true><<<row_grid(T), ROW_WARPS * 32, 0, stream>>>(
            T, D, vec, X, score, pos, gate, gamma_all, valid_rows, routed, rscore, h_hi, h_lo);
    else
        scatter_ln_split_kernel<false><<<row_grid(T), ROW_WARPS * 32, 0, stream>>>(
            T, D, vec, X, score, pos, gate, gamma_all, valid_rows, routed, rscore, h_hi, h_lo);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

namespace {
// in[i,:] -> the row at address dst[i]
__global__ void __launch_bounds__(ROW_WARPS * 32)
rows_to_ptrs_kernel(long long n, int D, int vec, const float* __restrict__ in, const unsigned long long* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const long long j = (long long)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (j >= n) return;
    const float* a = in + j * D;
    float* o = reinterpret_cast<float*>(dst[j]);
    if (vec && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
        for (int i = lane; i < D / 4; i += 32) reinterpret_cast<float4*>(o)[i] = reinterpret_cast<const float4*>(a)[i];
    } else {
        for (int i = lane; i < D; i += 32) o[i] = a[i];
    }
}
}  // namespace

int launch_rows_to_ptrs(long long n, int D, const float* in, const unsigned long long* dst, cudaStream_t stream) {
    if (n < 0 || D <= 0 || !in || !dst) {
        set_error("rows_to_ptrs: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (n == 0) return INFMOE_OK;
    const int vec = (D % 4 == 0) && aligned16(in);
    rows_to_ptrs_kernel<<<row_grid(n), ROW_WARPS * 32, 0, stream>>>(n, D, vec, in, dst);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_gather(long long T, int D, const float* in, const int* pos, float* out, cudaStream_t stream,
                  const int* valid_rows) {
    if (T < 0 || D <= 0 || !in || !pos || !out) {
        set_error("expert_gather: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (T == 0) return INFMOE_OK;
    const int vec = (D % 4 == 0) && aligned16(in) && aligned16(out);
    gather_kernel<<<row_grid(T), ROW_WARPS * 32, 0, stream>>>(T, D, vec, in, pos, valid_rows, out);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_mix_gather(long long T, int D, const int* pos, const float* routed, const float* post,
                      const float* coeff, float* out, cudaStream_t stream, const int* valid_rows) {
    if (T < 0 || D <= 0 || !pos || !routed || !post || !coeff || !out) {
        set_error("expert_mix_gather: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (T == 0) return INFMOE_OK;
    const int vec = (D % 4 == 0) && aligned16(routed) && aligned16(post) && aligned16(out);
    mix_gather_kernel<<<row_grid(T), ROW_WARPS * 32, 0, stream>>>(T, D, vec, pos, routed, post, coeff, valid_rows,
                                                                  out);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_layernorm(float* out, const float* in, long long n, int D, const float* gamma, cudaStream_t stream) {
    if (n < 0 || D <= 0 || !out || !in || !gamma) {
        set_error("layernorm: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (n == 0) return INFMOE_OK;
    const int vec = (D % 4 == 0) && aligned16(in) && aligned16(out) && aligned16(gamma);
    layernorm_kernel<<<row_grid(n), ROW_WARPS * 32, 0, stream>>>(n, D, vec, in, gamma, out);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_ln_split(long long n, int D, const float* in, const float* gamma, float* h_hi, float* h_lo, bool pack,
                    cudaStream_t stream) {
    if (n == 0) return INFMOE_OK;
    const int vec = (D % 4 == 0) && aligned16(in) && aligned16(gamma);
    if (pack)
        ln_split_kernel<true><<<row_grid(n), ROW_WARPS * 32, 0, stream>>>(n, D, vec, in, gamma, h_hi, h_lo);
    else
        ln_split_kernel<false><<<row_grid(n), ROW_WARPS * 32, 0, stream>>>(n, D, vec, in, gamma, h_hi, h_lo);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_retile(const float* src0, const float* src1, int M, int K, float* dst, cudaStream_t stream) {
    const int MB = (M + 127) / 128, KB = (K + 31) / 32;
    const long long segs = (long long)MB * KB * 128;
    retile_kernel<<<(unsigned)((segs + 7) / 8), 256, 0, stream>>>(src0, src1, M, K, MB, KB, dst);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_gelu_dot(const float* a, float* b, size_t len, cudaStream_t stream) {
    if (!a || !b) {
        set_error("gelu_dot: bad argument");
        return INFMOE_ERR_INVALID_ARGUMENT;
    }
    if (len == 0) return INFMOE_OK;
    const unsigned grid = (unsigned)((len + 255) / 256 < 148 * 16 ? (len + 255) / 256 : 148 * 16);
    gelu_dot_kernel<<<grid, 256, 0, stream>>>(a, b, len);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

namespace {
__global__ void fill_int_kernel(int* dst, int value) { *dst = value; }
}  // namespace

int launch_fill_int(int* dst, int value, cudaStream_t stream) {
    fill_int_kernel<<<1, 1, 0, stream>>>(dst, value);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

int launch_split(const float* src, float* hi, float* lo, size_t len, cudaStream_t stream) {
    if (len == 0) return INFMOE_OK;
    const bool vec = aligned16(src) && aligned16(hi) && aligned16(lo);
    const size_t len4 = vec ? len / 4 : 0;
    const size_t work = len4 ? len4 : len;
    const unsigned grid = (unsigned)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
    split_kernel<<<grid, 256, 0, stream>>>(src, hi, lo, len4, len);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

}  // namespace infmoe
