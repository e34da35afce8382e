// Shared host/device helpers of the B200 MoE-layer kernels.
#pragma once

#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>
#include <cstdio>

#include "infmoe_c.h"

namespace infmoe {

// ---------------------------------------------------------------------------
// Error plumbing: nothing in this library exits the process (the reference's
// CUDA_SAFE_CALL does, plugin/utility.h:15-21); every failure becomes a status.
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

#define INFMOE_CUDA_TRY(call)                                                                              \
    do {                                                                                                   \
        cudaError_t err__ = (call);                                                                        \
        if (err__ != cudaSuccess) {                                                                        \
            ::infmoe::set_error("CUDA error %d (%s) at %s:%d", (int)err__, cudaGetErrorString(err__),      \
                                __FILE__, __LINE__);                                                       \
            return INFMOE_ERR_CUDA;                                                                        \
        }                                                                                                  \
    } while (0)

#define INFMOE_TRY(call)                \
    do {                                \
        int rc__ = (call);              \
        if (rc__ != INFMOE_OK) return rc__; \
    } while (0)

// Bits of the device-side status word.
enum : int32_t {
    STATUS_NO_EXPERT = 1,      // a token selected no expert (NaN scores)
    STATUS_BAD_GATE = 2,       // gate index outside [0, E)
    STATUS_WAIT_TIMEOUT = 4,   // a bounded mbarrier wait ran out inside a GEMM kernel
    STATUS_BAD_SHAPE = 8,
};

// Process-wide count of kernels launched by this library.
extern long long g_kernel_launches;
inline void note_launch(int n = 1) { g_kernel_launches += n; }

#ifdef __CUDACC__
// ---------------------------------------------------------------------------
// Canonical FP32 reductions.  Routing must agree bit for bit with the CPU
// checker, so the summation order is fixed: lane l of a warp owns elements
// k = 4*(l + 32*i) + c (i ascending, c = 0..3), accumulates them in that order
// with explicit round-to-nearest adds / fused multiply-adds, and the 32 lane
// partials are combined by a butterfly (xor 16, 8, 4, 2, 1).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_xor_sum(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// Loads elements [base, base+4) of a row; `vec` says the row is 16-byte aligned
// with D % 4 == 0.  Elements at or beyond D read as 0 and must be skipped by the caller.
__device__ __forceinline__ float4 load_row4(const float* __restrict__ row, int base, int D, bool vec) {
    if (vec) return *reinterpret_cast<const float4*>(row + base);
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (base + 0 < D) r.x = row[base + 0];
    if (base + 1 < D) r.y = row[base + 1];
    if (base + 2 < D) r.z = row[base + 2];
    if (base + 3 < D) r.w = row[base + 3];
    return r;
}

// LayerNorm statistics of one row held by a full warp (true LayerNorm: mean
// subtracted, biased variance, eps 1e-6; reference plugin/cuda/ops/layernorm.cu:126-149).
__device__ __forceinline__ void warp_row_stats(const float* __restrict__ row, int D, bool vec, float& mean,
                                               float& rstd) {
    const int lane = threadIdx.x & 31;
    // Same additions in the same order either way; the vector form (D a multiple of 4, aligned rows) has no
    // per-element bounds checks and keeps eight loads in flight.
    float s = 0.f;
    if (vec) {
#pragma unroll 8
        for (int base = 4 * lane; base < D; base += 128) {
            const float4 v = *reinterpret_cast<const float4*>(row + base);
            s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, v.x), v.y), v.z), v.w);
        }
    } else {
        for (int base = 4 * lane; base < D; base += 128) {
            const float4 v = load_row4(row, base, D, false);
            s = __fadd_rn(s, v.x);
            if (base + 1 < D) s = __fadd_rn(s, v.y);
            if (base + 2 < D) s = __fadd_rn(s, v.z);
            if (base + 3 < D) s = __fadd_rn(s, v.w);
        }
    }
    mean = __fdiv_rn(warp_xor_sum(s), (float)D);
    float q = 0.f;
    if (vec) {
#pragma unroll 8
        for (int base = 4 * lane; base < D; base += 128) {
            const float4 v = *reinterpret_cast<const float4*>(row + base);
            float d = __fsub_rn(v.x, mean);
            q = __fmaf_rn(d, d, q);
            d = __fsub_rn(v.y, mean);
            q = __fmaf_rn(d, d, q);
            d = __fsub_rn(v.z, mean);
            q = __fmaf_rn(d, d, q);
            d = __fsub_rn(v.w, mean);
            q = __fmaf_rn(d, d, q);
        }
    } else {
        for (int base = 4 * lane; base < D; base += 128) {
            const float4 v = load_row4(row, base, D, false);
            float d = __fsub_rn(v.x, mean);
            q = __fmaf_rn(d, d, q);
            if (base + 1 < D) { d = __fsub_rn(v.y, mean); q = __fmaf_rn(d, d, q); }
            if (base + 2 < D) { d = __fsub_rn(v.z, mean); q = __fmaf_rn(d, d, q); }
            if (base + 3 < D) { d = __fsub_rn(v.w, mean); q = __fmaf_rn(d, d, q); }
        }
    }
    const float var = __fdiv_rn(warp_xor_sum(q), (float)D);
    rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, 1e-6f)));
}

// gamma * ((x - mean) * rstd), reference plugin/cuda/ops/layernorm.cu:158-161.
__device__ __forceinline__ float ln_apply(float x, float mean, float rstd, float gamma) {
    return __fmul_rn(gamma, __fmul_rn(__fsub_rn(x, mean), rstd));
}

// Splits an FP32 value into a TF32-representable head and an FP32 remainder:
// hi = x rounded to 10 mantissa bits (round to nearest, ties away), lo = x - hi (exact).
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    lo = __fsub_rn(x, hi);
}

// Two FP32 values rounded to BF16 (round to nearest even) in one 32-bit word: `even` in the lower half.
__device__ __forceinline__ uint32_t pack_bf16x2(float even, float odd) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(odd), "f"(even));
    return r;
}

// Token operand of the tensor-core GEMM, per value x: hi = x rounded to TF32 (FP32 plane `hi`), and the BF16
// roundings of hi and of lo = x - hi in a packed plane.  The packed plane has one 128-byte group per 32 values
// of a row: 32 x bf16(hi) followed by 32 x bf16(lo); rows are padded with zeros to a multiple of 32 values.
__host__ __device__ __forceinline__ size_t pack_pitch(int K) { return (size_t)((K + 31) / 32) * 64; }   // in BF16 elements
// Stores the packed entries of four consecutive values k0..k0+3 (k0 a multiple of 4) of one row.
__device__ __forceinline__ void store_pack4(uint16_t* __restrict__ pack_row, int k0, const float hi[4], const float lo[4]) {
    uint16_t* g = pack_row + (size_t)(k0 >> 5) * 64 + (k0 & 31);
    *reinterpret_cast<uint2*>(g) = make_uint2(pack_bf16x2(hi[0], hi[1]), pack_bf16x2(hi[2], hi[3]));
    *reinterpret_cast<uint2*>(g + 32) = make_uint2(pack_bf16x2(lo[0], lo[1]), pack_bf16x2(lo[2], lo[3]));
}

// base_layer output mix (plugin/cuda/moe.cu:115-127, sigmoid plugin/cuda/common.cuh:24-27):
// out = alpha * expert_output + (1 - alpha) * input with alpha = sigmoid(score).  One fixed rounding sequence, so
// that the stand-alone combine kernel and the GEMM epilogue that fuses it give the same bits.
__device__ __forceinline__ float mix_alpha(float score) { return 1.0f / (1.0f + expf(-score)); }
__device__ __forceinline__ float mix_value(float alpha, float beta, float post, float routed) {
    return __fmaf_rn(alpha, post, __fmul_rn(beta, routed));
}

// gelu(a) * b in the reference's evaluation order (plugin/cuda/ops/gelu.cu:8-15).
__device__ __forceinline__ float gelu_dot(float a, float b) {
    const float cdf = 0.5f * (1.0f + tanhf(a * (0.035677408136300125f * a * a + 0.7978845608028654f)));
    return a * cdf * b;
}
// The same function with 0.5 (1 + tanh(u)) written as the logistic 1 / (1 + exp(-2u)): a handful of instructions
// instead of tanhf's few dozen, for the tensor-core path, whose results are held to a tolerance rather than to the
// reference's bits.  ex2.approx and the approximate division are each good to 2 ulp; for u so negative that
// exp(-2u) overflows the quotient is 0, which is the limit.
__device__ __forceinline__ float gelu_dot_fast(float a, float b) {
    const float u = a * (0.035677408136300125f * a * a + 0.7978845608028654f);
    const float cdf = __fdividef(1.0f, 1.0f + __expf(-2.0f * u));
    return a * cdf * b;
}
#endif  // __CUDACC__

}  // namespace infmoe
