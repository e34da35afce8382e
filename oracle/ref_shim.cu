// C entry points around the reference's own CUDA kernels (compiled unmodified
// from the reference checkout; see the Makefile).  TEST INFRASTRUCTURE ONLY:
// used on a GPU box to pin the CPU oracle against what the reference's kernels
// really compute, and to time the reference's kernel sequence.  All pointers
// are device pointers unless named h_*.
#include <cuda_runtime.h>
#include <cublas_v2.h>
#include <cstdint>
#include <cstdio>

#include "moe.h"   // reference: plugin/cuda/moe.h
#include "ops.h"   // reference: plugin/cuda/ops.h

extern "C" {

// layernorm_gpu<float,float>, plugin/cuda/ops/layernorm.cu:179-188 (gamma only, eps 1e-6)
int ref_layernorm(float* out, const float* in, int n1, int n2, const float* gamma) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, 0) != cudaSuccess) return 1;
    layernorm_gpu<float, float>(out, in, n1, n2, (double)1e-6, gamma, nullptr, (uint64_t)prop.maxGridSize[1], 0);
    return (int)cudaDeviceSynchronize();
}

// moe_expert_select, plugin/cuda/moe.cu:147-159
int ref_select(int token_num, int expert_num, const float* aff, int* gate, float* weight) {
    moe_expert_select(token_num, expert_num, aff, gate, weight, 0);
    return (int)cudaDeviceSynchronize();
}

// moe_expert_count, plugin/cuda/moe.cu:161-212; h_count[E] must be zeroed and
// h_offset[E+1] carry offset[E] = T, as the caller does at MoELayerPlugin.cc:350-351
int ref_count(int token_num, int expert_num, const int* gate, int* pos, int* h_count, int* h_offset) {
    moe_expert_count(token_num, expert_num, gate, pos, h_count, h_offset, 0);
    return (int)cudaDeviceSynchronize();
}

// moe_expert_scatter, plugin/cuda/moe.cu:214-228
int ref_scatter(int token_num, int token_len, const float* in, const float* coeff, int* pos, float* routed,
                float* routed_coeff) {
    moe_expert_scatter(token_num, token_len, in, coeff, pos, routed, routed_coeff, 0);
    return (int)cudaDeviceSynchronize();
}

// moe_expert_gather, plugin/cuda/moe.cu:230-240
int ref_gather(int token_num, int token_len, const float* routed, const int* pos, float* out) {
    moe_expert_gather(token_num, token_len, routed, pos, out, 0);
    return (int)cudaDeviceSynchronize();
}

// moe_expert_base_layer_fused_mix_and_gather, plugin/cuda/moe.cu:242-258
int ref_mix_gather(int token_num, int token_len, const int* pos, const float* routed, const float* post,
                   float* coeff, float* out) {
    moe_expert_base_layer_fused_mix_and_gather(token_num, token_len, pos, routed, post, coeff, out, 0);
    return (int)cudaDeviceSynchronize();
}

// fused_gelu_dot_gpu<float>, plugin/cuda/ops/gelu.cu:18-25: B = gelu(A) * B
int ref_gelu_dot(float* A, float* B, size_t len) {
    fused_gelu_dot_gpu<float>(A, B, len, 0);
    return (int)cudaDeviceSynchronize();
}

// The three cuBLAS calls + kernels of T5FFLayer::run (plugin/sublayers/T5FFLayer.cc:99-138)
// with the same arguments, on the default stream.  ws holds h[n*D] | a[n*F] | b[n*F].
int ref_t5ff_run(int n, int D, int F, const float* ln_w, const float* wi0, const float* wi1, const float* wo,
                 const float* x, float* y, float* ws) {
    static cublasHandle_t handle = nullptr;
    if (!handle && cublasCreate_v2(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, 0) != cudaSuccess) return 1;
    float* h = ws;
    float* a = ws + (size_t)n * D;
    float* b = a + (size_t)n * F;
    layernorm_gpu<float, float>(h, x, n, D, (double)1e-6, ln_w, nullptr, (uint64_t)prop.maxGridSize[1], 0);
    float alpha = 1.0f, beta = 0.0f;
    cublasSetStream_v2(handle, 0);
    if (cublasSgemm_v2(handle, CUBLAS_OP_T, CUBLAS_OP_N, F, n, D, &alpha, wi0, D, h, D, &beta, a, F)) return 2;
    if (cublasSgemm_v2(handle, CUBLAS_OP_T, CUBLAS_OP_N, F, n, D, &alpha, wi1, D, h, D, &beta, b, F)) return 2;
    fused_gelu_dot_gpu<float>(a, b, (size_t)n * F, 0);
    beta = 1.0f;
    cudaMemcpyAsync(y, x, sizeof(float) * (size_t)n * D, cudaMemcpyDeviceToDevice, 0);
    if (cublasSgemm_v2(handle, CUBLAS_OP_T, CUBLAS_OP_N, D, n, F, &alpha, wo, F, b, F, &beta, y, D)) return 2;
    return (int)cudaDeviceSynchronize();
}

// Gating scores as at plugin/MoELayerPlugin.cc:334-336.
int ref_gating_sgemm(int T, int D, int E, const float* centroids, const float* x, float* aff) {
    static cublasHandle_t handle = nullptr;
    if (!handle && cublasCreate_v2(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    float alpha = 1.0f, beta = 0.0f;
    if (cublasSgemm_v2(handle, CUBLAS_OP_T, CUBLAS_OP_N, E, T, D, &alpha, centroids, D, x, D, &beta, aff, E)) return 2;
    return (int)cudaDeviceSynchronize();
}

}  // extern "C"
