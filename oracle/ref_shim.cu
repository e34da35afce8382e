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


// ---------------------------------------------------------------------------------------------
// The reference's kernel sequence for one whole layer call, as MoELayerPlugin::enqueue issues it
// (plugin/MoELayerPlugin.cc:279-416), used only to time "the reference's kernels + cuBLAS on this
// box".  The TensorRT plugin itself cannot be built here, so the order of launches, copies and
// host synchronisations is restated around the reference's own functions: layer norm (:324),
// gating SGEMM + sync (:334-337), select, count, scatter (each synchronises inside moe.cu), then per
// non-empty expert four weight copies into slot (j+1) % mc while expert j runs on slot j % mc
// (:360-394), a sync of all slot streams (:399-401) and the final gather / mix (:407-412).
// Expert weights are taken from the four pointer tables (pinned host memory for the literal
// behaviour).  ws must hold mc * (4D + 12DF + 4T(D + 2F)) + 4(TE + 2T + 2TD) + 8T bytes (:253-273).
// flags: bit 0 = layer norm before scoring (cpm_2), bit 1 = base_layer mix,
//        bit 2 = gather the expert output (the literal reference gathers the scattered input, :411).
// ---------------------------------------------------------------------------------------------
int ref_layer_call(int T, int D, int E, int F, int mc, int flags, const float* x, const float* centroids,
                   const float* gating_ln, const float* const* ln_w, const float* const* wi0,
                   const float* const* wi1, const float* const* wo, int copy_kind, char* ws, float* out) {
    static cublasHandle_t handle = nullptr;
    static cudaStream_t streams[16] = {};
    if (mc < 1 || mc > 16) return 3;
    if (!handle && cublasCreate_v2(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    for (int i = 0; i < mc; ++i)
        if (!streams[i] && cudaStreamCreate(&streams[i]) != cudaSuccess) return 1;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, 0) != cudaSuccess) return 1;
    const uint64_t max_grid_y = (uint64_t)prop.maxGridSize[1];
    cudaStream_t stream = 0;
    const size_t weight_bytes = sizeof(float) * ((size_t)D + 3 * (size_t)D * F);
    const size_t slot_bytes = weight_bytes + sizeof(float) * (size_t)T * ((size_t)D + 2 * (size_t)F);
    float* moe = (float*)(ws + slot_bytes * mc);
    float* aff = moe;
    int* gate = (int*)(moe + (size_t)T * E);
    int* pos = gate + T;
    float* routed = (float*)(pos + T);
    float* post = routed + (size_t)T * D;
    float* coeff = post + (size_t)T * D;
    float* rcoeff = coeff + T;

    const float* aff_in = x;
    if (flags & 1) {
        layernorm_gpu<float, float>(routed, x, T, D, (double)1e-6, gating_ln, nullptr, max_grid_y, stream);
        aff_in = routed;
    }
    float alpha = 1.0f, beta = 0.0f;
    cublasSetStream_v2(handle, stream);
    if (cublasSgemm_v2(handle, CUBLAS_OP_T, CUBLAS_OP_N, E, T, D, &alpha, centroids, D, aff_in, D, &beta, aff, E)) return 2;
    cudaStreamSynchronize(stream);
    moe_expert_select(T, E, aff, gate, coeff, stream);
    int* h_offset = new int[E + 1]();
    int* h_count = new int[E]();
    h_offset[E] = T;
    moe_expert_count(T, E, gate, pos, h_count, h_offset, stream);
    moe_expert_scatter(T, D, x, coeff, pos, routed, rcoeff, stream);

    auto copy_weights = [&](char* slot, int e, cudaStream_t s) {
        const cudaMemcpyKind kind = copy_kind ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
        float* dst = (float*)slot;
        cudaMemcpyAsync(dst, ln_w[e], sizeof(float) * D, kind, s);
        cudaMemcpyAsync(dst + D, wi0[e], sizeof(float) * (size_t)D * F, kind, s);
        cudaMemcpyAsync(dst + D + (size_t)D * F, wi1[e], sizeof(float) * (size_t)D * F, kind, s);
        cudaMemcpyAsync(dst + D + 2 * (size_t)D * F, wo[e], sizeof(float) * (size_t)D * F, kind, s);
    };
    int next = 0;
    while (next < E && h_count[next] == 0) ++next;
    if (next < E) copy_weights(ws, next, streams[0]);
    cudaStreamSynchronize(stream);
    for (int e = next, j = 0; e < E; e = next, ++j) {
        const int cur = j % mc, nxt = (j + 1) % mc;
        cudaStreamSynchronize(streams[nxt]);
        next = e + 1;
        while (next < E && h_count[next] == 0) ++next;
        if (next < E) copy_weights(ws + slot_bytes * nxt, next, streams[nxt]);
        // T5FFLayer::run on this expert's rows (plugin/sublayers/T5FFLayer.cc:90-141)
        cudaStream_t s = streams[cur];
        cublasSetStream_v2(handle, s);
        const int n = h_count[e];
        const float* w = (const float*)(ws + slot_bytes * cur);
        float* scratch = (float*)(ws + slot_bytes * cur + weight_bytes);
        float* h = scratch;
        float* a = h + (size_t)n * D;
        float* b = a + (size_t)n * F;
        const float* xin = routed + (size_t)h_offset[e] * D;
        float* y = post + (size_t)h_offset[e] * D;
        layernorm_gpu<float, float>(h, xin, n, D, (double)1e-6, w, nullptr, max_grid_y, s);
        beta = 0.0f;
        cublasSgemm_v2(handle, CUBLAS_OP_T, CUBLAS_OP_N, F, n, D, &alpha, w + D, D, h, D, &beta, a, F);
        cublasSgemm_v2(handle, CUBLAS_OP_T, CUBLAS_OP_N, F, n, D, &alpha, w + D + (size_t)D * F, D, h, D, &beta, b, F);
        fused_gelu_dot_gpu<float>(a, b, (size_t)n * F, s);
        beta = 1.0f;
        cudaMemcpyAsync(y, xin, sizeof(float) * (size_t)n * D, cudaMemcpyDeviceToDevice, s);
        cublasSgemm_v2(handle, CUBLAS_OP_T, CUBLAS_OP_N, D, n, F, &alpha, w + D + 2 * (size_t)D * F, F, b, F, &beta, y, D);
    }
    delete[] h_offset;
    delete[] h_count;
    for (int i = 0; i < mc; ++i) cudaStreamSynchronize(streams[i]);
    cublasSetStream_v2(handle, stream);
    if (flags & 2)
        moe_expert_base_layer_fused_mix_and_gather(T, D, pos, routed, post, rcoeff, out, stream);
    else
        moe_expert_gather(T, D, (flags & 4) ? post : routed, pos, out, stream);
    return (int)cudaDeviceSynchronize();
}

}  // extern "C"
