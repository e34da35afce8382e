// Exact-FP32 grouped expert FFN on CUDA cores.  This is the path for shapes the
// tensor-core kernels cannot take (row strides that are not multiples of 16
// bytes, i.e. d_model or d_ff not divisible by 4) and the cross-check used while
// validating the tcgen05 kernels on the device.  It is not a fallback for a
// missing GPU: it runs on the same device from the same buffers.
//
// Math (T5FFLayer::run, plugin/sublayers/T5FFLayer.cc:112-138), per expert e on
// its rows [offset[e], offset[e+1]):
//   g = gelu(h wi_0^T) * (h wi_1^T)        h = h_hi + h_lo (exact recombination)
//   y = x + g wo^T
// Activations are stored as TF32 head/tail planes; head + tail is the original
// FP32 value exactly, so these kernels compute with full FP32 inputs.  Weights are
// raw FP32 in the tile-contiguous layout of the tensor-core path; wi_0 and wi_1 share
// one matrix with interleaved rows (row 2f = wi_0[f], row 2f+1 = wi_1[f]).
#include "common.cuh"

namespace infmoe {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

// Finds the (expert, first row, valid rows) of row-tile `tile` when every expert's
// rows are tiled separately by TM.  Returns false when `tile` is past the end.
__device__ bool locate_tile(const int* __restrict__ offset, int e_begin, int e_end, int tile, int& expert,
                            int& row0, int& rows) {
    int seen = 0;
    for (int e = e_begin; e < e_end; ++e) {
        const int beg = offset[e], cnt = offset[e + 1] - beg;
        const int nt = (cnt + TM - 1) / TM;
        if (tile < seen + nt) {
            expert = e;
            row0 = beg + (tile - seen) * TM;
            rows = min(TM, beg + cnt - row0);
            return true;
        }
        seen += nt;
    }
    return false;
}

// DUAL = true : out_hi/out_lo[j][n] = split(gelu(A W0^T) * (A W1^T))   (N = d_ff, K = d_model)
// DUAL = false: out_hi[j][n] = resid[j][n] + A W0^T                      (N = d_model, K = d_ff)
template <bool DUAL>
__global__ void __launch_bounds__(256)
ffn_simt_kernel(const int* __restrict__ offset, int e_begin, int e_end, int N, int K,
                const float* __restrict__ a_hi, const float* __restrict__ a_lo,
                const float* __restrict__ w, const int* __restrict__ slot_of_expert, const float* __restrict__ resid,
                float* __restrict__ out_hi, float* __restrict__ out_lo) {
    __shared__ float As[TK][TM + 1];
    __shared__ float B0s[TK][TN + 1];
    __shared__ float B1s[DUAL ? TK : 1][TN + 1];
    __shared__ int s_info[4];
    if (threadIdx.x == 0) {
        int e = 0, r0 = 0, rows = 0;
        const bool ok = locate_tile(offset, e_begin, e_end, blockIdx.y, e, r0, rows);
        s_info[0] = ok ? 1 : 0;
        s_info[1] = e;
        s_info[2] = r0;
        s_info[3] = rows;
    }
    __syncthreads();
    if (!s_info[0]) return;
    const int expert = s_info[1], row0 = s_info[2], rows = s_info[3];
    const int slot = slot_of_expert ? slot_of_expert[expert] : expert;
    const int n0 = blockIdx.x * TN;
    // tile-contiguous weight plane: 128 x 32 tiles, tile (mb, kb) at (mb * KB + kb) * 4096 floats
    const int Mw = DUAL ? 2 * N : N, MBw = (Mw + 127) / 128, KBw = (K + 31) / 32;
    const size_t wbase = (size_t)slot * (size_t)MBw * (size_t)KBw * 4096;
    auto w_at = [&](int m, int k) -> float {
        return w[wbase + ((size_t)(m >> 7) * KBw + (k >> 5)) * 4096 + (size_t)(m & 127) * 32 + (k & 31)];
    };

    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc0[4][4], acc1[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc0[i][j] = acc1[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int i = threadIdx.x; i < TM * TK; i += 256) {
            const int r = i / TK, k = i % TK;
            float v = 0.f;
            if (r < rows && k0 + k < K) {
                const size_t o = (size_t)(row0 + r) * K + k0 + k;
                v = a_hi[o] + a_lo[o];
            }
            As[k][r] = v;
        }
        for (int i = threadIdx.x; i < TN * TK; i += 256) {
            const int n = i / TK, k = i % TK;
            float v0 = 0.f, v1 = 0.f;
            if (n0 + n < N && k0 + k < K) {
                if (DUAL) {
                    v0 = w_at(2 * (n0 + n), k0 + k);
                    v1 = w_at(2 * (n0 + n) + 1, k0 + k);
                } else {
                    v0 = w_at(n0 + n, k0 + k);
                }
            }
            B0s[k][n] = v0;
            if (DUAL) B1s[k][n] = v1;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b0[4], b1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b0[j] = B0s[k][tx * 4 + j];
                b1[j] = DUAL ? B1s[k][tx * 4 + j] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc0[i][j] = fmaf(a[i], b0[j], acc0[i][j]);
                    if (DUAL) acc1[i][j] = fmaf(a[i], b1[j], acc1[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const size_t o = (size_t)(row0 + r) * N + n;
            if (DUAL) {
                float hi, lo;
                split_tf32(gelu_dot(acc0[i][j], acc1[i][j]), hi, lo);
                out_hi[o] = hi;
                out_lo[o] = lo;
            } else {
                out_hi[o] = resid[o] + acc0[i][j];
            }
        }
    }
}

}  // namespace

// Grouped FFN over experts [e_begin, e_end); T rows in expert-contiguous order.
//   h_hi/h_lo [T][D], g_hi/g_lo [T][F] (scratch), routed [T][D], post [T][D]
//   slot_of_expert (device, may be NULL = identity) maps expert -> weight slot.
int launch_ffn_simt(long long T, int D, int F, int e_begin, int e_end, const int* offset, const int* slot_of_expert,
                    const float* h_hi, const float* h_lo, const float* w01, const float* wo, const float* routed,
                    float* g_hi, float* g_lo, float* post, cudaStream_t stream) {
    if (T == 0 || e_begin >= e_end) return INFMOE_OK;
    const unsigned row_tiles = (unsigned)((T + TM - 1) / TM + (e_end - e_begin));
    dim3 g1((F + TN - 1) / TN, row_tiles), g2((D + TN - 1) / TN, row_tiles);
    ffn_simt_kernel<true><<<g1, 256, 0, stream>>>(offset, e_begin, e_end, F, D, h_hi, h_lo, w01, slot_of_expert,
                                                  nullptr, g_hi, g_lo);
    ffn_simt_kernel<false><<<g2, 256, 0, stream>>>(offset, e_begin, e_end, D, F, g_hi, g_lo, wo, slot_of_expert,
                                                   routed, post, nullptr);
    note_launch(2);
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

}  // namespace infmoe
