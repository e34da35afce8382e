// Launchers of the CUDA kernels (defined in route.cu, dispatch.cu, rows.cu, ffn_simt.cu, ffn_umma.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>

namespace infmoe {

int launch_route(const float* X, const float* C, const float* gamma, long long T, int D, int E, int* gate,
                 float* score, int* status, cudaStream_t stream);
int make_f32_row_map(CUtensorMap* map, const void* base, long long K, long long rows, int box_rows);
int launch_select_top1(long long T, int E, const float* aff, int* gate, float* weight, int* status,
                       cudaStream_t stream);
// region_count != NULL: the T slots are regions of region_size slots, of which only the first region_count[s]
// hold rows (receive buffer of the expert-parallel path); the other slots are skipped silently.
int launch_dispatch(const int* gate, long long T, int E, int* pos, int* count, int* offset, int* status,
                    cudaStream_t stream, const int* region_count = nullptr, int region_size = 0);
int launch_scatter(long long T, int D, const float* X, const float* coeff, const int* pos, float* routed,
                   float* rcoeff, cudaStream_t stream);
// valid_rows (device, may be NULL): rows at or past *valid_rows are skipped (tokens without an expert sit at
// the tail of pos[]; the dispatch kernel stores their start in offset[E]).  routed may be NULL.
int launch_scatter_ln_split(long long T, int D, const float* X, const float* score, const int* pos, const int* gate,
                            const float* gamma_all, const int* valid_rows, float* routed, float* rscore, float* h_hi,
                            float* h_lo, bool pack, cudaStream_t stream);
int launch_gather(long long T, int D, const float* in, const int* pos, float* out, cudaStream_t stream,
                  const int* valid_rows = nullptr);
int launch_mix_gather(long long T, int D, const int* pos, const float* routed, const float* post,
                      const float* coeff, float* out, cudaStream_t stream, const int* valid_rows = nullptr);
int launch_layernorm(float* out, const float* in, long long n, int D, const float* gamma, cudaStream_t stream);
int launch_gelu_dot(const float* a, float* b, size_t len, cudaStream_t stream);
int launch_split(const float* src, float* hi, float* lo, size_t len, cudaStream_t stream);
int launch_fill_int(int* dst, int value, cudaStream_t stream);   // *dst = value, stream ordered
// Tile-contiguous weight layout (see rows.cu); src1 != NULL interleaves the rows of two matrices.
int launch_retile(const float* src0, const float* src1, int M, int K, float* dst, cudaStream_t stream);
inline size_t tiled_elems(int M, int K) { return (size_t)((M + 127) / 128) * 128 * (size_t)((K + 31) / 32) * 32; }
int launch_ln_split(long long n, int D, const float* in, const float* gamma, float* h_hi, float* h_lo, bool pack,
                    cudaStream_t stream);
// Bytes of the second activation plane of a [rows][K] operand: FP32 tail plane (CUDA-core GEMM) or packed BF16
// plane with rows padded to whole groups of 32 values (tensor-core GEMM); the larger of the two.
inline size_t second_plane_bytes(long long rows, int K) { return (size_t)rows * (size_t)((K + 31) / 32) * 128; }

// Expert weights live in two raw FP32 planes in tile-contiguous layout (128 x 32 tiles, see launch_retile):
// w01 [slots] x tiled(2F x D) (row 2f = wi_0[f], row 2f+1 = wi_1[f]) and wo [slots] x tiled(D x F).  
// Activations travel as two planes: hi = value rounded to TF32 (FP32 [rows][K]) and either lo = value - hi
// (FP32 [rows][K], CUDA-core GEMM) or the packed BF16 plane of common.cuh (tensor-core GEMM).
int launch_ffn_simt(long long T, int D, int F, int e_begin, int e_end, const int* offset, const int* slot_of_expert,
                    const float* h_hi, const float* h_lo, const float* w01, const float* wo, const float* routed,
                    float* g_hi, float* g_lo, float* post, cudaStream_t stream);

// A one-warp kernel that waits, with the GEMM's bounded wait and the given limit, on a barrier nobody completes.
int launch_wait_probe(unsigned long long limit_ns, int* status, unsigned long long* waited_ns, cudaStream_t stream);

bool ffn_umma_supported(int D, int F, int E);
// out_pos != NULL: `post` is the layer output in token order, row j of the experts' result goes to row out_pos[j]
// (and mix_score != NULL applies the base_layer output mix on the way): the combine step fused into the epilogue.
// out_row_ptr != NULL: row out_pos[j] is written to the address out_row_ptr[out_pos[j]] instead.
int launch_ffn_umma(long long T, int D, int F, int E, int e_begin, int e_end, const int* offset,
                    const int* slot_of_expert, int slots, const float* h_hi, const float* h_lo, const float* w01,
                    const float* wo, const float* routed, float* g_hi, float* g_lo, float* post, int* status,
                    int num_sms, cudaStream_t stream, cudaEvent_t mid_event = nullptr, const int* out_pos = nullptr,
                    const float* mix_score = nullptr, const unsigned long long* out_row_ptr = nullptr);
// Rows of `in` [n][D] copied to the addresses dst[i] (one per row; they may point into a peer GPU's memory).
int launch_rows_to_ptrs(long long n, int D, const float* in, const unsigned long long* dst, cudaStream_t stream);

}  // namespace infmoe
