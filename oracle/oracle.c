/*
 * CPU oracle for the InfMoE MoE-layer path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference plugin's
 * MoELayerPlugin::enqueue path.  It is the checker that the CUDA path is
 * compared with; it is never linked into, called from, or shipped with the
 * product library.  Only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg load it.
 *
 * Parity status: the reference ships no tests, golden vectors or CPU path, so
 * the pins are (1) hand-derived known-answer cases whose arithmetic is exact
 * in FP32 (tests/golden), and (2) on a GPU box, outputs of the reference's own
 * kernels (plugin/cuda/moe.cu, ops/layernorm.cu, ops/gelu.cu) compiled
 * unmodified into oracle/_ref.  The four GEMMs of the reference run inside
 * cuBLAS (closed, unpinned version): for those the parity is "unpinned" and
 * anchored on the call sites' documented meaning (C = A * B^T in FP32).
 *
 * Each function names the reference file:line it follows.
 *
 * Two precisions:
 *   - "canonical FP32": a fixed summation order that the CUDA routing kernel
 *     reproduces exactly (fmaf + lane-strided partial sums + xor tree), so
 *     gate/score/pos are compared bit for bit;
 *   - FP64-accumulated: the accuracy yardstick for the layer output
 *     (relative L2 error <= 1e-5).
 *
 * Build: gcc -O2 -ffp-contract=off -mavx2 -mfma -fopenmp -shared -fPIC
 * (contraction must stay off so that only the explicit fmaf() calls fuse).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <immintrin.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { ORACLE_OK = 0, ORACLE_ERR_NAN = 1, ORACLE_ERR_ARG = 2, ORACLE_ERR_ALLOC = 3 };

enum { VARIANT_DEFAULT = 0, VARIANT_CPM2 = 1, VARIANT_BASE_LAYER = 2 };

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* Canonical FP32 building blocks                                             */
/* ------------------------------------------------------------------------- */

/* Butterfly sum over 32 "lanes": v[l] += v[l ^ off] for off = 16,8,4,2,1.
 * Every lane ends with the same bits; this is what a warp's __shfl_xor_sync
 * reduction computes. */
static inline float lanes_xor_sum(float v[32]) {
    float t[32];
    for (int off = 16; off >= 1; off >>= 1) {
        for (int l = 0; l < 32; ++l) t[l] = v[l] + v[l ^ off];
        memcpy(v, t, sizeof(t));
    }
    return v[0];
}

/* Canonical mean / reciprocal standard deviation of one row.
 * Math: plugin/cuda/ops/layernorm.cu:126-130 (sigma2 / n2, biased) and :149
 * (rsqrt(sigma2 + eps)), eps = 1e-6 cast to float (:187).  The reference
 * accumulates with Welford/Chan merges (:30-56); here the order is the fixed
 * two-pass one described in the header: lane l owns elements
 * k = 4*(l + 32*i) + c, i ascending, c = 0..3. */
static void canon_row_stats(const float* x, int D, float* mean_out, float* rstd_out) {
    float s[32], v[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int base = 4 * l; base < D; base += 128)
            for (int c = 0; c < 4 && base + c < D; ++c) acc = acc + x[base + c];
        s[l] = acc;
    }
    const float mean = lanes_xor_sum(s) / (float)D;
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int base = 4 * l; base < D; base += 128)
            for (int c = 0; c < 4 && base + c < D; ++c) {
                const float d = x[base + c] - mean;
                acc = fmaf(d, d, acc);
            }
        v[l] = acc;
    }
    const float var = lanes_xor_sum(v) / (float)D;
    *mean_out = mean;
    *rstd_out = 1.0f / sqrtf(var + 1e-6f);
}

/* out[k] = gamma[k] * ((x[k] - mean) * rstd)   -- layernorm.cu:158-161 (gamma only). */
static void canon_layernorm_row(const float* x, const float* gamma, int D, float* out) {
    float mean, rstd;
    canon_row_stats(x, D, &mean, &rstd);
    for (int k = 0; k < D; ++k) out[k] = gamma[k] * ((x[k] - mean) * rstd);
}

/* Canonical dot product: lane-strided fmaf partials, xor tree. */
static float canon_dot(const float* a, const float* b, int D) {
    float p[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int base = 4 * l; base < D; base += 128)
            for (int c = 0; c < 4 && base + c < D; ++c) acc = fmaf(a[base + c], b[base + c], acc);
        p[l] = acc;
    }
    return lanes_xor_sum(p);
}

/* LayerNorm of n rows, canonical order.  Follows layernorm_gpu as called at
 * MoELayerPlugin.cc:324 and T5FFLayer.cc:102 (gamma != NULL, beta == NULL). */
ORACLE_API void oracle_layernorm(const float* x, const float* gamma, int64_t n, int D, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < n; ++t) canon_layernorm_row(x + t * D, gamma, D, out + t * D);
}

/* The reference's own accumulation order for one row, as launched by
 * layernorm_gpu (layernorm.cu:179-188: block (32,4) = 128 threads):
 * per-thread Welford over groups of 4 consecutive elements strided by 4*128
 * (:76-87), 5 Chan merges with lane (x + 2^l) & 31 inside each warp (:89-95),
 * then the shared-memory tree over the 4 warps (:98-124).  Used to measure the
 * distance between the canonical order and the reference's order. */
static void welford_push(float curr, float* mu, float* s2, float* cnt) {
    *cnt = *cnt + 1.0f;
    float delta = curr - *mu;
    float lmean = *mu + delta / *cnt;
    *mu = lmean;
    float delta2 = curr - lmean;
    *s2 = *s2 + delta * delta2;
}
static void chan_merge(float muB, float s2B, float cntB, float* mu, float* s2, float* cnt) {
    float delta = muB - *mu;
    float nA = *cnt, nB = cntB;
    *cnt = *cnt + cntB;
    float nX = *cnt;
    if (nX > 0.0f) {
        nA = nA / nX;
        nB = nB / nX;
        *mu = nA * (*mu) + nB * muB;
        *s2 = *s2 + s2B + delta * delta * nA * nB * nX;
    } else {
        *mu = 0.0f;
        *s2 = 0.0f;
    }
}
ORACLE_API void oracle_layernorm_reference_order(const float* x, const float* gamma, int64_t n, int D, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < n; ++t) {
        const float* row = x + t * D;
        float mu[128], s2[128], cnt[128];
        for (int thr = 0; thr < 128; ++thr) {
            mu[thr] = s2[thr] = cnt[thr] = 0.0f;
            int l = 4 * thr;
            for (; l + 3 < D; l += 4 * 128)
                for (int k = 0; k < 4; ++k) welford_push(row[l + k], &mu[thr], &s2[thr], &cnt[thr]);
            for (; l < D; ++l) welford_push(row[l], &mu[thr], &s2[thr], &cnt[thr]);
        }
        for (int w = 0; w < 4; ++w) {
            for (int step = 0; step <= 4; ++step) {
                float nmu[32], ns2[32], ncnt[32];
                for (int lane = 0; lane < 32; ++lane) {
                    int src = (lane + (1 << step)) & 31;
                    nmu[lane] = mu[32 * w + lane];
                    ns2[lane] = s2[32 * w + lane];
                    ncnt[lane] = cnt[32 * w + lane];
                    chan_merge(mu[32 * w + src], s2[32 * w + src], cnt[32 * w + src], &nmu[lane], &ns2[lane],
                               &ncnt[lane]);
                }
                memcpy(&mu[32 * w], nmu, sizeof(nmu));
                memcpy(&s2[32 * w], ns2, sizeof(ns2));
                memcpy(&cnt[32 * w], ncnt, sizeof(ncnt));
            }
        }
        /* inter-warp tree: offset 2 (warps 2,3 -> 0,1), then offset 1 (warp 1 -> 0) */
        for (int offset = 2; offset > 0; offset /= 2)
            for (int w = 0; w < offset; ++w)
                chan_merge(mu[32 * (w + offset)], s2[32 * (w + offset)], cnt[32 * (w + offset)], &mu[32 * w],
                           &s2[32 * w], &cnt[32 * w]);
        const float mean = mu[0];
        const float sigma2 = s2[0] / (float)D;
        const float invvar = 1.0f / sqrtf(sigma2 + 1e-6f);
        for (int k = 0; k < D; ++k) out[t * D + k] = gamma[k] * (invvar * (row[k] - mean));
    }
}

/* ------------------------------------------------------------------------- */
/* Routing: MoELayerPlugin.cc:312-345 + moe.cu:21-28,61-75                    */
/* ------------------------------------------------------------------------- */

/* gate[t] = first index of the maximum score (strict '>' scan from -FLT_MAX,
 * moe.cu:26-27,62-67); score[t] = that maximum.  gamma != NULL selects the
 * cpm_2 pre-gating LayerNorm (MoELayerPlugin.cc:315-327).  centroids are
 * [E][D] row-major (cuBLAS call MoELayerPlugin.cc:334-336: OP_T, lda = D).
 * aff (nullable) receives all T*E scores.  Returns ORACLE_ERR_NAN when a row
 * selects nothing (reference: device assert, moe.cu:70). */
ORACLE_API int oracle_route(const float* X, const float* centroids, const float* gamma, int64_t T, int D, int E,
                            int32_t* gate, float* score, float* aff) {
    int bad = 0;
#pragma omp parallel
    {
        float* xs = (float*)malloc(sizeof(float) * (size_t)(D > 0 ? D : 1));
#pragma omp for schedule(static)
        for (int64_t t = 0; t < T; ++t) {
            const float* row = X + t * D;
            const float* src = row;
            if (gamma) {
                canon_layernorm_row(row, gamma, D, xs);
                src = xs;
            }
            float best = -FLT_MAX;
            int32_t best_e = -1;
            for (int e = 0; e < E; ++e) {
                const float s = canon_dot(src, centroids + (int64_t)e * D, D);
                if (aff) aff[t * E + e] = s;
                if (s > best) {
                    best = s;
                    best_e = e;
                }
            }
            gate[t] = best_e;
            score[t] = best;
            if (best_e < 0) {
#pragma omp atomic write
                bad = 1;
            }
        }
        free(xs);
    }
    return bad ? ORACLE_ERR_NAN : ORACLE_OK;
}

/* Top-1 over a given score matrix: moe_expert_select, moe.cu:13-76,147-159. */
ORACLE_API int oracle_select_top1(const float* aff, int64_t T, int E, int32_t* gate, float* score) {
    int bad = 0;
    for (int64_t t = 0; t < T; ++t) {
        float best = -FLT_MAX;
        int32_t best_e = -1;
        for (int e = 0; e < E; ++e) {
            const float s = aff[t * E + e];
            if (s > best) {
                best = s;
                best_e = e;
            }
        }
        gate[t] = best_e;
        if (score) score[t] = best;
        if (best_e < 0) bad = 1;
    }
    return bad ? ORACLE_ERR_NAN : ORACLE_OK;
}

/* FP64 scores, for counting near-tie flips between FP32 and FP64 argmax. */
ORACLE_API void oracle_route_f64(const float* X, const float* centroids, const float* gamma, int64_t T, int D, int E,
                                 int32_t* gate, double* top1, double* top2) {
#pragma omp parallel
    {
        double* xs = (double*)malloc(sizeof(double) * (size_t)(D > 0 ? D : 1));
#pragma omp for schedule(static)
        for (int64_t t = 0; t < T; ++t) {
            const float* row = X + t * D;
            if (gamma) {
                double m = 0, v = 0;
                for (int k = 0; k < D; ++k) m += row[k];
                m /= D;
                for (int k = 0; k < D; ++k) v += (row[k] - m) * (row[k] - m);
                v /= D;
                const double r = 1.0 / sqrt(v + 1e-6);
                for (int k = 0; k < D; ++k) xs[k] = (double)gamma[k] * ((row[k] - m) * r);
            } else {
                for (int k = 0; k < D; ++k) xs[k] = row[k];
            }
            double b1 = -DBL_MAX, b2 = -DBL_MAX;
            int32_t be = -1;
            for (int e = 0; e < E; ++e) {
                const float* c = centroids + (int64_t)e * D;
                double s = 0;
                for (int k = 0; k < D; ++k) s += xs[k] * (double)c[k];
                if (s > b1) {
                    b2 = b1;
                    b1 = s;
                    be = e;
                } else if (s > b2) {
                    b2 = s;
                }
            }
            gate[t] = be;
            if (top1) top1[t] = b1;
            if (top2) top2[t] = b2;
        }
        free(xs);
    }
}

/* ------------------------------------------------------------------------- */
/* Dispatch: moe_expert_count, moe.cu:161-212 (this is host code in the       */
/* reference; restated with the same three loops)                             */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_dispatch(const int32_t* gate, int64_t T, int E, int32_t* count, int32_t* offset,
                               int32_t* pos) {
    for (int e = 0; e < E; ++e) count[e] = 0;
    for (int64_t t = 0; t < T; ++t) {
        if (gate[t] < 0 || gate[t] >= E) return ORACLE_ERR_NAN; /* moe.cu:184 assert */
        count[gate[t]]++;
    }
    offset[0] = 0;
    for (int e = 1; e < E; ++e) offset[e] = offset[e - 1] + count[e - 1]; /* moe.cu:187-190 */
    offset[E] = (int32_t)T;                                               /* MoELayerPlugin.cc:351 */
    int32_t* cursor = (int32_t*)malloc(sizeof(int32_t) * (size_t)(E > 0 ? E : 1));
    if (!cursor) return ORACLE_ERR_ALLOC;
    memcpy(cursor, offset, sizeof(int32_t) * (size_t)E);
    for (int64_t t = 0; t < T; ++t) pos[cursor[gate[t]]++] = (int32_t)t; /* moe.cu:198-200 */
    free(cursor);
    return ORACLE_OK;
}

/* Scatter: batch_scatter_feature_and_weight_kernel, moe.cu:98-113. */
ORACLE_API void oracle_scatter(const float* X, const float* score, const int32_t* pos, int64_t T, int D,
                               float* routed, float* rscore) {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < T; ++j) {
        memcpy(routed + j * D, X + (int64_t)pos[j] * D, sizeof(float) * (size_t)D);
        if (rscore && score) rscore[j] = score[pos[j]];
    }
}

/* Gather: batch_gather_kernel, moe.cu:89-96. */
ORACLE_API void oracle_gather(const float* in, const int32_t* pos, int64_t T, int D, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < T; ++j) memcpy(out + (int64_t)pos[j] * D, in + j * D, sizeof(float) * (size_t)D);
}

/* base_layer mix + gather: fused_batch_mix_and_gather_kernel, moe.cu:115-127;
 * sigmoid(x) = 1 / (1 + exp(-x)), common.cuh:24-27. */
ORACLE_API void oracle_mix_gather(const float* post, const float* routed, const float* rscore, const int32_t* pos,
                                  int64_t T, int D, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < T; ++j) {
        const float alpha = 1.0f / (1.0f + expf(-rscore[j]));
        float* o = out + (int64_t)pos[j] * D;
        for (int k = 0; k < D; ++k) o[k] = alpha * post[j * D + k] + (1.0f - alpha) * routed[j * D + k];
    }
}

/* gelu(a) * b: gelu_dot functor, ops/gelu.cu:6-16 (cdf first, then a*cdf*b). */
static inline float gelu_dot_f32(float a, float b) {
    const float cdf = 0.5f * (1.0f + tanhf(a * (0.035677408136300125f * a * a + 0.7978845608028654f)));
    return a * cdf * b;
}
ORACLE_API void oracle_gelu_dot(const float* a, float* b, int64_t n) {
    for (int64_t i = 0; i < n; ++i) b[i] = gelu_dot_f32(a[i], b[i]);
}

/* ------------------------------------------------------------------------- */
/* FP32 GEMM  C[M][N] (+)= A[M][K] * B[N][K]^T  (both operands K-contiguous), */
/* the shape of every cublasSgemm_v2(OP_T, OP_N, ...) call on the path        */
/* (T5FFLayer.cc:114-116,122-124,136-138).  Blocked, AVX2 6x16 micro-kernel,  */
/* OpenMP over column panels: this is also the timed CPU baseline.            */
/* ------------------------------------------------------------------------- */
#define GEMM_KB 256
#define GEMM_NR 16
#define GEMM_MR 6

static void micro_6x16(int kb, const float* A, int lda, const float* Bp, float* C, int ldc, int mr, int nr,
                       int accumulate) {
    __m256 acc[GEMM_MR][2];
    for (int i = 0; i < GEMM_MR; ++i) acc[i][0] = acc[i][1] = _mm256_setzero_ps();
    for (int k = 0; k < kb; ++k) {
        const __m256 b0 = _mm256_loadu_ps(Bp + (size_t)k * GEMM_NR);
        const __m256 b1 = _mm256_loadu_ps(Bp + (size_t)k * GEMM_NR + 8);
        for (int i = 0; i < GEMM_MR; ++i) {
            const __m256 a = _mm256_set1_ps(i < mr ? A[(size_t)i * lda + k] : 0.0f);
            acc[i][0] = _mm256_fmadd_ps(a, b0, acc[i][0]);
            acc[i][1] = _mm256_fmadd_ps(a, b1, acc[i][1]);
        }
    }
    float tmp[GEMM_NR];
    for (int i = 0; i < mr; ++i) {
        _mm256_storeu_ps(tmp, acc[i][0]);
        _mm256_storeu_ps(tmp + 8, acc[i][1]);
        float* c = C + (size_t)i * ldc;
        if (accumulate)
            for (int j = 0; j < nr; ++j) c[j] += tmp[j];
        else
            for (int j = 0; j < nr; ++j) c[j] = tmp[j];
    }
}

/* beta = 0 when accumulate == 0, beta = 1 otherwise. */
static void sgemm_nt(int M, int N, int K, const float* A, int lda, const float* B, int ldb, float* C, int ldc,
                     int accumulate) {
    if (M <= 0 || N <= 0) return;
    const int npanels = (N + GEMM_NR - 1) / GEMM_NR;
#pragma omp parallel
    {
        float* Bp = (float*)aligned_alloc(64, sizeof(float) * GEMM_KB * GEMM_NR);
#pragma omp for schedule(dynamic, 4)
        for (int p = 0; p < npanels; ++p) {
            const int n0 = p * GEMM_NR;
            const int nr = N - n0 < GEMM_NR ? N - n0 : GEMM_NR;
            for (int k0 = 0; k0 < K; k0 += GEMM_KB) {
                const int kb = K - k0 < GEMM_KB ? K - k0 : GEMM_KB;
                for (int k = 0; k < kb; ++k)
                    for (int j = 0; j < GEMM_NR; ++j)
                        Bp[(size_t)k * GEMM_NR + j] = j < nr ? B[(size_t)(n0 + j) * ldb + k0 + k] : 0.0f;
                for (int m0 = 0; m0 < M; m0 += GEMM_MR) {
                    const int mr = M - m0 < GEMM_MR ? M - m0 : GEMM_MR;
                    micro_6x16(kb, A + (size_t)m0 * lda + k0, lda, Bp, C + (size_t)m0 * ldc + n0, ldc, mr, nr,
                               accumulate || k0 > 0);
                }
            }
        }
        free(Bp);
    }
}

ORACLE_API void oracle_sgemm_nt(int M, int N, int K, const float* A, const float* B, float* C, int accumulate) {
    sgemm_nt(M, N, K, A, K, B, K, C, N, accumulate);
}

/* ------------------------------------------------------------------------- */
/* T5_FF expert: T5FFLayer::run, T5FFLayer.cc:90-141                          */
/*   h = LN(x; ln_w)          (:99-103)                                       */
/*   a = h wi_0^T, b = h wi_1^T   (:112-124)                                  */
/*   g = gelu(a) * b          (:126, gelu.cu:8-15)                            */
/*   y = x + g wo^T           (:128-138; D2D copy then SGEMM beta = 1)        */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_expert_ffn_f32(const float* x, int64_t n, int D, int F, const float* ln_w, const float* wi0,
                                     const float* wi1, const float* wo, float* y) {
    if (n <= 0) return ORACLE_OK;
    float* h = (float*)malloc(sizeof(float) * (size_t)n * D);
    float* a = (float*)malloc(sizeof(float) * (size_t)n * F);
    float* b = (float*)malloc(sizeof(float) * (size_t)n * F);
    if (!h || !a || !b) {
        free(h);
        free(a);
        free(b);
        return ORACLE_ERR_ALLOC;
    }
    oracle_layernorm(x, ln_w, n, D, h);
    sgemm_nt((int)n, F, D, h, D, wi0, D, a, F, 0);
    sgemm_nt((int)n, F, D, h, D, wi1, D, b, F, 0);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n * (int64_t)F; ++i) b[i] = gelu_dot_f32(a[i], b[i]);
    memcpy(y, x, sizeof(float) * (size_t)n * D);
    sgemm_nt((int)n, D, F, b, F, wo, F, y, D, 1);
    free(h);
    free(a);
    free(b);
    return ORACLE_OK;
}

/* Same expert with FP64 accumulation and FP64 transcendental evaluation. */
ORACLE_API int oracle_expert_ffn_f64(const float* x, int64_t n, int D, int F, const float* ln_w, const float* wi0,
                                     const float* wi1, const float* wo, double* y) {
    if (n <= 0) return ORACLE_OK;
    int fail = 0;
#pragma omp parallel
    {
        double* h = (double*)malloc(sizeof(double) * (size_t)D);
        double* g = (double*)malloc(sizeof(double) * (size_t)F);
        if (!h || !g) {
#pragma omp atomic write
            fail = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (int64_t r = 0; r < n; ++r) {
            if (!h || !g) continue;
            const float* row = x + r * D;
            double m = 0, v = 0;
            for (int k = 0; k < D; ++k) m += row[k];
            m /= D;
            for (int k = 0; k < D; ++k) v += (row[k] - m) * (row[k] - m);
            v /= D;
            const double rs = 1.0 / sqrt(v + 1e-6);
            for (int k = 0; k < D; ++k) h[k] = (double)ln_w[k] * ((row[k] - m) * rs);
            for (int f = 0; f < F; ++f) {
                const float* w0 = wi0 + (size_t)f * D;
                const float* w1 = wi1 + (size_t)f * D;
                double a = 0, b = 0;
                for (int k = 0; k < D; ++k) {
                    a += h[k] * (double)w0[k];
                    b += h[k] * (double)w1[k];
                }
                const double cdf = 0.5 * (1.0 + tanh(a * (0.035677408136300125 * a * a + 0.7978845608028654)));
                g[f] = a * cdf * b;
            }
            for (int d = 0; d < D; ++d) {
                const float* w = wo + (size_t)d * F;
                double s = 0;
                for (int f = 0; f < F; ++f) s += g[f] * (double)w[f];
                y[r * D + d] = (double)row[d] + s;
            }
        }
        free(h);
        free(g);
    }
    return fail ? ORACLE_ERR_ALLOC : ORACLE_OK;
}

/* ------------------------------------------------------------------------- */
/* Whole layer: MoELayerPlugin::enqueue, MoELayerPlugin.cc:279-416            */
/* ------------------------------------------------------------------------- */
/* Expert weights are passed as arrays of E pointers (NULL allowed for an
 * expert that receives no rows).  literal_gather != 0 reproduces the literal
 * reference for cpm_2/default, whose final gather reads the scattered input
 * instead of the expert output (MoELayerPlugin.cc:411); 0 gathers the expert
 * output, which is what the product implements.
 * Optional outputs (may be NULL): gate[T], score[T], count[E], offset[E+1], pos[T]. */
ORACLE_API int oracle_layer_forward_f32(const float* X, int64_t T, int D, int F, int E, int variant,
                                        const float* centroids, const float* gating_ln_w,
                                        const float* const* ln_w, const float* const* wi0,
                                        const float* const* wi1, const float* const* wo, int literal_gather,
                                        float* out, int32_t* gate_o, float* score_o, int32_t* count_o,
                                        int32_t* offset_o, int32_t* pos_o) {
    if (T <= 0) return ORACLE_OK;
    if (variant == VARIANT_CPM2 && !gating_ln_w) return ORACLE_ERR_ARG; /* MoELayerPlugin.cc:76-79 */
    int32_t* gate = (int32_t*)malloc(sizeof(int32_t) * (size_t)T);
    int32_t* pos = (int32_t*)malloc(sizeof(int32_t) * (size_t)T);
    int32_t* count = (int32_t*)malloc(sizeof(int32_t) * (size_t)(E + 1));
    int32_t* offset = (int32_t*)malloc(sizeof(int32_t) * (size_t)(E + 1));
    float* score = (float*)malloc(sizeof(float) * (size_t)T);
    float* rscore = (float*)malloc(sizeof(float) * (size_t)T);
    float* routed = (float*)malloc(sizeof(float) * (size_t)T * D);
    float* post = (float*)malloc(sizeof(float) * (size_t)T * D);
    int rc = ORACLE_OK;
    if (!gate || !pos || !count || !offset || !score || !rscore || !routed || !post) rc = ORACLE_ERR_ALLOC;
    if (!rc) rc = oracle_route(X, centroids, variant == VARIANT_CPM2 ? gating_ln_w : NULL, T, D, E, gate, score, NULL);
    if (!rc) rc = oracle_dispatch(gate, T, E, count, offset, pos);
    if (!rc) {
        oracle_scatter(X, score, pos, T, D, routed, rscore); /* always the un-normalised X: MoELayerPlugin.cc:354 */
        for (int e = 0; e < E && !rc; ++e) {
            if (count[e] == 0) continue; /* MoELayerPlugin.cc:362,384 */
            rc = oracle_expert_ffn_f32(routed + (int64_t)offset[e] * D, count[e], D, F, ln_w[e], wi0[e], wi1[e],
                                       wo[e], post + (int64_t)offset[e] * D);
        }
    }
    if (!rc) {
        if (variant == VARIANT_BASE_LAYER)
            oracle_mix_gather(post, routed, rscore, pos, T, D, out); /* :407-409 */
        else
            oracle_gather(literal_gather ? routed : post, pos, T, D, out); /* :411 */
        if (gate_o) memcpy(gate_o, gate, sizeof(int32_t) * (size_t)T);
        if (score_o) memcpy(score_o, score, sizeof(float) * (size_t)T);
        if (count_o) memcpy(count_o, count, sizeof(int32_t) * (size_t)E);
        if (offset_o) memcpy(offset_o, offset, sizeof(int32_t) * (size_t)(E + 1));
        if (pos_o) memcpy(pos_o, pos, sizeof(int32_t) * (size_t)T);
    }
    free(gate);
    free(pos);
    free(count);
    free(offset);
    free(score);
    free(rscore);
    free(routed);
    free(post);
    return rc;
}

/* FP64-accumulated layer that takes the routing decision as an INPUT (gate,
 * score from the canonical FP32 oracle), so that a near-tie flip is counted
 * separately and does not pollute the L2 figure.  Output is double[T][D]. */
ORACLE_API int oracle_layer_forward_f64(const float* X, int64_t T, int D, int F, int E, int variant,
                                        const int32_t* gate, const float* score, const float* const* ln_w,
                                        const float* const* wi0, const float* const* wi1,
                                        const float* const* wo, double* out) {
    if (T <= 0) return ORACLE_OK;
    int32_t* pos = (int32_t*)malloc(sizeof(int32_t) * (size_t)T);
    int32_t* count = (int32_t*)malloc(sizeof(int32_t) * (size_t)(E + 1));
    int32_t* offset = (int32_t*)malloc(sizeof(int32_t) * (size_t)(E + 1));
    float* routed = (float*)malloc(sizeof(float) * (size_t)T * D);
    float* rscore = (float*)malloc(sizeof(float) * (size_t)T);
    double* post = (double*)malloc(sizeof(double) * (size_t)T * D);
    int rc = ORACLE_OK;
    if (!pos || !count || !offset || !routed || !rscore || !post) rc = ORACLE_ERR_ALLOC;
    if (!rc) rc = oracle_dispatch(gate, T, E, count, offset, pos);
    if (!rc) {
        oracle_scatter(X, score, pos, T, D, routed, rscore);
        for (int e = 0; e < E && !rc; ++e) {
            if (count[e] == 0) continue;
            rc = oracle_expert_ffn_f64(routed + (int64_t)offset[e] * D, count[e], D, F, ln_w[e], wi0[e], wi1[e],
                                       wo[e], post + (int64_t)offset[e] * D);
        }
    }
    if (!rc) {
#pragma omp parallel for schedule(static)
        for (int64_t j = 0; j < T; ++j) {
            double* o = out + (int64_t)pos[j] * D;
            if (variant == VARIANT_BASE_LAYER) {
                const double alpha = 1.0 / (1.0 + exp(-(double)rscore[j]));
                for (int k = 0; k < D; ++k) o[k] = alpha * post[j * D + k] + (1.0 - alpha) * (double)routed[j * D + k];
            } else {
                for (int k = 0; k < D; ++k) o[k] = post[j * D + k];
            }
        }
    }
    free(pos);
    free(count);
    free(offset);
    free(routed);
    free(rscore);
    free(post);
    return rc;
}
