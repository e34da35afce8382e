// Grouped expert FFN on the Blackwell tensor cores (sm_100a): tcgen05.mma
// kind::tf32 with TMEM accumulators, operands staged by TMA, 3xTF32 error
// compensation so the products keep FP32 accuracy.
//
// Replaces, for all experts at once, the per-expert sequence of
// T5FFLayer::run (plugin/sublayers/T5FFLayer.cc:112-138):
//   cublasSgemm_v2 x2 (wi_0, wi_1) -> fused_gelu_dot_gpu -> cudaMemcpyAsync D2D -> cublasSgemm_v2 (beta = 1)
//
// Two launches of one kernel template (the weights are the M-side operand):
//   EPI_GELU_PAIR  g = gelu(h wi_0^T) * (h wi_1^T)   K = d_model, weight rows = 2 * d_ff
//                  (rows of wi_0 and wi_1 are stored interleaved: row 2f = wi_0[f], row 2f+1 = wi_1[f],
//                   so both halves of the gate land in neighbouring TMEM lanes of ONE accumulator)
//   EPI_RESIDUAL   y = x + g wo^T                     K = d_ff,    weight rows = d_model
//
// Orientation.  Weight rows sit on the MMA's M side (always a full 128-row
// tile), the tokens of one expert on the N side (any multiple of 16 up to
// NMAX).  An expert with 139 tokens therefore costs one N=144 tile instead of
// two 128-token tiles, and a decode step with 1..64 tokens runs N=16..64 MMAs.
// The accumulator is D^T: TMEM lane = weight row, TMEM column = token.
//
// 3xTF32.  Every operand is stored as two FP32 planes: hi = x rounded to TF32
// and lo = x - hi (exact).  Per 8-wide k step three MMAs accumulate
// lo*hi + hi*lo + hi*hi into the same FP32 accumulator; the dropped lo*lo term
// is below 2^-22 relative.
//
// Chunked accumulation.  The tensor core adds into its FP32 accumulator with
// truncation, not round-to-nearest: measured on B200, one accumulator carried
// over K = 1024..2048 drifts by about 1.5e-5 relative, and the drift grows
// linearly with the number of MMAs.  So TMEM only ever holds the sum of one K
// chunk of 256 (96 MMAs); two TMEM accumulators alternate, and the accumulate
// warps add each finished chunk into a running sum in registers with
// round-to-nearest adds while the tensor core already works on the next chunk.
// The same double buffering hides the epilogue behind the next tile's MMAs.
//
// Pipeline per CTA (persistent, one CTA per SM, 320 threads):
//   warp 0      TMA producer: per k block loads the weight tile (box 128 x BK)
//               and the token tile (boxes 32 x BK) of both planes into a
//               STAGES-deep shared-memory ring, completion on mbarriers
//   warp 1      allocates TMEM, issues tcgen05.mma from one lane, commits each
//               stage back to the producer and each K chunk to the accumulate warps
//   warps 2..9  accumulate + epilogue: tcgen05.ld the chunk (one TMEM lane quarter
//               and every other 16-column slice per warp), add into registers; after
//               the last chunk gelu*dot + TF32 split (lane pairs exchange a and b by
//               shuffle) or residual add, stores contiguous over the weight-row index
// Tiles are (expert, 128-row weight block, token chunk); the list is derived in
// the kernel from offset[E+1], so no host synchronisation is needed.  Every
// mbarrier wait is bounded: on expiry the CTA raises STATUS_WAIT_TIMEOUT, lets
// copies in flight land, frees its TMEM and returns.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace infmoe {

namespace {

constexpr int UMMA_M = 128;
constexpr int MAX_EXPERTS = 1024;
constexpr unsigned long long WAIT_LIMIT_NS = 4000000000ull;  // 4 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Bounded wait.  Returns false when the wait was abandoned (limit reached here or in another role).
__device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int i = 0; i < 2048; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    while (true) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Brings a weight box into L2 without touching shared memory.
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, both operands K-major, FP32 accumulate.
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <int BK>
struct Swz {
    static_assert(BK == 16 || BK == 32, "BK must give 64- or 128-byte shared-memory rows");
    static constexpr int ROW_BYTES = BK * 4;
    static constexpr uint64_t LAYOUT = BK == 32 ? 2 : 4;          // UMMA layout type: SWIZZLE_128B / SWIZZLE_64B
    static constexpr uint64_t SBO = (8 * ROW_BYTES) >> 4;         // 8-row group pitch, 16-byte units
};

// Shared-memory matrix descriptor of a K-major swizzled tile (rows of BK floats, 8-row swizzle groups).
template <int BK>
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address
    d |= (uint64_t)1 << 16;                      // leading byte offset: not used by swizzled K-major layouts
    d |= Swz<BK>::SBO << 32;                     // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                      // descriptor version of sm_100
    d |= Swz<BK>::LAYOUT << 61;
    return d;
}

// Instruction descriptor: FP32 accumulate, TF32 x TF32, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(UMMA_M >> 4) << 24);
}

enum { EPI_GELU_PAIR = 0, EPI_RESIDUAL = 1 };

constexpr int EPI_WARPS = 8;                        // two warps per TMEM lane quarter
constexpr int GEMM_THREADS = (2 + EPI_WARPS) * 32;  // producer, MMA issuer, accumulate/epilogue warps
constexpr int ACC_STRIDE = 256;                     // TMEM columns between the two accumulator buffers
constexpr int TMEM_COLS = 512;
constexpr int K_CHUNK = 256;                        // K extent accumulated inside the tensor core at a time

template <int BK, int NMAX, int STAGES>
struct Cfg {
    static constexpr int W_TILE = UMMA_M * BK * 4;
    static constexpr int A_TILE = NMAX * BK * 4;
    static constexpr int STAGE = 2 * W_TILE + 2 * A_TILE;           // hi and lo planes of both operands
    static constexpr int SMEM = STAGES * STAGE + 1024;              // + slack to align the ring to 1024 bytes
    static constexpr int KB_PER_CHUNK = K_CHUNK / BK;
    static constexpr int SLICES = NMAX / 32;                        // 16-column slices owned by one epilogue thread
    static_assert(NMAX % 32 == 0 && NMAX <= ACC_STRIDE, "token chunk");
    static_assert(W_TILE % 1024 == 0 && A_TILE % 1024 == 0, "tiles must keep 1024-byte alignment");
};

struct GemmArgs {
    const int* offset;          // [E+1] first routed row of each expert
    const int* slot_of_expert;  // expert -> weight slot (NULL: identity)
    int E, e_begin, e_end;      // experts [e_begin, e_end) are processed
    int M_total;                // weight rows: 2 * d_ff (wi_0 / wi_1 rows interleaved) or d_model
    int K;
    float* out_hi;              // GELU_PAIR: g_hi [T][M_total / 2]; RESIDUAL: y [T][M_total]
    float* out_lo;              // GELU_PAIR: g_lo
    const float* resid;         // RESIDUAL: x [T][M_total]
    int* status;
    int prefetch;               // L2 prefetch distance of the weight stream, in k blocks
};

struct TileInfo {
    int expert, slot, mb, row0, n_tok, n_pad;
};

template <int NMAX>
__device__ __forceinline__ void chunking(int cnt, int& nch, int& csz) {
    nch = (cnt + NMAX - 1) / NMAX;
    csz = nch ? (((cnt + nch - 1) / nch + 15) & ~15) : 0;  // balanced chunks, multiple of 16, <= NMAX
}

template <int NMAX>
__device__ __forceinline__ TileInfo decode_tile(int tile, const int* s_prefix, const GemmArgs& a) {
    int lo = a.e_begin, hi = a.e_end - 1;  // last e with s_prefix[e] <= tile
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    TileInfo t;
    t.expert = lo;
    t.slot = a.slot_of_expert ? a.slot_of_expert[lo] : lo;
    const int beg = a.offset[lo], cnt = a.offset[lo + 1] - beg;
    int nch, csz;
    chunking<NMAX>(cnt, nch, csz);
    const int local = tile - s_prefix[lo];
    t.mb = local / nch;                 // chunk-minor: CTAs working side by side share the weight tile in L2
    const int c = local % nch;
    t.row0 = beg + c * csz;
    t.n_tok = min(csz, beg + cnt - t.row0);
    t.n_pad = (t.n_tok + 15) & ~15;
    return t;
}

template <int EPI, int BK, int NMAX, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
ffn_umma_kernel(const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
                const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                const GemmArgs args) {
    using C = Cfg<BK, NMAX, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[STAGES];
    __shared__ __align__(8) uint64_t s_empty[STAGES];
    __shared__ __align__(8) uint64_t s_acc_full[2];
    __shared__ __align__(8) uint64_t s_acc_empty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_prefix[MAX_EXPERTS + 1];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int MB = (args.M_total + UMMA_M - 1) / UMMA_M;
    const int KB = (args.K + BK - 1) / BK;

    // ---- tile schedule: exclusive prefix of tiles per expert -------------------------------
    if (warp == 0) {
        int carry = 0;
        for (int e0 = 0; e0 < args.E; e0 += 32) {
            const int e = e0 + lane;
            int nt = 0;
            if (e < args.E && e >= args.e_begin && e < args.e_end) {
                int nch, csz;
                chunking<NMAX>(args.offset[e + 1] - args.offset[e], nch, csz);
                nt = nch * MB;
            }
            int incl = nt;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += n;
            }
            if (e < args.E) s_prefix[e] = carry + incl - nt;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) s_prefix[args.E] = carry;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&s_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&s_acc_full[b]), 1);
            mbar_init(smem_u32(&s_acc_empty[b]), EPI_WARPS * 32);
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    const int total_tiles = s_prefix[args.E];
    volatile int* abort_flag = &s_abort;

    if (warp == 0) {
        // ================= TMA producer =================
        // Optional L2 prefetch cursor PF k blocks ahead of the loads (INFMOE_GEMM_PREFETCH).  Measured
        // on B200 it does not help this kernel (the weight stream already runs at ~75% of the copy
        // bandwidth; distances >= 8 k blocks thrash L2), so it is off by default.
        if (lane == 0) {
            const int PF = args.prefetch;    // look-ahead in k blocks
            uint32_t it = 0;
            int la_tile = blockIdx.x, la_kb = 0, la_m0 = 0, la_slot = 0;
            bool la_valid = la_tile < total_tiles;
            if (la_valid) {
                const TileInfo t = decode_tile<NMAX>(la_tile, s_prefix, args);
                la_m0 = t.mb * UMMA_M;
                la_slot = t.slot;
            }
            auto prefetch_next = [&]() {
                if (!la_valid) return;
                tma_prefetch_3d(&map_w_hi, la_kb * BK, la_m0, la_slot);
                tma_prefetch_3d(&map_w_lo, la_kb * BK, la_m0, la_slot);
                if (++la_kb == KB) {
                    la_kb = 0;
                    la_tile += gridDim.x;
                    la_valid = la_tile < total_tiles;
                    if (la_valid) {
                        const TileInfo t = decode_tile<NMAX>(la_tile, s_prefix, args);
                        la_m0 = t.mb * UMMA_M;
                        la_slot = t.slot;
                    }
                }
            };
            for (int i = 0; i < PF; ++i) prefetch_next();
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                const TileInfo t = decode_tile<NMAX>(tile, s_prefix, args);
                const int nbox = (t.n_pad + 31) >> 5;
                const uint32_t bytes = 2 * C::W_TILE + 2 * nbox * 32 * BK * 4;
                bool ok = true;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    prefetch_next();
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&s_full[s]);
                    mbar_expect_tx(bar, bytes);
                    const uint32_t base = ring + s * C::STAGE;
                    const int k0 = kb * BK, m0 = t.mb * UMMA_M;
                    tma_load_3d(base, &map_w_hi, bar, k0, m0, t.slot);
                    tma_load_3d(base + C::W_TILE, &map_w_lo, bar, k0, m0, t.slot);
                    const uint32_t a_hi = base + 2 * C::W_TILE, a_lo = a_hi + C::A_TILE;
                    for (int b = 0; b < nbox; ++b) {
                        tma_load_2d(a_hi + b * 32 * BK * 4, &map_a_hi, bar, k0, t.row0 + b * 32);
                        tma_load_2d(a_lo + b * 32 * BK * 4, &map_a_lo, bar, k0, t.row0 + b * 32);
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            uint32_t it = 0, chunk = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                const TileInfo t = decode_tile<NMAX>(tile, s_prefix, args);
                const uint32_t idesc = make_idesc(t.n_pad);
                bool ok = true;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int kc = kb % C::KB_PER_CHUNK;
                    const uint32_t buf = chunk & 1;
                    if (kc == 0) {  // a new K chunk starts in accumulator `buf`: it must have been drained
                        if (!mbar_wait(smem_u32(&s_acc_empty[buf]), ((chunk >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                    }
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(smem_u32(&s_full[s]), ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t base = ring + s * C::STAGE;
                    const uint32_t a_hi = base + 2 * C::W_TILE, a_lo = a_hi + C::A_TILE;
                    const uint32_t d = tmem_base + buf * ACC_STRIDE;
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ++ks) {
                        const uint32_t koff = ks * 32;  // 8 TF32 = 32 bytes along K inside the swizzled row
                        const uint64_t d_a_hi = make_smem_desc<BK>(a_hi + koff);
                        const uint64_t d_a_lo = make_smem_desc<BK>(a_lo + koff);
                        const uint64_t d_w_hi = make_smem_desc<BK>(base + koff);
                        const uint64_t d_w_lo = make_smem_desc<BK>(base + C::W_TILE + koff);
                        umma_tf32(d, d_w_lo, d_a_hi, idesc, (kc | ks) ? 1u : 0u);   // small terms first
                        umma_tf32(d, d_w_hi, d_a_lo, idesc, 1u);
                        umma_tf32(d, d_w_hi, d_a_hi, idesc, 1u);
                    }
                    umma_commit(smem_u32(&s_empty[s]));  // stage reusable once these MMAs have read it
                    if (kc == C::KB_PER_CHUNK - 1 || kb == KB - 1) {
                        umma_commit(smem_u32(&s_acc_full[buf]));  // chunk complete: hand it to the accumulate warps
                        ++chunk;
                    }
                }
                if (!ok) break;
            }
        }
    } else {
        // ================= accumulate + epilogue (warps 2..9) =================
        // The tensor core adds into its FP32 accumulator with truncation, so a long K loop inside
        // TMEM drifts.  Each K chunk is therefore accumulated from zero in TMEM and added to a
        // running sum in registers with round-to-nearest adds.
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;       // even or odd 16-column slices
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        uint32_t chunk = 0;
        const int NC = (KB + C::KB_PER_CHUNK - 1) / C::KB_PER_CHUNK;
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
            const TileInfo t = decode_tile<NMAX>(tile, s_prefix, args);
            const int nsl = t.n_pad >> 4;
            float sum[C::SLICES][16];
#pragma unroll
            for (int i = 0; i < C::SLICES; ++i)
#pragma unroll
                for (int c = 0; c < 16; ++c) sum[i][c] = 0.f;
            bool ok = true;
            for (int ch = 0; ch < NC; ++ch, ++chunk) {
                const uint32_t buf = chunk & 1;
                if (!mbar_wait(smem_u32(&s_acc_full[buf]), (chunk >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int i = 0; i < C::SLICES; ++i) {
                    const int sl = 2 * i + half;
                    if (sl < nsl) {
                        uint32_t r[16];
                        tmem_ld16(tlane + buf * ACC_STRIDE + sl * 16, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 16; ++c) sum[i][c] = __fadd_rn(sum[i][c], __uint_as_float(r[c]));
                    }
                }
                tc_fence_before();
                mbar_arrive(smem_u32(&s_acc_empty[buf]));
            }
            if (!ok) break;
            const int m = t.mb * UMMA_M + q * 32 + lane;
            const bool m_ok = m < args.M_total;
#pragma unroll
            for (int i = 0; i < C::SLICES; ++i) {
                const int sl = 2 * i + half;
                if (sl >= nsl) continue;     // uniform across the warp
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int col = sl * 16 + c;
                    const float v = sum[i][c];
                    if (EPI == EPI_GELU_PAIR) {
                        // even weight row = wi_0 (a), odd row = wi_1 (b) of the same d_ff index
                        const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                        const float a = (lane & 1) ? other : v, b = (lane & 1) ? v : other;
                        float hi, lo;
                        split_tf32(gelu_dot(a, b), hi, lo);
                        if (col < t.n_tok && m_ok) {
                            const size_t o = (size_t)(t.row0 + col) * (size_t)(args.M_total >> 1) + (size_t)(m >> 1);
                            if (lane & 1) args.out_lo[o] = lo; else args.out_hi[o] = hi;
                        }
                    } else {
                        if (col < t.n_tok && m_ok) {
                            const size_t o = (size_t)(t.row0 + col) * (size_t)args.M_total + (size_t)m;
                            args.out_hi[o] = __fadd_rn(args.resid[o], v);
                        }
                    }
                }
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (s_abort) {
        if (threadIdx.x == 0 && args.status) atomicOr(args.status, STATUS_WAIT_TIMEOUT);
        // let bulk copies that were already issued land before the shared memory is released
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// rank-3 map over a plane [slots][rows][K] (K contiguous); box = BK x box_rows x 1
int make_map(CUtensorMap* map, const float* base, uint64_t K, uint64_t rows, uint64_t slots, int bk, int box_rows,
             int rank) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return INFMOE_ERR_CUDA;
    }
    cuuint64_t dims[3] = {K, rows, slots};
    cuuint64_t strides[2] = {K * 4, K * rows * 4};
    cuuint32_t box[3] = {(cuuint32_t)bk, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle swz = bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, (void*)base, dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with %d (K=%llu rows=%llu slots=%llu box=%dx%d)", (int)r,
                  (unsigned long long)K, (unsigned long long)rows, (unsigned long long)slots, bk, box_rows);
        return INFMOE_ERR_CUDA;
    }
    return INFMOE_OK;
}

template <int EPI, int BK, int NMAX, int STAGES>
int launch_one(const GemmArgs& args, long long T, int slots, const float* w_hi, const float* w_lo, const float* a_hi,
               const float* a_lo, int num_ctas, cudaStream_t stream) {
    using C = Cfg<BK, NMAX, STAGES>;
    static_assert(C::SMEM + 8192 <= 227 * 1024, "shared-memory ring too large");
    CUtensorMap m[4];
    INFMOE_TRY(make_map(&m[0], w_hi, args.K, args.M_total, slots, BK, UMMA_M, 3));
    INFMOE_TRY(make_map(&m[1], w_lo, args.K, args.M_total, slots, BK, UMMA_M, 3));
    INFMOE_TRY(make_map(&m[2], a_hi, args.K, (uint64_t)T, 1, BK, 32, 2));
    INFMOE_TRY(make_map(&m[3], a_lo, args.K, (uint64_t)T, 1, BK, 32, 2));
    auto kern = ffn_umma_kernel<EPI, BK, NMAX, STAGES>;
    INFMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    kern<<<num_ctas, GEMM_THREADS, C::SMEM, stream>>>(m[0], m[1], m[2], m[3], args);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

}  // namespace

bool ffn_umma_supported(int D, int F, int E) {
    return D % 4 == 0 && F % 4 == 0 && D >= 8 && F >= 8 && E <= MAX_EXPERTS;
}

// Grouped FFN over experts [e_begin, e_end); T rows in expert-contiguous order.
//   h_hi/h_lo [T][D], g_hi/g_lo [T][F] (scratch), routed [T][D], post [T][D]
//   w01 planes [slots][2F][D]: row 2f = wi_0[f], row 2f+1 = wi_1[f];  wo planes [slots][D][F]
int launch_ffn_umma(long long T, int D, int F, int E, int e_begin, int e_end, const int* offset,
                    const int* slot_of_expert, int slots, const float* h_hi, const float* h_lo, const float* w01_hi,
                    const float* w01_lo, const float* wo_hi, const float* wo_lo, const float* routed, float* g_hi,
                    float* g_lo, float* post, int* status, int num_sms, cudaStream_t stream, cudaEvent_t mid_event) {
    if (T == 0 || e_begin >= e_end) return INFMOE_OK;
    if (!ffn_umma_supported(D, F, E)) {
        set_error("ffn_umma: unsupported shape D=%d F=%d E=%d", D, F, E);
        return INFMOE_ERR_UNSUPPORTED;
    }
    GemmArgs a1{};
    a1.offset = offset;
    a1.slot_of_expert = slot_of_expert;
    a1.E = E;
    a1.e_begin = e_begin;
    a1.e_end = e_end;
    a1.M_total = 2 * F;
    a1.K = D;
    a1.out_hi = g_hi;
    a1.out_lo = g_lo;
    a1.resid = nullptr;
    a1.status = status;
    static const int prefetch = [] {
        const char* v = getenv("INFMOE_GEMM_PREFETCH");
        return v ? atoi(v) : 0;
    }();
    a1.prefetch = prefetch;
    GemmArgs a2 = a1;
    a2.M_total = D;
    a2.K = F;
    a2.out_hi = post;
    a2.out_lo = nullptr;
    a2.resid = routed;
    // Tile shape: k block (floats), token chunk, pipeline depth.  INFMOE_GEMM_TILE selects another
    // instantiation for tuning runs.
    static const int variant = [] {
        const char* v = getenv("INFMOE_GEMM_TILE");
        return v ? atoi(v) : 0;
    }();
#define INFMOE_LAUNCH_PAIR(BK, NMAX, STAGES)                                                                        \
    do {                                                                                                             \
        INFMOE_TRY((launch_one<EPI_GELU_PAIR, BK, NMAX, STAGES>(a1, T, slots, w01_hi, w01_lo, h_hi, h_lo, num_sms,    \
                                                                stream)));                                           \
        if (mid_event) INFMOE_CUDA_TRY(cudaEventRecord(mid_event, stream));                                          \
        INFMOE_TRY((launch_one<EPI_RESIDUAL, BK, NMAX, STAGES>(a2, T, slots, wo_hi, wo_lo, g_hi, g_lo, num_sms,       \
                                                               stream)));                                            \
    } while (0)
    switch (variant) {
        case 1: INFMOE_LAUNCH_PAIR(32, 192, 2); break;
        case 2: INFMOE_LAUNCH_PAIR(16, 192, 5); break;
        case 3: INFMOE_LAUNCH_PAIR(16, 256, 4); break;
        default: INFMOE_LAUNCH_PAIR(32, 160, 3); break;   // 128-byte rows: fewest TMA requests per byte
    }
#undef INFMOE_LAUNCH_PAIR
    return INFMOE_OK;
}

}  // namespace infmoe
