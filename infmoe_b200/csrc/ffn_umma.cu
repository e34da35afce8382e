// Grouped expert FFN on the Blackwell tensor cores (sm_100a): tcgen05.mma with
// TMEM accumulators and a TMEM A operand, operands staged by TMA, split-operand
// error compensation so the products keep FP32 accuracy.
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
// Split operands.  x = hi + lo with hi = x rounded to TF32 and lo = x - hi (exact).
// w * x = hi(w) hi(x) + lo(w) hi(x) + hi(w) lo(x) + (a term below 2^-22).  The head product runs as
// kind::tf32 MMAs (K = 8 each).  The two correction products are 2^-11 of the result, so their
// operands only need 8 significant bits: they run as kind::f16 MMAs on BF16 copies (K = 16 each,
// twice the work per instruction and per joule).  A k block of 32 therefore costs 4 BF16 + 4 TF32
// MMAs into the same FP32 accumulator instead of 12 TF32 MMAs; measured on B200 the layer output
// stays at 2e-6 relative L2 of the FP64 oracle, and the step is no longer held at the power cap
// (SM clock 1.9 GHz instead of 1.4 GHz under sustained load).
//   * Token operand (N side, read from shared memory by the MMA): the producers of the activations
//     (scatter + LayerNorm, GEMM-1 epilogue) write a head plane (FP32 values rounded to TF32) and a
//     packed BF16 plane (per 32 values: 32 x bf16(head), 32 x bf16(tail)); both are small and reused
//     by every weight tile.
//   * Weight operand (M side): the raw FP32 matrix is streamed from HBM exactly once, from a
//     tile-contiguous copy made at load time (each 128 x 32 tile is 16 KB of consecutive addresses,
//     and a CTA's tiles follow one another).  Four transform warps read each tile from shared memory,
//     split it in registers with integer arithmetic and store head, bf16(tail) and bf16(head) into
//     TMEM (tcgen05.st); the MMAs take their A operand from TMEM.  Weights therefore cost 4 bytes per
//     element in HBM, L2 and shared memory, and the MMA reads only the token tile from shared memory.
//
// Chunked accumulation.  The tensor core adds into its FP32 accumulator with
// truncation, not round-to-nearest: measured on B200, one accumulator carried
// over K = 1024..2048 drifts by about 1.5e-5 relative, and the drift grows
// linearly with the number of MMAs.  So a TMEM accumulator only ever holds the
// sum of one chunk of 8 k blocks (64 MMAs, the first one overwriting; the first
// chunk of a tile is 12 or 16 blocks, see chunk_ends); the accumulate warps add
// each finished chunk into a running sum in registers with round-to-nearest adds.
//
// Two MMA issuers, one accumulator each.  One thread can keep the tensor pipe full only while it does
// nothing but issue; the barrier waits before a k block and the commits after it leave the pipe idle
// (measured with one issuer: ~900 of ~1870 cycles per k block).  Two warps therefore issue alternate
// k blocks: the barrier waits of one overlap the issue of the other.
// MMAs issued by different threads into one accumulator complete correctly but in no defined order
// (checked on B200 with integer-valued operands: no update is lost), and the truncating accumulate
// is not associative, so each issuer owns a TMEM accumulator: the MMAs into one accumulator all
// come from one thread, in k order, and the result does not depend on timing.  The chunk boundaries
// of the two accumulators are half a chunk apart, so while one accumulator is read out the other
// issuer keeps the pipe busy; the same overlap hides the epilogue behind the next tile's MMAs.
//
// Pipeline per CTA (persistent, one CTA per SM, 16 warps in four warpgroups, so that setmaxnreg can move
// registers from the single-thread roles to the warps that hold the running sums: 56 / 168 / 120 per thread):
//   warp 0        TMA producer of the weight ring (W_STAGES x 16 KB, raw FP32)
//   warp 1, 3     MMA issuers for even / odd k blocks into accumulator 0 / 1 (warp 1 also owns the TMEM
//                 allocation); a commit per k block frees the token stage and the TMEM weight buffer,
//                 a commit per chunk hands the issuer's accumulator to the accumulate warps
//   warp 2        TMA producer of the token ring (T_STAGES x two planes)
//   warps 4..11   accumulate + epilogue: tcgen05.ld the chunk (one TMEM lane quarter and every other
//                 16-column slice per warp), add into registers; after the last chunk gelu*dot and its
//                 split (lane pairs exchange a and b by shuffle) or residual add, stores contiguous
//                 over the weight-row index
//   warps 12..15  transform: weight tile shared memory -> registers -> head / packed BF16 -> TMEM
// TMEM columns: accumulators at 0 and 192 (a token chunk has up to 192 tokens), two weight buffers (32 head + 32
// packed columns) at 384 and 448.  Two buffers feed the MMAs as well as three did; the 64 columns went to the
// accumulators, because an expert with more tokens than a chunk holds costs a second pass over its weights, and
// with 128 tokens per expert on average a limit of 160 is exceeded by one expert in a few hundred, which is enough
// to give one rank in four of an expert-parallel run an extra round of tiles.
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
// Same with a suspend-time hint: the thread may sleep in hardware for up to `ns` nanoseconds and is woken when
// the phase completes, instead of polling.  Polling warps take issue slots from the working warps of their
// scheduler: with every waiting role polling, the transform warps ran 2-3x slower than alone.
__device__ __forceinline__ bool mbar_try_wait_sleep(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the wait was abandoned (limit reached here or in another role).
// The slow path is a real function call (about 200 cycles on B200); the common case, a barrier
// that is already complete, is a single inlined try_wait (about 17 cycles).
static __device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               unsigned long long limit_ns) {
    const unsigned long long t0 = global_ns();
    while (true) {
        for (int i = 0; i < 16; ++i)
            if (mbar_try_wait_sleep(bar, parity, 100000u)) return true;   // sleeps, up to 0.1 ms at a time
        if (*abort_flag) return false;
        if (global_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait_limited(bar, parity, abort_flag, WAIT_LIMIT_NS);
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]^T: A is 128 lanes x 8 columns of TF32, B is K-major in shared memory.
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with BF16 operands (K = 16 per instruction): A is 128 lanes x 8 columns holding two BF16 each.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
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

// Stores 32 consecutive TMEM columns of this thread's lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// Register redistribution between warpgroups (four consecutive warps): every warp of the group executes it.
template <int REGS>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS)); }
template <int REGS>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS)); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

constexpr int BK = 32;                     // k block: 32 floats = one 128-byte swizzled row
constexpr int ROW_BYTES = BK * 4;

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzled rows (8-row groups of 1024 bytes).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);    // start address
    d |= (uint64_t)1 << 16;                       // leading byte offset: not used by swizzled K-major layouts
    d |= (uint64_t)((8 * ROW_BYTES) >> 4) << 32;  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                       // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}

// Instruction descriptors: FP32 accumulate, both operands K-major, M = 128, N = n; operand format 2 = TF32
// (kind::tf32), 1 = BF16 (kind::f16).
__device__ __forceinline__ uint32_t make_idesc(int n, uint32_t fmt) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(UMMA_M >> 4) << 24);
}

enum { EPI_GELU_PAIR = 0, EPI_RESIDUAL = 1 };

// Roles by warpgroup (four consecutive warps), so that registers can be moved between them (setmaxnreg): the four
// single-thread roles give most of theirs to the accumulate warps, which hold the running sums of up to 12 slices.
constexpr int W_WARP = 0;                             // TMA producer of the weight ring
constexpr int MMA1_WARP = 1;                          // MMA issuer of the even k blocks; owns the TMEM allocation
constexpr int TOKEN_WARP = 2;                         // TMA producer of the token ring
constexpr int MMA2_WARP = 3;                          // MMA issuer of the odd k blocks
constexpr int EPI_WARP0 = 4;
constexpr int EPI_WARPS = 8;                          // two warps per TMEM lane quarter
constexpr int XF_WARP0 = EPI_WARP0 + EPI_WARPS;
constexpr int XF_WARPS = 4;                           // one transform warp per TMEM lane quarter
constexpr int GEMM_THREADS = (XF_WARP0 + XF_WARPS) * 32;
constexpr int REGS_SINGLE_ROLES = 56, REGS_EPILOGUE = 168, REGS_TRANSFORM = 120;   // per thread, after setmaxnreg
static_assert(4 * 32 * REGS_SINGLE_ROLES + EPI_WARPS * 32 * REGS_EPILOGUE + XF_WARPS * 32 * REGS_TRANSFORM <=
                  GEMM_THREADS * 128, "the roles share the registers the CTA was launched with (128 per thread)");
constexpr int ACC_STRIDE = 192;                       // TMEM columns between the two accumulators
constexpr int WBUF_COL = 2 * ACC_STRIDE;              // first TMEM column of the weight head/tail buffers
constexpr int WBUF_STRIDE = 2 * BK;                   // head (BK columns) then tail (BK columns)
constexpr int WBUFS = 2;                              // TMEM weight head/tail buffers
// A ring of n buffers whose consecutive uses alternate between the two MMA issuers needs one barrier per
// (buffer, issuer) pair, so that each issuer observes every phase of the barriers it waits on: a waiter
// that skips phases of a shared barrier can take a stale completion for its own.
constexpr int barrier_period(int n) { return n % 2 ? 2 * n : n; }
constexpr int PW = barrier_period(WBUFS);
constexpr int TMEM_COLS = 512;
constexpr int CHUNK_BLOCKS = 8;                       // k blocks (of 8 MMAs) one accumulator takes between two drains
constexpr int W_TILE = UMMA_M * ROW_BYTES;            // 16 KB of raw FP32 weights per k block

template <int NMAX, int W_STAGES, int T_STAGES>
struct Cfg {
    static constexpr int A_TILE = NMAX * ROW_BYTES;                 // one plane of the token tile
    static constexpr int A_STAGE = 2 * A_TILE;
    static constexpr int SMEM = W_STAGES * W_TILE + T_STAGES * A_STAGE + 1024;   // + slack for 1024-byte alignment
    static constexpr int PA = barrier_period(T_STAGES);             // barriers of the token ring
    static constexpr int SLICES = (NMAX / 16 + 1) / 2;              // 16-column slices owned by one epilogue thread
    static_assert(NMAX % 16 == 0 && NMAX <= ACC_STRIDE, "token chunk");
    static_assert(A_TILE % 1024 == 0, "tiles must keep 1024-byte alignment");
};

struct GemmArgs {
    const int* offset;          // [E+1] first routed row of each expert
    const int* slot_of_expert;  // expert -> weight slot (NULL: identity)
    int E, e_begin, e_end;      // experts [e_begin, e_end) are processed
    int M_total;                // weight rows: 2 * d_ff (wi_0 / wi_1 rows interleaved) or d_model
    int K;
    float* out_hi;              // GELU_PAIR: g_hi [T][M_total / 2]; RESIDUAL: y [T][M_total]
    float* out_lo;              // GELU_PAIR: g_lo
    const float* resid;         // RESIDUAL: the rows the experts were applied to, indexed like the output: row
                                // out_pos[j] (or j) of x [rows][M_total]; no routed copy of x is needed
    const int* out_pos;         // RESIDUAL: row j is written to row out_pos[j] of y (NULL: row j), i.e. the combine
                                // step moe_expert_gather (plugin/cuda/moe.cu:89-96) fused into the epilogue
    const float* mix_score;     // RESIDUAL: routed scores for the base_layer output mix (NULL: no mix)
    const unsigned long long* out_row_ptr;   // RESIDUAL: address of output row i (i = out_pos[j] or j) instead of
                                             // y + i * M_total; the rows may live in another GPU's memory
    int* status;
};

// True when k block kb (of KB) of a tile is the last one of a chunk of its accumulator (each accumulator
// takes every other k block).  Chunks are CHUNK_BLOCKS own blocks long, except the first one of a tile, which
// is 12 blocks for the even and 16 for the odd k blocks: the accumulate warps are still busy with the previous
// tile's epilogue when a tile starts, and an accumulator that needs draining before they are back stalls its
// MMA issuer.  The different first lengths also keep the two accumulators half a chunk apart, so that they
// are never drained at the same time.
__device__ __forceinline__ bool chunk_ends(int kb, int KB) {
    const int first = (kb & 1) ? 2 * CHUNK_BLOCKS : CHUNK_BLOCKS + CHUNK_BLOCKS / 2;
    const int done = (kb >> 1) + 1 - first;      // own blocks past the first chunk, counting this one
    return (done >= 0 && done % CHUNK_BLOCKS == 0) || kb + 2 >= KB;
}

// Tensor maps of the two token planes, one per box height 16, 32, ... 160 rows: a tile's load fetches exactly
// the rows its MMAs read (n_pad), not the largest tile's worth.
constexpr int TOKEN_BOXES = 12;
struct TokenMaps {
    CUtensorMap hi[TOKEN_BOXES], pk[TOKEN_BOXES];
};

struct TileInfo {
    int expert, slot, mb, row0, n_tok, n_pad;
};

template <int NMAX>
__device__ __forceinline__ void chunking(int cnt, int& nch, int& csz) {
    nch = (cnt + NMAX - 1) / NMAX;
    csz = nch ? (((cnt + nch - 1) / nch + 15) & ~15) : 0;  // balanced chunks, multiple of 16, <= NMAX
}

// Tiles are listed by expert in order of falling token count (s_order: list position -> expert, s_prefix: first
// tile of each list position), so the long tiles of the busiest experts are handed out first and the short ones
// fill the end of the schedule.
template <int NMAX>
__device__ __forceinline__ TileInfo decode_tile(int tile, const int* s_prefix, const short* s_order, const GemmArgs& a) {
    int lo = 0, hi = a.E - 1;  // last list position with s_prefix[.] <= tile
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    TileInfo t;
    const int ex = s_order[lo];
    t.expert = ex;
    t.slot = a.slot_of_expert ? a.slot_of_expert[ex] : ex;
    const int beg = a.offset[ex], cnt = a.offset[ex + 1] - beg;
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

// Tile of this CTA in round j of the schedule: the CTAs walk the list forwards in even rounds and backwards in odd
// ones, so that over two rounds every CTA gets one tile from each end of a stretch of the (sorted) list.
__device__ __forceinline__ int tile_of_round(int j) {
    const int G = (int)gridDim.x, b = (int)blockIdx.x;
    return j * G + ((j & 1) ? G - 1 - b : b);
}

template <int EPI, int NMAX, int W_STAGES, int T_STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
ffn_umma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ TokenMaps token_maps,
                const GemmArgs args) {
    using C = Cfg<NMAX, W_STAGES, T_STAGES>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_w_full[W_STAGES];    // TMA -> transform
    __shared__ __align__(8) uint64_t s_w_empty[W_STAGES];   // transform -> TMA
    // k block `it` (counted over all tiles of the CTA) uses token stage it % T_STAGES with barrier it % PA, and
    // TMEM weight buffer it % WBUFS with barrier it % PW; it is issued by MMA issuer it & 1
    __shared__ __align__(8) uint64_t s_a_full[C::PA];       // TMA -> MMA: token stage filled
    __shared__ __align__(8) uint64_t s_a_empty[C::PA];      // MMA -> TMA: token stage consumed
    __shared__ __align__(8) uint64_t s_wb_ready[PW];        // transform -> MMA: TMEM weight buffer filled
    __shared__ __align__(8) uint64_t s_wb_free[PW];         // MMA -> transform: TMEM weight buffer consumed
    __shared__ __align__(8) uint64_t s_acc_full[2];         // MMA issuer i -> accumulate warps: chunk of accumulator i done
    __shared__ __align__(8) uint64_t s_acc_empty[2];        // accumulate warps -> MMA issuer i: chunk read out
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_prefix[MAX_EXPERTS + 1];
    __shared__ int s_cnt[MAX_EXPERTS];
    __shared__ short s_order[MAX_EXPERTS];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t w_ring = ring, a_ring = ring + W_STAGES * W_TILE;
    const int MB = (args.M_total + UMMA_M - 1) / UMMA_M;
    const int KB = (args.K + BK - 1) / BK;

    // ---- tile schedule: experts by falling token count, exclusive prefix of their tiles ---------
    for (int e = threadIdx.x; e < args.E; e += GEMM_THREADS)
        s_cnt[e] = (e >= args.e_begin && e < args.e_end) ? args.offset[e + 1] - args.offset[e] : 0;
    __syncthreads();
    for (int e = threadIdx.x; e < args.E; e += GEMM_THREADS) {
        const int c = s_cnt[e];
        int rank = 0;   // experts that come before e: more tokens, or as many and a lower index
        for (int o = 0; o < args.E; ++o) {
            const int co = s_cnt[o];
            rank += (co > c || (co == c && o < e)) ? 1 : 0;
        }
        s_order[rank] = (short)e;
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int e0 = 0; e0 < args.E; e0 += 32) {
            const int e = e0 + lane;   // list position
            int nt = 0;
            if (e < args.E) {
                int nch, csz;
                chunking<NMAX>(s_cnt[s_order[e]], nch, csz);
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
        for (int s = 0; s < W_STAGES; ++s) {
            mbar_init(smem_u32(&s_w_full[s]), 1);
            mbar_init(smem_u32(&s_w_empty[s]), XF_WARPS * 32);
        }
        for (int s = 0; s < C::PA; ++s) {
            mbar_init(smem_u32(&s_a_full[s]), 1);
            mbar_init(smem_u32(&s_a_empty[s]), 1);
        }
        for (int s = 0; s < PW; ++s) {
            mbar_init(smem_u32(&s_wb_ready[s]), XF_WARPS * 32);
            mbar_init(smem_u32(&s_wb_free[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&s_acc_full[b]), 1);
            mbar_init(smem_u32(&s_acc_empty[b]), EPI_WARPS * 32);
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA1_WARP) {
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

    if (warp < EPI_WARP0) {
    setmaxnreg_dec<REGS_SINGLE_ROLES>();   // warps 0..3: one thread each does the work; the registers go to the others
    if (warp == W_WARP) {
        // ================= TMA producer, weights =================
        // Runs up to W_STAGES k blocks ahead of the transform warps, independently of the token ring.
        if (lane == 0) {
            uint32_t it = 0;
            for (int round = 0, tile; (tile = tile_of_round(round)) < total_tiles && !*abort_flag; ++round) {
                const TileInfo t = decode_tile<NMAX>(tile, s_prefix, s_order, args);
                bool ok = true;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % W_STAGES;
                    if (!mbar_wait(smem_u32(&s_w_empty[s]), ((it / W_STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&s_w_full[s]);
                    mbar_expect_tx(bar, W_TILE);
                    tma_load_2d(w_ring + s * W_TILE, &map_w, bar, 0, ((t.slot * MB + t.mb) * KB + kb) * UMMA_M);
                }
                if (!ok) break;
            }
        }
    } else if (warp == TOKEN_WARP) {
        // ================= TMA producer, tokens (head and tail planes) =================
        if (lane == 0) {
            uint32_t it = 0;
            for (int round = 0, tile; (tile = tile_of_round(round)) < total_tiles && !*abort_flag; ++round) {
                const TileInfo t = decode_tile<NMAX>(tile, s_prefix, s_order, args);
                // one box of n_pad rows per plane (rows past the chunk's tokens belong to the next expert or are
                // zero-filled past the end; they only feed accumulator columns that are never stored)
                const CUtensorMap* map_hi = &token_maps.hi[(t.n_pad >> 4) - 1];
                const CUtensorMap* map_pk = &token_maps.pk[(t.n_pad >> 4) - 1];
                const uint32_t a_bytes = 2 * t.n_pad * ROW_BYTES;
                bool ok = true;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % T_STAGES;
                    if (it >= (uint32_t)T_STAGES) {   // the stage's previous k block must have been consumed
                        const uint32_t prev = it - T_STAGES;
                        if (!mbar_wait(smem_u32(&s_a_empty[prev % C::PA]), (prev / C::PA) & 1, abort_flag)) { ok = false; break; }
                    }
                    const uint32_t bar = smem_u32(&s_a_full[it % C::PA]);
                    mbar_expect_tx(bar, a_bytes);
                    // head plane: 32 floats of the row; packed plane: the row's 64 BF16 of this k block
                    const uint32_t a_hi = a_ring + s * C::A_STAGE, a_pk = a_hi + C::A_TILE;
                    tma_load_2d(a_hi, map_hi, bar, kb * BK, t.row0);
                    tma_load_2d(a_pk, map_pk, bar, kb * 2 * BK, t.row0);
                }
                if (!ok) break;
            }
        }
    } else if (warp == MMA1_WARP || warp == MMA2_WARP) {
        // ================= MMA issuers =================
        // Warp 1 issues the even k blocks (counted over all tiles of the CTA) into accumulator 0, the
        // other warp the odd ones into accumulator 1.  The whole warp runs the loop so that addresses
        // and descriptors stay warp-uniform; one lane issues the tcgen05 instructions.
        const uint32_t mine = warp == MMA1_WARP ? 0u : 1u;
        const bool leader = lane == 0;
        const uint32_t d = tmem_base + mine * ACC_STRIDE;
        const uint32_t acc_empty = smem_u32(&s_acc_empty[mine]), acc_full = smem_u32(&s_acc_full[mine]);
        uint32_t it = 0, rounds = 0;   // rounds: hand-overs of this issuer's accumulator so far
        for (int round = 0, tile; (tile = tile_of_round(round)) < total_tiles && !*abort_flag; ++round) {
            const TileInfo t = decode_tile<NMAX>(tile, s_prefix, s_order, args);
            const uint32_t idesc_tf32 = make_idesc(t.n_pad, 2u), idesc_bf16 = make_idesc(t.n_pad, 1u);
            bool ok = true, entered = false;   // entered: the accumulator has been taken over for the current chunk
            for (int kb = 0; kb < KB; ++kb, ++it) {
                if ((it & 1u) != mine) continue;
                if (!entered) {  // the accumulator's previous chunk must have been read out
                    if (!mbar_wait(acc_empty, rounds & 1, abort_flag)) { ok = false; break; }
                }
                const int s = it % T_STAGES;
                const uint32_t wb = it % WBUFS;
                if (!mbar_wait(smem_u32(&s_a_full[it % C::PA]), (it / C::PA) & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(smem_u32(&s_wb_ready[it % PW]), (it / PW) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const bool first = !entered;       // first k block of a chunk: its first MMA overwrites the accumulator
                entered = true;
                if (leader) {
                    const uint32_t a_hi = a_ring + s * C::A_STAGE, a_pk = a_hi + C::A_TILE;
                    const uint32_t w_hi = tmem_base + WBUF_COL + wb * WBUF_STRIDE, w_pk = w_hi + BK;
                    const uint64_t d_a_hi = make_smem_desc(a_hi), d_a_pk = make_smem_desc(a_pk);
                    // corrections first (small terms), in BF16 with K = 16 per instruction: tail(w) x head(x) and
                    // head(w) x tail(x).  In the packed token row bf16(head) is bytes 0..63, bf16(tail) bytes 64..127;
                    // 32 bytes along K = 2 units of the descriptor address.
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j) {
                        umma_bf16_ts(d, w_pk + 8 * j, d_a_pk + 2 * j, idesc_bf16, (first && j == 0) ? 0u : 1u);
                        umma_bf16_ts(d, w_pk + 16 + 8 * j, d_a_pk + 4 + 2 * j, idesc_bf16, 1u);
                    }
                    // head(w) x head(x) in TF32, K = 8 per instruction
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ++ks) umma_tf32_ts(d, w_hi + ks * 8, d_a_hi + 2 * ks, idesc_tf32, 1u);
                    // token stage and TMEM weight buffer are free once these MMAs have completed
                    umma_commit(smem_u32(&s_a_empty[it % C::PA]));
                    umma_commit(smem_u32(&s_wb_free[it % PW]));
                    if (chunk_ends(kb, KB)) umma_commit(acc_full);
                }
                if (chunk_ends(kb, KB)) {
                    ++rounds;
                    entered = false;
                }
            }
            if (!ok) break;
        }
    }
    } else if (warp < XF_WARP0) {
        setmaxnreg_inc<REGS_EPILOGUE>();   // takes what the other warpgroups gave back
        // ================= accumulate + epilogue (warps 4..11) =================
        // Each chunk is accumulated in TMEM (its first MMA overwrites the accumulator) and added
        // here, with round-to-nearest adds, to a running sum in registers; then the accumulator
        // goes back to its MMA issuer.  The chunks of the two accumulators are taken in the fixed
        // order of their last k block.
        const int q = warp & 3;                 // TMEM lane quarter this warp may access
        const int half = (warp - EPI_WARP0) >> 2;   // even or odd 16-column slices
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        // first hand-over: both accumulators are free
        mbar_arrive(smem_u32(&s_acc_empty[0]));
        mbar_arrive(smem_u32(&s_acc_empty[1]));
        uint32_t it = 0, rounds0 = 0, rounds1 = 0;      // rounds: hand-overs of accumulator 0 / 1 so far
        for (int round = 0, tile; (tile = tile_of_round(round)) < total_tiles && !*abort_flag; ++round) {
            const TileInfo t = decode_tile<NMAX>(tile, s_prefix, s_order, args);
            const int nsl = t.n_pad >> 4;
            float sum[C::SLICES][16];
#pragma unroll
            for (int i = 0; i < C::SLICES; ++i)
#pragma unroll
                for (int c = 0; c < 16; ++c) sum[i][c] = 0.f;
            bool ok = true;
            for (int kb = 0; kb < KB; ++kb, ++it) {
                if (!chunk_ends(kb, KB)) continue;
                const uint32_t buf = it & 1;
                const uint32_t par = (buf ? rounds1 : rounds0) & 1;
                if (buf) ++rounds1; else ++rounds0;
                // the warp stays converged for the .aligned TMEM instructions, also when a wait is abandoned
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_acc_full[buf]), par, abort_flag))) { ok = false; break; }
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
                // RESIDUAL: output row and mix coefficient of the slice's 16 token columns, one column per lane
                // (lanes 16..31 repeat them), handed out by shuffle below
                int lane_row = 0;
                float lane_alpha = 0.f;
                unsigned long long lane_ptr = 0;
                if (EPI == EPI_RESIDUAL) {
                    const int lc = sl * 16 + (lane & 15);
                    const int r = t.row0 + lc;
                    lane_row = (lc < t.n_tok && args.out_pos) ? args.out_pos[r] : r;
                    if (args.mix_score && lc < t.n_tok) lane_alpha = mix_alpha(args.mix_score[r]);
                    if (lc < t.n_tok)
                        lane_ptr = args.out_row_ptr
                                       ? args.out_row_ptr[lane_row]
                                       : (unsigned long long)(args.out_hi + (size_t)lane_row * (size_t)args.M_total);
                }
                if (EPI == EPI_GELU_PAIR) {
                    // Even weight row = wi_0 (a), odd row = wi_1 (b) of the same d_ff index f, so a lane pair holds
                    // (a, b) of f for all 16 token columns.  The pair splits the columns: the even lane takes the
                    // even ones, the odd lane the odd ones; one shuffle per column pair hands each lane the half
                    // it lacks, and every gelu is evaluated once.
                    const int F = args.M_total >> 1, f = m >> 1;
                    const bool odd = lane & 1;
#pragma unroll
                    for (int c = 0; c < 16; c += 2) {
                        const float got = __shfl_xor_sync(0xffffffffu, odd ? sum[i][c] : sum[i][c + 1], 1);
                        const float a = odd ? got : sum[i][c], b = odd ? sum[i][c + 1] : got;
                        const float g = gelu_dot_fast(a, b);
                        const uint32_t hb = (__float_as_uint(g) + 0x1000u) & 0xffffe000u;   // TF32 head, as split_tf32
                        const float hi = __uint_as_float(hb), lo = __fsub_rn(g, hi);
                        const int col = sl * 16 + c + (odd ? 1 : 0);
                        // Packed plane: neighbouring f (lanes two apart, same column) exchange their halves so that
                        // every lane stores one 32-bit word, even f the pair of heads, odd f the pair of tails.
                        const uint32_t hl = pack_bf16x2(hi, lo);
                        const uint32_t nb = __shfl_xor_sync(0xffffffffu, hl, 2);
                        // The packed plane is zero padded to whole groups of 32 (weight rows past the matrix are
                        // zero in the tiled layout, so those values are 0).
                        if (col < t.n_tok) {
                            if (f < F) args.out_hi[(size_t)(t.row0 + col) * (size_t)F + (size_t)f] = hi;
                            if (f < ((F + 31) & ~31)) {
                                uint16_t* gp = reinterpret_cast<uint16_t*>(args.out_lo) +
                                               (size_t)(t.row0 + col) * pack_pitch(F) + (size_t)(f >> 5) * 64 + (f & 31);
                                if (!(f & 1)) *reinterpret_cast<uint32_t*>(gp) = (hl & 0xffffu) | (nb << 16);
                                else *reinterpret_cast<uint32_t*>(gp + 31) = (nb >> 16) | (hl & 0xffff0000u);
                            }
                        }
                    }
                    continue;
                }
                // The residual values of the slice's 16 columns are fetched first, all in flight together: issued
                // one by one between the stores (which may alias them as far as the compiler knows) each would
                // cost a trip to L2 or HBM, 80 in a row per thread, and the next tile's first chunk would wait.
                float xres[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int resid_row = __shfl_sync(0xffffffffu, lane_row, c);
                    xres[c] = (sl * 16 + c < t.n_tok && m_ok)
                                  ? args.resid[(size_t)resid_row * (size_t)args.M_total + (size_t)m] : 0.f;
                }
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int col = sl * 16 + c;
                    const unsigned long long out_row = __shfl_sync(0xffffffffu, lane_ptr, c);
                    const float alpha = __shfl_sync(0xffffffffu, lane_alpha, c);
                    if (col < t.n_tok && m_ok) {
                        const float x = xres[c];
                        float y = __fadd_rn(x, sum[i][c]);
                        if (args.mix_score) y = mix_value(alpha, 1.0f - alpha, y, x);
                        reinterpret_cast<float*>(out_row)[m] = y;
                    }
                }
            }
        }
    } else {
        // ================= transform =================
        setmaxnreg_dec<REGS_TRANSFORM>();
        // Thread = one weight row of the tile.  The row's 128 bytes are read from the swizzled
        // shared-memory tile (16-byte chunk c of row r sits at chunk c ^ (r & 7)), split into
        // TF32 head and tail, and stored into this thread's TMEM lane.
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16) + WBUF_COL;
        const uint8_t* w_ring_ptr = smem_raw + (w_ring - smem_u32(smem_raw));
        // Software pipeline: the tile of k block it + 1 is read from shared memory and split (and its slot
        // handed back to the producer) right after the buffer of k block `it` has been handed to the MMA
        // issuers, i.e. while this warp would otherwise wait for the next TMEM buffer to come free.
        int my_tiles = 0;
        for (int round = 0; tile_of_round(round) < total_tiles; ++round) ++my_tiles;
        const uint32_t total_it = (uint32_t)my_tiles * (uint32_t)KB;
        float4 v[8];
        bool ok = total_it > 0 && !*abort_flag;
        auto fetch = [&](uint32_t it) -> bool {
            const int s = it % W_STAGES;
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_w_full[s]), (it / W_STAGES) & 1, abort_flag))) return false;
            const uint8_t* row = w_ring_ptr + s * W_TILE + r * ROW_BYTES;
#pragma unroll
            for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const float4*>(row + ((c ^ (r & 7)) << 4));
            mbar_arrive(smem_u32(&s_w_empty[s]));   // the tile is in registers: its slot can be refilled
            return true;
        };
        // hi: the 32 values rounded to TF32; pk: 16 words of bf16(tail) pairs, then 16 words of bf16(head) pairs.
        // Integer arithmetic only (the conversion instructions are several times slower than the ALU here):
        // head = (bits + 0x1000) & ~0x1fff is cvt.rna.tf32 for every finite value; the BF16 halves keep the upper
        // 16 bits of head and tail (the head has 11 significant bits, so its BF16 copy drops 3 of them; the
        // error this adds to a correction product is below 2^-19 of the full product).
        uint32_t hi[32], pk[32];
        auto split = [&]() {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float x[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
                uint32_t h[4], l[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    h[j] = (__float_as_uint(x[j]) + 0x1000u) & 0xffffe000u;
                    l[j] = __float_as_uint(__fsub_rn(x[j], __uint_as_float(h[j])));
                    hi[4 * c + j] = h[j];
                }
                pk[2 * c] = __byte_perm(l[0], l[1], 0x7632);          // upper halves: l[0] low, l[1] high
                pk[2 * c + 1] = __byte_perm(l[2], l[3], 0x7632);
                pk[16 + 2 * c] = __byte_perm(h[0], h[1], 0x7632);
                pk[16 + 2 * c + 1] = __byte_perm(h[2], h[3], 0x7632);
            }
        };
        if (ok) ok = fetch(0);
        if (ok) split();
        for (uint32_t it = 0; ok && it < total_it; ++it) {
            // the MMAs that read this TMEM buffer WBUFS k blocks ago must be done
            if (it >= (uint32_t)WBUFS) {
                const uint32_t prev = it - WBUFS;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_wb_free[prev % PW]), (prev / PW) & 1, abort_flag))) break;
            }
            tc_fence_after();
            const uint32_t dst = tlane + (it % WBUFS) * WBUF_STRIDE;
            tmem_st32(dst, hi);
            tmem_st32(dst + BK, pk);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(smem_u32(&s_wb_ready[it % PW]));
            // the next tile is read and split while this buffer is already on its way to the MMA issuers and
            // the buffer after it is still being consumed
            if (it + 1 < total_it) {
                ok = fetch(it + 1);
                if (ok) split();
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
    if (warp == MMA1_WARP) {
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

// map over an FP32 plane [slots][rows][K] (K contiguous), or over the packed BF16 plane [rows][K] with K counted
// in BF16 elements; box = 128 bytes x box_rows (x 1), 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, uint64_t K, uint64_t rows, uint64_t slots, int box_rows, int rank,
             bool bf16 = false) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return INFMOE_ERR_CUDA;
    }
    cuuint64_t dims[3] = {K, rows, slots};
    const uint64_t esz = bf16 ? 2 : 4;
    cuuint64_t strides[2] = {K * esz, K * rows * esz};
    cuuint32_t box[3] = {(cuuint32_t)(ROW_BYTES / esz), (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                          (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with %d (K=%llu rows=%llu slots=%llu box=%dx%d)", (int)r,
                  (unsigned long long)K, (unsigned long long)rows, (unsigned long long)slots, BK, box_rows);
        return INFMOE_ERR_CUDA;
    }
    return INFMOE_OK;
}

// The token maps of a call depend only on the two plane pointers, K and the row count, which repeat from call
// to call (same workspace): the last few sets are kept per host thread instead of being encoded again.
int token_maps(TokenMaps* out, const float* a_hi, const float* a_lo, int K, long long T) {
    struct Entry {
        const float *hi = nullptr, *lo = nullptr;
        int K = 0;
        long long T = 0;
        TokenMaps maps;
    };
    static thread_local Entry cache[4];
    static thread_local int next = 0;
    for (const Entry& e : cache)
        if (e.hi == a_hi && e.lo == a_lo && e.K == K && e.T == T) {
            *out = e.maps;
            return INFMOE_OK;
        }
    Entry& e = cache[next];
    next = (next + 1) % 4;
    e.hi = nullptr;   // stays invalid if an encode fails
    for (int b = 0; b < TOKEN_BOXES; ++b) {
        INFMOE_TRY(make_map(&e.maps.hi[b], a_hi, (uint64_t)K, (uint64_t)T, 1, 16 * (b + 1), 2));
        INFMOE_TRY(make_map(&e.maps.pk[b], a_lo, pack_pitch(K), (uint64_t)T, 1, 16 * (b + 1), 2, true));
    }
    e.hi = a_hi;
    e.lo = a_lo;
    e.K = K;
    e.T = T;
    *out = e.maps;
    return INFMOE_OK;
}

template <int EPI, int NMAX, int W_STAGES, int T_STAGES>
int launch_one(const GemmArgs& args, long long T, int slots, const float* w, const float* a_hi, const float* a_lo,
               int num_ctas, cudaStream_t stream) {
    using C = Cfg<NMAX, W_STAGES, T_STAGES>;
    static_assert(C::SMEM + 12288 <= 227 * 1024, "shared-memory rings too large");
    static_assert(NMAX <= 16 * TOKEN_BOXES, "a token tile needs a tensor map of its height");
    CUtensorMap map_w;
    TokenMaps tm;
    // weights: tile-contiguous plane = a [slots * MB * KB * 128][32] matrix, one 16 KB tile per box
    const uint64_t w_rows = (uint64_t)slots * ((args.M_total + UMMA_M - 1) / UMMA_M) * ((args.K + BK - 1) / BK) * UMMA_M;
    INFMOE_TRY(make_map(&map_w, w, BK, w_rows, 1, UMMA_M, 2));
    INFMOE_TRY(token_maps(&tm, a_hi, a_lo, args.K, T));
    auto kern = ffn_umma_kernel<EPI, NMAX, W_STAGES, T_STAGES>;
    INFMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    kern<<<num_ctas, GEMM_THREADS, C::SMEM, stream>>>(map_w, tm, args);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

// One warp waits on a barrier that nothing ever completes, through the same bounded wait the GEMM roles use, with
// a caller-chosen limit: the way to see the expiry path (flag, status bit, orderly return) without a real stall.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int* status, unsigned long long* waited_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int s_abort;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const unsigned long long t0 = global_ns();
    const bool done = mbar_wait_limited(smem_u32(&bar), 0, &s_abort, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!done && s_abort) atomicOr(status, STATUS_WAIT_TIMEOUT);
        *waited_ns = global_ns() - t0;
    }
}

}  // namespace

// Tensor map over a row-major FP32 matrix [rows][K] with boxes of 32 floats x box_rows rows and the 128-byte swizzle
// (for the other kernels of the library; K * 4 and the base address must be multiples of 16 bytes).
int make_f32_row_map(CUtensorMap* map, const void* base, long long K, long long rows, int box_rows) {
    return make_map(map, base, (uint64_t)K, (uint64_t)rows, 1, box_rows, 2);
}

int launch_wait_probe(unsigned long long limit_ns, int* status, unsigned long long* waited_ns, cudaStream_t stream) {
    wait_probe_kernel<<<1, 32, 0, stream>>>(limit_ns, status, waited_ns);
    note_launch();
    INFMOE_CUDA_TRY(cudaGetLastError());
    return INFMOE_OK;
}

bool ffn_umma_supported(int D, int F, int E) {
    return D % 4 == 0 && F % 4 == 0 && D >= 8 && F >= 8 && E <= MAX_EXPERTS;
}

// Grouped FFN over experts [e_begin, e_end); T rows in expert-contiguous order.
//   h_hi/h_lo [T][D], g_hi/g_lo [T][F] (scratch), routed [T][D], post [T][D]
//   w01 [slots] x tiled(2F x D) raw FP32: row 2f = wi_0[f], row 2f+1 = wi_1[f];  wo [slots] x tiled(D x F);
//   tiled = 128 x 32 tiles stored contiguously (launch_retile), so a CTA streams its weights as one
//   sequential run of 16 KB tiles
int launch_ffn_umma(long long T, int D, int F, int E, int e_begin, int e_end, const int* offset,
                    const int* slot_of_expert, int slots, const float* h_hi, const float* h_lo, const float* w01,
                    const float* wo, const float* routed, float* g_hi, float* g_lo, float* post, int* status,
                    int num_sms, cudaStream_t stream, cudaEvent_t mid_event, const int* out_pos,
                    const float* mix_score, const unsigned long long* out_row_ptr) {
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
    GemmArgs a2 = a1;
    a2.M_total = D;
    a2.K = F;
    a2.out_hi = post;
    a2.out_lo = nullptr;
    a2.resid = routed;
    a2.out_pos = out_pos;
    a2.mix_score = mix_score;
    a2.out_row_ptr = out_row_ptr;
    // Shapes: token chunk, weight stages (16 KB each), token stages.  INFMOE_GEMM_TILE selects another instantiation
    // for tuning runs.
    static const int variant = [] {
        const char* v = getenv("INFMOE_GEMM_TILE");
        return v ? atoi(v) : 0;
    }();
#define INFMOE_LAUNCH_PAIR(NMAX, WS, TS)                                                                         \
    do {                                                                                                          \
        INFMOE_TRY((launch_one<EPI_GELU_PAIR, NMAX, WS, TS>(a1, T, slots, w01, h_hi, h_lo, num_sms, stream)));    \
        if (mid_event) INFMOE_CUDA_TRY(cudaEventRecord(mid_event, stream));                                       \
        INFMOE_TRY((launch_one<EPI_RESIDUAL, NMAX, WS, TS>(a2, T, slots, wo, g_hi, g_lo, num_sms, stream)));      \
    } while (0)
    switch (variant) {
        case 1: INFMOE_LAUNCH_PAIR(160, 5, 3); break;
        case 2: INFMOE_LAUNCH_PAIR(144, 4, 4); break;
        default: INFMOE_LAUNCH_PAIR(192, 4, 3); break;
    }
#undef INFMOE_LAUNCH_PAIR
    return INFMOE_OK;
}

}  // namespace infmoe
