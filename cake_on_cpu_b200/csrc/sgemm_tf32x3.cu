// FP32 SGEMM on the 5th-generation tensor cores with split-precision operands
// ("3xTF32"): every FP32 value v is written as hi + lo with hi = tf32(v) and
// lo = tf32(v - hi); A*B is then hi*hi + hi*lo + lo*hi accumulated in FP32 in
// tensor memory.  The dropped lo*lo term and the rounding of lo are of relative
// size 2^-22, the same order as FP32 rounding itself.
//
// Role in the CAKE design.  The reference packs A and B into contiguous
// operation blocks (src/pack_k_first.cpp, src/pack_ob.cpp) and walks CB blocks
// in K-first / M-first / N-first order calling a register-tile outer-product
// microkernel (src/cake_sgemm_k_first.cpp:9-153, src/kernels/haswell/dense.cpp:8).
// Here:
//   * packing     -> one bandwidth-bound pass that splits each operand into its
//                    hi / lo planes (B is transposed on the way so that both
//                    operands are K-major), then TMA boxes staged in a ring of
//                    128-byte-swizzled shared-memory tiles;
//   * CB block    -> a BM x BN tile of C held in tensor memory while K streams
//                    through (K innermost); the schedule is the order in which
//                    the persistent CTAs take tiles;
//   * microkernel -> tcgen05.mma kind::tf32, 128 x BN x 8 per instruction.
//
// Two kernels share this file.  Both: one CTA per SM, warp 0 issues TMA loads, warp 1 issues the MMAs
// and owns the tensor-memory allocation.  The plain kernel has four more warps that drain finished
// accumulators; the chunked kernel has three warp groups, the eight warps of the last two drain accumulators
// (tcgen05.ld) while the MMAs already fill the other accumulator buffer.  Each exists in two forms,
// chosen by the template parameter PAIR: one CTA per 128 x BN tile, or the two CTAs of a cluster on one
// 256 x BN tile (tcgen05 cta_group::2, see Cfg), which is what products with more than 128 rows run.
//
// Accumulation in chunks of K.  The tensor core adds into tensor memory with
// truncation, so the error of one long accumulation grows linearly with K (at
// K = 8192 and uniform(-1, 1) operands about 6e-3 absolute, six times the 1e-3
// that the reference's own checker allows, src/util.cpp:139-169).  A tile's K range
// is therefore cut into chunks (CHUNK_KB slices of 32): each chunk is accumulated
// from zero in one of the two buffers, and the drain warps fold finished chunks
// into a running sum held in registers with round-to-nearest FP32 adds, so only
// the chunk length, not K, sets the truncation error.  The fold overlaps the MMAs
// of the next chunk; the last chunk is added on the way out to global memory.
// Reading an accumulator out of tensor memory while MMAs run is not free: each fold costs the MMAs
// about 1150 cycles (0.6 us, the time of nine of them), whether the loads are 32 or 64 columns wide, one
// or two in flight, bunched or spread over the chunk, so the chunk length trades accuracy for speed.
// Largest absolute error against float64 (64 sampled rows, uniform(-1, 1)) and time per product in a loop
// of 40 products (6 at 16384^3) on pairs of SMs, for one unbroken accumulation / chunks of 1024 / 512 /
// 256 of K:
//    4096^3: 3.0e-3 / 7.8e-4 / 3.3e-4 / 1.9e-4,   0.526 / 0.539 / 0.554 / 0.614 ms
//    8192^3: 8.3e-3 / 1.1e-3 / 5.6e-4 / 2.6e-4,   4.37-4.67 / 4.55-4.65 / 4.86-4.99 / 4.99-5.14 ms (power-capped)
//   16384^3: 2.6e-2 / 1.5e-3 / 7.5e-4 / 4.2e-4,   38.0-38.3 / 38.1-39.9 / 40.3-40.5 / 44.0-44.5 ms
// (the exact-FP32 FFMA kernel: 2.3e-4 at 3000^3, 3.7e-4 at 4096^3 and, against the reference's own result,
// 9.5e-4 at 8192^3).  Rule: chunks of 1024 of K at every K: 0 to 4 % of the time for an error that no
// longer grows with K (normalised by the row and column norms: 3e-7 instead of 2.3e-6 at 8192^3, against
// a gate of 1e-5 that an unbroken accumulation would approach at K = 32768).  The "chunk_kb" option sets
// another length; a value of at least K / 32 means one unbroken accumulation (the plain kernel).
#include <cuda.h>

#include <stdlib.h>
#include <string.h>
#include <atomic>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "tcgen05.cuh"

namespace cakeb200 {
bool tune_lookup(int M, int N, int K, int sched, int* tile_n, int* band, int* k_pieces, int* cluster);  // tune.cpp

namespace {

using namespace ptx;

constexpr int BM = 128;          // rows of C per tile = TMEM lanes
constexpr int BK = 32;           // K per pipeline stage: 32 floats = one 128-byte swizzle row
constexpr int UMMA_K = 8;        // K of one tcgen05.mma kind::tf32
constexpr int NUM_THREADS = 192;           // plain kernel: TMA warp, MMA warp, four drain warps
constexpr int CHUNKED_THREADS = 384;   // chunked kernel: warp group 0 = TMA warp, MMA warp, two idle warps; groups 1 and 2 = drain warps
constexpr int EPI_WARPS = 8;      // two per quarter of the tensor-memory lanes, each taking half of the columns
constexpr int CHUNK_KB = 32;      // default chunk: 32 slices of 32 = 1024 of K

// PAIR: two CTAs of a cluster (the two SMs of one processor pair) work on one 256 x BN tile of C with
// tcgen05.mma.cta_group::2.  Each CTA stages its 128 rows of A and its half of the tile's BN rows of B^T; the
// MMAs, issued by the even CTA, read both halves of B (the other CTA's half comes over the link between
// the two SMs) and write 128 accumulator rows into each CTA's tensor memory.  Per MMA an SM then reads
// half as much of B from its shared memory and a pipeline stage shrinks from 96 KB to 64 KB (BN = 256),
// which takes the 3xTF32 loop (three MMAs per 8 of K, all reading shared memory) off the shared-memory
// bandwidth limit of the single-CTA form: 8192^3 kernel 4.12 -> 3.64 ms.
// Hand-overs in a pair: the stage-full barriers are the leader's (armed for the bytes of both CTAs, both
// CTAs' loads count on them); stage-empty and accumulator-full live in each CTA and the MMA commit arrives
// on both copies; accumulator-empty is the leader's and the drain warps of both CTAs arrive on it.
template <int BN, bool PAIR>
struct Cfg {
    static constexpr int B_ROWS = PAIR ? BN / 2 : BN;   // rows of B^T staged by one CTA
    static constexpr int A_BYTES = BM * BK * 4;       // one plane of A per stage
    static constexpr int B_BYTES = B_ROWS * BK * 4;   // one plane of B per stage
    static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    static constexpr int STAGES = STAGE_BYTES > 64 * 1024 ? 2 : (STAGE_BYTES > 48 * 1024 ? 3 : 4);
    static constexpr int TILE_M = PAIR ? 2 * BM : BM;   // rows of C per tile
    static constexpr int TMEM_COLS = 2 * BN;      // two accumulator buffers
    static constexpr int EPI_BYTES = 4 * 32 * 32 * 4;          // plain kernel: one 32 x 32 patch per drain warp
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + EPI_BYTES;
    static constexpr int SMEM_BYTES_CHUNKED = SMEM_BYTES + (EPI_WARPS - 4) * 32 * 32 * 4;  // eight patches
};

// Work of one unit (a CTA, or a pair of CTAs): first whole tiles taken round-robin (tile = unit + i * units
// for tiles below dp_tiles), then the K-range pieces listed for it in `units`.  A piece
// that covers only part of K stores its accumulator in a slot of `partials`; a separate
// kernel adds the slots of each tile up in a fixed order.
struct Tf32x3Args {
    float* C;
    float* partials;         // [slot][BM x BN]; in a pair the odd CTA's halves follow at slot + slot_count
    int slot_count;
    const int4* units;       // {tile, first k-block, end k-block, slot or -1 = whole K, store to C}
    const int* cta_begin;    // pieces of unit b are [cta_begin[b], cta_begin[b + 1])
    int dp_tiles;
    int M, N, K;
    int ldc;
    int tiles_m, tiles_n;
    int kblocks;             // 32-deep slices of K of this launch
    int kb_first;            // first slice (a deep product is run as several launches over ranges of K)
    unsigned drain_backoff;  // ns the drain warps sleep between polls for the next accumulator
    int chunk_kb;            // slices of 32 accumulated in tensor memory before they are folded into the running sum
    int order, band;         // tile walk, see tile_coords
    int accumulate;          // for tiles stored straight to C
    int out_p;               // > 0: N axis is (image, position), see GemmProblem::out_p
    long long out_image_stride;
    const float* bias;       // length N, added to every row (nullptr: none)
    int* status_word;
};

// Timeline of CTA 0 (diagnostic build only, -DCAKEB200_ROLE_TIMERS): nanosecond stamps in status_word[16 + 2 * slot].
#ifdef CAKEB200_ROLE_TIMERS
#define STAMP(slot) do { if (blockIdx.x == 0) ((unsigned long long*) (args.status_word + 16))[slot] = global_ns(); } while (0)
#define STAMP_CYCLES(slot) do { if (blockIdx.x == 0) ((unsigned long long*) (args.status_word + 16))[slot] = (unsigned long long) clock64(); } while (0)
#else
#define STAMP(slot)
#define STAMP_CYCLES(slot)
#endif

struct WorkPiece {
    int tile, kb0, kb1, slot;
};

// The it-th piece of this CTA; every role of the CTA walks the same sequence.
__device__ __forceinline__ bool work_piece(const Tf32x3Args& a, int it, WorkPiece& w, int b, int g) {
    const int whole = (b < a.dp_tiles) ? (a.dp_tiles - b + g - 1) / g : 0;
    if (it < whole) {
        w.tile = b + it * g; w.kb0 = a.kb_first; w.kb1 = a.kb_first + a.kblocks; w.slot = -1;
        return true;
    }
    if (a.units == nullptr) return false;
    const int u = a.cta_begin[b] + (it - whole);
    if (u >= a.cta_begin[b + 1]) return false;
    const int4 p = a.units[u];
    w.tile = p.x; w.kb0 = p.y; w.kb1 = p.z; w.slot = p.w;
    return true;
}

// Accumulator hand-overs of one piece: its K range in chunks (an empty range still hands over once, zeros).
__device__ __forceinline__ int piece_chunks(const WorkPiece& w, int chunk_kb) {
    const int n = w.kb1 - w.kb0;
    return n <= 0 ? 1 : (n + chunk_kb - 1) / chunk_kb;
}

// ------------------------------------------------------------------ the kernel

// The plain kernel: every tile's (or piece's) K range is one unbroken accumulation in tensor memory.
// Four drain warps, no running sums, 192 threads.  It is what runs when no K range is longer than a
// chunk (K up to 1024 under the rule, K pieces of a deep product with few tiles, or on request).
template <int BN, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sgemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                    const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                    const Tf32x3Args args) {
    using C_ = Cfg<BN, PAIR>;
    constexpr int STAGES = C_::STAGES;
    extern __shared__ uint8_t smem_raw[];
    // swizzled tiles need 1024-byte alignment
    uint8_t* tiles = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint64_t* bars = (uint64_t*) (tiles + STAGES * C_::STAGE_BYTES);
    // bars[0..S): full, [S..2S): empty, [2S..2S+2): accumulator full, [2S+2..2S+4): accumulator empty
    uint32_t* tmem_slot = (uint32_t*) (bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // within the pair; rank 0 ("leader") issues the MMAs
    // position among the units that take tiles: CTAs, or pairs of CTAs
    const int cta = PAIR ? (int) blockIdx.x >> 1 : (int) blockIdx.x, ctas = PAIR ? (int) gridDim.x >> 1 : (int) gridDim.x;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), PAIR ? 8 : 4);  // one arrival per drain warp (of both CTAs of a pair)
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x == 0) STAMP(0);
    if (warp == 1) tmem_alloc<PAIR>(smem_u32(tmem_slot), (uint32_t) C_::TMEM_COLS);  // belongs to the MMA warp (of both CTAs of a pair)
    tcgen05_fence_before();
    sync_all_t<PAIR>();  // in a pair: both CTAs' barriers exist before anything arrives on them
    tcgen05_fence_after();
    if (threadIdx.x == 0) STAMP(1);
    const uint32_t tmem_base = *tmem_slot;

    WorkPiece w;

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int it = 0; ok && work_piece(args, it, w, cta, ctas); it++) {
                int tm, tn;
                tile_coords(w.tile, args.tiles_m, args.tiles_n, args.order, args.band, tm, tn);
                const int a_row = tm * C_::TILE_M + (int) rank * BM, b_row = tn * BN + (int) rank * C_::B_ROWS;
                for (int kb = w.kb0; kb < w.kb1; kb++) {
                    ok = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, args.status_word, 100 + stage);
                    if (!ok) break;
                    const uint32_t base = smem_u32(tiles + stage * C_::STAGE_BYTES);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), (PAIR ? 2 : 1) * C_::STAGE_BYTES);
                    tma_load_2d_t<PAIR>(base, &map_a_hi, kb * BK, a_row, full_bar(stage));
                    tma_load_2d_t<PAIR>(base + C_::A_BYTES, &map_a_lo, kb * BK, a_row, full_bar(stage));
                    tma_load_2d_t<PAIR>(base + 2 * C_::A_BYTES, &map_b_hi, kb * BK, b_row, full_bar(stage));
                    tma_load_2d_t<PAIR>(base + 2 * C_::A_BYTES + C_::B_BYTES, &map_b_lo, kb * BK, b_row, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // Gave up: let the loads already issued land before the CTA goes away.
                // A stage's loads have landed once its full barrier completed the phase
                // the producer last armed; poll each briefly (bounded).
                const unsigned long long t0 = global_ns();
                if (rank == 0) {
                    for (int s = 0; s < STAGES; s++) {
                        const uint32_t armed = (s < stage) ? phase : (phase ^ 1);
                        while (!mbar_try_wait(full_bar(s), armed) && (long long) (global_ns() - t0) < 20000000LL) {}
                    }
                } else {
                    // the odd CTA of a pair has no barrier of its own to poll: a fixed margin (loads take microseconds)
                    while ((long long) (global_ns() - t0) < 200000LL) __nanosleep(1000);
                }
            }
        }
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_tf32(C_::TILE_M, BN);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (; ok && work_piece(args, local, w, cta, ctas); local++) {
                const int kb0 = w.kb0, kb1 = w.kb1;
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                ok = mbar_wait(acc_empty_bar(buf), acc_phase ^ 1, abort_flag, args.status_word, 200 + buf);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t) (buf * BN);
                uint32_t accumulate = 0;
                for (int kb = kb0; kb < kb1; kb++) {
                    ok = mbar_wait(full_bar(stage), phase, abort_flag, args.status_word, 300 + stage);
                    if (!ok) break;
                    if (local == 0 && kb == kb0) { STAMP(2); STAMP_CYCLES(9); }
                    tcgen05_fence_after();
                    const uint32_t base = smem_u32(tiles + stage * C_::STAGE_BYTES);
                    const uint64_t a_hi = make_kmajor_sw128_desc(base);
                    const uint64_t a_lo = make_kmajor_sw128_desc(base + C_::A_BYTES);
                    const uint64_t b_hi = make_kmajor_sw128_desc(base + 2 * C_::A_BYTES);
                    const uint64_t b_lo = make_kmajor_sw128_desc(base + 2 * C_::A_BYTES + C_::B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        // advance 8 floats = 32 bytes inside the 128-byte swizzle row (16-byte units)
                        const uint64_t adv = (uint64_t) (k * UMMA_K * 4 >> 4);
                        umma_tf32_t<PAIR>(d_tmem, a_lo + adv, b_hi + adv, idesc, accumulate);
                        umma_tf32_t<PAIR>(d_tmem, a_hi + adv, b_lo + adv, idesc, 1);
                        umma_tf32_t<PAIR>(d_tmem, a_hi + adv, b_hi + adv, idesc, 1);
                        accumulate = 1;
                    }
                    umma_commit_t<PAIR>(empty_bar(stage));  // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_t<PAIR>(acc_full_bar(buf));  // accumulator complete
                STAMP(3); STAMP_CYCLES(10);
            }
        }
    } else {
        // ----------------------------------------------------------- epilogue
        // tcgen05.ld hands each thread one row of the accumulator (32 columns per load), so
        // storing from those registers would touch 32 different rows per instruction.  Every
        // 32 x 32 chunk therefore goes through a swizzled shared-memory patch of the warp and
        // comes back with eight lanes per row: a store instruction then covers 4 rows x 128
        // contiguous bytes.
        const int quarter = warp & 3;  // a warp may only touch TMEM lanes [32*(warp%4), +32)
        const uint32_t patch = smem_u32(tiles + STAGES * C_::STAGE_BYTES + 256) + (uint32_t) quarter * 4096u;
        const int sub_r = lane >> 3, sub_c = lane & 7;
        const bool c_vec = (args.ldc % 4 == 0) && (((uintptr_t) args.C) % 16 == 0);
        const bool p_vec = (args.out_p % 4 == 0) && (args.out_image_stride % 4 == 0) && (((uintptr_t) args.C) % 16 == 0);
        int local = 0;
        bool ok = true;
        for (; ok && work_piece(args, local, w, cta, ctas); local++) {
            int tm, tn;
            tile_coords(w.tile, args.tiles_m, args.tiles_n, args.order, args.band, tm, tn);
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            ok = mbar_wait(acc_full_bar(buf), acc_phase, abort_flag, args.status_word, 400 + buf);
            ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below need the whole warp
            if (!ok) break;
            if (warp == 2 && lane == 0) STAMP(4);
            tcgen05_fence_after();
            const bool empty_range = w.kb0 >= w.kb1;  // a piece with no K range contributes zeros
            const uint32_t t_addr = tmem_base + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (buf * BN);
            const int row0 = tm * C_::TILE_M + (int) rank * BM + quarter * 32;
            // a piece of K: the whole accumulator goes to its slot, unclipped (rows and columns
            // beyond the matrix are zeros computed from zero-filled operand tiles)
            float* slot = (w.slot >= 0) ? args.partials + ((long long) (w.slot + (int) rank * args.slot_count) * BM + quarter * 32) * BN : nullptr;
            float v[32];
            if (!empty_range) {
                tmem_ld32(t_addr, v);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = 0.0f;
            }
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                if (!empty_range) tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; j++)
                    st_shared_v4(patch + (uint32_t) lane * 128u + (uint32_t) ((j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1],
                                 v[4 * j + 2], v[4 * j + 3]);
                __syncwarp();
                if (!empty_range) {
                    if (c + 1 < BN / 32) {
                        tmem_ld32(t_addr + (uint32_t) ((c + 1) * 32), v);  // lands while this chunk is stored
                    } else {
                        // the accumulator has been read out: hand the buffer back before the stores
                        tcgen05_fence_before();
                        if (lane == 0) mbar_arrive_t<PAIR>(acc_empty_bar(buf));
                    }
                }
                const int col = tn * BN + c * 32 + sub_c * 4;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = i * 4 + sub_r;
                    float4 o = ld_shared_v4(patch + (uint32_t) r * 128u + (uint32_t) ((sub_c ^ (r & 7)) << 4));
                    const int row = row0 + r;
                    if (args.bias != nullptr && slot == nullptr) {
                        if (col < args.N) o.x += __ldg(args.bias + col);
                        if (col + 1 < args.N) o.y += __ldg(args.bias + col + 1);
                        if (col + 2 < args.N) o.z += __ldg(args.bias + col + 2);
                        if (col + 3 < args.N) o.w += __ldg(args.bias + col + 3);
                    }
                    if (slot != nullptr) {
                        *reinterpret_cast<float4*>(slot + (long long) r * BN + c * 32 + sub_c * 4) = o;
                    } else if (row < args.M && col < args.N) {
                        if (args.out_p > 0) {
                            // convolution output: columns are (image, position); rows are output channels
                            const int img = col / args.out_p, pos = col - img * args.out_p;
                            float* dst = args.C + (long long) img * args.out_image_stride + (long long) row * args.out_p + pos;
                            if (p_vec && pos + 4 <= args.out_p && col + 4 <= args.N) {
                                *reinterpret_cast<float4*>(dst) = o;
                            } else {
                                const float e[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    const int cj = col + j;
                                    if (cj < args.N) {
                                        const int im = cj / args.out_p, ps = cj - im * args.out_p;
                                        args.C[(long long) im * args.out_image_stride + (long long) row * args.out_p + ps] = e[j];
                                    }
                                }
                            }
                        } else {
                            float* dst = args.C + (long long) row * args.ldc + col;
                            if (c_vec && col + 4 <= args.N) {
                                if (args.accumulate) {
                                    const float4 old = *reinterpret_cast<const float4*>(dst);
                                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                                }
                                *reinterpret_cast<float4*>(dst) = o;
                            } else {
                                const float e[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                for (int j = 0; j < 4; j++)
                                    if (col + j < args.N) dst[j] = args.accumulate ? dst[j] + e[j] : e[j];
                            }
                        }
                    }
                }
                __syncwarp();  // the patch is rewritten by the next chunk
            }
            if (empty_range) {
                tcgen05_fence_before();
                if (lane == 0) mbar_arrive_t<PAIR>(acc_empty_bar(buf));
            }
        }
    }

    if (lane == 0 && (warp == 2 || warp == 4)) STAMP(5 + (warp == 4));
    if (threadIdx.x == 0) STAMP(7);
    tcgen05_fence_before();
    sync_all_t<PAIR>();  // in a pair: neither CTA frees tensor memory or leaves while the other may still touch it
    if (threadIdx.x == 0) STAMP(8);
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_free<PAIR>(tmem_base, (uint32_t) C_::TMEM_COLS);
    }
}

// The chunked kernel.
template <int BN, bool PAIR>
__global__ void __launch_bounds__(CHUNKED_THREADS, 1)
sgemm_tf32x3_chunked_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                    const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                    const Tf32x3Args args) {
    using C_ = Cfg<BN, PAIR>;
    constexpr int STAGES = C_::STAGES;
    extern __shared__ uint8_t smem_raw[];
    // swizzled tiles need 1024-byte alignment
    uint8_t* tiles = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint64_t* bars = (uint64_t*) (tiles + STAGES * C_::STAGE_BYTES);
    // bars[0..S): full, [S..2S): empty, [2S..2S+2): accumulator full, [2S+2..2S+4): accumulator empty
    uint32_t* tmem_slot = (uint32_t*) (bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // within the pair; rank 0 ("leader") issues the MMAs
    // position among the units that take tiles: CTAs, or pairs of CTAs
    const int cta = PAIR ? (int) blockIdx.x >> 1 : (int) blockIdx.x, ctas = PAIR ? (int) gridDim.x >> 1 : (int) gridDim.x;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), (PAIR ? 2 : 1) * EPI_WARPS);  // one arrival per drain warp (of both CTAs of a pair)
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x == 0) STAMP(0);
    if (warp == 1) tmem_alloc<PAIR>(smem_u32(tmem_slot), (uint32_t) C_::TMEM_COLS);  // belongs to the MMA warp (of both CTAs of a pair)
    tcgen05_fence_before();
    sync_all_t<PAIR>();  // in a pair: both CTAs' barriers exist before anything arrives on them
    tcgen05_fence_after();
    if (threadIdx.x == 0) STAMP(1);
    const uint32_t tmem_base = *tmem_slot;

    WorkPiece w;

    // Registers follow the roles: the drain warps each hold half a row of the running sum (up to 128
    // values) next to a 32-column load, the other warp group needs a handful.  The launch gives every
    // thread 168; group 0 hands most of its share back and groups 1 and 2 take it.
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
        // ------------------------------------------------------- TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int it = 0; ok && work_piece(args, it, w, cta, ctas); it++) {
                int tm, tn;
                tile_coords(w.tile, args.tiles_m, args.tiles_n, args.order, args.band, tm, tn);
                const int a_row = tm * C_::TILE_M + (int) rank * BM, b_row = tn * BN + (int) rank * C_::B_ROWS;
                for (int kb = w.kb0; kb < w.kb1; kb++) {
                    ok = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, args.status_word, 100 + stage);
                    if (!ok) break;
                    const uint32_t base = smem_u32(tiles + stage * C_::STAGE_BYTES);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), (PAIR ? 2 : 1) * C_::STAGE_BYTES);
                    tma_load_2d_t<PAIR>(base, &map_a_hi, kb * BK, a_row, full_bar(stage));
                    tma_load_2d_t<PAIR>(base + C_::A_BYTES, &map_a_lo, kb * BK, a_row, full_bar(stage));
                    tma_load_2d_t<PAIR>(base + 2 * C_::A_BYTES, &map_b_hi, kb * BK, b_row, full_bar(stage));
                    tma_load_2d_t<PAIR>(base + 2 * C_::A_BYTES + C_::B_BYTES, &map_b_lo, kb * BK, b_row, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // Gave up: let the loads already issued land before the CTA goes away.
                // A stage's loads have landed once its full barrier completed the phase
                // the producer last armed; poll each briefly (bounded).
                const unsigned long long t0 = global_ns();
                if (rank == 0) {
                    for (int s = 0; s < STAGES; s++) {
                        const uint32_t armed = (s < stage) ? phase : (phase ^ 1);
                        while (!mbar_try_wait(full_bar(s), armed) && (long long) (global_ns() - t0) < 20000000LL) {}
                    }
                } else {
                    // the odd CTA of a pair has no barrier of its own to poll: a fixed margin (loads take microseconds)
                    while ((long long) (global_ns() - t0) < 200000LL) __nanosleep(1000);
                }
            }
        }
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_tf32(C_::TILE_M, BN);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0, handover = 0;
            bool ok = true;
            for (; ok && work_piece(args, local, w, cta, ctas); local++) {
                const int chunks = piece_chunks(w, args.chunk_kb);
                for (int ci = 0; ok && ci < chunks; ci++, handover++) {
                    const int kb0 = w.kb0 + ci * args.chunk_kb, kb1 = min(w.kb1, kb0 + args.chunk_kb);
                    const int buf = handover & 1;
                    const uint32_t acc_phase = (handover >> 1) & 1;
                    ok = mbar_wait(acc_empty_bar(buf), acc_phase ^ 1, abort_flag, args.status_word, 200 + buf);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t) (buf * BN);
                    uint32_t accumulate = 0;
                    for (int kb = kb0; kb < kb1; kb++) {
                        ok = mbar_wait(full_bar(stage), phase, abort_flag, args.status_word, 300 + stage);
                        if (!ok) break;
                        if (local == 0 && ci == 0 && kb == kb0) { STAMP(2); STAMP_CYCLES(9); }
                        tcgen05_fence_after();
                        const uint32_t base = smem_u32(tiles + stage * C_::STAGE_BYTES);
                        const uint64_t a_hi = make_kmajor_sw128_desc(base);
                        const uint64_t a_lo = make_kmajor_sw128_desc(base + C_::A_BYTES);
                        const uint64_t b_hi = make_kmajor_sw128_desc(base + 2 * C_::A_BYTES);
                        const uint64_t b_lo = make_kmajor_sw128_desc(base + 2 * C_::A_BYTES + C_::B_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; k++) {
                            // advance 8 floats = 32 bytes inside the 128-byte swizzle row (16-byte units)
                            const uint64_t adv = (uint64_t) (k * UMMA_K * 4 >> 4);
                            umma_tf32_t<PAIR>(d_tmem, a_lo + adv, b_hi + adv, idesc, accumulate);
                            umma_tf32_t<PAIR>(d_tmem, a_hi + adv, b_lo + adv, idesc, 1);
                            umma_tf32_t<PAIR>(d_tmem, a_hi + adv, b_hi + adv, idesc, 1);
                            accumulate = 1;
                        }
                        umma_commit_t<PAIR>(empty_bar(stage));  // stage reusable once these MMAs have read it
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
                    if (!ok) break;
                    umma_commit_t<PAIR>(acc_full_bar(buf));  // chunk complete
                    STAMP(3); STAMP_CYCLES(10);
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        // ----------------------------------------------------------- drain warps
        // Eight warps: warp w may only touch tensor-memory lanes [32 * (w % 4), +32), so two warps
        // share each quarter of the rows and take half of the columns each.  A thread owns one
        // row of its half: COLS / 32 loads of 32 columns.  Chunks that are not the last of their
        // piece are folded into `sum`; the last one is added to `sum` and stored.
        // tcgen05.ld hands each thread one row of the accumulator, so storing from those
        // registers would touch 32 different rows per instruction.  Every 32 x 32 block
        // therefore goes through a swizzled shared-memory patch of the warp and comes back with
        // eight lanes per row: a store instruction then covers 4 rows x 128 contiguous bytes.
        constexpr int COLS = BN / 2, LOADS = COLS / 32;
        const int ew = warp - 4;
        const int quarter = warp & 3, half = ew >> 2;
        const uint32_t patch = smem_u32(tiles + STAGES * C_::STAGE_BYTES + 256) + (uint32_t) ew * 4096u;
        const int sub_r = lane >> 3, sub_c = lane & 7;
        const bool c_vec = (args.ldc % 4 == 0) && (((uintptr_t) args.C) % 16 == 0);
        const bool p_vec = (args.out_p % 4 == 0) && (args.out_image_stride % 4 == 0) && (((uintptr_t) args.C) % 16 == 0);
        float sum[COLS];
        int local = 0, handover = 0;
        bool ok = true;
        for (; ok && work_piece(args, local, w, cta, ctas); local++) {
            int tm, tn;
            tile_coords(w.tile, args.tiles_m, args.tiles_n, args.order, args.band, tm, tn);
            const int chunks = piece_chunks(w, args.chunk_kb);
            const bool empty_range = w.kb0 >= w.kb1;  // a piece with no K range contributes zeros
            for (int ci = 0; ok && ci < chunks; ci++, handover++) {
                const int buf = handover & 1;
                const uint32_t acc_phase = (handover >> 1) & 1;
                ok = mbar_wait_for(acc_full_bar(buf), acc_phase, abort_flag, args.status_word, 400 + buf, WAIT_LIMIT_NS, args.drain_backoff);
                ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below need the whole warp
                if (!ok) break;
                if (warp == 4 && lane == 0) STAMP(4);
                tcgen05_fence_after();
                const uint32_t t_addr = tmem_base + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (buf * BN + half * COLS);
                float v[32];
                if (ci + 1 < chunks) {
                    // fold: sum (+)= chunk, round to nearest; 64 columns per load and wait (a tensor-memory
                    // load queues behind the MMAs already issued, so fewer, wider loads shorten the fold)
                    float v2[64];
#pragma unroll
                    for (int c = 0; c < LOADS; c += 2) {
                        tmem_ld64(t_addr + (uint32_t) (c * 32), v2);
                        tmem_ld_wait();
                        if (ci == 0) {
#pragma unroll
                            for (int j = 0; j < 64; j++) sum[c * 32 + j] = v2[j];
                        } else {
#pragma unroll
                            for (int j = 0; j < 64; j++) sum[c * 32 + j] += v2[j];
                        }
                    }
                    tcgen05_fence_before();
                    if (lane == 0) mbar_arrive_t<PAIR>(acc_empty_bar(buf));
                    continue;
                }
                // last chunk of the piece: out it goes
                const int row0 = tm * C_::TILE_M + (int) rank * BM + quarter * 32;
                // a piece of K: the whole accumulator goes to its slot, unclipped (rows and columns
                // beyond the matrix are zeros computed from zero-filled operand tiles)
                float* slot = (w.slot >= 0) ? args.partials + ((long long) (w.slot + (int) rank * args.slot_count) * BM + quarter * 32) * BN + half * COLS : nullptr;
                if (!empty_range) {
                    tmem_ld32(t_addr, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = 0.0f;
                }
#pragma unroll
                for (int c = 0; c < LOADS; c++) {
                    if (!empty_range) tmem_ld_wait();
                    if (ci > 0) {
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] += sum[c * 32 + j];
                    }
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        st_shared_v4(patch + (uint32_t) lane * 128u + (uint32_t) ((j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1],
                                     v[4 * j + 2], v[4 * j + 3]);
                    __syncwarp();
                    if (!empty_range) {
                        if (c + 1 < LOADS) {
                            tmem_ld32(t_addr + (uint32_t) ((c + 1) * 32), v);  // lands while this block is stored
                        } else {
                            // the accumulator has been read out: hand the buffer back before the stores
                            tcgen05_fence_before();
                            if (lane == 0) mbar_arrive_t<PAIR>(acc_empty_bar(buf));
                        }
                    }
                    const int col = tn * BN + half * COLS + c * 32 + sub_c * 4;
                    // not unrolled: the enclosing loop over c is (the running sums are indexed by it), and 32 copies of the
                    // store logic run once per tile, straight through, from a cold instruction cache (measured: the drain
                    // of a tile took 34 us against 8 us in the plain kernel)
#pragma unroll 1
                    for (int i = 0; i < 8; i++) {
                        const int r = i * 4 + sub_r;
                        float4 o = ld_shared_v4(patch + (uint32_t) r * 128u + (uint32_t) ((sub_c ^ (r & 7)) << 4));
                        const int row = row0 + r;
                        if (args.bias != nullptr && slot == nullptr) {
                            if (col < args.N) o.x += __ldg(args.bias + col);
                            if (col + 1 < args.N) o.y += __ldg(args.bias + col + 1);
                            if (col + 2 < args.N) o.z += __ldg(args.bias + col + 2);
                            if (col + 3 < args.N) o.w += __ldg(args.bias + col + 3);
                        }
                        if (slot != nullptr) {
                            *reinterpret_cast<float4*>(slot + (long long) r * BN + c * 32 + sub_c * 4) = o;
                        } else if (row < args.M && col < args.N) {
                            if (args.out_p > 0) {
                                // convolution output: columns are (image, position); rows are output channels
                                const int img = col / args.out_p, pos = col - img * args.out_p;
                                float* dst = args.C + (long long) img * args.out_image_stride + (long long) row * args.out_p + pos;
                                if (p_vec && pos + 4 <= args.out_p && col + 4 <= args.N) {
                                    *reinterpret_cast<float4*>(dst) = o;
                                } else {
                                    const float e[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                    for (int j = 0; j < 4; j++) {
                                        const int cj = col + j;
                                        if (cj < args.N) {
                                            const int im = cj / args.out_p, ps = cj - im * args.out_p;
                                            args.C[(long long) im * args.out_image_stride + (long long) row * args.out_p + ps] = e[j];
                                        }
                                    }
                                }
                            } else {
                                float* dst = args.C + (long long) row * args.ldc + col;
                                if (c_vec && col + 4 <= args.N) {
                                    if (args.accumulate) {
                                        const float4 old = *reinterpret_cast<const float4*>(dst);
                                        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                                    }
                                    *reinterpret_cast<float4*>(dst) = o;
                                } else {
                                    const float e[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                    for (int j = 0; j < 4; j++)
                                        if (col + j < args.N) dst[j] = args.accumulate ? dst[j] + e[j] : e[j];
                                }
                            }
                        }
                    }
                    __syncwarp();  // the patch is rewritten by the next block
                }
                if (empty_range) {
                    tcgen05_fence_before();
                    if (lane == 0) mbar_arrive_t<PAIR>(acc_empty_bar(buf));
                }
            }
        }
    }

    if (lane == 0 && (warp == 2 || warp == 4)) STAMP(5 + (warp == 4));
    if (threadIdx.x == 0) STAMP(7);
    tcgen05_fence_before();
    sync_all_t<PAIR>();  // in a pair: neither CTA frees tensor memory or leaves while the other may still touch it
    if (threadIdx.x == 0) STAMP(8);
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_free<PAIR>(tmem_base, (uint32_t) C_::TMEM_COLS);
    }
}

// ------------------------------------------------------------- operand split


// A (M x K, leading dimension lda) -> hi / lo planes with leading dimension Kp
__global__ void __launch_bounds__(256)
split_rows_kernel(const float* __restrict__ A, float* __restrict__ hi, float* __restrict__ lo, int M, int K, int lda, int Kp) {
    const long long total = (long long) M * Kp;
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long) gridDim.x * blockDim.x) {
        const int m = (int) (i / Kp), k = (int) (i - (long long) m * Kp);
        float h = 0.f, l = 0.f;
        if (k < K) split_tf32(__ldg(A + (long long) m * lda + k), h, l);
        hi[i] = h;
        lo[i] = l;
    }
}

// Same split, four elements per thread: needs K % 4 == 0 (then Kp == K), lda % 4 == 0 and a 16-byte aligned A.
__global__ void __launch_bounds__(256)
split_rows_vec4_kernel(const float4* __restrict__ A, float4* __restrict__ hi, float4* __restrict__ lo, int M, int K4, int lda4) {
    const long long total = (long long) M * K4;
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long) gridDim.x * blockDim.x) {
        const int m = (int) (i / K4), k = (int) (i - (long long) m * K4);
        const float4 v = __ldg(A + (long long) m * lda4 + k);
        float4 h, l;
        split_tf32(v.x, h.x, l.x);
        split_tf32(v.y, h.y, l.y);
        split_tf32(v.z, h.z, l.z);
        split_tf32(v.w, h.w, l.w);
        hi[i] = h;
        lo[i] = l;
    }
}

// B (K x N, leading dimension ldb) -> transposed hi / lo planes (N x Kp): 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float* __restrict__ B, float* __restrict__ hi, float* __restrict__ lo, int K, int N, int ldb, int Kp) {
    __shared__ float t[32][33];
    const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int k = k0 + r, n = n0 + tx;
        t[r][tx] = (k < K && n < N) ? __ldg(B + (long long) k * ldb + n) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int n = n0 + r, k = k0 + tx;
        if (n < N && k < Kp) {
            float h, l;
            split_tf32(t[tx][r], h, l);
            hi[(long long) n * Kp + k] = h;
            lo[(long long) n * Kp + k] = l;
        }
    }
}

// im2col fused with the operand split: the K x N matrix of the convolution-as-GEMM
// route (reference examples/cake_conv.cpp:1178-1213; row k = (cin, hf, wf), column
// n = (image, ho, wo), zero padding) is never materialised; its transposed hi / lo
// planes (N x Kp, k fastest) are written straight from the NCHW input.
__global__ void __launch_bounds__(256)
im2col_split_kernel(const float* __restrict__ in, float* __restrict__ hi, float* __restrict__ lo, int batch, int cin,
                    int H, int W, int hf, int wf, int stride, int pad, int Ho, int Wo, int Kg, int Kp) {
    const long long total = (long long) batch * Ho * Wo * Kp;
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long) gridDim.x * blockDim.x) {
        const long long n = i / Kp;
        const int k = (int) (i - n * Kp);
        float h = 0.f, l = 0.f;
        if (k < Kg) {
            const int fw = k % wf, fh = (k / wf) % hf, ci = k / (wf * hf);
            const int wo = (int) (n % Wo), ho = (int) ((n / Wo) % Ho), b = (int) (n / ((long long) Wo * Ho));
            const int y = ho * stride - pad + fh, x = wo * stride - pad + fw;
            if (y >= 0 && y < H && x >= 0 && x < W)
                split_tf32(__ldg(in + (((long long) b * cin + ci) * H + y) * W + x), h, l);
        }
        hi[i] = h;
        lo[i] = l;
    }
}

// Same planes, one CTA per output row (image b, row ho): the hf input rows of every
// channel that this output row touches are staged in shared memory once (coalesced
// reads), then each thread owns a few k = (cin, hf, wf) and walks along wo, so the
// (cin, hf, wf) decode happens once per k and the plane writes are coalesced along k.
__global__ void __launch_bounds__(256)
im2col_split_rows_kernel(const float* __restrict__ in, float* __restrict__ hi, float* __restrict__ lo, int cin, int H, int W,
                         int hf, int wf, int stride, int pad, int Ho, int Wo, int Kg, int Kp) {
    extern __shared__ float patch[];  // [cin][hf][W]
    const int b = blockIdx.x / Ho, ho = blockIdx.x - b * Ho;
    const int rows = cin * hf;
    for (int e = threadIdx.x; e < rows * W; e += blockDim.x) {
        const int r = e / W, x = e - r * W;
        const int ci = r / hf, fh = r - ci * hf;
        const int y = ho * stride - pad + fh;
        patch[e] = (y >= 0 && y < H) ? __ldg(in + (((long long) b * cin + ci) * H + y) * W + x) : 0.0f;
    }
    __syncthreads();
    const long long row_base = ((long long) b * Ho + ho) * Wo;
    for (int k = threadIdx.x; k < Kp; k += blockDim.x) {
        const bool real = k < Kg;
        const int ci = k / (hf * wf), r = k - ci * (hf * wf);
        const int fh = r / wf, fw = r - fh * wf;
        const float* src = patch + (ci * hf + fh) * W;
        for (int wo = 0; wo < Wo; wo++) {
            const int x = wo * stride - pad + fw;
            float h = 0.f, l = 0.f;
            if (real && x >= 0 && x < W) split_tf32(src[x], h, l);
            const long long o = (row_base + wo) * Kp + k;
            hi[o] = h;
            lo[o] = l;
        }
    }
}

// A tile whose K range was cut into pieces: its partial accumulators sit in `count`
// consecutive slots and are added up in slot order (ascending K), then stored to C.
struct TilePieces {
    int tm, tn, first_slot, count;
};

template <int BN>
__global__ void __launch_bounds__(256)
reduce_pieces_kernel(const float* __restrict__ partials, const TilePieces* __restrict__ tiles, float* __restrict__ C, int M,
                     int N, int ldc, int accumulate, int out_p, long long out_image_stride, const float* __restrict__ bias) {
    const TilePieces t = tiles[blockIdx.x];
    const float* base = partials + (long long) t.first_slot * (BM * BN);
    // gridDim.y CTAs share a tile, each taking a band of its rows
    const int rows_per = BM / (int) gridDim.y, r_lo = (int) blockIdx.y * rows_per;
    for (int i = threadIdx.x; i < rows_per * BN / 4; i += blockDim.x) {
        const int r = r_lo + i / (BN / 4), c = (i % (BN / 4)) * 4;
        float4 s = *reinterpret_cast<const float4*>(base + (long long) r * BN + c);
        for (int p = 1; p < t.count; p++) {
            const float4 v = *reinterpret_cast<const float4*>(base + (long long) p * (BM * BN) + (long long) r * BN + c);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        const int row = t.tm * BM + r, col = t.tn * BN + c;
        if (row >= M) continue;
        const float e[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (col + j >= N) break;
            long long at;
            if (out_p > 0) {
                const int img = (col + j) / out_p, pos = (col + j) - img * out_p;
                at = (long long) img * out_image_stride + (long long) row * out_p + pos;
            } else {
                at = (long long) row * ldc + col + j;
            }
            const float v = bias ? e[j] + __ldg(bias + col + j) : e[j];
            C[at] = accumulate ? C[at] + v : v;
        }
    }
}

// The same sum for a K-sharded product: the rows of every summed tile go to the rank that owns them,
// over NVLink, with plain stores into that rank's memory (the slot reserved there for this rank), as
// soon as the tile is summed.  The CTA that finishes last tells every owner that this rank's rows are
// complete.  Nothing here waits: the owners wait (bounded) in sum_owner_slots_kernel.
template <int BN>
__global__ void __launch_bounds__(256)
reduce_pieces_to_owners_kernel(const float* __restrict__ partials, const TilePieces* __restrict__ tiles, int M, int N,
                               const OwnerSlots os) {
    const TilePieces t = tiles[blockIdx.x];
    const float* base = partials + (long long) t.first_slot * (BM * BN);
    const int rows_per = BM / (int) gridDim.y, r_lo = (int) blockIdx.y * rows_per;
    const bool vec = (N % 4 == 0);
    for (int i = threadIdx.x; i < rows_per * BN / 4; i += blockDim.x) {
        const int r = r_lo + i / (BN / 4), c = (i % (BN / 4)) * 4;
        const int row = t.tm * BM + r, col = t.tn * BN + c;
        if (row >= M || col >= N) continue;
        float4 s = *reinterpret_cast<const float4*>(base + (long long) r * BN + c);
        for (int p = 1; p < t.count; p++) {
            const float4 v = *reinterpret_cast<const float4*>(base + (long long) p * (BM * BN) + (long long) r * BN + c);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        int o = 0;
        while (o + 1 < os.world && row >= os.row_lo[o + 1]) o++;
        float* dst = os.base[o] + (long long) (row - os.row_lo[o]) * N + col;
        if (vec) {
            *reinterpret_cast<float4*>(dst) = s;  // N % 4 == 0 and col % 4 == 0: whole and 16-byte aligned
        } else {
            const float e[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (col + j < N) dst[j] = e[j];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();  // this CTA's rows are visible to the owners before it is counted
        const unsigned total = gridDim.x * gridDim.y;
        if (atomicAdd(os.done, 1u) == total - 1) {
            *os.done = 0;  // ready for the next product on this stream
            __threadfence_system();
            for (int o = 0; o < os.world; o++) *reinterpret_cast<volatile int*>(os.flag[o]) = os.epoch;
        }
    }
}

// ------------------------------------------------------------- host side

typedef CUresult (*encode_fn_t)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_fn_t encode_fn() {
    static encode_fn_t fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (encode_fn_t) p;
        else
            cudaGetLastError();
    });
    return fn;
}

}  // namespace

int encode_tiled_f32(CUtensorMap* map, const float* base, int rank, const unsigned long long* dims,
                     const unsigned long long* strides_bytes, const unsigned* box, bool swizzle128) {
    encode_fn_t enc = encode_fn();
    if (!enc) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return CAKEB200_ERR_CUDA;
    }
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], estr[5] = {1, 1, 1, 1, 1};
    for (int i = 0; i < rank; i++) { d[i] = dims[i]; b[i] = box[i]; }
    for (int i = 0; i + 1 < rank; i++) st[i] = strides_bytes[i];
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t) rank, (void*) base, d, st, b, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d (rank %d)", (int) r, rank);
        return CAKEB200_ERR_CUDA;
    }
    return CAKEB200_OK;
}

namespace {

// rows x K plane (leading dimension Kp floats), boxes of box_rows x 32 floats, 128-byte swizzle, zero fill
int make_map(CUtensorMap* map, const float* base, int rows, int K, int Kp, int box_rows) {
    encode_fn_t enc = encode_fn();
    if (!enc) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return CAKEB200_ERR_CUDA;
    }
    cuuint64_t dims[2] = {(cuuint64_t) K, (cuuint64_t) rows};
    cuuint64_t strides[1] = {(cuuint64_t) Kp * 4};
    cuuint32_t box[2] = {(cuuint32_t) BK, (cuuint32_t) box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*) base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d (rows %d, K %d, Kp %d)", (int) r, rows, K, Kp);
        return CAKEB200_ERR_CUDA;
    }
    return CAKEB200_OK;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int padded_k(int K) { return (K + 3) / 4 * 4; }  // TMA row pitch must be a multiple of 16 bytes

// Choices that can be overridden per shape (0 = the rule below): tile width, band height of the tile
// walk, K pieces per tile of the ragged last wave, chunk length of the accumulation.  They come from
// cakeb200_set_option and the tuning cache (resolve_tunables); the rules are what an untuned shape gets.
struct Tunables {
    int bn = 0, band = 0, pieces = 0, chunk_kb = 0;
    int pair = 0;  // cluster shape: 1 = pairs of SMs wherever possible, 2 = single SMs
};

// What applies to one product: an explicit override wins, then the tuning cache's entry for the
// shape, then the rule (a field left 0).
Tunables resolve_tunables(int M, int N, int K, int order) {
    Tunables t;
    t.bn = option_get(OPT_TILE_N); t.band = option_get(OPT_BAND); t.pieces = option_get(OPT_K_PIECES); t.chunk_kb = option_get(OPT_CHUNK_KB);
    t.pair = option_get(OPT_PAIR);
    int w = 0, b = 0, p = 0, c = 0;
    if (tune_lookup(M, N, K, order, &w, &b, &p, &c)) {
        if (!t.bn) t.bn = w;
        if (!t.band) t.band = b;
        if (!t.pieces) t.pieces = p;
        if (!t.pair) t.pair = c;
    }
    return t;
}

// Columns of C per tile.  256 halves the reads of A per flop and its MMAs run about 30 % better per
// flop than 128-wide ones, so it is what large products want.  A shallow product with fewer 128 x 256
// tiles than SMs leaves most of the machine to the K cut alone, which has little K to cut, and 128-wide
// tiles then give twice the tiles to spread (measured: 2048^3 0.145 -> 0.117 ms, 1024^3 0.053 -> 0.048 ms;
// 3000^3 and larger are faster with 256, and so is a deep product with few tiles, 1024 x 262144 x 1024:
// 2.6 ms against 3.4 ms, because its K cut fills the machine by itself).  On pairs of SMs (`pair_units` of
// them, 0 = single-SM form) a product whose 256 x 256 tiles fill at least three quarters of one wave runs
// them whole, with no cut along K and no reduction (2048^3: 64 tiles on 74 pairs, 0.107 -> 0.099 ms).
inline int tile_width(int M, int N, int K, int sm_count, const Tunables& t, int pair_units = 0) {
    if ((t.bn == 128 || t.bn == 256) && !(t.bn == 256 && N <= 128)) return t.bn;
    if (N <= 128) return 128;
    const long long wide_tiles = (long long) ((M + BM - 1) / BM) * ((N + 255) / 256);
    if (pair_units > 0) {
        const long long pair_tiles = (long long) ((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
        if (pair_tiles <= pair_units && pair_tiles * 4 >= 3LL * pair_units) return 256;
    }
    return (wide_tiles <= sm_count && K <= 4096) ? 128 : 256;
}
int pair_clusters();
bool use_pair(int M, int mode);
// With 128-wide tiles an MMA of either form is bound by its issue, not by shared memory, and the single-SM
// form spreads twice as many tiles: 1 to 6 % faster on the shapes that get narrow tiles (1024^3: 0.0351
// against 0.0372 ms).  Under the rule pairs are therefore for 256-wide tiles.
inline bool pair_pays(int bn, int mode) { return mode == 1 || bn == 256; }

// Band height of the tile walk.  Tiles that run together should cover a patch of C with
// few distinct A and B panels; 8 rows (or columns) per band measured best on the square,
// the tall and the wide benchmark shapes alike (12 and 16 were equal on squares and up
// to 20 % slower on the 65536 x 1024 x 1024 and 1024 x 1024 x 65536 products).
int band_for(int order, int tiles_m, int tiles_n, const Tunables& t) {
    const int band = t.band > 0 ? t.band : 8;
    return std::max(1, std::min(band, order == CAKEB200_SCHED_NKM ? tiles_n : tiles_m));
}

// How the tiles of one product are spread over the persistent CTAs.  Whole waves of
// tiles are taken round-robin, one whole-K tile per CTA per wave.  When the tile count
// is not a multiple of the CTA count, the last full wave plus the remainder (or all
// tiles, when there are fewer tiles than CTAs) is laid out as one long row of k-blocks
// and cut into equal shares, so every CTA finishes at the same time; tiles that end up
// cut get their pieces summed by reduce_pieces_kernel.  This is how the K-first schedule
// keeps all cores busy on shapes with few output blocks (src/cake_sgemm_k_first.cpp:75-98).
struct HostPlan {
    int grid = 0, dp_tiles = 0, slots = 0, longest_kb = 0;  // longest_kb: slices of the longest K piece
    std::vector<int4> units;
    std::vector<int> cta_begin;
    std::vector<TilePieces> pieces;
};

// `sm_count` is the number of units that take tiles: SMs, or pairs of SMs (`pair`, whose tiles are 256 rows
// high and whose partial tiles are two 128-row halves, the odd CTA's `slots` further on).
HostPlan build_plan(int tiles_m, int tiles_n, int kblocks, int order, int sm_count, const Tunables& tn, bool pair) {
    HostPlan p;
    const int band = band_for(order, tiles_m, tiles_n, tn);
    const long long T = (long long) tiles_m * tiles_n;
    const int G = (int) std::min<long long>(T, sm_count);
    p.grid = G;
    p.dp_tiles = (int) T;
    p.cta_begin.assign(G + 1, 0);
    if (G == 0) return p;
    // Whole waves are taken round-robin.  The R tiles left over (fewer than there are SMs)
    // would occupy only R SMs for a whole tile time, so each of them is cut into s equal
    // K ranges.  Pieces are numbered K-range-major: pieces that run at the same time read
    // the same K range of the operands, which keeps them shared in L2 (a cut that staggers
    // the K ranges over the CTAs turned out DRAM-bound).  s minimises
    // ceil(R*s / SMs) / s tile times plus the cost of writing and re-reading the partial tiles.
    const int R = (int) (T % sm_count);
    if (R == 0 || kblocks < 16) return p;
    const int s_max = std::min(std::min(32, kblocks / 8), std::max(1, (4 * sm_count) / R));
    const double tile_us = 1.17 * kblocks, slot_us = pair ? 0.18 : 0.09, fixed_us = 8.0;
    int best_s = 1;
    double best = tile_us;
    // (Pieces of very different lengths were timed on 1024 x 262144 x 1024, 32 tiles: 4, 9 and 18 pieces per
    // tile give 2.64, 2.57 and 2.58 ms, so beyond filling the SMs the choice of s hardly matters.)
    for (int s = 2; s <= s_max; s++) {
        const long long rounds = ((long long) R * s + sm_count - 1) / sm_count;
        const double cost = tile_us * rounds / s + slot_us * R * s + fixed_us;
        if (cost < best * 0.97) { best = cost; best_s = s; }
    }
    if (tn.pieces >= 1 && (long long) tn.pieces * R <= 4LL * sm_count + 4 && tn.pieces <= kblocks)
        best_s = tn.pieces;  // the selector's choice for this shape
    if (best_s == 1) return p;
    const int s = best_s;
    p.dp_tiles = (int) T - R;
    p.grid = (int) std::min<long long>((long long) sm_count, std::max<long long>(G, (long long) R * s));
    p.slots = R * s;
    const int per = (kblocks + s - 1) / s;
    p.longest_kb = per;
    std::vector<std::vector<int4>> per_cta(p.grid);
    for (int q = 0; q < s; q++)
        for (int r = 0; r < R; r++) {
            const int u = q * R + r;
            const int k0 = std::min(kblocks, q * per), k1 = std::min(kblocks, k0 + per);
            per_cta[u % p.grid].push_back(make_int4(p.dp_tiles + r, k0, k1, r * s + q));
        }
    p.cta_begin.assign(p.grid + 1, 0);
    for (int c = 0; c < p.grid; c++) {
        p.cta_begin[c] = (int) p.units.size();
        p.units.insert(p.units.end(), per_cta[c].begin(), per_cta[c].end());
    }
    p.cta_begin[p.grid] = (int) p.units.size();
    for (int r = 0; r < R; r++) {
        int tm, tn;
        tile_coords(p.dp_tiles + r, tiles_m, tiles_n, order, band, tm, tn);
        if (pair) {
            p.pieces.push_back({2 * tm, tn, r * s, s});
            p.pieces.push_back({2 * tm + 1, tn, p.slots + r * s, s});
        } else {
            p.pieces.push_back({tm, tn, r * s, s});
        }
    }
    return p;
}

// Device copies of plans, cached per device by shape.  A slot is overwritten only after
// the last kernel that read it has finished (event), so asynchronous callers may queue
// many products ahead.
struct PlanKey {
    int tiles_m, tiles_n, kblocks, order, sm_count, bn, band, pieces, pair;  // band, pieces: the overrides in force (0 = rule)
    bool operator==(const PlanKey& o) const {
        return tiles_m == o.tiles_m && tiles_n == o.tiles_n && kblocks == o.kblocks && order == o.order &&
               sm_count == o.sm_count && bn == o.bn && band == o.band && pieces == o.pieces && pair == o.pair;
    }
};
struct DevicePlan {
    PlanKey key = {};
    bool valid = false;
    int grid = 0, dp_tiles = 0, slots = 0, num_pieces = 0, longest_kb = 0;
    char* dev = nullptr;
    size_t dev_bytes = 0;
    const int4* units = nullptr;
    const int* cta_begin = nullptr;
    const TilePieces* pieces = nullptr;
    cudaEvent_t last_use = nullptr;
    unsigned long long stamp = 0;
    bool pinned = false;  // recorded into a CUDA graph: the table must stay where it is for good
};
constexpr int PLAN_SLOTS = 16, PLAN_DEVICES = 64;
DevicePlan g_plans[PLAN_DEVICES][PLAN_SLOTS];
unsigned long long g_plan_clock = 0;
std::mutex g_plan_mutex;

int get_plan(int tiles_m, int tiles_n, int kblocks, int order, int sm_count, int bn, const Tunables& tn, bool pair,
             cudaStream_t stream, DevicePlan** out) {
    int dev = 0;
    CAKE_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= PLAN_DEVICES) dev = 0;
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    const PlanKey key = {tiles_m, tiles_n, kblocks, order, sm_count, bn, tn.band, tn.pieces, pair ? 1 : 0};
    DevicePlan* slots = g_plans[dev];
    DevicePlan* victim = nullptr;
    for (int i = 0; i < PLAN_SLOTS; i++) {
        if (slots[i].valid && slots[i].key == key) {
            slots[i].stamp = ++g_plan_clock;
            *out = &slots[i];
            return CAKEB200_OK;
        }
        if (!slots[i].valid) { victim = &slots[i]; break; }
        if (!slots[i].pinned && (!victim || slots[i].stamp < victim->stamp)) victim = &slots[i];
    }
    if (!victim) {
        set_error("every cached tile plan of this device is part of a captured CUDA graph (16 shapes)");
        return CAKEB200_ERR_ARG;
    }
    {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) cudaGetLastError();
        if (capturing != cudaStreamCaptureStatusNone) {
            set_error("first use of a shape during stream capture: call it once outside the capture (the tile plan is uploaded then)");
            return CAKEB200_ERR_ARG;
        }
    }
    const HostPlan hp = build_plan(tiles_m, tiles_n, kblocks, order, sm_count, tn, pair);
    const size_t units_b = align_up(hp.units.size() * sizeof(int4) + 16, 256);
    const size_t begin_b = align_up(hp.cta_begin.size() * sizeof(int), 256);
    const size_t pieces_b = align_up(hp.pieces.size() * sizeof(TilePieces) + 16, 256);
    const size_t need = units_b + begin_b + pieces_b;
    if (victim->last_use) CAKE_CUDA_OK(cudaEventSynchronize(victim->last_use));
    else CAKE_CUDA_OK(cudaEventCreateWithFlags(&victim->last_use, cudaEventDisableTiming));
    if (need > victim->dev_bytes) {
        if (victim->dev) CAKE_CUDA_OK(cudaFree(victim->dev));
        victim->dev = nullptr;
        victim->dev_bytes = 0;
        CAKE_CUDA_OK(cudaMalloc((void**) &victim->dev, need));
        victim->dev_bytes = need;
    }
    victim->valid = false;
    if (!hp.units.empty())
        CAKE_CUDA_OK(cudaMemcpyAsync(victim->dev, hp.units.data(), hp.units.size() * sizeof(int4), cudaMemcpyHostToDevice, stream));
    CAKE_CUDA_OK(cudaMemcpyAsync(victim->dev + units_b, hp.cta_begin.data(), hp.cta_begin.size() * sizeof(int),
                                 cudaMemcpyHostToDevice, stream));
    if (!hp.pieces.empty())
        CAKE_CUDA_OK(cudaMemcpyAsync(victim->dev + units_b + begin_b, hp.pieces.data(), hp.pieces.size() * sizeof(TilePieces),
                                     cudaMemcpyHostToDevice, stream));
    CAKE_CUDA_OK(cudaStreamSynchronize(stream));  // the host vectors die with this scope
    victim->key = key;
    victim->grid = hp.grid; victim->dp_tiles = hp.dp_tiles; victim->slots = hp.slots; victim->longest_kb = hp.longest_kb;
    victim->num_pieces = (int) hp.pieces.size();
    victim->units = hp.units.empty() ? nullptr : (const int4*) victim->dev;
    victim->cta_begin = (const int*) (victim->dev + units_b);
    victim->pieces = (const TilePieces*) (victim->dev + units_b + begin_b);
    victim->stamp = ++g_plan_clock;
    victim->valid = true;
    *out = victim;
    return CAKEB200_OK;
}

// bytes of partial-tile slots a product may need (an upper bound that does not depend on the plan)
size_t partial_slot_bytes(int sm_count) { return (size_t) (4 * sm_count + 16) * BM * 256 * sizeof(float); }

// Pairs of CTAs (clusters of two) of the largest pair kernel that the device runs at once; 0: it cannot. Per device.
int pair_clusters() {
    static std::mutex m;
    static int cached[PLAN_DEVICES];  // 0 = not asked yet, -1 = unavailable
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PLAN_DEVICES) { cudaGetLastError(); return 0; }
    std::lock_guard<std::mutex> lock(m);
    if (cached[dev] == 0) {
        cached[dev] = -1;
        int sms = 0, n = 0;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.blockDim = dim3(CHUNKED_THREADS);
        cfg.dynamicSmemBytes = Cfg<256, true>::SMEM_BYTES_CHUNKED;
        cfg.attrs = at; cfg.numAttrs = 1;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms >= 2 &&
            cudaFuncSetAttribute(sgemm_tf32x3_chunked_kernel<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<256, true>::SMEM_BYTES_CHUNKED) == cudaSuccess) {
            cfg.gridDim = dim3((unsigned) (sms / 2 * 2));
            if (cudaOccupancyMaxActiveClusters(&n, sgemm_tf32x3_chunked_kernel<256, true>, &cfg) == cudaSuccess && n > 0) cached[dev] = n;
        }
        cudaGetLastError();
    }
    return cached[dev] > 0 ? cached[dev] : 0;
}

// Whether a product with M rows runs its tiles on pairs of SMs.  Not for a single row of tiles, and under
// the rule not where padding the rows to 256 instead of 128 would add more than 7 % of work.
bool use_pair(int M, int mode) {  // mode: 0 = rule, 1 = wherever possible, 2 = never
    if (mode == 2 || M <= BM) return false;
    if (pair_clusters() <= 0) return false;
    if (mode == 1) return true;
    const long long p256 = (M + 2 * BM - 1) / (2 * BM) * (2LL * BM), p128 = (M + BM - 1) / BM * (long long) BM;
    return p256 * 100 <= p128 * 107;
}
inline int tile_rows(bool pair) { return pair ? 2 * BM : BM; }
inline int tile_units(bool pair, int sm_count) { return pair ? pair_clusters() : sm_count; }

template <int BN, bool PAIR>
cudaError_t run_kernel(bool chunked, int grid_units, cudaStream_t stream, const CUtensorMap& ma_hi, const CUtensorMap& ma_lo,
                       const CUtensorMap& mb_hi, const CUtensorMap& mb_lo, const Tf32x3Args& args) {
    using C_ = Cfg<BN, PAIR>;
    // the shared-memory opt-in is a property of the kernel on one device: once per device a product runs on
    static std::atomic<unsigned long long> opted_in{0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !(opted_in.load() >> dev & 1)) {
        e = cudaFuncSetAttribute(sgemm_tf32x3_kernel<BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(sgemm_tf32x3_chunked_kernel<BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES_CHUNKED);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) opted_in.fetch_or(1ULL << dev);
    }
    if constexpr (PAIR) {
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned) (2 * grid_units));
        cfg.blockDim = dim3(chunked ? CHUNKED_THREADS : NUM_THREADS);
        cfg.dynamicSmemBytes = chunked ? C_::SMEM_BYTES_CHUNKED : C_::SMEM_BYTES;
        cfg.stream = stream;
        cfg.attrs = at; cfg.numAttrs = 1;
        return chunked ? cudaLaunchKernelEx(&cfg, sgemm_tf32x3_chunked_kernel<BN, PAIR>, ma_hi, ma_lo, mb_hi, mb_lo, args)
                       : cudaLaunchKernelEx(&cfg, sgemm_tf32x3_kernel<BN, PAIR>, ma_hi, ma_lo, mb_hi, mb_lo, args);
    } else {
        if (chunked)
            sgemm_tf32x3_chunked_kernel<BN, PAIR><<<grid_units, CHUNKED_THREADS, C_::SMEM_BYTES_CHUNKED, stream>>>(ma_hi, ma_lo, mb_hi, mb_lo, args);
        else
            sgemm_tf32x3_kernel<BN, PAIR><<<grid_units, NUM_THREADS, C_::SMEM_BYTES, stream>>>(ma_hi, ma_lo, mb_hi, mb_lo, args);
        return cudaGetLastError();
    }
}

#ifdef CAKEB200_ROLE_TIMERS
void print_timeline(int* status_word, cudaStream_t stream, bool chunked) {
    unsigned long long h[12];
    cudaStreamSynchronize(stream);
    cudaMemcpy(h, status_word + 16, sizeof(h), cudaMemcpyDeviceToHost);
    fprintf(stderr, "K1 %s timeline of CTA 0 (us after entry): ready %.2f, first MMA %.2f, last commit %.2f, last acc_full seen %.2f, "
            "drain warp 2 done %.2f, drain warp 4 done %.2f, thread 0 at exit %.2f, after final sync %.2f; first MMA to last commit %llu cycles\n", chunked ? "chunked" : "plain",
            (h[1] - h[0]) * 1e-3, (h[2] - h[0]) * 1e-3, (h[3] - h[0]) * 1e-3, (h[4] - h[0]) * 1e-3, (h[5] - h[0]) * 1e-3,
            (h[6] - h[0]) * 1e-3, (h[7] - h[0]) * 1e-3, (h[8] - h[0]) * 1e-3, h[10] - h[9]);
}
#endif

// plan == nullptr: whole-K tiles only, taken round-robin (no table, no partial slots).  A plan must have been
// built for the same PAIR (tile rows and unit count).
template <int BN, bool PAIR>
int launch(const GemmProblem& g, float* a_hi, float* a_lo, float* b_hi, float* b_lo, float* partials, DevicePlan* plan,
           int* status_word, int sm_count, cudaStream_t stream, int* launches, const Tunables& tn) {
    using C_ = Cfg<BN, PAIR>;
    const int units = tile_units(PAIR, sm_count);
    const int Kp = padded_k(g.K);
    alignas(64) CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    int rc;
    if ((rc = make_map(&ma_hi, a_hi, g.M, g.K, Kp, BM))) return rc;
    if ((rc = make_map(&ma_lo, a_lo, g.M, g.K, Kp, BM))) return rc;
    if ((rc = make_map(&mb_hi, b_hi, g.N, g.K, Kp, C_::B_ROWS))) return rc;
    if ((rc = make_map(&mb_lo, b_lo, g.N, g.K, Kp, C_::B_ROWS))) return rc;

    Tf32x3Args a;
    a.C = g.C;
    a.partials = partials;
    a.slot_count = plan ? plan->slots : 0;
    a.M = g.M; a.N = g.N; a.K = g.K;
    a.ldc = g.ldc;
    a.tiles_m = (g.M + C_::TILE_M - 1) / C_::TILE_M;
    a.tiles_n = (g.N + BN - 1) / BN;
    a.kblocks = (g.K + BK - 1) / BK;
    a.kb_first = 0;
    // Chunk length of the accumulation.  Rule: 1024 of K.
    a.chunk_kb = tn.chunk_kb > 0 ? tn.chunk_kb : CHUNK_KB;
    a.drain_backoff = 400;  // a chunk lasts tens of microseconds; measured +0.4 % at 8192^3 against plain polling
    a.order = g.order;
    a.band = band_for(g.order, a.tiles_m, a.tiles_n, tn);
    a.accumulate = g.accumulate;
    a.out_p = g.out_p;
    a.out_image_stride = g.out_image_stride;
    a.bias = g.bias;
    a.status_word = status_word;
    const long long tiles = (long long) a.tiles_m * a.tiles_n;
    if (tiles > 0x7fffffffLL) {
        set_error("sgemm_tf32x3: too many tiles");
        return CAKEB200_ERR_TOO_LARGE;
    }
    int grid;  // units that take tiles: CTAs, or pairs of CTAs
    if (plan && plan->units && partials) {
        a.units = plan->units; a.cta_begin = plan->cta_begin; a.dp_tiles = plan->dp_tiles;
        grid = plan->grid;
    } else {
        a.units = nullptr; a.cta_begin = nullptr; a.dp_tiles = (int) tiles;
        grid = (int) std::min<long long>(tiles, units);
    }
    // the chunked kernel only where some K range is longer than a chunk (whole tiles; pieces are shorter)
    auto run = [&](const Tf32x3Args& args) {
        const int longest = (plan && a.units && plan->dp_tiles == 0 && plan->longest_kb > 0) ? plan->longest_kb : args.kblocks;
        const cudaError_t e = run_kernel<BN, PAIR>(args.chunk_kb < longest, grid, stream, ma_hi, ma_lo, mb_hi, mb_lo, args);
#ifdef CAKEB200_ROLE_TIMERS
        print_timeline(status_word, stream, args.chunk_kb < longest);
#endif
        return e;
    };
    // A very deep product with many tiles is run as several launches over ranges of K, each adding to C.
    // Within one launch the CTAs of a wave share their A and B panels through L2 only while they work on
    // nearby slices of K; over thousands of slices they drift apart and the panels come from DRAM once per
    // CTA (32768^3: 400 ms in one launch, 313 ms in ranges of 8192, at the cost of re-reading C three times).
    const int total_kb = a.kblocks;
    const int range_kb = (total_kb > 512 && tiles * (PAIR ? 2 : 1) >= 4LL * sm_count && g.out_p == 0) ? 256 : total_kb;
    if (g.owners && !(range_kb == total_kb && a.units && plan->num_pieces > 0 && plan->dp_tiles == 0)) {
        set_error("sgemm_tf32x3: a K-sharded product needs a shape whose tiles are all cut into K pieces");
        return CAKEB200_ERR_ARG;
    }
    if (range_kb < total_kb) {
        a.units = nullptr; a.cta_begin = nullptr; a.dp_tiles = (int) tiles;
        grid = (int) std::min<long long>(tiles, units);
        for (int first = 0; first < total_kb; first += range_kb) {
            a.kb_first = first;
            a.kblocks = std::min(range_kb, total_kb - first);
            a.accumulate = (first > 0) ? 1 : g.accumulate;
            a.bias = (first > 0) ? nullptr : g.bias;
            CAKE_CUDA_OK(run(a));
            if (launches) (*launches)++;
        }
        return CAKEB200_OK;
    }
    CAKE_CUDA_OK(run(a));
    if (launches) (*launches)++;
    if (g.owners) {
        reduce_pieces_to_owners_kernel<BN><<<dim3(plan->num_pieces, 16), 256, 0, stream>>>(partials, plan->pieces, g.M, g.N, *g.owners);
        CAKE_CUDA_OK(cudaGetLastError());
        if (launches) (*launches)++;
    } else if (a.units && plan->num_pieces > 0) {
        reduce_pieces_kernel<BN><<<dim3(plan->num_pieces, 16), 256, 0, stream>>>(partials, plan->pieces, g.C, g.M, g.N, g.ldc, g.accumulate,
                                                                      g.out_p, g.out_image_stride, g.bias);
        CAKE_CUDA_OK(cudaGetLastError());
        if (launches) (*launches)++;
    }
    if (a.units) {
        // inside a stream capture the table becomes part of the graph: it is pinned instead of tracked by an event
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) cudaGetLastError();
        if (capturing != cudaStreamCaptureStatusNone) plan->pinned = true;
        else CAKE_CUDA_OK(cudaEventRecord(plan->last_use, stream));
    }
    return CAKEB200_OK;
}

// The instantiation for a tile width and form.
int launch_as(int bn, bool pair, const GemmProblem& g, float* a_hi, float* a_lo, float* b_hi, float* b_lo, float* partials,
              DevicePlan* plan, int* status_word, int sm_count, cudaStream_t stream, int* launches, const Tunables& tn) {
    if (pair)
        return (bn == 256) ? launch<256, true>(g, a_hi, a_lo, b_hi, b_lo, partials, plan, status_word, sm_count, stream, launches, tn)
                           : launch<128, true>(g, a_hi, a_lo, b_hi, b_lo, partials, plan, status_word, sm_count, stream, launches, tn);
    return (bn == 256) ? launch<256, false>(g, a_hi, a_lo, b_hi, b_lo, partials, plan, status_word, sm_count, stream, launches, tn)
                       : launch<128, false>(g, a_hi, a_lo, b_hi, b_lo, partials, plan, status_word, sm_count, stream, launches, tn);
}

// rows [0, M) of A (leading dimension lda) -> hi / lo planes
int run_split_rows(const float* A, float* hi, float* lo, int M, int K, int lda, int Kp, int sm_count, cudaStream_t stream) {
    if (M <= 0) return CAKEB200_OK;
    const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (((uintptr_t) A | (uintptr_t) hi | (uintptr_t) lo) % 16 == 0);
    if (vec) {
        const long long total = (long long) M * (K / 4);
        const int blocks = (int) std::min<long long>((total + 255) / 256, (long long) sm_count * 16);
        split_rows_vec4_kernel<<<blocks, 256, 0, stream>>>((const float4*) A, (float4*) hi, (float4*) lo, M, K / 4, lda / 4);
    } else {
        const long long total = (long long) M * Kp;
        const int blocks = (int) std::min<long long>((total + 255) / 256, (long long) sm_count * 16);
        split_rows_kernel<<<blocks, 256, 0, stream>>>(A, hi, lo, M, K, lda, Kp);
    }
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}

int run_split_transpose(const float* B, float* hi, float* lo, int K, int N, int ldb, int Kp, cudaStream_t stream) {
    dim3 grid((N + 31) / 32, (Kp + 31) / 32);
    if (grid.y > 65535) {
        set_error("sgemm_tf32x3: K too large for the transpose grid");
        return CAKEB200_ERR_TOO_LARGE;
    }
    split_transpose_kernel<<<grid, 256, 0, stream>>>(B, hi, lo, K, N, ldb, Kp);
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}

}  // namespace

// ---- row-band interface: lets the host-pointer driver overlap copies with compute.
// Planes for the whole product are laid out once; B is split once; then each band of
// rows is split and multiplied as soon as its rows have arrived.

// slots_for_sms > 0 also reserves room for partial tiles, so that a whole product multiplied
// through tf32x3_multiply_rows can balance its tiles over that many SMs
size_t tf32x3_plane_bytes(int M, int N, int K, int slots_for_sms) {
    const size_t Kp = (size_t) padded_k(K);
    return 2 * align_up((size_t) M * Kp * 4, 1024) + 2 * align_up((size_t) N * Kp * 4, 1024) + 2048 +
           (slots_for_sms > 0 ? partial_slot_bytes(slots_for_sms) : 0);
}

int tf32x3_planes(int M, int N, int K, void* scratch, size_t scratch_bytes, Tf32x3Planes* out, int slots_for_sms) {
    if (tf32x3_plane_bytes(M, N, K, slots_for_sms) > scratch_bytes) {
        set_error("sgemm_tf32x3: scratch too small for the operand planes");
        return CAKEB200_ERR_ARG;
    }
    const int Kp = padded_k(K);
    const size_t a_bytes = align_up((size_t) M * Kp * 4, 1024), b_bytes = align_up((size_t) N * Kp * 4, 1024);
    char* base = (char*) align_up((size_t) scratch, 1024);
    out->a_hi = (float*) base;
    out->a_lo = (float*) (base + a_bytes);
    out->b_hi = (float*) (base + 2 * a_bytes);
    out->b_lo = (float*) (base + 2 * a_bytes + b_bytes);
    out->partials = slots_for_sms > 0 ? (float*) (base + 2 * a_bytes + 2 * b_bytes) : nullptr;
    out->M = M;
    out->Kp = Kp;
    return CAKEB200_OK;
}

int tf32x3_split_B(const float* B, int ldb, int K, int N, const Tf32x3Planes& p, cudaStream_t stream) {
    return run_split_transpose(B, p.b_hi, p.b_lo, K, N, ldb, p.Kp, stream);
}

// B planes of a convolution: n = (image, ho, wo) rows, k = (cin, hf, wf) columns
int tf32x3_split_im2col(const float* in, int batch, int cin, int H, int W, int hf, int wf, int stride, int pad,
                        const Tf32x3Planes& p, int sm_count, cudaStream_t stream) {
    const int Ho = (H + 2 * pad - hf) / stride + 1, Wo = (W + 2 * pad - wf) / stride + 1;
    const long long total = (long long) batch * Ho * Wo * p.Kp;
    if (total <= 0) return CAKEB200_OK;
    const size_t patch_bytes = (size_t) cin * hf * W * sizeof(float);
    if (patch_bytes <= 200 * 1024 && (long long) batch * Ho <= 0x7fffffffLL) {
        CAKE_CUDA_OK(cudaFuncSetAttribute(im2col_split_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) patch_bytes));
        im2col_split_rows_kernel<<<batch * Ho, 256, patch_bytes, stream>>>(in, p.b_hi, p.b_lo, cin, H, W, hf, wf, stride, pad,
                                                                          Ho, Wo, cin * hf * wf, p.Kp);
        CAKE_CUDA_OK(cudaGetLastError());
        return CAKEB200_OK;
    }
    const int blocks = (int) std::min<long long>((total + 255) / 256, (long long) sm_count * 32);
    im2col_split_kernel<<<blocks, 256, 0, stream>>>(in, p.b_hi, p.b_lo, batch, cin, H, W, hf, wf, stride, pad, Ho, Wo,
                                                    cin * hf * wf, p.Kp);
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}

int tf32x3_split_A_rows(const float* A, int lda, int r0, int rows, int K, const Tf32x3Planes& p, int sm_count,
                        cudaStream_t stream) {
    return run_split_rows(A + (size_t) r0 * lda, p.a_hi + (size_t) r0 * p.Kp, p.a_lo + (size_t) r0 * p.Kp, rows, K, lda,
                          p.Kp, sm_count, stream);
}

int tf32x3_multiply_rows(const Tf32x3Planes& p, float* C, int ldc, int r0, int rows, int N, int K, int order,
                         int accumulate, int* status_word, int sm_count, cudaStream_t stream, int out_p,
                         long long out_image_stride) {
    GemmProblem g = {};
    g.C = C + (size_t) r0 * ldc;
    g.M = rows; g.N = N; g.K = K;
    g.ldc = ldc;
    g.batch = 1;
    g.order = order;
    g.accumulate = accumulate;
    g.out_p = out_p;
    g.out_image_stride = out_image_stride;
    float* a_hi = p.a_hi + (size_t) r0 * p.Kp;
    float* a_lo = p.a_lo + (size_t) r0 * p.Kp;
    DevicePlan* plan = nullptr;
    const Tunables tn = resolve_tunables(rows, N, K, order);
    // of the whole product, so that every band of rows uses one width
    const int bn = tile_width(p.M, N, K, sm_count, tn, use_pair(p.M, tn.pair) ? pair_clusters() : 0);
    const bool pair = use_pair(rows, tn.pair) && pair_pays(bn, tn.pair);
    if (p.partials && r0 == 0 && rows == p.M) {  // the whole product at once: balance its tiles
        int rc = get_plan((rows + tile_rows(pair) - 1) / tile_rows(pair), (N + bn - 1) / bn, (K + BK - 1) / BK, order,
                          tile_units(pair, sm_count), bn, tn, pair, stream, &plan);
        if (rc) return rc;
    }
    return launch_as(bn, pair, g, a_hi, a_lo, p.b_hi, p.b_lo, p.partials, plan, status_word, sm_count, stream, nullptr, tn);
}

// scratch = A hi/lo planes + transposed B hi/lo planes + slots for the partial tiles of the last wave (worst case)
size_t tf32x3_scratch_bytes(int M, int N, int K, int sm_count) {
    const size_t Kp = (size_t) padded_k(K);
    const size_t a = align_up((size_t) M * Kp * 4, 1024), b = align_up((size_t) N * Kp * 4, 1024);
    return 2 * a + 2 * b + partial_slot_bytes(sm_count) + 2048;
}

int tf32x3_tile_rows(int M, int N, int K, int order, int sm_count) {
    const Tunables tn = resolve_tunables(M, N, K, order);
    const bool by_rows = use_pair(M, tn.pair);
    const int bn = tile_width(M, N, K, sm_count, tn, by_rows ? pair_clusters() : 0);
    return tile_rows(by_rows && pair_pays(bn, tn.pair));
}

size_t tf32x3_one_plane_bytes(int rows, int K) { return align_up((size_t) rows * padded_k(K) * 4, 1024); }

int tf32x3_make_planes(const float* mat, int rows, int K, int ld, bool transpose, float* hi, float* lo, int sm_count,
                       cudaStream_t stream) {
    const int Kp = padded_k(K);
    return transpose ? run_split_transpose(mat, hi, lo, K, rows, ld, Kp, stream) : run_split_rows(mat, hi, lo, rows, K, ld, Kp, sm_count, stream);
}

bool tf32x3_all_tiles_in_pieces(int M, int N, int K, int order, int sm_count) {
    if (M <= 0 || N <= 0 || K <= 0 || sm_count <= 0) return false;
    // the same choices as launch_sgemm_tf32x3 makes for this shape
    const Tunables tn = resolve_tunables(M, N, K, order);
    const bool by_rows = use_pair(M, tn.pair);
    const int bn = tile_width(M, N, K, sm_count, tn, by_rows ? pair_clusters() : 0), kblocks = (K + BK - 1) / BK;
    const bool pair = by_rows && pair_pays(bn, tn.pair);
    const int tm = (M + tile_rows(pair) - 1) / tile_rows(pair), units = tile_units(pair, sm_count);
    const long long tiles = (long long) tm * ((N + bn - 1) / bn);
    if (tiles >= units) return false;
    const HostPlan hp = build_plan(tm, (N + bn - 1) / bn, kblocks, order, units, tn, pair);
    return hp.dp_tiles == 0 && !hp.pieces.empty();
}

int launch_sgemm_tf32x3(const GemmProblem& g, void* scratch, size_t scratch_bytes, int* status_word, int sm_count,
                        cudaStream_t stream, cakeb200_stats* stats, cudaEvent_t* prepass_events) {
    if (g.batch != 1) {
        set_error("sgemm_tf32x3: batched products are not supported by this kernel");
        return CAKEB200_ERR_ARG;
    }
    const int Kp = padded_k(g.K);
    const size_t a_bytes = align_up((size_t) g.M * Kp * 4, 1024), b_bytes = align_up((size_t) g.N * Kp * 4, 1024);
    char* base = (char*) align_up((size_t) scratch, 1024);
    // planes the caller kept from an earlier split are used where they lie; the others go to the scratch arena
    float* a_hi = g.a_hi ? const_cast<float*>(g.a_hi) : (float*) base;
    float* a_lo = g.a_hi ? const_cast<float*>(g.a_lo) : (float*) (base + a_bytes);
    float* b_hi = g.b_hi ? const_cast<float*>(g.b_hi) : (float*) (base + 2 * a_bytes);
    float* b_lo = g.b_hi ? const_cast<float*>(g.b_lo) : (float*) (base + 2 * a_bytes + b_bytes);
    float* partials = (float*) (base + 2 * a_bytes + 2 * b_bytes);

    const Tunables tn = resolve_tunables(g.M, g.N, g.K, g.order);
    const bool by_rows = use_pair(g.M, tn.pair);
    const int bn = tile_width(g.M, g.N, g.K, sm_count, tn, by_rows ? pair_clusters() : 0);
    const bool pair = by_rows && pair_pays(bn, tn.pair);
    const size_t need = 2 * a_bytes + 2 * b_bytes + partial_slot_bytes(sm_count) + 1024;
    if (need > scratch_bytes) {
        set_error("sgemm_tf32x3: scratch too small (%zu < %zu)", scratch_bytes, need);
        return CAKEB200_ERR_ARG;
    }
    if ((g.a_hi && !g.a_lo) || (g.b_hi && !g.b_lo) || (((uintptr_t) a_hi | (uintptr_t) a_lo | (uintptr_t) b_hi | (uintptr_t) b_lo) % 16)) {
        set_error("sgemm_tf32x3: operand planes come in hi / lo pairs, 16-byte aligned");
        return CAKEB200_ERR_ARG;
    }

    if (prepass_events) CAKE_CUDA_OK(cudaEventRecord(prepass_events[0], stream));
    int rc = CAKEB200_OK;
    int split_launches = 0;
    // both operand planes are K-major; an operand already stored that way (A as given, B
    // transposed, e.g. the N x K weight of a linear layer) is split in place, the other
    // kind is transposed through shared memory on the way
    if (!g.a_hi) {
        if (g.trans_a) rc = run_split_transpose(g.A, a_hi, a_lo, g.K, g.M, g.lda, Kp, stream);
        else rc = run_split_rows(g.A, a_hi, a_lo, g.M, g.K, g.lda, Kp, sm_count, stream);
        if (rc) return rc;
        split_launches++;
    }
    if (!g.b_hi) {
        if (g.trans_b) rc = run_split_rows(g.B, b_hi, b_lo, g.N, g.K, g.ldb, Kp, sm_count, stream);
        else rc = run_split_transpose(g.B, b_hi, b_lo, g.K, g.N, g.ldb, Kp, stream);
        if (rc) return rc;
        split_launches++;
    }
    if (prepass_events) CAKE_CUDA_OK(cudaEventRecord(prepass_events[1], stream));

    DevicePlan* plan = nullptr;
    if ((rc = get_plan((g.M + tile_rows(pair) - 1) / tile_rows(pair), (g.N + bn - 1) / bn, (g.K + BK - 1) / BK, g.order,
                       tile_units(pair, sm_count), bn, tn, pair, stream, &plan)))
        return rc;
    int launches = split_launches;
    rc = launch_as(bn, pair, g, a_hi, a_lo, b_hi, b_lo, partials, plan, status_word, sm_count, stream, &launches, tn);
    if (rc) return rc;
    if (stats) {
        stats->launches += launches;
        stats->tile_m = tile_rows(pair); stats->tile_n = bn; stats->tile_k = BK;
    }
    return CAKEB200_OK;
}

}  // namespace cakeb200

// ------------------------------------------------- self-test of the bounded wait
//
// One CTA waits on an mbarrier that nothing ever arrives at, with a limit of `limit_us`
// microseconds, through the same wait routine the product kernels use.  The wait must give
// up, record where in the status word and let the kernel return normally; the host then
// reports CAKEB200_ERR_DEVICE_TIMEOUT and the context stays usable.  This is how the
// containment of a stalled pipeline is exercised without stalling anything for real.
namespace cakeb200 {
namespace {
__global__ void bounded_wait_selftest_kernel(int* status_word, long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait_for(smem_u32(&bar), 0, &abort_flag, status_word, 900, limit_ns);
    __syncthreads();
}
// The same for a pair of CTAs: the leader waits for an arrival that its peer would send to the leader's barrier
// and never does (as if the peer's drain warps had stalled).  The leader gives up, and both CTAs still meet
// at the cluster barrier that ends every pair kernel, so neither leaves while the other could touch it.
__global__ void __launch_bounds__(32) bounded_wait_pair_selftest_kernel(int* status_word, long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    const uint32_t rank = cluster_ctarank();
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 2);  // one arrival from each CTA; only the leader's own ever comes
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    cluster_sync_all();
    if (threadIdx.x == 0 && rank == 0) {
        mbar_arrive_leader(smem_u32(&bar));
        mbar_wait_for(smem_u32(&bar), 0, &abort_flag, status_word, 901, limit_ns);
    }
    cluster_sync_all();
}
}  // namespace

int launch_bounded_wait_selftest(int* status_word, int limit_us, cudaStream_t stream, bool pair) {
    if (pair) {
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2);
        cfg.blockDim = dim3(32);
        cfg.stream = stream;
        cfg.attrs = at; cfg.numAttrs = 1;
        CAKE_CUDA_OK(cudaLaunchKernelEx(&cfg, bounded_wait_pair_selftest_kernel, status_word, (long long) limit_us * 1000));
        return CAKEB200_OK;
    }
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status_word, (long long) limit_us * 1000);
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}
}  // namespace cakeb200

// ------------------------------------------------- entry point that allocates nothing
//
// Some callers may not allocate device memory at the moment they need a product:
// code that runs inside another framework's memory pool and must not disturb it, a
// real-time loop whose memory budget was fixed at start-up, a library that is handed
// a stream and buffers and told to stay off the allocator.  cakeb200_sgemm grows a
// scratch arena with cudaMalloc on first use and again whenever a larger shape shows
// up, so those callers cannot use it.  This variant runs the same 3xTF32 kernels with
// the split operand planes in a fixed array that is part of the library image.
//
// The array costs CAKEB200_NOALLOC_SCRATCH_BYTES of device memory on every GPU that
// loads the library, from load until the process exits.
namespace {

constexpr size_t NOALLOC_HEADER = 1024;  // status word, then padding up to the plane alignment
static __device__ __align__(256) unsigned char g_noalloc_scratch[CAKEB200_NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device
// address; the address is looked up once per device, with that device current.
constexpr int NOALLOC_MAX_DEVICES = 64;
unsigned char* g_noalloc_addr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_noalloc_mutex;

int noalloc_scratch(unsigned char** out) {
    int dev = -1;
    CAKE_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        cakeb200::set_error("device index %d out of range", dev);
        return CAKEB200_ERR_NO_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_addr[dev]) {
        void* p = nullptr;
        CAKE_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_noalloc_addr[dev] = (unsigned char*) p;
    }
    *out = g_noalloc_addr[dev];
    return CAKEB200_OK;
}

// device memory of the device `dev` (the kernels run there; memory of another GPU may not even be mapped)
bool noalloc_on_device(const void* p, int dev) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (a.type == cudaMemoryTypeManaged) return true;
    return a.type == cudaMemoryTypeDevice && a.device == dev;
}

}  // namespace

// bytes of the built-in array a shape uses: header + two planes of A + two planes of B
static size_t noalloc_scratch_need(int M, int N, int K) {
    const size_t Kp = (size_t) cakeb200::padded_k(K);
    return NOALLOC_HEADER + 2 * cakeb200::align_up((size_t) M * Kp * 4, 1024) + 2 * cakeb200::align_up((size_t) N * Kp * 4, 1024);
}

extern "C" int cakeb200_sgemm_noalloc(const float* A, const float* B, float* C, int M, int N, int K, void* stream) {
    using namespace cakeb200;
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) {
        set_error("cakeb200_sgemm_noalloc: null pointer or non-positive dimension");
        return CAKEB200_ERR_ARG;
    }
    int cur_dev = -1;
    CAKE_CUDA_OK(cudaGetDevice(&cur_dev));
    if (!noalloc_on_device(A, cur_dev) || !noalloc_on_device(B, cur_dev) || !noalloc_on_device(C, cur_dev)) {
        set_error("cakeb200_sgemm_noalloc: A, B and C must be device pointers of the current device %d (staging a host "
                  "operand would allocate; another GPU's memory is not reachable from the kernels)", cur_dev);
        return CAKEB200_ERR_ARG;
    }
    const size_t need = noalloc_scratch_need(M, N, K);
    if (need > (size_t) CAKEB200_NOALLOC_SCRATCH_BYTES) {
        set_error("cakeb200_sgemm_noalloc: M=%d N=%d K=%d needs %zu bytes of scratch, the built-in array holds %zu; "
                  "use cakeb200_sgemm for this shape",
                  M, N, K, need, (size_t) CAKEB200_NOALLOC_SCRATCH_BYTES);
        return CAKEB200_ERR_TOO_LARGE;
    }
    unsigned char* base = nullptr;
    int rc = noalloc_scratch(&base);
    if (rc) return rc;
    int dev = 0, sm_count = 0;
    CAKE_CUDA_OK(cudaGetDevice(&dev));
    CAKE_CUDA_OK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    cudaStream_t s = (cudaStream_t) stream;

    const int Kp = padded_k(K);
    const size_t a_bytes = align_up((size_t) M * Kp * 4, 1024), b_bytes = align_up((size_t) N * Kp * 4, 1024);
    int* status_word = (int*) base;
    float* a_hi = (float*) (base + NOALLOC_HEADER);
    float* a_lo = (float*) (base + NOALLOC_HEADER + a_bytes);
    float* b_hi = (float*) (base + NOALLOC_HEADER + 2 * a_bytes);
    float* b_lo = (float*) (base + NOALLOC_HEADER + 2 * a_bytes + b_bytes);

    // The array keeps whatever the previous call left.  The status word must start
    // at zero; the planes need no clearing because the split pass rewrites every
    // element this shape will read, padding columns included.
    CAKE_CUDA_OK(cudaMemsetAsync(status_word, 0, 256, s));
    {
        const long long total = (long long) M * Kp;
        const int blocks = (int) std::min<long long>((total + 255) / 256, (long long) sm_count * 16);
        split_rows_kernel<<<blocks, 256, 0, s>>>(A, a_hi, a_lo, M, K, K, Kp);
        dim3 grid((N + 31) / 32, (Kp + 31) / 32);
        if (grid.y > 65535) {
            set_error("cakeb200_sgemm_noalloc: K too large");
            return CAKEB200_ERR_TOO_LARGE;
        }
        split_transpose_kernel<<<grid, 256, 0, s>>>(B, b_hi, b_lo, K, N, N, Kp);
        CAKE_CUDA_OK(cudaGetLastError());
    }
    GemmProblem g = {};
    g.A = A; g.B = B; g.C = C;
    g.M = M; g.N = N; g.K = K;
    g.lda = K; g.ldb = N; g.ldc = N;
    g.batch = 1;
    g.order = CAKEB200_SCHED_KMN;
    // whole-K tiles only: cutting tiles along K would need slots for partial tiles, i.e. more scratch
    const int bn_na = N > 128 ? 256 : 128, mode_na = option_get(OPT_PAIR);
    rc = launch_as(bn_na, use_pair(M, mode_na) && pair_pays(bn_na, mode_na), g, a_hi, a_lo, b_hi, b_lo, nullptr, nullptr, status_word, sm_count, s, nullptr,
                   Tunables());
    if (rc) return rc;
    int word[4] = {0, 0, 0, 0};
    CAKE_CUDA_OK(cudaMemcpyAsync(word, status_word, sizeof(word), cudaMemcpyDeviceToHost, s));
    CAKE_CUDA_OK(cudaStreamSynchronize(s));
    if (word[0] != 0) {
        set_error("cakeb200_sgemm_noalloc: device-side wait gave up (where %d, block %d)", word[1], word[2]);
        return CAKEB200_ERR_DEVICE_TIMEOUT;
    }
    return CAKEB200_OK;
}
