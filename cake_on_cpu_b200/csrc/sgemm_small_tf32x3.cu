// Batches of small FP32 products on the tensor cores (3xTF32), operands split in the kernel.
//
// The reference's small-matrix path (cake_gemm_small / schedule_*_small,
// src/cake_sgemm.cpp:614-721, src/cake_sgemm_small.cpp:7-236) skips packing because a
// small matrix does not repay a separate pass over it.  The same holds here: for a
// product of 96 x 96 matrices the operand-split pass of the large-matrix path would
// write and re-read three times the bytes of the operands.  So this kernel reads A and
// B as the caller stores them, and a group of producer warps does what the reference's
// packing does -- lay the operands out the way the multiplier wants them -- on the way
// into shared memory: each value is split into its TF32 hi and lo parts and written into
// 128-byte-swizzled K-major tiles (B is transposed by the choice of which thread writes
// what); when tensor memory has room next to the two accumulators (N <= 192) the split A
// operand is stored there instead (tcgen05.st, a thread per row) and costs no shared-memory
// bandwidth when the multiplier reads it.  One tcgen05.mma issuer consumes the tiles; the accumulator of one product is a
// 128 x N block of tensor memory; four warps drain it while the next product is already
// being multiplied into the second block.
//
// Getting the operands on chip: a loader thread brings raw FP32 boxes of A (M x 32) and B
// (32 x N) into a ring of shared-memory buffers with TMA, several stages ahead, so that
// enough bytes are in flight per SM to keep HBM busy; the producer warps then work from
// shared memory to shared memory.  When the operands do not meet TMA's alignment rules
// (leading dimensions and strides in multiples of 4 floats, 16-byte aligned bases) or the
// tiles leave no room for the ring, the producer warps read global memory themselves.
//
// One CTA per SM walks the batch: product i goes to CTA i mod gridDim.x.  Limits:
// M <= 128, N <= 256 (one accumulator per product); K is arbitrary (zero-filled to a
// multiple of 32).  Rows of the 128-row tile beyond M are never written and hold
// whatever the shared memory held: they only feed accumulator rows that are never
// stored, since every row of the result depends on its own row of A alone.
//
// Every wait is bounded; a wait that runs out records where in the status word, raises
// the CTA's abort flag, and the CTA frees its tensor memory and returns.
#include <stdlib.h>
#include <string.h>
#include <algorithm>

#include "common.cuh"
#include "tcgen05.cuh"

namespace cakeb200 {
namespace {

using namespace ptx;

constexpr int BM = 128, BK = 32, UMMA_K = 8;
constexpr int PROD_WARPS = 16, EPI_WARPS = 4, EPI_GROUPS = 1;  // a second epilogue group (one per accumulator) was tried: no gain
constexpr int PROD_THREADS = PROD_WARPS * 32;
constexpr int FIRST_EPI_WARP = 2, FIRST_PROD_WARP = FIRST_EPI_WARP + EPI_GROUPS * EPI_WARPS;
constexpr int NUM_THREADS = 32 * (FIRST_PROD_WARP + PROD_WARPS);  // MMA, loader, 4 epilogue, 16 producer warps
constexpr int A_ITER = (BM * 8 + PROD_THREADS - 1) / PROD_THREADS;    // float4 chunks of A per producer thread and stage
constexpr int B_ITER = (256 * 8 + PROD_THREADS - 1) / PROD_THREADS;   // float4 chunks of B (N up to 256)
constexpr int EPI_BYTES = EPI_GROUPS * EPI_WARPS * 32 * 32 * 4;
constexpr int MAX_SMEM = 227 * 1024;
constexpr int MAX_RING = 8;

// Role timers (diagnostic build only, -DCAKEB200_ROLE_TIMERS): CTA 0 adds up the clock cycles its roles
// spend waiting and working into status_word[16 + 2 * slot] (64-bit counters).
#ifdef CAKEB200_ROLE_TIMERS
#define TIMER_DECL long long _t0 = 0
#define TIMER_START() _t0 = clock64()
#define TIMER_ADD(slot) do { if (blockIdx.x == 0) atomicAdd((unsigned long long*) (a.status_word + 16) + (slot), (unsigned long long) (clock64() - _t0)); } while (0)
#else
#define TIMER_DECL
#define TIMER_START()
#define TIMER_ADD(slot)
#endif

struct SmallArgs {
    const float* A;
    const float* B;
    float* C;
    const float* bias;
    int M, N, K;
    int lda, ldb, ldc;
    long long stride_a, stride_b, stride_c;
    int batch;
    int accumulate;
    int kblocks;       // ceil(K / 32)
    int npad;          // N rounded up to a multiple of 16: the N of the MMA
    int a_plane;       // bytes of one split plane of A per stage: M rounded up to 8 rows, 128 bytes each
    int b_plane;       // bytes of one split plane of B per stage: npad * 128
    int stage_bytes;   // 2 * a_plane + 2 * b_plane
    int stages;        // split stages
    int ring;          // raw stages filled by TMA (0: producers read global memory)
    int raw_a_bytes, raw_b_bytes, raw_bytes;
    int raw_tx;        // bytes the two TMA boxes of a raw stage deliver: (M + npad) * 128
    int acc_stride;    // tensor-memory columns between the two accumulators (multiple of 32)
    int tmem_cols;     // power of two >= 2 * acc_stride
    uint32_t idesc;
    int a_vec;         // rows of A may be read as float4 (direct mode)
    int a_tmem;        // the split A operand lives in tensor memory (first column a_col0), not in shared memory
    int a_col0;
    int* status_word;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
sgemm_small_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          const SmallArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t* raws = tiles + a.stages * a.stage_bytes;
    uint64_t* bars = (uint64_t*) (raws + a.ring * a.raw_bytes);
    // bars: split full [S], split empty [S], raw full [R], raw empty [R], accumulator full x2, accumulator empty x2
    uint32_t* tmem_slot = (uint32_t*) (bars + 28);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);
    volatile int* sync_flags = abort_flag + 1;  // [0]: producers, [1], [2]: epilogue (alternating)
    uint8_t* patches = (uint8_t*) bars + 256;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = a.stages, R = a.ring;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
    auto raw_full_bar = [&](int r) { return bar0 + 8u * (2 * S + r); };
    auto raw_empty_bar = [&](int r) { return bar0 + 8u * (2 * S + R + r); };
    auto acc_full_bar = [&](int b) { return bar0 + 8u * (2 * S + 2 * R + b); };
    auto acc_empty_bar = [&](int b) { return bar0 + 8u * (2 * S + 2 * R + 2 + b); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full_bar(s), 1);           // one producer thread, after the producers' own barrier
            mbar_init(empty_bar(s), 1);          // tcgen05.commit
        }
        for (int r = 0; r < R; r++) {
            mbar_init(raw_full_bar(r), 1);       // the loader's expect_tx arrival
            mbar_init(raw_empty_bar(r), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), EPI_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t) a.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // --------------------------------------------------------- MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            TIMER_DECL;
            for (int item = blockIdx.x; ok && item < a.batch; item += gridDim.x, local++) {
                const int buf = local & 1;
                TIMER_START();
                ok = mbar_wait(acc_empty_bar(buf), ((local >> 1) & 1) ^ 1, abort_flag, a.status_word, 200 + buf);
                TIMER_ADD(0);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t) (buf * a.acc_stride);
                uint32_t accumulate = 0;
                for (int kb = 0; kb < a.kblocks; kb++) {
                    TIMER_START();
                    ok = mbar_wait(full_bar(stage), phase, abort_flag, a.status_word, 300 + stage);
                    TIMER_ADD(1);
                    if (!ok) break;
                    TIMER_START();
                    tcgen05_fence_after();
                    const uint32_t base = smem_u32(tiles + stage * a.stage_bytes);
                    const uint64_t b_hi = make_kmajor_sw128_desc(base + 2 * a.a_plane);
                    const uint64_t b_lo = make_kmajor_sw128_desc(base + 2 * a.a_plane + a.b_plane);
                    if (a.a_tmem) {
                        const uint32_t t_hi = tmem_base + (uint32_t) (a.a_col0 + stage * 2 * BK), t_lo = t_hi + BK;
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; k++) {
                            const uint64_t adv = (uint64_t) (k * UMMA_K * 4 >> 4);
                            const uint32_t col = (uint32_t) (k * UMMA_K);
                            umma_tf32_ts(d_tmem, t_lo + col, b_hi + adv, a.idesc, accumulate);
                            umma_tf32_ts(d_tmem, t_hi + col, b_lo + adv, a.idesc, 1);
                            umma_tf32_ts(d_tmem, t_hi + col, b_hi + adv, a.idesc, 1);
                            accumulate = 1;
                        }
                    } else {
                        const uint64_t a_hi = make_kmajor_sw128_desc(base);
                        const uint64_t a_lo = make_kmajor_sw128_desc(base + a.a_plane);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; k++) {
                            const uint64_t adv = (uint64_t) (k * UMMA_K * 4 >> 4);
                            umma_tf32(d_tmem, a_lo + adv, b_hi + adv, a.idesc, accumulate);
                            umma_tf32(d_tmem, a_hi + adv, b_lo + adv, a.idesc, 1);
                            umma_tf32(d_tmem, a_hi + adv, b_hi + adv, a.idesc, 1);
                            accumulate = 1;
                        }
                    }
                    umma_commit(empty_bar(stage));
                    TIMER_ADD(2);
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(acc_full_bar(buf));
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------- loader of raw boxes
        if (lane == 0 && R > 0) {
            int r = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < a.batch; item += gridDim.x) {
                for (int kb = 0; kb < a.kblocks; kb++) {
                    TIMER_DECL;
                    TIMER_START();
                    ok = mbar_wait(raw_empty_bar(r), phase ^ 1, abort_flag, a.status_word, 500 + r);
                    TIMER_ADD(3);
                    if (!ok) break;
                    const uint32_t dst = smem_u32(raws + r * a.raw_bytes);
                    mbar_expect_tx(raw_full_bar(r), (uint32_t) a.raw_tx);
                    tma_load_3d(dst, &map_a, kb * BK, 0, item, raw_full_bar(r));
                    tma_load_3d(dst + (uint32_t) a.raw_a_bytes, &map_b, 0, kb * BK, item, raw_full_bar(r));
                    if (++r == R) { r = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // gave up: let the boxes already requested land before the CTA goes away (bounded)
                const unsigned long long t0 = global_ns();
                for (int q = 0; q < R; q++) {
                    const uint32_t armed = (q < r) ? phase : (phase ^ 1);
                    while (!mbar_try_wait(raw_full_bar(q), armed) && (long long) (global_ns() - t0) < 20000000LL) {}
                }
            }
        }
    } else if (warp < FIRST_PROD_WARP) {
        // ----------------------------------------------------------- epilogue
        const int quarter = warp & 3;  // a warp may only touch TMEM lanes [32*(warp%4), +32)
        const uint32_t patch = smem_u32(patches) + (uint32_t) (warp - FIRST_EPI_WARP) * 4096u;
        const int sub_r = lane >> 3, sub_c = lane & 7;
        const bool c_vec = (a.ldc % 4 == 0) && (a.stride_c % 4 == 0) && (((uintptr_t) a.C) % 16 == 0);
        const int chunks = (a.npad + 31) / 32;
        // Epilogue group g (of EPI_GROUPS) handles the CTA's products g, g + EPI_GROUPS, ...; with one group the
        // accumulators alternate, with two each accumulator would have its own group.
        const int grp = (warp - FIRST_EPI_WARP) / EPI_WARPS;
        const bool poller = (warp - FIRST_EPI_WARP) % EPI_WARPS == 0 && lane == 0;
        bool ok = true;
        for (int local = grp; ok; local += EPI_GROUPS) {
            const long long item_ll = (long long) blockIdx.x + (long long) local * gridDim.x;
            if (item_ll >= a.batch) break;
            const int item = (int) item_ll;
            const int buf = local & 1;
            TIMER_DECL;
            TIMER_START();
            if (poller)
                sync_flags[1 + buf] = mbar_wait(acc_full_bar(buf), (local >> 1) & 1, abort_flag, a.status_word, 400 + buf) ? 1 : 0;
            named_barrier_sync(2 + grp, EPI_WARPS * 32);
            if (warp == FIRST_EPI_WARP && lane == 0) TIMER_ADD(4);
            TIMER_START();
            ok = sync_flags[1 + buf] != 0;
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (buf * a.acc_stride);
            float* Ci = a.C + (long long) item * a.stride_c;
            if (quarter * 32 >= a.M) {  // none of this warp's 32 rows belongs to the matrix
                tcgen05_fence_before();
                if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                continue;
            }
            float v[32];
            tmem_ld32(t_addr, v);
#pragma unroll 1
            for (int c = 0; c < chunks; c++) {
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; j++)
                    st_shared_v4(patch + (uint32_t) lane * 128u + (uint32_t) ((j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1],
                                 v[4 * j + 2], v[4 * j + 3]);
                __syncwarp();
                if (c + 1 < chunks) {
                    tmem_ld32(t_addr + (uint32_t) ((c + 1) * 32), v);
                } else {
                    tcgen05_fence_before();
                    if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                }
                const int col = c * 32 + sub_c * 4;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = i * 4 + sub_r;
                    float4 o = ld_shared_v4(patch + (uint32_t) r * 128u + (uint32_t) ((sub_c ^ (r & 7)) << 4));
                    const int row = quarter * 32 + r;
                    if (row >= a.M || col >= a.N) continue;
                    float e[4] = {o.x, o.y, o.z, o.w};
                    float* dst = Ci + (long long) row * a.ldc + col;
                    if (a.bias != nullptr) {
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            if (col + j < a.N) e[j] += __ldg(a.bias + col + j);
                    }
                    if (c_vec && col + 4 <= a.N) {
                        float4 w = make_float4(e[0], e[1], e[2], e[3]);
                        if (a.accumulate) {
                            const float4 old = *reinterpret_cast<const float4*>(dst);
                            w.x += old.x; w.y += old.y; w.z += old.z; w.w += old.w;
                        }
                        *reinterpret_cast<float4*>(dst) = w;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            if (col + j < a.N) dst[j] = a.accumulate ? dst[j] + e[j] : e[j];
                    }
                }
                __syncwarp();
            }
            if (warp == FIRST_EPI_WARP && lane == 0) TIMER_ADD(5);
        }
    } else {
        // ----------------------------------------------------------- producers
        // Thread t of the 512 producer threads owns, in every stage, the 16-byte chunks
        // t, t + 512, ... of A (chunk = 4 consecutive k of one row; 8 lanes cover one
        // 128-byte row, so reads are contiguous and the swizzled stores hit every bank once)
        // and of B (chunk = 4 consecutive k of one column n; consecutive lanes own
        // consecutive n, so the four reads of a warp are contiguous rows of B and the
        // stores again spread over all banks: this is where B gets transposed).
        const int t = threadIdx.x - 32 * FIRST_PROD_WARP;
        const int a_chunks = a.M * 8, b_chunks = a.npad * 8;
        int stage = 0, r = 0;
        uint32_t phase = 0, raw_phase = 0;
        bool ok = true;

        auto store_a = [&](uint32_t base, int idx, float4 v) {
            const int row = idx >> 3, chunk = idx & 7;
            float4 h, l;
            split_tf32(v.x, h.x, l.x);
            split_tf32(v.y, h.y, l.y);
            split_tf32(v.z, h.z, l.z);
            split_tf32(v.w, h.w, l.w);
            const uint32_t at = base + (uint32_t) row * 128u + (uint32_t) ((chunk ^ (row & 7)) << 4);
            st_shared_v4(at, h.x, h.y, h.z, h.w);
            st_shared_v4(at + (uint32_t) a.a_plane, l.x, l.y, l.z, l.w);
        };
        auto store_b = [&](uint32_t base, int chunk, int n, const float* v) {
            float h[4], l[4];
#pragma unroll
            for (int j = 0; j < 4; j++) split_tf32(v[j], h[j], l[j]);
            const uint32_t at = base + 2 * (uint32_t) a.a_plane + (uint32_t) n * 128u + (uint32_t) ((chunk ^ (n & 7)) << 4);
            st_shared_v4(at, h[0], h[1], h[2], h[3]);
            st_shared_v4(at + (uint32_t) a.b_plane, l[0], l[1], l[2], l[3]);
        };
        // One thread polls the mbarriers; the other 511 sleep on a hardware barrier instead of
        // spending issue slots on polling.
        auto wait_both = [&](bool with_raw) {
            TIMER_DECL;
            TIMER_START();
            if (t == 0) {
                bool mine = true;
                if (with_raw) mine = mbar_wait(raw_full_bar(r), raw_phase, abort_flag, a.status_word, 600 + r);
                TIMER_ADD(6);
                if (mine) mine = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, a.status_word, 100 + stage);
                sync_flags[0] = mine ? 1 : 0;
                TIMER_ADD(7);
            }
            named_barrier_sync(1, PROD_THREADS);
            return sync_flags[0] != 0;
        };

        if (R > 0 && a.a_tmem) {
            // A goes to tensor memory, B to shared memory.  Producer warps 0-7 take A: a thread owns one row
            // (its tensor-memory lane: warp % 4 selects the 32 lanes a warp may write) and 16 of the 32 k of a
            // stage, read from the 128-byte-swizzled raw box (conflict-free 16-byte loads although consecutive
            // lanes are consecutive rows).  Producer warps 8-15 take B as in the other mode.
            const int pw = t >> 5;
            const bool a_side = pw < 8;
            const int quarter = warp & 3, half = (pw >> 2) & 1, row = quarter * 32 + lane;
            constexpr int B_THREADS = PROD_THREADS / 2, B_IT = (192 * 8 + B_THREADS - 1) / B_THREADS;  // N up to 192
            const int tb = t - B_THREADS;
            uint32_t b_src[B_IT], b_dst[B_IT];
#pragma unroll
            for (int it = 0; it < B_IT; it++) {
                const int idx = (a_side ? 0 : tb) + it * B_THREADS, chunk = idx / a.npad, n = idx - chunk * a.npad;
                b_src[it] = (uint32_t) (chunk * 4 * a.npad + n) * 4u;
                b_dst[it] = (uint32_t) n * 128u + (uint32_t) ((chunk ^ (n & 7)) << 4);
            }
            const uint32_t b_row = (uint32_t) a.npad * 4u;
            for (int item = blockIdx.x; ok && item < a.batch; item += gridDim.x) {
                for (int kb = 0; kb < a.kblocks; kb++) {
                    ok = wait_both(true);
                    if (!ok) break;
                    TIMER_DECL;
                    TIMER_START();
                    const uint32_t base = smem_u32(tiles + stage * a.stage_bytes);
                    const uint32_t raw_a = smem_u32(raws + r * a.raw_bytes), raw_b = raw_a + (uint32_t) a.raw_a_bytes;
                    if (a_side) {
                        tcgen05_fence_after();  // the MMAs that read this slice of tensor memory have completed
                        float v[16], h[16], l[16];
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const int c = half * 4 + q;
                            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (row < a.M) x = ld_shared_v4(raw_a + (uint32_t) row * 128u + (uint32_t) ((c ^ (row & 7)) << 4));
                            v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
                        }
#pragma unroll
                        for (int j = 0; j < 16; j++) split_tf32(v[j], h[j], l[j]);
                        const uint32_t dst = tmem_base + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (a.a_col0 + stage * 2 * BK);
                        tmem_st16(dst + (uint32_t) (half * 16), h);
                        tmem_st16(dst + (uint32_t) (BK + half * 16), l);
                        tmem_st_wait();
                        tcgen05_fence_before();
                    } else {
                        float vb[B_IT][4];
#pragma unroll
                        for (int it = 0; it < B_IT; it++)
                            if (tb + it * B_THREADS < b_chunks) {
#pragma unroll
                                for (int j = 0; j < 4; j++) vb[it][j] = ld_shared_f32(raw_b + b_src[it] + (uint32_t) j * b_row);
                            }
#pragma unroll
                        for (int it = 0; it < B_IT; it++)
                            if (tb + it * B_THREADS < b_chunks) {
                                float h[4], l[4];
#pragma unroll
                                for (int j = 0; j < 4; j++) split_tf32(vb[it][j], h[j], l[j]);
                                st_shared_v4(base + b_dst[it], h[0], h[1], h[2], h[3]);
                                st_shared_v4(base + b_dst[it] + (uint32_t) a.b_plane, l[0], l[1], l[2], l[3]);
                            }
                        fence_proxy_async_smem();
                    }
                    if (t == 0) TIMER_ADD(8);
                    named_barrier_sync(1, PROD_THREADS);
                    if (t == 0) {
                        mbar_arrive(full_bar(stage));
                        mbar_arrive(raw_empty_bar(r));
                        TIMER_ADD(9);
                    }
                    if (++stage == S) { stage = 0; phase ^= 1; }
                    if (++r == R) { r = 0; raw_phase ^= 1; }
                }
            }
        } else if (R > 0) {
            // per-thread offsets of its chunks: where to read in the raw boxes, where to write in the split planes
            uint32_t a_src[A_ITER], a_dst[A_ITER], b_src[B_ITER], b_dst[B_ITER];
#pragma unroll
            for (int it = 0; it < A_ITER; it++) {
                const int idx = t + it * PROD_THREADS, row = idx >> 3, chunk = idx & 7;
                a_src[it] = (uint32_t) idx * 16u;
                a_dst[it] = (uint32_t) row * 128u + (uint32_t) ((chunk ^ (row & 7)) << 4);
            }
#pragma unroll
            for (int it = 0; it < B_ITER; it++) {
                const int idx = t + it * PROD_THREADS, chunk = idx / a.npad, n = idx - chunk * a.npad;
                b_src[it] = (uint32_t) (chunk * 4 * a.npad + n) * 4u;
                b_dst[it] = 2 * (uint32_t) a.a_plane + (uint32_t) n * 128u + (uint32_t) ((chunk ^ (n & 7)) << 4);
            }
            const uint32_t b_row = (uint32_t) a.npad * 4u;
            for (int item = blockIdx.x; ok && item < a.batch; item += gridDim.x) {
                for (int kb = 0; kb < a.kblocks; kb++) {
                    ok = wait_both(true);
                    if (!ok) break;
                    TIMER_DECL;
                    TIMER_START();
                    const uint32_t base = smem_u32(tiles + stage * a.stage_bytes);
                    const uint32_t raw_a = smem_u32(raws + r * a.raw_bytes), raw_b = raw_a + (uint32_t) a.raw_a_bytes;
                    // all reads of the stage first, so that their latencies overlap
                    float4 va[A_ITER];
                    float vb[B_ITER][4];
#pragma unroll
                    for (int it = 0; it < A_ITER; it++)
                        if (t + it * PROD_THREADS < a_chunks) va[it] = ld_shared_v4(raw_a + a_src[it]);
#pragma unroll
                    for (int it = 0; it < B_ITER; it++)
                        if (t + it * PROD_THREADS < b_chunks) {
#pragma unroll
                            for (int j = 0; j < 4; j++) vb[it][j] = ld_shared_f32(raw_b + b_src[it] + (uint32_t) j * b_row);
                        }
#pragma unroll
                    for (int it = 0; it < A_ITER; it++)
                        if (t + it * PROD_THREADS < a_chunks) {
                            float4 h, l;
                            split_tf32(va[it].x, h.x, l.x);
                            split_tf32(va[it].y, h.y, l.y);
                            split_tf32(va[it].z, h.z, l.z);
                            split_tf32(va[it].w, h.w, l.w);
                            st_shared_v4(base + a_dst[it], h.x, h.y, h.z, h.w);
                            st_shared_v4(base + a_dst[it] + (uint32_t) a.a_plane, l.x, l.y, l.z, l.w);
                        }
#pragma unroll
                    for (int it = 0; it < B_ITER; it++)
                        if (t + it * PROD_THREADS < b_chunks) {
                            float h[4], l[4];
#pragma unroll
                            for (int j = 0; j < 4; j++) split_tf32(vb[it][j], h[j], l[j]);
                            st_shared_v4(base + b_dst[it], h[0], h[1], h[2], h[3]);
                            st_shared_v4(base + b_dst[it] + (uint32_t) a.b_plane, l[0], l[1], l[2], l[3]);
                        }
                    if (t == 0) TIMER_ADD(8);
                    fence_proxy_async_smem();
                    named_barrier_sync(1, PROD_THREADS);
                    if (t == 0) {
                        mbar_arrive(full_bar(stage));
                        mbar_arrive(raw_empty_bar(r));
                        TIMER_ADD(9);
                    }
                    if (++stage == S) { stage = 0; phase ^= 1; }
                    if (++r == R) { r = 0; raw_phase ^= 1; }
                }
            }
        } else {
            // operands read straight from global memory; the loads of the next stage are
            // issued before the wait for its buffer
            float4 ra[A_ITER];
            float rb[B_ITER][4];
            auto fetch = [&](int item, int kb) {
                const float* Ai = a.A + (long long) item * a.stride_a;
                const float* Bi = a.B + (long long) item * a.stride_b;
#pragma unroll
                for (int it = 0; it < A_ITER; it++) {
                    const int idx = t + it * PROD_THREADS;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (idx < a_chunks) {
                        const int row = idx >> 3, k = kb * BK + (idx & 7) * 4;
                        const float* src = Ai + (long long) row * a.lda + k;
                        if (a.a_vec && k + 4 <= a.K) {
                            v = __ldg(reinterpret_cast<const float4*>(src));
                        } else {
                            if (k < a.K) v.x = __ldg(src);
                            if (k + 1 < a.K) v.y = __ldg(src + 1);
                            if (k + 2 < a.K) v.z = __ldg(src + 2);
                            if (k + 3 < a.K) v.w = __ldg(src + 3);
                        }
                    }
                    ra[it] = v;
                }
#pragma unroll
                for (int it = 0; it < B_ITER; it++) {
                    const int idx = t + it * PROD_THREADS;
#pragma unroll
                    for (int j = 0; j < 4; j++) rb[it][j] = 0.f;
                    if (idx < b_chunks) {
                        const int chunk = idx / a.npad, n = idx - chunk * a.npad;
                        const int k = kb * BK + chunk * 4;
                        if (n < a.N) {
                            const float* src = Bi + (long long) k * a.ldb + n;
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                if (k + j < a.K) rb[it][j] = __ldg(src + (long long) j * a.ldb);
                        }
                    }
                }
            };
            int item = blockIdx.x, kb = 0;
            if (item < a.batch) fetch(item, 0);
            while (ok && item < a.batch) {
                ok = wait_both(false);
                if (!ok) break;
                const uint32_t base = smem_u32(tiles + stage * a.stage_bytes);
#pragma unroll
                for (int it = 0; it < A_ITER; it++) {
                    const int idx = t + it * PROD_THREADS;
                    if (idx < a_chunks) store_a(base, idx, ra[it]);
                }
#pragma unroll
                for (int it = 0; it < B_ITER; it++) {
                    const int idx = t + it * PROD_THREADS;
                    if (idx < b_chunks) {
                        const int chunk = idx / a.npad;
                        store_b(base, chunk, idx - chunk * a.npad, rb[it]);
                    }
                }
                fence_proxy_async_smem();
                named_barrier_sync(1, PROD_THREADS);
                if (t == 0) mbar_arrive(full_bar(stage));
                if (++stage == S) { stage = 0; phase ^= 1; }
                if (++kb == a.kblocks) { kb = 0; item += gridDim.x; }
                if (item < a.batch) fetch(item, kb);
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t) a.tmem_cols)
                     : "memory");
    }
}

}  // namespace

bool small_tf32x3_fits(int M, int N, int K) { return M >= 1 && M <= BM && N >= 1 && N <= 256 && K >= 1; }

// `batch` products C_i (+)= A_i B_i (+ bias), row-major with leading dimensions and strides between items.
int launch_sgemm_small_tf32x3(const GemmProblem& g, int* status_word, int sm_count, cudaStream_t stream) {
    if (g.batch <= 0) return CAKEB200_OK;
    if (!small_tf32x3_fits(g.M, g.N, g.K) || g.trans_a || g.trans_b || g.out_p > 0) {
        set_error("sgemm_small_tf32x3: needs M <= 128, N <= 256 and untransposed operands (M=%d N=%d K=%d)", g.M, g.N, g.K);
        return CAKEB200_ERR_ARG;
    }
    SmallArgs a = {};
    a.A = g.A; a.B = g.B; a.C = g.C; a.bias = g.bias;
    a.M = g.M; a.N = g.N; a.K = g.K;
    a.lda = g.lda; a.ldb = g.ldb; a.ldc = g.ldc;
    a.stride_a = g.stride_a; a.stride_b = g.stride_b; a.stride_c = g.stride_c;
    a.batch = g.batch;
    a.accumulate = g.accumulate;
    a.kblocks = (g.K + BK - 1) / BK;
    a.npad = (g.N + 15) / 16 * 16;
    a.a_plane = (g.M + 7) / 8 * 8 * 128;
    a.b_plane = a.npad * 128;
    a.stage_bytes = 2 * a.a_plane + 2 * a.b_plane;
    a.acc_stride = (a.npad + 31) / 32 * 32;
    a.tmem_cols = 32;
    while (a.tmem_cols < 2 * a.acc_stride) a.tmem_cols *= 2;
    a.idesc = make_idesc_tf32(BM, a.npad);
    a.a_vec = (g.lda % 4 == 0) && (g.stride_a % 4 == 0) && (((uintptr_t) g.A) % 16 == 0);
    a.status_word = status_word;
    // the 128-row MMA reads 16 KB from the start of an A plane whatever M is; the epilogue
    // patches at the end of the allocation keep that inside shared memory
    const int fixed = 1024 /*alignment*/ + 256 /*barriers*/ + EPI_BYTES;
    a.raw_a_bytes = g.M * 128;
    a.raw_b_bytes = a.npad * 128;
    a.raw_bytes = (a.raw_a_bytes + a.raw_b_bytes + 127) / 128 * 128;
    a.raw_tx = (g.M + a.npad) * 128;
    const bool tma_ok = (g.lda % 4 == 0) && (g.ldb % 4 == 0) && (g.stride_a % 4 == 0) && (g.stride_b % 4 == 0) &&
                        (((uintptr_t) g.A | (uintptr_t) g.B) % 16 == 0) && option_get(OPT_SMALL_OPERANDS) != 2;
    // two split stages (one being multiplied, one being filled); the rest of shared memory goes to the
    // ring of raw boxes, whose depth is what keeps enough bytes in flight (measured at 96^3: ring of
    // 2 / 3 / 4 boxes -> 0.145 / 0.126 / 0.124 ms for 4096 products; a third split stage instead: 0.139 ms)
    a.stages = 2;
    a.ring = tma_ok ? std::min(MAX_RING, (MAX_SMEM - fixed - a.stages * a.stage_bytes) / a.raw_bytes) : 0;
    // With room in tensor memory next to the two accumulators (N up to 192) the split A operand goes there:
    // shared memory then holds only B's planes and raw boxes (A's box 128-byte swizzled, in 1 KiB units).
    if (tma_ok && a.acc_stride <= 192 && option_get(OPT_SMALL_OPERANDS) != 1) {
        SmallArgs t = a;
        t.a_tmem = 1;
        t.a_col0 = 2 * t.acc_stride;
        t.tmem_cols = 512;
        t.a_plane = 0;
        t.stage_bytes = 2 * t.b_plane;
        t.raw_a_bytes = (g.M * 128 + 1023) / 1024 * 1024;
        t.raw_bytes = t.raw_a_bytes + t.raw_b_bytes;
        t.stages = std::min(4, (512 - t.a_col0) / (2 * BK));
        t.ring = std::min(MAX_RING, (MAX_SMEM - fixed - t.stages * t.stage_bytes) / t.raw_bytes);
        while (t.ring < 3 && t.stages > 2) {
            t.stages--;
            t.ring = std::min(MAX_RING, (MAX_SMEM - fixed - t.stages * t.stage_bytes) / t.raw_bytes);
        }
        if (t.ring >= 2 && t.stages >= 2) a = t;
    }
    if (a.ring < 2) {
        a.ring = 0;
        a.stages = std::min(6, (MAX_SMEM - fixed) / a.stage_bytes);
    }
    if (a.stages < 2) {
        set_error("sgemm_small_tf32x3: not enough shared memory for two stages");
        return CAKEB200_ERR_ARG;
    }
    alignas(64) CUtensorMap map_a, map_b;
    memset(&map_a, 0, sizeof(map_a));
    memset(&map_b, 0, sizeof(map_b));
    if (a.ring > 0) {
        // A as {K, M, batch} with boxes of 32 x M x 1; B as {N, K, batch} with boxes of npad x 32 x 1;
        // elements outside the matrix (K tail, columns N..npad) arrive as zeros
        const unsigned long long da[3] = {(unsigned long long) g.K, (unsigned long long) g.M, (unsigned long long) g.batch};
        const unsigned long long sa[2] = {(unsigned long long) g.lda * 4, (unsigned long long) (g.stride_a > 0 ? g.stride_a : (long long) g.M * g.lda) * 4};
        const unsigned ba[3] = {(unsigned) BK, (unsigned) g.M, 1};
        const unsigned long long db[3] = {(unsigned long long) g.N, (unsigned long long) g.K, (unsigned long long) g.batch};
        const unsigned long long sb[2] = {(unsigned long long) g.ldb * 4, (unsigned long long) (g.stride_b > 0 ? g.stride_b : (long long) g.K * g.ldb) * 4};
        const unsigned bb[3] = {(unsigned) a.npad, (unsigned) BK, 1};
        int rc;
        if ((rc = encode_tiled_f32(&map_a, g.A, 3, da, sa, ba, a.a_tmem != 0))) return rc;
        if ((rc = encode_tiled_f32(&map_b, g.B, 3, db, sb, bb, false))) return rc;
    }
    const int smem = a.stages * a.stage_bytes + a.ring * a.raw_bytes + fixed;
    CAKE_CUDA_OK(cudaFuncSetAttribute(sgemm_small_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int grid = std::min(g.batch, sm_count);
    sgemm_small_tf32x3_kernel<<<grid, NUM_THREADS, smem, stream>>>(map_a, map_b, a);
    CAKE_CUDA_OK(cudaGetLastError());
#ifdef CAKEB200_ROLE_TIMERS
    {
        unsigned long long h[16];
        cudaStreamSynchronize(stream);
        cudaMemcpy(h, status_word + 16, sizeof(h), cudaMemcpyDeviceToHost);
        cudaMemset(status_word + 16, 0, sizeof(h));
        fprintf(stderr, "small-batch role timers (cycles, CTA 0): mma[wait_acc %llu wait_full %llu issue %llu] loader[wait %llu] "
                "epilogue[wait %llu work %llu] producer0[wait_raw %llu +wait_empty %llu convert %llu +publish %llu] slices/CTA %d\n",
                h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[7], h[8], h[9], (a.batch + grid - 1) / grid * a.kblocks);
    }
#endif
    return CAKEB200_OK;
}

}  // namespace cakeb200
