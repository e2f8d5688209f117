// Convolution as an implicit product on the tensor cores (3xTF32), stride 1, NCHW.
//
// The reference computes a convolution as im2col followed by one cake_sgemm
// (examples/cake_conv.cpp:1007-1066 with im_2_col at :1178-1213): the patch matrix is
// written out, packed and multiplied.  Here the patch matrix never exists, neither in
// HBM nor as TF32 planes.  A tile is up to 128 output positions times up to 128 output
// channels; the positions are whole output rows of one image or, when that saves a round
// of tiles on the machine, a run of 128 consecutive positions of the whole batch (which can
// start in the middle of a row and continue into the next images: one input box per image).  For each group of 32 input channels one TMA
// box brings the input rows those positions need into shared memory (rows above and below
// the image arrive as zeros), and for every filter tap (fh, fw) the producer warps build
// the 128 x 32 operand tile "position x channel" from that box -- a shifted window, read
// along the positions and split into TF32 hi and lo parts -- and store it with tcgen05.st
// into tensor memory, where tcgen05.mma takes its A operand from (a thread's position is
// its lane, the 32 channels are 32 columns), so this operand costs no shared-memory
// bandwidth at all.  The filters are the B operand: they are split once into hi / lo
// planes whose K axis is ordered (channel group, fh, fw, channel) to match, and TMA brings
// their 32-wide slices into 128-byte-swizzled shared-memory tiles.  tcgen05.mma accumulates
// all channel groups and taps of a tile in tensor memory; the epilogue stores it to NCHW
// (a warp's 32 lanes are 32 consecutive positions of one channel: contiguous).
//
// Measured on the way: one tcgen05.mma kind::tf32 of 128 x N x 8 takes about 80-90 cycles for
// every N up to 128 (and 188 for N = 256), whether A comes from shared or from tensor
// memory and whether consecutive instructions share an accumulator or not.  A tile of 64
// output channels therefore runs at half the tensor rate; 128 channels per tile is the
// smallest efficient width, and wider layers are cut into 128-channel tiles.
//
// Warps: 0 MMA issuer, 1 loader of input boxes, 2 loader of filter slices, 4-7 epilogue,
// 8-15 producers in two groups.  Every wait is bounded (status word + abort flag, as in the other
// tcgen05 kernels).
#include <stdlib.h>
#include <string.h>
#include <algorithm>

#include "common.cuh"
#include "tcgen05.cuh"

namespace cakeb200 {
namespace {

using namespace ptx;

constexpr int BM = 128, BK = 32, UMMA_K = 8;
constexpr int FIRST_EPI_WARP = 4, EPI_WARPS = 4, FIRST_PROD_WARP = 8, PROD_WARPS = 8;
constexpr int PROD_THREADS = PROD_WARPS * 32;
constexpr int GROUPS = 2, GROUP_THREADS = PROD_THREADS / GROUPS;  // producer groups; one thread per position
static_assert(GROUP_THREADS == BM, "one producer thread per position");
constexpr int NUM_THREADS = 32 * (FIRST_PROD_WARP + PROD_WARPS);
constexpr int A_COLS = 2 * BK;  // tensor-memory columns of one slice of the patch operand: 32 hi + 32 lo
constexpr int MAX_SMEM = 227 * 1024;
constexpr int MAX_RING = 4;

// Role timers (diagnostic build only, -DCAKEB200_ROLE_TIMERS): CTA 0 adds up the clock cycles each role
// spends in its waits and in its work into status_word[16 + slot].
#ifdef CAKEB200_ROLE_TIMERS
#define TIMER_DECL long long _t0 = 0
#define TIMER_START() _t0 = clock64()
#define TIMER_ADD(slot) do { if (blockIdx.x == 0) atomicAdd((unsigned long long*) (a.status_word + 16) + (slot), (unsigned long long) (clock64() - _t0)); } while (0)
#else
#define TIMER_DECL
#define TIMER_START()
#define TIMER_ADD(slot)
#endif

struct ConvArgs {
    float* out;
    const float* bias;
    int batch, cin, H, W, cout, hf, wf, pad, Ho, Wo;
    int flat;            // tiles are runs of 128 positions of the whole batch (else whole rows of one image)
    int rows_per_tile;   // row tiles: output rows of one image per tile
    int groups;          // row tiles: tiles per image
    int plane;           // Ho * Wo
    long long positions; // batch * plane
    int segs;            // images a tile can touch (1 for row tiles): input boxes per raw stage
    int box_bytes;       // one input box: box_w * 32 * 4
    int bn, ntiles;      // output channels per tile, tiles along the channels
    int ncg;             // groups of 32 input channels
    int kblocks;         // ncg * hf * wf
    int box_w;           // floats per channel in an input box
    int raw_bytes;       // one raw stage: segs * box_bytes
    int b_plane;         // bytes of one filter plane per stage: bn * 128
    int stage_bytes;     // 2 * b_plane (the patch operand of a stage lives in tensor memory)
    int a_col0;          // first tensor-memory column of the patch operand ring
    int stages, ring;
    int acc_stride, tmem_cols;
    uint32_t idesc;
    long long tiles;
    int* status_word;
};

// Filters F[cout][cin][hf][wf] -> hi / lo planes [cout][KP], KP = kblocks * 32, with
// k = ((group * hf + fh) * wf + fw) * 32 + channel in group; channels beyond cin are zeros.
__global__ void __launch_bounds__(256)
split_filters_kernel(const float* __restrict__ F, float* __restrict__ hi, float* __restrict__ lo, int cout, int cin, int hf,
                     int wf, int kblocks) {
    const long long total = (long long) cout * kblocks * 32;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += (long long) gridDim.x * 256) {
        const int c = (int) (i & 31);
        const long long q = i >> 5;
        const int kb = (int) (q % kblocks), co = (int) (q / kblocks);
        const int fw = kb % wf, fh = (kb / wf) % hf, g = kb / (wf * hf);
        const int ch = g * 32 + c;
        float h = 0.f, l = 0.f;
        if (ch < cin) split_tf32(__ldg(F + (((long long) co * cin + ch) * hf + fh) * wf + fw), h, l);
        hi[i] = h;
        lo[i] = l;
    }
}

// The positions of a tile come from up to three images: a segment is a run of consecutive positions
// [p0, p0 + n) of image img, served by one input box that starts at the (16-byte aligned) beginning of
// the first input row the run needs.
struct Seg {
    int img, p0, n, x_al, dx;
};
__device__ __forceinline__ int tile_segments(const ConvArgs& a, long long tile, Seg* seg, int& nt, int& npos) {
    nt = (int) (tile % a.ntiles);
    const long long mt = tile / a.ntiles;
    int count = 0;
    if (a.flat) {
        long long fp = mt * BM;
        npos = (int) min((long long) BM, a.positions - fp);
        int left = npos;
        while (left > 0 && count < 3) {
            Seg& s = seg[count++];
            s.img = (int) (fp / a.plane);
            s.p0 = (int) (fp - (long long) s.img * a.plane);
            s.n = min(left, a.plane - s.p0);
            fp += s.n;
            left -= s.n;
        }
    } else {
        const int oh0 = (int) (mt % a.groups) * a.rows_per_tile;
        npos = min(a.rows_per_tile, a.Ho - oh0) * a.Wo;
        seg[0].img = (int) (mt / a.groups);
        seg[0].p0 = oh0 * a.Wo;
        seg[0].n = npos;
        count = 1;
    }
    for (int i = 0; i < count; i++) {
        const int x = (seg[i].p0 / a.Wo - a.pad) * a.W;  // first input row of the run, as an index into the image plane
        seg[i].dx = ((x % 4) + 4) % 4;                   // TMA needs a 16-byte aligned start; the remainder is added when reading
        seg[i].x_al = x - seg[i].dx;
    }
    return count;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_tf32x3_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_f_hi,
                   const __grid_constant__ CUtensorMap map_f_lo, const ConvArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t* raws = tiles + a.stages * a.stage_bytes;
    uint64_t* bars = (uint64_t*) (raws + a.ring * a.raw_bytes);
    // bars: full [S], empty [S], raw full [R], raw empty [R], accumulator full x2, accumulator empty x2
    uint32_t* tmem_slot = (uint32_t*) (bars + 24);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);
    volatile int* sync_flags = abort_flag + 1;

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
            mbar_init(full_bar(s), 2);   // the producing group's representative + the filter loader's expect_tx
            mbar_init(empty_bar(s), 1);  // tcgen05.commit
        }
        for (int r = 0; r < R; r++) {
            mbar_init(raw_full_bar(r), 1);
            mbar_init(raw_empty_bar(r), GROUPS);
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

    const int taps = a.hf * a.wf;

    if (warp == 0) {
        // --------------------------------------------------------- MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            TIMER_DECL;
            for (long long tile = blockIdx.x; ok && tile < a.tiles; tile += gridDim.x, local++) {
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
                    const uint32_t p_hi = tmem_base + (uint32_t) (a.a_col0 + stage * A_COLS), p_lo = p_hi + BK;
                    const uint64_t f_hi = make_kmajor_sw128_desc(base);
                    const uint64_t f_lo = make_kmajor_sw128_desc(base + a.b_plane);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        const uint64_t adv = (uint64_t) (k * UMMA_K * 4 >> 4);
                        const uint32_t col = (uint32_t) (k * UMMA_K);  // one column per TF32 element
                        umma_tf32_ts(d_tmem, p_lo + col, f_hi + adv, a.idesc, accumulate);
                        umma_tf32_ts(d_tmem, p_hi + col, f_lo + adv, a.idesc, 1);
                        umma_tf32_ts(d_tmem, p_hi + col, f_hi + adv, a.idesc, 1);
                        accumulate = 1;
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
        // ------------------------------------------------ loader of input boxes
        if (lane == 0) {
            int r = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < a.tiles; tile += gridDim.x) {
                Seg seg[3];
                int nt, npos;
                const int nseg = tile_segments(a, tile, seg, nt, npos);
                for (int g = 0; g < a.ncg; g++) {
                    TIMER_DECL;
                    TIMER_START();
                    ok = mbar_wait(raw_empty_bar(r), phase ^ 1, abort_flag, a.status_word, 500 + r);
                    TIMER_ADD(3);
                    if (!ok) break;
                    mbar_expect_tx(raw_full_bar(r), (uint32_t) (nseg * a.box_bytes));
                    for (int i = 0; i < nseg; i++)
                        tma_load_3d(smem_u32(raws + r * a.raw_bytes + i * a.box_bytes), &map_in, seg[i].x_al, g * 32, seg[i].img,
                                    raw_full_bar(r));
                    if (++r == R) { r = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                const unsigned long long t0 = global_ns();
                for (int q = 0; q < R; q++) {
                    const uint32_t armed = (q < r) ? phase : (phase ^ 1);
                    while (!mbar_try_wait(raw_full_bar(q), armed) && (long long) (global_ns() - t0) < 20000000LL) {}
                }
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------- loader of filter slices
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < a.tiles; tile += gridDim.x) {
                const int nt = (int) (tile % a.ntiles);
                for (int kb = 0; kb < a.kblocks; kb++) {
                    TIMER_DECL;
                    TIMER_START();
                    ok = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, a.status_word, 700 + stage);
                    TIMER_ADD(4);
                    if (!ok) break;
                    const uint32_t base = smem_u32(tiles + stage * a.stage_bytes);
                    mbar_expect_tx(full_bar(stage), (uint32_t) (2 * a.b_plane));
                    tma_load_2d(base, &map_f_hi, kb * BK, nt * a.bn, full_bar(stage));
                    tma_load_2d(base + (uint32_t) a.b_plane, &map_f_lo, kb * BK, nt * a.bn, full_bar(stage));
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                const unsigned long long t0 = global_ns();
                for (int q = 0; q < S; q++) {
                    const uint32_t armed = (q < stage) ? phase : (phase ^ 1);
                    while (!mbar_try_wait(full_bar(q), armed) && (long long) (global_ns() - t0) < 20000000LL) {}
                }
            }
        }
    } else if (warp >= FIRST_EPI_WARP && warp < FIRST_PROD_WARP) {
        // ----------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        const int pos = quarter * 32 + lane;
        const int chunks = (a.bn + 31) / 32;
        const long long plane = (long long) a.Ho * a.Wo;
        int local = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < a.tiles; tile += gridDim.x, local++) {
            Seg seg[3];
            int nt, npos;
            const int nseg = tile_segments(a, tile, seg, nt, npos);
            const int buf = local & 1;
            TIMER_DECL;
            TIMER_START();
            if (warp == FIRST_EPI_WARP && lane == 0)
                sync_flags[1 + buf] = mbar_wait(acc_full_bar(buf), (local >> 1) & 1, abort_flag, a.status_word, 400 + buf) ? 1 : 0;
            named_barrier_sync(3, EPI_WARPS * 32);
            if (warp == FIRST_EPI_WARP && lane == 0) TIMER_ADD(5);
            TIMER_START();
            ok = sync_flags[1 + buf] != 0;
            if (!ok) break;
            tcgen05_fence_after();
            if (quarter * 32 >= npos) {  // none of this warp's positions exists
                tcgen05_fence_before();
                if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                continue;
            }
            const uint32_t t_addr = tmem_base + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (buf * a.acc_stride);
            // this thread's position: which image, where in its plane
            float* dst0 = a.out;
            for (int i = 0, first = 0; i < nseg; first += seg[i].n, i++)
                if (pos >= first && pos < first + seg[i].n)
                    dst0 = a.out + ((long long) seg[i].img * a.cout) * plane + seg[i].p0 + (pos - first);
            float v[32];
#pragma unroll 1
            for (int c = 0; c < chunks; c++) {
                float w[32];
                tmem_ld32(t_addr + (uint32_t) (c * 32), v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j++) w[j] = v[j];
                if (c + 1 == chunks) {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                }
                if (pos < npos) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int co = nt * a.bn + c * 32 + j;
                        if (c * 32 + j < a.bn && co < a.cout)
                            dst0[(long long) co * plane] = a.bias ? w[j] + __ldg(a.bias + co) : w[j];
                    }
                }
            }
            if (warp == FIRST_EPI_WARP && lane == 0) TIMER_ADD(6);
        }
    } else if (warp >= FIRST_PROD_WARP) {
        // ----------------------------------------------------------- producers
        // Two groups of four warps take the stages in turn (group g builds every second 32-deep
        // slice), so that one slice is being built while the previous one is being published.
        // Inside a group thread i owns output position i, which is also lane i of tensor memory:
        // consecutive lanes are consecutive positions, so the reads of the box are contiguous.
        const int t = threadIdx.x - 32 * FIRST_PROD_WARP;
        const int grp = t / GROUP_THREADS, pos = t % GROUP_THREADS;
        const int bar_id = 1 + grp;
        const uint32_t chan_stride = (uint32_t) a.box_w * 4u;
        long long kcount = 0, rcount = 0;  // slices and input boxes consumed so far by this CTA
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < a.tiles; tile += gridDim.x) {
            Seg seg[3];
            int nt, npos;
            const int nseg = tile_segments(a, tile, seg, nt, npos);
            // this thread's position: which box, and where in it tap (0, 0) of the position lies
            const bool live = pos < npos;
            int ow = 0, lin0 = 0;
            uint32_t box_off = 0;
            for (int i = 0, first = 0; i < nseg; first += seg[i].n, i++)
                if (pos >= first && pos < first + seg[i].n) {
                    const int p = seg[i].p0 + (pos - first);
                    const int oh = p / a.Wo;
                    ow = p - oh * a.Wo;
                    lin0 = (oh - seg[i].p0 / a.Wo) * a.W + ow - a.pad + seg[i].dx;
                    box_off = (uint32_t) (i * a.box_bytes);
                }
            for (int g = 0; ok && g < a.ncg; g++, rcount++) {
                const int r = (int) (rcount % R);
                const uint32_t raw_phase = (uint32_t) ((rcount / R) & 1);
                bool box_seen = false;
                for (int tap = 0; tap < taps; tap++, kcount++) {
                    if ((int) (kcount % GROUPS) != grp) continue;
                    const int stage = (int) (kcount % S);
                    const uint32_t phase = (uint32_t) ((kcount / S) & 1);
                    TIMER_DECL;
                    TIMER_START();
                    if (pos == 0) {
                        bool mine = true;
                        if (!box_seen) mine = mbar_wait(raw_full_bar(r), raw_phase, abort_flag, a.status_word, 600 + r);
                        if (pos == 0 && grp == 0) TIMER_ADD(7);
                        if (mine) mine = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, a.status_word, 100 + stage);
                        sync_flags[3 + grp] = mine ? 1 : 0;
                    }
                    if (pos == 0 && grp == 0) TIMER_ADD(8);
                    named_barrier_sync(bar_id, GROUP_THREADS);
                    ok = sync_flags[3 + grp] != 0;
                    if (!ok) break;
                    box_seen = true;
                    tcgen05_fence_after();  // the MMAs that read this slice of tensor memory have completed
                    if (pos == 0 && grp == 0) TIMER_ADD(9);
                    {
                        // every lane runs the stores (they are warp-wide); positions that do not exist and
                        // taps that fall beside the image contribute zeros
                        const int fh = tap / a.wf, fw = tap - fh * a.wf;
                        const int col = ow - a.pad + fw;
                        const bool inside = live && col >= 0 && col < a.W;
                        const uint32_t src = smem_u32(raws + r * a.raw_bytes) + box_off + (uint32_t) (lin0 + fh * a.W + fw) * 4u;
                        // this thread's lane of tensor memory is its position; columns are the 32 channels, hi then lo
                        const uint32_t dst = tmem_base + ((uint32_t) (pos & ~31) << 16) + (uint32_t) (a.a_col0 + stage * A_COLS);
#pragma unroll
                        for (int half = 0; half < 2; half++) {
                            float vals[16], h[16], l[16];
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                vals[j] = inside ? ld_shared_f32(src + (uint32_t) (half * 16 + j) * chan_stride) : 0.f;
#pragma unroll
                            for (int j = 0; j < 16; j++) split_tf32(vals[j], h[j], l[j]);
                            tmem_st16(dst + (uint32_t) (half * 16), h);
                            tmem_st16(dst + (uint32_t) (BK + half * 16), l);
                        }
                        tmem_st_wait();
                    }
                    if (pos == 0 && grp == 0) TIMER_ADD(10);
                    tcgen05_fence_before();
                    if (pos == 0 && grp == 0) TIMER_ADD(11);
                    named_barrier_sync(bar_id, GROUP_THREADS);
                    if (pos == 0) mbar_arrive(full_bar(stage));
                    if (pos == 0 && grp == 0) TIMER_ADD(12);
                }
                if (!ok) break;
                if (!box_seen) {
                    // no slice of this box fell to this group (1 x 1 filters): still wait for the box before
                    // releasing it, so that a release can never overtake the load it belongs to
                    if (pos == 0)
                        sync_flags[3 + grp] = mbar_wait(raw_full_bar(r), raw_phase, abort_flag, a.status_word, 650 + r) ? 1 : 0;
                    named_barrier_sync(bar_id, GROUP_THREADS);
                    ok = sync_flags[3 + grp] != 0;
                    if (!ok) break;
                }
                if (pos == 0) mbar_arrive(raw_empty_bar(r));  // this group is done with the box
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

// Shared-memory and tensor-memory layout for a tiling whose tiles touch `segs` images and need
// `rows` input-row spans per image; false when it does not fit.
bool layout(ConvArgs& a, int segs, int span_rows) {
    a.segs = segs;
    a.box_w = ((span_rows + a.hf - 1) * a.W + 3 + 3) / 4 * 4;  // +3 floats of alignment slack, rounded to 16 bytes
    if (a.box_w > 256) return false;                            // TMA boxes hold at most 256 elements per dimension
    a.box_bytes = a.box_w * 32 * 4;
    a.raw_bytes = segs * a.box_bytes;
    a.b_plane = a.bn * 128;
    a.stage_bytes = 2 * a.b_plane;
    const int fixed = 1024 + 256;
    // tensor memory: two accumulators, the rest is the ring of patch-operand slices (64 columns each)
    a.acc_stride = (a.bn + 31) / 32 * 32;
    a.a_col0 = 2 * a.acc_stride;
    a.tmem_cols = 512;
    a.stages = std::min(6, (a.tmem_cols - a.a_col0) / A_COLS);
    a.ring = std::min(MAX_RING, (MAX_SMEM - fixed - a.stages * a.stage_bytes) / a.raw_bytes);
    while (a.ring < 2 && a.stages > 2) {  // trade a split stage for input boxes
        a.stages--;
        a.ring = std::min(MAX_RING, (MAX_SMEM - fixed - a.stages * a.stage_bytes) / a.raw_bytes);
    }
    return a.ring >= 2 && a.stages >= 2;
}

// Geometry of the launch; returns false when the convolution does not fit this kernel.
bool plan(ConvArgs& a, const float* in, int batch, int cin, int H, int W, int cout, int hf, int wf, int stride, int pad,
          int sm_count) {
    if (stride != 1) return false;
    a.batch = batch; a.cin = cin; a.H = H; a.W = W; a.cout = cout; a.hf = hf; a.wf = wf; a.pad = pad;
    a.Ho = H + 2 * pad - hf + 1;
    a.Wo = W + 2 * pad - wf + 1;
    if (a.Ho < 1 || a.Wo < 1 || a.Wo > BM) return false;
    if (((long long) H * W) % 4 != 0 || ((uintptr_t) in) % 16 != 0) return false;  // TMA: channel stride in 16-byte units
    if ((long long) H * W * 4 >= (1LL << 32) || (long long) cin * H * W * 4 >= (1LL << 40)) return false;
    a.plane = a.Ho * a.Wo;
    a.positions = (long long) batch * a.plane;
    a.bn = cout >= 128 ? 128 : (cout + 15) / 16 * 16;
    a.ntiles = (cout + a.bn - 1) / a.bn;
    a.ncg = (cin + 31) / 32;
    a.kblocks = a.ncg * hf * wf;
    a.idesc = make_idesc_tf32(BM, a.bn);

    // (a) tiles of whole output rows of one image: at most 128 positions, input box at most 256 floats
    int rows = std::min(a.Ho, BM / a.Wo);
    rows = std::min(rows, 253 / W - hf + 1);
    const bool rows_ok = rows >= 1;
    const long long row_tiles = rows_ok ? (long long) batch * ((a.Ho + rows - 1) / rows) * a.ntiles : 0;
    // (b) tiles of 128 consecutive positions of the whole batch: full tiles whatever Ho * Wo is, but a run of
    // 128 positions can start in the middle of a row and cross into the next images
    const int span = std::min(a.Ho, (BM + a.Wo - 2) / a.Wo + 1);
    const int segs = a.plane >= BM ? 2 : a.plane >= BM / 2 ? 3 : 0;  // images a run of 128 positions can touch
    const long long flat_tiles = (a.positions + BM - 1) / BM * a.ntiles;
    ConvArgs f = a;
    f.flat = 1;
    const bool flat_ok = segs > 0 && option_get(OPT_CONV_ROUTE) != 2 && layout(f, segs, span);
    // flat tiles when they save a round of tiles on the machine (or when row tiles do not fit at all)
    const long long sms = std::max(sm_count, 1);
    const bool take_flat = flat_ok && (!rows_ok || option_get(OPT_CONV_ROUTE) == 3 ||
                                       (flat_tiles + sms - 1) / sms < (row_tiles + sms - 1) / sms);
    if (take_flat) {
        a = f;
        a.tiles = flat_tiles;
        return true;
    }
    if (!rows_ok) return false;
    a.flat = 0;
    a.rows_per_tile = rows;
    a.groups = (a.Ho + rows - 1) / rows;
    a.tiles = row_tiles;
    return layout(a, 1, rows);
}

}  // namespace

int conv_tf32x3_describe(int batch, int cin, int H, int W, int cout, int hf, int wf, int stride, int pad, int sm_count,
                         cakeb200_conv_plan* out) {
    ConvArgs a = {};
    memset(out, 0, sizeof(*out));
    out->route = 2;
    if (!plan(a, nullptr, batch, cin, H, W, cout, hf, wf, stride, pad, sm_count > 0 ? sm_count : 148)) return CAKEB200_OK;
    out->route = a.flat ? 1 : 0;
    out->tiles = (int) a.tiles;
    out->channel_tile = a.bn;
    out->positions_tile = a.flat ? BM : a.rows_per_tile * a.Wo;
    out->k_slices = a.kblocks;
    out->stages = a.stages;
    out->ring = a.ring;
    out->smem_bytes = a.stages * a.stage_bytes + a.ring * a.raw_bytes + 1024 + 256;
    return CAKEB200_OK;
}

bool conv_tf32x3_fits(const float* in, int batch, int cin, int H, int W, int cout, int hf, int wf, int stride, int pad) {
    ConvArgs a = {};
    return plan(a, in, batch, cin, H, W, cout, hf, wf, stride, pad, 148);
}

size_t conv_tf32x3_scratch_bytes(int cin, int cout, int hf, int wf) {
    const size_t kp = (size_t) ((cin + 31) / 32) * hf * wf * 32;
    return 2 * ((size_t) cout * kp * 4 + 1024) + 1024;
}

// out[batch][cout][Ho][Wo] = conv(in[batch][cin][H][W], filters[cout][cin][hf][wf]) (+ bias per channel), stride 1.
int launch_conv_tf32x3(const float* in, const float* filters, float* out, const float* bias, int batch, int cin, int H,
                       int W, int cout, int hf, int wf, int pad, void* scratch, size_t scratch_bytes, int* status_word,
                       int sm_count, cudaStream_t stream, int* launches) {
    ConvArgs a = {};
    if (!plan(a, in, batch, cin, H, W, cout, hf, wf, 1, pad, sm_count)) {
        set_error("conv_tf32x3: this geometry is not covered by the implicit kernel");
        return CAKEB200_ERR_ARG;
    }
    if (conv_tf32x3_scratch_bytes(cin, cout, hf, wf) > scratch_bytes) {
        set_error("conv_tf32x3: scratch too small");
        return CAKEB200_ERR_ARG;
    }
    a.out = out;
    a.bias = bias;
    a.status_word = status_word;
    const long long kp = (long long) a.kblocks * 32;
    const size_t plane_bytes = ((size_t) cout * kp * 4 + 1023) / 1024 * 1024;
    float* f_hi = (float*) (((uintptr_t) scratch + 1023) / 1024 * 1024);
    float* f_lo = (float*) ((char*) f_hi + plane_bytes);
    const long long total = (long long) cout * kp;
    const int blocks = (int) std::min<long long>((total + 255) / 256, 148 * 8);
    split_filters_kernel<<<blocks, 256, 0, stream>>>(filters, f_hi, f_lo, cout, cin, hf, wf, a.kblocks);
    CAKE_CUDA_OK(cudaGetLastError());

    alignas(64) CUtensorMap map_in, map_hi, map_lo;
    int rc;
    {
        const unsigned long long d[3] = {(unsigned long long) H * W, (unsigned long long) cin, (unsigned long long) batch};
        const unsigned long long s[2] = {(unsigned long long) H * W * 4, (unsigned long long) cin * H * W * 4};
        const unsigned b[3] = {(unsigned) a.box_w, 32u, 1u};
        if ((rc = encode_tiled_f32(&map_in, in, 3, d, s, b, false))) return rc;
    }
    {
        const unsigned long long d[2] = {(unsigned long long) kp, (unsigned long long) cout};
        const unsigned long long s[1] = {(unsigned long long) kp * 4};
        const unsigned b[2] = {(unsigned) BK, (unsigned) a.bn};
        if ((rc = encode_tiled_f32(&map_hi, f_hi, 2, d, s, b, true))) return rc;
        if ((rc = encode_tiled_f32(&map_lo, f_lo, 2, d, s, b, true))) return rc;
    }
    const int smem = a.stages * a.stage_bytes + a.ring * a.raw_bytes + 1024 + 256;
    CAKE_CUDA_OK(cudaFuncSetAttribute(conv_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int grid = (int) std::min<long long>(a.tiles, sm_count);
    conv_tf32x3_kernel<<<grid, NUM_THREADS, smem, stream>>>(map_in, map_hi, map_lo, a);
    CAKE_CUDA_OK(cudaGetLastError());
    if (launches) *launches += 2;
#ifdef CAKEB200_ROLE_TIMERS
    {
        unsigned long long h[16];
        cudaStreamSynchronize(stream);
        cudaMemcpy(h, status_word + 16, sizeof(h), cudaMemcpyDeviceToHost);
        cudaMemset(status_word + 16, 0, sizeof(h));
        fprintf(stderr, "conv role timers (cycles, CTA 0): mma[wait_acc %llu wait_full %llu issue %llu] raw_loader[wait %llu] "
                "filter_loader[wait %llu] epilogue[wait %llu work %llu] producer0[raw %llu +empty %llu +bar %llu +convert %llu "
                "+fence %llu +publish %llu] kblocks/CTA %lld\n", h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[7], h[8], h[9],
                h[10], h[11], h[12], (a.tiles + grid - 1) / grid * a.kblocks);
    }
#endif
    return CAKEB200_OK;
}

}  // namespace cakeb200
