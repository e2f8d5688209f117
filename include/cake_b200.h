/* cake_b200.h -- the C ABI of the B200 implementation of the CAKE SGEMM path.
 *
 * Plain pointers and sizes only.  Every matrix is FP32, row-major, dense, with
 * the leading dimension equal to its column count (A[m*K+k], B[k*N+n],
 * C[m*N+n]) exactly as in vnatesh/CAKE_on_CPU (src/util.cpp:183).  Each data
 * pointer may be a HOST pointer (pageable or pinned) or a DEVICE pointer of the
 * current CUDA device; host operands are copied to the device and the result is
 * copied back inside the call.  All entry points return CAKEB200_OK (0) or a
 * negative status; cakeb200_last_error() gives the text.  Nothing here calls
 * exit() and no kernel traps: device-side waits are bounded and report through
 * CAKEB200_ERR_DEVICE_TIMEOUT.
 *
 * The C++ API of the reference (include/cake.h of this repository, same
 * prototypes as the reference's include/cake.h:12-76) is a thin layer over
 * these functions.
 */
#ifndef CAKE_B200_H
#define CAKE_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    CAKEB200_OK = 0,
    CAKEB200_ERR_ARG = -1,            /* bad size / null pointer / unknown enum */
    CAKEB200_ERR_CUDA = -2,           /* a CUDA runtime call failed */
    CAKEB200_ERR_NO_DEVICE = -3,      /* no usable sm_100 device */
    CAKEB200_ERR_DEVICE_TIMEOUT = -4, /* a bounded device-side wait gave up */
    CAKEB200_ERR_TOO_LARGE = -5       /* exceeds a documented fixed limit */
};

/* Block schedules, same numbering as `enum sched` (reference include/common.h:105). */
enum { CAKEB200_SCHED_KMN = 0, CAKEB200_SCHED_MKN = 1, CAKEB200_SCHED_NKM = 2, CAKEB200_SCHED_NA = 3 };

/* Which arithmetic kernel computes the contraction. */
enum {
    CAKEB200_KERNEL_AUTO = 0,
    CAKEB200_KERNEL_TF32X3 = 1, /* tcgen05 tensor cores, FP32 split into two TF32 terms, 3 MMAs */
    CAKEB200_KERNEL_FFMA = 2    /* exact FP32 fused multiply-add on the CUDA cores */
};

/* Timings of the last call on this thread, milliseconds, from CUDA events. */
typedef struct cakeb200_stats {
    float ms_h2d;     /* host -> device copies (0 for device operands) */
    float ms_prepass; /* operand split / pack kernels */
    float ms_gemm;    /* the contraction kernel(s) */
    float ms_d2h;     /* device -> host copy of the result */
    int kernel;       /* CAKEB200_KERNEL_* that ran */
    int sched;        /* CAKEB200_SCHED_* that ordered the tiles */
    int tile_m, tile_n, tile_k;
    int launches;     /* kernels of this library launched by the call */
} cakeb200_stats;

/* Machine description the block-sizing formulas consume; mirrors the fields of
 * cake_cntx_t that the reference reads (reference include/common.h:138-151). */
typedef struct cakeb200_cntx {
    double alpha_n;
    int mr, nr;
    int L1, L2, L3;
    int ncores;
} cakeb200_cntx;

/* Field-for-field the reference's blk_dims_t (reference include/common.h:108-135). */
typedef struct cakeb200_blk_dims {
    int m_c, k_c, n_c, m_c1, k_c1, n_c1;
    int m_c1_last_core, n_c1_last_core, k_c1_last_core;
    int mr_rem, nr_rem, k_rem;
    int p_l, pm_l, pn_l, pm, pn;
    int m_pad, k_pad, n_pad;
    int Mb, Kb, Nb;
    int M_padded, N_padded;
    int sch;
} cakeb200_blk_dims;

const char* cakeb200_last_error(void);
void cakeb200_get_stats(cakeb200_stats* out);

/* Number of visible CUDA devices with compute capability 10.x. */
int cakeb200_device_count(void);

/* The devices a host-pointer product with p > 1 is spread over by the C++ API (in the reference p
 * is the OpenMP thread count, src/cake_sgemm.cpp:19; here it bounds the GPUs).  cc_major[d] is the
 * compute-capability major of visible device d; the result starts with `current` (when it is a
 * 10.x device) and continues with the other 10.x devices in ordinal order, at most
 * min(p, cap if cap > 0, M / 512) of them; returns how many were written to `out` (room for
 * n_devices).  `cap` is the CAKE_NGPU environment variable in the C++ API.  Pure host logic. */
int cakeb200_select_devices(const int* cc_major, int n_devices, int current, int p, int cap, int M, int* out);

/* Fills a context for the current device: L1 = shared memory per SM,
 * L2 = device L2 bytes, L3 = min(HBM bytes, INT_MAX), ncores = visible devices,
 * mr x nr = 128 x 256 (the MMA tile).  Replaces cake_query_cntx()
 * (reference src/block_sizing.cpp:40-75). */
int cakeb200_query_cntx(cakeb200_cntx* out);

/* Measured dense TF32 tensor rate of the current device, TFLOP/s: every SM issues
 * tcgen05.mma kind::tf32 128 x 256 x 8 back to back on operand tiles resident in shared
 * memory for about `ms_target` milliseconds (<= 0: about 2 ms, and the result of an earlier
 * call on this device is returned if there is one).  The 3xTF32 product issues three MMAs per
 * FP32-class multiply-add, so its roofline is a third of this figure.  `ms` (optional) receives
 * the duration of the measured launch.  Replaces the machine peak the reference hard-codes in
 * its context (peak_flops = 600e9, reference src/block_sizing.cpp:49-50). */
int cakeb200_tf32_peak(float ms_target, float* tflops, float* ms, void* stream);

/* C = A*B (accumulate == 0) or C += A*B (accumulate != 0).
 * Replaces cake_sgemm() (reference src/cake_sgemm.cpp:9-175; prototype
 * include/cake.h:12-14).  `sched` orders the output tiles (KMN: K innermost
 * per tile with a snake over tiles; MKN: M-fastest; NKM: N-fastest; NA: derive
 * from the shape as derive_schedule does, reference src/block_sizing.cpp:434-462).
 * `stream` is a cudaStream_t (NULL = the CUDA default stream, as in the CUDA
 * runtime); work is ordered after what the caller queued on that stream before
 * the call, and the call returns after its own work has finished.  Host
 * operands with many rows are streamed in bands of rows: band i is multiplied
 * while band i+1 is still being copied in and band i-1 is being copied out. */
int cakeb200_sgemm(const float* A, const float* B, float* C, int M, int N, int K,
                   int accumulate, int sched, int kernel, void* stream);

/* cakeb200_sgemm for a B that is still being completed when the call is made: the kernels of the
 * call wait for `b_ready` (a cudaEvent_t already recorded by the caller; NULL = nothing to wait for)
 * in addition to the work queued on `stream`, while host rows of A start moving to the device at
 * once.  For one product spread over several GPUs, where each GPU copies its own slice of B from the
 * host and the slices are gathered from the peers over NVLink into a B in this GPU's memory
 * (the reference shares one packed B among all its cores, reference
 * src/cake_sgemm_k_first.cpp:85-129): the gather runs on another stream and records `b_ready`. */
int cakeb200_sgemm_after(const float* A, const float* B, float* C, int M, int N, int K,
                         int accumulate, int sched, int kernel, void* stream, void* b_ready);

/* Overrides of the large-matrix kernel's own choices, process-wide, 0 = back to the library's rule:
 *   "tile_n"   128 or 256: columns of C per tile;
 *   "band"     tile rows (columns for N-first) per band of the tile walk (rule: 8);
 *   "k_pieces" K ranges each tile of the ragged last wave is cut into (rule: a cost model);
 *   "chunk_kb" 32-deep slices of K accumulated in tensor memory before they are folded into the
 *              FP32 running sum (rule: 32, i.e. 1024 of K; a value >= K / 32 means one unbroken
 *              accumulation, which is 0 to 4 % faster and whose truncation error grows with K);
 * and, so that tests can reach every code path of the other kernels:
 *   "conv_route" 1 = im2col planes + the large-matrix kernel, 2 / 3 = the implicit kernel tiled by
 *              whole rows of one image / by runs of 128 positions across images (rule: by geometry);
 *   "small_operands" of the batched tensor-core kernel: 1 = A's split planes in shared memory
 *              instead of tensor memory, 2 = operands read from global memory instead of by TMA;
 *   "pack_scalar" 1 = pack / unpack move one element per thread instead of 16 bytes.
 *   "pair"      form of the large-matrix tensor-core kernels: 1 = 256-row tiles on pairs of SMs
 *               (tcgen05 cta_group::2) wherever the product has more than 128 rows, 2 = always one
 *               CTA per 128-row tile; rule: pairs for 256-wide tiles, unless padding M to a multiple
 *               of 256 instead of 128 adds more than 7 % of rows.  Both forms give the same bits when no tile is
 *               cut along K ("k_pieces" 1).
 * They take the place of the block sizes a caller of the reference forces with mcu / kcu / ncu
 * (reference include/cake.h:12-14, src/block_sizing.cpp:363-368) and of update_mr_nr
 * (src/block_sizing.cpp:78-83): on a GPU the blocks a caller may pin are the tile, the walk and
 * the cut along K.  The tuning cache (cakeb200_tune) applies them per shape.  cakeb200_get_option
 * returns the override in force, -1 for an unknown name. */
int cakeb200_set_option(const char* name, int value);
int cakeb200_get_option(const char* name);

/* ---- An operand kept in the kernel's preferred form across products.
 *
 * The reference lets a caller pack an operand once and pass packedA / packedB = 1 to every later
 * cake_sgemm (reference src/cake_sgemm.cpp:40-85 skips pack_A / pack_B then; used with stationary
 * weights in examples/cake_conv.cpp:1032-1055).  The tensor-core kernel's preferred form is not a
 * blocked copy but the operand's two TF32 planes (hi = tf32(v), lo = tf32(v - hi), K-major), so that
 * is what is kept: cakeb200_planes_create splits a matrix once into device memory owned by the object
 * (is_b == 0: `mat` is A, rows x K row-major; is_b != 0: `mat` is B, K x rows row-major, and its
 * transposed planes are stored), and cakeb200_sgemm_planes multiplies with planes standing in for A,
 * for B or for both (pass NULL for the planes of an operand that is given as a matrix, and the matrix
 * pointer may be NULL where planes are given).  The operand's split pass, a third of the time of a
 * product with little reuse, is then not repeated.  Host or device pointers for the matrices and C;
 * the call blocks like cakeb200_sgemm.  The C++ API's pack_A / pack_B record such planes next to the
 * layout-exact packed buffer, which is how cake_sgemm(..., packedA = 1) finds them. */
typedef struct cakeb200_planes cakeb200_planes;
int cakeb200_planes_create(const float* mat, int rows, int K, int is_b, cakeb200_planes** out, void* stream);
int cakeb200_planes_destroy(cakeb200_planes* p);
int cakeb200_sgemm_planes(const cakeb200_planes* A_planes, const float* A, const cakeb200_planes* B_planes, const float* B,
                          float* C, int M, int N, int K, int accumulate, int sched, void* stream);

/* ---- Tile-shape selection with a persistent cache.
 *
 * Replaces the reference's block-size autotuner (reference src/autotune_sa.cpp:13-82 and
 * include/autotune.h:82-86: random-step search over (m_c, k_c, n_c) with a visited set; dead
 * code there, not compiled by its Makefile).  On a GPU the blocks worth searching are the tile
 * width, the cluster shape (one or two CTAs per tile), the band height of the tile walk and the
 * cut of the last wave's tiles along K.
 *
 * cakeb200_tune times the large-matrix kernel on the caller's operands (device pointers; C is
 * overwritten with the product every time) at up to `trials` points of that grid, walking it by
 * random steps from the rule's own choice; the fastest point is then run in turns with the rule's
 * choice and recorded for (M, N, K, schedule) when it is at least 3 % faster, else the rule itself
 * is recorded (tile_n = 0); later products of that shape use the entry.  After the call cakeb200_get_stats reports the winning
 * tile_n, its time (ms_gemm) and the points evaluated (launches).  Explicit options
 * (cakeb200_set_option) still win over the cache.  The search changes the process-wide options
 * while it runs: no other thread should multiply meanwhile.
 *
 * The cache lives in the process; _save / _load write and read it as JSON (they return the number
 * of entries, or a negative status), and the file named by the environment variable
 * CAKE_AUTOTUNE_CACHE is loaded on first use and rewritten after every cakeb200_tune.  _put / _get
 * / _clear edit it directly (_get returns 1 when the shape has an entry, else 0); `sched` is a
 * resolved schedule (KMN, MKN or NKM).
 *
 * cakeb200_tune_search is the search alone, host logic: `cost` returns the time of a point in
 * milliseconds (<= 0: not a valid point) and may be anything, which is how the search is tested
 * without a device. */
typedef double (*cakeb200_tune_cost)(int tile_n, int band, int k_pieces, void* user);
/* The _shape forms add the cluster shape to the grid: `cluster` 1 = the two CTAs of a thread-block
 * cluster on one 256-row tile (a pair of SMs), 2 = one CTA per 128-row tile, 0 = the library's rule
 * (the "pair" option has the same values).  cakeb200_tune searches and records all four choices;
 * the forms without _shape leave the cluster shape to the rule. */
typedef double (*cakeb200_tune_cost_shape)(int tile_n, int cluster, int band, int k_pieces, void* user);
int cakeb200_tune_search_shape(int M, int N, int K, int sm_count, int trials, unsigned long long seed,
                               cakeb200_tune_cost_shape cost, void* user, int* tile_n, int* cluster, int* band,
                               int* k_pieces, float* best_ms, int* evaluated);
int cakeb200_tune_put_shape(int M, int N, int K, int sched, int tile_n, int cluster, int band, int k_pieces, float ms);
int cakeb200_tune_get_shape(int M, int N, int K, int sched, int* tile_n, int* cluster, int* band, int* k_pieces, float* ms);
int cakeb200_tune(const float* A, const float* B, float* C, int M, int N, int K, int sched, int trials, void* stream);
int cakeb200_tune_search(int M, int N, int K, int sm_count, int trials, unsigned long long seed, cakeb200_tune_cost cost,
                         void* user, int* tile_n, int* band, int* k_pieces, float* best_ms, int* evaluated);
int cakeb200_tune_put(int M, int N, int K, int sched, int tile_n, int band, int k_pieces, float ms);
int cakeb200_tune_get(int M, int N, int K, int sched, int* tile_n, int* band, int* k_pieces, float* ms);
int cakeb200_tune_clear(void);
int cakeb200_tune_save(const char* path);
int cakeb200_tune_load(const char* path);

/* Same, but only enqueues on `stream` (device pointers required, no host copies,
 * no synchronisation).  For callers that time or overlap the work themselves.
 * It can be recorded into a CUDA graph by stream capture once the same shape has
 * been called outside a capture (that call sizes the scratch arena and uploads
 * the tile plan); a later call with a shape that needs a larger arena moves the
 * arena and invalidates graphs recorded before, so call the largest shape first. */
int cakeb200_sgemm_async(const float* A, const float* B, float* C, int M, int N, int K,
                         int accumulate, int sched, int kernel, void* stream);

/* C[M x N] (+)= op(A) * op(B) (+ bias) on device operands, enqueued on `stream`.
 * trans_a = 0: A is M x K row-major with leading dimension lda; 1: A points at a
 * K x M row-major matrix (lda >= M) and its transpose is multiplied.  trans_b
 * likewise (0: K x N, ldb >= N; 1: N x K, ldb >= K).  `bias` (length N, or NULL)
 * is added to every row in the kernel's epilogue.  This is the product the
 * reference's PyTorch layer needs without its copies: forward y = x W^T + b with
 * the weight used where it lies (replaces weight.t().contiguous(), the cake_sgemm
 * call and the scalar bias loop of reference src/linear.cpp:22-46), and
 * dW = dY^T X with dY used where it lies (replaces the transposed copy at
 * reference src/linear.cpp:76-84). */
int cakeb200_sgemm_ex(const float* A, int lda, int trans_a, const float* B, int ldb, int trans_b,
                      float* C, int ldc, int M, int N, int K, const float* bias,
                      int accumulate, int sched, int kernel, void* stream);

/* Device-side timing of cakeb200_sgemm_async without synchronising: between
 * _begin and _end every asynchronous product (up to 256) records CUDA events on
 * its stream before the operand-split pass, after it and after the contraction
 * kernel(s); _end waits for the last one and returns the summed durations in
 * milliseconds.  Replaces the reference's DEBUG timing printouts around pack /
 * GEMM / unpack (reference src/cake_sgemm.cpp:32-168). */
int cakeb200_profile_begin(void);
int cakeb200_profile_end(float* ms_prepass, float* ms_kernel, int* calls);

/* `batch` independent products of identical shape, item i at A + i*M*K etc.
 * Replaces the small-matrix entry points cake_gemm_small / schedule_*_small
 * (reference include/cake.h:52-72, src/cake_sgemm_small.cpp:7-236), whose live
 * equivalent in the reference is one cake_sgemm call per item.  `kernel`:
 * CAKEB200_KERNEL_FFMA = exact FP32; CAKEB200_KERNEL_TF32X3 = tensor cores with
 * the operands split inside the kernel (needs M <= 128 and N <= 256);
 * CAKEB200_KERNEL_AUTO picks the tensor-core kernel for a batch that fills most
 * SMs with reasonably full tiles. */
int cakeb200_sgemm_batched(const float* A, const float* B, float* C, int M, int N, int K,
                           int batch, int kernel, void* stream);

/* Self-test of the fault containment: one CTA waits, through the wait routine of the
 * tensor-core kernels, on a barrier that nothing ever signals; after `limit_us`
 * microseconds (1 .. 1e6) the wait gives up, the kernel returns normally and the call
 * reports CAKEB200_ERR_DEVICE_TIMEOUT with "where 900" in the error text.  The device
 * context stays usable.  (The reference stops the process with exit(1) on its errors,
 * reference src/cake_sgemm.cpp:49-52.) */
int cakeb200_selftest_bounded_wait(int limit_us, void* stream);
/* The same for the kernels that run on pairs of SMs: in a cluster of two CTAs the leader waits for
 * an arrival its peer never sends, gives up after `limit_us` ("where 901"), and both CTAs still
 * leave through the cluster barrier that ends those kernels. */
int cakeb200_selftest_bounded_wait_pair(int limit_us, void* stream);

/* ---- One product with K sharded over the GPUs of one box, one process per GPU.
 *
 * For shapes whose M and N are too small to give every GPU its own rows or columns of C
 * (deep, narrow products such as 1024 x 262144 x 1024).  Rank r holds columns
 * [k0, k1) of A and the same rows of B, multiplies them, and while its tiles are being
 * summed stores each row of the partial result straight into the memory of the rank
 * that owns that row (plain stores over NVLink into a slot reserved for rank r); the
 * owner then adds the `world` slots in rank order.  Nothing but those rows crosses the
 * link, no library collective is involved, and the result does not depend on timing.
 * This is the reference's K-first core split (src/cake_sgemm_k_first.cpp:85-129: every
 * core adds its share of K into a private copy of the block, the copies are combined
 * afterwards) with GPUs in place of cores.
 *
 * Rows are owned in whole 128-row tiles: cakeb200_kshard_rows gives [lo, hi) of a rank.
 * Call order on every rank: create -> exchange the 64-byte handles between the
 * processes by any means -> connect_ipc -> any number of (partial, finish) pairs, the
 * same number on every rank, all on one stream -> a barrier of the caller's -> destroy.
 * partial and finish must alternate: a second partial before the finish of the first is
 * refused (CAKEB200_ERR_ARG), because the slots alternate between two sets by product
 * number and an owner may still be reading the set a third product would write.  A finish
 * that gave up waiting leaves the product open: call finish again (the late rank may still
 * arrive) or destroy the object; a new partial is refused until a finish has succeeded.  A
 * partial whose launch failed publishes nothing and does not count.
 * cakeb200_kshard_finish blocks until this rank's rows are complete; it waits at most
 * `wait_limit_us` (0: 2 s) for the other ranks and otherwise returns
 * CAKEB200_ERR_DEVICE_TIMEOUT with "where 910" and the missing rank in the error text,
 * leaving the context usable.  cakeb200_kshard_supported tells (without a device when
 * sm_count > 0) whether a shape is one this path takes: products with few tiles and a
 * deep K; others return CAKEB200_ERR_ARG from cakeb200_kshard_partial and are summed
 * with a reduce-scatter by the caller.  world <= 8.
 *
 * cakeb200_kshard_connect_local wires up objects that all live in this process on one
 * device, so that the whole exchange can be exercised on a single GPU: run `partial` for
 * every rank, then `finish` for every rank. */
#define CAKEB200_IPC_HANDLE_BYTES 64
typedef struct cakeb200_kshard cakeb200_kshard;
int cakeb200_kshard_rows(int M, int world, int rank, int* lo, int* hi);
int cakeb200_kshard_supported(int M, int N, int K_local, int sm_count);
int cakeb200_kshard_create(int world, int rank, int M, int N, cakeb200_kshard** out, unsigned char* ipc_handle);
int cakeb200_kshard_connect_ipc(cakeb200_kshard* x, const unsigned char* handles /* world x 64 bytes, by rank */);
int cakeb200_kshard_connect_local(cakeb200_kshard* x, cakeb200_kshard* const* all /* world objects, by rank */);
int cakeb200_kshard_partial(cakeb200_kshard* x, const float* A, int lda, const float* B, int ldb, int K_local, void* stream);
int cakeb200_kshard_finish(cakeb200_kshard* x, float* C_block, int wait_limit_us, void* stream);
int cakeb200_kshard_destroy(cakeb200_kshard* x);

/* y (+)= A x for an M x K matrix.  col_major != 0: A[k*M + m], the layout of the
 * reference's matrix-vector driver; else row-major A[m*K + k], the N = 1 case of
 * cake_sgemm.  accumulate != 0 adds to y, which is what the reference's driver
 * does with the C it is handed.  Replaces cake_sgemv / schedule_mvm and the
 * 8 x 8 microkernel (reference examples/cake_gemv.cpp:87-140, 424-489, 716-765). */
int cakeb200_sgemv(const float* A, const float* x, float* y, int M, int K, int col_major,
                   int accumulate, void* stream);

/* C = A*B where A is mostly zero: A is compacted on the device to a per-row
 * list of (column, value) and only the nonzeros are multiplied.  Replaces the
 * sparse microkernel cake_sp_sgemm_haswell_6x16 (reference
 * src/kernels/haswell/sparse.cpp:7-131), which the reference never schedules. */
int cakeb200_sp_sgemm(const float* A, const float* B, float* C, int M, int N, int K,
                      int kernel, void* stream);

/* NCHW convolution through im2col + SGEMM: out[b][co][ho][wo].  Replaces the
 * GEMM route of the reference's convolution example (im_2_col + cake_sgemm,
 * reference examples/cake_conv.cpp:1007-1066,1178-1213), extended with batch,
 * stride and zero padding.  On the tensor-core path a stride-1 convolution runs
 * as an implicit product (the patch matrix is built on chip, never in memory);
 * other geometries build split im2col planes first; CAKEB200_KERNEL_FFMA
 * materialises the FP32 im2col matrix and multiplies exactly. */
int cakeb200_conv2d(const float* in, const float* filters, float* out, int batch, int cin,
                    int H, int W, int cout, int hf, int wf, int stride, int pad,
                    int kernel, void* stream);

/* How cakeb200_conv2d lays a convolution out on the tensor-core path (host logic only, needs no device):
 * route 0 = implicit product, tiles of whole output rows of one image; 1 = implicit product, tiles of 128
 * consecutive positions of the batch; 2 = im2col planes + the large-matrix kernel (strides, rows wider than
 * 128 outputs, image areas that are not a multiple of 4 floats).  The other fields describe the implicit
 * kernel's launch (0 for route 2).  The GPU counterpart of choosing m_c / k_c / n_c for the convolution's
 * GEMM (reference examples/cake_conv.cpp:1028-1056 through init_block_dims). */
typedef struct cakeb200_conv_plan {
    int route;
    int tiles;            /* tiles of positions x tiles of channels */
    int channel_tile;     /* output channels per tile (N of the MMA) */
    int positions_tile;   /* positions per tile (at most 128) */
    int k_slices;         /* 32-deep slices of K per tile: ceil(cin / 32) * hf * wf */
    int stages, ring;     /* split stages in tensor memory / shared memory, input boxes in flight */
    int smem_bytes;
} cakeb200_conv_plan;
int cakeb200_conv_plan_query(int batch, int cin, int H, int W, int cout, int hf, int wf, int stride, int pad,
                             int sm_count, cakeb200_conv_plan* out);

/* im2col alone (reference examples/cake_conv.cpp:1178-1213): col[(cin,hf,wf)][(b,ho,wo)]. */
int cakeb200_im2col(const float* in, float* col, int batch, int cin, int H, int W,
                    int hf, int wf, int stride, int pad, void* stream);

/* Block sizing: replaces init_block_dims / get_cache_dims / derive_schedule
 * (reference src/block_sizing.cpp:304-595) and set_schedule
 * (reference src/cake_sgemm.cpp:768-787).  `cntx->alpha_n` is updated as the
 * reference does. */
int cakeb200_init_block_dims(int M, int N, int K, int p, cakeb200_blk_dims* x, cakeb200_cntx* cntx,
                             int sched, int mcu, int kcu, int ncu);
int cakeb200_derive_schedule(int M, int N, int K, int p, int mc_ret, const cakeb200_cntx* cntx);
int cakeb200_set_schedule(int sched, int M, int N, int K);

/* Byte sizes of the packed operands: replaces cake_sgemm_packed_{A,B,C}_size
 * (reference src/pack_helper.cpp:5-87). */
size_t cakeb200_packed_A_size(int M, int K, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* cntx, int sched);
size_t cakeb200_packed_B_size(int K, int N, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* cntx);
size_t cakeb200_packed_C_size(int M, int N, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* cntx, int sched);

/* Layout-exact packing on the device: the output buffer holds exactly the
 * bytes the reference's packers produce for the same block dimensions
 * (padding positions are zero).  Replace pack_A / pack_B / pack_C / unpack_C
 * (reference src/pack_helper.cpp:92-184 and the routines they dispatch to in
 * src/pack_{k,m,n}_first.cpp, src/unpack_{k,m,n}_first.cpp, src/pack_ob.cpp). */
int cakeb200_pack_A(const float* A, float* A_p, int M, int K, int p, const cakeb200_blk_dims* x,
                    const cakeb200_cntx* cntx, void* stream);
int cakeb200_pack_B(const float* B, float* B_p, int K, int N, int p, const cakeb200_blk_dims* x,
                    const cakeb200_cntx* cntx, void* stream);
int cakeb200_pack_C(const float* C, float* C_p, int M, int N, int p, const cakeb200_blk_dims* x,
                    const cakeb200_cntx* cntx, void* stream);
int cakeb200_unpack_C(float* C, const float* C_p, int M, int N, int p, const cakeb200_blk_dims* x,
                      const cakeb200_cntx* cntx, void* stream);
/* Inverses of pack_A / pack_B, used when cake_sgemm is handed pre-packed operands. */
int cakeb200_unpack_A(float* A, const float* A_p, int M, int K, int p, const cakeb200_blk_dims* x,
                      const cakeb200_cntx* cntx, void* stream);
int cakeb200_unpack_B(float* B, const float* B_p, int K, int N, int p, const cakeb200_blk_dims* x,
                      const cakeb200_cntx* cntx, void* stream);

/* C = A*B for callers that must not allocate device memory.  This entry point has
 * no counterpart in the reference; it exists for hosts of this library that are
 * not allowed to touch the allocator when they need a product: code living inside
 * another framework's memory pool, a loop whose memory was budgeted at start-up, a
 * plug-in that is given a stream and buffers and nothing else.  cakeb200_sgemm
 * cannot serve them because it grows its scratch arena with cudaMalloc the first
 * time a larger shape arrives.
 *
 * Same kernels as cakeb200_sgemm with CAKEB200_KERNEL_TF32X3, but the split operand
 * planes live in a fixed device array inside the library image.  The call makes no
 * cudaMalloc, cudaFree or other allocating call.
 *   - A, B, C must be DEVICE pointers (copying a host operand would need a buffer).
 *   - Limit: 1024 + 2*roundup1024(4*M*ceil4(K)) + 2*roundup1024(4*N*ceil4(K)) bytes
 *     must fit in CAKEB200_NOALLOC_SCRATCH_BYTES (17 MiB).  With the arguments in this
 *     function's order: M = N = K = 1024 fits (16 MiB of planes); so does M = 2048,
 *     N = 1024, K = 512 (12 MiB); M = 2048, N = 512, K = 1024 (20 MiB) does not.  Larger
 *     shapes return CAKEB200_ERR_TOO_LARGE and compute nothing.
 *   - A, B and C must belong to the current device (CAKEB200_ERR_ARG otherwise).
 *   - The array occupies that much memory on every GPU that loads the library,
 *     until the process exits.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress).  With CUDA's default lazy module loading that first call, or
 *     the first kernel launch of this library, is also when the driver loads the library's
 *     module and reserves the array, which is an allocation in effect and synchronises.
 *     Make one call (any small product) at start-up, outside any stream capture, before
 *     the region that must not allocate; or start the process with CUDA_MODULE_LOADING=EAGER.
 *   - All calls on a device share the one array: two calls whose work overlaps on
 *     the GPU (different streams, or different threads) race on it.  Issue them
 *     one after the other.  Each call clears the state it needs at its start, so
 *     what an earlier call left behind does not matter.
 *   - `stream` is a cudaStream_t (NULL = the default stream).  Every call synchronises
 *     `stream` before it returns (it reads the device-side status word back). */
#define CAKEB200_NOALLOC_SCRATCH_BYTES (17u << 20)
int cakeb200_sgemm_noalloc(const float* A, const float* B, float* C, int M, int N, int K, void* stream);

#ifdef __cplusplus
}
#endif
#endif
