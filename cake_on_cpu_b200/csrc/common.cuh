// Shared declarations for the sm_100a kernels and the C-ABI layer above them.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "cake_b200.h"

namespace cakeb200 {

// Last error text of the calling thread, returned by cakeb200_last_error().
void set_error(const char* fmt, ...);

#define CAKE_CUDA_OK(expr)                                                              \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess) {                                                        \
            cakeb200::set_error("%s failed at %s:%d: %s", #expr, __FILE__, __LINE__,    \
                                cudaGetErrorString(_e));                                \
            return CAKEB200_ERR_CUDA;                                                   \
        }                                                                               \
    } while (0)

// One dense product C[M x N] (+)= A[M x K] * B[K x N], all row-major FP32 in
// device memory.  `batch` independent products are laid `stride_*` elements apart.
struct GemmProblem {
    const float* A;
    const float* B;
    float* C;
    int M, N, K;
    int lda, ldb, ldc;
    long long stride_a, stride_b, stride_c;
    int batch;
    int accumulate;  // 0: C = A*B, 1: C += A*B (the reference's beta != 0 behaviour)
    int order;       // tile rasterisation: CAKEB200_SCHED_*
    int band;        // tile rows (columns for N-first) per band of the rasterisation; 0 = the kernel's default
    // 3xTF32 path only: when out_p > 0 the N axis is (image, position) with out_p positions per image and
    // element (m, n) is stored at C[(n / out_p) * out_image_stride + m * out_p + n % out_p] (NCHW convolution output)
    int out_p;
    long long out_image_stride;
    // operands stored transposed: trans_a -> A points at a K x M row-major matrix (lda >= M),
    // trans_b -> B points at an N x K row-major matrix (ldb >= K); the product is op(A) * op(B)
    int trans_a, trans_b;
    const float* bias;  // length N, added to every row of the result (nullptr: none)
    // 3xTF32 path only: operands already split into TF32 hi / lo planes by an earlier call (both K-major with
    // leading dimension ceil4(K): a_* is M x Kp, b_* is N x Kp, i.e. B transposed).  Where set, the operand's
    // split pass is skipped and A (B) itself is not read.
    const float *a_hi, *a_lo, *b_hi, *b_lo;
    // 3xTF32 path only, K-sharded product over several GPUs: when set, the rows of the result are not
    // stored at C but sent to the ranks that own them (see OwnerSlots)
    const struct OwnerSlots* owners;
};

// Where the rows of one rank's partial product go when K is sharded over the GPUs of a box.  Rows
// [row_lo[o], row_lo[o+1]) of the result belong to rank o; this rank's partial sums of those rows are
// stored, dense with N columns, from base[o] on, which is memory of rank o's GPU (mapped into this
// process) reserved for this source rank.  When every row has been stored, flag[o] (also in rank o's
// memory) is set to `epoch`.
constexpr int MAX_RANKS = 8;
struct OwnerSlots {
    float* base[MAX_RANKS];
    int* flag[MAX_RANKS];
    int row_lo[MAX_RANKS + 1];
    int world;
    int epoch;
    unsigned* done;  // counter in this GPU's memory: CTAs of the storing kernel that have finished
};

// Per-device state: scratch arena that grows on demand and is reused between calls.
struct DeviceState {
    int device = -1;
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    void* staging[3] = {nullptr, nullptr, nullptr};
    size_t staging_bytes[3] = {0, 0, 0};
    int sm_count = 0;
    int* status_word = nullptr;  // device-side error flag written by bounded waits
    cudaStream_t stream = nullptr;
    cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // 4,5 bracket the operand-split pass
    // host-operand pipeline: copies in and out run on their own streams, ordered by per-band events
    static constexpr int MAX_BANDS = 32;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t band_in[MAX_BANDS] = {}, band_done[MAX_BANDS] = {}, fence[3] = {};
    // optional device-side timing of the asynchronous entry point (cakeb200_profile_begin / _end)
    static constexpr int MAX_PROFILE = 256;
    bool profiling = false;
    int profile_count = 0;
    cudaEvent_t profile_ev[3 * MAX_PROFILE] = {};
};
DeviceState* device_state();  // state of the current device (created on first use)
int ensure_scratch(DeviceState* st, size_t bytes);

// exact-FP32 FFMA path (sgemm_ffma.cu)
int launch_sgemm_ffma(const GemmProblem& g, cudaStream_t stream);  // untransposed operands only
int launch_transpose_copy(const float* src, float* dst, int rows, int cols, int ld_src, cudaStream_t stream);
// one CTA runs a bounded wait that must give up (sgemm_tf32x3.cu)
int launch_bounded_wait_selftest(int* status_word, int limit_us, cudaStream_t stream, bool pair = false);
// Process-wide overrides set through cakeb200_set_option (abi.cu); 0 = the library's own rule.
enum Option { OPT_TILE_N, OPT_BAND, OPT_K_PIECES, OPT_CHUNK_KB, OPT_CONV_ROUTE, OPT_SMALL_OPERANDS, OPT_PACK_SCALAR, OPT_PAIR, OPT_COUNT };
int option_get(int id);
// 16 page-locked ints of the calling host thread (nullptr if they could not be had): landing place for small
// device-to-host reads; words 0-3 are the status word's, 8-9 a 64-bit count (abi.cu)
int* pinned_host_words();
// issue rate of dense TF32 MMAs on every SM (peak_tf32.cu)
int measure_tf32_peak(int* status_word, int sm_count, float ms_target, cudaStream_t stream, float* tflops, float* ms_out);
// batches of small products on the tensor cores, operands split inside the kernel (sgemm_small_tf32x3.cu)
bool small_tf32x3_fits(int M, int N, int K);
int launch_sgemm_small_tf32x3(const GemmProblem& g, int* status_word, int sm_count, cudaStream_t stream);
// matrix-vector product (gemv.cu); scratch holds the partial vectors of the K slices
size_t sgemv_scratch_bytes(int M, int K, int sm_count);
int launch_sgemv(const float* A, const float* x, float* y, int M, int K, int lda, int col_major, int accumulate,
                 void* scratch, size_t scratch_bytes, int sm_count, cudaStream_t stream, int* launches);
// stride-1 convolution as an implicit product (conv_tf32x3.cu); scratch holds the split filter planes
bool conv_tf32x3_fits(const float* in, int batch, int cin, int H, int W, int cout, int hf, int wf, int stride, int pad);
size_t conv_tf32x3_scratch_bytes(int cin, int cout, int hf, int wf);
int conv_tf32x3_describe(int batch, int cin, int H, int W, int cout, int hf, int wf, int stride, int pad, int sm_count,
                         cakeb200_conv_plan* out);
int launch_conv_tf32x3(const float* in, const float* filters, float* out, const float* bias, int batch, int cin, int H,
                       int W, int cout, int hf, int wf, int pad, void* scratch, size_t scratch_bytes, int* status_word,
                       int sm_count, cudaStream_t stream, int* launches);
// 3xTF32 tcgen05 path (sgemm_tf32x3.cu); needs scratch for the split operand planes
size_t tf32x3_scratch_bytes(int M, int N, int K, int sm_count);
// row-band interface of the 3xTF32 path (operand planes laid out once, rows multiplied band by band)
struct Tf32x3Planes {
    float *a_hi, *a_lo, *b_hi, *b_lo;
    float* partials;  // room for partial tiles (nullptr: none reserved)
    int M, Kp;
};
size_t tf32x3_plane_bytes(int M, int N, int K, int slots_for_sms = 0);
int tf32x3_planes(int M, int N, int K, void* scratch, size_t scratch_bytes, Tf32x3Planes* out, int slots_for_sms = 0);
int tf32x3_split_B(const float* B, int ldb, int K, int N, const Tf32x3Planes& p, cudaStream_t stream);
int tf32x3_split_A_rows(const float* A, int lda, int r0, int rows, int K, const Tf32x3Planes& p, int sm_count,
                        cudaStream_t stream);
int tf32x3_split_im2col(const float* in, int batch, int cin, int H, int W, int hf, int wf, int stride, int pad,
                        const Tf32x3Planes& p, int sm_count, cudaStream_t stream);
int tf32x3_multiply_rows(const Tf32x3Planes& p, float* C, int ldc, int r0, int rows, int N, int K, int order,
                         int accumulate, int* status_word, int sm_count, cudaStream_t stream, int out_p = 0,
                         long long out_image_stride = 0);
int launch_sgemm_tf32x3(const GemmProblem& g, void* scratch, size_t scratch_bytes, int* status_word,
                        int sm_count, cudaStream_t stream, cakeb200_stats* stats, cudaEvent_t* prepass_events);
// hi / lo planes of one operand, for callers that keep an operand split across many products (weights):
// bytes of one plane and the split itself (transpose: `mat` is K x rows row-major, as B is; else rows x K)
size_t tf32x3_one_plane_bytes(int rows, int K);
// rows of C per tile of a product: 256 where it runs on pairs of SMs, else 128
int tf32x3_tile_rows(int M, int N, int K, int order, int sm_count);
int tf32x3_make_planes(const float* mat, int rows, int K, int ld, bool transpose, float* hi, float* lo, int sm_count,
                       cudaStream_t stream);
// true when the tile plan of this shape cuts every tile into K pieces, so that the kernel that sums the
// pieces is the only one that stores rows of the result (the condition for GemmProblem::owners)
bool tf32x3_all_tiles_in_pieces(int M, int N, int K, int order, int sm_count);
// K-sharded product, second half (kshard.cu): wait (bounded) for every rank's flag, then
// out[i] = sum over source ranks r of slots[r * slot_floats + i], i < count, in rank order
int launch_sum_owner_slots(const float* slots, long long slot_floats, int world, float* out, long long count,
                           const int* flags, int epoch, long long limit_ns, int* status_word, int sm_count,
                           cudaStream_t stream);


#ifdef __CUDACC__
// Linear tile index -> tile coordinates.  K always runs innermost inside a tile (the
// accumulator stays in place), so what remains of the reference's block schedules on a
// GPU is the order in which tiles are taken.  As in the reference, the name gives the
// loop nest from the outside in:
//   M-first (MKN) and K-first (KMN): M outermost.  Bands of `band` tile rows, each walked
//       column by column; the direction alternates from band to band, the analogue of the
//       snaking CB-block traversal of src/cake_sgemm_k_first.cpp:28-71 and
//       src/cake_sgemm_m_first.cpp:26-60.
//   N-first (NKM): N outermost.  Bands of `band` tile columns, each walked row by row
//       (src/cake_sgemm_n_first.cpp:26-60).
// Tiles that run at the same time (consecutive ids) therefore cover a compact
// band x (SMs / band) patch of C and share their A and B panels through L2.
__host__ __device__ __forceinline__ void tile_coords(int id, int tiles_m, int tiles_n, int order, int band, int& tm,
                                                     int& tn) {
    if (order == CAKEB200_SCHED_NKM) {
        const int per = band * tiles_m;
        const int b = id / per, first = b * band;
        const int cols = (band < tiles_n - first) ? band : tiles_n - first;
        const int in_band = id - b * per;
        tn = first + in_band % cols;
        tm = in_band / cols;
        if (b & 1) tm = tiles_m - 1 - tm;
    } else {
        const int per = band * tiles_n;
        const int b = id / per, first = b * band;
        const int rows = (band < tiles_m - first) ? band : tiles_m - first;
        const int in_band = id - b * per;
        tm = first + in_band % rows;
        tn = in_band / rows;
        if (b & 1) tn = tiles_n - 1 - tn;
    }
}
#endif

}  // namespace cakeb200
