// Matrix-vector product y (+)= A x, the skinny end of the SGEMM path.
//
// The reference has a separate driver for it (cake_sgemv / schedule_mvm,
// examples/cake_gemv.cpp:424-489, 716-765, with the 8 x 8 microkernel at :87-140): the
// matrix is column-major (A[k*M + m]), blocks of rows go to cores, and inside a block the
// microkernel streams A once, broadcasting one x[k] per column.  A matrix-vector product
// does one multiply-add per element of A, so it is bound by reading A from HBM and
// nothing else; the kernels below are plain streaming kernels sized to keep every SM's
// memory pipeline full.
//
// Column-major A (the reference's layout): consecutive threads own consecutive rows m, so
// a warp reads 128 contiguous floats of one column at a time; K is cut into slices
// (blockIdx.y) so that even a matrix with few rows fills the machine, every slice writes a
// partial vector, and a second kernel adds the slices in a fixed order (deterministic).
// Row-major A (the N = 1 case of cake_sgemm): one warp per row, 16-byte loads along the
// row, a shuffle reduction at the end.
#include <algorithm>

#include "common.cuh"

namespace cakeb200 {
namespace {

constexpr int COL_THREADS = 256;

// partial[s][m] = sum over k in slice s of A[k*M + m] * x[k]; V = rows per thread (4: float4 loads)
template <int V>
__global__ void __launch_bounds__(COL_THREADS)
sgemv_cols_kernel(const float* __restrict__ A, const float* __restrict__ x, float* __restrict__ partial, int M, int K,
                  int k_per_slice) {
    const int m = (blockIdx.x * COL_THREADS + threadIdx.x) * V;
    if (m >= M) return;
    const int k0 = blockIdx.y * k_per_slice, k1 = min(K, k0 + k_per_slice);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; j++) acc[j] = 0.f;
    const float* col = A + (long long) k0 * M + m;
    int k = k0;
    // four columns in flight per thread
    for (; k + 4 <= k1; k += 4, col += 4LL * M) {
        float a[4][V];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (V == 4) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(col + (long long) u * M));
                a[u][0] = v.x; a[u][1] = v.y; a[u][2] = v.z; a[u][3] = v.w;
            } else {
                a[u][0] = __ldg(col + (long long) u * M);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const float xv = __ldg(x + k + u);
#pragma unroll
            for (int j = 0; j < V; j++) acc[j] = fmaf(a[u][j], xv, acc[j]);
        }
    }
    for (; k < k1; k++, col += M) {
        const float xv = __ldg(x + k);
        if (V == 4) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(col));
            acc[0] = fmaf(v.x, xv, acc[0]); acc[1] = fmaf(v.y, xv, acc[1]);
            acc[2] = fmaf(v.z, xv, acc[2]); acc[3] = fmaf(v.w, xv, acc[3]);
        } else {
            acc[0] = fmaf(__ldg(col), xv, acc[0]);
        }
    }
    float* out = partial + (long long) blockIdx.y * M + m;
#pragma unroll
    for (int j = 0; j < V; j++) out[j] = acc[j];
}

// y[m] = (accumulate ? y[m] : 0) + partial[0][m] + partial[1][m] + ...
__global__ void __launch_bounds__(256)
sgemv_sum_slices_kernel(const float* __restrict__ partial, float* __restrict__ y, int M, int slices, int accumulate) {
    const int m = blockIdx.x * 256 + threadIdx.x;
    if (m >= M) return;
    float s = accumulate ? y[m] : 0.f;
    for (int i = 0; i < slices; i++) s += partial[(long long) i * M + m];
    y[m] = s;
}

// row-major A: one warp per row
__global__ void __launch_bounds__(256)
sgemv_rows_kernel(const float* __restrict__ A, const float* __restrict__ x, float* __restrict__ y, int M, int K, int lda,
                  int vec, int accumulate) {
    const int warp = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    const float* row = A + (long long) warp * lda;
    float acc = 0.f;
    if (vec) {
        const int k4 = K / 4;
        for (int i = lane; i < k4; i += 32) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(row) + i);
            const float4 b = __ldg(reinterpret_cast<const float4*>(x) + i);
            acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
            acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
        }
        for (int k = k4 * 4 + lane; k < K; k += 32) acc = fmaf(__ldg(row + k), __ldg(x + k), acc);
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(__ldg(row + k), __ldg(x + k), acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) y[warp] = accumulate ? y[warp] + acc : acc;
}

// How a column-major product is cut: CTAs along the rows, slices along K.  About eight CTAs per SM,
// slices of at least 64 columns (in whole groups of four), at most 512 slices.
struct ColPlan {
    int row_ctas, slices, k_per_slice;
};
ColPlan col_plan(int M, int K, bool v4, int sm_count) {
    ColPlan p;
    const int rows_per_cta = COL_THREADS * (v4 ? 4 : 1);
    p.row_ctas = (M + rows_per_cta - 1) / rows_per_cta;
    int slices = std::max(1, std::min(512, (8 * sm_count + p.row_ctas - 1) / p.row_ctas));
    slices = std::max(1, std::min(slices, K / 64));
    p.k_per_slice = ((K + slices - 1) / slices + 3) / 4 * 4;
    p.slices = (K + p.k_per_slice - 1) / p.k_per_slice;
    return p;
}

}  // namespace

size_t sgemv_scratch_bytes(int M, int K, int sm_count) {
    const ColPlan a = col_plan(M, K, true, sm_count), b = col_plan(M, K, false, sm_count);
    return (size_t) std::max(a.slices, b.slices) * M * 4;
}

// A column-major (A[k*M + m], col_major != 0) or row-major with leading dimension lda.
int launch_sgemv(const float* A, const float* x, float* y, int M, int K, int lda, int col_major, int accumulate,
                 void* scratch, size_t scratch_bytes, int sm_count, cudaStream_t stream, int* launches) {
    if (M <= 0 || K <= 0) return CAKEB200_OK;
    if (!col_major) {
        const int vec = (lda % 4 == 0) && (((uintptr_t) A | (uintptr_t) x) % 16 == 0);
        const long long blocks = ((long long) M * 32 + 255) / 256;
        sgemv_rows_kernel<<<(unsigned) blocks, 256, 0, stream>>>(A, x, y, M, K, lda, vec, accumulate);
        CAKE_CUDA_OK(cudaGetLastError());
        if (launches) *launches += 1;
        return CAKEB200_OK;
    }
    const bool v4 = (M % 4 == 0) && (((uintptr_t) A) % 16 == 0);
    const ColPlan cp = col_plan(M, K, v4, sm_count);
    const int row_ctas = cp.row_ctas, slices = cp.slices, k_per_slice = cp.k_per_slice;
    if ((size_t) slices * M * 4 > scratch_bytes) {
        set_error("sgemv: scratch too small");
        return CAKEB200_ERR_ARG;
    }
    float* partial = (float*) scratch;
    dim3 grid((unsigned) row_ctas, (unsigned) slices);
    if (v4) sgemv_cols_kernel<4><<<grid, COL_THREADS, 0, stream>>>(A, x, partial, M, K, k_per_slice);
    else sgemv_cols_kernel<1><<<grid, COL_THREADS, 0, stream>>>(A, x, partial, M, K, k_per_slice);
    CAKE_CUDA_OK(cudaGetLastError());
    sgemv_sum_slices_kernel<<<(M + 255) / 256, 256, 0, stream>>>(partial, y, M, slices, accumulate);
    CAKE_CUDA_OK(cudaGetLastError());
    if (launches) *launches += 2;
    return CAKEB200_OK;
}

}  // namespace cakeb200
