// Sparse-A SGEMM: C = A*B with A mostly zero.
//
// The reference's sparse microkernel (cake_sp_sgemm_haswell_6x16,
// src/kernels/haswell/sparse.cpp:7-131) walks the stored columns of an A tile
// and, for every nonzero a[m,k], issues C[m,:] = fma(a, B[k,:], C[m,:]); zeros
// issue nothing.  Here A is first compacted on the device into per-row
// (column, value) lists with warp ballots (each 32-column chunk yields a bitmap
// whose popcount places the survivors), then a CTA that owns BM rows x BN
// columns of C streams BK-deep slabs of B through shared memory and lets every
// warp replay its rows' nonzeros against the slab.  Per C element the FMAs run
// over k ascending, so the result equals the row-skipping CPU order bit for bit.
#include <cstdlib>

#include "common.cuh"

namespace cakeb200 {
namespace {

// nonzeros per row; one warp per row, 128-bit loads when the row is aligned
__global__ void __launch_bounds__(256) row_nnz_kernel(const float* __restrict__ A, int M, int K, int* __restrict__ cnt) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    const float* row = A + (long long) warp * K;
    int n = 0;
    for (int k = lane; k < K; k += 32) n += (__ldg(row + k) != 0.0f);
    for (int o = 16; o; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
    if (lane == 0) cnt[warp] = n;
}

// exclusive scan of cnt[0..M) into ptr[0..M]; single CTA, M is at most a few 100k
__global__ void __launch_bounds__(1024) row_ptr_kernel(const int* __restrict__ cnt, int M, long long* __restrict__ ptr) {
    __shared__ long long part[1024];
    const int t = threadIdx.x;
    const int per = (M + 1023) / 1024;
    const int lo = min(t * per, M), hi = min(lo + per, M);
    long long s = 0;
    for (int i = lo; i < hi; i++) s += cnt[i];
    part[t] = s;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
        long long v = (t >= o) ? part[t - o] : 0;
        __syncthreads();
        part[t] += v;
        __syncthreads();
    }
    long long run = (t == 0) ? 0 : part[t - 1];
    for (int i = lo; i < hi; i++) {
        ptr[i] = run;
        run += cnt[i];
    }
    if (t == 1023) ptr[M] = part[1023];
}

// warp-level compaction: ballot -> bitmap of survivors, popcount of the lower lanes -> slot
__global__ void __launch_bounds__(256)
compact_rows_kernel(const float* __restrict__ A, int M, int K, const long long* __restrict__ ptr,
                    int* __restrict__ cols, float* __restrict__ vals, int* status) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    const float* row = A + (long long) warp * K;
    long long base = ptr[warp];
    const long long limit = ptr[warp + 1];
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        const float v = (k < K) ? __ldg(row + k) : 0.0f;
        const unsigned bitmap = __ballot_sync(0xffffffffu, v != 0.0f);
        if (v != 0.0f) {
            const long long slot = base + __popc(bitmap & ((1u << lane) - 1u));
            if (slot >= limit || slot < 0) {  // the row holds more nonzeros than were counted: record, do not write
                if (atomicCAS(status, 0, 2) == 0) { status[1] = 11; status[2] = warp; }
            } else {
                cols[slot] = k;
                vals[slot] = v;
            }
        }
        base += __popc(bitmap);
    }
}

// 128-bit variants for rows that are 16-byte aligned (K % 4 == 0): a warp step covers 128 columns.
__global__ void __launch_bounds__(256) row_nnz_vec4_kernel(const float4* __restrict__ A, int M, int K4, int* __restrict__ cnt) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    const float4* row = A + (long long) warp * K4;
    int n = 0;
    for (int k = lane; k < K4; k += 32) {
        const float4 v = __ldg(row + k);
        n += (v.x != 0.0f) + (v.y != 0.0f) + (v.z != 0.0f) + (v.w != 0.0f);
    }
    for (int o = 16; o; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
    if (lane == 0) cnt[warp] = n;
}

__global__ void __launch_bounds__(256)
compact_rows_vec4_kernel(const float4* __restrict__ A, int M, int K4, const long long* __restrict__ ptr,
                         int* __restrict__ cols, float* __restrict__ vals, int* status) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    const float4* row = A + (long long) warp * K4;
    long long base = ptr[warp];
    const long long limit = ptr[warp + 1];
    for (int k0 = 0; k0 < K4; k0 += 32) {
        const int k4 = k0 + lane;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k4 < K4) v = __ldg(row + k4);
        const float e[4] = {v.x, v.y, v.z, v.w};
        // survivors of this lane, then an exclusive prefix over the lanes: ascending column order is kept
        const int mine = (e[0] != 0.0f) + (e[1] != 0.0f) + (e[2] != 0.0f) + (e[3] != 0.0f);
        int incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        long long slot = base + incl - mine;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (e[j] != 0.0f) {
                if (slot >= limit || slot < 0) {  // more nonzeros than were counted: record, do not write
                    if (atomicCAS(status, 0, 2) == 0) { status[1] = 11; status[2] = warp; }
                } else {
                    cols[slot] = k4 * 4 + j;
                    vals[slot] = e[j];
                }
                slot++;
            }
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
    }
}

constexpr int SP_BM = 64, SP_BN = 128, SP_BK = 64, SP_WARPS = 8, SP_ROWS = SP_BM / SP_WARPS;

template <bool VEC>
__global__ void __launch_bounds__(SP_WARPS * 32)
spmm_rows_kernel(const long long* __restrict__ ptr, const int* __restrict__ cols, const float* __restrict__ vals,
                 const float* __restrict__ B, float* __restrict__ C, int M, int N, int K, int* status) {
    __shared__ __align__(16) float Bs[SP_BK][SP_BN];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * SP_BM + warp * SP_ROWS, n0 = blockIdx.y * SP_BN;  // row blocks fastest: a strip of B stays in L2

    long long cur[SP_ROWS], end[SP_ROWS];
    float acc[SP_ROWS][4];
#pragma unroll
    for (int r = 0; r < SP_ROWS; r++) {
        const int m = m0 + r;
        cur[r] = (m < M) ? ptr[m] : 0;
        end[r] = (m < M) ? ptr[m + 1] : 0;
        if (cur[r] < 0 || end[r] < cur[r] || end[r] > (long long) M * K) {  // corrupt row list: record, skip the row
            if (lane == 0 && atomicCAS(status, 0, 2) == 0) { status[1] = 13; status[2] = m; }
            cur[r] = end[r] = 0;
        }
        acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;
    }

    for (int k0 = 0; k0 < K; k0 += SP_BK) {
        __syncthreads();  // previous slab fully consumed
        for (int i = threadIdx.x; i < SP_BK * SP_BN / 4; i += SP_WARPS * 32) {
            const int r = i / (SP_BN / 4), c = (i % (SP_BN / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + r < K) {
                const float* src = B + (long long) (k0 + r) * N + n0 + c;
                if (VEC) {
                    if (n0 + c < N) v = __ldg(reinterpret_cast<const float4*>(src));
                } else {
                    if (n0 + c + 0 < N) v.x = __ldg(src + 0);
                    if (n0 + c + 1 < N) v.y = __ldg(src + 1);
                    if (n0 + c + 2 < N) v.z = __ldg(src + 2);
                    if (n0 + c + 3 < N) v.w = __ldg(src + 3);
                }
            }
            *reinterpret_cast<float4*>(&Bs[r][c]) = v;
        }
        __syncthreads();
        const int k_hi = k0 + SP_BK;
#pragma unroll
        for (int r = 0; r < SP_ROWS; r++) {
            long long c = cur[r];
            const long long e = end[r];
            while (c < e) {
                const int k = __ldg(cols + c);  // same address in every lane: one broadcast load
                if (k >= k_hi) break;
                if (k < k0) {  // list not ascending: record and drop the rest of the row
                    if (lane == 0 && atomicCAS(status, 0, 2) == 0) { status[1] = 12; status[2] = m0 + r; }
                    c = e;
                    break;
                }
                const float a = __ldg(vals + c);
                const float4 b = *reinterpret_cast<const float4*>(&Bs[k - k0][lane * 4]);
                acc[r][0] = fmaf(a, b.x, acc[r][0]);
                acc[r][1] = fmaf(a, b.y, acc[r][1]);
                acc[r][2] = fmaf(a, b.z, acc[r][2]);
                acc[r][3] = fmaf(a, b.w, acc[r][3]);
                c++;
            }
            cur[r] = c;
        }
    }

#pragma unroll
    for (int r = 0; r < SP_ROWS; r++) {
        const int m = m0 + r, n = n0 + lane * 4;
        if (m >= M) continue;
        float* dst = C + (long long) m * N + n;
        if (VEC) {
            if (n < N) *reinterpret_cast<float4*>(dst) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (n + j < N) dst[j] = acc[r][j];
        }
    }
}

// Very sparse A: each 64-deep slab of B would be staged for a handful of nonzeros, so
// the slab staging is dropped.  One warp owns one row of A and a 512-column slab of C;
// it loads 32 (column, value) pairs at a time, broadcasts them with shuffles and, for
// each nonzero, reads the matching piece of row k of B straight from L2 (four
// independent 128-bit loads per lane).  Same FMA order per element as the staged kernel.
constexpr int SG_BN = 512;

template <bool VEC>
__global__ void __launch_bounds__(256)
spmm_gather_kernel(const long long* __restrict__ ptr, const int* __restrict__ cols, const float* __restrict__ vals,
                   const float* __restrict__ B, float* __restrict__ C, int M, int N, int K, int* status) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // row groups run fastest, strips of columns slowest: the CTAs resident at one time work on one or two
    // strips of B (512 columns x K rows, 17 MB at K = 8192), which then stay in L2 while every row visits them
    const int m = blockIdx.x * 8 + warp, n0 = blockIdx.y * SG_BN;
    if (m >= M) return;
    long long c = ptr[m], e = ptr[m + 1];
    if (c < 0 || e < c || e > (long long) M * K) {  // corrupt row list: record, produce zeros
        if (lane == 0 && atomicCAS(status, 0, 2) == 0) { status[1] = 13; status[2] = m; }
        c = e = 0;
    }
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    for (; c < e; c += 32) {
        const long long mine = c + lane;
        const int my_k = (mine < e) ? __ldg(cols + mine) : 0;
        const float my_a = (mine < e) ? __ldg(vals + mine) : 0.0f;
        const int cnt = (int) min((long long) 32, e - c);
#pragma unroll 4
        for (int t = 0; t < cnt; t++) {
            int k = __shfl_sync(0xffffffffu, my_k, t);
            const float a = __shfl_sync(0xffffffffu, my_a, t);
            if ((unsigned) k >= (unsigned) K) {  // never for a list built by compact_rows_kernel
                if (lane == 0 && atomicCAS(status, 0, 2) == 0) { status[1] = 14; status[2] = m; }
                continue;
            }
            const float* brow = B + (long long) k * N + n0 + lane * 4;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int col = n0 + j * 128 + lane * 4;
                float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
                if (VEC) {
                    if (col < N) b = __ldg(reinterpret_cast<const float4*>(brow + j * 128));
                } else {
                    if (col + 0 < N) b.x = __ldg(brow + j * 128 + 0);
                    if (col + 1 < N) b.y = __ldg(brow + j * 128 + 1);
                    if (col + 2 < N) b.z = __ldg(brow + j * 128 + 2);
                    if (col + 3 < N) b.w = __ldg(brow + j * 128 + 3);
                }
                acc[j][0] = fmaf(a, b.x, acc[j][0]);
                acc[j][1] = fmaf(a, b.y, acc[j][1]);
                acc[j][2] = fmaf(a, b.z, acc[j][2]);
                acc[j][3] = fmaf(a, b.w, acc[j][3]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int col = n0 + j * 128 + lane * 4;
        float* dst = C + (long long) m * N + col;
        if (VEC) {
            if (col < N) *reinterpret_cast<float4*>(dst) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (col + q < N) dst[q] = acc[j][q];
        }
    }
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct SparseLayout {
    int* cnt;
    long long* ptr;
    int* cols;
    float* vals;
};
SparseLayout layout_of(void* scratch, int M, int K) {
    SparseLayout l;
    char* base = (char*) scratch;
    l.cnt = (int*) base;
    base += align_up((size_t) M * 4, 256);
    l.ptr = (long long*) base;
    base += align_up(((size_t) M + 1) * 8, 256);
    l.cols = (int*) base;
    base += align_up((size_t) M * K * 4, 256);
    l.vals = (float*) base;
    return l;
}

// CAKEB200_DEBUG_SYNC=1: wait after every kernel and name the one that failed
int after_kernel(const char* what, cudaStream_t stream) {
    static const bool debug_sync = getenv("CAKEB200_DEBUG_SYNC") != nullptr;
    if (!debug_sync) return CAKEB200_OK;
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("sparse: %s failed: %s", what, cudaGetErrorString(e));
        return CAKEB200_ERR_CUDA;
    }
    return CAKEB200_OK;
}

}  // namespace

// Scratch layout: [cnt: M ints][ptr: M+1 int64][cols: nnz ints][vals: nnz floats].
// The compacted lists are sized for the worst case (every entry nonzero) so the
// whole call needs a single allocation and no device->host round trip.
size_t sparse_scratch_bytes(int M, int K) {
    const size_t cells = (size_t) M * K;
    return align_up((size_t) M * 4, 256) + align_up(((size_t) M + 1) * 8, 256) + align_up(cells * 4, 256) * 2;
}

// Step 1: count, scan, compact.  Returns the number of nonzeros (one 8-byte read-back:
// the caller picks the multiply kernel, or the dense tensor-core product, from the density).
int sp_compact(const float* A, int M, int K, void* scratch, int* status_word, cudaStream_t stream,
               long long* nnz, int* launches) {
    const SparseLayout l = layout_of(scratch, M, K);
    int rc;
    const int row_blocks = (M + 7) / 8;  // 8 warps (rows) per 256-thread CTA
    const bool vec = (K % 4 == 0) && ((uintptr_t) A % 16 == 0);
    if (vec)
        row_nnz_vec4_kernel<<<row_blocks, 256, 0, stream>>>((const float4*) A, M, K / 4, l.cnt);
    else
        row_nnz_kernel<<<row_blocks, 256, 0, stream>>>(A, M, K, l.cnt);
    if ((rc = after_kernel("row_nnz_kernel", stream))) return rc;
    row_ptr_kernel<<<1, 1024, 0, stream>>>(l.cnt, M, l.ptr);
    if ((rc = after_kernel("row_ptr_kernel", stream))) return rc;
    if (vec)
        compact_rows_vec4_kernel<<<row_blocks, 256, 0, stream>>>((const float4*) A, M, K / 4, l.ptr, l.cols, l.vals, status_word);
    else
        compact_rows_kernel<<<row_blocks, 256, 0, stream>>>(A, M, K, l.ptr, l.cols, l.vals, status_word);
    CAKE_CUDA_OK(cudaGetLastError());
    if ((rc = after_kernel("compact_rows_kernel", stream))) return rc;
    long long stack_total = 0;
    int* pinned = pinned_host_words();
    long long* total = pinned ? reinterpret_cast<long long*>(pinned + 8) : &stack_total;
    CAKE_CUDA_OK(cudaMemcpyAsync(total, l.ptr + M, sizeof(*total), cudaMemcpyDeviceToHost, stream));
    CAKE_CUDA_OK(cudaStreamSynchronize(stream));
    if (nnz) *nnz = *total;
    if (launches) *launches += 3;
    return CAKEB200_OK;
}

// Step 2: multiply the compacted rows.  Below 10 % nonzeros rows are gathered from L2
// one nonzero at a time; above, slabs of B are staged in shared memory and shared by 64 rows.
int sp_multiply(const float* B, float* C, int M, int N, int K, void* scratch, long long nnz, int* status_word,
                cudaStream_t stream, int* launches) {
    const SparseLayout l = layout_of(scratch, M, K);
    int rc;
    const bool vec = (N % 4 == 0) && (((uintptr_t) B | (uintptr_t) C) % 16 == 0);
    // measured at 8192^3: the gathering kernel takes 0.25 ms + 1.1 ms per percent of nonzeros up to 5 % and beyond;
    // the staged kernel (slabs of B shared by 64 rows) only pays once most 64-deep slabs are needed by most rows
    const bool gather = (double) nnz < 0.10 * (double) M * (double) K;
    if (gather) {
        dim3 grid((M + 7) / 8, (N + SG_BN - 1) / SG_BN);
        if (grid.y > 65535) {
            set_error("sparse product: too many column strips");
            return CAKEB200_ERR_TOO_LARGE;
        }
        if (vec)
            spmm_gather_kernel<true><<<grid, 256, 0, stream>>>(l.ptr, l.cols, l.vals, B, C, M, N, K, status_word);
        else
            spmm_gather_kernel<false><<<grid, 256, 0, stream>>>(l.ptr, l.cols, l.vals, B, C, M, N, K, status_word);
    } else {
        dim3 grid((M + SP_BM - 1) / SP_BM, (N + SP_BN - 1) / SP_BN);
        if (grid.y > 65535) {
            set_error("sparse product: too many column strips");
            return CAKEB200_ERR_TOO_LARGE;
        }
        if (vec)
            spmm_rows_kernel<true><<<grid, SP_WARPS * 32, 0, stream>>>(l.ptr, l.cols, l.vals, B, C, M, N, K, status_word);
        else
            spmm_rows_kernel<false><<<grid, SP_WARPS * 32, 0, stream>>>(l.ptr, l.cols, l.vals, B, C, M, N, K, status_word);
    }
    CAKE_CUDA_OK(cudaGetLastError());
    if ((rc = after_kernel(gather ? "spmm_gather_kernel" : "spmm_rows_kernel", stream))) return rc;
    if (launches) *launches += 1;
    return CAKEB200_OK;
}

}  // namespace cakeb200
