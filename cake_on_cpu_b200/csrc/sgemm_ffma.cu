// Exact-FP32 SGEMM on the CUDA cores (FFMA), register-tiled.
//
// This is the B200 counterpart of the reference's outer-product register-tile
// microkernel (cake_sgemm_haswell_6x16, src/kernels/haswell/dense.cpp:8-203)
// together with the m_reg / n_reg loops that drive it
// (src/cake_sgemm_k_first.cpp:113-127): every C element is one chain of fused
// multiply-adds over k ascending, a single rounding per step, as on the CPU.
//
// One CTA owns a BM x BN tile of C and streams BK-deep slices of A and B through
// double-buffered shared memory (the CPU's "packing" of operation blocks becomes
// this staging); each thread keeps a TM x TN accumulator in registers.  The
// order in which CTAs take tiles is the schedule (K-first / M-first / N-first).
#include "common.cuh"

namespace cakeb200 {
namespace {

template <int BM, int BN, int BK, int TM, int TN, bool VEC>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_ffma_kernel(GemmProblem g, int tiles_m, int tiles_n) {
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr int CM = TM / 4, CN = TN / 4;  // 4-wide chunks per thread along M and N
    constexpr int PAD = 4;
    __shared__ __align__(16) float As[2][BK][BM + PAD];
    __shared__ __align__(16) float Bs[2][BK][BN + PAD];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    int tm, tn;
    tile_coords(blockIdx.x, tiles_m, tiles_n, g.order, g.band > 0 ? g.band : 8, tm, tn);
    const int m0 = tm * BM, n0 = tn * BN;
    const float* __restrict__ A = g.A + (long long) blockIdx.z * g.stride_a;
    const float* __restrict__ B = g.B + (long long) blockIdx.z * g.stride_b;
    float* __restrict__ C = g.C + (long long) blockIdx.z * g.stride_c;
    const int M = g.M, N = g.N, K = g.K;

    constexpr int A_ELEMS = VEC ? BM * BK / 4 : BM * BK;
    constexpr int B_ELEMS = VEC ? BK * BN / 4 : BK * BN;
    constexpr int A_IT = (A_ELEMS + NT - 1) / NT, B_IT = (B_ELEMS + NT - 1) / NT;
    float4 ra[VEC ? A_IT : 1], rb[VEC ? B_IT : 1];
    float sa[VEC ? 1 : A_IT], sb[VEC ? 1 : B_IT];

    auto fetch = [&](int k0) {
        if constexpr (VEC) {
#pragma unroll
            for (int it = 0; it < A_IT; it++) {
                int i = tid + it * NT;
                int r = i / (BK / 4), c = (i % (BK / 4)) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < A_ELEMS && m0 + r < M && k0 + c < K)
                    v = __ldg(reinterpret_cast<const float4*>(A + (long long) (m0 + r) * g.lda + k0 + c));
                ra[it] = v;
            }
#pragma unroll
            for (int it = 0; it < B_IT; it++) {
                int i = tid + it * NT;
                int r = i / (BN / 4), c = (i % (BN / 4)) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < B_ELEMS && k0 + r < K && n0 + c < N)
                    v = __ldg(reinterpret_cast<const float4*>(B + (long long) (k0 + r) * g.ldb + n0 + c));
                rb[it] = v;
            }
        } else {
#pragma unroll
            for (int it = 0; it < A_IT; it++) {
                int i = tid + it * NT;
                int r = i / BK, c = i % BK;
                sa[it] = (i < A_ELEMS && m0 + r < M && k0 + c < K) ? __ldg(A + (long long) (m0 + r) * g.lda + k0 + c) : 0.f;
            }
#pragma unroll
            for (int it = 0; it < B_IT; it++) {
                int i = tid + it * NT;
                int r = i / BN, c = i % BN;
                sb[it] = (i < B_ELEMS && k0 + r < K && n0 + c < N) ? __ldg(B + (long long) (k0 + r) * g.ldb + n0 + c) : 0.f;
            }
        }
    };
    auto stage = [&](int buf) {
        if constexpr (VEC) {
#pragma unroll
            for (int it = 0; it < A_IT; it++) {
                int i = tid + it * NT;
                if (i < A_ELEMS) {
                    int r = i / (BK / 4), c = (i % (BK / 4)) * 4;
                    As[buf][c + 0][r] = ra[it].x;
                    As[buf][c + 1][r] = ra[it].y;
                    As[buf][c + 2][r] = ra[it].z;
                    As[buf][c + 3][r] = ra[it].w;
                }
            }
#pragma unroll
            for (int it = 0; it < B_IT; it++) {
                int i = tid + it * NT;
                if (i < B_ELEMS) {
                    int r = i / (BN / 4), c = (i % (BN / 4)) * 4;
                    *reinterpret_cast<float4*>(&Bs[buf][r][c]) = rb[it];
                }
            }
        } else {
#pragma unroll
            for (int it = 0; it < A_IT; it++) {
                int i = tid + it * NT;
                if (i < A_ELEMS) As[buf][i % BK][i / BK] = sa[it];
            }
#pragma unroll
            for (int it = 0; it < B_IT; it++) {
                int i = tid + it * NT;
                if (i < B_ELEMS) Bs[buf][i / BN][i % BN] = sb[it];
            }
        }
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    const int KT = (K + BK - 1) / BK;
    if (KT > 0) {
        fetch(0);
        stage(0);
    }
    __syncthreads();
    for (int kt = 0; kt < KT; kt++) {
        const int buf = kt & 1;
        if (kt + 1 < KT) fetch((kt + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], b[TN];
#pragma unroll
            for (int c = 0; c < CM; c++) {
                float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][c * (BM / CM) + ty * 4]);
                a[c * 4 + 0] = v.x; a[c * 4 + 1] = v.y; a[c * 4 + 2] = v.z; a[c * 4 + 3] = v.w;
            }
#pragma unroll
            for (int c = 0; c < CN; c++) {
                float4 v = *reinterpret_cast<const float4*>(&Bs[buf][kk][c * (BN / CN) + tx * 4]);
                b[c * 4 + 0] = v.x; b[c * 4 + 1] = v.y; b[c * 4 + 2] = v.z; b[c * 4 + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < KT) stage(buf ^ 1);
        __syncthreads();
    }

#pragma unroll
    for (int ci = 0; ci < CM; ci++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int row = m0 + ci * (BM / CM) + ty * 4 + i;
            if (row >= M) continue;
            float* crow = C + (long long) row * g.ldc;
#pragma unroll
            for (int cj = 0; cj < CN; cj++) {
                const int col = n0 + cj * (BN / CN) + tx * 4;
                float* a4 = acc[ci * 4 + i] + cj * 4;
                if constexpr (VEC) {
                    if (col < N) {
                        float4 v = make_float4(a4[0], a4[1], a4[2], a4[3]);
                        if (g.bias) {
                            const float4 b = __ldg(reinterpret_cast<const float4*>(g.bias + col));
                            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                        }
                        if (g.accumulate) {
                            float4 o = *reinterpret_cast<const float4*>(crow + col);
                            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                        }
                        *reinterpret_cast<float4*>(crow + col) = v;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (col + j < N) {
                            const float v = g.bias ? a4[j] + __ldg(g.bias + col + j) : a4[j];
                            crow[col + j] = g.accumulate ? crow[col + j] + v : v;
                        }
                }
            }
        }
}

template <int BM, int BN, int BK, int TM, int TN>
int launch_cfg(const GemmProblem& g, cudaStream_t stream) {
    const int tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + BN - 1) / BN;
    const long long tiles = (long long) tiles_m * tiles_n;
    if (tiles > 0x7fffffffLL || g.batch > 65535) {
        set_error("sgemm_ffma: grid too large (%lld tiles, batch %d)", tiles, g.batch);
        return CAKEB200_ERR_TOO_LARGE;
    }
    dim3 grid((unsigned) tiles, 1, (unsigned) g.batch), block((BM / TM) * (BN / TN));
    const bool vec = (g.lda % 4 == 0) && (g.ldb % 4 == 0) && (g.ldc % 4 == 0) && (g.stride_a % 4 == 0) &&
                     (g.stride_b % 4 == 0) && (g.stride_c % 4 == 0) &&
                     (((uintptr_t) g.A | (uintptr_t) g.B | (uintptr_t) g.C | (uintptr_t) g.bias) % 16 == 0) &&
                     // a float4 never straddles the edge of the matrix (views inside a wider allocation)
                     (g.K % 4 == 0) && (g.N % 4 == 0);
    if (vec)
        sgemm_ffma_kernel<BM, BN, BK, TM, TN, true><<<grid, block, 0, stream>>>(g, tiles_m, tiles_n);
    else
        sgemm_ffma_kernel<BM, BN, BK, TM, TN, false><<<grid, block, 0, stream>>>(g, tiles_m, tiles_n);
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}

// dst[c][r] = src[r][c] for a rows x cols row-major matrix (leading dimension ld_src); dst is cols x rows, dense
__global__ void __launch_bounds__(256)
transpose_copy_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int cols, int ld_src) {
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int i = ty; i < 32; i += 8)
        if (r0 + i < rows && c0 + tx < cols) tile[i][tx] = src[(long long) (r0 + i) * ld_src + c0 + tx];
    __syncthreads();
    for (int i = ty; i < 32; i += 8)
        if (c0 + i < cols && r0 + tx < rows) dst[(long long) (c0 + i) * rows + r0 + tx] = tile[tx][i];
}

}  // namespace

int launch_transpose_copy(const float* src, float* dst, int rows, int cols, int ld_src, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return CAKEB200_OK;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32);
    if (grid.y > 65535) {
        set_error("transpose: too many rows (%d)", rows);
        return CAKEB200_ERR_TOO_LARGE;
    }
    transpose_copy_kernel<<<grid, 256, 0, stream>>>(src, dst, rows, cols, ld_src);
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}

// Tile shape selection (the GPU analogue of get_cache_dims picking m_c / n_c,
// src/block_sizing.cpp:304-429): big tiles when the grid still fills the SMs.
int launch_sgemm_ffma(const GemmProblem& g, cudaStream_t stream) {
    if (g.M <= 0 || g.N <= 0 || g.batch <= 0) return CAKEB200_OK;
    // padded work of each tile size, weighted by how efficient that tile's inner loop is;
    // a large tile is penalised when it leaves most SMs without a CTA
    const int sizes[3] = {128, 96, 64};
    const double weight[3] = {1.0, 1.1, 1.35};
    int best = 2;
    double best_cost = 0;
    for (int i = 0; i < 3; i++) {
        const int t = sizes[i];
        const double tiles = (double) ((g.M + t - 1) / t) * ((g.N + t - 1) / t) * g.batch;
        double cost = tiles * t * t * weight[i];
        if (tiles < 120) cost *= 120.0 / tiles;
        if (i == 0 || cost < best_cost) { best = i; best_cost = cost; }
    }
    if (best == 0) return launch_cfg<128, 128, 16, 8, 8>(g, stream);
    if (best == 1) return launch_cfg<96, 96, 16, 8, 8>(g, stream);
    return launch_cfg<64, 64, 16, 4, 4>(g, stream);
}

}  // namespace cakeb200
