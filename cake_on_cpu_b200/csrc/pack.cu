// Layout-exact packing and unpacking on the device.
//
// The reference reorders A, B and C into "operation blocks" (OBs) laid out in
// the order its schedules consume them (src/pack_{k,m,n}_first.cpp,
// src/unpack_{k,m,n}_first.cpp) and, inside an OB, into register-tile panels
// (src/pack_ob.cpp:40-60 for A, :105-140 for B, :253-288 / :393-411 for C).
// The B200 GEMM kernels do not need these buffers -- they stage tiles through
// shared memory themselves -- but callers of the reference API do size, fill
// and pass them, so the library produces byte-identical buffers: the host walks
// the block structure once and emits one descriptor per OB, and a single
// bandwidth-bound kernel moves every element (padding positions become zero).
#include <vector>

#include "common.cuh"

namespace cakeb200 {
namespace {

enum { OB_A = 0, OB_B = 1, OB_C = 2 };

struct ObDesc {
    long long mat_off;     // first element of the block in the row-major matrix
    long long packed_off;  // first element of the block in the packed buffer
    int rows, cols;        // block extent (rows multiple of m_r for A/C, cols multiple of n_r for B/C)
    int row0, col0;        // global coordinates used for the bounds test
};

// Element e of a packed block -> (row, col) inside the block.  IDX is 32-bit for
// every block a cache-sized blocking produces; 64-bit only for huge user-defined blocks.
template <int KIND, typename IDX>
__device__ __forceinline__ void ob_coords(IDX e, int rows, int cols, int mr, int nr, int& r, int& c) {
    if (KIND == OB_A) {  // [row panel][k][row in panel]
        const IDX per_panel = (IDX) cols * mr;
        const IDX panel = e / per_panel;
        const unsigned rem = (unsigned) (e - panel * per_panel);
        const unsigned k = rem / (unsigned) mr;
        c = (int) k;
        r = (int) panel * mr + (int) (rem - k * mr);
    } else if (KIND == OB_B) {  // [col panel][k][col in panel]
        const IDX per_panel = (IDX) rows * nr;
        const IDX panel = e / per_panel;
        const unsigned rem = (unsigned) (e - panel * per_panel);
        const unsigned k = rem / (unsigned) nr;
        r = (int) k;
        c = (int) panel * nr + (int) (rem - k * nr);
    } else {  // [col panel][row panel][m_r x n_r tile, row-major]
        const IDX per_panel = (IDX) rows * nr;
        const IDX panel = e / per_panel;
        const unsigned rem = (unsigned) (e - panel * per_panel);
        const unsigned tile = (unsigned) (mr * nr);
        const unsigned rp = rem / tile;
        const unsigned t = rem - rp * tile;
        const unsigned tr = t / (unsigned) nr;
        r = (int) (rp * mr + tr);
        c = (int) panel * nr + (int) (t - tr * nr);
    }
}

template <int KIND, bool UNPACK, typename IDX>
__device__ __forceinline__ void ob_move_block(const ObDesc& d, float* __restrict__ mat, float* __restrict__ packed, int ld,
                                              int row_limit, int col_limit, int mr, int nr) {
    const IDX elems = (IDX) d.rows * (IDX) d.cols;
    const IDX step = (IDX) gridDim.y * blockDim.x;
    for (IDX e = (IDX) blockIdx.y * blockDim.x + threadIdx.x; e < elems; e += step) {
        int r, c;
        ob_coords<KIND, IDX>(e, d.rows, d.cols, mr, nr, r, c);
        const bool inside = (d.row0 + r < row_limit) && (d.col0 + c < col_limit);
        const long long m_idx = d.mat_off + (long long) r * ld + c;
        if (UNPACK) {
            if (inside) mat[m_idx] = packed[d.packed_off + (long long) e];
        } else {
            packed[d.packed_off + (long long) e] = inside ? __ldg(mat + m_idx) : 0.0f;
        }
    }
}

template <int KIND, bool UNPACK>
__global__ void __launch_bounds__(256)
ob_move_kernel(const ObDesc* __restrict__ descs, float* __restrict__ mat, float* __restrict__ packed,
               int ld, int row_limit, int col_limit, int mr, int nr) {
    const ObDesc d = descs[blockIdx.x];
    if ((long long) d.rows * d.cols < 0x7fffffffLL - (long long) gridDim.y * blockDim.x)
        ob_move_block<KIND, UNPACK, unsigned>(d, mat, packed, ld, row_limit, col_limit, mr, nr);
    else
        ob_move_block<KIND, UNPACK, long long>(d, mat, packed, ld, row_limit, col_limit, mr, nr);
}

struct Split {
    int used, full, step, last;
    int extent(int core) const { return core == used - 1 ? last : step; }
};
// K-first: the M extent of a CB block is divided over cores (src/cake_sgemm_k_first.cpp:75-98)
Split rows_of_block(const cakeb200_blk_dims& x, int m, int p, int mr) {
    if (m == x.Mb - 1 && x.m_pad) return {x.p_l, mr * x.mr_rem, x.m_c1, x.m_c1_last_core};
    return {p, p * x.m_c, x.m_c, x.m_c};
}
// M-/N-first: the K extent of a CB block is divided over cores (src/cake_sgemm_m_first.cpp:60-96)
Split depth_of_block(const cakeb200_blk_dims& x, int k, int p) {
    if (k == x.Kb - 1 && x.k_pad) return {x.p_l, x.k_rem, x.k_c1, x.k_c1_last_core};
    return {p, p * x.k_c, x.k_c, x.k_c};
}
int cols_of_block(const cakeb200_blk_dims& x, int n) { return (n == x.Nb - 1 && x.n_pad) ? x.n_c1 : x.n_c; }
int first_col(const cakeb200_blk_dims& x, int n, int N) { return (n == x.Nb - 1 && x.n_pad) ? N - N % x.n_c : n * x.n_c; }

// pack_A_single_buf_{k,m,n}_first: src/pack_k_first.cpp:7-76, src/pack_m_first.cpp:7-78, src/pack_n_first.cpp:8-79
void describe_A(std::vector<ObDesc>& out, int M, int K, int p, const cakeb200_blk_dims& x, int mr) {
    long long off = 0;
    (void) M;
    if (x.sch == CAKEB200_SCHED_KMN) {
        for (int m = 0; m < x.Mb; m++) {
            const Split s = rows_of_block(x, m, p, mr);
            for (int k = 0; k < x.Kb; k++) {
                const int kc = (k == x.Kb - 1 && x.k_pad) ? x.k_c1 : x.k_c;
                for (int core = 0; core < s.used; core++) {
                    const int row = m * p * x.m_c + core * s.step;
                    out.push_back({(long long) row * K + (long long) k * x.k_c, off + (long long) core * s.step * kc,
                                   s.extent(core), kc, row, 0});
                }
                off += (long long) s.full * kc;
            }
        }
        return;
    }
    const bool m_first = x.sch == CAKEB200_SCHED_MKN;
    const int span = m_first ? x.m_c : p * x.m_c;
    const int outer = m_first ? x.Kb : x.Mb, inner = m_first ? x.Mb : x.Kb;
    for (int o = 0; o < outer; o++)
        for (int i = 0; i < inner; i++) {
            const int k = m_first ? o : i, m = m_first ? i : o;
            const Split s = depth_of_block(x, k, p);
            const int rows = (m == x.Mb - 1 && x.m_pad) ? x.m_c1 : span;
            for (int core = 0; core < s.used; core++)
                out.push_back({(long long) m * span * K + (long long) k * p * x.k_c + (long long) core * s.step,
                               off + (long long) core * s.step * rows, rows, s.extent(core), m * span, 0});
            off += (long long) s.full * rows;
        }
}

// pack_B_{k,m,n}_first: src/pack_k_first.cpp:187-283, src/pack_m_first.cpp:83-144, src/pack_n_first.cpp:84-144
void describe_B(std::vector<ObDesc>& out, int K, int N, int p, const cakeb200_blk_dims& x) {
    long long off = 0;
    (void) K;
    if (x.sch == CAKEB200_SCHED_KMN) {
        for (int n = 0; n < x.Nb; n++) {
            const int cols = cols_of_block(x, n), c0 = first_col(x, n, N);
            for (int k = 0; k < x.Kb; k++) {
                const int kc = (k == x.Kb - 1 && x.k_pad) ? x.k_c1 : x.k_c;
                out.push_back({(long long) k * x.k_c * N + (long long) n * x.n_c, off, kc, cols, 0, c0});
                off += (long long) kc * cols;
            }
        }
        return;
    }
    const bool m_first = x.sch == CAKEB200_SCHED_MKN;
    const int outer = m_first ? x.Nb : x.Kb, inner = m_first ? x.Kb : x.Nb;
    for (int o = 0; o < outer; o++)
        for (int i = 0; i < inner; i++) {
            const int n = m_first ? o : i, k = m_first ? i : o;
            const int cols = cols_of_block(x, n), c0 = first_col(x, n, N);
            const Split s = depth_of_block(x, k, p);
            for (int core = 0; core < s.used; core++)
                out.push_back({(long long) (k * p * x.k_c + core * s.step) * N + (long long) n * x.n_c,
                               off + (long long) core * s.step * cols, s.extent(core), cols, 0, c0});
            off += (long long) s.full * cols;
        }
}

// pack_C_single_buf_* / unpack_C_single_buf_*: src/pack_k_first.cpp:404-472, src/unpack_k_first.cpp:5-67,
// src/pack_m_first.cpp:148-200, src/unpack_m_first.cpp:5-49, src/pack_n_first.cpp:155-209,
// src/unpack_n_first.cpp:5-49.  N-first uses the block offsets of the schedule and the unpacker
// (src/cake_sgemm_n_first.cpp:98), the only self-consistent choice for ragged shapes.
void describe_C(std::vector<ObDesc>& out, int M, int N, int p, const cakeb200_blk_dims& x, int mr) {
    if (x.sch == CAKEB200_SCHED_KMN) {
        long long off = 0;
        for (int n = 0; n < x.Nb; n++) {
            const int cols = cols_of_block(x, n), c0 = first_col(x, n, N);
            for (int m = 0; m < x.Mb; m++) {
                const Split s = rows_of_block(x, m, p, mr);
                for (int core = 0; core < s.used; core++) {
                    const int row = m * p * x.m_c + core * s.step;
                    out.push_back({(long long) row * N + (long long) n * x.n_c, off + (long long) core * s.step * cols,
                                   s.extent(core), cols, row, c0});
                }
                off += (long long) s.full * cols;
            }
        }
        return;
    }
    const bool m_first = x.sch == CAKEB200_SCHED_MKN;
    const int span = m_first ? x.m_c : p * x.m_c;
    for (int m = 0; m < x.Mb; m++) {
        const int rows = (m == x.Mb - 1 && x.m_pad) ? x.m_c1 : span;
        for (int n = 0; n < x.Nb; n++) {
            const int cols = cols_of_block(x, n), c0 = first_col(x, n, N);
            const long long off = m_first ? (long long) x.M_padded * n * x.n_c + (long long) m * x.m_c * cols
                                          : (long long) x.N_padded * m * span + (long long) n * rows * x.n_c;
            out.push_back({(long long) m * span * N + (long long) n * x.n_c, off, rows, cols, m * span, c0});
        }
    }
    (void) M;
}

template <int KIND, bool UNPACK>
int run_move(std::vector<ObDesc>& descs, float* mat, float* packed, int ld, int row_limit, int col_limit,
             int mr, int nr, cudaStream_t stream) {
    if (descs.empty()) return CAKEB200_OK;
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    const size_t bytes = descs.size() * sizeof(ObDesc);
    int rc = ensure_scratch(st, bytes);
    if (rc) return rc;
    CAKE_CUDA_OK(cudaMemcpyAsync(st->scratch, descs.data(), bytes, cudaMemcpyHostToDevice, stream));
    CAKE_CUDA_OK(cudaStreamSynchronize(stream));  // descs is a host temporary
    long long biggest = 0;
    for (const ObDesc& d : descs) biggest = std::max(biggest, (long long) d.rows * d.cols);
    // enough CTAs per block to cover it with ~8 elements per thread, capped
    int chunks = (int) std::min<long long>(std::max<long long>((biggest + 2047) / 2048, 1), 1024);
    while ((long long) chunks * descs.size() > (1LL << 22) && chunks > 1) chunks /= 2;
    dim3 grid((unsigned) descs.size(), (unsigned) chunks);
    ob_move_kernel<KIND, UNPACK><<<grid, 256, 0, stream>>>((const ObDesc*) st->scratch, mat, packed, ld,
                                                           row_limit, col_limit, mr, nr);
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}

bool bad(const void* a, const void* b, const cakeb200_blk_dims* x, const cakeb200_cntx* c, int p) {
    if (!a || !b || !x || !c || p <= 0 || c->mr <= 0 || c->nr <= 0 || x->sch < 0 || x->sch > CAKEB200_SCHED_NKM) {
        set_error("pack: bad argument");
        return true;
    }
    return false;
}

}  // namespace

// Device-pointer implementations behind the C ABI (pointer-kind handling lives in abi.cu).
int pack_A_dev(const float* A, float* A_p, int M, int K, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* c,
               bool unpack, cudaStream_t s) {
    if (bad(A, A_p, x, c, p)) return CAKEB200_ERR_ARG;
    std::vector<ObDesc> d;
    describe_A(d, M, K, p, *x, c->mr);
    return unpack ? run_move<OB_A, true>(d, (float*) A, A_p, K, M, K, c->mr, c->nr, s)
                  : run_move<OB_A, false>(d, (float*) A, A_p, K, M, K, c->mr, c->nr, s);
}
int pack_B_dev(const float* B, float* B_p, int K, int N, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* c,
               bool unpack, cudaStream_t s) {
    if (bad(B, B_p, x, c, p)) return CAKEB200_ERR_ARG;
    std::vector<ObDesc> d;
    describe_B(d, K, N, p, *x);
    return unpack ? run_move<OB_B, true>(d, (float*) B, B_p, N, K, N, c->mr, c->nr, s)
                  : run_move<OB_B, false>(d, (float*) B, B_p, N, K, N, c->mr, c->nr, s);
}
int pack_C_dev(const float* C, float* C_p, int M, int N, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* c,
               bool unpack, cudaStream_t s) {
    if (bad(C, C_p, x, c, p)) return CAKEB200_ERR_ARG;
    std::vector<ObDesc> d;
    describe_C(d, M, N, p, *x, c->mr);
    return unpack ? run_move<OB_C, true>(d, (float*) C, C_p, N, M, N, c->mr, c->nr, s)
                  : run_move<OB_C, false>(d, (float*) C, C_p, N, M, N, c->mr, c->nr, s);
}

}  // namespace cakeb200
