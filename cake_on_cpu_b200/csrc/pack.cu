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
#include <stdlib.h>
#include <string.h>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace cakeb200 {
namespace {

enum { OB_A = 0, OB_B = 1, OB_C = 2 };

thread_local int g_last_width = 1;  // floats per access of this thread's last pack / unpack call

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

// Four packed elements per thread.  For B and C a quad is four consecutive columns of one row of a
// register-tile panel (n_r is a multiple of 4), on both sides a 16-byte access.
template <int KIND, bool UNPACK>
__device__ __forceinline__ void ob_move_block_quads(const ObDesc& d, float* __restrict__ mat, float* __restrict__ packed,
                                                    int ld, int row_limit, int col_limit, int mr, int nr) {
    const unsigned quads = (unsigned) ((long long) d.rows * d.cols / 4);
    const unsigned step = gridDim.y * blockDim.x;
    for (unsigned q = blockIdx.y * blockDim.x + threadIdx.x; q < quads; q += step) {
        int r, c;
        ob_coords<KIND, unsigned>(q * 4u, d.rows, d.cols, mr, nr, r, c);
        float4* pk = reinterpret_cast<float4*>(packed + d.packed_off) + q;
        float* m = mat + d.mat_off + (long long) r * ld + c;
        const bool row_in = d.row0 + r < row_limit;
        if (row_in && d.col0 + c + 3 < col_limit) {
            if (UNPACK) *reinterpret_cast<float4*>(m) = *pk;
            else *pk = __ldg(reinterpret_cast<const float4*>(m));
        } else {  // quad on the ragged edge of the matrix
            if (UNPACK) {
                const float4 v = *pk;
                const float e[4] = {v.x, v.y, v.z, v.w};
                for (int j = 0; j < 4; j++)
                    if (row_in && d.col0 + c + j < col_limit) m[j] = e[j];
            } else {
                float e[4];
                for (int j = 0; j < 4; j++) e[j] = (row_in && d.col0 + c + j < col_limit) ? __ldg(m + j) : 0.0f;
                *pk = make_float4(e[0], e[1], e[2], e[3]);
            }
        }
    }
}

// A: a thread owns V (4 or 2) consecutive k of one row panel: MR rows are read as V-wide vectors along k
// (coalesced across the warp) and leave as V * MR contiguous packed floats ([k][row in panel]), written
// 16 bytes at a time.  V = 2 serves block depths k_c that are even but not multiples of 4.
template <bool UNPACK, int MR, int V>
__device__ __forceinline__ void ob_move_block_a_vec(const ObDesc& d, float* __restrict__ mat, float* __restrict__ packed,
                                                    int ld, int row_limit, int col_limit) {
    static_assert((V * MR) % 4 == 0, "a thread's packed floats must be whole 16-byte pieces");
    const unsigned kq = (unsigned) d.cols / V;  // vectors of k per panel
    const unsigned items = (unsigned) (d.rows / MR) * kq;
    const unsigned step = gridDim.y * blockDim.x;
    for (unsigned i = blockIdx.y * blockDim.x + threadIdx.x; i < items; i += step) {
        const unsigned panel = i / kq, k = (i - panel * kq) * V;
        float4* pk = reinterpret_cast<float4*>(packed + d.packed_off + (long long) panel * d.cols * MR + (long long) k * MR);
        float* m = mat + d.mat_off + (long long) panel * MR * ld + k;
        const bool k_in = d.col0 + (int) k + V - 1 < col_limit;
        float w[V * MR];  // w[j * MR + r] = element (row r, k + j)
        if (UNPACK) {
#pragma unroll
            for (int j = 0; j < V * MR / 4; j++) {
                const float4 v = pk[j];
                w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
            }
#pragma unroll
            for (int r = 0; r < MR; r++) {
                if (d.row0 + (int) panel * MR + r >= row_limit) continue;
                float* dst = m + (long long) r * ld;
                if (k_in) {
                    if (V == 4) *reinterpret_cast<float4*>(dst) = make_float4(w[r], w[MR + r], w[2 * MR + r], w[3 * MR + r]);
                    else *reinterpret_cast<float2*>(dst) = make_float2(w[r], w[MR + r]);
                } else {
#pragma unroll
                    for (int j = 0; j < V; j++)
                        if (d.col0 + (int) k + j < col_limit) dst[j] = w[j * MR + r];
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < MR; r++) {
                float e[4] = {0.f, 0.f, 0.f, 0.f};
                if (d.row0 + (int) panel * MR + r < row_limit) {
                    const float* src = m + (long long) r * ld;
                    if (k_in) {
                        if (V == 4) {
                            const float4 v = __ldg(reinterpret_cast<const float4*>(src));
                            e[0] = v.x; e[1] = v.y; e[2] = v.z; e[3] = v.w;
                        } else {
                            const float2 v = __ldg(reinterpret_cast<const float2*>(src));
                            e[0] = v.x; e[1] = v.y;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < V; j++)
                            if (d.col0 + (int) k + j < col_limit) e[j] = __ldg(src + j);
                    }
                }
#pragma unroll
                for (int j = 0; j < V; j++) w[j * MR + r] = e[j];
            }
#pragma unroll
            for (int j = 0; j < V * MR / 4; j++) pk[j] = make_float4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        }
    }
}

// `vec` (4, 2 or 1): floats per access that every block of the call allows (decided on the host: alignment
// of the buffers, of every block offset and of the leading dimension; n_r a multiple of 4 for B and C, the
// block depth k_c a multiple of 4 or 2 for A).
template <int KIND, bool UNPACK>
__global__ void __launch_bounds__(256)
ob_move_kernel(const ObDesc* __restrict__ descs, float* __restrict__ mat, float* __restrict__ packed,
               int ld, int row_limit, int col_limit, int mr, int nr, int vec) {
    const ObDesc d = descs[blockIdx.x];
    if (vec > 1 && (long long) d.rows * d.cols < 0x7fffffffLL) {
        if (KIND == OB_A) {
            if (mr == 6 && vec == 4) return ob_move_block_a_vec<UNPACK, 6, 4>(d, mat, packed, ld, row_limit, col_limit);
            if (mr == 6 && vec == 2) return ob_move_block_a_vec<UNPACK, 6, 2>(d, mat, packed, ld, row_limit, col_limit);
            if (mr == 8 && vec == 4) return ob_move_block_a_vec<UNPACK, 8, 4>(d, mat, packed, ld, row_limit, col_limit);
            if (mr == 8 && vec == 2) return ob_move_block_a_vec<UNPACK, 8, 2>(d, mat, packed, ld, row_limit, col_limit);
        } else {
            return ob_move_block_quads<KIND, UNPACK>(d, mat, packed, ld, row_limit, col_limit, mr, nr);
        }
    }
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

// Descriptor tables on the device, kept for the shapes seen last: a caller that packs the same
// shape again (every layer call of a network, every step of a benchmark) skips the upload and the
// synchronisation it needs.  An entry is recognised by the descriptors themselves.
struct TableEntry {
    int device = -1;
    std::vector<ObDesc> host;
    ObDesc* dev = nullptr;
    unsigned long long used = 0;
};
constexpr int TABLES = 12;
TableEntry g_tables[TABLES];
unsigned long long g_table_clock = 0;
std::mutex g_table_mutex;

int device_table(int device, const std::vector<ObDesc>& descs, cudaStream_t stream, const ObDesc** out) {
    std::lock_guard<std::mutex> lock(g_table_mutex);
    const size_t bytes = descs.size() * sizeof(ObDesc);
    TableEntry* victim = &g_tables[0];
    for (TableEntry& e : g_tables) {
        if (e.dev && e.device == device && e.host.size() == descs.size() && memcmp(e.host.data(), descs.data(), bytes) == 0) {
            e.used = ++g_table_clock;
            *out = e.dev;
            return CAKEB200_OK;
        }
        if (e.used < victim->used) victim = &e;
    }
    if (victim->dev) {
        cudaFree(victim->dev);  // waits for kernels that may still read the old table
        victim->dev = nullptr;
    }
    CAKE_CUDA_OK(cudaMalloc((void**) &victim->dev, bytes));
    victim->host = descs;
    victim->device = device;
    victim->used = ++g_table_clock;
    CAKE_CUDA_OK(cudaMemcpyAsync(victim->dev, victim->host.data(), bytes, cudaMemcpyHostToDevice, stream));
    CAKE_CUDA_OK(cudaStreamSynchronize(stream));
    *out = victim->dev;
    return CAKEB200_OK;
}

template <int KIND, bool UNPACK>
int run_move(std::vector<ObDesc>& descs, float* mat, float* packed, int ld, int row_limit, int col_limit,
             int mr, int nr, cudaStream_t stream) {
    if (descs.empty()) return CAKEB200_OK;
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    const ObDesc* table = nullptr;
    int rc = device_table(st->device, descs, stream, &table);
    if (rc) return rc;
    long long biggest = 0;
    for (const ObDesc& d : descs) biggest = std::max(biggest, (long long) d.rows * d.cols);
    // wide moves need every address involved to be a multiple of the width
    auto allows = [&](int w) {
        if (ld % w != 0 || ((uintptr_t) mat) % (4 * w) != 0 || ((uintptr_t) packed) % 16 != 0) return false;
        if (KIND == OB_A ? !(mr == 6 || mr == 8) : (w != 4 || nr % 4 != 0)) return false;
        for (const ObDesc& d : descs) {
            if (d.mat_off % w != 0 || d.packed_off % 4 != 0 || d.col0 % w != 0) return false;
            if (KIND == OB_A ? (d.cols % w != 0 || d.rows % mr != 0) : (d.cols % nr != 0)) return false;
        }
        return true;
    };
    int vec = allows(4) ? 4 : (KIND == OB_A && allows(2)) ? 2 : 1;
    if (option_get(OPT_PACK_SCALAR)) vec = 1;  // for tests: the one-element-per-thread path
    g_last_width = vec;
    // enough CTAs per block to cover it with ~8 elements (2 quads) per thread, capped
    int chunks = (int) std::min<long long>(std::max<long long>((biggest + 2047) / 2048, 1), 1024);
    while ((long long) chunks * descs.size() > (1LL << 22) && chunks > 1) chunks /= 2;
    dim3 grid((unsigned) descs.size(), (unsigned) chunks);
    ob_move_kernel<KIND, UNPACK><<<grid, 256, 0, stream>>>(table, mat, packed, ld,
                                                           row_limit, col_limit, mr, nr, vec);
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

int last_pack_width() { return g_last_width; }

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
