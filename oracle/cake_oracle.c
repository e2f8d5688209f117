/* TEST INFRASTRUCTURE ONLY -- see cake_oracle.h.  Plain C, no intrinsics.
 *
 * Each function names the reference file:line it restates (paths are relative
 * to the vnatesh/CAKE_on_CPU tree).  The floating-point operation ORDER of the
 * reference is kept exactly: every C element is a chain of single-rounding
 * fused multiply-adds over k, k-blocks visited in the schedule's snake order,
 * so results match the reference's AVX2 build bit for bit.
 */
#include "cake_oracle.h"

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ context */

/* cake_query_cntx, src/block_sizing.cpp:40-75: the x86 register tile is 6x16. */
void oracle_cntx_init(oracle_cntx_t* c, int L1, int L2, int L3, int ncores) {
    c->alpha_n = 1.0;
    c->mr = 6;
    c->nr = 16;
    c->L1 = L1;
    c->L2 = L2;
    c->L3 = L3;
    c->ncores = ncores;
}

/* ----------------------------------------------------------- block sizing */

/* derive_schedule, src/block_sizing.cpp:434-462.  The reference keeps the
 * cut-offs in `float` while the right-hand sides are evaluated in double. */
int oracle_derive_schedule(int M, int N, int K, int p, int mc_ret, const oracle_cntx_t* c) {
    float m = (float) (p * mc_ret), k = m, n = m;
    float K_cut_M = (float) ((2.0 * M) / (1.0 + (M * ((2.0 / k) - (1.0 / m)))));
    float K_cut_N = (float) ((2.0 * N) / (1.0 + (N * ((2.0 / k) - (1.0 / n)))));
    m = (float) (c->alpha_n * p * mc_ret);
    n = m;
    float N_cut_M = (float) (M / (1.0 + (M * ((1.0 / n) - (1.0 / m)))));
    float M_cut_N = (float) (N / (1.0 + (N * ((1.0 / m) - (1.0 / n)))));
    if (((float) N <= N_cut_M) && ((float) K <= K_cut_M)) return ORACLE_MKN;
    if (((float) M <= M_cut_N) && ((float) K <= K_cut_N)) return ORACLE_NKM;
    return ORACLE_KMN;
}

/* set_schedule, src/cake_sgemm.cpp:768-787 (exported, unused by cake_sgemm). */
int oracle_set_schedule(int sch, int M, int N, int K) {
    if (sch != ORACLE_NA) return sch;
    if (M >= 2 * K && M >= N) return ORACLE_MKN;
    if (K >= M && K >= N) return ORACLE_KMN;
    if (N >= 2 * K && N >= M) return ORACLE_NKM;
    return ORACLE_KMN;
}

static int round_down_nonzero(int v, int q) {
    v -= v % q;
    return v == 0 ? q : v;
}

/* get_cache_dims, src/block_sizing.cpp:304-429 (type_size = 4). */
static void cache_dims(int M, int N, int K, int p, oracle_cntx_t* c, int sch,
                       int mcu, int kcu, int ncu, int* m_c, int* k_c, int* n_c, int* sch_out) {
    const int mr = c->mr, nr = c->nr;
    const float type_size = 4;
    int b = 2 * nr;
    int mc_L2 = (int) ((-b + sqrt(b * b + 4 * (((double) c->L2) / (2 * type_size)))) / 2.0);
    mc_L2 -= mc_L2 % mr;
    int mc_L3 = (int) sqrt((((double) c->L3) / (2 * type_size)) /
                           (c->ncores * (1 + 1.0 + 1.0 * c->ncores)));
    mc_L3 -= mc_L3 % mr;
    c->alpha_n = ((double) mc_L3) / mc_L2; /* the reference mutates its context here (:336) */

    int mc_ret = mc_L2;
    if (M < p * mr) {
        mc_ret = mr;
    } else if (M < p * mc_L2) {
        int a = M / p;
        mc_ret = (a < mr) ? mr : a + (mr - (a % mr)); /* adds a full mr when a % mr == 0 (:346-349) */
    }

    *sch_out = (sch == ORACLE_NA) ? oracle_derive_schedule(M, N, K, p, mc_ret, c) : sch;

    if (mcu && ncu && kcu) {
        *m_c = mcu; *k_c = kcu; *n_c = ncu;
        c->alpha_n = 1.0;
        return;
    }
    int nc_ret;
    if (*sch_out == ORACLE_NKM) {
        nc_ret = round_down_nonzero(mc_ret, nr);
        mc_ret = round_down_nonzero((int) (c->alpha_n * mc_ret), mr);
    } else {
        nc_ret = round_down_nonzero((int) (c->alpha_n * p * mc_ret), nr);
    }
    *m_c = mc_ret; *k_c = mc_ret; *n_c = nc_ret;
}

static int ceil_div_d(int a, int b) { return (int) ceil(((double) a) / b); }

/* init_block_dims, src/block_sizing.cpp:465-595. */
void oracle_init_block_dims(int M, int N, int K, int p, oracle_blk_t* x, oracle_cntx_t* c,
                            int sch, int mcu, int kcu, int ncu) {
    const int mr = c->mr, nr = c->nr;
    memset(x, 0, sizeof(*x));
    cache_dims(M, N, K, p, c, sch, mcu, kcu, ncu, &x->m_c, &x->k_c, &x->n_c, &x->sch);

    x->n_pad = (N % x->n_c) ? 1 : 0;
    x->nr_rem = (int) ceil(((double) (N % x->n_c) / nr));
    x->n_c1 = x->nr_rem * nr;
    x->Nb = (N / x->n_c) + x->n_pad;
    x->N_padded = (N - (N % x->n_c)) + x->n_c1;

    if (x->sch == ORACLE_KMN) {
        const int pm = p * x->m_c;
        x->k_pad = (K % x->k_c) ? 1 : 0;
        x->m_pad = (M % pm) ? 1 : 0;
        x->mr_rem = ceil_div_d(M % pm, mr);
        int per_core = ceil_div_d(x->mr_rem, p);
        x->p_l = per_core ? ceil_div_d(x->mr_rem, per_core) : 0;
        x->m_c1 = per_core * mr;
        x->m_c1_last_core = (per_core - (x->p_l * per_core - x->mr_rem)) * mr;
        x->k_c1 = K % x->k_c;
        x->Mb = (M / pm) + x->m_pad;
        x->Kb = (K / x->k_c) + x->k_pad;
        x->M_padded = mr * x->mr_rem + (M / pm) * pm;
        x->pm = p; x->pn = 1;
        return;
    }

    /* MKN and NKM split K over the p "cores" of a block (:518-587) */
    const int pk = p * x->k_c;
    x->k_pad = (K % pk) ? 1 : 0;
    x->k_rem = K % pk;
    x->k_c1 = ceil_div_d(x->k_rem, p);
    x->p_l = x->k_c1 ? ceil_div_d(x->k_rem, x->k_c1) : 0;
    x->k_c1_last_core = x->k_rem - x->k_c1 * (x->p_l - 1);
    x->Kb = (K / pk) + x->k_pad;
    if (x->sch == ORACLE_MKN) {
        x->m_pad = (M % x->m_c) ? 1 : 0;
        x->mr_rem = ceil_div_d(M % x->m_c, mr);
        x->m_c1 = x->mr_rem * mr;
        x->Mb = (M / x->m_c) + x->m_pad;
        x->M_padded = (M / x->m_c) * x->m_c + x->m_c1;
        x->pm = p; x->pn = 1;
    } else {
        const int pm = p * x->m_c;
        x->m_pad = (M % pm) ? 1 : 0;
        x->mr_rem = ceil_div_d(M % pm, mr);
        x->m_c1 = x->mr_rem * mr;
        x->Mb = (M / pm) + x->m_pad;
        x->M_padded = (M / pm) * pm + x->m_c1;
        x->pm = 1; x->pn = p;
    }
}

void oracle_block_dims_flat(int M, int N, int K, int p, oracle_cntx_t* c, int sch,
                            int mcu, int kcu, int ncu, int* out26) {
    oracle_blk_t x;
    oracle_init_block_dims(M, N, K, p, &x, c, sch, mcu, kcu, ncu);
    memcpy(out26, &x, 26 * sizeof(int));
}

/* cake_sgemm_packed_{A,B,C}_size, src/pack_helper.cpp:5-87 (bytes). */
static int padded_M(int M, int p, const oracle_blk_t* x, const oracle_cntx_t* c, int sch) {
    int blk = (sch == ORACLE_MKN) ? x->m_c : p * x->m_c;
    return (M / blk) * blk + c->mr * ceil_div_d(M % blk, c->mr);
}
static int padded_N(int N, const oracle_blk_t* x, const oracle_cntx_t* c) {
    return (N - (N % x->n_c)) + c->nr * (int) ceil(((double) (N % x->n_c) / c->nr));
}
size_t oracle_packed_A_size(int M, int K, int p, const oracle_blk_t* x, const oracle_cntx_t* c, int sch) {
    return (size_t) (padded_M(M, p, x, c, sch) * K) * sizeof(float);
}
size_t oracle_packed_B_size(int K, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c) {
    (void) p;
    return (size_t) (K * padded_N(N, x, c)) * sizeof(float);
}
size_t oracle_packed_C_size(int M, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c, int sch) {
    return (size_t) (padded_M(M, p, x, c, sch) * padded_N(N, x, c)) * sizeof(float);
}

/* -------------------------------------------------------- operation blocks */

/* pack_ob_A_single_buf, src/pack_ob.cpp:40-60: an m_c x k_c block of A becomes
 * panels of m_r rows; inside a panel k runs slowest, the m_r rows fastest.
 * Rows at or beyond M are zero.  `A` points at the block's first element. */
static void ob_pack_A(const float* A, float* out, int M, int K, int row0, int rows, int kc, int mr) {
    size_t w = 0;
    for (int r = 0; r < rows; r += mr)
        for (int k = 0; k < kc; k++)
            for (int j = 0; j < mr; j++)
                out[w++] = (row0 + r + j < M) ? A[(size_t) (r + j) * K + k] : 0.0f;
}

/* pack_ob_B_single_buf, src/pack_ob.cpp:105-140: panels of n_r columns, each
 * k_c rows of n_r contiguous values; columns at or beyond N are zero. */
static void ob_pack_B(const float* B, float* out, int N, int col0, int kc, int cols, int nr) {
    size_t w = 0;
    for (int q = 0; q < cols; q += nr)
        for (int k = 0; k < kc; k++)
            for (int j = 0; j < nr; j++)
                out[w++] = (col0 + q + j < N) ? B[(size_t) k * N + q + j] : 0.0f;
}

/* pack_ob_C_single_buf / unpack_ob_C_single_buf, src/pack_ob.cpp:253-288,393-411:
 * n_r-column panels outermost, then m_r-row panels, then an m_r x n_r row-major tile. */
static void ob_pack_C(const float* C, float* out, int M, int N, int row0, int col0,
                      int rows, int cols, int mr, int nr) {
    size_t w = 0;
    for (int q = 0; q < cols; q += nr)
        for (int r = 0; r < rows; r += mr)
            for (int i = 0; i < mr; i++)
                for (int j = 0; j < nr; j++, w++)
                    out[w] = (col0 + q + j < N && row0 + r + i < M) ? C[(size_t) (r + i) * N + q + j] : 0.0f;
}
static void ob_unpack_C(float* C, const float* in, int M, int N, int row0, int col0,
                        int rows, int cols, int mr, int nr) {
    size_t w = 0;
    for (int q = 0; q < cols; q += nr)
        for (int r = 0; r < rows; r += mr)
            for (int i = 0; i < mr; i++)
                for (int j = 0; j < nr; j++, w++)
                    if (col0 + q + j < N && row0 + r + i < M) C[(size_t) (r + i) * N + q + j] = in[w];
}

/* The register-tile product, src/kernels/haswell/dense.cpp:8-203: every element
 * of the m_r x n_r tile receives one fused multiply-add per k, k ascending. */
static void ukernel(const float* Ap, const float* Bp, float* Ct, int mr, int nr, int kc) {
    for (int k = 0; k < kc; k++) {
        const float* a = Ap + (size_t) k * mr;
        const float* b = Bp + (size_t) k * nr;
        for (int i = 0; i < mr; i++) {
            const float ai = a[i];
            float* crow = Ct + (size_t) i * nr;
            for (int j = 0; j < nr; j++) crow[j] = __builtin_fmaf(ai, b[j], crow[j]);
        }
    }
}

/* The m_reg / n_reg loops shared by all schedules (src/cake_sgemm_k_first.cpp:113-127,
 * cake_sgemm_m_first.cpp:100-108, cake_sgemm_n_first.cpp:100-108). */
static void ob_multiply(const float* Ap, const float* Bp, float* Cp, int rows, int cols, int kc,
                        int mr, int nr) {
    for (int q = 0; q < cols / nr; q++)
        for (int r = 0; r < rows / mr; r++)
            ukernel(Ap + (size_t) r * mr * kc, Bp + (size_t) q * kc * nr,
                    Cp + (size_t) q * rows * nr + (size_t) r * mr * nr, mr, nr, kc);
}

/* ---------------------------------------------------- geometry of a visit */

typedef struct {
    int used;   /* cores (K-first: row slabs; M/N-first: K slices) active in this block */
    int full;   /* extent of the whole block along the split dimension */
    int step;   /* extent owned by every core but the last */
    int last;   /* extent owned by the last active core */
} split_t;

/* K-first splits the M extent of a block over cores (src/cake_sgemm_k_first.cpp:75-98). */
static split_t split_rows_kmn(const oracle_blk_t* x, int m, int p, int mr) {
    split_t s;
    if (m == x->Mb - 1 && x->m_pad) {
        s.used = x->p_l; s.full = mr * x->mr_rem; s.step = x->m_c1; s.last = x->m_c1_last_core;
    } else {
        s.used = p; s.full = p * x->m_c; s.step = x->m_c; s.last = x->m_c;
    }
    return s;
}
/* M-first / N-first split the K extent (src/cake_sgemm_m_first.cpp:60-96). */
static split_t split_k(const oracle_blk_t* x, int k, int p) {
    split_t s;
    if (k == x->Kb - 1 && x->k_pad) {
        s.used = x->p_l; s.full = x->k_rem; s.step = x->k_c1; s.last = x->k_c1_last_core;
    } else {
        s.used = p; s.full = p * x->k_c; s.step = x->k_c; s.last = x->k_c;
    }
    return s;
}
static int core_extent(const split_t* s, int core) { return core == s->used - 1 ? s->last : s->step; }

static int ncols_of(const oracle_blk_t* x, int n) { return (n == x->Nb - 1 && x->n_pad) ? x->n_c1 : x->n_c; }
static int col0_of(const oracle_blk_t* x, int n, int N) {
    return (n == x->Nb - 1 && x->n_pad) ? (N - (N % x->n_c)) : n * x->n_c;
}

/* ------------------------------------------------------------------ packers */

/* pack_A_single_buf_k_first (src/pack_k_first.cpp:7-76),
 * pack_A_single_buf_m_first (src/pack_m_first.cpp:7-78),
 * pack_A_single_buf_n_first (src/pack_n_first.cpp:8-79). */
void oracle_pack_A(const float* A, float* A_p, int M, int K, int p, const oracle_blk_t* x, const oracle_cntx_t* c) {
    const int mr = c->mr;
    size_t off = 0;
    if (x->sch == ORACLE_KMN) {
        for (int m = 0; m < x->Mb; m++) {
            split_t s = split_rows_kmn(x, m, p, mr);
            for (int k = 0; k < x->Kb; k++) {
                int kc = (k == x->Kb - 1 && x->k_pad) ? x->k_c1 : x->k_c;
                const float* base = A + (size_t) m * p * x->m_c * K + (size_t) k * x->k_c;
                for (int core = 0; core < s.used; core++)
                    ob_pack_A(base + (size_t) core * s.step * K, A_p + off + (size_t) core * s.step * kc,
                              M, K, m * p * x->m_c + core * s.step, core_extent(&s, core), kc, mr);
                off += (size_t) s.full * kc;
            }
        }
        return;
    }
    const int m_first = (x->sch == ORACLE_MKN);
    const int mblk = m_first ? x->m_c : p * x->m_c;
    /* M-first walks k outermost, N-first walks m outermost */
    const int outer_n = m_first ? x->Kb : x->Mb, inner_n = m_first ? x->Mb : x->Kb;
    for (int o = 0; o < outer_n; o++)
        for (int i = 0; i < inner_n; i++) {
            int k = m_first ? o : i, m = m_first ? i : o;
            split_t s = split_k(x, k, p);
            int rows = (m == x->Mb - 1 && x->m_pad) ? x->m_c1 : mblk;
            const float* base = A + (size_t) m * mblk * K + (size_t) k * p * x->k_c;
            for (int core = 0; core < s.used; core++)
                ob_pack_A(base + (size_t) core * s.step, A_p + off + (size_t) core * s.step * rows,
                          M, K, m * mblk, rows, core_extent(&s, core), mr);
            off += (size_t) s.full * rows;
        }
}

/* pack_B_k_first (src/pack_k_first.cpp:187-283), pack_B_m_first
 * (src/pack_m_first.cpp:83-144), pack_B_n_first (src/pack_n_first.cpp:84-144). */
void oracle_pack_B(const float* B, float* B_p, int K, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c) {
    const int nr = c->nr;
    size_t off = 0;
    (void) K;
    if (x->sch == ORACLE_KMN) {
        for (int n = 0; n < x->Nb; n++) {
            int cols = ncols_of(x, n), col0 = col0_of(x, n, N);
            for (int k = 0; k < x->Kb; k++) {
                int kc = (k == x->Kb - 1 && x->k_pad) ? x->k_c1 : x->k_c;
                ob_pack_B(B + (size_t) k * x->k_c * N + (size_t) n * x->n_c, B_p + off, N, col0, kc, cols, nr);
                off += (size_t) kc * cols;
            }
        }
        return;
    }
    const int m_first = (x->sch == ORACLE_MKN);
    const int outer_n = m_first ? x->Nb : x->Kb, inner_n = m_first ? x->Kb : x->Nb;
    for (int o = 0; o < outer_n; o++)
        for (int i = 0; i < inner_n; i++) {
            int n = m_first ? o : i, k = m_first ? i : o;
            int cols = ncols_of(x, n), col0 = col0_of(x, n, N);
            split_t s = split_k(x, k, p);
            const float* base = B + (size_t) k * p * x->k_c * N + (size_t) n * x->n_c;
            for (int core = 0; core < s.used; core++)
                ob_pack_B(base + (size_t) core * s.step * N, B_p + off + (size_t) core * s.step * cols,
                          N, col0, core_extent(&s, core), cols, nr);
            off += (size_t) s.full * cols;
        }
}

/* One walker serves pack_C and unpack_C of all three schedules:
 * pack_C_single_buf_k_first (src/pack_k_first.cpp:404-472) / unpack (src/unpack_k_first.cpp:5-67),
 * _m_first (src/pack_m_first.cpp:148-200, src/unpack_m_first.cpp:5-49),
 * _n_first (src/pack_n_first.cpp:155-209, src/unpack_n_first.cpp:5-49).
 * For N-first the block offsets are those the schedule and the unpacker use
 * (src/cake_sgemm_n_first.cpp:98, src/unpack_n_first.cpp:45); the reference's
 * N-first pack_C uses a different offset for ragged edge blocks
 * (src/pack_n_first.cpp:205) and is only self-consistent for aligned shapes. */
static void walk_C(float* C, float* C_p, int M, int N, int p, const oracle_blk_t* x,
                   const oracle_cntx_t* c, int unpack) {
    const int mr = c->mr, nr = c->nr;
    if (x->sch == ORACLE_KMN) {
        size_t off = 0;
        for (int n = 0; n < x->Nb; n++) {
            int cols = ncols_of(x, n), col0 = col0_of(x, n, N);
            for (int m = 0; m < x->Mb; m++) {
                split_t s = split_rows_kmn(x, m, p, mr);
                int row_base = (m == x->Mb - 1 && x->m_pad) ? (M - (M % (p * x->m_c))) : m * p * x->m_c;
                for (int core = 0; core < s.used; core++) {
                    float* Cb = C + (size_t) (m * p * x->m_c + core * s.step) * N + (size_t) n * x->n_c;
                    float* Pb = C_p + off + (size_t) core * s.step * cols;
                    if (unpack) ob_unpack_C(Cb, Pb, M, N, row_base + core * s.step, col0, core_extent(&s, core), cols, mr, nr);
                    else        ob_pack_C(Cb, Pb, M, N, row_base + core * s.step, col0, core_extent(&s, core), cols, mr, nr);
                }
                off += (size_t) s.full * cols;
            }
        }
        return;
    }
    const int m_first = (x->sch == ORACLE_MKN);
    const int mblk = m_first ? x->m_c : p * x->m_c;
    for (int m = 0; m < x->Mb; m++) {
        int ragged_m = (m == x->Mb - 1 && x->m_pad);
        int rows = ragged_m ? x->m_c1 : mblk;
        int row0 = ragged_m ? (M - (M % mblk)) : m * mblk;
        for (int n = 0; n < x->Nb; n++) {
            int cols = ncols_of(x, n), col0 = col0_of(x, n, N);
            size_t off = m_first ? (size_t) x->M_padded * n * x->n_c + (size_t) m * x->m_c * cols
                                 : (size_t) x->N_padded * m * mblk + (size_t) n * rows * x->n_c;
            float* Cb = C + (size_t) m * mblk * N + (size_t) n * x->n_c;
            if (unpack) ob_unpack_C(Cb, C_p + off, M, N, row0, col0, rows, cols, mr, nr);
            else        ob_pack_C(Cb, C_p + off, M, N, row0, col0, rows, cols, mr, nr);
        }
    }
}
void oracle_pack_C(const float* C, float* C_p, int M, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c) {
    walk_C((float*) C, C_p, M, N, p, x, c, 0);
}
void oracle_unpack_C(float* C, const float* C_p, int M, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c) {
    walk_C(C, (float*) C_p, M, N, p, x, c, 1);
}

void oracle_packed_sizes(int M, int N, int K, int p, oracle_cntx_t* c, int sch, size_t* out3) {
    oracle_blk_t x;
    oracle_init_block_dims(M, N, K, p, &x, c, sch, 0, 0, 0);
    out3[0] = oracle_packed_A_size(M, K, p, &x, c, x.sch);
    out3[1] = oracle_packed_B_size(K, N, p, &x, c);
    out3[2] = oracle_packed_C_size(M, N, p, &x, c, x.sch);
}

void oracle_pack(int which, const float* src, float* dst, int M, int N, int K, int p,
                 oracle_cntx_t* c, int sch) {
    oracle_blk_t x;
    oracle_init_block_dims(M, N, K, p, &x, c, sch, 0, 0, 0);
    switch (which) {
        case 0: oracle_pack_A(src, dst, M, K, p, &x, c); break;
        case 1: oracle_pack_B(src, dst, K, N, p, &x, c); break;
        case 2: oracle_pack_C(src, dst, M, N, p, &x, c); break;
        default: oracle_unpack_C(dst, src, M, N, p, &x, c); break;
    }
}

/* ---------------------------------------------------------------- schedules */

/* schedule_KMN, src/cake_sgemm_k_first.cpp:9-153.  Blocks are visited n
 * ascending, m snaking with n, k snaking with (n, m); each core accumulates its
 * m_c x n_c slab of C over all k-blocks in a zeroed private buffer and then
 * writes it straight to C. */
static void run_KMN(const float* A_p, const float* B_p, float* C, int M, int N, int K, int p,
                    const oracle_blk_t* x, const oracle_cntx_t* c) {
    const int mr = c->mr, nr = c->nr;
    for (int n = 0; n < x->Nb; n++) {
        int cols = ncols_of(x, n), col0 = col0_of(x, n, N);
        for (int mi = 0; mi < x->Mb; mi++) {
            int m = (n % 2) ? x->Mb - 1 - mi : mi;
            int k_fwd = ((n + m) % 2) == 0;
            split_t s = split_rows_kmn(x, m, p, mr);
            int row_base = (m == x->Mb - 1 && x->m_pad) ? (M - (M % (p * x->m_c))) : m * p * x->m_c;
#pragma omp parallel for schedule(static)
            for (int core = 0; core < s.used; core++) {
                int rows = core_extent(&s, core);
                float* slab = (float*) calloc((size_t) x->m_c * x->n_c, sizeof(float));
                for (int ki = 0; ki < x->Kb; ki++) {
                    int k = k_fwd ? ki : x->Kb - 1 - ki;
                    int kc = (k == x->Kb - 1 && x->k_pad) ? x->k_c1 : x->k_c;
                    size_t a = (size_t) m * p * x->m_c * K + (size_t) k * s.full * x->k_c + (size_t) core * s.step * kc;
                    size_t b = (size_t) n * K * x->n_c + (size_t) k * x->k_c * cols;
                    ob_multiply(A_p + a, B_p + b, slab, rows, cols, kc, mr, nr);
                }
                ob_unpack_C(C + (size_t) (m * p * x->m_c + core * s.step) * N + (size_t) n * x->n_c, slab,
                            M, N, row_base + core * s.step, col0, rows, cols, mr, nr);
                free(slab);
            }
        }
    }
}

/* schedule_MKN (src/cake_sgemm_m_first.cpp:4-113) and schedule_NKM
 * (src/cake_sgemm_n_first.cpp:4-113).  K is the only dimension whose visiting
 * order changes a result: k-blocks go forward for even outer index and
 * backward for odd, and inside a k-block the p slices are taken in order. */
static void run_MKN_NKM(const float* A_p, const float* B_p, float* C_p, int M, int N, int K, int p,
                        const oracle_blk_t* x, const oracle_cntx_t* c) {
    const int mr = c->mr, nr = c->nr;
    const int m_first = (x->sch == ORACLE_MKN);
    const int mblk = m_first ? x->m_c : p * x->m_c;
    const int outer_n = m_first ? x->Nb : x->Mb, par_n = m_first ? x->Mb : x->Nb;
    (void) M; (void) N;
    for (int o = 0; o < outer_n; o++)
        for (int ki = 0; ki < x->Kb; ki++) {
            int k = (o % 2) ? x->Kb - 1 - ki : ki;
            split_t s = split_k(x, k, p);
#pragma omp parallel for schedule(static)
            for (int q = 0; q < par_n; q++) {
                int m = m_first ? q : o, n = m_first ? o : q;
                int rows = (m == x->Mb - 1 && x->m_pad) ? x->m_c1 : mblk;
                int cols = ncols_of(x, n);
                for (int core = 0; core < s.used; core++) {
                    int kc = core_extent(&s, core);
                    size_t a, b, cc;
                    if (m_first) {
                        a = (size_t) k * x->M_padded * p * x->k_c + (size_t) m * x->m_c * s.full + (size_t) core * rows * s.step;
                        b = (size_t) n * K * x->n_c + (size_t) k * p * x->k_c * cols + (size_t) core * s.step * cols;
                        cc = (size_t) n * x->M_padded * x->n_c + (size_t) m * x->m_c * cols;
                    } else {
                        a = (size_t) m * mblk * K + (size_t) rows * k * p * x->k_c + (size_t) core * rows * s.step;
                        b = (size_t) k * p * x->k_c * x->N_padded + (size_t) n * x->n_c * s.full + (size_t) core * s.step * cols;
                        cc = (size_t) m * mblk * x->N_padded + (size_t) rows * n * x->n_c;
                    }
                    ob_multiply(A_p + a, B_p + b, C_p + cc, rows, cols, kc, mr, nr);
                }
            }
        }
}

/* cake_sgemm, src/cake_sgemm.cpp:9-175.  `alpha` is never applied by the
 * reference; K-first overwrites C; M-first / N-first start from packed C when
 * beta != 0 (adding A*B on top, unscaled) and from zeros otherwise. */
int oracle_cake_sgemm(const float* A, const float* B, float* C, int M, int N, int K, int p,
                      oracle_cntx_t* c, int sch, float beta, int mcu, int kcu, int ncu) {
    oracle_blk_t x;
    oracle_init_block_dims(M, N, K, p, &x, c, sch, mcu, kcu, ncu);
    float* A_p = (float*) malloc(oracle_packed_A_size(M, K, p, &x, c, x.sch) + 64);
    float* B_p = (float*) malloc(oracle_packed_B_size(K, N, p, &x, c) + 64);
    oracle_pack_A(A, A_p, M, K, p, &x, c);
    oracle_pack_B(B, B_p, K, N, p, &x, c);
    if (x.sch == ORACLE_KMN) {
        run_KMN(A_p, B_p, C, M, N, K, p, &x, c);
    } else {
        size_t csz = oracle_packed_C_size(M, N, p, &x, c, x.sch);
        float* C_p = (float*) calloc(csz / sizeof(float) + 16, sizeof(float));
        if (beta != 0) oracle_pack_C(C, C_p, M, N, p, &x, c);
        run_MKN_NKM(A_p, B_p, C_p, M, N, K, p, &x, c);
        oracle_unpack_C(C, C_p, M, N, p, &x, c);
        free(C_p);
    }
    free(A_p);
    free(B_p);
    return x.sch;
}

/* ------------------------------------------------------------------ variants */

/* im_2_col, examples/cake_conv.cpp:1178-1213, extended with a batch dimension
 * and zero padding: row index k = (cin, hf, wf), column index n = (b, ho, wo). */
void oracle_im2col(const float* in, float* col, int batch, int cin, int H, int W,
                   int hf, int wf, int stride, int pad) {
    const int Ho = (H + 2 * pad - hf) / stride + 1, Wo = (W + 2 * pad - wf) / stride + 1;
    const size_t Ncol = (size_t) batch * Ho * Wo;
    for (int ci = 0; ci < cin; ci++)
        for (int fh = 0; fh < hf; fh++)
            for (int fw = 0; fw < wf; fw++) {
                float* row = col + (size_t) ((ci * hf + fh) * wf + fw) * Ncol;
                for (int b = 0; b < batch; b++)
                    for (int ho = 0; ho < Ho; ho++)
                        for (int wo = 0; wo < Wo; wo++) {
                            int h = ho * stride - pad + fh, w = wo * stride - pad + fw;
                            float v = 0.0f;
                            if (h >= 0 && h < H && w >= 0 && w < W)
                                v = in[(((size_t) b * cin + ci) * H + h) * W + w];
                            row[((size_t) b * Ho + ho) * Wo + wo] = v;
                        }
            }
}

/* GEMM route of examples/cake_conv.cpp:1007-1066: C[Cout x (b,ho,wo)] = F * im2col. */
void oracle_conv2d(const float* in, const float* filt, float* out, int batch, int cin, int H, int W,
                   int cout, int hf, int wf, int stride, int pad, int p, oracle_cntx_t* c) {
    const int Ho = (H + 2 * pad - hf) / stride + 1, Wo = (W + 2 * pad - wf) / stride + 1;
    const int Kg = cin * hf * wf, Ng = batch * Ho * Wo;
    float* col = (float*) malloc((size_t) Kg * Ng * sizeof(float));
    float* Cg = (float*) calloc((size_t) cout * Ng, sizeof(float));
    oracle_im2col(in, col, batch, cin, H, W, hf, wf, stride, pad);
    oracle_cake_sgemm(filt, col, Cg, cout, Ng, Kg, p, c, ORACLE_NA, 0.0f, 0, 0, 0);
    for (int b = 0; b < batch; b++)
        for (int co = 0; co < cout; co++)
            memcpy(out + ((size_t) b * cout + co) * Ho * Wo, Cg + (size_t) co * Ng + (size_t) b * Ho * Wo,
                   (size_t) Ho * Wo * sizeof(float));
    free(col);
    free(Cg);
}

/* The reference's small-matrix schedules compute nothing
 * (src/cake_sgemm_small.cpp:68-71); the live path for a small product is
 * cake_sgemm itself, called once per item. */
void oracle_sgemm_batched(const float* A, const float* B, float* C, int M, int N, int K,
                          int batch, int p, oracle_cntx_t* c) {
    for (int i = 0; i < batch; i++)
        oracle_cake_sgemm(A + (size_t) i * M * K, B + (size_t) i * K * N, C + (size_t) i * M * N,
                          M, N, K, p, c, ORACLE_NA, 0.0f, 0, 0, 0);
}

/* cake_sp_sgemm_haswell_6x16, src/kernels/haswell/sparse.cpp:7-126: for each
 * stored column k of A (ascending), every nonzero a[m,k] issues
 * C[m,:] = fma(a, B[k,:], C[m,:]); zeros issue nothing.  Pinned: bit-identical to that
 * microkernel driven tile by tile over whole matrices (oracle/ref_sparse_driver.cpp,
 * tests/test_oracle_vs_reference.py) and to its stored outputs (tests/golden/). */
void oracle_sp_sgemm(const float* A, const float* B, float* C, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        float* crow = C + (size_t) m * N;
        for (int n = 0; n < N; n++) crow[n] = 0.0f;
        for (int k = 0; k < K; k++) {
            float a = A[(size_t) m * K + k];
            if (a == 0.0f) continue;
            const float* brow = B + (size_t) k * N;
            for (int n = 0; n < N; n++) crow[n] = __builtin_fmaf(a, brow[n], crow[n]);
        }
    }
}

/* cake_sgemv of the reference's matrix-vector example: schedule_mvm
 * (examples/cake_gemv.cpp:424-489) walks blocks of rows and, inside, blocks of k in
 * ascending order, and its microkernel cake_sgemv_haswell_8x8_col (:87-140) loads C,
 * issues c = fma(A[k*M + m], B[k], c) for k ascending and stores C.  Per output
 * element that is one chain of fused multiply-adds over k = 0 .. K-1 on top of the
 * value C held on entry; A is column-major (A[k*M + m]).  Pinned: bit-identical to that
 * microkernel driven eight rows at a time (oracle/ref_gemv_driver.cpp; the example is a
 * stand-alone program, so only the microkernel is compiled, not its main), and to its
 * stored outputs (tests/golden/). */
void oracle_sgemv(const float* A, const float* B, float* C, int M, int K) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        float c = C[m];
        for (int k = 0; k < K; k++) c = __builtin_fmaf(A[(size_t) k * M + m], B[k], c);
        C[m] = c;
    }
}

/* --------------------------------------------------------------- generators */

static inline uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline float u01(uint64_t seed, uint64_t i) {
    return (float) (splitmix64(seed * 0x9E3779B97F4A7C15ull + i) >> 40) * (1.0f / 16777216.0f);
}
/* uniform in [-1, 1), the range of rand_init (src/util.cpp:259-267) */
void oracle_fill_uniform(float* x, size_t n, unsigned long long seed) {
    for (size_t i = 0; i < n; i++) x[i] = u01(seed, i) * 2.0f - 1.0f;
}
/* Box-Muller, as normalRandom does (src/util.cpp:270-280) */
void oracle_fill_normal(float* x, size_t n, unsigned long long seed, float sigma) {
    for (size_t i = 0; i < n; i++) {
        float u1 = u01(seed, 2 * i), u2 = u01(seed, 2 * i + 1);
        if (u1 < 1e-7f) u1 = 1e-7f;
        x[i] = sigma * sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
    }
}
void oracle_fill_sparse(float* x, size_t n, unsigned long long seed, unsigned long long mask_seed,
                        double density) {
    for (size_t i = 0; i < n; i++)
        x[i] = ((double) u01(mask_seed, i) < density) ? u01(seed, i) * 2.0f - 1.0f : 0.0f;
}
