/* TEST INFRASTRUCTURE ONLY: C-ABI wrapper around the UNMODIFIED reference
 * (vnatesh/CAKE_on_CPU), compiled from the reference's own sources where
 * they lie by oracle/Makefile into oracle/_ref/libcake_ref.so.
 *
 * Every function here forwards to the reference function named in its
 * comment; nothing is re-implemented.  Used by tests (parity oracle) and by
 * the CPU-baseline leg of bench.py, never by the product path.
 */
#include "cake.h"

int ref_shim_ncores = 1;

extern "C" {

/* Deterministic context: same fields cake_query_cntx() fills
 * (src/block_sizing.cpp:40-75) but with caller-given cache sizes, so block
 * sizes (and therefore summation order) do not depend on the host. */
void* ref_ctx_make(int L1, int L2, int L3, int ncores) {
    cake_cntx_t* c = (cake_cntx_t*) malloc(sizeof(cake_cntx_t));
    c->blis_cntx = NULL;
    c->alpha_n = 1.0;
    c->peak_dram_bw = 32 * 1e9;
    c->peak_flops = 600 * 1e9;
    c->mr = MR_MIN;
    c->nr = NR_MIN;
    c->m_map = 0;
    c->n_map = 0;
    c->L1 = L1;
    c->L2 = L2;
    c->L3 = L3;
    c->ncores = ncores;
    ref_shim_ncores = ncores;
    return c;
}

/* cake_query_cntx(), src/block_sizing.cpp:40 (lscpu-derived cache sizes). */
void* ref_ctx_query(void) {
    cake_cntx_t* c = cake_query_cntx();
    ref_shim_ncores = c->ncores;
    return c;
}

void ref_ctx_get(void* ctx, int* out6, double* alpha_n) {
    cake_cntx_t* c = (cake_cntx_t*) ctx;
    out6[0] = c->mr; out6[1] = c->nr; out6[2] = c->L1;
    out6[3] = c->L2; out6[4] = c->L3; out6[5] = c->ncores;
    *alpha_n = c->alpha_n;
}

void ref_ctx_free(void* ctx) { free(ctx); }

/* cake_sgemm(), src/cake_sgemm.cpp:9.  variant: 0 = cake_sgemm,
 * 1 = cake_sgemm_online (src/cake_sgemm.cpp:397), 2 = cake_sgemm_2d (:179). */
double ref_cake_sgemm(float* A, float* B, float* C, int M, int N, int K, int p, void* ctx,
                      int sch, float beta, int mcu, int kcu, int ncu, int variant) {
    cake_cntx_t* c = (cake_cntx_t*) ctx;
    switch (variant) {
        case 1:  return cake_sgemm_online(A, B, C, M, N, K, p, c, NULL, 0, 0, 1, beta, (enum sched) sch, mcu, kcu, ncu);
        case 2:  return cake_sgemm_2d(A, B, C, M, N, K, p, c, NULL, 0, 0, 1, beta, (enum sched) sch, mcu, kcu, ncu);
        default: return cake_sgemm(A, B, C, M, N, K, p, c, NULL, 0, 0, 1, beta, (enum sched) sch, mcu, kcu, ncu);
    }
}

/* init_block_dims(), src/block_sizing.cpp:465; fields in struct order
 * (include/common.h:108-135), 26 ints. */
void ref_init_block_dims(int M, int N, int K, int p, void* ctx, int sch,
                         int mcu, int kcu, int ncu, int* out26) {
    blk_dims_t x;
    memset(&x, 0, sizeof(x));
    init_block_dims(M, N, K, p, &x, (cake_cntx_t*) ctx, (enum sched) sch, NULL, 4, mcu, kcu, ncu);
    int v[26] = {x.m_c, x.k_c, x.n_c, x.m_c1, x.k_c1, x.n_c1, x.m_c1_last_core, x.n_c1_last_core,
                 x.k_c1_last_core, x.mr_rem, x.nr_rem, x.k_rem, x.p_l, x.pm_l, x.pn_l, x.pm, x.pn,
                 x.m_pad, x.k_pad, x.n_pad, x.Mb, x.Kb, x.Nb, x.M_padded, x.N_padded, (int) x.sch};
    memcpy(out26, v, sizeof(v));
}

/* derive_schedule(), src/block_sizing.cpp:434 */
int ref_derive_schedule(int M, int N, int K, int p, int mc_ret, void* ctx) {
    return (int) derive_schedule(M, N, K, p, mc_ret, (cake_cntx_t*) ctx);
}

/* set_schedule(), src/cake_sgemm.cpp:768 */
int ref_set_schedule(int sch, int M, int N, int K) {
    return (int) set_schedule((enum sched) sch, M, N, K);
}

/* cake_sgemm_packed_{A,B,C}_size(), src/pack_helper.cpp:5-87 (bytes) */
void ref_packed_sizes(int M, int N, int K, int p, void* ctx, int sch, size_t* out3) {
    cake_cntx_t* c = (cake_cntx_t*) ctx;
    blk_dims_t x;
    memset(&x, 0, sizeof(x));
    init_block_dims(M, N, K, p, &x, c, (enum sched) sch, NULL, 4, 0, 0, 0);
    out3[0] = cake_sgemm_packed_A_size(M, K, p, &x, c, x.sch);
    out3[1] = cake_sgemm_packed_B_size(K, N, p, &x, c);
    out3[2] = cake_sgemm_packed_C_size(M, N, p, &x, c, x.sch);
}

/* pack_A / pack_B / pack_C / unpack_C, src/pack_helper.cpp:92-184.
 * which: 0 = A, 1 = B, 2 = C, 3 = unpack C (src is the packed buffer). */
void ref_pack(int which, float* src, float* dst, int M, int N, int K, int p, void* ctx, int sch) {
    cake_cntx_t* c = (cake_cntx_t*) ctx;
    blk_dims_t x;
    memset(&x, 0, sizeof(x));
    omp_set_num_threads(p);
    init_block_dims(M, N, K, p, &x, c, (enum sched) sch, NULL, 4, 0, 0, 0);
    switch (which) {
        case 0: pack_A(src, dst, M, K, p, &x, c, x.sch); break;
        case 1: pack_B(src, dst, K, N, p, &x, c, x.sch); break;
        case 2: pack_C(src, dst, M, N, p, &x, c, x.sch); break;
        case 3: unpack_C(dst, src, M, N, p, &x, c, x.sch); break;
    }
}

/* rand_init(), src/util.cpp:259, after srand(seed) (examples/cake_conv.cpp:924 uses srand(1)). */
void ref_rand_init(unsigned seed, float* mat, int r, int cols) {
    srand(seed);
    rand_init(mat, r, cols);
}

/* cake_sgemm_checker(), src/util.cpp:173: returns 0 when |C - naive| <= 1e-3 everywhere. */
int ref_checker(float* A, float* B, float* C, int N, int M, int K) {
    return (int) cake_sgemm_checker(A, B, C, N, M, K);
}

}  /* extern "C" */
