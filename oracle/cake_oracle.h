/* TEST INFRASTRUCTURE ONLY -- never linked into or called from the product path.
 *
 * Plain-C restatement of the SGEMM path of vnatesh/CAKE_on_CPU: block sizing,
 * schedule derivation, the K-first / M-first / N-first block schedules, the
 * pack / unpack routines and the variants built on top of them (im2col
 * convolution, batched small GEMM, sparse-A row-skipping product).
 *
 * Parity status: PINNED for the dense path.  tests/test_oracle_vs_reference.py
 * checks every function below bit-for-bit against the unmodified reference
 * compiled from its own sources (oracle/_ref/libcake_ref.so), and
 * tests/golden/ holds outputs of that reference for hosts where it is absent.
 * The sparse restatement follows a reference kernel that the reference never
 * builds or calls (src/kernels/haswell/sparse.cpp:7-131): parity UNPINNED for
 * it beyond agreement with the dense product on the densified operand.
 */
#ifndef CAKE_ORACLE_H
#define CAKE_ORACLE_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_KMN = 0, ORACLE_MKN = 1, ORACLE_NKM = 2, ORACLE_NA = 3 };

/* include/common.h:138-151 (the fields the SGEMM path reads) */
typedef struct oracle_cntx_t {
    double alpha_n;
    int mr, nr;
    int L1, L2, L3;
    int ncores;
} oracle_cntx_t;

/* include/common.h:108-135, same field order */
typedef struct oracle_blk_t {
    int m_c, k_c, n_c;
    int m_c1, k_c1, n_c1;
    int m_c1_last_core, n_c1_last_core, k_c1_last_core;
    int mr_rem, nr_rem, k_rem;
    int p_l, pm_l, pn_l, pm, pn;
    int m_pad, k_pad, n_pad;
    int Mb, Kb, Nb;
    int M_padded, N_padded;
    int sch;
} oracle_blk_t;

void oracle_cntx_init(oracle_cntx_t* c, int L1, int L2, int L3, int ncores);

int  oracle_derive_schedule(int M, int N, int K, int p, int mc_ret, const oracle_cntx_t* c);
int  oracle_set_schedule(int sch, int M, int N, int K);
void oracle_init_block_dims(int M, int N, int K, int p, oracle_blk_t* x, oracle_cntx_t* c,
                            int sch, int mcu, int kcu, int ncu);
/* 26 ints in struct order, for comparison with the reference */
void oracle_block_dims_flat(int M, int N, int K, int p, oracle_cntx_t* c, int sch,
                            int mcu, int kcu, int ncu, int* out26);

size_t oracle_packed_A_size(int M, int K, int p, const oracle_blk_t* x, const oracle_cntx_t* c, int sch);
size_t oracle_packed_B_size(int K, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c);
size_t oracle_packed_C_size(int M, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c, int sch);

void oracle_pack_A(const float* A, float* A_p, int M, int K, int p, const oracle_blk_t* x, const oracle_cntx_t* c);
void oracle_pack_B(const float* B, float* B_p, int K, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c);
void oracle_pack_C(const float* C, float* C_p, int M, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c);
void oracle_unpack_C(float* C, const float* C_p, int M, int N, int p, const oracle_blk_t* x, const oracle_cntx_t* c);

/* which: 0 = pack A, 1 = pack B, 2 = pack C, 3 = unpack C (src packed -> dst) */
void oracle_pack(int which, const float* src, float* dst, int M, int N, int K, int p,
                 oracle_cntx_t* c, int sch);
void oracle_packed_sizes(int M, int N, int K, int p, oracle_cntx_t* c, int sch, size_t* out3);

/* C = A*B through pack -> schedule -> unpack, exactly as the reference orders
 * its floating-point operations.  Returns the schedule that ran. */
int oracle_cake_sgemm(const float* A, const float* B, float* C, int M, int N, int K, int p,
                      oracle_cntx_t* c, int sch, float beta, int mcu, int kcu, int ncu);

/* im2col with batch and zero padding; K index (cin,hf,wf), N index (b,ho,wo). */
void oracle_im2col(const float* in, float* col, int batch, int cin, int H, int W,
                   int hf, int wf, int stride, int pad);
/* NCHW convolution = filters[Cout x Cin*hf*wf] * im2col, through oracle_cake_sgemm.
 * out is NCHW [batch][cout][Ho][Wo]. */
void oracle_conv2d(const float* in, const float* filt, float* out, int batch, int cin, int H, int W,
                   int cout, int hf, int wf, int stride, int pad, int p, oracle_cntx_t* c);

/* batch of independent small products, one oracle_cake_sgemm per item */
void oracle_sgemm_batched(const float* A, const float* B, float* C, int M, int N, int K,
                          int batch, int p, oracle_cntx_t* c);

/* sparse-A product with the row-skipping outer-product order of the
 * reference's sparse microkernel (zero entries of A contribute no operation). */
void oracle_sp_sgemm(const float* A, const float* B, float* C, int M, int N, int K);

/* C[m] += sum_k A[k*M + m] * B[k], one fused multiply-add chain per element over ascending k
 * (reference examples/cake_gemv.cpp:87-140, 424-489); pinned against that microkernel. */
void oracle_sgemv(const float* A, const float* B, float* C, int M, int K);

/* seeded generators shared by tests and benches (counter based, stateless) */
void oracle_fill_uniform(float* x, size_t n, unsigned long long seed);
void oracle_fill_normal(float* x, size_t n, unsigned long long seed, float sigma);
void oracle_fill_sparse(float* x, size_t n, unsigned long long seed, unsigned long long mask_seed,
                        double density);

#ifdef __cplusplus
}
#endif
#endif
