/* cake.h -- the C++ API of CAKE SGEMM, served by B200 kernels.
 *
 * Source compatible with the reference library's public header: code written
 * against vnatesh/CAKE_on_CPU's include/cake.h (and the headers it pulls in:
 * common.h, tiling.h, packing.h, util.h) compiles against this file and links
 * against libcake_b200.so instead of libcake.so.  Names, argument order,
 * default arguments and struct fields are the reference's; what each argument
 * means on a GPU is stated next to it.  Every function is a thin layer over the
 * C ABI in cake_b200.h.
 *
 * Differences a caller can observe:
 *   - errors are reported (message on stderr, negative return time) instead of
 *     exit(1);
 *   - data pointers may be host or device pointers;
 *   - `p` bounds the number of GPUs used instead of the number of CPU threads.
 */
#pragma once

/* the standard headers the reference's common.h makes visible to its callers */
#include <math.h>
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "cake_b200.h"

/* ------------------------------------------------------------------ types
 * Same members, same order as the reference (include/common.h:105-159). */

enum sched { KMN, MKN, NKM, NA };

typedef struct blk_dims_t {
    int m_c, k_c, n_c;
    int m_c1, k_c1, n_c1;
    int m_c1_last_core, n_c1_last_core, k_c1_last_core;
    int mr_rem, nr_rem, k_rem;
    int p_l, pm_l, pn_l, pm, pn;
    int m_pad, k_pad, n_pad;
    int Mb, Kb, Nb;
    int M_padded, N_padded;
    enum sched sch;
} blk_dims_t;

typedef struct cake_cntx_t {
    void* blis_cntx;     /* unused (NULL); kept so the struct stays layout compatible */
    double alpha_n;      /* aspect of the CB block; rewritten by get_cache_dims as in the reference */
    double peak_dram_bw; /* bytes/s of device memory */
    double peak_flops;   /* FP32-equivalent flop/s of the 3xTF32 tensor path */
    int mr, nr;          /* register tile of the reference = MMA tile here (128 x 256) */
    int m_map, n_map;    /* kernel_map indices of the reference; always 0 */
    int L1, L2, L3;      /* shared memory per SM, device L2, device memory (capped at INT_MAX) */
    int ncores;          /* visible B200 devices */
} cake_cntx_t;

typedef struct cache_dims_t {
    int m_c, k_c, n_c;
    enum sched sch;
} cache_dims_t;

#define cake_max(x, y) (((x) >= (y)) ? (x) : (y))
#define cake_min(x, y) (((x) <= (y)) ? (x) : (y))

/* ------------------------------------------------------------- the product
 * reference: include/cake.h:12-14, src/cake_sgemm.cpp:9-175.
 *   A (M x K), B (K x N), C (M x N): row-major FP32, host or device pointers.
 *   p          upper bound on the GPUs to use (host pointers: C is split by row
 *              blocks of M over min(p, ncores) devices, B replicated).
 *   cake_cntx  NULL = query the current device.
 *   argv       ignored, as in the reference.
 *   packedA/B  the pointer is a buffer produced by pack_A / pack_B with the same
 *              (M, N, K, p, cake_cntx, sch).
 *   alpha      accepted and ignored, exactly like the reference.
 *   beta       K-first overwrites C; M-first / N-first ADD A*B to C when
 *              beta != 0 (no scaling), as the reference does.
 *   sch        NA = derive from the shape (derive_schedule); otherwise forced.
 *              The schedule fixes the order in which tiles of C are produced.
 *   mcu,kcu,ncu  all non-zero = user block sizes for the packed layouts.
 * Returns the wall time of the whole call in seconds, negative on error. */
double cake_sgemm(float* A, float* B, float* C, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                  char* argv[] = NULL, bool packedA = 0, bool packedB = 0, float alpha = 1, float beta = 0,
                  enum sched sch = NA, int mcu = 0, int kcu = 0, int ncu = 0);

/* Variants of the K-first driver (reference include/cake.h:36-47): on-the-fly
 * packing (src/cake_sgemm.cpp:397-468), 2-D core grid (:179-247), 2-D small
 * (:253-318) and the test driver.  A GPU kernel always stages tiles on the fly
 * and tiles C in two dimensions, so all of them are the K-first product. */
double cake_sgemm_online(float* A, float* B, float* C, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                         char* argv[] = NULL, bool packedA = 0, bool packedB = 0, float alpha = 1, float beta = 0,
                         enum sched sch = NA, int mcu = 0, int kcu = 0, int ncu = 0);
double cake_sgemm_2d(float* A, float* B, float* C, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                     char* argv[] = NULL, bool packedA = 0, bool packedB = 0, float alpha = 1, float beta = 0,
                     enum sched sch = NA, int mcu = 0, int kcu = 0, int ncu = 0);
double cake_sgemm_2d_small(float* A, float* B, float* C, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                           char* argv[] = NULL, bool packedA = 0, bool packedB = 0, float alpha = 1, float beta = 0,
                           enum sched sch = NA);
double cake_sgemm_test(float* A, float* B, float* C, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                       char* argv[] = NULL, bool packedA = 0, bool packedB = 0, float alpha = 1, float beta = 0,
                       enum sched sch = NA);

/* Schedules on packed operands (reference include/cake.h:15-23).  K-first
 * writes the product to C (C_p is per-core scratch in the reference and is not
 * touched here); M-first / N-first add the product into the packed C_p. */
void schedule(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
              blk_dims_t* x, enum sched sch, bool sparse, bool small);
void schedule_KMN(float* A_p, float* B_p, float* C, float** C_p, int M, int N, int K, int p,
                  cake_cntx_t* cake_cntx, blk_dims_t* x);
void schedule_MKN(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                  blk_dims_t* x);
void schedule_NKM(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                  blk_dims_t* x);

/* The other K-first schedule entry points of the reference (include/cake.h:26-33).  _online, _2d
 * and _2d_small take PLAIN A, B, C; their A_p / B_p / C_p arguments are the reference's per-core
 * packing scratch, which has no role here (tiles are staged inside the kernel) and is left
 * untouched.  _C_unpacked takes A and B packed for K-first and ADDS the product into C_p, a plain
 * matrix with leading dimension x->N_padded (src/cake_sgemm_k_first.cpp:986-1104). */
void schedule_KMN_online(float* A, float* B, float* C, float** A_p, float* B_p, float** C_p, int M, int N, int K,
                         int p, cake_cntx_t* cake_cntx, blk_dims_t* x);
void schedule_KMN_C_unpacked(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p,
                             cake_cntx_t* cake_cntx, blk_dims_t* x);
void schedule_KMN_2d(float* A, float* B, float* C, float* A_p, float* B_p, float** C_p, int M, int N, int K, int p,
                     cake_cntx_t* cake_cntx, blk_dims_t* x);
void schedule_KMN_2d_small(float* A, float* B, float* C, float* A_p, float* B_p, float** C_p, int M, int N, int K,
                           int p, cake_cntx_t* cake_cntx, blk_dims_t* x);

/* Packing-free schedules for small matrices (reference include/cake.h:57-69,
 * src/cake_sgemm_small.cpp:7-236).  In the reference their microkernel call is commented out and
 * they compute nothing; here they do what that microkernel is written for
 * (src/kernels/haswell/dense.cpp:206-207): C += A*B with A stored by columns (A_p[k*M + m]), B and
 * C plain row-major.  The _A_packed / _B_packed / _C_packed forms take that one operand in the
 * layout of pack_A(NKM) / pack_B(MKN) / pack_C(KMN) and the other two plain row-major. */
void schedule_KMN_small(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                        blk_dims_t* x);
void schedule_MKN_small(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                        blk_dims_t* x);
void schedule_NKM_small(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                        blk_dims_t* x);
void schedule_NKM_small_A_packed(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p,
                                 cake_cntx_t* cake_cntx, blk_dims_t* x);
void schedule_MKN_small_B_packed(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p,
                                 cake_cntx_t* cake_cntx, blk_dims_t* x);
void schedule_KMN_small_C_packed(float* A_p, float* B_p, float* C_p, int M, int N, int K, int p,
                                 cake_cntx_t* cake_cntx, blk_dims_t* x);

/* Small-matrix path (reference include/cake.h:52-53, src/cake_sgemm.cpp:614-721).
 * Returns true and computes C = A*B with the exact-FP32 kernel, without any
 * operand pre-pass, when the product is too small to amortise one; returns
 * false (C untouched) otherwise. */
bool cake_gemm_small(float* A, float* B, float* C, int M, int N, int K, int p, blk_dims_t* x,
                     cake_cntx_t* cake_cntx, enum sched sch, char* argv[] = NULL);

/* Six-buffer form of the same (reference include/cake.h:71-72); the packed scratch is not used. */
bool cake_gemm_small(float* A, float* A_p, float* B, float* B_p, float* C, float* C_p, int M, int N, int K, int p,
                     blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch);

/* Batch of independent small products, item i at A + i*M*K, B + i*K*N,
 * C + i*M*N.  The reference has no batched entry; its equivalent is one
 * cake_sgemm per item. */
double cake_sgemm_small_batched(float* A, float* B, float* C, int M, int N, int K, int batch, int p,
                                cake_cntx_t* cake_cntx);

/* Sparse-A product (the reference ships only the microkernel,
 * src/kernels/haswell/sparse.cpp:7-131).  density_hint <= 0 = unknown. */
double cake_sp_sgemm(float* A, float* B, float* C, int M, int N, int K, int p, cake_cntx_t* cake_cntx,
                     float density_hint = -1.0f);

/* Matrix-vector product of the reference's driver (examples/cake_gemv.cpp:7-9, 716-765), same
 * signature: A is column-major (A[k*M + m]), B is the vector of length K, and C (length M) is
 * added to, as the reference's microkernel does with the C it is handed.  argv, packedA, alpha,
 * beta and sch are accepted and ignored, as there. */
double cake_sgemv(float* A, float* B, float* C, int M, int K, int p, cake_cntx_t* cake_cntx, char* argv[] = NULL,
                  bool packedA = 0, float alpha = 1, float beta = 0, enum sched sch = NA);

/* Convolution through im2col + SGEMM (reference examples/cake_conv.cpp:1007-1066).
 * in: [batch][Cin][H][W], filters: [Cout][Cin][Hf][Wf], out: [batch][Cout][Ho][Wo]. */
double cake_sconv_im2col(float* in, float* filters, float* out, int batch, int Cin, int H, int W, int Cout,
                         int Hf, int Wf, int stride, int pad, int p, cake_cntx_t* cake_cntx);
/* im_2_col of the reference (examples/cake_conv.cpp:1178-1213): single image,
 * no padding; returns a malloc'd K x N matrix the caller frees. */
float* im_2_col(float* In, int Wf, int Hf, int Win, int Hin, int Wout, int Hout, int Cin, int Cout, int s);

/* choose a schedule from the shape alone (reference src/cake_sgemm.cpp:768-787) */
enum sched set_schedule(enum sched sch, int M, int N, int K);

/* ------------------------------------------------------- context and tiling
 * reference: include/tiling.h:10-51, src/block_sizing.cpp. */
double clamp_val(double d, double min, double max);
cake_cntx_t* cake_query_cntx();                    /* malloc'd; caller frees with free() */
cake_cntx_t* cake_query_cntx_torch(int L2, int L3); /* same, with caller-given cache sizes */
void update_mr_nr(cake_cntx_t* cake_cntx, int m_r, int n_r);
int get_cache_size(int level);       /* 1: shared memory per SM, 2: L2, 3: device memory */
int get_num_physical_cores();        /* visible B200 devices */
int lcm(int n1, int n2);
enum sched derive_schedule(int M, int N, int K, int p, int mc_ret, cake_cntx_t* cake_cntx);
cache_dims_t* get_cache_dims(int M, int N, int K, int p, cake_cntx_t* cake_cntx, enum sched sch, char* argv[],
                             float type_size = 4, int mcu = 0, int kcu = 0, int ncu = 0);
void init_block_dims(int M, int N, int K, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch,
                     char* argv[], float type_size = 4, int mcu = 0, int kcu = 0, int ncu = 0);
void init_block_dims_2d(int M, int N, int K, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch,
                        char* argv[], float type_size = 4, int mcu = 0, int kcu = 0, int ncu = 0);
void init_block_dims_2d_small(int M, int N, int K, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch,
                              char* argv[], float type_size = 4);
int grid_dims_2d(int M, int N, int K, int p, int ncores);

/* ------------------------------------------------------------------ packing
 * reference: include/packing.h:6-72, src/pack_helper.cpp.  Buffers are
 * byte-identical to the reference's for the same block dimensions. */
size_t cake_sgemm_packed_A_size(int M, int K, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch);
size_t cake_sgemm_packed_B_size(int K, int N, int p, blk_dims_t* x, cake_cntx_t* cake_cntx);
size_t cake_sgemm_packed_C_size(int M, int N, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch);
double pack_A(float* A, float* A_p, int M, int K, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch);
void pack_B(float* B, float* B_p, int K, int N, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch);
void pack_C(float* C, float* C_p, int M, int N, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch);
void unpack_C(float* C, float* C_p, int M, int N, int p, blk_dims_t* x, cake_cntx_t* cake_cntx, enum sched sch);

/* -------------------------------------------------------------------- util
 * reference: include/util.h:6-26, src/util.cpp. */
int run_tests();
bool cake_sgemm_checker(float* A, float* B, float* C, int N, int M, int K); /* note the N, M, K order */
bool mat_equals(float* C, float* C_check, int M, int N);
void rand_init(float* mat, int r, int c);
float rand_gen();
float normalRandom();
void print_array(float* arr, int len);
void print_mat(float* arr, int r, int c);
void print_schedule(enum sched sch);
