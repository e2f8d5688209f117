// Drives the C++ API of include/cake.h the way a caller of the reference
// library would (compare the reference's examples/cake_sgemm_test.cpp:5-90 and
// the packed-operand calls in examples/cake_conv.cpp:1028-1056).
// Exit code 0 = every check printed CORRECT.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "cake.h"

static int failures = 0;
static void expect(bool ok, const char* what) {
    if (!ok) {
        printf("FAILED: %s\n", what);
        failures++;
    }
}

int main(int argc, char* argv[]) {
    int M = 777, K = 515, N = 1030, p = 4;
    if (argc > 3) { M = atoi(argv[1]); K = atoi(argv[2]); N = atoi(argv[3]); }
    std::vector<float> A((size_t) M * K), B((size_t) K * N), C((size_t) M * N);
    srand(1);
    rand_init(A.data(), M, K);
    rand_init(B.data(), K, N);

    cake_cntx_t* cntx = cake_query_cntx();
    printf("context: mr=%d nr=%d L1=%d L2=%d L3=%d ncores=%d\n", cntx->mr, cntx->nr, cntx->L1, cntx->L2, cntx->L3, cntx->ncores);
    expect(cntx->ncores >= 1 && cntx->L2 > 0, "cake_query_cntx");

    const enum sched all[] = {KMN, MKN, NKM, NA};
    for (enum sched s : all) {
        std::fill(C.begin(), C.end(), -7.f);
        double t = cake_sgemm(A.data(), B.data(), C.data(), M, N, K, p, cntx, NULL, 0, 0, 1, 0, s);
        expect(t > 0, "cake_sgemm returned a time");
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "cake_sgemm result");
    }
    // NULL context = query internally
    expect(cake_sgemm(A.data(), B.data(), C.data(), M, N, K, p, NULL) > 0, "cake_sgemm with NULL context");
    expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "NULL-context result");

    // pre-packed operands, K-first (examples/cake_conv.cpp:1028-1056)
    {
        blk_dims_t x;
        init_block_dims(M, N, K, p, &x, cntx, KMN, NULL);
        std::vector<float> A_p(cake_sgemm_packed_A_size(M, K, p, &x, cntx, KMN) / 4);
        std::vector<float> B_p(cake_sgemm_packed_B_size(K, N, p, &x, cntx) / 4);
        expect(pack_A(A.data(), A_p.data(), M, K, p, &x, cntx, KMN) >= 0, "pack_A");
        pack_B(B.data(), B_p.data(), K, N, p, &x, cntx, KMN);
        std::fill(C.begin(), C.end(), -7.f);
        expect(cake_sgemm(A_p.data(), B_p.data(), C.data(), M, N, K, p, cntx, NULL, 1, 1, 1, 0, KMN) > 0, "packed cake_sgemm");
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "packed operands result");
        std::fill(C.begin(), C.end(), -7.f);
        schedule_KMN(A_p.data(), B_p.data(), C.data(), NULL, M, N, K, p, cntx, &x);
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "schedule_KMN result");
        // a packed buffer moved to another address is not one the library kept planes for: it is unpacked instead
        std::vector<float> A_moved(A_p), B_moved(B_p);
        std::fill(C.begin(), C.end(), -7.f);
        expect(cake_sgemm(A_moved.data(), B_moved.data(), C.data(), M, N, K, p, cntx, NULL, 1, 1, 1, 0, KMN) > 0, "packed cake_sgemm, moved buffers");
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "moved packed operands result");
        // the same address refilled with another operand's packed image (without pack_A): the kept planes must not be used
        std::vector<float> A2((size_t) M * K), A2_p(A_p.size());
        rand_init(A2.data(), M, K);
        pack_A(A2.data(), A2_p.data(), M, K, p, &x, cntx, KMN);
        memcpy(A_p.data(), A2_p.data(), A_p.size() * sizeof(float));
        std::fill(C.begin(), C.end(), -7.f);
        expect(cake_sgemm(A_p.data(), B_p.data(), C.data(), M, N, K, p, cntx, NULL, 1, 1, 1, 0, KMN) > 0, "packed cake_sgemm, refilled buffer");
        expect(cake_sgemm_checker(A2.data(), B.data(), C.data(), N, M, K) == 0, "refilled packed operand result");
        // one operand packed, the other plain
        std::fill(C.begin(), C.end(), -7.f);
        expect(cake_sgemm(A.data(), B_p.data(), C.data(), M, N, K, p, cntx, NULL, 0, 1, 1, 0, KMN) > 0, "cake_sgemm, packed B only");
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "packed B only result");
    }
    // M-first on packed operands accumulates into packed C; unpack_C brings it back
    {
        blk_dims_t x;
        init_block_dims(M, N, K, p, &x, cntx, MKN, NULL);
        std::vector<float> A_p(cake_sgemm_packed_A_size(M, K, p, &x, cntx, MKN) / 4);
        std::vector<float> B_p(cake_sgemm_packed_B_size(K, N, p, &x, cntx) / 4);
        std::vector<float> C_p(cake_sgemm_packed_C_size(M, N, p, &x, cntx, MKN) / 4, 0.f);
        pack_A(A.data(), A_p.data(), M, K, p, &x, cntx, MKN);
        pack_B(B.data(), B_p.data(), K, N, p, &x, cntx, MKN);
        schedule(A_p.data(), B_p.data(), C_p.data(), M, N, K, p, cntx, &x, MKN, 0, 0);
        std::fill(C.begin(), C.end(), -7.f);
        unpack_C(C.data(), C_p.data(), M, N, p, &x, cntx, MKN);
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "schedule(MKN) + unpack_C result");
    }
    // beta != 0 with M-first adds to C (the reference's flag semantics)
    {
        std::vector<float> C1((size_t) M * N), C2((size_t) M * N, 1.5f);
        cake_sgemm(A.data(), B.data(), C1.data(), M, N, K, p, cntx, NULL, 0, 0, 1, 0, MKN);
        cake_sgemm(A.data(), B.data(), C2.data(), M, N, K, p, cntx, NULL, 0, 0, 1, 1, MKN);
        double worst = 0;
        for (size_t i = 0; i < C1.size(); i++) worst = std::max(worst, (double) fabsf(C2[i] - C1[i] - 1.5f));
        expect(worst < 1e-3, "beta flag adds to C");
    }
    // the other K-first drivers and their schedule entry points (reference include/cake.h:26-47): plain operands
    {
        std::fill(C.begin(), C.end(), -7.f);
        expect(cake_sgemm_online(A.data(), B.data(), C.data(), M, N, K, p, cntx) > 0, "cake_sgemm_online");
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "cake_sgemm_online result");
        std::fill(C.begin(), C.end(), -7.f);
        expect(cake_sgemm_2d(A.data(), B.data(), C.data(), M, N, K, p, cntx) > 0, "cake_sgemm_2d");
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "cake_sgemm_2d result");
        std::fill(C.begin(), C.end(), -7.f);
        expect(cake_sgemm_2d_small(A.data(), B.data(), C.data(), M, N, K, p, cntx) > 0, "cake_sgemm_2d_small");
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "cake_sgemm_2d_small result");
        blk_dims_t x;
        init_block_dims_2d(M, N, K, p, &x, cntx, KMN, NULL);
        expect(x.pm * x.pn == p, "init_block_dims_2d grid");
        std::fill(C.begin(), C.end(), -7.f);
        schedule_KMN_online(A.data(), B.data(), C.data(), NULL, NULL, NULL, M, N, K, p, cntx, &x);
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "schedule_KMN_online result");
        std::fill(C.begin(), C.end(), -7.f);
        schedule_KMN_2d(A.data(), B.data(), C.data(), NULL, NULL, NULL, M, N, K, p, cntx, &x);
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "schedule_KMN_2d result");
        blk_dims_t xs;
        init_block_dims_2d_small(M, N, K, p, &xs, cntx, KMN, NULL);
        expect(xs.pm * xs.pn == p && xs.m_c >= M / xs.pm && xs.n_c >= N / xs.pn && xs.k_c > 0, "init_block_dims_2d_small");
        std::fill(C.begin(), C.end(), -7.f);
        schedule_KMN_2d_small(A.data(), B.data(), C.data(), NULL, NULL, NULL, M, N, K, p, cntx, &xs);
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "schedule_KMN_2d_small result");
    }
    // K-first on packed A and B adding into a plain C with the padded row pitch
    {
        blk_dims_t x;
        init_block_dims(M, N, K, p, &x, cntx, KMN, NULL);
        std::vector<float> A_p(cake_sgemm_packed_A_size(M, K, p, &x, cntx, KMN) / 4);
        std::vector<float> B_p(cake_sgemm_packed_B_size(K, N, p, &x, cntx) / 4);
        pack_A(A.data(), A_p.data(), M, K, p, &x, cntx, KMN);
        pack_B(B.data(), B_p.data(), K, N, p, &x, cntx, KMN);
        std::vector<float> C_wide((size_t) x.M_padded * x.N_padded, 0.f);
        schedule_KMN_C_unpacked(A_p.data(), B_p.data(), C_wide.data(), M, N, K, p, cntx, &x);
        for (int m = 0; m < M; m++) memcpy(&C[(size_t) m * N], &C_wide[(size_t) m * x.N_padded], (size_t) N * sizeof(float));
        expect(cake_sgemm_checker(A.data(), B.data(), C.data(), N, M, K) == 0, "schedule_KMN_C_unpacked result");
    }
    // packing-free small schedules: A stored by columns, C added to; and the forms with one packed operand
    {
        const int m = 111, k = 96, n = 211;
        std::vector<float> a((size_t) m * k), at((size_t) k * m), b((size_t) k * n), c((size_t) m * n);
        rand_init(a.data(), m, k);
        rand_init(b.data(), k, n);
        for (int i = 0; i < m; i++)
            for (int j = 0; j < k; j++) at[(size_t) j * m + i] = a[(size_t) i * k + j];
        blk_dims_t x;
        typedef void (*small_fn)(float*, float*, float*, int, int, int, int, cake_cntx_t*, blk_dims_t*);
        const small_fn plain[] = {schedule_KMN_small, schedule_MKN_small, schedule_NKM_small};
        const enum sched order[] = {KMN, MKN, NKM};
        for (int i = 0; i < 3; i++) {
            init_block_dims(m, n, k, p, &x, cntx, order[i], NULL);
            std::fill(c.begin(), c.end(), 0.f);
            plain[i](at.data(), b.data(), c.data(), m, n, k, p, cntx, &x);
            expect(cake_sgemm_checker(a.data(), b.data(), c.data(), n, m, k) == 0, "schedule_*_small result");
        }
        init_block_dims(m, n, k, p, &x, cntx, NKM, NULL);
        std::vector<float> a_p(cake_sgemm_packed_A_size(m, k, p, &x, cntx, NKM) / 4);
        pack_A(a.data(), a_p.data(), m, k, p, &x, cntx, NKM);
        std::fill(c.begin(), c.end(), 0.f);
        schedule_NKM_small_A_packed(a_p.data(), b.data(), c.data(), m, n, k, p, cntx, &x);
        expect(cake_sgemm_checker(a.data(), b.data(), c.data(), n, m, k) == 0, "schedule_NKM_small_A_packed result");
        init_block_dims(m, n, k, p, &x, cntx, MKN, NULL);
        std::vector<float> b_p(cake_sgemm_packed_B_size(k, n, p, &x, cntx) / 4);
        pack_B(b.data(), b_p.data(), k, n, p, &x, cntx, MKN);
        std::fill(c.begin(), c.end(), 0.f);
        schedule_MKN_small_B_packed(a.data(), b_p.data(), c.data(), m, n, k, p, cntx, &x);
        expect(cake_sgemm_checker(a.data(), b.data(), c.data(), n, m, k) == 0, "schedule_MKN_small_B_packed result");
        init_block_dims(m, n, k, p, &x, cntx, KMN, NULL);
        std::vector<float> c_p(cake_sgemm_packed_C_size(m, n, p, &x, cntx, KMN) / 4, 0.f);
        schedule_KMN_small_C_packed(a.data(), b.data(), c_p.data(), m, n, k, p, cntx, &x);
        std::fill(c.begin(), c.end(), -7.f);
        unpack_C(c.data(), c_p.data(), m, n, p, &x, cntx, KMN);
        expect(cake_sgemm_checker(a.data(), b.data(), c.data(), n, m, k) == 0, "schedule_KMN_small_C_packed result");
        // six-buffer form of the small-matrix entry point
        std::fill(c.begin(), c.end(), -7.f);
        expect(cake_gemm_small(a.data(), NULL, b.data(), NULL, c.data(), NULL, m, n, k, p, &x, cntx, NA), "cake_gemm_small (six buffers)");
        expect(cake_sgemm_checker(a.data(), b.data(), c.data(), n, m, k) == 0, "cake_gemm_small (six buffers) result");
    }
    // small-matrix entry point
    {
        const int m = 96;
        std::vector<float> a(m * m), b(m * m), c(m * m);
        rand_init(a.data(), m, m);
        rand_init(b.data(), m, m);
        blk_dims_t x;
        expect(cake_gemm_small(a.data(), b.data(), c.data(), m, m, m, p, &x, cntx, NA), "cake_gemm_small took the product");
        expect(cake_sgemm_checker(a.data(), b.data(), c.data(), m, m, m) == 0, "cake_gemm_small result");
    }
    // matrix-vector driver of the reference's example (examples/cake_gemv.cpp:771-813): column-major A, C added to
    {
        const int m = 1000, k = 700;
        std::vector<float> a((size_t) m * k), x(k), y(m, 0.25f), want(m, 0.25f);
        rand_init(a.data(), m, k);
        rand_init(x.data(), k, 1);
        expect(cake_sgemv(a.data(), x.data(), y.data(), m, k, p, cntx) > 0, "cake_sgemv returned a time");
        for (int kk = 0; kk < k; kk++)
            for (int mm = 0; mm < m; mm++) want[mm] += a[(size_t) kk * m + mm] * x[kk];
        double worst = 0;
        for (int mm = 0; mm < m; mm++) worst = std::max(worst, (double) fabsf(want[mm] - y[mm]));
        expect(worst < 1e-3, "cake_sgemv result");
    }
    // a batch of small products (tensor-core kernel for a batch this large)
    {
        const int m = 96, batch = 200;
        std::vector<float> a((size_t) batch * m * m), b((size_t) batch * m * m), c((size_t) batch * m * m, -7.f);
        rand_init(a.data(), batch * m, m);
        rand_init(b.data(), batch * m, m);
        expect(cake_sgemm_small_batched(a.data(), b.data(), c.data(), m, m, m, batch, p, cntx) > 0, "cake_sgemm_small_batched");
        for (int i : {0, 77, 199})
            expect(cake_sgemm_checker(a.data() + (size_t) i * m * m, b.data() + (size_t) i * m * m, c.data() + (size_t) i * m * m,
                                      m, m, m) == 0, "batched item result");
    }
    expect(set_schedule(NA, 4000, 100, 100) == MKN && set_schedule(NA, 100, 100, 4000) == KMN &&
           set_schedule(NA, 100, 4000, 100) == NKM, "set_schedule");
    free(cntx);
    printf(failures ? "%d FAILURES\n" : "ALL CORRECT\n", failures);
    return failures ? 1 : 0;
}
