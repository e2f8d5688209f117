/* TEST INFRASTRUCTURE ONLY: drives the reference's sparse microkernel
 * cake_sp_sgemm_haswell_6x16 (reference src/kernels/haswell/sparse.cpp:7-126), tile by tile,
 * so that the oracle's restatement of the row-skipping product can be pinned against it.
 *
 * The reference ships this microkernel without any packer or schedule (the dispatcher's
 * sparse arms are comments, src/cake_sgemm.cpp:731-753), and the rest of its file does not
 * compile (the 3x32 kernel uses undeclared variables).  oracle/Makefile therefore cuts the
 * file at the end of its first function, into oracle/_ref/, and compiles that next to this
 * driver; nothing of it is kept in the repository.
 *
 * What the driver supplies is only the operand layout the kernel reads, taken from its body:
 *   A         the nonzeros of an m_r x k tile, column after column, rows ascending;
 *   nnz_outer[j], k_inds[j]   count and source row of B for the j-th stored column; columns
 *             without nonzeros come last (the kernel stops at the first empty one it meets
 *             at a multiple of four);
 *   loc_m     the row (0..5) of every stored nonzero;
 *   B         a panel of k rows x 16 floats, row r at B + 16 * r, 32-byte aligned;
 *   C         the 6 x 16 tile, row-major contiguous, loaded, added to and stored.
 * No arithmetic happens here. */
#include <cstdlib>
#include <cstring>
#include <vector>

void cake_sp_sgemm_haswell_6x16(float* A, float* B, float* C, int m, int n, int k, int* nnz_outer, int* k_inds, int* loc_m);

extern "C" int ref_sp_sgemm(const float* A, const float* B, float* C, int M, int N, int K) {
    const int MR = 6, NR = 16;
    float* panel = nullptr;
    if (posix_memalign((void**) &panel, 64, (size_t) (K > 0 ? K : 1) * NR * sizeof(float))) return -1;
    std::vector<float> vals((size_t) MR * K + 1);
    std::vector<int> nnz_outer(K + 4), k_inds(K + 4), loc_m((size_t) MR * K + 1);
    alignas(64) float tile[MR * NR];
    for (int n0 = 0; n0 < N; n0 += NR) {
        const int cols = (N - n0 < NR) ? N - n0 : NR;
        for (int k = 0; k < K; k++) {  // B panel: k rows of 16, columns beyond N zero
            memset(panel + (size_t) k * NR, 0, NR * sizeof(float));
            memcpy(panel + (size_t) k * NR, B + (size_t) k * N + n0, cols * sizeof(float));
        }
        for (int m0 = 0; m0 < M; m0 += MR) {
            const int rows = (M - m0 < MR) ? M - m0 : MR;
            int stored = 0, nz = 0;
            for (int k = 0; k < K; k++) {  // stored columns in ascending k, empty ones left out (they would come last)
                int cnt = 0;
                for (int r = 0; r < rows; r++) {
                    const float a = A[(size_t) (m0 + r) * K + k];
                    if (a != 0.0f) {
                        vals[nz] = a;
                        loc_m[nz] = r;
                        nz++;
                        cnt++;
                    }
                }
                if (cnt) {
                    nnz_outer[stored] = cnt;
                    k_inds[stored] = k;
                    stored++;
                }
            }
            for (int j = stored; j < K + 4; j++) { nnz_outer[j] = 0; k_inds[j] = 0; }
            memset(tile, 0, sizeof(tile));
            cake_sp_sgemm_haswell_6x16(vals.data(), panel, tile, MR, NR, K, nnz_outer.data(), k_inds.data(), loc_m.data());
            for (int r = 0; r < rows; r++) memcpy(C + (size_t) (m0 + r) * N + n0, tile + r * NR, cols * sizeof(float));
        }
    }
    free(panel);
    return 0;
}
