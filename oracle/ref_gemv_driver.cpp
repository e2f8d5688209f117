/* TEST INFRASTRUCTURE ONLY: drives the reference's matrix-vector microkernel
 * cake_sgemv_haswell_8x8_col (reference examples/cake_gemv.cpp:87-140), eight rows at a time, so
 * that the oracle's restatement of the matrix-vector product can be pinned against it.
 *
 * The microkernel lives in a stand-alone example program (its file has a main and its own copies
 * of the library's helpers), so oracle/Makefile cuts that one function out of the example into
 * oracle/_ref/ and compiles it next to this driver; nothing of it is kept in the repository.
 * The example's schedule (schedule_mvm, :424-489) calls the kernel per block of rows and, inside,
 * per block of k in ascending order, with C loaded and stored in between; per element that is the
 * one chain over all of k that a single call with k = K performs.  No arithmetic happens here:
 * the driver only pads M to a multiple of eight (the kernel always loads eight rows). */
#include <cstdlib>
#include <cstring>
#include <vector>

void cake_sgemv_haswell_8x8_col(float* A, float* B, float* C, int m, int k, int M);

/* y (length M) += A x, A column-major: A[k * M + m] */
extern "C" int ref_sgemv(const float* A, const float* x, float* y, int M, int K) {
    const int Mp = (M + 7) / 8 * 8;
    std::vector<float> a((size_t) Mp * K, 0.0f), c(Mp, 0.0f), b(x, x + K);
    for (int k = 0; k < K; k++) memcpy(&a[(size_t) k * Mp], A + (size_t) k * M, (size_t) M * sizeof(float));
    memcpy(c.data(), y, (size_t) M * sizeof(float));
    for (int m0 = 0; m0 < Mp; m0 += 8) cake_sgemv_haswell_8x8_col(a.data() + m0, b.data(), c.data() + m0, 8, K, Mp);
    memcpy(y, c.data(), (size_t) M * sizeof(float));
    return 0;
}
