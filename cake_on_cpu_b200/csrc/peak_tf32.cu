// Issue-rate measurement of tcgen05.mma kind::tf32: what the tensor pipe of this GPU
// delivers when nothing but the instruction stream limits it.  One CTA per SM, operand
// tiles resident in shared memory (no loads inside the timed loop), one thread issuing
// 128 x 256 x 8 MMAs back to back into a tensor-memory accumulator, exactly the
// instruction the large-matrix kernel issues.  The 3xTF32 product needs three such
// MMAs per FP32-class multiply-add, so its roofline is this rate divided by three.
//
// The reference sizes its blocks from a hard-coded machine peak (peak_flops = 600e9,
// src/block_sizing.cpp:49-50); here the figure is measured on the device it runs on.
#include <algorithm>

#include "common.cuh"
#include "tcgen05.cuh"

namespace cakeb200 {
namespace {

using namespace ptx;

constexpr int PK_BM = 128, PK_BN = 256, PK_BK = 32;
constexpr int PK_SMEM = (PK_BM + PK_BN) * PK_BK * 4 + 1024 + 64;

__global__ void __launch_bounds__(128, 1) tf32_peak_kernel(int iters, int* status_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint64_t* bar = (uint64_t*) (tiles + (PK_BM + PK_BN) * PK_BK * 4);
    uint32_t* tmem_slot = (uint32_t*) (bar + 1);
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    // operand values: small non-zero numbers, so the multipliers toggle as in a real product
    float* f = (float*) tiles;
    for (int i = threadIdx.x; i < (PK_BM + PK_BN) * PK_BK; i += blockDim.x) {
        float hi, lo;
        split_tf32(0.25f + 0.001f * (float) ((i * 37 + (int) blockIdx.x) & 255), hi, lo);
        f[i] = hi;
    }
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = make_idesc_tf32(PK_BM, PK_BN);
        const uint64_t a = make_kmajor_sw128_desc(smem_u32(tiles));
        const uint64_t b = make_kmajor_sw128_desc(smem_u32(tiles) + PK_BM * PK_BK * 4);
        for (int it = 0; it < iters; it++) {
            // two accumulators in turn, four k-steps of 8 each: the issue pattern of one pipeline stage
            const uint32_t d = tmem_base + (uint32_t) ((it & 1) * PK_BN);
#pragma unroll
            for (int k = 0; k < PK_BK / 8; k++) umma_tf32(d, a + (uint64_t) (k * 2), b + (uint64_t) (k * 2), idesc, (it > 1 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(bar));
        mbar_wait(smem_u32(bar), 0, &abort_flag, status_word, 950);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace

// TFLOP/s of dense TF32 MMAs over `ms_target` milliseconds (roughly) of back-to-back issue on every SM.
int measure_tf32_peak(int* status_word, int sm_count, float ms_target, cudaStream_t stream, float* tflops, float* ms_out) {
    CAKE_CUDA_OK(cudaFuncSetAttribute(tf32_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM));
    cudaEvent_t e0, e1;
    CAKE_CUDA_OK(cudaEventCreate(&e0));
    CAKE_CUDA_OK(cudaEventCreate(&e1));
    const double flop_per_iter = 2.0 * PK_BM * PK_BN * PK_BK;
    int iters = 2000;
    float ms = 0.f;
    for (int round = 0; round < 3; round++) {  // first round warms up and sizes the second
        CAKE_CUDA_OK(cudaEventRecord(e0, stream));
        tf32_peak_kernel<<<sm_count, 128, PK_SMEM, stream>>>(iters, status_word);
        CAKE_CUDA_OK(cudaGetLastError());
        CAKE_CUDA_OK(cudaEventRecord(e1, stream));
        CAKE_CUDA_OK(cudaEventSynchronize(e1));
        CAKE_CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
        if (round == 0 && ms > 0.f) iters = (int) std::min(4.0e6, std::max(1000.0, iters * (double) ms_target / ms));
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (tflops) *tflops = (float) (flop_per_iter * iters * sm_count / (ms * 1e-3) / 1e12);
    if (ms_out) *ms_out = ms;
    return CAKEB200_OK;
}

}  // namespace cakeb200
