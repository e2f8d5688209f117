// Second half of a product whose K dimension is sharded over the GPUs of one box.
//
// The reference splits a block of C's rows over cores and lets every core add its share of K
// into a private buffer before the buffers are combined (the K-first schedule,
// src/cake_sgemm_k_first.cpp:85-129).  Across GPUs the same idea applies to shapes whose
// M and N are too small to give every GPU a block of rows or columns: each rank multiplies
// its range of K, and while it sums its tiles it stores the rows of the result straight
// into the memory of the rank that owns them (reduce_pieces_to_owners_kernel in
// sgemm_tf32x3.cu), one slot per source rank.  The kernel below runs on the owner: it
// waits until every source rank has flagged its slot complete and adds the slots in rank
// order, so the result does not depend on arrival order.
//
// The wait is bounded.  A rank that never arrives (it failed, or it is simply seconds
// behind) makes the kernel record the missing rank in the device status word and return;
// the host reports CAKEB200_ERR_DEVICE_TIMEOUT and the context stays usable.
#include <algorithm>

#include "common.cuh"

namespace cakeb200 {
namespace {

__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

constexpr int WHERE_OWNER_WAIT = 910;  // status_word[1] of a wait that gave up here; status_word[2] = the missing rank

__global__ void __launch_bounds__(256)
sum_owner_slots_kernel(const float* __restrict__ slots, long long slot_floats, int world, float* __restrict__ out,
                       long long count, const int* flags, int epoch, long long limit_ns, int* status_word) {
    __shared__ int arrived;
    if (threadIdx.x == 0) {
        arrived = 1;
        const unsigned long long t0 = timer_ns();
        for (int r = 0; r < world && arrived; r++) {
            const volatile int* f = flags + r;
            // epochs only grow; the difference form survives a wrap of the counter
            while ((int) (*f - epoch) < 0) {
                if ((long long) (timer_ns() - t0) > limit_ns) {
                    arrived = 0;
                    if (atomicCAS(status_word, 0, 1) == 0) {
                        status_word[1] = WHERE_OWNER_WAIT;
                        status_word[2] = r;
                    }
                    break;
                }
                __nanosleep(200);
            }
        }
        __threadfence_system();  // the slots are read after the flags
    }
    __syncthreads();
    if (!arrived) return;
    const long long stride = (long long) gridDim.x * blockDim.x, first = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    const bool vec = (count % 4 == 0) && (slot_floats % 4 == 0) && ((((uintptr_t) slots | (uintptr_t) out) & 15) == 0);
    if (vec) {
        for (long long i = first; i < count / 4; i += stride) {
            float4 s = __ldcv(reinterpret_cast<const float4*>(slots) + i);
            for (int r = 1; r < world; r++) {
                const float4 v = __ldcv(reinterpret_cast<const float4*>(slots + (long long) r * slot_floats) + i);
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            reinterpret_cast<float4*>(out)[i] = s;
        }
    } else {
        for (long long i = first; i < count; i += stride) {
            float s = __ldcv(slots + i);
            for (int r = 1; r < world; r++) s += __ldcv(slots + (long long) r * slot_floats + i);
            out[i] = s;
        }
    }
}

}  // namespace

int launch_sum_owner_slots(const float* slots, long long slot_floats, int world, float* out, long long count,
                           const int* flags, int epoch, long long limit_ns, int* status_word, int sm_count,
                           cudaStream_t stream) {
    if (count <= 0) return CAKEB200_OK;
    const long long work = (count + 3) / 4;
    const int blocks = (int) std::max<long long>(1, std::min<long long>((work + 255) / 256, (long long) sm_count * 4));
    sum_owner_slots_kernel<<<blocks, 256, 0, stream>>>(slots, slot_floats, world, out, count, flags, epoch, limit_ns, status_word);
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}

}  // namespace cakeb200
