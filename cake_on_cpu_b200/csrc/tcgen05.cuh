// Inline-PTX wrappers shared by the tcgen05 kernels: mbarriers with bounded waits,
// TMA tile loads, tcgen05.mma / commit / ld, shared-memory matrix descriptors and the
// TF32 hi/lo split.  sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cakeb200 {

// Host: tiled FP32 tensor map of `rank` dimensions (innermost first; strides of dimensions 1.. in bytes),
// out-of-range elements read as zero.  Implemented next to the driver entry-point lookup in sgemm_tf32x3.cu.
int encode_tiled_f32(CUtensorMap* map, const float* base, int rank, const unsigned long long* dims,
                     const unsigned long long* strides_bytes, const unsigned* box, bool swizzle128);

namespace ptx {

constexpr long long WAIT_LIMIT_NS = 2000000000LL;  // 2 s per wait, far above any legitimate stall

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when the
// barrier did not flip within WAIT_LIMIT_NS or another role already gave up.
// `backoff_ns` > 0: once the quick polls have failed the thread sleeps that long between polls (for waits
// that are expected to take many microseconds: a polling warp takes issue slots and power from the warps
// that feed the tensor cores).
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word,
                                              int where, long long limit_ns, unsigned backoff_ns = 0) {
    // short waits are the common case: poll a while before touching the (slow) global timer
#pragma unroll 1
    for (int i = 0; i < 64; i++)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (backoff_ns) __nanosleep(backoff_ns);
        if ((++spins & (backoff_ns ? 63 : 1023)) == 0) {
            if (*abort_flag) return false;
            if ((long long) (global_ns() - t0) > limit_ns) {
                *abort_flag = 1;
                if (atomicCAS(status_word, 0, 1) == 0) {
                    status_word[1] = where;
                    status_word[2] = (int) blockIdx.x;
                }
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_word, int where) {
    return mbar_wait_for(bar, parity, abort_flag, status_word, where, WAIT_LIMIT_NS);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same product with the A operand in tensor memory (lane = row, one 32-bit column per TF32 element).
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- two CTAs of a cluster working as one (cta_group::2).  The pair is (even rank, even rank + 1); the
// even one ("leader") issues the MMAs, which read A rows and B rows from both CTAs' shared memory at the
// same offsets and write 128 accumulator rows into each CTA's tensor memory.

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of both CTAs.
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Shared-memory addresses of the two CTAs of a pair differ in this bit; clearing it names the same
// offset in the leader.
constexpr uint32_t PAIR_LEADER_MASK = 0xFEFFFFFFu;

// Tile load by either CTA of the pair into its own shared memory; the bytes are counted on the
// LEADER's mbarrier at the offset of `bar`.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar & PAIR_LEADER_MASK)
        : "memory");
}
// D (256 x N, 128 rows in each CTA's tensor memory) (+)= A (128 rows per CTA) x B (N / 2 rows per CTA).
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier at this offset in BOTH CTAs once every pair MMA issued so far has finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t) 3)
                 : "memory");
}
// Arrive on the leader's mbarrier at the offset of `bar` (from either CTA).
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PAIR_LEADER_MASK) : "memory");
}

// One source for the single-CTA and the pair form of a kernel: PAIR selects the instruction variants.
template <bool PAIR>
__device__ __forceinline__ void tma_load_2d_t(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    if constexpr (PAIR) tma_load_2d_pair(dst, map, x, y, bar);
    else tma_load_2d(dst, map, x, y, bar);
}
template <bool PAIR>
__device__ __forceinline__ void umma_tf32_t(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if constexpr (PAIR) umma_tf32_pair(tmem_d, desc_a, desc_b, idesc, accumulate);
    else umma_tf32(tmem_d, desc_a, desc_b, idesc, accumulate);
}
template <bool PAIR>
__device__ __forceinline__ void umma_commit_t(uint32_t bar) {
    if constexpr (PAIR) umma_commit_pair(bar);
    else umma_commit(bar);
}
// Arrive on the barrier the MMA issuer waits on: this CTA's, or the leader's in a pair.
template <bool PAIR>
__device__ __forceinline__ void mbar_arrive_t(uint32_t bar) {
    if constexpr (PAIR) mbar_arrive_leader(bar);
    else mbar_arrive(bar);
}
// Tensor-memory allocation by one whole warp (the same warp of both CTAs in a pair, same `slot` offset).
template <bool PAIR>
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
    if constexpr (PAIR) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
}
template <bool PAIR>
__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t cols) {
    if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
// Every thread of the CTA, or of both CTAs of the pair.
template <bool PAIR>
__device__ __forceinline__ void sync_all_t() {
    if constexpr (PAIR) cluster_sync_all();
    else __syncthreads();
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// 64 consecutive columns of the thread's lane in one instruction.
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}
// Each thread writes 16 consecutive columns of its own lane (the warp covers lanes [32 * (warp % 4), +32)).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
    float o;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(o) : "r"(addr) : "memory");
    return o;
}
__device__ __forceinline__ float4 ld_shared_v4(uint32_t addr) {
    float4 o;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(o.x), "=f"(o.y), "=f"(o.z), "=f"(o.w) : "r"(addr) : "memory");
    return o;
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes
// and 128-byte swizzled: 8-row groups are 1024 bytes apart (stride byte offset),
// the leading byte offset is unused for swizzled K-major layouts (encoded 1),
// descriptor version 1 (sm_100), layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((smem_addr & 0x3FFFF) >> 4);   // start address, 16-byte units
    d |= (uint64_t) 1 << 16;                        // leading byte offset (ignored)
    d |= (uint64_t) (1024 >> 4) << 32;              // stride byte offset
    d |= (uint64_t) 1 << 46;                        // descriptor version
    d |= (uint64_t) 2 << 61;                        // SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::tf32: D = F32, A = B = TF32, both K-major,
// N in units of 8 at bit 17, M in units of 16 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (m >> 4) << 24);
}


// v = hi + lo with hi = tf32(v) (round to nearest on the 13 dropped mantissa bits) and
// lo = tf32(v - hi) (the exact remainder, rounded again).
__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) {
    const uint32_t b = __float_as_uint(v);
    hi = __uint_as_float((b + 0x1000u) & 0xFFFFE000u);
    const float r = v - hi;
    lo = __uint_as_float((__float_as_uint(r) + 0x1000u) & 0xFFFFE000u);
}

// Hardware barrier `id` (1..15; 0 is __syncthreads) among `threads` threads of the CTA (a multiple of 32).
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Makes this thread's earlier shared-memory writes visible to the asynchronous proxy
// (tcgen05.mma and TMA read shared memory through it).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace ptx
}  // namespace cakeb200
