// The C ABI (include/cake_b200.h): argument checking, host/device pointer
// handling, kernel selection and timing.  No arithmetic happens here and there
// is no CPU fallback: every product is computed by a kernel of this library.
#include <algorithm>
#include <atomic>
#include <climits>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <mutex>

#include "common.cuh"

namespace cakeb200 {

int pack_A_dev(const float*, float*, int, int, int, const cakeb200_blk_dims*, const cakeb200_cntx*, bool, cudaStream_t);
int pack_B_dev(const float*, float*, int, int, int, const cakeb200_blk_dims*, const cakeb200_cntx*, bool, cudaStream_t);
int pack_C_dev(const float*, float*, int, int, int, const cakeb200_blk_dims*, const cakeb200_cntx*, bool, cudaStream_t);
int last_pack_width();
size_t sparse_scratch_bytes(int M, int K);
int sp_compact(const float* A, int M, int K, void* scratch, int* status_word, cudaStream_t stream, long long* nnz,
               int* launches);
int sp_multiply(const float* B, float* C, int M, int N, int K, void* scratch, long long nnz, int* status_word,
                cudaStream_t stream, int* launches);
int launch_im2col(const float*, float*, int, int, int, int, int, int, int, int, cudaStream_t);

namespace {
thread_local char g_error[512] = "";
thread_local cakeb200_stats g_stats = {};
std::mutex g_state_mutex;
constexpr int MAX_DEVICES = 64;
DeviceState* g_states[MAX_DEVICES] = {};
}  // namespace

namespace {
std::atomic<int> g_options[OPT_COUNT];
const char* const g_option_names[OPT_COUNT] = {"tile_n", "band", "k_pieces", "chunk_kb", "conv_route", "small_operands", "pack_scalar", "pair"};
}  // namespace
int option_get(int id) { return (id >= 0 && id < OPT_COUNT) ? g_options[id].load() : 0; }

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

DeviceState* device_state() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        cudaGetLastError();
        set_error("no CUDA device is current");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_state_mutex);
    if (g_states[dev]) return g_states[dev];
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaGetDeviceProperties failed");
        return nullptr;
    }
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major, prop.minor);
        return nullptr;
    }
    DeviceState* st = new DeviceState();
    st->device = dev;
    st->sm_count = prop.multiProcessorCount;
    bool ok = cudaStreamCreateWithFlags(&st->stream, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < 6 && ok; i++) ok = cudaEventCreate(&st->ev[i]) == cudaSuccess;
    ok = ok && cudaMalloc((void**) &st->status_word, 256) == cudaSuccess;
    ok = ok && cudaMemset(st->status_word, 0, 256) == cudaSuccess;
    if (!ok) {
        set_error("device state creation failed: %s", cudaGetErrorString(cudaGetLastError()));
        delete st;
        return nullptr;
    }
    g_states[dev] = st;
    return st;
}

// Grow-only arena.  Growing waits for the device first: an earlier call's
// kernels may still be reading the old block.
static int grow(void** p, size_t* have, size_t need) {
    if (need <= *have) return CAKEB200_OK;
    CAKE_CUDA_OK(cudaDeviceSynchronize());
    if (*p) CAKE_CUDA_OK(cudaFree(*p));
    *p = nullptr;
    *have = 0;
    const size_t want = (need + (size_t(1) << 21) - 1) & ~((size_t(1) << 21) - 1);
    CAKE_CUDA_OK(cudaMalloc(p, want));
    *have = want;
    return CAKEB200_OK;
}
int ensure_scratch(DeviceState* st, size_t bytes) { return grow(&st->scratch, &st->scratch_bytes, bytes); }

namespace {

bool on_device(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// A matrix argument that may live on the host: `dev` is where kernels see it.
struct Operand {
    const void* user = nullptr;
    void* dev = nullptr;
    size_t bytes = 0;
    bool host = false;
};

int stage_in(DeviceState* st, int slot, Operand& op, const void* user, size_t bytes, bool copy, cudaStream_t s) {
    op.user = user;
    op.bytes = bytes;
    op.host = !on_device(user);
    if (!op.host) {
        op.dev = const_cast<void*>(user);
        return CAKEB200_OK;
    }
    int rc = grow(&st->staging[slot], &st->staging_bytes[slot], bytes);
    if (rc) return rc;
    op.dev = st->staging[slot];
    if (copy) CAKE_CUDA_OK(cudaMemcpyAsync(op.dev, user, bytes, cudaMemcpyHostToDevice, s));
    return CAKEB200_OK;
}

int stage_out(const Operand& op, cudaStream_t s) {
    if (op.host) CAKE_CUDA_OK(cudaMemcpyAsync(const_cast<void*>(op.user), op.dev, op.bytes, cudaMemcpyDeviceToHost, s));
    return CAKEB200_OK;
}

// Page-locked landing place for the status word, one per host thread: a device-to-host copy into
// pageable memory goes through the driver's staging buffer and costs the blocking call tens of
// microseconds; into page-locked memory it is a plain DMA.  Falls back to the caller's stack array.
struct HostStatus {
    int* word = nullptr;
    HostStatus() {
        if (cudaHostAlloc((void**) &word, 64, cudaHostAllocPortable) != cudaSuccess) {
            cudaGetLastError();
            word = nullptr;
        }
    }
    ~HostStatus() {
        if (word) cudaFreeHost(word);
        cudaGetLastError();  // at process exit the runtime may already be gone
    }
};

}  // namespace
int* pinned_host_words() {
    static thread_local HostStatus pinned;
    return pinned.word;
}
namespace {

int check_status_word(DeviceState* st, cudaStream_t s) {
    int stack_word[4] = {0, 0, 0, 0};
    int* pinned = pinned_host_words();
    int* host_word = pinned ? pinned : stack_word;
    CAKE_CUDA_OK(cudaMemcpyAsync(host_word, st->status_word, sizeof(stack_word), cudaMemcpyDeviceToHost, s));
    CAKE_CUDA_OK(cudaStreamSynchronize(s));
    if (host_word[0] != 0) {
        set_error("device-side wait gave up (code %d, where %d, info %d)", host_word[0], host_word[1], host_word[2]);
        cudaMemsetAsync(st->status_word, 0, 256, s);
        cudaStreamSynchronize(s);
        return CAKEB200_ERR_DEVICE_TIMEOUT;
    }
    return CAKEB200_OK;
}

// Queried once per device: the property calls cost milliseconds, far too much per product.
void b200_cntx(DeviceState* st, cakeb200_cntx* c) {
    static std::mutex m;
    static cakeb200_cntx cached[MAX_DEVICES];
    static bool have[MAX_DEVICES] = {};
    std::lock_guard<std::mutex> lock(m);
    if (!have[st->device]) {
        cudaDeviceProp prop;
        cudaGetDeviceProperties(&prop, st->device);
        size_t free_b = 0, total_b = 0;
        cudaMemGetInfo(&free_b, &total_b);
        int ndev = 0;
        cudaGetDeviceCount(&ndev);
        cakeb200_cntx& k = cached[st->device];
        k.alpha_n = 1.0;
        k.mr = 128;
        k.nr = 256;
        k.L1 = (int) prop.sharedMemPerMultiprocessor;
        k.L2 = prop.l2CacheSize;
        k.L3 = (int) std::min<size_t>(total_b, (size_t) INT_MAX);
        k.ncores = ndev;
        have[st->device] = true;
    }
    *c = cached[st->device];
}

// Tile order for a shape when the caller leaves the schedule open: the same
// MEMA rule as derive_schedule with the device L2 in the role of the cache that
// holds a CB block (src/block_sizing.cpp:434-462).
int resolve_schedule(DeviceState* st, int M, int N, int K, int sched) {
    if (sched != CAKEB200_SCHED_NA) return sched;
    cakeb200_cntx c;
    b200_cntx(st, &c);
    c.ncores = 1;
    cakeb200_blk_dims x;
    if (cakeb200_init_block_dims(M, N, K, 1, &x, &c, CAKEB200_SCHED_NA, 0, 0, 0) != CAKEB200_OK) return CAKEB200_SCHED_KMN;
    return x.sch;
}

// The tensor-core path pays a fixed operand-split pass; tiny products run on FFMA.
int resolve_kernel(int kernel, long long M, long long N, long long K, long long batch) {
    if (kernel != CAKEB200_KERNEL_AUTO) return kernel;
    if (batch > 1) return CAKEB200_KERNEL_FFMA;
    if (M >= 256 && N >= 256 && K >= 64 && M * N * K >= (1LL << 27)) return CAKEB200_KERNEL_TF32X3;
    return CAKEB200_KERNEL_FFMA;
}

int run_dense(DeviceState* st, GemmProblem& g, int kernel, cudaStream_t s, bool timed) {
    // a product with a single column or a single row is a matrix-vector product: stream the matrix once
    if (kernel != CAKEB200_KERNEL_TF32X3 && g.batch == 1 && !g.trans_a && !g.trans_b && !g.bias && g.out_p == 0 &&
        ((g.N == 1 && g.ldb == 1 && g.ldc == 1) || (g.M == 1 && g.ldb == g.N && g.N > 1))) {
        const bool column = g.N == 1;  // C (M x 1) = A x   else   C (1 x N) = B^T a, B read as column-major N x K
        const int rows = column ? g.M : g.N;
        int rc = ensure_scratch(st, sgemv_scratch_bytes(rows, g.K, st->sm_count));
        if (rc) return rc;
        int launches = 0;
        rc = column ? launch_sgemv(g.A, g.B, g.C, g.M, g.K, g.lda, 0, g.accumulate, st->scratch, st->scratch_bytes, st->sm_count, s,
                                   &launches)
                    : launch_sgemv(g.B, g.A, g.C, g.N, g.K, g.N, 1, g.accumulate, st->scratch, st->scratch_bytes, st->sm_count, s,
                                   &launches);
        g_stats.kernel = CAKEB200_KERNEL_FFMA;
        g_stats.launches += launches;
        return rc;
    }
    kernel = resolve_kernel(kernel, g.M, g.N, g.K, g.batch);
    g_stats.kernel = kernel;
    if (kernel == CAKEB200_KERNEL_FFMA) {
        g_stats.launches += 1;
        return launch_sgemm_ffma(g, s);
    }
    if (kernel != CAKEB200_KERNEL_TF32X3) {
        set_error("unknown kernel id %d", kernel);
        return CAKEB200_ERR_ARG;
    }
    const size_t need = tf32x3_scratch_bytes(g.M, g.N, g.K, st->sm_count);
    int rc = ensure_scratch(st, need);
    if (rc) return rc;
    g_stats.ms_prepass = timed ? -1.0f : 0.0f;  // -1: events 4,5 hold the split-pass time
    return launch_sgemm_tf32x3(g, st->scratch, st->scratch_bytes, st->status_word, st->sm_count, s, &g_stats,
                               timed ? &st->ev[4] : nullptr);
}

bool bad_dims(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) {
        set_error("matrix dimensions must be positive (M=%d N=%d K=%d)", M, N, K);
        return true;
    }
    return false;
}

float elapsed(cudaEvent_t a, cudaEvent_t b) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, a, b) != cudaSuccess) cudaGetLastError();
    return ms;
}

int ensure_pipeline(DeviceState* st) {
    if (st->copy_in) return CAKEB200_OK;
    CAKE_CUDA_OK(cudaStreamCreateWithFlags(&st->copy_in, cudaStreamNonBlocking));
    CAKE_CUDA_OK(cudaStreamCreateWithFlags(&st->copy_out, cudaStreamNonBlocking));
    for (int i = 0; i < DeviceState::MAX_BANDS; i++) {
        CAKE_CUDA_OK(cudaEventCreateWithFlags(&st->band_in[i], cudaEventDisableTiming));
        CAKE_CUDA_OK(cudaEventCreateWithFlags(&st->band_done[i], cudaEventDisableTiming));
    }
    for (int i = 0; i < 3; i++) CAKE_CUDA_OK(cudaEventCreateWithFlags(&st->fence[i], cudaEventDisableTiming));
    return CAKEB200_OK;
}

// Host operands, large M: the product is cut into bands of rows.  While band i is
// multiplied, the rows of band i+1 are still arriving over PCIe and the result rows
// of band i-1 are already leaving; only B has to be complete before the first band.
// This is the GPU form of the reference's on-the-fly packing driver, which packs
// block i+1 while block i is multiplied (src/cake_sgemm_k_first.cpp:633-813).
int sgemm_host_pipelined(DeviceState* st, const float* A, const float* B, float* C, GemmProblem g, int kernel,
                         cudaStream_t s, cudaEvent_t b_ready) {
    const int M = g.M, N = g.N, K = g.K;
    int rc;
    static const bool debug_timing = getenv("CAKEB200_DEBUG_TIMING") != nullptr;
    timespec h0, h1, h2;
    clock_gettime(CLOCK_MONOTONIC, &h0);
    if ((rc = ensure_pipeline(st))) return rc;
    kernel = resolve_kernel(kernel, M, N, K, 1);
    g_stats.kernel = kernel;
    const bool b_host = !on_device(B);
    if ((rc = grow(&st->staging[0], &st->staging_bytes[0], (size_t) M * K * 4))) return rc;
    if (b_host && (rc = grow(&st->staging[1], &st->staging_bytes[1], (size_t) K * N * 4))) return rc;
    if ((rc = grow(&st->staging[2], &st->staging_bytes[2], (size_t) M * N * 4))) return rc;
    float* dA = (float*) st->staging[0];
    const float* dB = b_host ? (const float*) st->staging[1] : B;
    float* dC = (float*) st->staging[2];
    Tf32x3Planes planes = {};
    if (kernel == CAKEB200_KERNEL_TF32X3) {
        if ((rc = ensure_scratch(st, tf32x3_plane_bytes(M, N, K)))) return rc;
        if ((rc = tf32x3_planes(M, N, K, st->scratch, st->scratch_bytes, &planes))) return rc;
    }

    // bands of whole tiles (128 rows, or 256 where the tensor-core kernel runs on pairs of SMs); enough of
    // them that the first and last are short
    const int tile_rows = (kernel == CAKEB200_KERNEL_TF32X3) ? tf32x3_tile_rows(M, N, K, g.order, st->sm_count) : 128;
    const int tiles = (M + tile_rows - 1) / tile_rows;
    const int bands = std::max(1, std::min(std::min(DeviceState::MAX_BANDS, 16), tiles / 2));
    CAKE_CUDA_OK(cudaEventRecord(st->ev[0], s));
    CAKE_CUDA_OK(cudaEventRecord(st->fence[0], s));
    CAKE_CUDA_OK(cudaStreamWaitEvent(st->copy_in, st->fence[0], 0));
    CAKE_CUDA_OK(cudaStreamWaitEvent(st->copy_out, st->fence[0], 0));
    if (b_host) {
        CAKE_CUDA_OK(cudaMemcpyAsync(st->staging[1], B, (size_t) K * N * 4, cudaMemcpyHostToDevice, st->copy_in));
        CAKE_CUDA_OK(cudaEventRecord(st->fence[1], st->copy_in));
        CAKE_CUDA_OK(cudaStreamWaitEvent(s, st->fence[1], 0));
    }
    // B being completed by someone else (a gather from other GPUs): only the kernels wait for it,
    // the rows of A keep arriving meanwhile
    if (b_ready) CAKE_CUDA_OK(cudaStreamWaitEvent(s, b_ready, 0));
    if (kernel == CAKEB200_KERNEL_TF32X3) {
        if ((rc = tf32x3_split_B(dB, N, K, N, planes, s))) return rc;
        g_stats.launches++;
        g_stats.tile_m = tile_rows; g_stats.tile_n = N > 128 ? 256 : 128; g_stats.tile_k = 32;
    }
    for (int b = 0; b < bands; b++) {
        const int r0 = (int) ((long long) tiles * b / bands) * tile_rows;
        const int r1 = (b == bands - 1) ? M : (int) ((long long) tiles * (b + 1) / bands) * tile_rows;
        const int rows = r1 - r0;
        if (rows <= 0) continue;
        CAKE_CUDA_OK(cudaMemcpyAsync(dA + (size_t) r0 * K, A + (size_t) r0 * K, (size_t) rows * K * 4,
                                     cudaMemcpyHostToDevice, st->copy_in));
        if (g.accumulate)
            CAKE_CUDA_OK(cudaMemcpyAsync(dC + (size_t) r0 * N, C + (size_t) r0 * N, (size_t) rows * N * 4,
                                         cudaMemcpyHostToDevice, st->copy_in));
        CAKE_CUDA_OK(cudaEventRecord(st->band_in[b], st->copy_in));
        if (b == bands - 1) CAKE_CUDA_OK(cudaEventRecord(st->ev[1], st->copy_in));
        CAKE_CUDA_OK(cudaStreamWaitEvent(s, st->band_in[b], 0));
        if (kernel == CAKEB200_KERNEL_TF32X3) {
            if ((rc = tf32x3_split_A_rows(dA, K, r0, rows, K, planes, st->sm_count, s))) return rc;
            if ((rc = tf32x3_multiply_rows(planes, dC, N, r0, rows, N, K, g.order, g.accumulate, st->status_word,
                                           st->sm_count, s)))
                return rc;
            g_stats.launches += 2;
        } else {
            GemmProblem band = g;
            band.A = dA + (size_t) r0 * K; band.B = dB; band.C = dC + (size_t) r0 * N;
            band.M = rows;
            if ((rc = launch_sgemm_ffma(band, s))) return rc;
            g_stats.launches += 1;
        }
        CAKE_CUDA_OK(cudaEventRecord(st->band_done[b], s));
        if (b == bands - 1) CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
        CAKE_CUDA_OK(cudaStreamWaitEvent(st->copy_out, st->band_done[b], 0));
        CAKE_CUDA_OK(cudaMemcpyAsync(C + (size_t) r0 * N, dC + (size_t) r0 * N, (size_t) rows * N * 4,
                                     cudaMemcpyDeviceToHost, st->copy_out));
    }
    CAKE_CUDA_OK(cudaEventRecord(st->ev[3], st->copy_out));
    CAKE_CUDA_OK(cudaEventRecord(st->fence[2], st->copy_out));
    CAKE_CUDA_OK(cudaStreamWaitEvent(s, st->fence[2], 0));
    clock_gettime(CLOCK_MONOTONIC, &h1);
    if ((rc = check_status_word(st, s))) return rc;
    clock_gettime(CLOCK_MONOTONIC, &h2);
    if (debug_timing)
        fprintf(stderr, "cakeb200 pipelined: %d bands, host enqueue %.3f ms, wait %.3f ms\n", bands,
                (h1.tv_sec - h0.tv_sec) * 1e3 + (h1.tv_nsec - h0.tv_nsec) * 1e-6,
                (h2.tv_sec - h1.tv_sec) * 1e3 + (h2.tv_nsec - h1.tv_nsec) * 1e-6);
    // the phases overlap; report the spans that do not: start -> last row arrived -> last band multiplied -> last row back
    g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
    g_stats.ms_gemm = elapsed(st->ev[1], st->ev[2]);
    g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
    return CAKEB200_OK;
}

int sgemm_impl(const float* A, const float* B, float* C, int M, int N, int K, int accumulate, int sched,
               int kernel, void* stream, bool blocking, cudaEvent_t b_ready = nullptr) {
    g_stats = cakeb200_stats();
    if (!A || !B || !C) {
        set_error("null matrix pointer");
        return CAKEB200_ERR_ARG;
    }
    if (bad_dims(M, N, K)) return CAKEB200_ERR_ARG;
    if (sched < 0 || sched > CAKEB200_SCHED_NA) {
        set_error("unknown schedule %d", sched);
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;  // NULL = the CUDA default stream, ordered with the caller's default-stream work

    GemmProblem g = {};
    g.M = M; g.N = N; g.K = K;
    g.lda = K; g.ldb = N; g.ldc = N;
    g.batch = 1;
    g.accumulate = accumulate ? 1 : 0;
    g.order = resolve_schedule(st, M, N, K, sched);
    g_stats.sched = g.order;

    if (!blocking) {
        if (!on_device(A) || !on_device(B) || !on_device(C)) {
            set_error("cakeb200_sgemm_async needs device pointers");
            return CAKEB200_ERR_ARG;
        }
        g.A = A; g.B = B; g.C = C;
        if (st->profiling && st->profile_count < DeviceState::MAX_PROFILE) {
            cudaEvent_t* e = &st->profile_ev[3 * st->profile_count];
            const bool tensor = resolve_kernel(kernel, M, N, K, 1) == CAKEB200_KERNEL_TF32X3;
            int rc = CAKEB200_OK;
            if (tensor) {
                const size_t need = tf32x3_scratch_bytes(M, N, K, st->sm_count);
                if ((rc = ensure_scratch(st, need))) return rc;
                g_stats.kernel = CAKEB200_KERNEL_TF32X3;
                rc = launch_sgemm_tf32x3(g, st->scratch, st->scratch_bytes, st->status_word, st->sm_count, s, &g_stats, e);
            } else {
                CAKE_CUDA_OK(cudaEventRecord(e[0], s));
                CAKE_CUDA_OK(cudaEventRecord(e[1], s));
                rc = run_dense(st, g, kernel, s, false);
            }
            if (rc) return rc;
            CAKE_CUDA_OK(cudaEventRecord(e[2], s));
            st->profile_count++;
            return CAKEB200_OK;
        }
        return run_dense(st, g, kernel, s, false);
    }

    if (!on_device(A) && !on_device(C) && M >= 1024) return sgemm_host_pipelined(st, A, B, C, g, kernel, s, b_ready);
    if (b_ready) CAKE_CUDA_OK(cudaStreamWaitEvent(s, b_ready, 0));

    Operand oa, ob, oc;
    int rc;
    static const bool host_timing = getenv("CAKEB200_DEBUG_TIMING") != nullptr;
    timespec t0, t1, t2, t3;
    if (host_timing) clock_gettime(CLOCK_MONOTONIC, &t0);
    CAKE_CUDA_OK(cudaEventRecord(st->ev[0], s));
    if ((rc = stage_in(st, 0, oa, A, (size_t) M * K * 4, true, s))) return rc;
    if ((rc = stage_in(st, 1, ob, B, (size_t) K * N * 4, true, s))) return rc;
    if ((rc = stage_in(st, 2, oc, C, (size_t) M * N * 4, g.accumulate != 0, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[1], s));
    if (host_timing) clock_gettime(CLOCK_MONOTONIC, &t1);
    g.A = (const float*) oa.dev; g.B = (const float*) ob.dev; g.C = (float*) oc.dev;
    if ((rc = run_dense(st, g, kernel, s, true))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
    if ((rc = stage_out(oc, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[3], s));
    if (host_timing) clock_gettime(CLOCK_MONOTONIC, &t2);
    if ((rc = check_status_word(st, s))) return rc;
    if (host_timing) {
        clock_gettime(CLOCK_MONOTONIC, &t3);
        auto us = [](const timespec& a, const timespec& b) { return (b.tv_sec - a.tv_sec) * 1e6 + (b.tv_nsec - a.tv_nsec) * 1e-3; };
        fprintf(stderr, "cakeb200 blocking call, host side: operands %.1f us, enqueue %.1f us, wait + status %.1f us\n", us(t0, t1),
                us(t1, t2), us(t2, t3));
    }
    g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
    g_stats.ms_prepass = (g_stats.ms_prepass < 0.f) ? elapsed(st->ev[4], st->ev[5]) : 0.f;
    const float mid = elapsed(st->ev[1], st->ev[2]);
    g_stats.ms_gemm = mid - g_stats.ms_prepass;
    g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
    return CAKEB200_OK;
}

// C = op(A) op(B) (+ bias) on device operands with leading dimensions, asynchronous on `stream`.
int sgemm_ex_impl(const float* A, int lda, int trans_a, const float* B, int ldb, int trans_b, float* C, int ldc, int M,
                  int N, int K, const float* bias, int accumulate, int sched, int kernel, void* stream) {
    g_stats = cakeb200_stats();
    if (!A || !B || !C) {
        set_error("null matrix pointer");
        return CAKEB200_ERR_ARG;
    }
    if (bad_dims(M, N, K)) return CAKEB200_ERR_ARG;
    if (sched < 0 || sched > CAKEB200_SCHED_NA) {
        set_error("unknown schedule %d", sched);
        return CAKEB200_ERR_ARG;
    }
    if (lda < (trans_a ? M : K) || ldb < (trans_b ? K : N) || ldc < N) {
        set_error("leading dimension smaller than the row length (lda=%d ldb=%d ldc=%d)", lda, ldb, ldc);
        return CAKEB200_ERR_ARG;
    }
    if (!on_device(A) || !on_device(B) || !on_device(C) || (bias && !on_device(bias))) {
        set_error("cakeb200_sgemm_ex needs device pointers");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;

    GemmProblem g = {};
    g.A = A; g.B = B; g.C = C;
    g.M = M; g.N = N; g.K = K;
    g.lda = lda; g.ldb = ldb; g.ldc = ldc;
    g.batch = 1;
    g.accumulate = accumulate ? 1 : 0;
    g.order = resolve_schedule(st, M, N, K, sched);
    g.trans_a = trans_a ? 1 : 0;
    g.trans_b = trans_b ? 1 : 0;
    g.bias = bias;
    g_stats.sched = g.order;
    if (resolve_kernel(kernel, M, N, K, 1) == CAKEB200_KERNEL_FFMA && (g.trans_a || g.trans_b)) {
        // the FFMA kernel reads row-major A and B: lay a transposed operand out that way first
        const size_t a_bytes = g.trans_a ? ((size_t) M * K * 4 + 255) / 256 * 256 : 0;
        const size_t b_bytes = g.trans_b ? (size_t) K * N * 4 : 0;
        int rc = ensure_scratch(st, a_bytes + b_bytes);
        if (rc) return rc;
        if (g.trans_a) {
            if ((rc = launch_transpose_copy(A, (float*) st->scratch, K, M, lda, s))) return rc;
            g.A = (const float*) st->scratch; g.lda = K; g.trans_a = 0;
            g_stats.launches += 1;
        }
        if (g.trans_b) {
            float* bt = (float*) ((char*) st->scratch + a_bytes);
            if ((rc = launch_transpose_copy(B, bt, N, K, ldb, s))) return rc;
            g.B = bt; g.ldb = N; g.trans_b = 0;
            g_stats.launches += 1;
        }
    }
    return run_dense(st, g, kernel, s, false);
}

typedef int (*pack_fn)(const float*, float*, int, int, int, const cakeb200_blk_dims*, const cakeb200_cntx*, bool, cudaStream_t);

// mat: rows x cols matrix, packed: packed buffer of packed_bytes; unpack moves packed -> mat.
int pack_impl(pack_fn fn, const float* mat, size_t mat_bytes, float* packed, size_t packed_bytes, int d0, int d1,
              int p, const cakeb200_blk_dims* x, const cakeb200_cntx* c, bool unpack, void* stream) {
    g_stats = cakeb200_stats();
    if (!mat || !packed || !x || !c) {
        set_error("null argument");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;  // NULL = the CUDA default stream, ordered with the caller's default-stream work
    Operand om, op;
    int rc;
    // unpack leaves matrix cells outside the packed image untouched, so the matrix is always copied in
    if ((rc = stage_in(st, 0, om, mat, mat_bytes, true, s))) return rc;
    if ((rc = stage_in(st, 1, op, packed, packed_bytes, unpack, s))) return rc;
    if ((rc = fn((const float*) om.dev, (float*) op.dev, d0, d1, p, x, c, unpack, s))) return rc;
    g_stats.launches = 1;
    g_stats.tile_k = last_pack_width();  // floats moved per access: 4 when every block allows 16-byte moves
    if ((rc = stage_out(unpack ? om : op, s))) return rc;
    CAKE_CUDA_OK(cudaStreamSynchronize(s));
    return CAKEB200_OK;
}

}  // namespace
}  // namespace cakeb200

using namespace cakeb200;

extern "C" {

const char* cakeb200_last_error(void) { return g_error; }

void cakeb200_get_stats(cakeb200_stats* out) {
    if (out) *out = g_stats;
}

int cakeb200_device_count(void) {
    int n = 0, good = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    for (int i = 0; i < n; i++) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) good++;
    }
    return good;
}

int cakeb200_query_cntx(cakeb200_cntx* out) {
    if (!out) return CAKEB200_ERR_ARG;
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    b200_cntx(st, out);
    return CAKEB200_OK;
}

int cakeb200_set_option(const char* name, int value) {
    if (!name || value < 0) {
        set_error("cakeb200_set_option: null name or negative value");
        return CAKEB200_ERR_ARG;
    }
    for (int i = 0; i < OPT_COUNT; i++) {
        if (strcmp(name, g_option_names[i])) continue;
        if ((i == OPT_TILE_N && value != 0 && value != 128 && value != 256) || (i == OPT_CONV_ROUTE && value > 3) ||
            (i == OPT_SMALL_OPERANDS && value > 2) || (i == OPT_PACK_SCALAR && value > 1) || (i == OPT_PAIR && value > 2)) {
            set_error("cakeb200_set_option: %d is not a value of '%s'", value, name);
            return CAKEB200_ERR_ARG;
        }
        g_options[i] = value;
        return CAKEB200_OK;
    }
    set_error("cakeb200_set_option: unknown option '%s'", name);
    return CAKEB200_ERR_ARG;
}

int cakeb200_get_option(const char* name) {
    if (!name) return -1;
    for (int i = 0; i < OPT_COUNT; i++)
        if (!strcmp(name, g_option_names[i])) return g_options[i];
    return -1;
}

int cakeb200_tf32_peak(float ms_target, float* tflops, float* ms, void* stream) {
    static std::mutex m;
    static float cached[MAX_DEVICES] = {};
    if (!tflops) {
        set_error("cakeb200_tf32_peak: null result pointer");
        return CAKEB200_ERR_ARG;
    }
    if (ms_target > 200.f) {
        set_error("cakeb200_tf32_peak: at most 200 ms");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    if (ms_target <= 0.f) {
        std::lock_guard<std::mutex> lock(m);
        if (cached[st->device] > 0.f) {
            *tflops = cached[st->device];
            if (ms) *ms = 0.f;
            return CAKEB200_OK;
        }
    }
    float got = 0.f, took = 0.f;
    int rc = measure_tf32_peak(st->status_word, st->sm_count, ms_target > 0.f ? ms_target : 2.0f, (cudaStream_t) stream, &got, &took);
    if (rc) return rc;
    if ((rc = check_status_word(st, (cudaStream_t) stream))) return rc;
    {
        std::lock_guard<std::mutex> lock(m);
        cached[st->device] = got;
    }
    *tflops = got;
    if (ms) *ms = took;
    return CAKEB200_OK;
}

// ---- an operand kept in the kernel's own form across products

struct cakeb200_planes {
    float *hi = nullptr, *lo = nullptr;
    int rows = 0, K = 0, is_b = 0, device = -1;
    size_t bytes = 0;  // of one plane
};

int cakeb200_planes_create(const float* mat, int rows, int K, int is_b, cakeb200_planes** out, void* stream) {
    g_stats = cakeb200_stats();
    if (!mat || !out || rows <= 0 || K <= 0) {
        set_error("cakeb200_planes_create: bad argument");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;
    cakeb200_planes* p = new cakeb200_planes();
    p->rows = rows; p->K = K; p->is_b = is_b ? 1 : 0; p->device = st->device;
    p->bytes = tf32x3_one_plane_bytes(rows, K);
    cudaError_t e = cudaMalloc((void**) &p->hi, 2 * p->bytes);
    if (e != cudaSuccess) {
        set_error("cakeb200_planes_create: %s", cudaGetErrorString(e));
        cudaGetLastError();
        delete p;
        return CAKEB200_ERR_CUDA;
    }
    p->lo = (float*) ((char*) p->hi + p->bytes);
    Operand om;
    // A: rows x K row-major.  B: K x rows row-major, split into its transposed planes (rows x K).
    int rc = stage_in(st, 0, om, mat, (size_t) rows * K * 4, true, s);
    if (!rc) rc = tf32x3_make_planes((const float*) om.dev, rows, K, is_b ? rows : K, is_b != 0, p->hi, p->lo, st->sm_count, s);
    if (!rc && cudaStreamSynchronize(s) != cudaSuccess) rc = CAKEB200_ERR_CUDA;
    if (rc) {
        cudaFree(p->hi);
        cudaGetLastError();
        delete p;
        return rc;
    }
    g_stats.launches = 1;
    *out = p;
    return CAKEB200_OK;
}

int cakeb200_planes_destroy(cakeb200_planes* p) {
    if (!p) return CAKEB200_OK;
    if (p->hi) {
        cudaDeviceSynchronize();  // a product still reading the planes finishes first
        cudaFree(p->hi);
        cudaGetLastError();
    }
    delete p;
    return CAKEB200_OK;
}

int cakeb200_sgemm_planes(const cakeb200_planes* A_planes, const float* A, const cakeb200_planes* B_planes, const float* B,
                          float* C, int M, int N, int K, int accumulate, int sched, void* stream) {
    g_stats = cakeb200_stats();
    if (!C || (!A_planes && !A) || (!B_planes && !B)) {
        set_error("cakeb200_sgemm_planes: every operand needs planes or a matrix");
        return CAKEB200_ERR_ARG;
    }
    if (bad_dims(M, N, K)) return CAKEB200_ERR_ARG;
    if (sched < 0 || sched > CAKEB200_SCHED_NA) {
        set_error("unknown schedule %d", sched);
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    if ((A_planes && (A_planes->is_b || A_planes->rows != M || A_planes->K != K || A_planes->device != st->device)) ||
        (B_planes && (!B_planes->is_b || B_planes->rows != N || B_planes->K != K || B_planes->device != st->device))) {
        set_error("cakeb200_sgemm_planes: the planes were made for another operand, shape or device");
        return CAKEB200_ERR_ARG;
    }
    cudaStream_t s = (cudaStream_t) stream;
    Operand oa, ob, oc;
    int rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[0], s));
    if (!A_planes && (rc = stage_in(st, 0, oa, A, (size_t) M * K * 4, true, s))) return rc;
    if (!B_planes && (rc = stage_in(st, 1, ob, B, (size_t) K * N * 4, true, s))) return rc;
    if ((rc = stage_in(st, 2, oc, C, (size_t) M * N * 4, accumulate != 0, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[1], s));
    GemmProblem g = {};
    g.A = (const float*) oa.dev; g.B = (const float*) ob.dev; g.C = (float*) oc.dev;
    g.M = M; g.N = N; g.K = K;
    g.lda = K; g.ldb = N; g.ldc = N;
    g.batch = 1;
    g.accumulate = accumulate ? 1 : 0;
    g.order = resolve_schedule(st, M, N, K, sched);
    if (A_planes) { g.a_hi = A_planes->hi; g.a_lo = A_planes->lo; }
    if (B_planes) { g.b_hi = B_planes->hi; g.b_lo = B_planes->lo; }
    g_stats.sched = g.order;
    g_stats.kernel = CAKEB200_KERNEL_TF32X3;
    if ((rc = ensure_scratch(st, tf32x3_scratch_bytes(M, N, K, st->sm_count)))) return rc;
    if ((rc = launch_sgemm_tf32x3(g, st->scratch, st->scratch_bytes, st->status_word, st->sm_count, s, &g_stats, &st->ev[4]))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
    if ((rc = stage_out(oc, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[3], s));
    if ((rc = check_status_word(st, s))) return rc;
    g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
    g_stats.ms_prepass = elapsed(st->ev[4], st->ev[5]);
    g_stats.ms_gemm = elapsed(st->ev[1], st->ev[2]) - g_stats.ms_prepass;
    g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
    return CAKEB200_OK;
}

// ---- tile-shape search on the device (the cache and the search itself are host logic, tune.cpp)

namespace {
struct TuneRun {
    DeviceState* st;
    GemmProblem g;
    cudaStream_t s;
    int reps;
    int rc;
};

// cost of one point of the grid: fastest of `reps` whole products (split pass + contraction) with the point forced
double tune_cost(int tile_n, int cluster, int band, int k_pieces, void* user) {
    TuneRun* r = (TuneRun*) user;
    if (cakeb200_set_option("tile_n", tile_n) || cakeb200_set_option("pair", cluster) || cakeb200_set_option("band", band) ||
        cakeb200_set_option("k_pieces", k_pieces))
        return -1;
    double best = -1;
    for (int i = 0; i < r->reps + 1; i++) {  // the first run uploads the tile plan of the point and is not timed
        if (cudaEventRecord(r->st->ev[0], r->s) != cudaSuccess) return -1;
        r->rc = launch_sgemm_tf32x3(r->g, r->st->scratch, r->st->scratch_bytes, r->st->status_word, r->st->sm_count, r->s, nullptr, nullptr);
        if (r->rc) return -1;
        if (cudaEventRecord(r->st->ev[1], r->s) != cudaSuccess || cudaEventSynchronize(r->st->ev[1]) != cudaSuccess) return -1;
        const double ms = elapsed(r->st->ev[0], r->st->ev[1]);
        if (i > 0 && (best < 0 || ms < best)) best = ms;
    }
    return best;
}
}  // namespace

int cakeb200_tune(const float* A, const float* B, float* C, int M, int N, int K, int sched, int trials, void* stream) {
    g_stats = cakeb200_stats();
    if (!A || !B || !C || bad_dims(M, N, K)) return CAKEB200_ERR_ARG;
    if (!on_device(A) || !on_device(B) || !on_device(C)) {
        set_error("cakeb200_tune needs device pointers");
        return CAKEB200_ERR_ARG;
    }
    if (sched < 0 || sched > CAKEB200_SCHED_NA || trials < 1 || trials > 1000) {
        set_error("cakeb200_tune: unknown schedule or trials outside 1..1000");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    TuneRun run = {};
    run.st = st;
    run.s = (cudaStream_t) stream;
    run.reps = 3;
    run.g.A = A; run.g.B = B; run.g.C = C;
    run.g.M = M; run.g.N = N; run.g.K = K;
    run.g.lda = K; run.g.ldb = N; run.g.ldc = N;
    run.g.batch = 1;
    run.g.order = resolve_schedule(st, M, N, K, sched);
    int rc = ensure_scratch(st, tf32x3_scratch_bytes(M, N, K, st->sm_count));
    if (rc) return rc;
    const int keep[4] = {cakeb200_get_option("tile_n"), cakeb200_get_option("band"), cakeb200_get_option("k_pieces"),
                         cakeb200_get_option("pair")};
    int tile_n = 0, cluster = 0, band = 0, k_pieces = 0, evaluated = 0;
    float best_ms = 0.f;
    rc = cakeb200_tune_search_shape(M, N, K, st->sm_count, trials, 0x5eedULL + (unsigned long long) M * 31 + N * 17 + K, tune_cost, &run,
                                    &tile_n, &cluster, &band, &k_pieces, &best_ms, &evaluated);
    // The clocks drift while dozens of candidates run, so times taken minutes apart do not compare.  The winner
    // is therefore run again in turns with the rule's own choice, and it replaces the rule only when it is
    // at least 3 % faster on the median of those turns.
    if (!rc) {
        double win[5], rule[5];
        bool ok = true;
        run.reps = 2;
        for (int i = 0; i < 5 && ok; i++) {
            rule[i] = tune_cost(0, 0, 0, 0, &run);
            win[i] = tune_cost(tile_n, cluster, band, k_pieces, &run);
            ok = rule[i] > 0 && win[i] > 0;
        }
        if (ok) {
            std::sort(win, win + 5);
            std::sort(rule, rule + 5);
            if (win[2] > 0.97 * rule[2]) {  // not clearly better: record the rule itself
                tile_n = 0; cluster = 0; band = 8; k_pieces = 0;
                best_ms = (float) rule[2];
            } else {
                best_ms = (float) win[2];
            }
        }
    }
    cakeb200_set_option("tile_n", keep[0]);
    cakeb200_set_option("band", keep[1]);
    cakeb200_set_option("k_pieces", keep[2]);
    cakeb200_set_option("pair", keep[3]);
    if (rc) return run.rc ? run.rc : rc;
    if ((rc = check_status_word(st, run.s))) return rc;
    if ((rc = cakeb200_tune_put_shape(M, N, K, run.g.order, tile_n, cluster, band, k_pieces, best_ms))) return rc;
    if (const char* path = getenv("CAKE_AUTOTUNE_CACHE")) cakeb200_tune_save(path);
    g_stats.tile_m = (cluster == 1 || (cluster == 0 && tf32x3_tile_rows(M, N, K, run.g.order, st->sm_count) == 256)) ? 256 : 128; g_stats.tile_n = tile_n; g_stats.tile_k = 32;
    g_stats.ms_gemm = best_ms;
    g_stats.launches = evaluated;
    g_stats.kernel = CAKEB200_KERNEL_TF32X3;
    g_stats.sched = run.g.order;
    return CAKEB200_OK;
}

int cakeb200_profile_begin(void) {
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    for (int i = 0; i < 3 * DeviceState::MAX_PROFILE; i++)
        if (!st->profile_ev[i]) CAKE_CUDA_OK(cudaEventCreate(&st->profile_ev[i]));
    st->profile_count = 0;
    st->profiling = true;
    return CAKEB200_OK;
}

int cakeb200_profile_end(float* ms_prepass, float* ms_kernel, int* calls) {
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    st->profiling = false;
    double pre = 0, ker = 0;
    for (int i = 0; i < st->profile_count; i++) {
        cudaEvent_t* e = &st->profile_ev[3 * i];
        CAKE_CUDA_OK(cudaEventSynchronize(e[2]));
        pre += elapsed(e[0], e[1]);
        ker += elapsed(e[1], e[2]);
    }
    if (ms_prepass) *ms_prepass = (float) pre;
    if (ms_kernel) *ms_kernel = (float) ker;
    if (calls) *calls = st->profile_count;
    st->profile_count = 0;
    return CAKEB200_OK;
}

int cakeb200_sgemm(const float* A, const float* B, float* C, int M, int N, int K, int accumulate, int sched,
                   int kernel, void* stream) {
    return sgemm_impl(A, B, C, M, N, K, accumulate, sched, kernel, stream, true);
}

int cakeb200_sgemm_after(const float* A, const float* B, float* C, int M, int N, int K, int accumulate, int sched,
                         int kernel, void* stream, void* b_ready) {
    return sgemm_impl(A, B, C, M, N, K, accumulate, sched, kernel, stream, true, (cudaEvent_t) b_ready);
}

int cakeb200_sgemm_async(const float* A, const float* B, float* C, int M, int N, int K, int accumulate, int sched,
                         int kernel, void* stream) {
    return sgemm_impl(A, B, C, M, N, K, accumulate, sched, kernel, stream, false);
}

int cakeb200_sgemm_ex(const float* A, int lda, int trans_a, const float* B, int ldb, int trans_b, float* C, int ldc, int M,
                      int N, int K, const float* bias, int accumulate, int sched, int kernel, void* stream) {
    return sgemm_ex_impl(A, lda, trans_a, B, ldb, trans_b, C, ldc, M, N, K, bias, accumulate, sched, kernel, stream);
}

int cakeb200_sgemm_batched(const float* A, const float* B, float* C, int M, int N, int K, int batch, int kernel,
                           void* stream) {
    g_stats = cakeb200_stats();
    if (!A || !B || !C || batch <= 0) {
        set_error("bad argument");
        return CAKEB200_ERR_ARG;
    }
    if (bad_dims(M, N, K)) return CAKEB200_ERR_ARG;
    if (kernel == CAKEB200_KERNEL_TF32X3 && !small_tf32x3_fits(M, N, K)) {
        set_error("the batched tensor-core kernel needs M <= 128 and N <= 256 (M=%d N=%d)", M, N);
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    // The tensor-core kernel wins once the 128-row tile is reasonably full and there are products
    // for most SMs; a few tiny products stay on the exact-FP32 kernel.
    const bool tensor = kernel == CAKEB200_KERNEL_TF32X3 ||
                        (kernel == CAKEB200_KERNEL_AUTO && small_tf32x3_fits(M, N, K) && M >= 48 && N >= 32 && K >= 32 &&
                         batch >= st->sm_count / 2);
    cudaStream_t s = (cudaStream_t) stream;  // NULL = the CUDA default stream, ordered with the caller's default-stream work
    Operand oa, ob, oc;
    int rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[0], s));
    if ((rc = stage_in(st, 0, oa, A, (size_t) batch * M * K * 4, true, s))) return rc;
    if ((rc = stage_in(st, 1, ob, B, (size_t) batch * K * N * 4, true, s))) return rc;
    if ((rc = stage_in(st, 2, oc, C, (size_t) batch * M * N * 4, false, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[1], s));
    GemmProblem g = {};
    g.A = (const float*) oa.dev; g.B = (const float*) ob.dev; g.C = (float*) oc.dev;
    g.M = M; g.N = N; g.K = K;
    g.lda = K; g.ldb = N; g.ldc = N;
    g.stride_a = (long long) M * K; g.stride_b = (long long) K * N; g.stride_c = (long long) M * N;
    g.order = CAKEB200_SCHED_MKN;
    if (tensor) {
        g.batch = batch;
        if ((rc = launch_sgemm_small_tf32x3(g, st->status_word, st->sm_count, s))) return rc;
        g_stats.launches++;
    }
    for (int done = 0; !tensor && done < batch; done += 65535) {  // gridDim.z limit
        GemmProblem part = g;
        part.batch = std::min(65535, batch - done);
        part.A += (long long) done * g.stride_a;
        part.B += (long long) done * g.stride_b;
        part.C += (long long) done * g.stride_c;
        if ((rc = launch_sgemm_ffma(part, s))) return rc;
        g_stats.launches++;
    }
    g_stats.kernel = tensor ? CAKEB200_KERNEL_TF32X3 : CAKEB200_KERNEL_FFMA;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
    if ((rc = stage_out(oc, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[3], s));
    if ((rc = check_status_word(st, s))) return rc;
    g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
    g_stats.ms_gemm = elapsed(st->ev[1], st->ev[2]);
    g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
    return CAKEB200_OK;
}

namespace {
int selftest_bounded_wait(int limit_us, void* stream, bool pair);
}
int cakeb200_selftest_bounded_wait(int limit_us, void* stream) { return selftest_bounded_wait(limit_us, stream, false); }
int cakeb200_selftest_bounded_wait_pair(int limit_us, void* stream) { return selftest_bounded_wait(limit_us, stream, true); }
namespace {
int selftest_bounded_wait(int limit_us, void* stream, bool pair) {
    g_stats = cakeb200_stats();
    if (limit_us < 1 || limit_us > 1000000) {
        set_error("limit must be between 1 us and 1 s");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;
    int rc = launch_bounded_wait_selftest(st->status_word, limit_us, s, pair);
    if (rc) return rc;
    return check_status_word(st, s);  // expected: CAKEB200_ERR_DEVICE_TIMEOUT, "where" 900 (901 for the pair)
}
}  // namespace

// ---- K-sharded product over the GPUs of one box: exchange object

struct cakeb200_kshard {
    int world = 0, rank = 0, M = 0, N = 0, device = -1;
    int row_lo[MAX_RANKS + 1] = {};
    long long slot_floats = 0;
    size_t bytes = 0;
    char* peer[MAX_RANKS] = {};    // peer[rank] is this rank's own buffer
    bool ipc_opened[MAX_RANKS] = {};
    bool connected = false;
    int epoch = 0;      // products started (partial)
    int finished = 0;   // products completed (finish); partial is refused while epoch != finished
};

namespace {
constexpr size_t KSHARD_HEADER = 1024;   // flags of the source ranks at byte 0, counter of finished CTAs at byte 128
constexpr size_t KSHARD_DONE_AT = 128;

void kshard_row_block(int M, int world, int rank, int* lo, int* hi) {
    const long long tiles = (M + 127) / 128;
    const long long a = tiles * rank / world * 128, b = tiles * (rank + 1) / world * 128;
    *lo = (int) std::min<long long>(a, M);
    *hi = (rank == world - 1) ? M : (int) std::min<long long>(b, M);
}
}  // namespace

int cakeb200_kshard_rows(int M, int world, int rank, int* lo, int* hi) {
    if (M < 0 || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || !lo || !hi) {
        set_error("kshard_rows: bad argument");
        return CAKEB200_ERR_ARG;
    }
    kshard_row_block(M, world, rank, lo, hi);
    return CAKEB200_OK;
}

int cakeb200_kshard_supported(int M, int N, int K_local, int sm_count) {
    if (sm_count <= 0) {
        DeviceState* st = device_state();
        if (!st) return 0;
        sm_count = st->sm_count;
    }
    return tf32x3_all_tiles_in_pieces(M, N, K_local, CAKEB200_SCHED_KMN, sm_count) ? 1 : 0;
}

int cakeb200_kshard_create(int world, int rank, int M, int N, cakeb200_kshard** out, unsigned char* ipc_handle) {
    if (!out || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || M < 1 || N < 1) {
        set_error("kshard_create: bad argument (world 1..%d)", MAX_RANKS);
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cakeb200_kshard* x = new cakeb200_kshard();
    x->world = world; x->rank = rank; x->M = M; x->N = N; x->device = st->device;
    int most = 0;
    for (int r = 0; r < world; r++) {
        int lo, hi;
        kshard_row_block(M, world, r, &lo, &hi);
        x->row_lo[r] = lo;
        x->row_lo[r + 1] = hi;
        most = std::max(most, hi - lo);
    }
    x->slot_floats = ((long long) most * N + 3) / 4 * 4;
    x->bytes = KSHARD_HEADER + (size_t) 2 * world * x->slot_floats * sizeof(float);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, x->bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, KSHARD_HEADER);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess && ipc_handle) {
        static_assert(sizeof(cudaIpcMemHandle_t) == CAKEB200_IPC_HANDLE_BYTES, "size of an IPC handle");
        cudaIpcMemHandle_t h;
        e = cudaIpcGetMemHandle(&h, p);
        if (e == cudaSuccess) memcpy(ipc_handle, &h, sizeof(h));
    }
    if (e != cudaSuccess) {
        set_error("kshard_create: %s", cudaGetErrorString(e));
        if (p) cudaFree(p);
        delete x;
        return CAKEB200_ERR_CUDA;
    }
    x->peer[rank] = (char*) p;
    x->connected = (world == 1);
    *out = x;
    return CAKEB200_OK;
}

int cakeb200_kshard_connect_ipc(cakeb200_kshard* x, const unsigned char* handles) {
    if (!x || !handles) {
        set_error("kshard_connect_ipc: null argument");
        return CAKEB200_ERR_ARG;
    }
    for (int r = 0; r < x->world; r++) {
        if (r == x->rank || x->peer[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t) r * CAKEB200_IPC_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        CAKE_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        x->peer[r] = (char*) p;
        x->ipc_opened[r] = true;
    }
    x->connected = true;
    return CAKEB200_OK;
}

int cakeb200_kshard_connect_local(cakeb200_kshard* x, cakeb200_kshard* const* all) {
    if (!x || !all) {
        set_error("kshard_connect_local: null argument");
        return CAKEB200_ERR_ARG;
    }
    for (int r = 0; r < x->world; r++) {
        if (!all[r] || all[r]->world != x->world || all[r]->rank != r || all[r]->M != x->M || all[r]->N != x->N ||
            all[r]->device != x->device) {
            set_error("kshard_connect_local: object %d does not belong to this product", r);
            return CAKEB200_ERR_ARG;
        }
        x->peer[r] = all[r]->peer[r];
    }
    x->connected = true;
    return CAKEB200_OK;
}

int cakeb200_kshard_partial(cakeb200_kshard* x, const float* A, int lda, const float* B, int ldb, int K_local, void* stream) {
    g_stats = cakeb200_stats();
    if (!x || !A || !B) {
        set_error("kshard_partial: null argument");
        return CAKEB200_ERR_ARG;
    }
    if (!x->connected) {
        set_error("kshard_partial: the ranks are not connected yet");
        return CAKEB200_ERR_ARG;
    }
    if (x->epoch != x->finished) {
        // the two slot sets alternate by product number: a second product may only start once this rank's
        // rows of the first have been summed, or an owner still reading set (epoch & 1) would be overwritten
        set_error("kshard_partial: the previous product has not been finished (call cakeb200_kshard_finish first)");
        return CAKEB200_ERR_ARG;
    }
    if (bad_dims(x->M, x->N, K_local)) return CAKEB200_ERR_ARG;
    if (lda < K_local || ldb < x->N || !on_device(A) || !on_device(B)) {
        set_error("kshard_partial: needs device operands with lda >= K and ldb >= N");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    if (st->device != x->device) {
        set_error("kshard_partial: called on device %d, created on device %d", st->device, x->device);
        return CAKEB200_ERR_ARG;
    }
    if (!tf32x3_all_tiles_in_pieces(x->M, x->N, K_local, CAKEB200_SCHED_KMN, st->sm_count)) {
        set_error("kshard_partial: shape %d x %d x %d is not one this path takes (cakeb200_kshard_supported)", x->M, K_local, x->N);
        return CAKEB200_ERR_ARG;
    }
    cudaStream_t s = (cudaStream_t) stream;
    int rc;
    if ((rc = ensure_scratch(st, tf32x3_scratch_bytes(x->M, x->N, K_local, st->sm_count)))) return rc;
    const int epoch = x->epoch + 1;  // counted only once the launch below has succeeded
    const int set = epoch & 1;
    OwnerSlots os = {};
    os.world = x->world;
    os.epoch = epoch;
    os.done = (unsigned*) (x->peer[x->rank] + KSHARD_DONE_AT);
    for (int o = 0; o < x->world; o++) {
        os.base[o] = (float*) (x->peer[o] + KSHARD_HEADER) + ((long long) set * x->world + x->rank) * x->slot_floats;
        os.flag[o] = (int*) x->peer[o] + x->rank;
        os.row_lo[o] = x->row_lo[o];
    }
    os.row_lo[x->world] = x->row_lo[x->world];
    GemmProblem g = {};
    g.A = A; g.B = B; g.C = nullptr;
    g.M = x->M; g.N = x->N; g.K = K_local;
    g.lda = lda; g.ldb = ldb; g.ldc = x->N;
    g.batch = 1;
    g.order = CAKEB200_SCHED_KMN;
    g.owners = &os;
    g_stats.kernel = CAKEB200_KERNEL_TF32X3;
    g_stats.sched = g.order;
    rc = launch_sgemm_tf32x3(g, st->scratch, st->scratch_bytes, st->status_word, st->sm_count, s, &g_stats, nullptr);
    if (rc == CAKEB200_OK) x->epoch = epoch;  // a failed launch publishes nothing: the peers' count is unchanged
    return rc;
}

int cakeb200_kshard_finish(cakeb200_kshard* x, float* C_block, int wait_limit_us, void* stream) {
    if (!x || x->epoch == x->finished) {
        set_error("kshard_finish: no product in flight");
        return CAKEB200_ERR_ARG;
    }
    const int rows = x->row_lo[x->rank + 1] - x->row_lo[x->rank];
    if (rows > 0 && (!C_block || !on_device(C_block))) {
        set_error("kshard_finish: needs a device pointer for this rank's rows");
        return CAKEB200_ERR_ARG;
    }
    if (wait_limit_us < 0 || wait_limit_us > 60 * 1000000) {
        set_error("kshard_finish: limit must be between 0 (default, 2 s) and 60 s");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;
    const int set = x->epoch & 1;
    const float* slots = (const float*) (x->peer[x->rank] + KSHARD_HEADER) + (long long) set * x->world * x->slot_floats;
    const long long limit_ns = wait_limit_us ? (long long) wait_limit_us * 1000 : 2000000000LL;
    int rc = launch_sum_owner_slots(slots, x->slot_floats, x->world, C_block, (long long) rows * x->N,
                                    (const int*) x->peer[x->rank], x->epoch, limit_ns, st->status_word, st->sm_count, s);
    if (rc) return rc;
    g_stats.launches += 1;
    rc = check_status_word(st, s);
    if (rc == CAKEB200_OK) x->finished = x->epoch;  // after a timeout the product stays open: finish may be called again
    return rc;
}

int cakeb200_kshard_destroy(cakeb200_kshard* x) {
    if (!x) return CAKEB200_OK;
    cudaDeviceSynchronize();
    for (int r = 0; r < x->world; r++)
        if (x->ipc_opened[r]) cudaIpcCloseMemHandle(x->peer[r]);
    if (x->peer[x->rank]) cudaFree(x->peer[x->rank]);
    cudaGetLastError();
    delete x;
    return CAKEB200_OK;
}

int cakeb200_sgemv(const float* A, const float* x, float* y, int M, int K, int col_major, int accumulate, void* stream) {
    g_stats = cakeb200_stats();
    if (!A || !x || !y) {
        set_error("null pointer");
        return CAKEB200_ERR_ARG;
    }
    if (bad_dims(M, 1, K)) return CAKEB200_ERR_ARG;
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;
    Operand oa, ox, oy;
    int rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[0], s));
    if ((rc = stage_in(st, 0, oa, A, (size_t) M * K * 4, true, s))) return rc;
    if ((rc = stage_in(st, 1, ox, x, (size_t) K * 4, true, s))) return rc;
    if ((rc = stage_in(st, 2, oy, y, (size_t) M * 4, accumulate != 0, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[1], s));
    if ((rc = ensure_scratch(st, sgemv_scratch_bytes(M, K, st->sm_count)))) return rc;
    int launches = 0;
    if ((rc = launch_sgemv((const float*) oa.dev, (const float*) ox.dev, (float*) oy.dev, M, K, K, col_major, accumulate ? 1 : 0,
                           st->scratch, st->scratch_bytes, st->sm_count, s, &launches)))
        return rc;
    g_stats.launches = launches;
    g_stats.kernel = CAKEB200_KERNEL_FFMA;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
    if ((rc = stage_out(oy, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[3], s));
    CAKE_CUDA_OK(cudaStreamSynchronize(s));
    g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
    g_stats.ms_gemm = elapsed(st->ev[1], st->ev[2]);
    g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
    return CAKEB200_OK;
}

int cakeb200_sp_sgemm(const float* A, const float* B, float* C, int M, int N, int K, int kernel, void* stream) {
    g_stats = cakeb200_stats();
    if (!A || !B || !C) {
        set_error("null matrix pointer");
        return CAKEB200_ERR_ARG;
    }
    if (bad_dims(M, N, K)) return CAKEB200_ERR_ARG;
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;  // NULL = the CUDA default stream, ordered with the caller's default-stream work
    Operand oa, ob, oc;
    int rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[0], s));
    if ((rc = stage_in(st, 0, oa, A, (size_t) M * K * 4, true, s))) return rc;
    if ((rc = stage_in(st, 1, ob, B, (size_t) K * N * 4, true, s))) return rc;
    if ((rc = stage_in(st, 2, oc, C, (size_t) M * N * 4, false, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[1], s));
    if (kernel != CAKEB200_KERNEL_AUTO && kernel != CAKEB200_KERNEL_TF32X3 && kernel != CAKEB200_KERNEL_FFMA) {
        set_error("unknown kernel id %d", kernel);
        return CAKEB200_ERR_ARG;
    }
    bool dense = kernel == CAKEB200_KERNEL_TF32X3;
    long long nnz = -1;
    if (!dense) {
        if ((rc = ensure_scratch(st, sparse_scratch_bytes(M, K)))) return rc;
        if ((rc = sp_compact((const float*) oa.dev, M, K, st->scratch, st->status_word, s, &nnz, &g_stats.launches)))
            return rc;
        // Skipping zeros pays only when almost everything is zero: the tensor cores multiply the whole
        // matrix faster than the CUDA cores gather rows of B for 3.5 % of it (measured at 8192^3: dense
        // 4.6 ms at any density; zero skipping 0.25 ms + 1.1 ms per percent of nonzeros).
        if (kernel == CAKEB200_KERNEL_AUTO && M >= 256 && N >= 256 && K >= 64 &&
            (double) M * N * K >= (double) (1LL << 27) && (double) nnz > 0.035 * (double) M * (double) K)
            dense = true;
    }
    if (dense) {
        // dense tensor-core product on the operand as given (zeros multiply like any value)
        GemmProblem g = {};
        g.A = (const float*) oa.dev; g.B = (const float*) ob.dev; g.C = (float*) oc.dev;
        g.M = M; g.N = N; g.K = K; g.lda = K; g.ldb = N; g.ldc = N; g.batch = 1;
        g.order = resolve_schedule(st, M, N, K, CAKEB200_SCHED_NA);
        if ((rc = run_dense(st, g, CAKEB200_KERNEL_TF32X3, s, false))) return rc;
    } else {
        if ((rc = sp_multiply((const float*) ob.dev, (float*) oc.dev, M, N, K, st->scratch, nnz, st->status_word, s,
                              &g_stats.launches)))
            return rc;
        g_stats.kernel = CAKEB200_KERNEL_FFMA;
    }
    CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
    if ((rc = stage_out(oc, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[3], s));
    if ((rc = check_status_word(st, s))) return rc;
    g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
    g_stats.ms_gemm = elapsed(st->ev[1], st->ev[2]);
    g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
    return CAKEB200_OK;
}

int cakeb200_im2col(const float* in, float* col, int batch, int cin, int H, int W, int hf, int wf, int stride,
                    int pad, void* stream) {
    g_stats = cakeb200_stats();
    if (!in || !col || batch <= 0 || cin <= 0 || H <= 0 || W <= 0 || hf <= 0 || wf <= 0 || stride <= 0 || pad < 0 ||
        H + 2 * pad < hf || W + 2 * pad < wf) {
        set_error("bad convolution geometry");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;  // NULL = the CUDA default stream, ordered with the caller's default-stream work
    const int Ho = (H + 2 * pad - hf) / stride + 1, Wo = (W + 2 * pad - wf) / stride + 1;
    Operand oi, oc;
    int rc;
    if ((rc = stage_in(st, 0, oi, in, (size_t) batch * cin * H * W * 4, true, s))) return rc;
    if ((rc = stage_in(st, 1, oc, col, (size_t) cin * hf * wf * batch * Ho * Wo * 4, false, s))) return rc;
    if ((rc = launch_im2col((const float*) oi.dev, (float*) oc.dev, batch, cin, H, W, hf, wf, stride, pad, s))) return rc;
    g_stats.launches = 1;
    if ((rc = stage_out(oc, s))) return rc;
    CAKE_CUDA_OK(cudaStreamSynchronize(s));
    return CAKEB200_OK;
}

int cakeb200_conv_plan_query(int batch, int cin, int H, int W, int cout, int hf, int wf, int stride, int pad, int sm_count,
                             cakeb200_conv_plan* out) {
    if (!out || batch <= 0 || cin <= 0 || cout <= 0 || H <= 0 || W <= 0 || hf <= 0 || wf <= 0 || stride <= 0 || pad < 0 ||
        H + 2 * pad < hf || W + 2 * pad < wf) {
        set_error("bad convolution geometry");
        return CAKEB200_ERR_ARG;
    }
    return conv_tf32x3_describe(batch, cin, H, W, cout, hf, wf, stride, pad, sm_count, out);
}

int cakeb200_conv2d(const float* in, const float* filters, float* out, int batch, int cin, int H, int W, int cout,
                    int hf, int wf, int stride, int pad, int kernel, void* stream) {
    g_stats = cakeb200_stats();
    if (!in || !filters || !out || batch <= 0 || cin <= 0 || cout <= 0 || H <= 0 || W <= 0 || hf <= 0 || wf <= 0 ||
        stride <= 0 || pad < 0 || H + 2 * pad < hf || W + 2 * pad < wf) {
        set_error("bad convolution geometry");
        return CAKEB200_ERR_ARG;
    }
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    cudaStream_t s = (cudaStream_t) stream;  // NULL = the CUDA default stream, ordered with the caller's default-stream work
    const int Ho = (H + 2 * pad - hf) / stride + 1, Wo = (W + 2 * pad - wf) / stride + 1;
    const int Kg = cin * hf * wf;
    const long long plane = (long long) Ho * Wo, Ng = plane * batch;
    if (Ng > INT_MAX) {
        set_error("im2col matrix has more than 2^31-1 columns");
        return CAKEB200_ERR_TOO_LARGE;
    }
    Operand oi, of, oo;
    int rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[0], s));
    if ((rc = stage_in(st, 0, oi, in, (size_t) batch * cin * H * W * 4, true, s))) return rc;
    if ((rc = stage_in(st, 1, of, filters, (size_t) cout * Kg * 4, true, s))) return rc;
    if ((rc = stage_in(st, 2, oo, out, (size_t) batch * cout * plane * 4, false, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[1], s));

    const bool tensor = kernel == CAKEB200_KERNEL_TF32X3 ||
                        (kernel == CAKEB200_KERNEL_AUTO && cout >= 32 && Kg >= 32 && Ng >= 512 &&
                         (double) cout * Kg * Ng >= (double) (1LL << 27));
    if (kernel != CAKEB200_KERNEL_AUTO && kernel != CAKEB200_KERNEL_TF32X3 && kernel != CAKEB200_KERNEL_FFMA) {
        set_error("unknown kernel id %d", kernel);
        return CAKEB200_ERR_ARG;
    }
    if (tensor && option_get(OPT_CONV_ROUTE) != 1 &&
        conv_tf32x3_fits((const float*) oi.dev, batch, cin, H, W, cout, hf, wf, stride, pad)) {
        // Implicit product: input rows come on chip by TMA, the patch operand is built in shared memory
        if ((rc = ensure_scratch(st, conv_tf32x3_scratch_bytes(cin, cout, hf, wf)))) return rc;
        int launches = 0;
        if ((rc = launch_conv_tf32x3((const float*) oi.dev, (const float*) of.dev, (float*) oo.dev, nullptr, batch, cin, H, W,
                                     cout, hf, wf, pad, st->scratch, st->scratch_bytes, st->status_word, st->sm_count, s,
                                     &launches)))
            return rc;
        g_stats.launches += launches;
        g_stats.kernel = CAKEB200_KERNEL_TF32X3;
        g_stats.tile_m = 128; g_stats.tile_n = cout >= 128 ? 128 : (cout + 15) / 16 * 16; g_stats.tile_k = 32;
        CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
        if ((rc = stage_out(oo, s))) return rc;
        CAKE_CUDA_OK(cudaEventRecord(st->ev[3], s));
        if ((rc = check_status_word(st, s))) return rc;
        g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
        g_stats.ms_gemm = elapsed(st->ev[1], st->ev[2]);
        g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
        g_stats.ms_prepass = 0.f;
        return CAKEB200_OK;
    }
    if (tensor) {
        // Tensor-core route for the other geometries (strides, very wide images): the filters are the A operand
        Tf32x3Planes planes;
        if ((rc = ensure_scratch(st, tf32x3_plane_bytes(cout, (int) Ng, Kg, st->sm_count)))) return rc;
        if ((rc = tf32x3_planes(cout, (int) Ng, Kg, st->scratch, st->scratch_bytes, &planes, st->sm_count))) return rc;
        if ((rc = tf32x3_split_A_rows((const float*) of.dev, Kg, 0, cout, Kg, planes, st->sm_count, s))) return rc;
        if ((rc = tf32x3_split_im2col((const float*) oi.dev, batch, cin, H, W, hf, wf, stride, pad, planes, st->sm_count, s)))
            return rc;
        if ((rc = tf32x3_multiply_rows(planes, (float*) oo.dev, (int) plane, 0, cout, (int) Ng, Kg, CAKEB200_SCHED_NKM, 0,
                                       st->status_word, st->sm_count, s, (int) plane, (long long) cout * plane)))
            return rc;
        g_stats.launches += 3;
        g_stats.kernel = CAKEB200_KERNEL_TF32X3;
        g_stats.tile_m = 128; g_stats.tile_n = Ng > 128 ? 256 : 128; g_stats.tile_k = 32;
        CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
        if ((rc = stage_out(oo, s))) return rc;
        CAKE_CUDA_OK(cudaEventRecord(st->ev[3], s));
        if ((rc = check_status_word(st, s))) return rc;
        g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
        g_stats.ms_gemm = elapsed(st->ev[1], st->ev[2]);
        g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
        return CAKEB200_OK;
    }

    // FFMA route: the im2col matrix lives in the scratch arena.
    const size_t col_bytes = (size_t) Kg * Ng * 4;
    if ((rc = ensure_scratch(st, col_bytes))) return rc;
    float* col = (float*) st->scratch;
    if ((rc = launch_im2col((const float*) oi.dev, col, batch, cin, H, W, hf, wf, stride, pad, s))) return rc;
    g_stats.launches++;

    // One strided product per image: out[b] (cout x Ho*Wo) = F (cout x Kg) * col[:, b*Ho*Wo ...]
    GemmProblem g = {};
    g.A = (const float*) of.dev; g.B = col; g.C = (float*) oo.dev;
    g.M = cout; g.N = (int) plane; g.K = Kg;
    g.lda = Kg; g.ldb = (int) Ng; g.ldc = (int) plane;
    g.stride_a = 0; g.stride_b = plane; g.stride_c = (long long) cout * plane;
    g.order = CAKEB200_SCHED_MKN;
    for (int done = 0; done < batch; done += 65535) {
        GemmProblem part = g;
        part.batch = std::min(65535, batch - done);
        part.B += (long long) done * g.stride_b;
        part.C += (long long) done * g.stride_c;
        if ((rc = launch_sgemm_ffma(part, s))) return rc;
        g_stats.launches++;
    }
    g_stats.kernel = CAKEB200_KERNEL_FFMA;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[2], s));
    if ((rc = stage_out(oo, s))) return rc;
    CAKE_CUDA_OK(cudaEventRecord(st->ev[3], s));
    CAKE_CUDA_OK(cudaStreamSynchronize(s));
    g_stats.ms_h2d = elapsed(st->ev[0], st->ev[1]);
    g_stats.ms_gemm = elapsed(st->ev[1], st->ev[2]);
    g_stats.ms_d2h = elapsed(st->ev[2], st->ev[3]);
    return CAKEB200_OK;
}

int cakeb200_pack_A(const float* A, float* A_p, int M, int K, int p, const cakeb200_blk_dims* x,
                    const cakeb200_cntx* c, void* stream) {
    if (!x || !c) return CAKEB200_ERR_ARG;
    return pack_impl(pack_A_dev, A, (size_t) M * K * 4, A_p, cakeb200_packed_A_size(M, K, p, x, c, x->sch), M, K, p, x, c, false, stream);
}
int cakeb200_unpack_A(float* A, const float* A_p, int M, int K, int p, const cakeb200_blk_dims* x,
                      const cakeb200_cntx* c, void* stream) {
    if (!x || !c) return CAKEB200_ERR_ARG;
    return pack_impl(pack_A_dev, A, (size_t) M * K * 4, (float*) A_p, cakeb200_packed_A_size(M, K, p, x, c, x->sch), M, K, p, x, c, true, stream);
}
int cakeb200_pack_B(const float* B, float* B_p, int K, int N, int p, const cakeb200_blk_dims* x,
                    const cakeb200_cntx* c, void* stream) {
    if (!x || !c) return CAKEB200_ERR_ARG;
    return pack_impl(pack_B_dev, B, (size_t) K * N * 4, B_p, cakeb200_packed_B_size(K, N, p, x, c), K, N, p, x, c, false, stream);
}
int cakeb200_unpack_B(float* B, const float* B_p, int K, int N, int p, const cakeb200_blk_dims* x,
                      const cakeb200_cntx* c, void* stream) {
    if (!x || !c) return CAKEB200_ERR_ARG;
    return pack_impl(pack_B_dev, B, (size_t) K * N * 4, (float*) B_p, cakeb200_packed_B_size(K, N, p, x, c), K, N, p, x, c, true, stream);
}
int cakeb200_pack_C(const float* C, float* C_p, int M, int N, int p, const cakeb200_blk_dims* x,
                    const cakeb200_cntx* c, void* stream) {
    if (!x || !c) return CAKEB200_ERR_ARG;
    return pack_impl(pack_C_dev, C, (size_t) M * N * 4, C_p, cakeb200_packed_C_size(M, N, p, x, c, x->sch), M, N, p, x, c, false, stream);
}
int cakeb200_unpack_C(float* C, const float* C_p, int M, int N, int p, const cakeb200_blk_dims* x,
                      const cakeb200_cntx* c, void* stream) {
    if (!x || !c) return CAKEB200_ERR_ARG;
    return pack_impl(pack_C_dev, C, (size_t) M * N * 4, (float*) C_p, cakeb200_packed_C_size(M, N, p, x, c, x->sch), M, N, p, x, c, true, stream);
}

}  // extern "C"
