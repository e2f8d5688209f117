// im2col for NCHW input: builds the K x N operand of the convolution-as-GEMM
// route (reference examples/cake_conv.cpp:1178-1213), extended with a batch
// dimension, stride and zero padding.  Row index k = (cin, hf, wf); column
// index n = (b, ho, wo).  One thread per output element, n fastest, so writes
// are fully coalesced and reads are contiguous runs of the input rows.
#include "common.cuh"

namespace cakeb200 {
namespace {

__global__ void __launch_bounds__(256)
im2col_kernel(const float* __restrict__ in, float* __restrict__ col, int batch, int cin, int H, int W,
              int hf, int wf, int stride, int pad, int Ho, int Wo) {
    const long long ncol = (long long) batch * Ho * Wo;
    const long long total = (long long) cin * hf * wf * ncol;
    for (long long idx = (long long) blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long) gridDim.x * blockDim.x) {
        const long long k = idx / ncol, n = idx - k * ncol;
        const int fw = (int) (k % wf), fh = (int) ((k / wf) % hf), ci = (int) (k / (wf * hf));
        const int wo = (int) (n % Wo), ho = (int) ((n / Wo) % Ho), b = (int) (n / ((long long) Wo * Ho));
        const int h = ho * stride - pad + fh, w = wo * stride - pad + fw;
        float v = 0.0f;
        if (h >= 0 && h < H && w >= 0 && w < W) v = __ldg(in + (((long long) b * cin + ci) * H + h) * W + w);
        col[idx] = v;
    }
}

}  // namespace

int launch_im2col(const float* in, float* col, int batch, int cin, int H, int W, int hf, int wf,
                  int stride, int pad, cudaStream_t stream) {
    const int Ho = (H + 2 * pad - hf) / stride + 1, Wo = (W + 2 * pad - wf) / stride + 1;
    const long long total = (long long) cin * hf * wf * batch * Ho * Wo;
    if (total <= 0) return CAKEB200_OK;
    DeviceState* st = device_state();
    if (!st) return CAKEB200_ERR_NO_DEVICE;
    const int blocks = (int) std::min<long long>((total + 255) / 256, (long long) st->sm_count * 64);
    im2col_kernel<<<blocks, 256, 0, stream>>>(in, col, batch, cin, H, W, hf, wf, stride, pad, Ho, Wo);
    CAKE_CUDA_OK(cudaGetLastError());
    return CAKEB200_OK;
}

}  // namespace cakeb200
