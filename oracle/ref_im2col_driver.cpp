/* TEST INFRASTRUCTURE ONLY: calls the reference's im_2_col (reference examples/cake_conv.cpp:1178-1213),
 * cut out of the stand-alone convolution example into oracle/_ref/ by oracle/Makefile, so that the
 * oracle's im2col restatement (k = (cin, hf, wf), n = (ho, wo)) can be pinned against it for the
 * case the reference covers: one image, no padding, stride 1 (its `s` argument is not used in the
 * index arithmetic).  Forwards only. */
#include <cstdlib>
#include <cstring>

float* im_2_col(float* In, int Wf, int Hf, int Win, int Hin, int Wout, int Hout, int Cin, int Cout, int s);

extern "C" int ref_im_2_col(const float* in, float* col, int cin, int H, int W, int hf, int wf) {
    const int Ho = H - hf + 1, Wo = W - wf + 1;
    float* mat = im_2_col(const_cast<float*>(in), wf, hf, W, H, Wo, Ho, cin, 0, 1);
    if (!mat) return -1;
    memcpy(col, mat, (size_t) cin * hf * wf * Ho * Wo * sizeof(float));
    free(mat);
    return 0;
}
