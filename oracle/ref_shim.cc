// TEST INFRASTRUCTURE ONLY.  C-callable doors into the reference's own CPU code.
//
// Compiled together with the reference's Tetris/tensor_utils.cc, taken where it
// lies in the reference checkout (never copied into this repository), into
// oracle/_ref/libtetris_ref.so.  The tests use it to pin the C restatement in
// host_conv2d.c and to generate tests/golden/; the benchmark may time it as the
// CPU baseline.  Nothing in the shipped library touches it.
#include <cstddef>
#include <vector>
#include <cstring>
#include "tensor_utils.h"  // the reference's header, found through -I

extern "C" {

// Tetris/tensor_utils.cc:136-170
void ref_host_conv2d(float *input, float *filter, float *output, int batch_size, int img_h,
                     int img_w, int in_channel, int out_channel, int kernel_size, int stride,
                     int padding) {
  HostConv2d(input, filter, output, batch_size, img_h, img_w, in_channel, out_channel,
             kernel_size, stride, padding);
}

// Tetris/tensor_utils.cc:17-19
int ref_float_equal(float x, float y) { return FloatEqual(x, y) ? 1 : 0; }

// Tetris/tensor_utils.cc:85-111 (in place, as the reference does it)
void ref_nchw_to_nhwc(float *t, int N, int C, int H, int W) { NCHW2NHWC(t, N, C, H, W); }
void ref_nhwc_to_nchw(float *t, int N, int C, int H, int W) { NHWC2NCHW(t, N, C, H, W); }
void ref_kcrs_to_krsc(float *t, int K, int C, int R, int S) { KCRS2KRSC(t, K, C, R, S); }
void ref_krsc_to_kcrs(float *t, int K, int C, int R, int S) { KRSC2KCRS(t, K, C, R, S); }

// Tetris/tensor_utils.cc:55-82.  Returns the malloc'd filter; the caller frees it
// with ref_free.  The header values come back through `cfg[8]` in file order:
// H W IC OC KS Pad S G.
float *ref_read_layer_file(const char *path, int batch_size, int *cfg) {
  int h, w, ic, oc, ks, s, p, g;
  float *f = ReadConfigAndDataFromFile(path, batch_size, "NHWC", h, w, ic, oc, ks, s, p, g);
  cfg[0] = h; cfg[1] = w; cfg[2] = ic; cfg[3] = oc; cfg[4] = ks; cfg[5] = p; cfg[6] = s; cfg[7] = g;
  return f;
}
void ref_free(void *p) { free(p); }

}  // extern "C"
