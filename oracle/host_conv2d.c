/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the sparse-filter convolution path.
 *
 * A plain-C restatement of the CPU direct convolution, tolerance compare and
 * layout transposes that the Tetris artifact uses to check its GPU kernel.
 * Nothing in the shipped library links, loads or calls this file: only the
 * tests, the smoke check and the CPU-baseline leg of the benchmark do, and
 * only as the checker.
 *
 * Parity pin: the reference holds no golden vectors for this path.  This port
 * is pinned against the reference's own tensor_utils.cc compiled unchanged
 * into oracle/_ref/libtetris_ref.so (see oracle/Makefile) -- bit-exact on
 * seeded inputs -- and against the fixtures under tests/golden/ that were
 * produced by that compiled reference.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (no -ffast-math, no
 * -mfma: every multiply and every add must round to FP32 on its own, as the
 * reference's x86-64 build does).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Output extent of a convolution; Tetris/tensor_utils.cc:140-141. */
static int out_extent(int in, int pad, int ks, int stride) {
  return (in + 2 * pad - ks) / stride + 1;
}

/*
 * One output plane (n, oc) of the reference's HostConv2d.
 * Follows Tetris/tensor_utils.cc:147-163: the output element is zeroed, then
 * taps are added in (ic, x, y) order straight into the FP32 output element;
 * taps that fall into the zero padding are skipped (tensor_utils.cc:155-156).
 * Zero weights are NOT skipped by the reference; `skip_zero` may skip them,
 * which cannot change any bit of the result: adding a product that is +/-0 to
 * an accumulator that is never -0 leaves it as it was.
 */
static void conv_plane(const float *in_n, const float *filt_oc, float *out_plane,
                       int img_h, int img_w, int in_channel, int ks, int stride,
                       int padding, int out_h, int out_w, int skip_zero) {
  for (int h = 0; h < out_h; ++h) {
    for (int w = 0; w < out_w; ++w) {
      float *o = &out_plane[(size_t)h * out_w + w];
      *o = 0.f;
      for (int ic = 0; ic < in_channel; ++ic) {
        const float *plane = in_n + (size_t)ic * img_h * img_w;
        const float *f = filt_oc + (size_t)ic * ks * ks;
        for (int x = 0; x < ks; ++x) {
          int ih = h * stride + x;
          if (ih < padding || ih >= img_h + padding) continue;
          for (int y = 0; y < ks; ++y) {
            int iw = w * stride + y;
            if (iw < padding || iw >= img_w + padding) continue;
            float wt = f[x * ks + y];
            if (skip_zero && wt == 0.f) continue;
            *o += plane[(size_t)(ih - padding) * img_w + (iw - padding)] * wt;
          }
        }
      }
    }
  }
}

/*
 * HostConv2d, Tetris/tensor_utils.cc:136-170.  NCHW input, OIHW filter, NCHW
 * output, single thread, loop nest n, oc, h, w, ic, x, y exactly as there.
 */
void oracle_host_conv2d(const float *input, const float *filter, float *output,
                        int batch_size, int img_h, int img_w, int in_channel,
                        int out_channel, int kernel_size, int stride, int padding) {
  int out_h = out_extent(img_h, padding, kernel_size, stride);
  int out_w = out_extent(img_w, padding, kernel_size, stride);
  for (int n = 0; n < batch_size; ++n)
    for (int oc = 0; oc < out_channel; ++oc)
      conv_plane(input + (size_t)n * in_channel * img_h * img_w,
                 filter + (size_t)oc * in_channel * kernel_size * kernel_size,
                 output + ((size_t)n * out_channel + oc) * out_h * out_w, img_h, img_w,
                 in_channel, kernel_size, stride, padding, out_h, out_w, 0);
}

/*
 * The same arithmetic spread over host threads: one (n, oc) output plane per
 * task.  Each output element is still produced by one thread in the
 * reference's (ic, x, y) order, so the result is bit-identical to
 * oracle_host_conv2d.  `skip_zero` != 0 skips zero weights (bit-identical, see
 * conv_plane) and is what makes model-sized checks affordable.
 */
void oracle_host_conv2d_mt(const float *input, const float *filter, float *output,
                           int batch_size, int img_h, int img_w, int in_channel,
                           int out_channel, int kernel_size, int stride, int padding,
                           int skip_zero) {
  int out_h = out_extent(img_h, padding, kernel_size, stride);
  int out_w = out_extent(img_w, padding, kernel_size, stride);
  long tasks = (long)batch_size * out_channel;
#pragma omp parallel for schedule(dynamic, 1)
  for (long t = 0; t < tasks; ++t) {
    int n = (int)(t / out_channel), oc = (int)(t % out_channel);
    conv_plane(input + (size_t)n * in_channel * img_h * img_w,
               filter + (size_t)oc * in_channel * kernel_size * kernel_size,
               output + ((size_t)n * out_channel + oc) * out_h * out_w, img_h, img_w,
               in_channel, kernel_size, stride, padding, out_h, out_w, skip_zero);
  }
}

/*
 * Depthwise convolution (groups == channels; filter is [C][1][KS][KS]).  The
 * reference reads `groups` from the layer file and ignores it
 * (Tetris/tensor_utils.cc:66, Tetris/spconv2d.cc:404-406), so there is no
 * grouped code to restate.  The oracle is HostConv2d applied to each (n, c)
 * plane as a 1-in 1-out convolution, which on NCHW planes is exact.
 */
void oracle_host_depthwise_conv2d(const float *input, const float *filter, float *output,
                                  int batch_size, int img_h, int img_w, int channels,
                                  int kernel_size, int stride, int padding) {
  int out_h = out_extent(img_h, padding, kernel_size, stride);
  int out_w = out_extent(img_w, padding, kernel_size, stride);
  long tasks = (long)batch_size * channels;
#pragma omp parallel for schedule(dynamic, 4)
  for (long t = 0; t < tasks; ++t) {
    int c = (int)(t % channels);
    conv_plane(input + (size_t)t * img_h * img_w, filter + (size_t)c * kernel_size * kernel_size,
               output + (size_t)t * out_h * out_w, img_h, img_w, 1, kernel_size, stride,
               padding, out_h, out_w, 0);
  }
}

/* FloatEqual, Tetris/tensor_utils.cc:17-19 (the arithmetic there is double). */
int oracle_float_equal(float x, float y) {
  return fabs((double)x - (double)y) <= 1e-5 * (fabs((double)x) + fabs((double)y)) + 1e-5;
}

/*
 * TensorEqual, Tetris/tensor_utils.cc:21-34: index of the first element that
 * fails FloatEqual, or -1 when all pass (the reference prints it and returns
 * false).
 */
long oracle_tensor_first_mismatch(const float *x, const float *y, size_t len) {
  for (size_t i = 0; i < len; ++i)
    if (!oracle_float_equal(x[i], y[i])) return (long)i;
  return -1;
}

/*
 * The acceptance check of this build: |x - y| <= rel * max(|x|, |y|) + abs_floor.
 * Returns the number of failing elements; *max_rel gets the largest relative
 * error over elements with |ref| > abs_floor, *n_floor the number of elements
 * that passed only thanks to the absolute floor.
 */
long oracle_tensor_compare(const float *got, const float *ref, size_t len, double rel,
                           double abs_floor, double *max_rel, long *n_floor) {
  long bad = 0, fl = 0;
  double mr = 0.0;
  for (size_t i = 0; i < len; ++i) {
    double a = got[i], b = ref[i], d = fabs(a - b);
    double m = fabs(a) > fabs(b) ? fabs(a) : fabs(b);
    if (!(d <= rel * m + abs_floor)) { ++bad; continue; }
    if (fabs(b) > abs_floor) { double r = d / fabs(b); if (r > mr) mr = r; }
    if (d > rel * m) ++fl;
  }
  if (max_rel) *max_rel = mr;
  if (n_floor) *n_floor = fl;
  return bad;
}

/* NCHW2NHWC / NHWC2NCHW, Tetris/tensor_utils.cc:85-111 (out of place here). */
void oracle_nchw_to_nhwc(const float *src, float *dst, int N, int C, int H, int W) {
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int h = 0; h < H; ++h)
        for (int w = 0; w < W; ++w)
          dst[(((size_t)n * H + h) * W + w) * C + c] = src[(((size_t)n * C + c) * H + h) * W + w];
}

void oracle_nhwc_to_nchw(const float *src, float *dst, int N, int C, int H, int W) {
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int h = 0; h < H; ++h)
        for (int w = 0; w < W; ++w)
          dst[(((size_t)n * C + c) * H + h) * W + w] = src[(((size_t)n * H + h) * W + w) * C + c];
}
