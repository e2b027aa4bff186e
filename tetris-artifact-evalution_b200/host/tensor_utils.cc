// Implementations for tensor_utils.h.  Semantics follow the reference (Tetris/tensor_utils.cc);
// the code is written for this project: a permutation helper serves all four layout changes and
// the convolution walks output planes with precomputed tap ranges instead of per-tap bounds tests.
#include "tensor_utils.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <random>
#include <vector>

namespace {

std::mt19937_64 &Engine() {
  static std::mt19937_64 engine(0x7e7215ULL);
  return engine;
}

// dst[a][c][b] = src[a][b][c] for `outer` blocks of a [rows][cols] matrix, through a copy.
void TransposeBlocks(float *data, size_t outer, size_t rows, size_t cols) {
  std::vector<float> copy(data, data + outer * rows * cols);
  for (size_t a = 0; a < outer; ++a) {
    const float *in = copy.data() + a * rows * cols;
    float *out = data + a * rows * cols;
    for (size_t r = 0; r < rows; ++r)
      for (size_t c = 0; c < cols; ++c) out[c * rows + r] = in[r * cols + c];
  }
}

}  // namespace

void SeedRand(uint64_t seed) { Engine().seed(seed); }

float RandFloat() {
  // 24 random bits -> [0, 1) exactly representable, then stretched to [-1, 1)
  const uint32_t bits = static_cast<uint32_t>(Engine()() >> 40);
  return static_cast<float>(bits) * (2.0f / 16777216.0f) - 1.0f;
}

bool FloatEqual(float x, float y) {
  const double dx = x, dy = y;
  return std::fabs(dx - dy) <= 1e-5 * (std::fabs(dx) + std::fabs(dy)) + 1e-5;
}

bool TensorEqual(float *tensor_x, float *tensor_y, size_t len) {
  for (size_t i = 0; i < len; ++i) {
    if (FloatEqual(tensor_x[i], tensor_y[i])) continue;
    std::cout << "pos = " << i << ", value_x = " << tensor_x[i] << ", value_y = " << tensor_y[i]
              << "\n";
    return false;
  }
  return true;
}

void GenRandTensor(float *tensor, size_t len) {
  std::generate(tensor, tensor + len, RandFloat);
}

void PrintConv2dConfig(int64_t nnz, int batch_size, std::string /*layout*/, int img_h, int img_w,
                       int in_channel, int out_channel, int kernel_size, int stride, int padding,
                       int /*groups*/) {
  const int64_t dense = (int64_t)out_channel * in_channel * kernel_size * kernel_size;
  std::cout << "[Config] sparsity = " << (1.0 - (double)nnz / (double)dense) << ", nnz = " << nnz
            << ", batch_size = " << batch_size << ", img_h = " << img_h << ", img_w = " << img_w
            << ", in_channel = " << in_channel << ", out_channel = " << out_channel
            << ", kernel_size = " << kernel_size << ", padding = " << padding
            << ", stride = " << stride << "\n\n";
}

float *ReadConfigAndDataFromFile(std::string weight_file, int batch_size, std::string layout,
                                 int &img_h, int &img_w, int &in_channel, int &out_channel,
                                 int &kernel_size, int &stride, int &padding, int &groups) {
  std::ifstream in(weight_file);
  if (!in) {
    std::cout << "Open file error.\n";
    std::exit(1);
  }
  in >> img_h >> img_w >> in_channel >> out_channel >> kernel_size >> padding >> stride >> groups;
  const size_t count = (size_t)out_channel * in_channel * kernel_size * kernel_size;
  float *filter = static_cast<float *>(std::malloc(count * sizeof(float)));
  int64_t nnz = 0;
  for (size_t i = 0; i < count; ++i) {
    float v = 0.f;
    in >> v;
    filter[i] = v;
    nnz += v != 0.f;
  }
  PrintConv2dConfig(nnz, batch_size, layout, img_h, img_w, in_channel, out_channel, kernel_size,
                    stride, padding, groups);
  return filter;
}

void NCHW2NHWC(float *src, int N, int C, int H, int W) { TransposeBlocks(src, N, C, (size_t)H * W); }
void NHWC2NCHW(float *src, int N, int C, int H, int W) { TransposeBlocks(src, N, (size_t)H * W, C); }
void KCRS2KRSC(float *src, int K, int C, int R, int S) { TransposeBlocks(src, K, C, (size_t)R * S); }
void KRSC2KCRS(float *src, int K, int C, int R, int S) { TransposeBlocks(src, K, (size_t)R * S, C); }

void HostConv2d(float *input, float *filter, float *output, int batch_size, int img_h, int img_w,
                int in_channel, int out_channel, int kernel_size, int stride, int padding) {
  const int out_h = (img_h + 2 * padding - kernel_size) / stride + 1;
  const int out_w = (img_w + 2 * padding - kernel_size) / stride + 1;
  const size_t plane = (size_t)img_h * img_w, taps = (size_t)kernel_size * kernel_size;
  for (int n = 0; n < batch_size; ++n) {
    const float *image = input + (size_t)n * in_channel * plane;
    for (int oc = 0; oc < out_channel; ++oc) {
      const float *weights = filter + (size_t)oc * in_channel * taps;
      float *out_plane = output + ((size_t)n * out_channel + oc) * out_h * out_w;
      for (int oh = 0; oh < out_h; ++oh) {
        // taps that stay inside the image for this output row / column
        const int top = oh * stride - padding;
        const int r_lo = std::max(0, -top), r_hi = std::min(kernel_size, img_h - top);
        for (int ow = 0; ow < out_w; ++ow) {
          const int left = ow * stride - padding;
          const int s_lo = std::max(0, -left), s_hi = std::min(kernel_size, img_w - left);
          float acc = 0.f;
          for (int ic = 0; ic < in_channel; ++ic) {
            const float *x = image + ic * plane;
            const float *w = weights + ic * taps;
            for (int r = r_lo; r < r_hi; ++r)
              for (int s = s_lo; s < s_hi; ++s)
                acc += x[(size_t)(top + r) * img_w + (left + s)] * w[r * kernel_size + s];
          }
          out_plane[(size_t)oh * out_w + ow] = acc;
        }
      }
    }
  }
}
