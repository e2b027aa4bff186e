// Host-side tensor helpers with the names and argument lists of the reference's tensor_utils.h
// (Tetris/tensor_utils.h:13-46), so host programs written against it compile unchanged.
// The implementations are this project's own (tensor_utils.cc here); the random generator is
// seedable instead of rand().
#ifndef TETRIS_B200_HOST_TENSOR_UTILS_H_
#define TETRIS_B200_HOST_TENSOR_UTILS_H_

#include <cstddef>
#include <cstdint>
#include <iostream>
#include <string>

// Timing protocol of the reference harness (Tetris/tensor_utils.h:10-11).
#ifndef REPEAT
#define REPEAT 100
#endif
#ifndef WARM
#define WARM 30
#endif

// Seeds RandFloat / GenRandTensor (the reference seeds rand() with the wall clock).
void SeedRand(uint64_t seed);

// Uniform in [-1, 1).
float RandFloat();

// |x - y| <= 1e-5 * (|x| + |y|) + 1e-5
bool FloatEqual(float x, float y);

// True when every element pair passes FloatEqual; prints the first mismatch otherwise.
bool TensorEqual(float *tensor_x, float *tensor_y, size_t len);

void GenRandTensor(float *tensor, size_t len);

void PrintConv2dConfig(int64_t nnz, int batch_size, std::string layout, int img_h, int img_w,
                       int in_channel, int out_channel, int kernel_size, int stride, int padding,
                       int groups);

// Reads a layer dump: header "H W IC OC KS Pad S G", then OC*IC*KS*KS floats (OIHW).  Returns a
// malloc'd filter the caller frees; prints the [Config] line; exits with status 1 if the file
// cannot be opened.
float *ReadConfigAndDataFromFile(std::string weight_file, int batch_size, std::string layout,
                                 int &img_h, int &img_w, int &in_channel, int &out_channel,
                                 int &kernel_size, int &stride, int &padding, int &groups);

// In-place layout changes of a host tensor.
void NCHW2NHWC(float *src, int N, int C, int H, int W);
void NHWC2NCHW(float *src, int N, int C, int H, int W);
// Filter layouts: K output maps, C input maps, R x S taps.
void KCRS2KRSC(float *src, int K, int C, int R, int S);
void KRSC2KCRS(float *src, int K, int C, int R, int S);

// Direct convolution on the host: NCHW input, OIHW filter, NCHW output, zero padding, taps
// accumulated in (ic, kernel row, kernel column) order into the FP32 output element.
void HostConv2d(float *input, float *filter, float *output, int batch_size, int img_h, int img_w,
                int in_channel, int out_channel, int kernel_size, int stride, int padding);

#endif  // TETRIS_B200_HOST_TENSOR_UTILS_H_
