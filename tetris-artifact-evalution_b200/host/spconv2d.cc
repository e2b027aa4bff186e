// spconv2d_test: the per-layer program of the reference (Tetris/spconv2d.cc:369-450) on the
// B200 engine.  Same contract:
//
//     spconv2d_test <weight_file> [batch]
//
// reads a layer dump (header "H W IC OC KS Pad S G" + OIHW floats), draws a random input, runs
// the sparse convolution and prints the lines the reference's Python drivers scrape
// (evalution/conv2d_timing.py:51-65):
//
//     [Config] sparsity = ..., nnz = ..., batch_size = ..., ...
//     Time of Spconv2d :<ms>ms
//     FLOPS of Spconv2d :<dense-equivalent binary TFLOP/s>T
//
// The reference compiles its self-check out (#define BENCHMARK); here it runs when the
// environment variable TETRIS_CHECK is set, and prints "Sparse Pass." / "Sparse Error." after
// comparing with HostConv2d under TensorEqual.  TETRIS_SEED fixes the random input.
#include <cuda_runtime.h>

#include <cassert>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <iostream>
#include <string>

#include "cuda_utils.h"
#include "spconv2d_kernel.cuh"
#include "spconv2d_utils.h"
#include "tensor_utils.h"

int main(int argc, char *argv[]) {
  std::cout << "args : " << argc;
  for (int i = 0; i < argc; ++i) std::cout << " " << argv[i];
  std::cout << "\n\n";
  assert(argc <= 3);

  const char *seed = std::getenv("TETRIS_SEED");
  SeedRand(seed ? std::strtoull(seed, nullptr, 10) : (uint64_t)std::time(nullptr));

  const int dev_id = 0;
  cudaDeviceProp prop;
  checkCudaErrors(cudaSetDevice(dev_id));
  checkCudaErrors(cudaGetDeviceProperties(&prop, dev_id));
  std::printf("GPU Device %d: \"%s\" with compute capability %d.%d\n\n", dev_id, prop.name, prop.major,
              prop.minor);

  const std::string layout = "NHWC";
  const int batch_size = argc >= 3 ? std::atoi(argv[2]) : 4;
  const std::string weight_file =
      argc >= 2 ? argv[1]
                : "./conv_weight_data/vgg19/vgg19-92-acc-71.7/"
                  "module8_0_module2_0_conv2d_3_H_56_W_56_IC_256_OC_256_KS_3_Pad_1_S_1_G_1";

  int img_h, img_w, in_channel, out_channel, kernel_size, stride, padding, groups;
  float *h_filter = ReadConfigAndDataFromFile(weight_file, batch_size, layout, img_h, img_w, in_channel,
                                              out_channel, kernel_size, stride, padding, groups);
  const int out_h = (img_h + padding * 2 - kernel_size) / stride + 1;
  const int out_w = (img_w + padding * 2 - kernel_size) / stride + 1;
  const size_t in_count = (size_t)batch_size * in_channel * img_h * img_w;
  const size_t out_count = (size_t)batch_size * out_channel * out_h * out_w;

  float *h_input = static_cast<float *>(std::malloc(in_count * sizeof(float)));
  float *h_sparse = static_cast<float *>(std::malloc(out_count * sizeof(float)));
  GenRandTensor(h_input, in_count);

  cudaStream_t cuda_stream;
  checkCudaErrors(cudaStreamCreate(&cuda_stream));
  CudaSparseConv2d<float, int, int>(h_input, h_filter, h_sparse, batch_size, img_h, img_w, in_channel,
                                    out_channel, kernel_size, stride, padding, cuda_stream, layout,
                                    /*apply_reorder=*/true);

  if (std::getenv("TETRIS_CHECK")) {
    float *h_check = static_cast<float *>(std::malloc(out_count * sizeof(float)));
    std::cout << "HostConv2d begin\n";
    HostConv2d(h_input, h_filter, h_check, batch_size, img_h, img_w, in_channel, out_channel,
               kernel_size, stride, padding);
    std::cout << "HostConv2d end\n";
    std::cout << (TensorEqual(h_sparse, h_check, out_count) ? "Sparse Pass.\n" : "Sparse Error.\n");
    std::free(h_check);
  }
  cudaStreamDestroy(cuda_stream);
  std::free(h_input);
  std::free(h_filter);
  std::free(h_sparse);
  return 0;
}
