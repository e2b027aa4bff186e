// Internal declarations of the engine: the filter handle, error plumbing and the launchers
// implemented in the individual .cu files.  Nothing here is part of the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <vector>

#include "../../include/tetris_b200.h"
#include "format.h"

struct tetris_filter {
  int in_channel, out_channel, kernel_size, groups;
  int oc_block, tile_ic;
  int n_oc_blocks, n_stages;
  int64_t nnz, n_ops;
  int max_prog_ops;        // longest program, in records
  int device;
  uint64_t *d_ops;         // program stream (n_ops records incl. tail padding)
  int32_t *d_prog_offsets; // n_oc_blocks * n_stages + 1 record indices
  float *d_dense;          // depthwise only: dense [C][KS*KS] filter
  // LIST form (format.h), consumed by the tiled kernel
  uint64_t *d_lists;       // n_list_units 8-byte units incl. tail padding
  int32_t *d_list_offsets; // n_oc_blocks * n_stages + 1 unit indices
  int64_t n_list_units;
  int max_list_units;      // longest piece, in 8-byte units
  int deterministic;       // 1: the tensor-core variant never splits a tile's K range (no atomic adds)
  void *plan_cache;        // tiled kernel: launch plan of the last conv shape (conv_tiled.cu)
  void *tc_state;          // tensor-core variant: split dense weights + tensor maps (conv_tc.cu)
  void *tc16_state;        // split-FP16 tensor-core variant: weight images + tensor maps (conv_tc16.cu)
};

namespace tetris {

void set_error(const char *fmt, ...);

#define TETRIS_CUDA_TRY(call)                                                              \
  do {                                                                                     \
    cudaError_t err__ = (call);                                                            \
    if (err__ != cudaSuccess) {                                                            \
      ::tetris::set_error("%s failed at %s:%d: %s", #call, __FILE__, __LINE__,             \
                          cudaGetErrorString(err__));                                      \
      return TETRIS_ERR_CUDA;                                                              \
    }                                                                                      \
  } while (0)

struct ConvShape {
  int N, H, W, IC, OC, KS, S, P, OH, OW;
  int relu = 0;  // fused epilogue: max(y, 0) at the store (tetris_conv2d_launch_fused)
};

// compress.cu: dense filter on the device -> program stream.  `d_scratch` holds
// n_programs + 1 ints (program lengths, then their exclusive scan) and one 64-bit
// nonzero counter after them.
size_t compress_scratch_bytes(int n_programs);
int compress_count(const float *d_filter, int IC, int OC, int KS, int K, int TIC, int B, int T,
                   int32_t *d_scratch, cudaStream_t st);
int compress_scan(const int32_t *d_scratch, int32_t *d_offsets, int n_programs, cudaStream_t st);
const unsigned long long *compress_nnz_ptr(const int32_t *d_scratch, int n_programs);
int compress_fill(const float *d_filter, int IC, int OC, int KS, int K, int TIC, int B, int T,
                  const int32_t *d_offsets, uint64_t *d_ops, int64_t n_ops, cudaStream_t st);

int list_count(const float *d_filter, int IC, int OC, int KS, int K, int TIC, int B, int T,
               int32_t *d_lens, cudaStream_t st);
int list_fill(const float *d_filter, int IC, int OC, int KS, int K, int TIC, int B, int T,
              const int32_t *d_offsets, uint64_t *d_units, int64_t n_units, cudaStream_t st);

// conv_generic.cu / conv_tiled.cu / depthwise.cu / layout.cu
int launch_conv_generic(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                        cudaStream_t st);
bool conv_tiled_supported(const tetris_filter *f, const ConvShape &s);
// allow_tc: let the plan's automatic choice switch to the tensor-core variant
int launch_conv_tiled(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                      cudaStream_t st, bool allow_tc);
int tune_conv_tiled(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                    cudaStream_t st, int max_candidates, float *best_ms);
int conv_auto_choice(const tetris_filter *f, const ConvShape &s, int *variant);
void *tiled_plan_cache_new();
// The plans tetris_conv2d_tune chose, as kTunedInts ints each: the conv shape (N, H, W, S, P),
// the kernel instance, the tile shape (NSEG, TH) and whether the tensor-core variant won.
constexpr int kTunedInts = 9;
void tiled_plans_export(const tetris_filter *f, std::vector<int32_t> *out);
void tiled_plans_import(const tetris_filter *f, const int32_t *plans, int n);
// conv kernel launches issued through the library by this process (all devices, all threads)
void count_launch();
// tetris_test_inject (failure-detection tests): 1 while the tensor-core kernels are asked to leave
// out every CTA's first activation load, with the poll limit their barrier waits then use.
int test_injection(unsigned *spin_limit);
void tiled_plan_cache_delete(void *cache);
int conv_tc_prepare(tetris_filter *f, const float *d_dense);
void conv_tc_state_delete(void *state);
bool conv_tc_supported(const tetris_filter *f, const ConvShape &s);
int launch_conv_tc(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                   cudaStream_t st);
int conv_tc_check_error(const tetris_filter *f);
int launch_conv_tc_gated(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st,
                         unsigned *gate);
int conv_tc16_prepare(tetris_filter *f, const float *d_dense);
void conv_tc16_state_delete(void *state);
bool conv_tc16_supported(const tetris_filter *f, const ConvShape &s);
int launch_conv_tc16(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st);
int conv_tc16_check_error(const tetris_filter *f);
int launch_depthwise(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                     cudaStream_t st);
int depthwise_check_error();
// chain.cu / api.cu: y = max(y, 0) in place; an automatic launch of one conv (with its fused
// options in s); whether the launch at hand rectified at its own store
int launch_relu_inplace(float *y, size_t n, cudaStream_t st);
int conv_dispatch_auto(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st);
void note_relu_fused();
int launch_nchw_to_nhwc(const float *src, float *dst, int N, int C, int H, int W, cudaStream_t st);
int launch_nhwc_to_nchw(const float *src, float *dst, int N, int C, int H, int W, cudaStream_t st);

}  // namespace tetris
