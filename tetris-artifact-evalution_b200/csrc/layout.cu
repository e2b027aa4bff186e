// Device-side layout transposes between NCHW and NHWC, out of place.
//
// The reference does these on the host through a temporary vector
// (Tetris/tensor_utils.cc:85-111).  Per image both are a 2-D transpose between a [C][H*W] and a
// [H*W][C] matrix, done here through a padded 32x32 shared-memory tile so that reads and writes
// are both coalesced.
#include "internal.h"

namespace tetris {
namespace {

// dst[n][col][row] = src[n][row][col] for a [rows][cols] matrix per image.
__global__ void __launch_bounds__(256)
transpose_kernel(const float *__restrict__ src, float *__restrict__ dst, int rows, int cols) {
  __shared__ float tile[32][33];
  const size_t img = (size_t)blockIdx.z * rows * cols;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + tx;
    if (r < rows && c < cols) tile[j][tx] = src[img + (size_t)r * cols + c];
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + tx;
    if (r < rows && c < cols) dst[img + (size_t)c * rows + r] = tile[tx][j];
  }
}

int launch_transpose(const float *src, float *dst, int N, int rows, int cols, cudaStream_t st) {
  if (N <= 0 || rows <= 0 || cols <= 0) return TETRIS_OK;
  const unsigned gy = (unsigned)((rows + 31) / 32);
  if (gy > 65535u || N > 65535) {
    set_error("layout transpose: shape too large for one launch");
    return TETRIS_ERR_UNSUPPORTED;
  }
  dim3 grid((unsigned)((cols + 31) / 32), gy, (unsigned)N);
  transpose_kernel<<<grid, 256, 0, st>>>(src, dst, rows, cols);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

}  // namespace

int launch_nchw_to_nhwc(const float *src, float *dst, int N, int C, int H, int W, cudaStream_t st) {
  return launch_transpose(src, dst, N, C, H * W, st);  // [C][HW] -> [HW][C]
}
int launch_nhwc_to_nchw(const float *src, float *dst, int N, int C, int H, int W, cudaStream_t st) {
  return launch_transpose(src, dst, N, H * W, C, st);  // [HW][C] -> [C][HW]
}

}  // namespace tetris
