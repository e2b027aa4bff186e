// Generic sparse-filter convolution: one thread per output pixel and output-channel block, any
// kernel size and stride, input taps read straight from global memory.  It is the fallback for
// shapes the tiled kernel does not cover (e.g. 7x7) and an independent second implementation of
// the program format for cross-checks.  NHWC in, NHWC out, as the reference kernel
// (Tetris/spconv2d_kernel.cu:51-160).
#include "internal.h"

namespace tetris {
namespace {

__global__ void __launch_bounds__(128)
conv_generic_kernel(const float *__restrict__ in, float *__restrict__ out,
                    const uint2 *__restrict__ ops, const int32_t *__restrict__ prog_offsets,
                    ConvShape s, int K, int TIC, int T) {
  const long long pix = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long npix = (long long)s.N * s.OH * s.OW;
  if (pix >= npix) return;
  const int b = blockIdx.y;
  const int ow = (int)(pix % s.OW);
  const int oh = (int)((pix / s.OW) % s.OH);
  const int n = (int)(pix / ((long long)s.OW * s.OH));
  const uint32_t c_group = (uint32_t)(K * s.KS), c_end = c_group + 1;

  float acc[kMaxOcBlock];
#pragma unroll
  for (int k = 0; k < kMaxOcBlock; ++k) acc[k] = 0.f;

  const float *img = in + (size_t)n * s.H * s.W * s.IC;
  for (int t = 0; t < T; ++t) {
    const uint2 *pc = ops + prog_offsets[b * T + t];
    int ic = 0, ih = -1;
    bool row_ok = false;
    for (;;) {
      const uint2 op = __ldg(pc++);
      if (op.y == c_end) break;
      if (op.y == c_group) {
        ic = t * TIC + (int)(op.x >> 8);
        ih = oh * s.S + (int)(op.x & 255u) - s.P;
        row_ok = ih >= 0 && ih < s.H;
        continue;
      }
      const int k = (int)op.y / s.KS, sx = (int)op.y - k * s.KS;
      const int iw = ow * s.S + sx - s.P;
      if (row_ok && iw >= 0 && iw < s.W)
        acc[k] = fmaf(__uint_as_float(op.x), __ldg(&img[((size_t)ih * s.W + iw) * s.IC + ic]), acc[k]);
    }
  }
  float *o = out + (size_t)pix * s.OC + (size_t)b * K;
  const int kn = min(K, s.OC - b * K);
  for (int k = 0; k < kn; ++k) o[k] = acc[k];
}

}  // namespace

int launch_conv_generic(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                        cudaStream_t st) {
  const long long npix = (long long)s.N * s.OH * s.OW;
  if (npix <= 0) return TETRIS_OK;
  dim3 grid((unsigned)((npix + 127) / 128), (unsigned)f->n_oc_blocks);
  conv_generic_kernel<<<grid, 128, 0, st>>>(in, out, reinterpret_cast<const uint2 *>(f->d_ops),
                                            f->d_prog_offsets, s, f->oc_block, f->tile_ic,
                                            f->n_stages);
  TETRIS_CUDA_TRY(cudaGetLastError());
  count_launch();
  return TETRIS_OK;
}

}  // namespace tetris
