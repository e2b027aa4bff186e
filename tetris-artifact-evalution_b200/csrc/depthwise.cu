// Depthwise convolution (groups == channels), dense filter, NHWC in / NHWC out.
//
// The reference has no grouped convolution: it reads `groups` from the layer file and ignores it
// (Tetris/tensor_utils.cc:66, Tetris/spconv2d.cc:404-406).  The MobileNet workload keeps its
// depthwise filters dense, so this is a plain bandwidth-bound stencil: lanes run along the
// channel axis (innermost in NHWC), so every global access is coalesced, and taps are added in
// (r, s) order -- the order the CPU loop nest uses (Tetris/tensor_utils.cc:152-153).
#include "internal.h"

namespace tetris {
namespace {

template <int KS>
__global__ void __launch_bounds__(256)
depthwise_kernel(const float *__restrict__ in, float *__restrict__ out,
                 const float *__restrict__ filt, ConvShape s) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)s.N * s.OH * s.OW * s.OC;
  if (idx >= total) return;
  const int c = (int)(idx % s.OC);
  long long pix = idx / s.OC;
  const int ow = (int)(pix % s.OW);
  pix /= s.OW;
  const int oh = (int)(pix % s.OH);
  const int n = (int)(pix / s.OH);
  const int ks = KS > 0 ? KS : s.KS;
  const float *img = in + (size_t)n * s.H * s.W * s.IC + c;
  const float *w = filt + (size_t)c * ks * ks;
  float acc = 0.f;
#pragma unroll
  for (int r = 0; r < ks; ++r) {
    const int ih = oh * s.S + r - s.P;
    if (ih < 0 || ih >= s.H) continue;
#pragma unroll
    for (int q = 0; q < ks; ++q) {
      const int iw = ow * s.S + q - s.P;
      if (iw < 0 || iw >= s.W) continue;
      acc = fmaf(__ldg(&w[r * ks + q]), __ldg(&img[((size_t)ih * s.W + iw) * s.IC]), acc);
    }
  }
  out[idx] = acc;
}

}  // namespace

int launch_depthwise(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                     cudaStream_t st) {
  const long long total = (long long)s.N * s.OH * s.OW * s.OC;
  if (total <= 0) return TETRIS_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (s.KS == 3)
    depthwise_kernel<3><<<blocks, 256, 0, st>>>(in, out, f->d_dense, s);
  else
    depthwise_kernel<0><<<blocks, 256, 0, st>>>(in, out, f->d_dense, s);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

}  // namespace tetris
