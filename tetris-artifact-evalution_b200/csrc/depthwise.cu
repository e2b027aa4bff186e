// Depthwise convolution (groups == channels), dense filter, NHWC in / NHWC out.
//
// The reference has no grouped convolution: it reads `groups` from the layer file and ignores it
// (Tetris/tensor_utils.cc:66, Tetris/spconv2d.cc:404-406).  The MobileNet workload keeps its
// depthwise filters dense, so this is a plain bandwidth-bound stencil.  Lanes run along the
// channel axis (innermost in NHWC) four channels at a time, so every global access is a
// coalesced 16-byte access; a thread produces a short run of output columns and keeps the input
// columns it has loaded in registers, so each input value is read once per filter row instead of
// once per tap.  Taps are added in (r, s) order -- the order the CPU loop nest uses
// (Tetris/tensor_utils.cc:152-153).
#include "internal.h"

namespace tetris {
namespace {

// How the 256 threads of a block are laid over the work: `qb` consecutive channel quads (a power
// of two, at most 32: the lanes of a warp read consecutive addresses) x `aw` x `ah` thread
// windows, i.e. a block computes a 2-D patch of the image, so that the input rows and columns
// neighbouring threads share are found in L1 (with a block one window tall the L2 -> SM traffic
// measured 3.2x the input).
struct DwGrid { int cq, wtiles, htiles, qb, aw, ah, qblocks, xblocks, yblocks; };

// 3x3, stride S, four channels per thread, TW output columns x RH output rows per thread.  The
// input rows are walked once: row `i` of the thread's window contributes to every output row
// whose three taps cover it, so an input value is loaded once per thread, not once per output row.
template <int S, int TW, int RH>
__global__ void __launch_bounds__(256)
depthwise3x3_kernel(const float4 *__restrict__ in, float4 *__restrict__ out,
                    const float *__restrict__ filt, ConvShape s, DwGrid g) {
  const int cq = g.cq;
  const int ql = threadIdx.x & (g.qb - 1), pos = threadIdx.x / g.qb;
  int blk = blockIdx.x;
  const int q = (blk % g.qblocks) * g.qb + ql; blk /= g.qblocks;
  const int wt = (blk % g.xblocks) * g.aw + pos % g.aw; blk /= g.xblocks;
  const int ht = (blk % g.yblocks) * g.ah + pos / g.aw;
  const int n = blk / g.yblocks;
  if (q >= cq || wt >= g.wtiles || ht >= g.htiles) return;
  const int ow0 = wt * TW, oh0 = ht * RH;

  float4 w[9];
#pragma unroll
  for (int t = 0; t < 9; ++t) {
    w[t].x = __ldg(&filt[(size_t)(4 * q + 0) * 9 + t]);
    w[t].y = __ldg(&filt[(size_t)(4 * q + 1) * 9 + t]);
    w[t].z = __ldg(&filt[(size_t)(4 * q + 2) * 9 + t]);
    w[t].w = __ldg(&filt[(size_t)(4 * q + 3) * 9 + t]);
  }
  float4 acc[RH][TW];
#pragma unroll
  for (int a = 0; a < RH; ++a)
#pragma unroll
    for (int j = 0; j < TW; ++j) acc[a][j] = make_float4(0.f, 0.f, 0.f, 0.f);

  constexpr int NCOL = (TW - 1) * S + 3;  // input columns this thread touches per row
  constexpr int NROW = (RH - 1) * S + 3;  // input rows of its window
  const int iw0 = ow0 * S - s.P, ih0 = oh0 * S - s.P;
  const float4 *img = in + (size_t)n * s.H * s.W * cq + q;
  // Taps are added in (r, s) order per output, the order of the CPU loop nest
  // (Tetris/tensor_utils.cc:152-153): window row i serves output row a with filter row r = i - a*S,
  // and i ascends.
#pragma unroll
  for (int i = 0; i < NROW; ++i) {
    const int ih = ih0 + i;
    if (ih < 0 || ih >= s.H) continue;
    float4 x[NCOL];
#pragma unroll
    for (int c = 0; c < NCOL; ++c) {
      const int iw = iw0 + c;
      x[c] = (iw >= 0 && iw < s.W) ? __ldg(&img[((size_t)ih * s.W + iw) * cq])
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int a = 0; a < RH; ++a) {
      const int r = i - a * S;
      if (r < 0 || r > 2) continue;
#pragma unroll
      for (int j = 0; j < TW; ++j)
#pragma unroll
        for (int t = 0; t < 3; ++t) {
          const float4 xv = x[j * S + t], wv = w[r * 3 + t];
          acc[a][j].x = fmaf(wv.x, xv.x, acc[a][j].x);
          acc[a][j].y = fmaf(wv.y, xv.y, acc[a][j].y);
          acc[a][j].z = fmaf(wv.z, xv.z, acc[a][j].z);
          acc[a][j].w = fmaf(wv.w, xv.w, acc[a][j].w);
        }
    }
  }
#pragma unroll
  for (int a = 0; a < RH; ++a) {
    if (oh0 + a >= s.OH) continue;
    float4 *o = out + (((size_t)n * s.OH + oh0 + a) * s.OW + ow0) * cq + q;
#pragma unroll
    for (int j = 0; j < TW; ++j)
      if (ow0 + j < s.OW) o[(size_t)j * cq] = acc[a][j];
  }
}

// Any kernel size / stride / channel count: one output element per thread.
__global__ void __launch_bounds__(256)
depthwise_any_kernel(const float *__restrict__ in, float *__restrict__ out,
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
  const float *img = in + (size_t)n * s.H * s.W * s.IC + c;
  const float *w = filt + (size_t)c * s.KS * s.KS;
  float acc = 0.f;
  for (int r = 0; r < s.KS; ++r) {
    const int ih = oh * s.S + r - s.P;
    if (ih < 0 || ih >= s.H) continue;
    for (int q = 0; q < s.KS; ++q) {
      const int iw = ow * s.S + q - s.P;
      if (iw < 0 || iw >= s.W) continue;
      acc = fmaf(__ldg(&w[r * s.KS + q]), __ldg(&img[((size_t)ih * s.W + iw) * s.IC]), acc);
    }
  }
  out[idx] = acc;
}

}  // namespace

int launch_depthwise(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                     cudaStream_t st) {
  const long long elems = (long long)s.N * s.OH * s.OW * s.OC;
  if (elems <= 0) return TETRIS_OK;
  const bool vec = s.KS == 3 && (s.S == 1 || s.S == 2) && (s.OC & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  if (vec) {
    constexpr int TW = 4;
    const int cq = s.OC / 4, wtiles = (s.OW + TW - 1) / TW;
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    float4 *out4 = reinterpret_cast<float4 *>(out);
    // Two output rows per thread where that still leaves a few thousand threads per SM in flight;
    // one row on the small late layers, where parallelism is what is short.
    int dev = 0, sms = 0;
    TETRIS_CUDA_TRY(cudaGetDevice(&dev));
    TETRIS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long threads1 = (long long)s.N * s.OH * wtiles * cq;
    const int RH = threads1 >= (long long)sms * 2048 * 2 ? 2 : 1;
    const int htiles = (s.OH + RH - 1) / RH;
    DwGrid g;
    g.cq = cq; g.wtiles = wtiles; g.htiles = htiles;
    g.qb = 8;
    while (g.qb < 32 && g.qb < cq) g.qb *= 2;
    const int windows = 256 / g.qb;                  // 32, 16 or 8 thread windows per block
    g.aw = windows >= 16 ? 4 : 2;
    while (g.aw > 1 && g.aw / 2 >= wtiles) g.aw /= 2;  // (narrow images: taller patches)
    g.ah = windows / g.aw;
    g.qblocks = (cq + g.qb - 1) / g.qb;
    g.xblocks = (wtiles + g.aw - 1) / g.aw;
    g.yblocks = (htiles + g.ah - 1) / g.ah;
    const unsigned blocks = (unsigned)((long long)g.qblocks * g.xblocks * g.yblocks * s.N);
    if (s.S == 1 && RH == 2)
      depthwise3x3_kernel<1, TW, 2><<<blocks, 256, 0, st>>>(in4, out4, f->d_dense, s, g);
    else if (s.S == 1)
      depthwise3x3_kernel<1, TW, 1><<<blocks, 256, 0, st>>>(in4, out4, f->d_dense, s, g);
    else if (RH == 2)
      depthwise3x3_kernel<2, TW, 2><<<blocks, 256, 0, st>>>(in4, out4, f->d_dense, s, g);
    else
      depthwise3x3_kernel<2, TW, 1><<<blocks, 256, 0, st>>>(in4, out4, f->d_dense, s, g);
  } else {
    depthwise_any_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, st>>>(in, out, f->d_dense, s);
  }
  TETRIS_CUDA_TRY(cudaGetLastError());
  count_launch();
  return TETRIS_OK;
}

}  // namespace tetris
