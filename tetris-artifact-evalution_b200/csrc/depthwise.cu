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
#include <cuda.h>

#include <algorithm>
#include <mutex>

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

// ---- 3x3 through an asynchronous pipeline -------------------------------------------------
// The kernel above is bound by latency (five dependent memory round trips per thread at half
// occupancy), not by bandwidth: kept for shapes this one does not cover (channels not a multiple
// of 32, unaligned tensors).  Here a persistent CTA walks tiles of TWO x 8 output pixels x 32
// channels; one thread issues, three to four tiles ahead, a TMA load of the tile's input patch
// with its halo (4-D box over the NHWC tensor, coordinates outside the image are filled with
// zeros: the padding) into a ring of shared-memory stages, and the 256 threads compute from
// shared memory: thread = (channel quad, pixel column, row group); it slides down its column,
// three 16-byte loads per input row, each input row feeding up to three output rows.  Taps are
// added in (r, s) order per output, as above.
constexpr uint32_t kDwSpinLimit = 1u << 22;
__device__ int g_dw_error;  // a bounded wait of the pipeline gave up (read and cleared by tetris_filter_check)

struct DwTmaParams {
  float4 *out;
  const float *filt;  // [C][9]
  int N, C, OH, OW, P;
  int tiles_x, tiles_y, cgs;
  int total;
};

__device__ __forceinline__ uint32_t dw_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool dw_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool dw_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (dw_try_wait(bar, parity)) return true;
    if ((i & 63) == 63) __nanosleep(32);
  }
  return false;
}

template <int S, int TWO>   // stride; output tile width (16, or 8 for stride 2 and for images up to 8 wide)
__global__ void __launch_bounds__(256, 2)
depthwise3x3_tma_kernel(const __grid_constant__ CUtensorMap map, const DwTmaParams p) {
  constexpr int THO = 8;                                  // output tile height
  constexpr int BX = (TWO - 1) * S + 3, BY = (THO - 1) * S + 3;  // input patch: 18 x 10, 10 x 10 or 17 x 17 pixels of 32 channels
  constexpr int kStage = BX * BY * 128;                   // bytes
  constexpr int NST = S == 1 ? 4 : 3;                     // stages (two CTAs per SM either way)
  constexpr int R = THO * TWO / 32;                       // output rows per thread: 4 or 2
  constexpr int NR = (R - 1) * S + 3;                     // input rows a thread walks
  extern __shared__ unsigned char dw_raw[];
  unsigned char *base = dw_raw + ((128 - (dw_smem_u32(dw_raw) & 127)) & 127);
  __shared__ uint64_t full[NST];
  const int tid = threadIdx.x, q = tid & 7, slot = tid >> 3;
  const int x = slot & (TWO - 1);
  const int row0 = (slot / TWO) * R;  // first output row of this thread within the tile
  if (tid == 0) {
    for (int i = 0; i < NST; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dw_smem_u32(&full[i])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int per_cg = p.tiles_x * p.tiles_y * p.N;
  auto issue = [&](int t, int s) {
    const int cg = t / per_cg;
    int rest = t - cg * per_cg;
    const int tx = rest % p.tiles_x; rest /= p.tiles_x;
    const int ty = rest % p.tiles_y;
    const int n = rest / p.tiles_y;
    const uint32_t bar = dw_smem_u32(&full[s]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)kStage) : "memory");
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dw_smem_u32(base + (size_t)s * kStage)), "l"(&map), "r"(bar), "r"(cg * 32), "r"(tx * TWO * S - p.P),
                   "r"(ty * THO * S - p.P), "r"(n) : "memory");
  };
  int issued = 0;
  if (tid == 0)
    for (int t = blockIdx.x; t < p.total && issued < NST - 1; t += gridDim.x, ++issued) issue(t, issued);
  float4 w[9];
  int cur_cg = -1;
  const int cq = p.C >> 2;
  bool ok = true;
  int k = 0;
  for (int t = blockIdx.x; t < p.total; t += gridDim.x, ++k) {
    if (tid == 0) {  // the stage tile k - 1 was read from is free again (the barrier at the end of that tile)
      const long long tn = (long long)t + (long long)(NST - 1) * gridDim.x;
      if (tn < p.total) { issue((int)tn, (k + NST - 1) % NST); ++issued; }
    }
    const int cg = t / per_cg;
    int rest = t - cg * per_cg;
    const int tx = rest % p.tiles_x; rest /= p.tiles_x;
    const int ty = rest % p.tiles_y;
    const int n = rest / p.tiles_y;
    if (cg != cur_cg) {
      cur_cg = cg;
      const float *f4 = p.filt + (size_t)(cg * 32 + 4 * q) * 9;
#pragma unroll
      for (int i = 0; i < 9; ++i) w[i] = make_float4(__ldg(f4 + i), __ldg(f4 + 9 + i), __ldg(f4 + 18 + i), __ldg(f4 + 27 + i));
    }
    ok = dw_wait(dw_smem_u32(&full[k % NST]), (uint32_t)(k / NST) & 1u, kDwSpinLimit);
    if (!__syncthreads_and(ok ? 1 : 0)) { ok = false; break; }
    const float4 *st = reinterpret_cast<const float4 *>(base + (size_t)(k % NST) * kStage);
    float4 acc[R];
#pragma unroll
    for (int a = 0; a < R; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const float4 *rowp = st + ((size_t)(row0 * S + i) * BX + x * S) * 8 + q;
      const float4 x0 = rowp[0], x1 = rowp[8], x2 = rowp[16];
#pragma unroll
      for (int a = 0; a < R; ++a) {
        const int r = i - a * S;
        if (r < 0 || r > 2) continue;
        const float4 w0 = w[r * 3], w1 = w[r * 3 + 1], w2 = w[r * 3 + 2];
        acc[a].x = fmaf(w0.x, x0.x, acc[a].x); acc[a].y = fmaf(w0.y, x0.y, acc[a].y);
        acc[a].z = fmaf(w0.z, x0.z, acc[a].z); acc[a].w = fmaf(w0.w, x0.w, acc[a].w);
        acc[a].x = fmaf(w1.x, x1.x, acc[a].x); acc[a].y = fmaf(w1.y, x1.y, acc[a].y);
        acc[a].z = fmaf(w1.z, x1.z, acc[a].z); acc[a].w = fmaf(w1.w, x1.w, acc[a].w);
        acc[a].x = fmaf(w2.x, x2.x, acc[a].x); acc[a].y = fmaf(w2.y, x2.y, acc[a].y);
        acc[a].z = fmaf(w2.z, x2.z, acc[a].z); acc[a].w = fmaf(w2.w, x2.w, acc[a].w);
      }
    }
    const int ow = tx * TWO + x;
#pragma unroll
    for (int a = 0; a < R; ++a) {
      const int oh = ty * THO + row0 + a;
      if (ow < p.OW && oh < p.OH) p.out[(((size_t)n * p.OH + oh) * p.OW + ow) * cq + cg * 8 + q] = acc[a];
    }
    __syncthreads();  // everybody is done with this stage before it is loaded again
  }
  if (!ok && tid == 0) {
    g_dw_error = 1;
    // loads already armed may still be in flight: wait (bounded) before the CTA gives up its shared memory
    for (int v = max(issued - NST, 0); v < issued; ++v) dw_wait(dw_smem_u32(&full[v % NST]), (uint32_t)(v / NST) & 1u, 1u << 16);
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

typedef CUresult (*DwEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
DwEncodeFn dw_get_encode() {
  static DwEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (DwEncodeFn)p;
  });
  return fn;
}

// The pipelined kernel's launch: 0 = launched, 1 = this shape is not covered (the caller falls
// back), otherwise a status.  Tensor maps of the inputs seen lately are kept per thread.
int launch_depthwise_tma(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st) {
  if (s.KS != 3 || (s.S != 1 && s.S != 2) || (s.OC & 31) != 0 || (reinterpret_cast<uintptr_t>(in) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return 1;
  DwEncodeFn enc = dw_get_encode();
  if (!enc) return 1;
  const int two = (s.S == 1 && s.OW > 8) ? 16 : 8, tho = 8;
  const int bx = (two - 1) * s.S + 3, by = (tho - 1) * s.S + 3;
  const int nst = s.S == 1 ? 4 : 3;
  int dev = 0, sms = 0;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  struct Entry { bool valid = false; int dev = 0; const float *in = nullptr; int N = 0, H = 0, W = 0, C = 0, S = 0, two = 0; CUtensorMap map; };
  static thread_local Entry cache[8];
  static thread_local int next = 0;
  Entry *e = nullptr;
  for (Entry &c : cache)
    if (c.valid && c.dev == dev && c.in == in && c.N == s.N && c.H == s.H && c.W == s.W && c.C == s.OC && c.S == s.S && c.two == two) { e = &c; break; }
  if (!e) {
    e = &cache[next];
    next = (next + 1) % 8;
    const cuuint64_t dims[4] = {(cuuint64_t)s.OC, (cuuint64_t)s.W, (cuuint64_t)s.H, (cuuint64_t)s.N};
    const cuuint64_t strides[3] = {(cuuint64_t)s.OC * 4, (cuuint64_t)s.W * s.OC * 4, (cuuint64_t)s.H * s.W * s.OC * 4};
    const cuuint32_t box[4] = {32, (cuuint32_t)bx, (cuuint32_t)by, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(&e->map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(in), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { e->valid = false; return 1; }
    e->valid = true; e->dev = dev; e->in = in; e->N = s.N; e->H = s.H; e->W = s.W; e->C = s.OC; e->S = s.S; e->two = two;
  }
  TETRIS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  DwTmaParams p;
  p.out = reinterpret_cast<float4 *>(out);
  p.filt = f->d_dense;
  p.N = s.N; p.C = s.OC; p.OH = s.OH; p.OW = s.OW; p.P = s.P;
  p.tiles_x = (s.OW + two - 1) / two;
  p.tiles_y = (s.OH + tho - 1) / tho;
  p.cgs = s.OC / 32;
  const long long total = (long long)p.tiles_x * p.tiles_y * s.N * p.cgs;
  if (total > 0x7FFFFFFFll / 8) return 1;
  p.total = (int)total;
  const size_t smem = (size_t)nst * bx * by * 128 + 128;
  static thread_local bool configured[16] = {false};
  if (dev >= 16 || !configured[dev]) {
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(depthwise3x3_tma_kernel<1, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 18 * 10 * 128 + 128));
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(depthwise3x3_tma_kernel<1, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 10 * 10 * 128 + 128));
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(depthwise3x3_tma_kernel<2, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 17 * 17 * 128 + 128));
    if (dev < 16) configured[dev] = true;
  }
  const unsigned grid = (unsigned)std::min<long long>(total, 2ll * sms);
  if (s.S == 1 && two == 16) depthwise3x3_tma_kernel<1, 16><<<grid, 256, smem, st>>>(e->map, p);
  else if (s.S == 1) depthwise3x3_tma_kernel<1, 8><<<grid, 256, smem, st>>>(e->map, p);
  else depthwise3x3_tma_kernel<2, 8><<<grid, 256, smem, st>>>(e->map, p);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // namespace

// 0 = no timeout seen so far, 1 = a bounded wait of the pipelined depthwise kernel gave up (cleared).
int depthwise_check_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_dw_error, sizeof(int)) != cudaSuccess) return 1;
  if (flag) { const int zero = 0; cudaMemcpyToSymbol(g_dw_error, &zero, sizeof(int)); }
  return flag;
}

int launch_depthwise(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                     cudaStream_t st) {
  const long long elems = (long long)s.N * s.OH * s.OW * s.OC;
  if (elems <= 0) return TETRIS_OK;
  {
    const int rc = launch_depthwise_tma(f, in, out, s, st);
    if (rc == 0) { count_launch(); return TETRIS_OK; }
    if (rc != 1) return rc;
  }
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
