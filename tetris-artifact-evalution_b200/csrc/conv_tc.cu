// Dense-contraction variant on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), FP32
// results by the three-pass split-TF32 scheme.
//
// Why it exists: the CUDA-core kernels need one data-dependent input word per multiply-add and
// are bound by the shared-memory pipe at 12-16 % of the FP32 peak (see the profile summaries).
// At the 80-95 % sparsities of the benchmark networks the same layer, computed DENSELY as an
// implicit GEMM on the tensor cores, needs 5-20x the multiply-adds at well over 20x the rate --
// the dense-contraction sub-case the design allows once a profile shows that it pays.  The
// weights keep their zeros here; sparsity is not exploited, precision is:
//
//   x = x_hi + x_lo, w = w_hi + w_lo with *_hi the TF32 truncation (what the tensor core reads
//   from an FP32 word) and *_lo the remainder; D += x_hi*w_hi + x_lo*w_hi + x_hi*w_lo in FP32
//   accumulators.  The dropped x_lo*w_lo term is 2^-22 relative; measured error against the CPU
//   convolution is ~1e-6, inside the 1e-4 bound of the path.
//
// One CTA computes a 128-pixel x 128-channel output tile.  GEMM view: M = pixels of a
// TW x TH x NB patch, N = output channels, K = (filter tap, 32-channel chunk).  Per K step:
//   * warp 0 (one thread): TMA tiled loads -- the activation patch shifted by the tap as a 4-D box
//     of the NHWC tensor (out-of-range coordinates are zero-filled: that is the padding), and the
//     w_hi / w_lo tiles -- into a 3-stage ring of 128-byte-swizzled shared tiles;
//   * warps 2-5: derive x_lo = x - trunc_tf32(x) next to the loaded tile (same offsets, so the
//     swizzle is preserved), publish it to the async proxy;
//   * warp 1 (one thread): 12 tcgen05.mma (4 K-slices x 3 passes) into the TMEM accumulator,
//     then tcgen05.commit frees the stage.
// Epilogue: warps 2-5 read their TMEM lane quarter (tcgen05.ld) and store 512 contiguous bytes per
// pixel (NHWC).  Every barrier wait is bounded: on a timeout an error flag is raised, all roles
// drain, TMEM is freed and the kernel returns; the host reports TETRIS_ERR_CUDA.
//
// No cluster launch, no multicast.  Covers stride 1, IC % 4 == 0 (TMA needs 16-byte strides).
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "internal.h"

namespace tetris {
namespace {

constexpr int BM = 128, KC = 32;  // tile rows (pixels), K chunk (32 floats = 128 B); BN = 64 or 128 channels
constexpr int kStages = 3;
constexpr int kTileBytes = BM * KC * 4;     // 16 KiB: one 128-row x 128-byte operand tile
constexpr int kStageBytes = 4 * kTileBytes; // x, x_lo, w_hi, w_lo
constexpr int kThreads = 192;               // warp 0 producer, warp 1 MMA, warps 2-5 convert + epilogue
constexpr uint32_t kSpinLimit = 1u << 22;

struct TcParams {
  float *out;
  int N, OH, OW, OC, P, KS;
  int TW, TH, NB;              // pixel patch of a tile: TW x TH x NB <= 128 rows
  int tiles_w, tiles_h, tiles_n;
  int n_chunks;                // ceil(IC / 32)
  int *error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Gives up when the limit is hit or when another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63) == 63) {
      if (*abort_flag) return false;
      __nanosleep(32);
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// K-major operand tile, 128-byte rows, 128B swizzle, 8-row atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_whi,
               const __grid_constant__ CUtensorMap map_wlo, const TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *base = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(base + kStages * kStageBytes);
  // barriers: full[s], conv[s], empty[s], accum
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * kStages + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar_full = [&](int s) { return smem_u32(&bars[s]); };
  auto bar_conv = [&](int s) { return smem_u32(&bars[kStages + s]); };
  auto bar_empty = [&](int s) { return smem_u32(&bars[2 * kStages + s]); };
  const uint32_t bar_accum = smem_u32(&bars[3 * kStages]);

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_conv(s), 4);
      mbar_init(bar_empty(s), 1);
    }
    mbar_init(bar_accum, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // ---- which tile ----
  int bx = blockIdx.x;
  const int tw = bx % p.tiles_w; bx /= p.tiles_w;
  const int th = bx % p.tiles_h;
  const int tn = bx / p.tiles_h;
  const int w0 = tw * p.TW, h0 = th * p.TH, n0 = tn * p.NB;
  const int oc0 = blockIdx.y * BN;
  const int taps = p.KS * p.KS;
  const int iters = taps * p.n_chunks;
  const uint32_t x_box_bytes = (uint32_t)(p.TW * p.TH * p.NB * KC * 4);

  if (warp == 0) {
    if (lane == 0) {
      for (int it = 0; it < iters; ++it) {
        const int s = it % kStages;
        if (!mbar_wait(bar_empty(s), ((it / kStages) & 1) ^ 1, abort_flag)) break;
        const int tap = it / p.n_chunks, chunk = it - tap * p.n_chunks;
        const int r = tap / p.KS, q = tap - r * p.KS;
        unsigned char *st = base + s * kStageBytes;
        mbar_expect_tx(bar_full(s), x_box_bytes + 2u * (uint32_t)(BN * KC * 4));
        tma_load_4d(smem_u32(st), &map_x, bar_full(s), chunk * KC, w0 + q - p.P, h0 + r - p.P, n0);
        tma_load_3d(smem_u32(st + 2 * kTileBytes), &map_whi, bar_full(s), chunk * KC, oc0, tap);
        tma_load_3d(smem_u32(st + 3 * kTileBytes), &map_wlo, bar_full(s), chunk * KC, oc0, tap);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % kStages;
        const uint32_t parity = (it / kStages) & 1;
        ok = mbar_wait(bar_full(s), parity, abort_flag) && mbar_wait(bar_conv(s), parity, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t st = smem_u32(base + s * kStageBytes);
#pragma unroll
        for (int k = 0; k < KC / 8; ++k) {
          const uint64_t dx = umma_desc(st + k * 32), dxl = umma_desc(st + kTileBytes + k * 32);
          const uint64_t dwh = umma_desc(st + 2 * kTileBytes + k * 32), dwl = umma_desc(st + 3 * kTileBytes + k * 32);
          umma_tf32(tmem_base, dx, dwh, idesc, (it | k) ? 1u : 0u);
          umma_tf32(tmem_base, dxl, dwh, idesc, 1u);
          umma_tf32(tmem_base, dx, dwl, idesc, 1u);
        }
        umma_commit(bar_empty(s));  // the stage may be refilled once these MMAs have read it
      }
      umma_commit(bar_accum);       // arrives when everything issued so far has completed
    }
  } else {
    // ---- warps 2..5: x_lo for every landed stage, then the epilogue ----
    const int ct = tid - 64;  // 0..127: the tile row this thread converts
    for (int it = 0; it < iters; ++it) {
      const int s = it % kStages;
      if (!mbar_wait(bar_full(s), (it / kStages) & 1, abort_flag)) break;
      const float4 *src = reinterpret_cast<const float4 *>(base + s * kStageBytes + ct * 128);
      float4 *dst = reinterpret_cast<float4 *>(base + s * kStageBytes + kTileBytes + ct * 128);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int jj = (j + lane) & 7;  // spread the lanes of a warp over the banks
        const float4 v = src[jj];
        float4 lo;
        lo.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
        lo.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
        lo.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
        lo.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
        dst[jj] = lo;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> tensor-core reads
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_conv(s));
    }
    const bool done = mbar_wait(bar_accum, 0, abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (done && !*abort_flag) {
      const int quarter = warp & 3;          // TMEM lanes this warp may read
      const int row = quarter * 32 + lane;   // tile row = pixel
      const int pw = row % p.TW, ph = (row / p.TW) % p.TH, pn = row / (p.TW * p.TH);
      const int ow = w0 + pw, oh = h0 + ph, n = n0 + pn;
      const bool row_ok = pn < p.NB && ow < p.OW && oh < p.OH && n < p.N;
      float *o = p.out + (((size_t)n * p.OH + oh) * p.OW + ow) * p.OC + oc0;
      const bool vec = (p.OC & 3) == 0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
              "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
              "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (!row_ok) continue;
        if (vec && oc0 + c0 + 32 <= p.OC) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4 *>(o + c0 + j) =
                make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (oc0 + c0 + j < p.OC) o[c0 + j] = __uint_as_float(v[j]);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.error_flag, 1);
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN) : "memory");
}

// Dense OIHW -> [tap][OC][ICP] in two FP32 tensors: the weight itself (the tensor core reads its
// TF32 truncation) and the remainder w - trunc(w).
__global__ void tc_weight_split_kernel(const float *__restrict__ filt, float *__restrict__ hi, float *__restrict__ lo,
                                       int OC, int IC, int KS, int ICP) {
  const long long total = (long long)KS * KS * OC * ICP;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ic = (int)(i % ICP);
    const int oc = (int)((i / ICP) % OC);
    const int tap = (int)(i / ((long long)ICP * OC));
    float w = 0.f;
    if (ic < IC) w = filt[((size_t)oc * IC + ic) * KS * KS + tap];
    hi[i] = w;
    lo[i] = w - __uint_as_float(__float_as_uint(w) & 0xFFFFE000u);
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                             const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeFn)p;
  });
  return fn;
}

int encode_map(CUtensorMap *map, void *ptr, int rank, const cuuint64_t *dims, const cuuint64_t *strides,
               const cuuint32_t *box) {
  EncodeFn enc = get_encode();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return TETRIS_ERR_UNSUPPORTED; }
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, ptr, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return TETRIS_ERR_CUDA; }
  return TETRIS_OK;
}

struct TcState {
  float *d_hi = nullptr, *d_lo = nullptr;
  int *d_error = nullptr;
  int icp = 0;
  CUtensorMap map_whi, map_wlo;      // weight tiles of 128 output channels
  CUtensorMap map_whi64, map_wlo64;  // ... and of 64
  // activation map of the last input pointer / shape
  std::mutex mutex;
  const float *last_in = nullptr;
  ConvShape last_shape{};
  CUtensorMap map_x;
  TcParams params{};
  dim3 grid;
  int bn = 128;
};

}  // namespace

void conv_tc_state_delete(void *state) {
  TcState *s = static_cast<TcState *>(state);
  if (!s) return;
  cudaFree(s->d_hi); cudaFree(s->d_lo); cudaFree(s->d_error);
  delete s;
}

// Builds the dense split weights and their tensor maps (called from filter creation, d_dense is
// the OIHW filter on the device).  Failure here is not fatal for the filter: the variant is then
// reported as unsupported.
int conv_tc_prepare(tetris_filter *f, const float *d_dense) {
  if (f->groups != 1 || (f->in_channel & 3) != 0) return TETRIS_OK;  // not covered: leave tc_state null
  TcState *s = new (std::nothrow) TcState();
  if (!s) return TETRIS_OK;
  const int KS = f->kernel_size, taps = KS * KS;
  s->icp = (f->in_channel + KC - 1) / KC * KC;
  const size_t elems = (size_t)taps * f->out_channel * s->icp;
  if (cudaMalloc(&s->d_hi, elems * 4) != cudaSuccess || cudaMalloc(&s->d_lo, elems * 4) != cudaSuccess ||
      cudaMalloc(&s->d_error, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    conv_tc_state_delete(s);
    return TETRIS_OK;
  }
  cudaMemset(s->d_error, 0, sizeof(int));
  tc_weight_split_kernel<<<(unsigned)std::min<size_t>((elems + 255) / 256, 4096), 256>>>(d_dense, s->d_hi, s->d_lo,
                                                                                        f->out_channel, f->in_channel, KS, s->icp);
  const cuuint64_t dims[3] = {(cuuint64_t)s->icp, (cuuint64_t)f->out_channel, (cuuint64_t)taps};
  const cuuint64_t strides[2] = {(cuuint64_t)s->icp * 4, (cuuint64_t)s->icp * 4 * f->out_channel};
  const cuuint32_t box[3] = {KC, 128, 1}, box64[3] = {KC, 64, 1};
  if (cudaGetLastError() != cudaSuccess || encode_map(&s->map_whi, s->d_hi, 3, dims, strides, box) ||
      encode_map(&s->map_wlo, s->d_lo, 3, dims, strides, box) ||
      encode_map(&s->map_whi64, s->d_hi, 3, dims, strides, box64) ||
      encode_map(&s->map_wlo64, s->d_lo, 3, dims, strides, box64)) {
    conv_tc_state_delete(s);
    return TETRIS_OK;
  }
  f->tc_state = s;
  return TETRIS_OK;
}

bool conv_tc_supported(const tetris_filter *f, const ConvShape &s) {
  if (!f->tc_state || f->groups != 1) return false;
  if (s.S != 1 || (s.IC & 3) != 0 || s.N < 1 || s.OH < 1 || s.OW < 1) return false;
  return true;
}

int launch_conv_tc(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st) {
  if (!conv_tc_supported(f, s) || (reinterpret_cast<uintptr_t>(in) & 15) != 0) {
    set_error("tensor-core variant covers stride 1, in_channel %% 4 == 0 and 16-byte aligned inputs only");
    return TETRIS_ERR_UNSUPPORTED;
  }
  TcState *t = static_cast<TcState *>(f->tc_state);
  CUtensorMap map_x;
  TcParams p;
  dim3 grid;
  int bn = 128;
  {
    std::lock_guard<std::mutex> lock(t->mutex);
    const ConvShape &l = t->last_shape;
    const bool hit = t->last_in == in && l.N == s.N && l.H == s.H && l.W == s.W && l.P == s.P && l.S == s.S;
    if (!hit) {
      // pixel patch: TW x TH x NB rows, at most 128, as full as possible
      int best_tw = 1, best_th = 1, best_nb = 1;
      double best = -1.0;
      for (int TW = 1; TW <= std::min(s.OW, 128); ++TW) {
        const int TH = std::min(s.OH, 128 / TW);
        if (TH < 1) continue;
        const int NB = (TH == s.OH && TW == s.OW) ? std::min(s.N, 128 / (TW * TH)) : 1;
        const double tiles = (double)((s.OW + TW - 1) / TW) * ((s.OH + TH - 1) / TH) * ((s.N + NB - 1) / NB);
        const double eff = (double)s.N * s.OH * s.OW / (tiles * 128.0);
        if (eff > best) { best = eff; best_tw = TW; best_th = TH; best_nb = NB; }
      }
      const cuuint64_t dims[4] = {(cuuint64_t)s.IC, (cuuint64_t)s.W, (cuuint64_t)s.H, (cuuint64_t)s.N};
      const cuuint64_t strides[3] = {(cuuint64_t)s.IC * 4, (cuuint64_t)s.IC * 4 * s.W, (cuuint64_t)s.IC * 4 * s.W * s.H};
      const cuuint32_t box[4] = {KC, (cuuint32_t)best_tw, (cuuint32_t)best_th, (cuuint32_t)best_nb};
      const int rc = encode_map(&t->map_x, const_cast<float *>(in), 4, dims, strides, box);
      if (rc) return rc;
      TcParams &q = t->params;
      q.N = s.N; q.OH = s.OH; q.OW = s.OW; q.OC = s.OC; q.P = s.P; q.KS = s.KS;
      q.TW = best_tw; q.TH = best_th; q.NB = best_nb;
      q.tiles_w = (s.OW + best_tw - 1) / best_tw;
      q.tiles_h = (s.OH + best_th - 1) / best_th;
      q.tiles_n = (s.N + best_nb - 1) / best_nb;
      q.n_chunks = t->icp / KC;
      q.error_flag = t->d_error;
      t->bn = s.OC <= 64 ? 64 : 128;
      t->grid = dim3((unsigned)(q.tiles_w * q.tiles_h * q.tiles_n), (unsigned)((s.OC + t->bn - 1) / t->bn));
      t->last_in = in;
      t->last_shape = s;
    }
    map_x = t->map_x;
    p = t->params;
    grid = t->grid;
    bn = t->bn;
  }
  p.out = out;
  const size_t smem = (size_t)kStages * kStageBytes + 1024 + 256;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(conv_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(conv_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 16) configured[dev] = true;
  }
  if (bn == 64)
    conv_tc_kernel<64><<<grid, kThreads, smem, st>>>(map_x, t->map_whi64, t->map_wlo64, p);
  else
    conv_tc_kernel<128><<<grid, kThreads, smem, st>>>(map_x, t->map_whi, t->map_wlo, p);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

// 0 = no timeout seen so far, 1 = a bounded wait gave up in some launch (the flag is cleared).
int conv_tc_check_error(const tetris_filter *f) {
  TcState *t = static_cast<TcState *>(f->tc_state);
  if (!t) return 0;
  int flag = 0;
  if (cudaMemcpy(&flag, t->d_error, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
  if (flag) cudaMemset(t->d_error, 0, sizeof(int));
  return flag;
}

}  // namespace tetris
