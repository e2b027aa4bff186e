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
//   x = x_hi + x_lo, w = w_hi + w_lo with *_hi the value rounded to TF32 (to nearest) and
//   *_lo the remainder; D += x_hi*w_hi + x_lo*w_hi + x_hi*w_lo in FP32 accumulators.  The
//   *_hi parts are rounded rather than left to the truncation the tensor core applies to a raw
//   FP32 word, so that the error terms (the truncation of the remainders and the dropped
//   x_lo*w_lo, about 2^-22 of a product each) have no preferred sign and do not add up over the
//   ~5000 products of a deep layer.
//
// The tensor core adds into its FP32 accumulator with truncation, so a long accumulation chain
// drifts toward zero (measured: 5e-5 absolute on outputs of 0.1 after the 1700 accumulation
// steps of a 512-channel 3x3 layer).  The chain is therefore cut: the tensor core accumulates
// four K steps (48 MMAs) from zero into a partial accumulator, and CUDA-core warps add the
// partial to the running sum, kept in registers, with round-to-nearest FP32 adds (measured
// error of the deep layers against the CPU convolution: below 4e-6 absolute).
//
// A persistent CTA (one per SM) walks 128-pixel x 128-channel (or x 64) output tiles.  GEMM
// view: M = pixels of a TW x TH x NB tile, N = output channels, K = (32-channel chunk, filter
// tap).  The M-side operand is fed to the tensor core from TENSOR MEMORY, the N-side operand
// from shared memory.  Every hand-over has its own ring with a full/empty barrier pair, so the
// roles run decoupled (measured: with one shared ring the barrier round trips, not the tensor
// pipe, set the pace):
//   * warp 0 (one thread): one TMA load per 32-channel chunk of the tile's pixels WITH THEIR
//     HALO -- a 4-D box (32 channels, TW+KS-1, TH+KS-1, NB) of the NHWC tensor; out-of-range
//     coordinates are zero-filled, which is the padding -- into a 2-deep ring of
//     128-byte-swizzled stages.  All KS*KS taps read their shifted rows from the one patch:
//     a box per tap moves 6x the bytes, and 128-byte rows scattered over L2 come in at only
//     ~25 B/clock/SM (measured), which made the activation loads as slow as the MMAs;
//   * warp 2 (one thread): one bulk copy per K step of a prepared {w_hi, w_lo} tile image into
//     a 5-deep ring (4-deep on layers with few K steps per item, see w_stages);
//   * warps 4-11: per K step read the patch rows of the tap (un-swizzling) and write
//     x_hi = tf32(x) and x_lo = x - x_hi into a 4-deep ring of 64 TMEM columns
//     (tcgen05.st); warps 4-7 take the even K steps, warps 8-11 the odd ones, because one
//     step's chain of waits, loads and stores is longer than an MMA period;
//   * warp 3 (one thread), the gatekeeper: waits per K step for the weights, for the drained
//     partial accumulator and for the free operand stage, and passes all three on as one
//     barrier, so that a converter warp waits once per K step and the MMA warp once;
//   * warp 1 (converged, one elected lane issues): 12 tcgen05.mma per K step (4 K-slices x 3
//     passes) into one of two partial accumulators in TMEM; after every K step one
//     tcgen05.commit releases the operand stages, and every fourth of those also hands the
//     partial accumulator over;
//   * warps 12-19: read the partial accumulator (tcgen05.ld; a warp may touch the TMEM lanes
//     of its quarter, two warps share a quarter and take half of the channels each), release
//     it, add it to the running sum; after the tile's last K step turn the sums through a
//     4 KiB staging block per warp so that eight lanes store one pixel's 128 contiguous bytes.
// Every barrier wait is bounded: on a timeout an error flag is raised, all roles drain, TMEM is
// freed and the kernel returns; the host reports TETRIS_ERR_CUDA.
//
// At stride > 1 a patch would hold S*S times the pixels it is used for, so there the loader
// falls back to one box per K step (the tile's input pixels of that tap, picked by the tensor
// map's element strides) in a 4-deep ring of 16 KiB stages.
//
// With at most 4 input channels (the stems of the networks) taps and channels are folded into
// one K axis, K = KS*KS*IC in chunks of 32, and the converter warps gather the activations from
// global memory themselves (TMA needs 16-byte strides; an NHWC pixel of 3 floats has 12).
//
// No cluster launch: every load is issued by one CTA for itself.  Covers strides 1-8, IC <= 4 or
// IC % 4 == 0.
#include <cuda.h>

#include <cstring>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "internal.h"

namespace tetris {
namespace {

constexpr int BM = 128, KC = 32;  // tile rows (pixels), K chunk (32 floats = 128 B); BN = 64 or 128 channels
constexpr int kXStages = 4;                 // activation stages: 4 of 16 KiB (a box per K step) or 2 of 32 KiB (patches)
constexpr int kWStages = 5;                 // ring of {w_hi, w_lo} tile pairs (shared memory, TMA target); the
                                            // fifth stage is given up for the store staging block on layers
                                            // with few K steps per tile (TcParams::w_stages)
constexpr int kAStages = 4;                 // ring of {x, x_lo} operand blocks (tensor memory)
constexpr int kTileBytes = BM * KC * 4;     // 16 KiB: one 128-row x 128-byte operand tile
constexpr int kPatchRows = 256;             // rows of 128 bytes an activation stage holds
constexpr int kPatchBytes = kPatchRows * KC * 4;
constexpr int kXBytes = 2 * kPatchBytes;     // shared memory of the activation ring, either way
constexpr int kStoreBytes = 8 * 32 * 32 * 4;  // store staging: per summing warp 32 rows x 32 channels
constexpr int kSmemTiles = kXBytes + kWStages * 2 * kTileBytes;  // the store staging block lies over the fifth weight stage
static_assert(kStoreBytes <= 2 * kTileBytes, "the store staging block must fit a weight stage");
constexpr int kPromote = 1;                 // K steps per group: one commit, releases the operand stages (per-step
                                            // release measured 1-4 % faster than per two steps: the operand ring
                                            // is only four deep)
constexpr int kSuper = 4;                   // groups accumulated on the tensor core before the FP32 add outside
constexpr int kTmemCols = 512;              // 2 partial accumulators (<= 128 columns each) + 4 x 64 operand columns
constexpr int kTmemA = 256;                 // first operand column
constexpr int kGroups = 8;                  // "group done" barriers in rotation (a group = kPromote K steps)
constexpr int kThreads = 640;               // warp 0 x loads, 1 MMA, 2 w loads, 4-11 convert, 12-19 sum + store
constexpr int kNumBars = 2 * kXStages + kWStages + 2 * kAStages + kGroups + 1 + 2;   // (... + one drain barrier + two partial-sum barriers)
constexpr uint32_t kSpinLimit = 1u << 22;

struct TcParams {
  float *out;
  int N, OH, OW, OC, P, KS;
  int TW, TH, NB;              // pixels of a tile: TW x TH x NB <= 128 rows
  int PW, PH;                  // the tile with its halo: PW = TW + KS - 1, PH = TH + KS - 1
  int per_tap, S;              // per_tap: one strided box per K step instead of a patch per chunk (stride > 1)
  int w_stages;                // weight stages in use: 5, or 4 with the fifth as store staging block
  int folded;                  // <= 4 input channels: K = (filter row, filter column, channel) folded into
                               // 32-wide chunks, activations gathered from global memory by the converters
  const float *in;             // activations (folded mode only)
  int H, W, IC;                // input extent (folded mode only)
  int tiles_w, tiles_h, tiles_n;
  int n_chunks;                // ceil(IC / 32)
  int ksplit;                  // work items per tile: each takes n_chunks / ksplit chunks and adds its result in
  int relu;                    // max(y, 0) at the store (never together with a split K range)
  int *error_flag;
  const float *w_tiles;        // weight tile images, see tc_weight_tiles_kernel
  int tma_store;               // the summing warps hand their staged blocks to TMA stores (see the epilogue)
  unsigned spin_limit;         // polls after which a barrier wait gives up (0: kSpinLimit)
  int withhold_first_load;     // failure-detection test only: every CTA leaves out its first activation load
  unsigned *gate;              // when set: the launch runs only if the magnitude in gate[0] asks for it (see launch_conv_tc_gated)
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
// Bounded wait.  Gives up when the limit (abort_flag[1]) is hit or when another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint32_t limit = (uint32_t)abort_flag[1];
  for (uint32_t i = 1; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63) == 63) {
      if (*abort_flag) return false;
      __nanosleep(32);
    }
  }
  *abort_flag = 1;
  return false;
}
// After a give-up: wait (bounded, whatever the abort flag says) for an asynchronous operation this
// thread started earlier, so that the CTA does not leave while a copy into its shared memory or
// an MMA on its tensor memory is still in flight.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 16); ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 63) == 63) __nanosleep(64);
  }
}
// The same for a whole converged warp, with one answer for all lanes.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, int lane) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// K-major operand tile, 128-byte rows, 128B swizzle, 8-row atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// FP32 -> TF32 (10 mantissa bits), round to nearest, ties away from zero; low 13 bits are zero.
// Integer form of cvt.rna.tf32.f32 for finite inputs (the conversion pipe runs at a quarter of
// the integer rate, and the converter warps round 64 values per K step each).
__device__ __forceinline__ uint32_t round_tf32(float v) { return (__float_as_uint(v) + 0x1000u) & 0xFFFFE000u; }
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
  return pred != 0;
}
// A-operand-in-TMEM form: D[tmem] (+)= A[tmem] * B[smem descriptor].
// The shared-memory descriptor is passed as its two words: the high word is a constant, the low
// word is the start address field plus a constant, so that stepping along K or to the w_lo tile
// is one integer add (the MMA thread's own instruction count is what limits the issue rate).
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t db_lo, uint32_t db_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\n.reg .b64 d;\nmov.b64 d, {%2, %3};\nsetp.ne.b32 p, %5, 0;\n"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], d, %4, p;\n}"
               ::"r"(tmem_d), "r"(tmem_a), "r"(db_lo), "r"(db_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}


template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_out, const TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  // A gated launch stands behind the split-FP16 variant, which left the largest |activation| it
  // saw (FP32 bits) in gate[0].  Recompute the layer when that does not fit FP16's window
  // (2048 or more after the variant's scaling, NaN, infinity) or when all activations are so
  // small (below 2^-8, not all zero) that FP16's absolute error would show; return otherwise.
  // Every CTA reads the word before it counts itself in gate[1]; the last one to do so clears
  // both for the next launch.
  if (p.gate) {
    unsigned *verdict = reinterpret_cast<unsigned *>(smem_raw);
    if (threadIdx.x == 0) {
      const unsigned m = *reinterpret_cast<volatile unsigned *>(p.gate);
      *verdict = (m >= 0x45000000u || (m != 0u && m < 0x3B800000u)) ? 1u : 0u;
      __threadfence();
      if (atomicAdd(p.gate + 1, 1u) == gridDim.x - 1) { p.gate[0] = 0u; p.gate[1] = 0u; }
    }
    __syncthreads();
    const unsigned run = *verdict;
    __syncthreads();
    if (!run) return;
  }
  unsigned char *xbase = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  unsigned char *wbase = xbase + kXBytes;
  unsigned char *store_base = wbase + 4 * 2 * kTileBytes;  // = weight stage 4, unused when w_stages == 4
  uint64_t *bars = reinterpret_cast<uint64_t *>(xbase + kSmemTiles);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar_xfull = [&](int s) { return smem_u32(&bars[s]); };
  auto bar_xempty = [&](int s) { return smem_u32(&bars[kXStages + s]); };
  auto bar_wfull = [&](int s) { return smem_u32(&bars[2 * kXStages + s]); };
  auto bar_afull = [&](int s) { return smem_u32(&bars[2 * kXStages + kWStages + s]); };
  auto bar_ready = [&](int s) { return smem_u32(&bars[2 * kXStages + kWStages + kAStages + s]); };
  auto bar_gdone = [&](int c) { return smem_u32(&bars[2 * kXStages + kWStages + 2 * kAStages + c]); };
  auto bar_pempty = [&](int b) { return smem_u32(&bars[kNumBars - 2 + b]); };
  auto bar_drain = [&]() { return smem_u32(&bars[kNumBars - 3]); };

  if (tid == 0) {
    // a patch is read by all eight converter warps, a per-tap box by the four that take its K step
    for (int s = 0; s < kXStages; ++s) { mbar_init(bar_xfull(s), 1); mbar_init(bar_xempty(s), p.per_tap ? 4 : 8); }
    for (int s = 0; s < kWStages; ++s) mbar_init(bar_wfull(s), 1);
    for (int s = 0; s < kAStages; ++s) { mbar_init(bar_afull(s), 4); mbar_init(bar_ready(s), 1); }
    for (int c = 0; c < kGroups; ++c) mbar_init(bar_gdone(c), 1);
    for (int b = 0; b < 2; ++b) mbar_init(bar_pempty(b), 8);
    mbar_init(bar_drain(), 1);
    abort_flag[0] = 0;
    abort_flag[1] = (int)(p.spin_limit ? p.spin_limit : kSpinLimit);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the whole tensor memory of the SM: this kernel runs one CTA per SM
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // Persistent CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the channel tile is the
  // fastest index, so CTAs that run side by side read the same activation patch.
  const int taps = p.folded ? 1 : p.KS * p.KS;  // K steps per channel chunk
  const int item_chunks = p.n_chunks / p.ksplit;            // chunks of a work item (ksplit divides n_chunks)
  const int iters = taps * item_chunks;                     // K steps of a work item
  const int tile_groups = (iters + kPromote - 1) / kPromote;  // groups of a tile
  const int tile_supers = (tile_groups + kSuper - 1) / kSuper;  // partial accumulators of a tile
  const int oc_tiles = (p.OC + BN - 1) / BN;
  // A work item is a tile, or -- when the tiles do not fill the last wave of CTAs well -- one
  // of ksplit slices of a tile's K range; the slices add their results into a zeroed output.
  const int total_tiles = p.tiles_w * p.tiles_h * p.tiles_n * oc_tiles * p.ksplit;
  auto decode = [&](int t, int &w0, int &h0, int &n0, int &oc0, int &chunk0) {
    chunk0 = (t % p.ksplit) * item_chunks; t /= p.ksplit;
    oc0 = (t % oc_tiles) * BN; t /= oc_tiles;
    w0 = (t % p.tiles_w) * p.TW; t /= p.tiles_w;
    h0 = (t % p.tiles_h) * p.TH;
    n0 = (t / p.tiles_h) * p.NB;
  };
  // One tcgen05.commit per group (= K step) tells everyone that the group's MMAs have
  // completed: the weight loader and the gatekeeper reuse the operand stages those MMAs read,
  // and after the last group of a partial sum the summing warps take the accumulator.  (A
  // commit costs the issuing thread 150-200 clocks, measured, so there is one per K step for
  // all purposes rather than one per ring.)  K step g of this CTA (counted across tiles) lies
  // in group group_of(g); a stage last used by step g - depth is free once that group is done.
  // The kGroups barriers rotate; eight are enough for every waiter to look at a group before
  // its barrier comes round again (the MMAs are at most two partial sums ahead of the summing
  // warps, the rings at most five K steps deep).
  auto group_of = [&](int g) { const int j = g / iters; return j * tile_groups + (g - j * iters) / kPromote; };
  auto wait_group = [&](int c) { return mbar_wait(bar_gdone(c % kGroups), (c / kGroups) & 1, abort_flag); };
  auto wait_group_warp = [&](int c) { return mbar_wait_warp(bar_gdone(c % kGroups), (c / kGroups) & 1, abort_flag, lane); };

  if (warp == 0) {
    // ---- activation loads ----
    if (lane == 0) {
      int u = 0;  // loads of this CTA, across tiles
      bool ok = true;
      if (p.folded) {
        // the converters gather the activations themselves
      } else if (!p.per_tap) {
        // One patch per 32-channel chunk: the tile plus its halo, shared by all taps.
        const uint32_t x_box_bytes = (uint32_t)(p.PW * p.PH * p.NB * KC * 4);
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
          int w0, h0, n0, oc0, chunk0;
          decode(t, w0, h0, n0, oc0, chunk0);
          for (int chunk = chunk0; chunk < chunk0 + item_chunks; ++chunk, ++u) {
            const int s = u & 1;
            if (!(ok = mbar_wait(bar_xempty(s), ((u >> 1) & 1) ^ 1, abort_flag))) break;
            if (u == 0 && p.withhold_first_load) continue;  // (test: this patch never arrives, its readers give up)
            mbar_expect_tx(bar_xfull(s), x_box_bytes);
            tma_load_4d(smem_u32(xbase + s * kPatchBytes), &map_x, bar_xfull(s), chunk * KC, w0 - p.P, h0 - p.P, n0);
          }
        }
        if (!ok || *abort_flag)  // the loads of the last lap may still be in flight
          for (int v = max(u - 2, p.withhold_first_load ? 1 : 0); v < u; ++v) mbar_drain(bar_xfull(v & 1), (uint32_t)(v >> 1) & 1u);
      } else {
        // Stride > 1: one box per K step, the tile's input pixels of that tap (every S-th
        // pixel; the tensor map carries the element strides).
        const uint32_t x_box_bytes = (uint32_t)(p.TW * p.TH * p.NB * KC * 4);
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
          int w0, h0, n0, oc0, chunk0;
          decode(t, w0, h0, n0, oc0, chunk0);
          for (int it = 0; it < iters; ++it, ++u) {
            const int s = u % kXStages;
            if (!(ok = mbar_wait(bar_xempty(s), ((u / kXStages) & 1) ^ 1, abort_flag))) break;
            if (u == 0 && p.withhold_first_load) continue;
            const int chunk = it / taps, tap = it - chunk * taps;
            const int r = tap / p.KS, q = tap - r * p.KS;
            mbar_expect_tx(bar_xfull(s), x_box_bytes);
            tma_load_4d(smem_u32(xbase + s * kTileBytes), &map_x, bar_xfull(s), (chunk0 + chunk) * KC, w0 * p.S + q - p.P, h0 * p.S + r - p.P, n0);
          }
        }
        if (!ok || *abort_flag)
          for (int v = max(u - kXStages, p.withhold_first_load ? 1 : 0); v < u; ++v) mbar_drain(bar_xfull(v % kXStages), (uint32_t)(v / kXStages) & 1u);
      }
    }
  } else if (warp == 2) {
    // ---- weight loads ----
    if (lane == 0) {
      int g = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int w0, h0, n0, oc0, chunk0;
        decode(t, w0, h0, n0, oc0, chunk0);
        for (int it = 0; it < iters; ++it, ++g) {
          const int s = g % p.w_stages;
          if (g >= p.w_stages && !(ok = wait_group(group_of(g - p.w_stages)))) break;
          // K step `it` of channel tile oc0 / BN: one contiguous {w_hi, w_lo} image
          const float *src = p.w_tiles + ((size_t)(chunk0 * taps + it) * oc_tiles + oc0 / BN) * (2 * BN * KC);
          mbar_expect_tx(bar_wfull(s), (uint32_t)(2 * BN * KC * 4));
          bulk_load(smem_u32(wbase + s * 2 * kTileBytes), src, (uint32_t)(2 * BN * KC * 4), bar_wfull(s));
        }
      }
      if (!ok || *abort_flag)  // the copies of the last lap may still be in flight
        for (int v = max(g - p.w_stages, 0); v < g; ++v) mbar_drain(bar_wfull(v % p.w_stages), (uint32_t)(v / p.w_stages) & 1u);
    }
  } else if (warp == 1) {
    // ---- MMA issue.  The whole warp runs the loop converged and one elected lane issues, so
    //      that descriptors, addresses and the instruction descriptor stay in uniform registers
    //      (with a single lane of a diverged warp every MMA pays for moving its operands there,
    //      and the issuing thread, not the tensor pipe, sets the pace). ----
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    int g = 0, c = 0, sbase = 0;  // K step, group and first partial of the tile, counted across tiles
    int sw = 0;                   // weight stage of K step g
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, sbase += tile_supers) {
      for (int it0 = 0; it0 < iters && ok; it0 += kPromote, ++c) {
        const int gi = it0 / kPromote;
        const bool fresh = gi % kSuper == 0;            // the first MMA of a partial overwrites it
        const int b = (sbase + gi / kSuper) & 1;
        // (the converters have also waited for the summing warps to drain this partial accumulator)
        const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
        const int it1 = min(it0 + kPromote, iters);
        for (int it = it0; it < it1; ++it, ++g) {
          const int sa = g % kAStages;  // a power of two; the weight stage `sw` is counted
          // one wait per K step: afull stands for all inputs of the step (see the converters)
          if (!(ok = mbar_wait_warp(bar_afull(sa), (g / kAStages) & 1, abort_flag, lane))) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t dw = umma_desc(smem_u32(wbase + sw * 2 * kTileBytes));
          const uint32_t dlo = (uint32_t)dw, dhi = (uint32_t)(dw >> 32);
          const uint32_t ta = tmem_base + (uint32_t)(kTmemA + sa * 2 * KC);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < KC / 8; ++k) {  // 32 bytes along K = 2 in the address field; w_lo follows w_hi
              umma_tf32_ts(tmem_d, ta + k * 8, dlo + 2 * k, dhi, idesc, (!fresh || it > it0 || k) ? 1u : 0u);
              umma_tf32_ts(tmem_d, ta + KC + k * 8, dlo + 2 * k, dhi, idesc, 1u);
              umma_tf32_ts(tmem_d, ta + k * 8, dlo + 2 * k + (BN * KC * 4 >> 4), dhi, idesc, 1u);
            }
          }
          __syncwarp();
          if (++sw == p.w_stages) sw = 0;
        }
        if (ok && elect_one()) umma_commit(bar_gdone(c % kGroups));  // arrives when the group's last MMA has completed
        __syncwarp();
      }
    }
    if (!ok || *abort_flag) {  // the MMAs issued so far may still be running
      if (elect_one()) umma_commit(bar_drain());
      __syncwarp();
      mbar_drain(bar_drain(), 0);
    }
  } else if (warp == 3) {
    // ---- gatekeeper (one thread): collects, per K step, the conditions under which the
    //      converters may store the step's operand and the MMAs may run -- the weights have
    //      landed; at the first K step of a partial sum the summing warps have drained the
    //      accumulator it goes into (two partial sums ago); the MMAs that read the operand stage
    //      four K steps ago have completed -- and passes them on as ONE barrier.  A wait costs
    //      a converter warp 150-300 clocks even on a completed phase, and the converters'
    //      per-step latency is what limits the kernel.
    if (lane == 0) {
      int g = 0, sbase = 0, cbase = 0, ws = 0;
      uint32_t wphase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, sbase += tile_supers, cbase += tile_groups) {
        for (int it = 0; it < iters; ++it, ++g) {
          if (!(ok = mbar_wait(bar_wfull(ws), wphase, abort_flag))) break;
          if (it % (kPromote * kSuper) == 0) {
            const int sp = sbase + it / (kPromote * kSuper);
            if (!(ok = mbar_wait(bar_pempty(sp & 1), ((sp >> 1) & 1) ^ 1, abort_flag))) break;
          }
          if (g >= kAStages) {  // group of K step g - 4: two groups back in this tile, or near the end of the last
            const int cprev = it >= kAStages      ? cbase + (it - kAStages) / kPromote
                              : iters >= kAStages ? cbase - tile_groups + (iters + it - kAStages) / kPromote
                                                  : group_of(g - kAStages);  // tiles of fewer than 4 K steps
            if (!(ok = wait_group(cprev))) break;
          }
          mbar_arrive(bar_ready(g % kAStages));
          if (++ws == p.w_stages) { ws = 0; wphase ^= 1u; }
        }
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ---- warps 4..11: shared activation tile -> {x_hi, x_lo} in tensor memory.  A warp may
    //      touch only the TMEM lanes of its quarter (warp % 4); two warps share a quarter and
    //      take 16 of the 32 K columns each.  Row r keeps its 16-byte chunk c at c ^ (r & 7).
    //      Every warp handles every K step, in order: a parity wait cannot tell phase n from
    //      phase n + 2, so no warp may run a whole ring ahead of another.
    const int quarter = warp & 3, set = (warp - 4) >> 2;
    const int row = quarter * 32 + lane;
    // patch row of this thread's pixel for tap (0, 0); rows past the tile read row 0
    const int pw = row % p.TW, ph = (row / p.TW) % p.TH, pn = row / (p.TW * p.TH);
    const int prow0 = pn < p.NB ? (pn * p.PH + ph) * p.PW + pw : 0;
    const bool live = pn < p.NB;
    // Everything that depends on the K step is counted along (no divisions in this loop: the
    // converters' own instruction count is on the critical path).
    int g = 0, u = 0;                        // K step and patch of this CTA, counted across tiles
    int seen_u = -1;                         // patch this warp has already waited for
    // folded mode: this thread's pixel per item, item coordinates counted along in mixed radix
    const int radix[4] = {p.ksplit, oc_tiles, p.tiles_w, p.tiles_h};
    int cur[5] = {0, 0, 0, 0, 0}, step[5] = {0, 0, 0, 0, 0};
    if (p.folded) {
      int a = blockIdx.x, b2 = gridDim.x;
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        cur[d] = a % radix[d]; a /= radix[d];
        step[d] = b2 % radix[d]; b2 /= radix[d];
      }
      cur[4] = a; step[4] = b2;
    }
    const int fold_row = p.KS * p.IC, fold_k = p.KS * fold_row;       // floats per filter row / per filter
    const uint32_t rcp_row = 65536u / (uint32_t)max(fold_row, 1) + 1u;  // exact quotients for indices < 256
    const uint32_t rcp_ic = 65536u / (uint32_t)max(p.IC, 1) + 1u;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int tap = 0, r = 0, q = 0;
      // folded mode: input position of this thread's pixel for filter tap (0, 0)
      int f_ih0 = 0, f_iw0 = 0, f_chunk0 = 0;
      const float *f_img = nullptr;
      bool f_live = false;
      if (p.folded) {
        const int n = cur[4] * p.NB + pn, oh = cur[3] * p.TH + ph, ow = cur[2] * p.TW + pw;
        f_chunk0 = cur[0] * item_chunks;
        f_live = live && n < p.N && oh < p.OH && ow < p.OW;
        f_ih0 = oh * p.S - p.P; f_iw0 = ow * p.S - p.P;
        f_img = p.in + (size_t)(f_live ? n : 0) * p.H * p.W * p.IC;
        int carry = 0;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          cur[d] += step[d] + carry;
          carry = cur[d] >= radix[d] ? 1 : 0;
          cur[d] -= carry ? radix[d] : 0;
        }
        cur[4] += step[4] + carry;
      }
      for (int it = 0; it < iters; ++it, ++g) {
        const int sa = g % kAStages;
        // activation stage, its phase, and whether this K step is the last to read it
        const int sx = p.per_tap ? g % kXStages : u & 1;
        const uint32_t xphase = (uint32_t)(p.per_tap ? g / kXStages : u >> 1) & 1u;
        const bool last_of_chunk = tap == taps - 1;
        if ((g & 1) == set) {
          // Read and split this tap's rows first: everything up to the tensor-memory store can
          // be done while the operand stage is still in use.
          uint32_t hi[32], lo[32];
          if (p.folded) {
            // K index k = (filter row, filter column, channel): within a filter row the
            // (column, channel) pairs are contiguous in the NHWC input, so element k of this
            // pixel is img[(ih0 + row) * W * IC + iw0 * IC + rem] where it exists.
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const uint32_t k = (uint32_t)((f_chunk0 + it) * KC + c);
              const uint32_t fr = (k * rcp_row) >> 16, rem = k - fr * (uint32_t)fold_row;
              const int ih = f_ih0 + (int)fr, iw = f_iw0 + (int)((rem * rcp_ic) >> 16);
              const bool inside = f_live && (int)k < fold_k && ih >= 0 && ih < p.H && iw >= 0 && iw < p.W;
              hi[c] = inside ? __float_as_uint(__ldg(f_img + ((long long)ih * p.W + f_iw0) * p.IC + (int)rem)) : 0u;
            }
          } else {
          if (p.per_tap || seen_u != u) {  // a patch is waited for once, at the first tap this warp reads
            if (!(ok = mbar_wait_warp(bar_xfull(sx), xphase, abort_flag, lane))) break;
            seen_u = u;
          }
          const int prow = p.per_tap ? row : live ? prow0 + r * p.PW + q : 0;
          const unsigned char *src = xbase + (p.per_tap ? sx * kTileBytes : sx * kPatchBytes) + prow * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 v = *reinterpret_cast<const uint4 *>(src + ((c ^ (prow & 7)) << 4));
            hi[4 * c + 0] = v.x; hi[4 * c + 1] = v.y; hi[4 * c + 2] = v.z; hi[4 * c + 3] = v.w;
          }
          }
          // The MMA warp waits for afull only (a wait costs it ~150 clocks in which nothing is
          // issued, and the tensor pipe holds only ~250 clocks of queued work), so afull stands
          // for everything the MMAs of this K step need; the gatekeeper has collected the rest.
          if (!(ok = mbar_wait_warp(bar_ready(sa), (g / kAStages) & 1, abort_flag, lane))) break;
          // (the split comes after the wait so that the loads above are in flight during it)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            // x_hi is rounded to nearest, so the remainder's sign is random; the tensor core
            // then truncates the (up to 13-bit) remainder itself, an error of 2^-22 |x| without
            // a preferred sign -- rounding it here as well would cost two more operations per value
            const float v = __uint_as_float(hi[c]);
            hi[c] = round_tf32(v);
            lo[c] = __float_as_uint(v - __uint_as_float(hi[c]));
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(kTmemA + sa * 2 * KC);
          tmem_st32(taddr, hi);
          tmem_st32(taddr + KC, lo);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(bar_afull(sa));
            if (p.per_tap && !p.folded) mbar_arrive(bar_xempty(sx));  // a per-tap box has this one reader set
          }
        }
        // The patch is released by every warp once its own last K step of the chunk is behind
        // the tensor-memory store.  (Releasing a stage right after the loads, ahead of long
        // waits, produced wrong results on the 56x56 and 112x112 layers.)
        if (last_of_chunk) {
          __syncwarp();
          if (lane == 0 && !p.per_tap && !p.folded) mbar_arrive(bar_xempty(sx));
          ++u;
          tap = 0; r = 0; q = 0;
        } else {
          ++tap;
          if (++q == p.KS) { q = 0; ++r; }
        }
      }
    }
  } else if (warp >= 12) {
    // ---- warps 12..19: running sum in registers, store at the end of the tile ----
    constexpr int NC = BN / 2;             // channels per thread
    const int quarter = warp & 3, half = (warp - 12) >> 2;
    const int row = quarter * 32 + lane;   // tile row = pixel = TMEM lane
    const int pw = row % p.TW, ph = (row / p.TW) % p.TH, pn = row / (p.TW * p.TH);
    // 16-byte stores and adds need a 16-byte aligned output as well as whole groups of four channels
    const bool vec = (p.OC & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    const bool vec8 = (p.OC & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0;
    const bool small_out = (unsigned long long)p.N * p.OH * p.OW * p.OC < (1ull << 34);  // 32-bit offsets in 16-byte units
    int cbase = 0, sp = 0;  // first group of the tile; partial sum, counted across tiles
    // Item t = blockIdx.x + k * gridDim.x in mixed radix (K slice, channel tile, tile column,
    // tile row, image group): decoded once here and advanced by digit-wise addition per item
    // (eight divisions per item cost this warp ~900 clocks, measured, and on short-K layers
    // these warps set the pace).
    const int radix[4] = {p.ksplit, oc_tiles, p.tiles_w, p.tiles_h};
    int cur[5], step[5];
    {
      int a = blockIdx.x, b2 = gridDim.x;
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        cur[d] = a % radix[d]; a /= radix[d];
        step[d] = b2 % radix[d]; b2 /= radix[d];
      }
      cur[4] = a; step[4] = b2;
    }
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, cbase += tile_groups) {
      float acc[NC];
#pragma unroll
      for (int j = 0; j < NC; ++j) acc[j] = 0.f;
      for (int si = 0; si < tile_supers; ++si, ++sp) {
        const int b = sp & 1;
        // the partial sum is complete when its last group is
        if (!(ok = wait_group_warp(cbase + min((si + 1) * kSuper, tile_groups) - 1))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * BN + half * NC);
#pragma unroll
        for (int c0 = 0; c0 < NC; c0 += 16) {
          uint32_t v[16];
          tmem_ld16(taddr + c0, v);
          if (c0 + 16 == NC) {  // everything is in registers: the tensor core may overwrite the partial
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pempty(b));
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c0 + j] += __uint_as_float(v[j]);
        }
      }
      if (!ok) break;
      if (p.relu) {
#pragma unroll
        for (int j = 0; j < NC; ++j) acc[j] = fmaxf(acc[j], 0.f);
      }
      // the item's tile coordinates, counted along in mixed radix (see `step` below)
      const int w0 = cur[2] * p.TW, h0 = cur[3] * p.TH, n0 = cur[4] * p.NB, oc0 = cur[1] * BN;
      {
        int carry = 0;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          cur[d] += step[d] + carry;
          carry = cur[d] >= radix[d] ? 1 : 0;
          cur[d] -= carry ? radix[d] : 0;
        }
        cur[4] += step[4] + carry;
      }
      const int ow = w0 + pw, oh = h0 + ph, n = n0 + pn;
      const bool row_ok = pn < p.NB && ow < p.OW && oh < p.OH && n < p.N && !*abort_flag;
      const int ocb = oc0 + half * NC;
      float *o = p.out + (((size_t)n * p.OH + oh) * p.OW + ow) * p.OC + ocb;
      if (p.tma_store) {
        // Short K ranges, tiles of one image with 32 % TW == 0 that are 128 pixels large or span
        // the image's height: the 32 rows of a warp are 32 / TW whole tile rows, so the warp's 4 KiB
        // staging block -- 32 rows of 32 channels in the 128-byte swizzle -- is exactly a box
        // {32 channels, TW, 32 / TW, 1} of the NHWC output.  One lane hands it to a TMA store
        // and the warp carries on: the store's shared-memory reads and global writes run
        // behind the next tile's sums (loading the rows back and storing them with the LSU took
        // the warps ~3000 clocks per tile, more than the MMAs of a two-step K range).  Rows and
        // channels outside the tensor are dropped by the store.
        float4 *stage = reinterpret_cast<float4 *>(store_base + (warp - 12) * 4096);
#pragma unroll
        for (int h = 0; h < NC / 32; ++h) {
          if (ocb + h * 32 >= p.OC) break;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the block's last store has read it
          __syncwarp();
#pragma unroll
          for (int qq = 0; qq < 8; ++qq)
            stage[lane * 8 + (qq ^ (lane & 7))] = make_float4(acc[h * 32 + 4 * qq], acc[h * 32 + 4 * qq + 1],
                                                               acc[h * 32 + 4 * qq + 2], acc[h * 32 + 4 * qq + 3]);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0 && !*abort_flag) {
            asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                         ::"l"(&map_out), "r"(smem_u32(stage)), "r"(ocb + h * 32), "r"(w0), "r"(h0 + quarter * (32 / p.TW)), "r"(n0) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        continue;
      }
      if (vec && ocb + NC <= p.OC && small_out && p.w_stages == 4) {
        // Coalesced path.  A thread holds 32..64 channels of ONE pixel, so stored directly the
        // 32 lanes of an instruction hit 32 different lines (32 passes through the memory pipe
        // per instruction, 2048 per tile, and the converter warps' traffic queues behind
        // them: measured ~3400 idle tensor-pipe clocks per tile).  Through a 4 KiB staging
        // block per warp the rows are turned so that eight lanes write one pixel's 128
        // contiguous bytes: 4 passes per instruction, 512 per tile.
        float4 *stage = reinterpret_cast<float4 *>(store_base + (warp - 12) * 4096);
        // this thread's pixel as an offset into the output in 16-byte units (invalid: all ones)
        const uint32_t off16 = row_ok ? (uint32_t)((o - p.out) >> 2) : 0xFFFFFFFFu;
#pragma unroll
        for (int h = 0; h < NC / 32; ++h) {
#pragma unroll
          for (int qq = 0; qq < 8; ++qq)  // 16-byte piece qq of row `lane` sits at piece qq ^ (lane & 7)
            stage[lane * 8 + (qq ^ (lane & 7))] = make_float4(acc[h * 32 + 4 * qq], acc[h * 32 + 4 * qq + 1],
                                                               acc[h * 32 + 4 * qq + 2], acc[h * 32 + 4 * qq + 3]);
          __syncwarp();
          // all loads first: a store through a generic pointer may alias the staging block as far
          // as the compiler knows, which would serialise load, store, load, ...
          float4 v[8];
          const int qq = lane & 7;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3);
            v[i] = stage[r * 8 + (qq ^ (r & 7))];
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t off = __shfl_sync(0xffffffffu, off16, 4 * i + (lane >> 3));
            float *dst = p.out + ((size_t)off << 2) + h * 32 + 4 * qq;
            if (off != 0xFFFFFFFFu) {
              if (p.ksplit > 1)  // a slice of the K range: add into the zeroed output
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v[i].x), "f"(v[i].y), "f"(v[i].z), "f"(v[i].w) : "memory");
              else
                *reinterpret_cast<float4 *>(dst) = v[i];
            }
          }
          __syncwarp();
        }
        continue;
      }
      if (!row_ok) continue;
      if (p.ksplit > 1) {  // a slice of the K range: add into the zeroed output
        if (vec && ocb + NC <= p.OC) {
#pragma unroll
          for (int j = 0; j < NC; j += 4)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + j), "f"(acc[j]), "f"(acc[j + 1]), "f"(acc[j + 2]), "f"(acc[j + 3]) : "memory");
        } else {
#pragma unroll
          for (int j = 0; j < NC; ++j)
            if (ocb + j < p.OC) atomicAdd(o + j, acc[j]);
        }
      } else if (vec8 && ocb + NC <= p.OC) {
        // 32 bytes per lane: the 32 lanes of a store write 32 different lines either way, so
        // wider stores halve the passes through the memory pipe, which the tile's stores
        // otherwise hold for ~4000 clocks while the converter warps queue behind them
#pragma unroll
        for (int j = 0; j < NC; j += 8)
          asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(o + j), "f"(acc[j]), "f"(acc[j + 1]), "f"(acc[j + 2]), "f"(acc[j + 3]),
                       "f"(acc[j + 4]), "f"(acc[j + 5]), "f"(acc[j + 6]), "f"(acc[j + 7]) : "memory");
      } else if (vec && ocb + NC <= p.OC) {
#pragma unroll
        for (int j = 0; j < NC; j += 4) *reinterpret_cast<float4 *>(o + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < NC; ++j)
          if (ocb + j < p.OC) o[j] = acc[j];
      }
    }
    if (p.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // this warp's stores are complete
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.error_flag, 1);
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// Dense OIHW -> the images the weight loader copies: for every (32-channel chunk, tap, channel
// tile) a block {w_hi, w_lo} of BN rows x 128 bytes each, rows = output channels, already in the
// 128-byte-swizzled order the tensor core reads (16-byte chunk j of row r sits at chunk
// j ^ (r & 7)), so that one contiguous bulk copy fills a stage.  Channels past IC or OC are zero.
__global__ void tc_weight_tiles_kernel(const float *__restrict__ filt, float *__restrict__ tiles,
                                       int OC, int IC, int KS, int n_chunks, int oc_tiles, int BN, int folded) {
  const long long total = (long long)(folded ? 1 : KS * KS) * n_chunks * oc_tiles * 2 * BN * KC;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(i % KC);
    const int row = (int)((i / KC) % BN);
    const int half = (int)((i / ((long long)KC * BN)) % 2);
    long long tile = i / ((long long)2 * KC * BN);
    const int oct = (int)(tile % oc_tiles); tile /= oc_tiles;
    const int k = (((col >> 2) ^ (row & 7)) << 2) | (col & 3);
    const int oc = oct * BN + row;
    float w = 0.f;
    if (folded) {  // K index = (filter row, filter column, channel), cut into chunks of 32
      const int kk = (int)tile * KC + k;
      const int tap = kk / IC, ic = kk - tap * IC;
      if (tap < KS * KS && oc < OC) w = filt[((size_t)oc * IC + ic) * KS * KS + tap];
    } else {
      const int tap = (int)(tile % (KS * KS));  // K steps run chunk-major, tap-minor
      const int chunk = (int)(tile / (KS * KS));
      const int ic = chunk * KC + k;
      if (ic < IC && oc < OC) w = filt[((size_t)oc * IC + ic) * KS * KS + tap];
    }
    const float h = __uint_as_float(round_tf32(w));
    tiles[i] = half ? __uint_as_float(round_tf32(w - h)) : h;
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
               const cuuint32_t *box, const cuuint32_t *estr) {
  EncodeFn enc = get_encode();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return TETRIS_ERR_UNSUPPORTED; }
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, ptr, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return TETRIS_ERR_CUDA; }
  return TETRIS_OK;
}

struct TcState {
  float *d_tiles = nullptr;  // weight tile images
  int *d_error = nullptr;
  int n_chunks = 0, bn = 128;  // K chunks per tap; channel tile (fixed by the filter: 64 up to 64 channels)
  bool folded = false;         // <= 4 input channels: taps and channels folded into one K axis
  // Launch set-ups (tensor map of the input, tile plan, grid), one per (input pointer, conv
  // shape) seen lately: a caller that rotates over a few buffers -- the pipelined host path has
  // four -- finds its map again instead of encoding one per launch.  Round-robin replacement.
  struct Setup {
    bool valid = false;
    bool gated = false;          // set-ups of gated launches never split the K range
    const float *in = nullptr;
    const float *out = nullptr;  // (the output's tensor map belongs to the set-up too)
    ConvShape shape{};
    CUtensorMap map_x, map_out;
    TcParams params{};
    dim3 grid;
  };
  static constexpr int kSetups = 8;
  std::mutex mutex;
  Setup setups[kSetups];
  int next_setup = 0;
};

}  // namespace

void conv_tc_state_delete(void *state) {
  TcState *s = static_cast<TcState *>(state);
  if (!s) return;
  cudaFree(s->d_tiles); cudaFree(s->d_error);
  delete s;
}

// Builds the dense split weights and their tensor maps (called from filter creation, d_dense is
// the OIHW filter on the device).  Failure here is not fatal for the filter: the variant is then
// reported as unsupported.
int conv_tc_prepare(tetris_filter *f, const float *d_dense) {
  const bool folded = f->in_channel <= 4;
  if (f->groups != 1 || (!folded && (f->in_channel & 3) != 0)) return TETRIS_OK;  // not covered: leave tc_state null
  TcState *s = new (std::nothrow) TcState();
  if (!s) return TETRIS_OK;
  const int KS = f->kernel_size, taps = KS * KS;
  s->folded = folded;
  s->n_chunks = folded ? (taps * f->in_channel + KC - 1) / KC : (f->in_channel + KC - 1) / KC;
  s->bn = f->out_channel <= 64 ? 64 : 128;
  const int oc_tiles = (f->out_channel + s->bn - 1) / s->bn;
  const size_t elems = (size_t)(folded ? 1 : taps) * s->n_chunks * oc_tiles * 2 * s->bn * KC;
  if (cudaMalloc(&s->d_tiles, elems * 4) != cudaSuccess || cudaMalloc(&s->d_error, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    conv_tc_state_delete(s);
    return TETRIS_OK;
  }
  cudaMemset(s->d_error, 0, sizeof(int));
  tc_weight_tiles_kernel<<<(unsigned)std::min<size_t>((elems + 255) / 256, 4096), 256>>>(
      d_dense, s->d_tiles, f->out_channel, f->in_channel, KS, s->n_chunks, oc_tiles, s->bn, folded ? 1 : 0);
  if (cudaGetLastError() != cudaSuccess) {
    conv_tc_state_delete(s);
    return TETRIS_OK;
  }
  f->tc_state = s;
  return TETRIS_OK;
}

bool conv_tc_supported(const tetris_filter *f, const ConvShape &s) {
  if (!f->tc_state || f->groups != 1) return false;
  if (s.S < 1 || s.S > 8 || s.N < 1 || s.OH < 1 || s.OW < 1) return false;
  return static_cast<TcState *>(f->tc_state)->folded || (s.IC & 3) == 0;
}

namespace {
int launch_conv_tc_impl(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st,
                        unsigned *gate);
}

int launch_conv_tc(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st) {
  return launch_conv_tc_impl(f, in, out, s, st, nullptr);
}

// The same launch, conditional on the device: the kernel decides from gate[0] whether to run (see
// the kernel's first lines).  Such a launch never splits a tile's K range (the zeroing of the
// output that the split needs cannot be made conditional), so it overwrites the whole output
// when it runs.
int launch_conv_tc_gated(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st,
                         unsigned *gate) {
  return launch_conv_tc_impl(f, in, out, s, st, gate);
}

namespace {
int launch_conv_tc_impl(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st,
                        unsigned *gate) {
  TcState *t = static_cast<TcState *>(f->tc_state);
  if (!conv_tc_supported(f, s) || (!t->folded && (reinterpret_cast<uintptr_t>(in) & 15) != 0)) {
    set_error("tensor-core variant covers strides up to 8, in_channel <= 4 or a multiple of 4, 16-byte aligned inputs");
    return TETRIS_ERR_UNSUPPORTED;
  }
  CUtensorMap map_x, map_out;
  TcParams p;
  dim3 grid;
  int bn = 128;
  {
    std::lock_guard<std::mutex> lock(t->mutex);
    TcState::Setup *su = nullptr;
    for (TcState::Setup &c : t->setups) {
      const ConvShape &l = c.shape;
      if (c.valid && c.in == in && c.out == out && c.gated == (gate != nullptr) && l.relu == s.relu && l.N == s.N && l.H == s.H && l.W == s.W && l.P == s.P && l.S == s.S) { su = &c; break; }
    }
    if (!su) {
      su = &t->setups[t->next_setup];
      t->next_setup = (t->next_setup + 1) % TcState::kSetups;
      su->valid = false;
      // pixels of a tile: TW x TH x NB rows, at most 128, as full as possible, and -- at stride
      // 1, where all taps read one patch -- such that the tile with its halo fits a stage
      // (1x1 filters have no halo to share either, and the per-K-step ring is four deep)
      const bool per_tap = s.S > 1 || s.KS == 1 || t->folded;
      const int halo = per_tap ? 0 : s.KS - 1;
      int best_tw = 0, best_th = 1, best_nb = 1;
      double best = -1.0;
      bool best_boxy = false;
      for (int TW = 1; TW <= std::min(s.OW, 128); ++TW) {
        int TH = std::min(s.OH, 128 / TW);
        while (TH > 1 && (TW + halo) * (TH + halo) > kPatchRows) --TH;
        if (TH < 1 || (TW + halo) * (TH + halo) > kPatchRows || (!t->folded && (TW * s.S > 256 || TH * s.S > 256))) continue;
        int NB = (TH == s.OH && TW == s.OW) ? std::min(s.N, 128 / (TW * TH)) : 1;
        while (NB > 1 && (TW + halo) * (TH + halo) * NB > kPatchRows) --NB;
        const double tiles = (double)((s.OW + TW - 1) / TW) * ((s.OH + TH - 1) / TH) * ((s.N + NB - 1) / NB);
        const double eff = (double)s.N * s.OH * s.OW / (tiles * 128.0);
        // (among equally full tiles, one whose rows fill a warp's 32 lanes: see tma_store below)
        // (a tile shorter than 128 rows qualifies when it spans the image's height: the rows past
        // its end then lie below the image and the store drops them)
        const bool boxy = NB == 1 && 32 % TW == 0 && (TW * TH == 128 || TH == s.OH);
        if (eff > best + 1e-9 || (eff > best - 1e-9 && boxy && !best_boxy)) { best = eff; best_tw = TW; best_th = TH; best_nb = NB; best_boxy = boxy; }
      }
      if (best_tw == 0) {
        set_error("tensor-core variant: no tile of this layer fits an activation stage");
        return TETRIS_ERR_UNSUPPORTED;
      }
      const int PW = best_tw + halo, PH = best_th + halo;
      const cuuint64_t dims[4] = {(cuuint64_t)s.IC, (cuuint64_t)s.W, (cuuint64_t)s.H, (cuuint64_t)s.N};
      const cuuint64_t strides[3] = {(cuuint64_t)s.IC * 4, (cuuint64_t)s.IC * 4 * s.W, (cuuint64_t)s.IC * 4 * s.W * s.H};
      // with element strides the box spans S times the pixels it loads
      const cuuint32_t box[4] = {KC, (cuuint32_t)(PW * s.S), (cuuint32_t)(PH * s.S), (cuuint32_t)best_nb};
      const cuuint32_t estr[4] = {1, (cuuint32_t)s.S, (cuuint32_t)s.S, 1};
      if (!t->folded) {  // (folded mode reads the activations with plain loads)
        const int rc = encode_map(&su->map_x, const_cast<float *>(in), 4, dims, strides, box, estr);
        if (rc) return rc;
      }
      TcParams &q = su->params;
      q.N = s.N; q.OH = s.OH; q.OW = s.OW; q.OC = s.OC; q.P = s.P; q.KS = s.KS;
      q.TW = best_tw; q.TH = best_th; q.NB = best_nb;
      q.PW = PW; q.PH = PH;
      q.per_tap = per_tap ? 1 : 0; q.S = s.S;
      q.folded = t->folded ? 1 : 0; q.in = in; q.H = s.H; q.W = s.W; q.IC = s.IC;
      q.tiles_w = (s.OW + best_tw - 1) / best_tw;
      q.tiles_h = (s.OH + best_th - 1) / best_th;
      q.tiles_n = (s.N + best_nb - 1) / best_nb;
      q.n_chunks = t->n_chunks;
      q.w_tiles = t->d_tiles;
      q.error_flag = t->d_error;
      int dev = 0, sms = 0;
      TETRIS_CUDA_TRY(cudaGetDevice(&dev));
      TETRIS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      const long long tiles = (long long)q.tiles_w * q.tiles_h * q.tiles_n * ((s.OC + t->bn - 1) / t->bn);
      // Split the K range of every tile into d work items when that fills the waves of CTAs
      // better (e.g. 448 tiles on 148 SMs: 4 waves for 3.03 waves of work).  Cost in K steps:
      // waves x (K steps + ~10 for filling and draining the pipeline per item), plus zeroing
      // the output that the items add into.  Measured on 28x28x512 -> 512: 0.396 ms unsplit,
      // 0.357 ms in two slices, 0.349 ms in four.
      const double iters = (double)(t->folded ? 1 : s.KS * s.KS) * q.n_chunks;
      const double zeroing = ((double)s.N * s.OH * s.OW * s.OC * 4 / 6.0e12 + 3e-6) * 1.9e9 / 1450.0;
      int best_d = 1;
      double best_cost = std::ceil((double)tiles / sms) * (iters + 10.0);
      q.relu = s.relu;
      for (int d = 2; d <= 8 && d <= q.n_chunks && !f->deterministic && !gate && !s.relu; ++d) {
        if (q.n_chunks % d) continue;
        const double cost = std::ceil((double)tiles * d / sms) * (iters / d + 10.0) + zeroing;
        if (cost < 0.96 * best_cost) { best_cost = cost; best_d = d; }
      }
      q.ksplit = best_d;
      // Few K steps per work item: the epilogue weighs more than a deep weight ring (measured:
      // 18-step tiles 8 % faster with the staged stores, 144-step tiles 13 % slower on 4 stages).
      q.w_stages = iters / best_d <= 40.0 ? 4 : 5;
      // TMA stores from the staging blocks (see the kernel's epilogue): short K ranges on large
      // images, whole tiles of one image whose rows fill a warp's 32 lanes
      q.tma_store = 0;
      std::memset(&su->map_out, 0, sizeof(su->map_out));
      if (q.w_stages == 4 && best_d == 1 && best_nb == 1 && 32 % best_tw == 0 && (best_tw * best_th == 128 || best_th == s.OH) &&
          (s.OC & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        const cuuint64_t odims[4] = {(cuuint64_t)s.OC, (cuuint64_t)s.OW, (cuuint64_t)s.OH, (cuuint64_t)s.N};
        const cuuint64_t ostrides[3] = {(cuuint64_t)s.OC * 4, (cuuint64_t)s.OC * 4 * s.OW, (cuuint64_t)s.OC * 4 * s.OW * s.OH};
        const cuuint32_t obox[4] = {32, (cuuint32_t)best_tw, (cuuint32_t)(32 / best_tw), 1};
        const cuuint32_t oestr[4] = {1, 1, 1, 1};
        if (encode_map(&su->map_out, out, 4, odims, ostrides, obox, oestr) == TETRIS_OK) q.tma_store = 1;
      }
      const long long total = tiles * best_d;
      su->grid = dim3((unsigned)std::min<long long>(total, sms));  // persistent: one CTA per SM
      su->in = in;
      su->out = out;
      su->gated = gate != nullptr;
      su->shape = s;
      su->valid = true;
    }
    map_x = su->map_x;
    map_out = su->map_out;
    p = su->params;
    grid = su->grid;
    bn = t->bn;
  }
  p.out = out;
  p.in = in;
  p.gate = gate;
  p.withhold_first_load = test_injection(&p.spin_limit);
  const size_t smem = (size_t)kSmemTiles + 1024 + kNumBars * 8 + 16;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(conv_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(conv_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 16) configured[dev] = true;
  }
  if (p.ksplit > 1)  // the work items add into the output
    TETRIS_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)s.N * s.OH * s.OW * s.OC * sizeof(float), st));
  if (bn == 64)
    conv_tc_kernel<64><<<grid, kThreads, smem, st>>>(map_x, map_out, p);
  else
    conv_tc_kernel<128><<<grid, kThreads, smem, st>>>(map_x, map_out, p);
  TETRIS_CUDA_TRY(cudaGetLastError());
  if (!gate) count_launch();
  if (p.relu) note_relu_fused();
  return TETRIS_OK;
}
}  // namespace

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
