// Dense contraction on the 5th-generation tensor cores in SPLIT FP16: the stride-1 layers' fast
// variant (tcgen05.mma kind::f16 + tcgen05.cp + TMEM + TMA).
//
// Arithmetic.  x = x_hi + x_lo and w' = w * 2^sh = w_hi + w_lo with *_hi the value rounded to
// FP16 (11 significant bits) and *_lo the FP16-rounded remainder; D += x_hi*w_hi + x_lo*w_hi +
// x_hi*w_lo in FP32 accumulators, scaled back by 2^-sh (exact) at the store; sh is chosen per
// OUTPUT CHANNEL, so channels of very different magnitude keep their own full precision.  The products are
// exact in FP32; what is dropped is x_lo*w_lo and the rounding of the remainders, about 2^-22 of
// a product each -- the same as the split-TF32 variant (conv_tc.cu), at twice the tensor-core
// rate and half the operand bytes.  sh puts a channel's largest |w'| at about 2^13: weights down
// to 2^-17 of the channel's largest keep a normal FP16 remainder.  Activations are
// scaled by a fixed 16 (their range is not known before the launch), which puts FP16's window at
// |x| < 2048 with remainders exact down to |x| = 2^-7 and an absolute error of at most 2e-9 per
// activation below that.  The conversion warps record the largest magnitude of the launch in
// global memory; the launcher has queued the split-TF32 variant behind this kernel, which
// starts, reads that maximum and recomputes the whole layer when it is 2048 or more (or NaN or
// infinity) -- FP16 would overflow -- or below 2^-8 -- all activations so small that the
// absolute error above would show in the relative accuracy -- and returns at once otherwise.
// Results are therefore FP32-accurate for any input.
//
// As in the split-TF32 variant the tensor core accumulates 48 MMAs (8 K steps) from zero into a
// partial accumulator and CUDA-core warps add the partials to a running sum in registers (the
// tensor core truncates when it adds into its accumulator; see conv_tc.cu).
//
// Structure.  GEMM view: M = 128 pixels = 16 groups of 8 consecutive output columns, N = 128
// (64) output channels, K = (32-channel chunk, filter tap).  What differs from conv_tc.cu is how
// the M-side operand reaches tensor memory.  There, converter warps rebuild the operand of every
// tap from the activation patch (nine times per patch for a 3x3 filter) and that conversion, not
// the tensor pipe, set the pace.  Here the patch is converted ONCE, in place, in shared memory
// (each 128-byte row of 32 FP32 channels becomes 32 x_hi and 32 x_lo FP16 values), and the
// operand of a tap is a WINDOW of the converted patch: tcgen05.cp copies 128 rows x 32 bytes from
// shared to tensor memory through a matrix descriptor whose start address is shifted by the
// tap's (row, column) offset and whose 8-row groups are PW rows apart (PW = patch width).  The
// 128-byte swizzle is a function of the shared-memory address, so a window that starts at any
// 128-byte row reads back exactly what the TMA load and the in-place conversion wrote.
//   * warp 0 (one thread): one TMA load per 32-channel chunk of the tile's pixels with their
//     halo (4-D box, out-of-range coordinates zero-filled = the padding) into a ring of stages;
//   * warps 4-7: convert a landed patch in place, one 128-byte row per thread, conflict-free;
//   * warp 3 (one elected lane): per K step four tcgen05.cp (x_hi and x_lo, two K slices each)
//     into one of the operand blocks; per GROUP of U K steps (U = 2, or 4 for 64-channel tiles
//     under filters larger than 1x1) one wait (the MMAs that read the block a lap ago are done)
//     and one commit;
//   * warp 2 (one thread): one bulk copy per group of K steps of prepared {w_hi, w_lo} tile images;
//   * warp 1 (one elected lane): 6 tcgen05.mma per K step; per group two waits (operands copied,
//     weights landed) and one commit.  The pipeline's unit is a group of K steps because a wait
//     costs a warp ~200 clocks and a commit ~250, against ~450 for the twelve MMAs of a pair;
//   * warps 8-15: partial accumulators -> running sum in registers -> staged, coalesced stores.
// Every barrier wait is bounded; on a timeout an error flag is raised, all roles drain, TMEM is
// freed and the kernel returns; the host reports TETRIS_ERR_CUDA.
//
// 1x1 filters take the same pipeline with M = 128 consecutive pixels of the flattened image
// (no halo, 100 % full tiles).  Mid-size images (28 x 28, 52 x 52 ...), which 8 x 16 tiles cut
// badly, are walked in their padded-width layout instead (`flat`, see launch_conv_tc16).  Covers stride 1, IC % 4 == 0 (TMA strides), KS <= 7.
// No cluster launch: every load is issued by one CTA for itself.
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <mutex>

#include "internal.h"

namespace tetris {
namespace {

constexpr int BM = 128, KC = 32;         // tile rows (pixels); K chunk (32 channels)
constexpr int kTW = 8, kTH = 16;         // a tile is 16 groups of 8 output columns
constexpr int kAStagesMax = 4;           // operand blocks in tensor memory: one per group of U K steps, 256 / (32 U) of them
constexpr int kStepCols = 32;            // per K step {x_hi k0, x_hi k1, x_lo k0, x_lo k1} x 8 columns
constexpr int kTmemCols = 512;           // 2 partial accumulators (<= 128 columns each) + 8 x 32 operand columns
constexpr int kTmemA = 256;
constexpr int kWStagesMax = 4, kXStagesMax = 6;   // weight stages hold a group of K steps
constexpr int kGroups = 16;              // "group done" barriers in rotation (a power of two, 2^4: see wait_group)
constexpr int kSuperSteps = 8;           // K steps (48 MMAs) accumulated on the tensor core before the FP32 add outside
constexpr int kThreads = 512;            // warp 0 x loads, 1 MMA, 2 w loads, 3 cp, 4-7 convert, 8-15 sum + store
constexpr int kStoreBytes = 8 * 4096;    // store staging: per summing warp 32 rows x 32 channels
constexpr int kNumBars = 3 * kXStagesMax + kWStagesMax + kAStagesMax + kGroups + 2 + 2;   // (... + two drain barriers + two partial-sum barriers)
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr float kXScale = 16.f;          // activations are multiplied by this before the split (undone in out_scale)

struct Tc16Params {
  float *out;
  int N, OH, OW, OC, P, KS;
  int linear;                  // 1x1 filters: a tile is 128 consecutive pixels of the flattened N*OH*OW image
  int flat;                    // a tile is 128 consecutive positions of one image laid out with its padded width
                               // PW = W + 2P (positions past OW in a row are computed and dropped)
  int PW;                      // patch width in pixels (kTW + KS - 1; flat mode: W + 2P); 8 in linear mode
  int PHI;                     // patch rows one image occupies in a stage
  int TH, NB;                  // output rows and images of a tile
  int box_rows;                // 128-byte rows a patch load delivers
  int x_stage_bytes, n_x;      // activation stage size and ring depth
  int n_w;                     // weight ring depth
  int tiles_w, tiles_h, tiles_n;
  int n_chunks, ksplit;
  // Tail split: the tiles that would form a last, nearly empty wave of CTAs (tiles tail_tile0 ...)
  // are cut into tail_d K slices each (work items tail_start ...); the slices leave their sums in
  // `scratch`, and whichever finishes last (tail_count) adds them up in slice order and stores.
  int tail_start, tail_tile0, tail_d;
  float *scratch;
  int *tail_count;
  int relu;                    // max(y, 0) at the store (never together with a split K range)
  long long total_pixels;      // N * OH * OW (linear mode)
  const float *out_scale;      // per output channel: 2^-sh[oc] / 16 (undoes the weight and activation scaling)
  int *error_flag;
  unsigned *gate;              // gate[0]: largest |activation| of the launch, as FP32 bits (see launch_conv_tc_gated)
  const __half *w_tiles;
  unsigned spin_limit;         // polls after which a barrier wait gives up (0: kSpinLimit)
  int withhold_first_load;     // failure-detection test only: every CTA leaves out its first activation load
  long long *prof;             // per-role clock totals of CTA 0 for TETRIS_TC16_PROF=1 (nullptr = off)
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
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
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
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// K-major operand, 128-byte rows, 128B swizzle; 8-row groups `sbo_bytes` apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t sbo_bytes) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
  return pred != 0;
}
// shared -> tensor memory: 128 rows x 32 bytes into 8 columns
__device__ __forceinline__ void tmem_cp(uint32_t taddr, uint32_t d_lo, uint32_t d_hi) {
  asm volatile("{\n.reg .b64 d;\nmov.b64 d, {%1, %2};\ntcgen05.cp.cta_group::1.128x256b [%0], d;\n}" ::"r"(taddr), "r"(d_lo), "r"(d_hi) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor], FP16 operands, FP32 accumulate
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t db_lo, uint32_t db_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\n.reg .b64 d;\nmov.b64 d, {%2, %3};\nsetp.ne.b32 p, %5, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d, %4, p;\n}"
               ::"r"(tmem_d), "r"(tmem_a), "r"(db_lo), "r"(db_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// BN: output channels of a tile.  U: K steps per pipeline group -- the unit the copy warp and the
// MMA warp wait, issue and commit by (2 for BN = 128; 4 for BN = 64, whose MMAs are short enough
// that a wait and a commit per pair of steps would set the pace).
template <int BN, int U>
__global__ void __launch_bounds__(kThreads, 1)
conv_tc16_kernel(const __grid_constant__ CUtensorMap map_x, const Tc16Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *xbase = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  unsigned char *wbase = xbase + (size_t)p.n_x * p.x_stage_bytes;
  constexpr int kWBytes = BN * 128;      // weights of one K step: BN rows of {w_hi (64 B), w_lo (64 B)}; a stage holds U
  constexpr int kAStages = 256 / (kStepCols * U);   // operand blocks in rotation (a power of two)
  constexpr int kSuper = kSuperSteps / U;           // groups per partial sum
  static_assert(kAStages <= kAStagesMax && kAStages * kStepCols * U == 256 && kSuper * U == kSuperSteps, "group size");
  unsigned char *store_base = wbase + (size_t)p.n_w * U * kWBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(store_base + kStoreBytes);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar_xfull = [&](int s) { return smem_u32(&bars[s]); };
  auto bar_xconv = [&](int s) { return smem_u32(&bars[kXStagesMax + s]); };
  auto bar_xempty = [&](int s) { return smem_u32(&bars[2 * kXStagesMax + s]); };
  auto bar_wfull = [&](int s) { return smem_u32(&bars[3 * kXStagesMax + s]); };
  auto bar_afull = [&](int s) { return smem_u32(&bars[3 * kXStagesMax + kWStagesMax + s]); };
  auto bar_gdone = [&](int c) { return smem_u32(&bars[3 * kXStagesMax + kWStagesMax + kAStagesMax + c]); };
  auto bar_pempty = [&](int b) { return smem_u32(&bars[kNumBars - 2 + b]); };
  auto bar_drain = [&](int b) { return smem_u32(&bars[kNumBars - 4 + b]); };

  if (tid == 0) {
    for (int s = 0; s < kXStagesMax; ++s) { mbar_init(bar_xfull(s), 1); mbar_init(bar_xconv(s), 4); mbar_init(bar_xempty(s), 1); }
    for (int s = 0; s < kWStagesMax; ++s) mbar_init(bar_wfull(s), 1);
    for (int s = 0; s < kAStages; ++s) mbar_init(bar_afull(s), 1);
    for (int c = 0; c < kGroups; ++c) mbar_init(bar_gdone(c), 1);
    for (int b = 0; b < 2; ++b) { mbar_init(bar_pempty(b), 8); mbar_init(bar_drain(b), 1); }
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
  // Timeline aid, compiled in with -DTETRIS_TC16_PROF only: clocks per role of CTA 0, in total
  // and inside its waits, printed by the launcher when the environment has TETRIS_TC16_PROF=1.
#ifdef TETRIS_TC16_PROF
  const bool prof_on = p.prof != nullptr && blockIdx.x == 0;
  long long pw[7] = {0, 0, 0, 0, 0, 0, 0};
  const long long prof_t0 = prof_on ? clock64() : 0;
#define TIMED(slot, expr) ([&]() { const long long t0_ = prof_on ? clock64() : 0; const bool r_ = (expr); if (prof_on) pw[slot] += clock64() - t0_; return r_; }())
#define PROF_OUT(role) do { if (prof_on && lane == 0) { p.prof[(role) * 8] = clock64() - prof_t0; for (int i_ = 0; i_ < 7; ++i_) p.prof[(role) * 8 + 1 + i_] = pw[i_]; } } while (0)
#define PROF_LAP(slot) do { if (prof_on) { const long long n_ = clock64(); pw[slot] += n_ - ts0; ts0 = n_; } } while (0)
#define PROF_START() long long ts0 = prof_on ? clock64() : 0
#else
#define TIMED(slot, expr) (expr)
#define PROF_OUT(role) do { } while (0)
#define PROF_LAP(slot) do { } while (0)
#define PROF_START() do { } while (0)
#endif

  // Persistent CTA: work items blockIdx.x, blockIdx.x + gridDim.x, ...; the channel tile is the
  // fastest index, so CTAs that run side by side read the same activation patch.
  const int taps = p.KS * p.KS;
  const int oc_tiles = (p.OC + BN - 1) / BN;
  const int total_tiles = p.tiles_w * p.tiles_h * p.tiles_n * oc_tiles;
  const int total_items = p.tail_start + (total_tiles - p.tail_tile0) * p.tail_d;
  // A work item is a tile, or one of ksplit equal slices of a tile's K range (all tiles), or --
  // for the tiles of the last wave -- one of tail_d slices.  The pipeline's unit is a GROUP of U K
  // steps (the last of an item may be shorter).
  struct Item { int tile, chunk0, chunks, iters, ngroups, supers; bool tail; int slice; };
  auto item_of = [&](int t) {
    Item it;
    it.tail = t >= p.tail_start;
    const int d = it.tail ? p.tail_d : p.ksplit, u = it.tail ? t - p.tail_start : t;
    it.slice = u % d;
    it.tile = (it.tail ? p.tail_tile0 : 0) + u / d;
    it.chunks = p.n_chunks / d;
    it.chunk0 = it.slice * it.chunks;
    it.iters = taps * it.chunks;
    it.ngroups = (it.iters + U - 1) / U;
    it.supers = (it.ngroups + kSuper - 1) / kSuper;
    return it;
  };
  auto decode = [&](int t, int &w0, int &h0, int &n0, int &oc0) {
    oc0 = (t % oc_tiles) * BN; t /= oc_tiles;
    w0 = (t % p.tiles_w) * kTW; t /= p.tiles_w;       // (linear mode: tiles_w = number of 128-pixel tiles)
    h0 = (t % p.tiles_h) * p.TH;
    n0 = (t / p.tiles_h) * p.NB;
  };
  // Group G of this CTA (counted across work items) signals bar_gdone(G % kGroups) when its MMAs
  // have completed.  Nobody looks at a group's barrier later than 16 groups after it: the rings are
  // at most 4 groups deep and the MMAs run at most two partial sums (8 groups) ahead of the summing warps.
  auto wait_group = [&](int G) { return mbar_wait(bar_gdone(G & (kGroups - 1)), (G >> 4) & 1, abort_flag); };
  auto wait_group_warp = [&](int G) { return mbar_wait_warp(bar_gdone(G & (kGroups - 1)), (G >> 4) & 1, abort_flag); };

  if (warp == 0) {
    // ---- activation loads: one patch (tile + halo) per 32-channel chunk ----
    if (lane == 0) {
      const uint32_t box_bytes = (uint32_t)p.box_rows * 128u;
      int s = 0, loads = 0;
      uint32_t phase = 1;  // (a fresh barrier lets the first lap through)
      bool ok = true;
      for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
        const Item it = item_of(t);
        int w0, h0, n0, oc0;
        decode(it.tile, w0, h0, n0, oc0);
        for (int chunk = it.chunk0; chunk < it.chunk0 + it.chunks; ++chunk) {
          if (!(ok = TIMED(0, mbar_wait(bar_xempty(s), phase, abort_flag)))) break;
          if (loads++ == 0 && p.withhold_first_load) {  // (test: this patch never arrives, its readers give up)
            if (++s == p.n_x) { s = 0; phase ^= 1u; }
            continue;
          }
          mbar_expect_tx(bar_xfull(s), box_bytes);
          if (p.linear)
            tma_load_4d(smem_u32(xbase + (size_t)s * p.x_stage_bytes), &map_x, bar_xfull(s), chunk * KC, (w0 / kTW) * BM, 0, 0);
          else if (p.flat)  // whole padded rows, from the row above the tile's first output row
            tma_load_4d(smem_u32(xbase + (size_t)s * p.x_stage_bytes), &map_x, bar_xfull(s), chunk * KC, -p.P,
                        ((w0 / kTW) * BM) / p.PW - p.P, n0);
          else
            tma_load_4d(smem_u32(xbase + (size_t)s * p.x_stage_bytes), &map_x, bar_xfull(s), chunk * KC, w0 - p.P, h0 - p.P, n0);
          if (++s == p.n_x) { s = 0; phase ^= 1u; }
        }
      }
      if (!ok || *abort_flag) {  // the loads of the last lap may still be in flight
        for (int v = max(loads - p.n_x, p.withhold_first_load ? 1 : 0); v < loads; ++v)
          mbar_drain(bar_xfull(v % p.n_x), (uint32_t)(v / p.n_x) & 1u);
      }
      PROF_OUT(0);
    }
  } else if (warp == 2) {
    // ---- weight loads: one bulk copy per group (the {w_hi, w_lo} images of its K steps lie
    //      back to back in global memory) ----
    if (lane == 0) {
      int G = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
        const Item it = item_of(t);
        const int iters = it.iters, ngroups = it.ngroups;
        int w0, h0, n0, oc0;
        decode(it.tile, w0, h0, n0, oc0);
        const __half *item = p.w_tiles + ((size_t)(oc0 / BN) * p.n_chunks + it.chunk0) * taps * (size_t)(BN * 64);
        for (int j = 0; j < ngroups; ++j, ++G) {
          const int s = G % p.n_w;
          if (G >= p.n_w && !(ok = TIMED(0, wait_group(G - p.n_w)))) break;
          const uint32_t bytes = (uint32_t)(min(U, iters - U * j) * kWBytes);
          mbar_expect_tx(bar_wfull(s), bytes);
          bulk_load(smem_u32(wbase + (size_t)s * U * kWBytes), item + (size_t)(U * j) * (BN * 64), bytes, bar_wfull(s));
        }
      }
      if (!ok || *abort_flag) {  // the copies of the last lap may still be in flight
        for (int v = max(G - p.n_w, 0); v < G; ++v) mbar_drain(bar_wfull(v % p.n_w), (uint32_t)(v / p.n_w) & 1u);
      }
      PROF_OUT(1);
    }
  } else if (warp == 3) {
    // ---- operand copies (converged warp, one elected lane issues, so that descriptors and
    //      addresses stay in uniform registers): per K step four tcgen05.cp -- the tap's window of
    //      the converted patch -> the step's operand block in tensor memory; one wait and one
    //      commit per pair.  Everything that depends on the K step is counted along: the issuing
    //      thread's own instructions, not the tensor unit, set the pace otherwise. ----
    const uint32_t sbo = (uint32_t)((p.linear || p.flat) ? 1024 : p.PW * 128);
    const uint32_t da_hi = (uint32_t)(smem_desc(0, sbo) >> 32);
    const uint32_t x0 = (uint32_t)smem_desc(smem_u32(xbase), sbo);       // descriptor (low word) of stage 0, tap (0, 0)
    const uint32_t stage_step = (uint32_t)(p.x_stage_bytes >> 4);        // ... one stage further
    const uint32_t row_step = (uint32_t)((p.PW - p.KS + 1) * 128 >> 4);  // ... from the end of a filter row to the next row
    int G = 0, sx = 0;
    uint32_t xd = x0, td = 0;  // descriptor of the current stage; offset of the current tap
    uint32_t xphase = 0;       // phase of the "converted" barrier of stage sx
    bool fresh_patch = true;   // the patch in stage sx has not been waited for yet
    bool ok = true;
    for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
      int r = 0, q = 0;  // tap of the next K step
      // flat mode: the tile's first position lies (P0 mod PW) rows into its first padded row
      const Item it = item_of(t);
      const int iters = it.iters, ngroups = it.ngroups;
      uint32_t td0 = 0;
      if (p.flat) {
        const int P0 = ((it.tile / oc_tiles) % p.tiles_w) * BM;
        td0 = (uint32_t)((P0 - (P0 / p.PW) * p.PW) * 8);
      }
      td = td0;
      for (int j = 0; j < ngroups; ++j, ++G) {
        const int sa = G & (kAStages - 1);
        const int ns = min(U, iters - U * j);
        // the MMAs that read this operand block (kAStages groups ago) are done
        if (G >= kAStages && !(ok = TIMED(0, wait_group_warp(G - kAStages)))) break;
        // per step: the window of its tap in the converted patch (waited for once per patch), and
        // the barrier that releases the patch if this step is its last
        uint32_t a[U], freed[U];
#pragma unroll
        for (int e = 0; e < U; ++e) {
          a[e] = 0; freed[e] = 0;
          if (e < ns && ok) {
            if (fresh_patch) {
              ok = TIMED(1, mbar_wait_warp(bar_xconv(sx), xphase, abort_flag));
              fresh_patch = false;
            }
            a[e] = xd + td;
            if (r == p.KS - 1 && q == p.KS - 1) {
              freed[e] = bar_xempty(sx);
              r = 0; q = 0; td = td0; fresh_patch = true;
              if (++sx == p.n_x) { sx = 0; xd = x0; xphase ^= 1u; } else xd += stage_step;
            }
            else if (++q == p.KS) { q = 0; ++r; td += row_step; }
            else td += 8;
          }
        }
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t ta = tmem_base + (uint32_t)(kTmemA + sa * (kStepCols * U));
        if (elect_one()) {
          // operand block of a K step: columns 0-7 / 8-15 x_hi of channels 0-15 / 16-31, 16-23 / 24-31 x_lo
          // (32 bytes along K = 2 in a descriptor's address field)
#pragma unroll
          for (int e = 0; e < U; ++e) {
            if (e < ns) {
              const uint32_t te = ta + (uint32_t)(e * kStepCols);
              tmem_cp(te, a[e], da_hi); tmem_cp(te + 8, a[e] + 2, da_hi); tmem_cp(te + 16, a[e] + 4, da_hi); tmem_cp(te + 24, a[e] + 6, da_hi);
              if (freed[e]) umma_commit(freed[e]);  // the patch has been read for the last time
            }
          }
          umma_commit(bar_afull(sa));
        }
        __syncwarp();
      }
    }
    if (!ok || *abort_flag) {  // the copies issued so far may still be running
      if (elect_one()) umma_commit(bar_drain(0));
      __syncwarp();
      mbar_drain(bar_drain(0), 0);
    }
    PROF_OUT(2);
  } else if (warp == 1) {
    // ---- MMA issue (converged warp, one elected lane): six tcgen05.mma per K step, one wait and
    //      one commit per group ----
    const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    const uint32_t dw_hi = (uint32_t)(smem_desc(0, 1024) >> 32);
    const uint32_t w0 = (uint32_t)smem_desc(smem_u32(wbase), 1024);
    int G = 0, sw = 0, sbase = 0, sp = 0;
    uint32_t wd = w0, wphase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
      const Item it = item_of(t);
      const int iters = it.iters, ngroups = it.ngroups;
      const int sbase0 = sbase;
      sbase += it.supers;
      for (int j = 0, jj = 0, si = 0; j < ngroups; ++j, ++G) {
        const int sa = G & (kAStages - 1);
        const uint32_t acc0 = jj == 0 ? 0u : 1u;  // the first MMA of a partial overwrites it
        const uint32_t tmem_d = tmem_base + (uint32_t)(((sbase0 + si) & 1) * BN);
        if (jj == 0) {  // first group of a partial sum: its accumulator has been drained (two partials ago)
          if (!(ok = TIMED(1, mbar_wait_warp(bar_pempty(sp & 1), ((sp >> 1) & 1) ^ 1, abort_flag)))) break;
          ++sp;
        }
        if (++jj == kSuper) { jj = 0; ++si; }
        if (!(ok = TIMED(2, mbar_wait_warp(bar_wfull(sw), wphase, abort_flag)))) break;  // the group's weights have landed
        if (!(ok = TIMED(0, mbar_wait_warp(bar_afull(sa), (G / kAStages) & 1, abort_flag)))) break;  // ... and its operand blocks
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        PROF_START();
        const int ns = min(U, iters - U * j);
        const uint32_t ta = tmem_base + (uint32_t)(kTmemA + sa * (kStepCols * U));
        const uint32_t dlo = wd;
        if (++sw == p.n_w) { sw = 0; wd = w0; wphase ^= 1u; } else wd += (uint32_t)(U * kWBytes >> 4);
        if (elect_one()) {
          // K slices of 16 channels: 32 bytes = 2 in the address field; w_lo sits 64 bytes after w_hi
#pragma unroll
          for (int e = 0; e < U; ++e) {
            if (e < ns) {
              const uint32_t te = ta + (uint32_t)(e * kStepCols), de = dlo + (uint32_t)(e * (kWBytes >> 4));
              umma_f16_ts(tmem_d, te, de, dw_hi, idesc, e == 0 ? acc0 : 1u);
              umma_f16_ts(tmem_d, te + 16, de, dw_hi, idesc, 1u);
              umma_f16_ts(tmem_d, te, de + 4, dw_hi, idesc, 1u);
              umma_f16_ts(tmem_d, te + 8, de + 2, dw_hi, idesc, 1u);
              umma_f16_ts(tmem_d, te + 24, de + 2, dw_hi, idesc, 1u);
              umma_f16_ts(tmem_d, te + 8, de + 6, dw_hi, idesc, 1u);
            }
          }
          PROF_LAP(3);
          umma_commit(bar_gdone(G & (kGroups - 1)));
          PROF_LAP(4);
        }
        __syncwarp();
      }
    }
    if (!ok || *abort_flag) {  // the MMAs issued so far may still be running
      if (elect_one()) umma_commit(bar_drain(1));
      __syncwarp();
      mbar_drain(bar_drain(1), 0);
    }
    PROF_OUT(3);
  } else if (warp >= 4 && warp < 8) {
    // ---- warps 4..7: a landed patch, in place: each 128-byte row of 32 FP32 channels becomes
    //      {x_hi[32], x_lo[32]} FP16.  One row per thread: the 16-byte chunks of row r sit at
    //      chunk ^ (r & 7) before and after, so the eight lanes of a quarter-warp touch eight
    //      different bank groups. ----
    const int ct = (warp - 4) * 32 + lane;
    int u = 0;
    bool ok = true;
    uint32_t seen_max = 0;
    for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
      const int item_chunks = item_of(t).chunks;
      for (int chunk = 0; chunk < item_chunks; ++chunk, ++u) {
        const int sx = u % p.n_x;
        if (!(ok = TIMED(0, mbar_wait_warp(bar_xfull(sx), (u / p.n_x) & 1, abort_flag)))) break;
        unsigned char *stage = xbase + (size_t)sx * p.x_stage_bytes;
        for (int row = ct; row < p.box_rows; row += 128) {
          uint4 *rp = reinterpret_cast<uint4 *>(stage + (size_t)row * 128);
          const int sw = row & 7;
          uint4 v[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) v[c] = rp[c ^ sw];
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float x0 = kXScale * __uint_as_float(v[c].x), x1 = kXScale * __uint_as_float(v[c].y),
                        x2 = kXScale * __uint_as_float(v[c].z), x3 = kXScale * __uint_as_float(v[c].w);
            seen_max = max(seen_max, max(max(v[c].x & 0x7FFFFFFFu, v[c].y & 0x7FFFFFFFu), max(v[c].z & 0x7FFFFFFFu, v[c].w & 0x7FFFFFFFu)));
            const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            hi[2 * c] = *reinterpret_cast<const uint32_t *>(&h01);
            hi[2 * c + 1] = *reinterpret_cast<const uint32_t *>(&h23);
            lo[2 * c] = pack_half2(x0 - f01.x, x1 - f01.y);
            lo[2 * c + 1] = pack_half2(x2 - f23.x, x3 - f23.y);
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            rp[c ^ sw] = make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
            rp[(c + 4) ^ sw] = make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
          }
        }
        // the writes above go through the generic proxy, tcgen05.cp reads through the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_xconv(sx));
      }
    }
    // the launch's largest magnitude: the guard kernel behind this one decides on it
    for (int d = 16; d; d >>= 1) seen_max = max(seen_max, __shfl_xor_sync(0xffffffffu, seen_max, d));
    if (lane == 0 && seen_max) atomicMax(p.gate, seen_max);
    if (warp == 4) PROF_OUT(4);
  } else if (warp >= 8) {
    // ---- warps 8..15: running sum in registers, store at the end of the work item ----
    constexpr int NC = BN / 2;             // channels per thread
    const int quarter = warp & 3, half = (warp - 8) >> 2;
    const int row = quarter * 32 + lane;   // tile row = pixel = TMEM lane
    const bool vec = (p.OC & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    const bool small_out = (unsigned long long)p.N * p.OH * p.OW * p.OC < (1ull << 34);  // 32-bit offsets in 16-byte units
    // output pixel of tile row r of the tile at (w0, h0, n0), in the launch's tile geometry
    auto row_pixel = [&](int r, int w0, int h0, int n0, bool &okr, size_t &pix) {
      if (p.linear) {
        const long long px = (long long)(w0 / kTW) * BM + r;
        okr = px < p.total_pixels;
        pix = (size_t)px;
      } else if (p.flat) {
        const int pos = (w0 / kTW) * BM + r, oh = pos / p.PW, ow = pos - oh * p.PW;
        okr = ow < p.OW && oh < p.OH && n0 < p.N;
        pix = ((size_t)n0 * p.OH + oh) * p.OW + ow;
      } else {
        const int g = r >> 3, in = g / p.PHI, ih = g - in * p.PHI;
        const int ow = w0 + (r & 7), oh = h0 + ih, n = n0 + in;
        okr = in < p.NB && ih < p.TH && ow < p.OW && oh < p.OH && n < p.N;
        pix = ((size_t)n * p.OH + oh) * p.OW + ow;
      }
    };
    int gbase = 0, sp = 0;  // first group of the item; partial sum, counted across items
    bool ok = true;
    for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
      int ngroups, tile_supers;
      { const Item head = item_of(t); ngroups = head.ngroups; tile_supers = head.supers; }
      const int gbase0 = gbase;
      gbase += ngroups;
      float acc[NC];
#pragma unroll
      for (int j = 0; j < NC; ++j) acc[j] = 0.f;
      for (int si = 0; si < tile_supers; ++si, ++sp) {
        const int b = sp & 1;
        if (!(ok = TIMED(0, wait_group_warp(gbase0 + min((si + 1) * kSuper, ngroups) - 1)))) break;  // the partial's last group
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
      // (the item is worked out again here rather than kept in registers across the sums above:
      // with 64 running sums per thread this role is the one that sets the kernel's register count)
      int t_again = t;
      asm volatile("" : "+r"(t_again));
      const Item it = item_of(t_again);
      int w0, h0, n0, oc0;
      decode(it.tile, w0, h0, n0, oc0);
      PROF_START();
      if (it.tail) {
        // A slice of a last-wave tile: leave the partial sums in the scratch block of (tile,
        // slice); the CTA that finishes a tile last adds the slices up in slice order (so the
        // result does not depend on who that is) and carries on to the store.
        float4 *mine = reinterpret_cast<float4 *>(p.scratch + ((size_t)((it.tile - p.tail_tile0) * p.tail_d + it.slice) * BM + row) * BN + half * NC);
#pragma unroll
        for (int j = 0; j < NC; j += 4) mine[j >> 2] = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        __threadfence();
        PROF_LAP(2);
        asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight summing warps
        int *verdict = reinterpret_cast<int *>(store_base);  // (the staging block is free between items)
        if (warp == 8 && lane == 0) {
          const int seen = atomicAdd(p.tail_count + (it.tile - p.tail_tile0), 1);
          *verdict = seen == p.tail_d - 1 ? 1 : 0;
          if (seen == p.tail_d - 1) p.tail_count[it.tile - p.tail_tile0] = 0;  // ready for the next launch
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const bool reducer = *verdict != 0;
        asm volatile("bar.sync 1, 256;" ::: "memory");  // (the staging block is written again below)
        PROF_LAP(3);
        if (!reducer) continue;
        __threadfence();
        // The slices are added position by position (a warp walks one row of the tile: coalesced
        // reads of the eight scratch blocks, coalesced stores) rather than into the per-thread
        // running sums: with those 64 registers held, the loads of the slices would go out one
        // at a time (measured: 36 us for one tile).
        constexpr int V = BN / 4;  // 16-byte pieces per tile row
        const float4 *blocks = reinterpret_cast<const float4 *>(p.scratch + (size_t)(it.tile - p.tail_tile0) * p.tail_d * BM * BN);
        const bool vec_out = (p.OC & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
        for (int idx = (warp - 8) * 32 + lane; idx < BM * V; idx += 256) {
          float4 v[8];
#pragma unroll
          for (int sl = 0; sl < 8; ++sl)
            v[sl] = sl < p.tail_d ? __ldcg(blocks + (size_t)sl * BM * V + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
          float4 sum = v[0];
#pragma unroll
          for (int sl = 1; sl < 8; ++sl) { sum.x += v[sl].x; sum.y += v[sl].y; sum.z += v[sl].z; sum.w += v[sl].w; }
          const int r2 = idx / V, oc = oc0 + 4 * (idx - r2 * V);
          bool ok2;
          size_t pix2;
          row_pixel(r2, w0, h0, n0, ok2, pix2);
          if (!ok2 || oc >= p.OC || *abort_flag) continue;
          float res[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            res[e] *= (oc + e < p.OC) ? __ldg(p.out_scale + oc + e) : 0.f;
            if (p.relu) res[e] = fmaxf(res[e], 0.f);
          }
          float *dst = p.out + pix2 * p.OC + oc;
          if (vec_out) *reinterpret_cast<float4 *>(dst) = make_float4(res[0], res[1], res[2], res[3]);
          else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (oc + e < p.OC) dst[e] = res[e];
          }
        }
        PROF_LAP(4);
        continue;
      }
      const bool add_up = !it.tail && p.ksplit > 1;  // a slice of a uniformly split K range: add into the zeroed output
      bool row_ok;
      size_t pix;
      row_pixel(row, w0, h0, n0, row_ok, pix);
      row_ok = row_ok && !*abort_flag;
      const int ocb = oc0 + half * NC;
      float *o = p.out + pix * p.OC + ocb;
      const bool coalesced = vec && ocb + NC <= p.OC && small_out;
      if (!coalesced) {  // (the coalesced path scales after the rows are turned: two loads per thread instead of NC)
#pragma unroll
        for (int j = 0; j < NC; ++j) acc[j] *= (ocb + j < p.OC) ? __ldg(p.out_scale + ocb + j) : 0.f;
        if (p.relu) {
#pragma unroll
          for (int j = 0; j < NC; ++j) acc[j] = fmaxf(acc[j], 0.f);
        }
      }
      if (coalesced) {
        // Coalesced path: a thread holds 32..64 channels of ONE pixel; through a 4 KiB staging
        // block per warp the rows are turned so that eight lanes write one pixel's 128
        // contiguous bytes (4 passes through the memory pipe per store instead of 32).
        float4 *stage = reinterpret_cast<float4 *>(store_base + (warp - 8) * 4096);
        const uint32_t off16 = row_ok ? (uint32_t)((o - p.out) >> 2) : 0xFFFFFFFFu;
#pragma unroll
        for (int h = 0; h < NC / 32; ++h) {
#pragma unroll
          for (int qq = 0; qq < 8; ++qq)  // 16-byte piece qq of row `lane` sits at piece qq ^ (lane & 7)
            stage[lane * 8 + (qq ^ (lane & 7))] = make_float4(acc[h * 32 + 4 * qq], acc[h * 32 + 4 * qq + 1],
                                                               acc[h * 32 + 4 * qq + 2], acc[h * 32 + 4 * qq + 3]);
          __syncwarp();
          float4 v[8];
          const int qq = lane & 7;
          // this lane's four channels of every row: the per-channel scale (a power of two, exact)
          const float4 sc = __ldg(reinterpret_cast<const float4 *>(p.out_scale + ocb + h * 32 + 4 * qq));
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3);
            v[i] = stage[r * 8 + (qq ^ (r & 7))];
            v[i].x *= sc.x; v[i].y *= sc.y; v[i].z *= sc.z; v[i].w *= sc.w;
            if (p.relu) { v[i].x = fmaxf(v[i].x, 0.f); v[i].y = fmaxf(v[i].y, 0.f); v[i].z = fmaxf(v[i].z, 0.f); v[i].w = fmaxf(v[i].w, 0.f); }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t off = __shfl_sync(0xffffffffu, off16, 4 * i + (lane >> 3));
            float *dst = p.out + ((size_t)off << 2) + h * 32 + 4 * qq;
            if (off != 0xFFFFFFFFu) {
              if (add_up)
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
      if (add_up) {
#pragma unroll
        for (int j = 0; j < NC; ++j)
          if (ocb + j < p.OC) atomicAdd(o + j, acc[j]);
      } else if (vec && ocb + NC <= p.OC) {
#pragma unroll
        for (int j = 0; j < NC; j += 4) *reinterpret_cast<float4 *>(o + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < NC; ++j)
          if (ocb + j < p.OC) o[j] = acc[j];
      }
    }
  }
  if (warp == 8) PROF_OUT(5);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.error_flag, 1);
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// Per output channel: the power of two that brings the channel's largest |w| into [2^12, 2^13)
// (1 for an all-zero channel), and its inverse divided by the activation scale.
__global__ void tc16_scales_kernel(const float *__restrict__ w, int per_oc, float *__restrict__ w_scale, float *__restrict__ out_scale) {
  const float *row = w + (size_t)blockIdx.x * per_oc;
  unsigned m = 0;
  for (int i = threadIdx.x; i < per_oc; i += blockDim.x) {
    const unsigned b = __float_as_uint(row[i]) & 0x7FFFFFFFu;
    if (b < 0x7F800000u) m = max(m, b);
  }
  __shared__ unsigned red[32];
  for (int d = 16; d; d >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, d));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) m = max(m, red[i]);
    int sh = 0;
    if (m) {
      int e;
      frexpf(__uint_as_float(m), &e);  // |w|max = f * 2^e, f in [0.5, 1)
      sh = min(100, max(-100, 13 - e));
    }
    w_scale[blockIdx.x] = ldexpf(1.f, sh);
    out_scale[blockIdx.x] = ldexpf(1.f, -sh) / kXScale;
  }
}

// Dense OIHW -> the images the weight loader copies: for every (32-channel chunk, tap, channel
// tile) BN rows of 128 bytes, row = output channel = {w_hi[32], w_lo[32]} FP16 of w * scale[oc], in
// the 128-byte-swizzled order the tensor core reads (16-byte piece j of row r sits at piece
// j ^ (r & 7)).  Channels past IC or OC are zero.
__global__ void tc16_weight_tiles_kernel(const float *__restrict__ filt, __half *__restrict__ tiles,
                                         int OC, int IC, int KS, int n_chunks, int oc_tiles, int BN, const float *__restrict__ scale) {
  const long long total = (long long)KS * KS * n_chunks * oc_tiles * BN * 64;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(i % 64);                 // FP16 position inside the stored row
    const int row = (int)((i / 64) % BN);
    long long tile = i / ((long long)64 * BN);     // images are stored [channel tile][chunk][tap]: the K steps of
    const int tap = (int)(tile % (KS * KS));       // a work item lie back to back
    tile /= KS * KS;
    const int chunk = (int)(tile % n_chunks);
    const int oct = (int)(tile / n_chunks);
    const int piece = (col >> 3) ^ (row & 7);      // logical 16-byte piece stored at this position
    const int k = ((piece & 3) << 3) | (col & 7);  // channel inside the chunk
    const bool is_lo = piece >= 4;
    const int oc = oct * BN + row, ic = chunk * KC + k;
    float w = 0.f;
    if (ic < IC && oc < OC) w = filt[((size_t)oc * IC + ic) * KS * KS + tap] * scale[oc];
    const __half h = __float2half_rn(w);
    tiles[i] = is_lo ? __float2half_rn(w - __half2float(h)) : h;
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

struct Tc16State {
  __half *d_tiles = nullptr;
  int *d_error = nullptr;
  unsigned *d_gate = nullptr;
  int n_chunks = 0, bn = 128;
  float *d_out_scale = nullptr;  // per output channel
  float *d_scratch = nullptr;    // tail split: one 128 x BN block of partial sums per CTA (allocated when a shape first needs it)
  int *d_tail_count = nullptr;   // tail split: finished slices per last-wave tile (all zero between launches)
  int sms = 0;
  struct Setup {
    bool valid = false;
    const float *in = nullptr;
    ConvShape shape{};
    CUtensorMap map_x;
    Tc16Params params{};
    dim3 grid;
    size_t smem = 0;
  };
  static constexpr int kSetups = 8;
  std::mutex mutex;
  Setup setups[kSetups];
  int next_setup = 0;
};

constexpr size_t kSmemBudget = 227 * 1024;

}  // namespace

void conv_tc16_state_delete(void *state) {
  Tc16State *s = static_cast<Tc16State *>(state);
  if (!s) return;
  cudaFree(s->d_tiles); cudaFree(s->d_error); cudaFree(s->d_gate); cudaFree(s->d_out_scale);
  cudaFree(s->d_scratch); cudaFree(s->d_tail_count);
  delete s;
}

// Builds the split FP16 weight images (called from filter creation and from the file loader;
// d_dense is the OIHW filter on the device).  Failure here is not fatal for the filter: the
// variant is then reported as unsupported.
int conv_tc16_prepare(tetris_filter *f, const float *d_dense) {
  if (f->groups != 1 || (f->in_channel & 3) != 0 || f->in_channel < 8 || f->kernel_size > 7) return TETRIS_OK;
  Tc16State *s = new (std::nothrow) Tc16State();
  if (!s) return TETRIS_OK;
  const int KS = f->kernel_size, taps = KS * KS;
  s->n_chunks = (f->in_channel + KC - 1) / KC;
  s->bn = f->out_channel <= 64 ? 64 : 128;
  const int oc_tiles = (f->out_channel + s->bn - 1) / s->bn;
  const size_t elems = (size_t)taps * s->n_chunks * oc_tiles * s->bn * 64;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&s->sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) s->sms = 0;
  if (s->sms < 1 || cudaMalloc(&s->d_tiles, elems * sizeof(__half)) != cudaSuccess || cudaMalloc(&s->d_error, sizeof(int)) != cudaSuccess ||
      cudaMalloc(&s->d_gate, 2 * sizeof(unsigned)) != cudaSuccess ||
      cudaMalloc(&s->d_tail_count, (size_t)s->sms * sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    conv_tc16_state_delete(s);
    return TETRIS_OK;
  }
  cudaMemset(s->d_error, 0, sizeof(int));
  cudaMemset(s->d_gate, 0, 2 * sizeof(unsigned));
  cudaMemset(s->d_tail_count, 0, (size_t)s->sms * sizeof(int));
  // per-channel scales: every output channel's largest |w| lands in [2^12, 2^13)
  float *d_w_scale = nullptr;
  if (cudaMalloc(&d_w_scale, f->out_channel * sizeof(float)) != cudaSuccess ||
      cudaMalloc(&s->d_out_scale, f->out_channel * sizeof(float)) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(d_w_scale);
    conv_tc16_state_delete(s);
    return TETRIS_OK;
  }
  tc16_scales_kernel<<<f->out_channel, 256>>>(d_dense, f->in_channel * taps, d_w_scale, s->d_out_scale);
  tc16_weight_tiles_kernel<<<(unsigned)std::min<size_t>((elems + 255) / 256, 4096), 256>>>(
      d_dense, s->d_tiles, f->out_channel, f->in_channel, KS, s->n_chunks, oc_tiles, s->bn, d_w_scale);
  const cudaError_t err = cudaGetLastError();
  cudaStreamSynchronize(0);  // (d_w_scale is freed next)
  cudaFree(d_w_scale);
  if (err != cudaSuccess) {
    conv_tc16_state_delete(s);
    return TETRIS_OK;
  }
  f->tc16_state = s;
  return TETRIS_OK;
}

// K steps per pipeline group of the kernel instance that serves channel tiles of `bn` and filters
// of `ks` x `ks`: four for 64-channel tiles, whose MMAs are short (measured on VGG-19 conv1_2 and
// the 64-channel 3x3 layers of ResNet-50: 3-4 % faster than pairs); 1x1 filters, where a group of
// four would wait for four patches at a time, and 128-channel tiles stay with pairs.
static int group_steps(int bn, int ks) { return bn == 64 && ks > 1 ? 4 : 2; }

bool conv_tc16_supported(const tetris_filter *f, const ConvShape &s) {
  if (!f->tc16_state || !f->tc_state || f->groups != 1) return false;  // (the split-TF32 variant is the out-of-range fallback)
  if (s.S != 1 || s.N < 1 || s.OH < 1 || s.OW < 1 || (s.IC & 3) != 0) return false;
  return conv_tc_supported(f, s);
}

int launch_conv_tc16(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st) {
  Tc16State *t = static_cast<Tc16State *>(f->tc16_state);
  if (!conv_tc16_supported(f, s) || (reinterpret_cast<uintptr_t>(in) & 15) != 0) {
    set_error("split-FP16 tensor-core variant covers stride 1, in_channel a multiple of 4 (at least 8), 16-byte aligned inputs");
    return TETRIS_ERR_UNSUPPORTED;
  }
  EncodeFn enc = get_encode();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return TETRIS_ERR_UNSUPPORTED; }
  CUtensorMap map_x;
  Tc16Params p;
  dim3 grid;
  size_t smem = 0;
  int bn = 128;
  {
    std::lock_guard<std::mutex> lock(t->mutex);
    Tc16State::Setup *su = nullptr;
    for (Tc16State::Setup &c : t->setups) {
      const ConvShape &l = c.shape;
      if (c.valid && c.in == in && l.relu == s.relu && l.N == s.N && l.H == s.H && l.W == s.W && l.P == s.P && l.S == s.S) { su = &c; break; }
    }
    if (!su) {
      su = &t->setups[t->next_setup];
      t->next_setup = (t->next_setup + 1) % Tc16State::kSetups;
      su->valid = false;
      Tc16Params &q = su->params;
      q = Tc16Params{};
      const int KS = s.KS, halo = KS - 1;
      q.N = s.N; q.OH = s.OH; q.OW = s.OW; q.OC = s.OC; q.P = s.P; q.KS = KS;
      q.linear = (KS == 1 && s.P == 0) ? 1 : 0;
      q.total_pixels = (long long)s.N * s.OH * s.OW;
      cuuint64_t dims[4], strides[3];
      cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
      if (q.linear) {
        q.PW = kTW; q.PHI = kTH; q.TH = kTH; q.NB = 1;
        q.box_rows = BM;
        q.tiles_w = (int)((q.total_pixels + BM - 1) / BM); q.tiles_h = 1; q.tiles_n = 1;
        dims[0] = (cuuint64_t)s.IC; dims[1] = (cuuint64_t)q.total_pixels; dims[2] = 1; dims[3] = 1;
        strides[0] = (cuuint64_t)s.IC * 4; strides[1] = strides[0] * dims[1]; strides[2] = strides[1];
        box[0] = KC; box[1] = BM; box[2] = 1; box[3] = 1;
      } else {
        q.PW = kTW + halo;
        const bool whole = s.OH <= kTH;                 // the image's rows fit one tile
        q.TH = whole ? s.OH : kTH;
        q.PHI = q.TH + halo;
        q.NB = whole ? std::max(1, std::min(s.N, (kTH + halo) / q.PHI)) : 1;
        while (q.NB > 1 && (q.NB - 1) * q.PHI + q.TH > kTH) --q.NB;  // every valid group index stays below 16
        q.box_rows = q.PW * q.PHI * q.NB;
        q.tiles_w = (s.OW + kTW - 1) / kTW;
        q.tiles_h = (s.OH + q.TH - 1) / q.TH;
        q.tiles_n = (s.N + q.NB - 1) / q.NB;
        // The other geometry: the image laid out with its padded width Wp = W + 2P, a tile = 128
        // consecutive positions of that layout (8-pixel groups simply follow one another, so a
        // window is again one descriptor).  Nothing is lost to tile shapes -- only the Wp - OW
        // positions per row that are no outputs -- at the price of a patch of whole padded rows.
        // Taken when it needs fewer tiles and the patches still fit beside three weight stages.
        const int Wp = s.W + 2 * s.P;
        const int span = (Wp - 1 + BM - 1) / Wp + 1;            // output rows a tile can touch
        const int nrows = span + halo;
        const long long tiles_flat = (long long)(((long long)s.OH * Wp + BM - 1) / BM) * s.N;
        const long long tiles_2d = (long long)q.tiles_w * q.tiles_h * q.tiles_n;
        const size_t flat_stage = ((size_t)(Wp * nrows + 8) * 128 + 1023) / 1024 * 1024;
        const size_t room = kSmemBudget - (1024 + kStoreBytes + kNumBars * 8 + 16) - 3 * (size_t)t->bn * 256;
        // (with room for two patches only -- a pair of K steps may need both -- it has to save 10 % of the tiles)
        if (Wp <= 256 && nrows <= 256 &&
            ((3 * flat_stage <= room && tiles_flat * 100 < tiles_2d * 97) || (2 * flat_stage <= room && tiles_flat * 100 < tiles_2d * 90))) {
          q.flat = 1;
          q.PW = Wp; q.PHI = nrows; q.TH = s.OH; q.NB = 1;
          q.box_rows = Wp * nrows;
          q.tiles_w = (int)(((long long)s.OH * Wp + BM - 1) / BM); q.tiles_h = 1; q.tiles_n = s.N;
        }
        dims[0] = (cuuint64_t)s.IC; dims[1] = (cuuint64_t)s.W; dims[2] = (cuuint64_t)s.H; dims[3] = (cuuint64_t)s.N;
        strides[0] = (cuuint64_t)s.IC * 4; strides[1] = strides[0] * s.W; strides[2] = strides[1] * s.H;
        box[0] = KC; box[1] = (cuuint32_t)q.PW; box[2] = (cuuint32_t)q.PHI; box[3] = (cuuint32_t)q.NB;
      }
      const CUresult r = enc(&su->map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(in), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return TETRIS_ERR_CUDA; }
      // a stage holds the patch and whatever the windows of the 16 groups reach beyond it
      const int reach_rows = q.linear ? BM : q.flat ? q.box_rows + 8 : (kTH + halo) * q.PW + halo + 8;
      q.x_stage_bytes = (std::max(reach_rows, q.box_rows) * 128 + 1023) / 1024 * 1024;
      q.n_chunks = t->n_chunks;
      q.w_tiles = t->d_tiles;
      q.error_flag = t->d_error;
      q.gate = t->d_gate;
      q.out_scale = t->d_out_scale;
      int dev = 0, sms = 0;
      TETRIS_CUDA_TRY(cudaGetDevice(&dev));
      TETRIS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      const long long tiles = (long long)q.tiles_w * q.tiles_h * q.tiles_n * ((s.OC + t->bn - 1) / t->bn);
      // K range split into d work items per tile when that fills the waves of CTAs better (as in the
      // split-TF32 variant; cost in K steps: waves x (K steps + ~12 per item) + zeroing the output)
      const double iters = (double)KS * KS * q.n_chunks;
      const double zeroing = ((double)s.N * s.OH * s.OW * s.OC * 4 / 6.0e12 + 3e-6) * 1.9e9 / 500.0;
      int best_d = 1;
      double best_cost = std::ceil((double)tiles / sms) * (iters + 12.0);
      q.relu = s.relu;
      for (int d = 2; d <= 8 && d <= q.n_chunks && !f->deterministic && !s.relu; ++d) {  // (a rectified sum cannot be added up from slices)
        if (q.n_chunks % d) continue;
        const double cost = std::ceil((double)tiles * d / sms) * (iters / d + 12.0) + zeroing;
        if (cost < 0.96 * best_cost) { best_cost = cost; best_d = d; }
      }
      q.ksplit = best_d;
      // Tail split: with T tiles on S CTAs the last wave holds T mod S tiles; when that is a small
      // remainder, each of those tiles is cut into d K slices (d a divisor of the chunk count, at
      // most one slice per CTA) that run side by side and are added up through the scratch blocks
      // -- in slice order, so the result stays bit-reproducible, and with no zeroing of the output.
      q.tail_tile0 = (int)tiles; q.tail_start = (int)tiles * best_d; q.tail_d = 1;
      q.scratch = t->d_scratch; q.tail_count = t->d_tail_count;
      if (best_d == 1 && tiles > sms && sms <= t->sms) {
        const int full = (int)(tiles / sms) * sms, rest = (int)tiles - full;
        int d = 0;
        // (writing the slices out and adding them up costs a tile about as much as 30 K steps:
        // the split has to save more than that)
        for (int c = 2; c <= 8 && c <= q.n_chunks; ++c)
          if (q.n_chunks % c == 0 && rest * c <= sms && iters * (c - 1) >= 32.0 * c) d = c;
        if (rest > 0 && d >= 2 && !t->d_scratch &&  // (10 MB per filter: only for filters that have such a shape)
            cudaMalloc(&t->d_scratch, (size_t)t->sms * BM * t->bn * sizeof(float)) != cudaSuccess) {
          cudaGetLastError();
          t->d_scratch = nullptr;
          d = 0;
        }
        if (rest > 0 && d >= 2) { q.tail_tile0 = full; q.tail_start = full; q.tail_d = d; q.scratch = t->d_scratch; }
      }
      // shared memory: activation ring, weight ring, store staging, barriers
      const size_t wbytes = (size_t)t->bn * 128 * group_steps(t->bn, KS);  // a weight stage holds a group of K steps
      const size_t fixed = 1024 + kStoreBytes + kNumBars * 8 + 16;
      const int chunks_per_item = q.n_chunks / best_d;
      q.n_w = kWStagesMax;
      q.n_x = (int)std::min<size_t>(kXStagesMax, (kSmemBudget - fixed - q.n_w * wbytes) / q.x_stage_bytes);
      while (q.n_x < 3 && q.n_w > 3) {  // (a group of K steps may straddle two patches: at least two stages, better three)
        --q.n_w;
        q.n_x = (int)std::min<size_t>(kXStagesMax, (kSmemBudget - fixed - q.n_w * wbytes) / q.x_stage_bytes);
      }
      if (q.n_x < 2) { set_error("split-FP16 variant: the activation patches of this layer do not fit shared memory"); return TETRIS_ERR_UNSUPPORTED; }
      if (KS > 1) q.n_x = std::min(q.n_x, 3);          // a patch feeds KS*KS steps: three stages are ample
      q.n_x = std::max(2, std::min(q.n_x, std::max(3, 2 * chunks_per_item)));  // (patches are fetched across work items)
      su->smem = fixed + (size_t)q.n_x * q.x_stage_bytes + (size_t)q.n_w * wbytes;
      su->grid = dim3((unsigned)std::min<long long>(q.tail_start + (tiles - q.tail_tile0) * q.tail_d, sms));  // persistent: one CTA per SM
      su->in = in;
      su->shape = s;
      su->valid = true;
    }
    map_x = su->map_x;
    p = su->params;
    grid = su->grid;
    smem = su->smem;
    bn = t->bn;
  }
  p.out = out;
  p.withhold_first_load = test_injection(&p.spin_limit);
#ifdef TETRIS_TC16_PROF
  static long long *d_prof = nullptr;
  const bool prof = getenv("TETRIS_TC16_PROF") != nullptr;
  if (prof) {
    if (!d_prof) cudaMalloc(&d_prof, 64 * sizeof(long long));
    cudaMemset(d_prof, 0, 64 * sizeof(long long));
    p.prof = d_prof;
  }
#endif
  static thread_local bool configured[16] = {false};
  int dev = 0;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(conv_tc16_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(conv_tc16_kernel<64, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(conv_tc16_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    if (dev < 16) configured[dev] = true;
  }
  if (p.ksplit > 1)  // the work items add into the output
    TETRIS_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)s.N * s.OH * s.OW * s.OC * sizeof(float), st));
  if (bn == 64 && group_steps(64, s.KS) == 4)
    conv_tc16_kernel<64, 4><<<grid, kThreads, smem, st>>>(map_x, p);
  else if (bn == 64)
    conv_tc16_kernel<64, 2><<<grid, kThreads, smem, st>>>(map_x, p);
  else
    conv_tc16_kernel<128, 2><<<grid, kThreads, smem, st>>>(map_x, p);
  TETRIS_CUDA_TRY(cudaGetLastError());
  count_launch();
  if (p.relu) note_relu_fused();
#ifdef TETRIS_TC16_PROF
  if (prof) {
    long long h[64];
    cudaDeviceSynchronize();
    cudaMemcpy(h, d_prof, sizeof(h), cudaMemcpyDeviceToHost);
    const char *names[6] = {"x loader (xempty)", "w loader (gdone)", "cp (gdone-4, xconv)", "mma (afull, pempty, wfull; mmas, commit)", "convert (xfull)", "sum (gdone)"};
    const long long tiles_ = (long long)p.tiles_w * p.tiles_h * p.tiles_n * ((s.OC + bn - 1) / bn);
    const long long items = (p.tail_start + (tiles_ - p.tail_tile0) * p.tail_d + grid.x - 1) / grid.x;
    const long long steps = (long long)(p.tail_start / grid.x) * s.KS * s.KS * (p.n_chunks / p.ksplit) + (long long)s.KS * s.KS * (p.n_chunks / p.tail_d);
    fprintf(stderr, "[tc16 prof] grid %u, items/CTA %lld, K steps/CTA %lld, n_x %d n_w %d\n", grid.x, items, steps, p.n_x, p.n_w);
    for (int r = 0; r < 6; ++r)
      fprintf(stderr, "[tc16 prof] %-42s total %9lld clk (%5.0f per K step); waits: %lld %lld %lld %lld %lld\n", names[r], h[r * 8],
              (double)h[r * 8] / (double)steps, h[r * 8 + 1], h[r * 8 + 2], h[r * 8 + 3], h[r * 8 + 4], h[r * 8 + 5]);
  }
#endif
  // The guard: the split-TF32 variant, queued behind; it returns at once unless the largest
  // activation of this launch lies outside FP16's useful window, in which case it recomputes the layer.
  return launch_conv_tc_gated(f, in, out, s, st, t->d_gate);
}

// 0 = no timeout seen so far, 1 = a bounded wait gave up in some launch (the flag is cleared).
int conv_tc16_check_error(const tetris_filter *f) {
  Tc16State *t = static_cast<Tc16State *>(f->tc16_state);
  if (!t) return 0;
  int flag = 0;
  if (cudaMemcpy(&flag, t->d_error, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
  if (flag) {
    // (a launch that gave up may have left the guard's words and the last-wave counters half way)
    cudaMemset(t->d_error, 0, sizeof(int));
    cudaMemset(t->d_gate, 0, 2 * sizeof(unsigned));
    cudaMemset(t->d_tail_count, 0, (size_t)t->sms * sizeof(int));
  }
  return flag;
}

}  // namespace tetris
