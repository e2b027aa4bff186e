// Tiled sparse-filter convolution for sm_100a: the hot kernel.
//
// Role of the reference's SparseConv2dKernel + LoadImg2SharedMem
// (Tetris/spconv2d_kernel.cu:13-160), re-designed:
//
//  * lanes are output PIXELS, not output channels, and the weights are warp-uniform.  A lane owns
//    P2 output columns of one tile row in two "planes" (two images of the batch, or the upper
//    and lower half of a tile when the batch is odd) for the K output channels of its warp's
//    block: K*P2 float2 accumulators.  The two planes share every weight, so each multiply-add
//    is one packed FP32 FMA (fma.rn.f32x2): half the issue slots of scalar FMAs.
//  * the weights of a block arrive as K lists of {weight, position} records (LIST form,
//    format.h), staged into shared memory next to the input tile.  The k loop is unrolled, so
//    accumulator row k is a compile-time register name; the record only carries a shared-memory
//    offset.  There is no per-record decode in the inner loop (the reference decodes y/x/ic with
//    shifts and masks per nonzero, Tetris/spconv2d_kernel.cu:103-105): positions are turned into
//    byte offsets once per staged list, 32 records at a time, one per lane.
//  * the input tile (with halo) is staged per input-channel stage by cp.async into a
//    double-buffered tile of float2 {plane0, plane1} laid out [channel][column parity][row]
//    [column]; lane `seg` of a row owns columns seg, seg+NSEG, seg+2*NSEG, ..., so for any
//    filter column shift the 32 lanes read 32 consecutive float2 -- a conflict-free 8-byte load
//    with no alignment constraint, which is what lets one code path serve every kernel size and
//    stride.  (TMA tiled loads do not fit this tile: the NHWC source is channel-innermost while
//    the tile is channel-outermost with two planes interleaved -- an element-wise gather.)
//  * records and input windows are prefetched one record ahead across list boundaries, so the
//    loop body is load-next / FMA-current with no dependent address arithmetic.
//
// The kernel moves one shared-memory word per multiply-add (the same ratio as the reference,
// see the profile summaries for what that bounds).  A variant that reused a register-resident
// window across the K channels through a jump-table interpreter (one indirect branch per weight)
// measured 5-7 TFLOP/s against 9-12 here and was removed.
//
// NHWC in, NHWC out, FP32, output fully overwritten -- the contract of the reference launcher
// (Tetris/spconv2d_kernel.cu:163-188).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <new>
#include <vector>

#include "internal.h"

namespace tetris {
namespace {

struct TiledParams {
  const float *in;
  float *out;
  const uint2 *lists;
  const int32_t *list_offsets;
  int N, H, W, IC, OC, OH, OW, P, KS, S;
  int NSEG, TH;          // lanes per tile row, tile rows; NSEG*TH lanes are in use
  int tiles_w, tiles_h;  // tiles along OW and along OH
  int pair_mode;         // 0: planes are images 2j and 2j+1; 1: upper/lower TH rows of one image
  int ROWS, COLS;        // staged input rows / columns per plane
  int RP;                // bytes per staged row
  int PLP;               // bytes per column-parity plane (ROWS * RP)
  int ICP;               // bytes per channel slab
  int stage_bytes;       // (TIC + 1) * ICP: the staged channels and one all-zero slab
  int n_entries;         // staging table entries: ROWS * COLS
  int list_bytes;        // shared bytes per warp and buffer for its staged list piece
  int T, B, TIC, tic_shift;
};

__device__ __forceinline__ void cp_async4(uint32_t dst, const float *src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds_u4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u1(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts_u1(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

template <int K, int P2, int WARPS, int MINB>
__global__ void __launch_bounds__(WARPS * 32, MINB) conv_tiled_kernel(const TiledParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(smem_raw);
  // layout: [input tile 0][input tile 1][lists 0: WARPS x list_bytes][lists 1]
  //         [staging table: n_entries x {goff plane 0, goff plane 1, soff, -}]
  const uint32_t lists0 = smem0 + 2 * p.stage_bytes;
  int4 *tab = reinterpret_cast<int4 *>(smem_raw + 2 * p.stage_bytes + 2 * WARPS * p.list_bytes);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- which tile ----
  int bx = blockIdx.x;
  const int tw = bx % p.tiles_w;
  bx /= p.tiles_w;
  const int th = bx % p.tiles_h;
  const int pr = bx / p.tiles_h;
  int n0, n1, h0, h1;
  bool v1;
  if (p.pair_mode == 0) {
    n0 = 2 * pr; n1 = n0 + 1; h0 = h1 = th * p.TH; v1 = n1 < p.N;
  } else {
    n0 = n1 = pr; h0 = th * 2 * p.TH; h1 = h0 + p.TH; v1 = h1 < p.OH;
  }
  const int w0 = tw * p.NSEG * P2;

  // ---- staging table: where every (input row, input column) of the tile comes from in global
  //      memory, per plane, and where it goes inside a channel slab ----
  for (int e = tid; e < p.n_entries; e += WARPS * 32) {
    const int ci = e % p.COLS, ri = e / p.COLS;
    const int iw = w0 * p.S + ci - p.P;
    const int ih0 = h0 * p.S + ri - p.P, ih1 = h1 * p.S + ri - p.P;
    const bool okw = iw >= 0 && iw < p.W;
    const bool ok0 = okw && ih0 >= 0 && ih0 < p.H;
    const bool ok1 = okw && v1 && ih1 >= 0 && ih1 < p.H;
    tab[e] = make_int4(ok0 ? (int)((((long long)n0 * p.H + ih0) * p.W + iw) * p.IC) : -1,
                       ok1 ? (int)((((long long)n1 * p.H + ih1) * p.W + iw) * p.IC) : -1,
                       (ci % p.S) * p.PLP + ri * p.RP + (ci / p.S) * 8, 0);
  }
  __syncthreads();

  const int b = blockIdx.y * WARPS + warp;  // output-channel block of this warp
  const bool warp_on = b < p.B;

  // staging role of this thread: plane (tid & 1), channel inside the stage, entry slot
  const int pl_s = tid & 1;
  const int icl_s = (tid >> 1) & (p.TIC - 1);
  const int pe0 = tid >> (1 + p.tic_shift), pe_step = (WARPS * 32) >> (1 + p.tic_shift);
  auto issue_stage = [&](int t, int buf) {
    if (warp_on) {  // this warp's list piece of the stage, 16 bytes per copy
      const int po = p.list_offsets[b * p.T + t], pn = p.list_offsets[b * p.T + t + 1];
      const uint32_t dst_p = lists0 + (buf * WARPS + warp) * p.list_bytes;
      for (int i = lane; 2 * i < pn - po; i += 32) cp_async16(dst_p + i * 16, p.lists + po + 2 * i);
    }
    const int ic = t * p.TIC + icl_s;
    if (ic < p.IC) {
      const float *src_c = p.in + ic;
      const uint32_t dst_c = smem0 + buf * p.stage_bytes + icl_s * p.ICP + pl_s * 4;
      for (int e = pe0; e < p.n_entries; e += pe_step) {
        const int4 ent = tab[e];
        const int g = pl_s ? ent.y : ent.x;
        cp_async4(dst_c + ent.z, src_c + (g >= 0 ? g : 0), g >= 0 ? 4 : 0);
      }
    }
    cp_async_commit();
  };

  // ---- this lane's pixels (compute role): columns seg + q*NSEG of tile row `row` ----
  // Idle lanes mirror the last active lane: same address, so their loads are broadcasts that
  // add no shared-memory wavefront.
  const bool lane_on = lane < p.NSEG * p.TH;
  const int lane_c = min(lane, p.NSEG * p.TH - 1);
  const int row = lane_c / p.NSEG;
  const int seg = lane_c % p.NSEG;
  uint32_t xoff[P2];
#pragma unroll
  for (int q = 0; q < P2; ++q) xoff[q] = (row * p.S) * p.RP + (q * p.NSEG + seg) * 8;

  float2 acc[K][P2];
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int q = 0; q < P2; ++q) acc[k][q] = make_float2(0.f, 0.f);

  // Channel slab TIC of each buffer stays zero: padding records point there, so a padded
  // multiply-add adds exactly 0 whatever the input holds.
  for (int i = tid * 4; i < p.ICP; i += WARPS * 32 * 4) {
    sts_u1(smem0 + p.TIC * p.ICP + i, 0u);
    sts_u1(smem0 + p.stage_bytes + p.TIC * p.ICP + i, 0u);
  }

  issue_stage(0, 0);
#pragma unroll 1
  for (int t = 0; t < p.T; ++t) {
    if (t + 1 < p.T) {
      issue_stage(t + 1, (t + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (warp_on) {
      const uint32_t sbase = smem0 + (t & 1) * p.stage_bytes;
      const uint32_t piece = lists0 + ((t & 1) * WARPS + warp) * p.list_bytes;
      const uint32_t recs = piece + (K + kListHeaderWords) * 4;
      // positions -> byte offsets inside the staged tile, one record per lane at a time
      // (the sentinel pair behind the last list is translated too)
      const int total = (int)lds_u1(piece + K * 4) + 2;
      for (int i = lane; i < total; i += 32) {
        const uint32_t pos = lds_u1(recs + i * 8 + 4);
        const uint32_t icl = pos >> 8, r = (pos >> 4) & 15u, s = pos & 15u;
        sts_u1(recs + i * 8 + 4, icl * p.ICP + r * p.RP + (s % p.S) * p.PLP + (s / p.S) * 8);
      }
      __syncwarp();
      // list lengths (even by construction), two 16-bit counts per register
      uint32_t cnt[K / 2];
#pragma unroll
      for (int k = 0; k < K; k += 2)
        cnt[k / 2] = lds_u1(piece + k * 4) | (lds_u1(piece + k * 4 + 4) << 16);
      uint32_t xb[P2];
#pragma unroll
      for (int q = 0; q < P2; ++q) xb[q] = sbase + xoff[q];

      // Two records per iteration, their windows in two register sets that swap roles, so the
      // prefetch needs no register copies: load pair i+1 while the FMAs of pair i issue.
      uint32_t rp = recs;
      uint4 rr = lds_u4(rp);  // records i (x, y) and i+1 (z, w)
      float2 xa[P2], xc[P2];
#pragma unroll
      for (int q = 0; q < P2; ++q) xa[q] = lds_f2(xb[q] + rr.y);
#pragma unroll
      for (int q = 0; q < P2; ++q) xc[q] = lds_f2(xb[q] + rr.w);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int n = (k & 1) ? (int)(cnt[k / 2] >> 16) : (int)(cnt[k / 2] & 0xffffu);
#pragma unroll 1
        for (int j = 0; j < n; j += 2) {
          const float wa = __uint_as_float(rr.x), wc = __uint_as_float(rr.z);
          rp += 16;
          rr = lds_u4(rp);  // the next pair: of this list, of the next one, or the sentinels
          const float2 wa2 = make_float2(wa, wa), wc2 = make_float2(wc, wc);
#pragma unroll
          for (int q = 0; q < P2; ++q) {
            acc[k][q] = __ffma2_rn(wa2, xa[q], acc[k][q]);
            xa[q] = lds_f2(xb[q] + rr.y);
          }
#pragma unroll
          for (int q = 0; q < P2; ++q) {
            acc[k][q] = __ffma2_rn(wc2, xc[q], acc[k][q]);
            xc[q] = lds_f2(xb[q] + rr.w);
          }
        }
      }
    }
    __syncthreads();
  }

  // ---- epilogue: NHWC stores, K consecutive channels per pixel ----
  if (!warp_on || !lane_on) return;
  const int oc0 = b * K;
  const int kn = min(K, p.OC - oc0);
  // 16-byte stores need a 16-byte aligned output as well as whole groups of four channels
  const bool vec = (p.OC & 3) == 0 && kn == K && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
#pragma unroll
  for (int pl = 0; pl < 2; ++pl) {
    const int n = pl ? n1 : n0;
    const int oh = (pl ? h1 : h0) + row;
    if ((pl == 1 && !v1) || oh >= p.OH) continue;
#pragma unroll
    for (int q = 0; q < P2; ++q) {
      const int ow = w0 + q * p.NSEG + seg;
      if (ow >= p.OW) continue;
      float *o = p.out + (((size_t)n * p.OH + oh) * p.OW + ow) * p.OC + oc0;
      if (vec) {
#pragma unroll
        for (int k4 = 0; k4 < K / 4; ++k4) {
          float4 v;
          v.x = pl ? acc[4 * k4 + 0][q].y : acc[4 * k4 + 0][q].x;
          v.y = pl ? acc[4 * k4 + 1][q].y : acc[4 * k4 + 1][q].x;
          v.z = pl ? acc[4 * k4 + 2][q].y : acc[4 * k4 + 2][q].x;
          v.w = pl ? acc[4 * k4 + 3][q].y : acc[4 * k4 + 3][q].x;
          *reinterpret_cast<float4 *>(o + 4 * k4) = v;
        }
      } else {
#pragma unroll
        for (int k = 0; k < K; ++k)
          if (k < kn) o[k] = pl ? acc[k][q].y : acc[k][q].x;
      }
    }
  }
}

// ---- host side: tile geometry -----------------------------------------------------------------
struct Plan {
  bool valid = false;
  ConvShape shape{};
  int instance = 0;  // which kernel template instance
  int use_tc = 0;  // automatic choice: 0 list kernel, 1 split-TF32 tensor-core variant, 2 split-FP16 tensor-core variant
  TiledParams p{};
  dim3 grid;
  size_t smem_bytes = 0;
};

// Row pitch in 8-byte slots: at least `need`, chosen so that the 16 lanes of a half-warp (one
// 128-byte shared-memory wavefront of 8-byte loads) fall into as many distinct slots mod 16 as
// possible.  Idle lanes mirror the last active one and add no slot.
int pick_row_slots(int need, int NSEG, int TH, int S) {
  int best = need, best_conf = 1 << 30;
  for (int rw = need; rw < need + 16; ++rw) {
    int conf = 0;
    for (int half = 0; half < 2; ++half) {
      int seen[16] = {0};
      for (int l = half * 16; l < half * 16 + 16; ++l) {
        if (l >= NSEG * TH) continue;
        const int row = l / NSEG, seg = l % NSEG;
        const int slot = (row * S * rw + seg) & 15;
        conf += seen[slot]++;
      }
    }
    if (conf < best_conf) { best_conf = conf; best = rw; }
  }
  return best;
}

constexpr size_t kSmemLimit = (size_t)225 * 1024;

struct Instance {
  int K, P2, WARPS, MINB;
};
constexpr Instance kInstances[] = {{8, 4, 8, 2}, {8, 2, 8, 3}, {16, 4, 4, 3}, {16, 2, 4, 4}};

// Estimated launch time (in SM clocks) of one instance with one tile shape, or a negative value
// if it does not fit.  The kernel is bound by the shared-memory data pipe (one wavefront per
// clock and SM), so the model counts wavefronts: P2 window loads of 2 wavefronts plus half
// a record load per weight record and warp, the staging stores, a fixed cost per CTA and per
// stage, and the rounding of the grid to whole waves of resident CTAs.
double plan_cost(const tetris_filter *f, const ConvShape &s, const Instance &inst, int NSEG, int TH,
                 int sm_count, size_t smem_limit, Plan *out) {
  const int P2 = inst.P2, TIC = f->tile_ic;
  const int pair_mode = (s.N % 2 == 0) ? 0 : 1;
  const int n_pairs = pair_mode ? s.N : s.N / 2;
  const int rows_per_tile = pair_mode ? 2 * TH : TH;
  const int tiles_w = (s.OW + NSEG * P2 - 1) / (NSEG * P2);
  const int tiles_h = (s.OH + rows_per_tile - 1) / rows_per_tile;
  const int ROWS = (TH - 1) * s.S + s.KS;
  const int COLS = (NSEG * P2 - 1) * s.S + s.KS;
  const int RW = pick_row_slots((COLS + s.S - 1) / s.S, NSEG, TH, s.S);
  const int RP = RW * 8, PLP = ROWS * RP;
  int ICP = s.S * PLP;
  if (((ICP / 8) & 1) == 0) ICP += 8;  // odd slot pitch: conflict-free staging stores
  const int n_entries = ROWS * COLS;
  const int list_bytes = (f->max_list_units * 8 + 15) / 16 * 16;
  const size_t smem = 2 * (size_t)(TIC + 1) * ICP + (size_t)n_entries * sizeof(int4) +
                      (size_t)2 * inst.WARPS * list_bytes;
  if (smem > smem_limit) return -1.0;
  const int ctas_y = (f->n_oc_blocks + inst.WARPS - 1) / inst.WARPS;
  const double ctas = (double)tiles_w * tiles_h * n_pairs * ctas_y;
  const int resident = (int)std::max<size_t>(1, std::min<size_t>((size_t)inst.MINB, smem_limit / smem));
  const double waves = ctas / ((double)sm_count * resident);
  const double rounding = std::ceil(waves) / waves;
  const double recs_per_block = 1.04 * (double)f->nnz / f->n_oc_blocks + 2.0 * f->n_stages;
  const double wl = 2.0;  // an 8-byte load takes two passes whatever the number of active lanes (measured)
  const double warp_blocks = (double)tiles_w * tiles_h * n_pairs * f->n_oc_blocks;
  const double wf_compute = warp_blocks * recs_per_block * (P2 * wl + 0.5);
  const double wf_staging = ctas * (double)f->n_stages * std::min(TIC, s.IC) * n_entries * 2 * 0.04;
  const double fixed = ctas * (2500.0 + 300.0 * f->n_stages) / resident;
  // a warp issues at most about one record per 36 clocks however idle the pipe is
  const double t_issue = warp_blocks * recs_per_block * 36.0 / ((double)resident * inst.WARPS);
  const double t = rounding * (std::max(wf_compute + wf_staging, t_issue) + fixed) / sm_count;
  if (out) {
    out->valid = true;
    out->shape = s;
    TiledParams &p = out->p;
    p.lists = reinterpret_cast<const uint2 *>(f->d_lists);
    p.list_offsets = f->d_list_offsets;
    p.N = s.N; p.H = s.H; p.W = s.W; p.IC = s.IC; p.OC = s.OC; p.OH = s.OH; p.OW = s.OW; p.P = s.P;
    p.KS = s.KS; p.S = s.S;
    p.NSEG = NSEG; p.TH = TH; p.tiles_w = tiles_w; p.tiles_h = tiles_h;
    p.pair_mode = pair_mode;
    p.ROWS = ROWS; p.COLS = COLS; p.RP = RP; p.PLP = PLP; p.ICP = ICP;
    p.stage_bytes = (TIC + 1) * ICP;
    p.n_entries = n_entries;
    p.list_bytes = list_bytes;
    p.T = f->n_stages; p.B = f->n_oc_blocks; p.TIC = TIC;
    p.tic_shift = 0;
    while ((1 << p.tic_shift) < TIC) ++p.tic_shift;
    out->grid = dim3((unsigned)(tiles_w * tiles_h * n_pairs), (unsigned)ctas_y);
    out->smem_bytes = smem;
  }
  return t;
}

struct Candidate {
  double cost;
  int instance, NSEG, TH;
};

// All (instance, tile shape) pairs that fit, cheapest first by the model.
int enumerate_plans(const tetris_filter *f, const ConvShape &s, int *sm_count_out,
                    std::vector<Candidate> *cands) {
  int dev = 0, sm_count = 0;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  TETRIS_CUDA_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  for (int i = 0; i < (int)(sizeof(kInstances) / sizeof(kInstances[0])); ++i) {
    if (kInstances[i].K != f->oc_block) continue;
    for (int NSEG = 1; NSEG <= 32; ++NSEG)
      for (int TH = 1; NSEG * TH <= 32; ++TH) {
        const double t = plan_cost(f, s, kInstances[i], NSEG, TH, sm_count, kSmemLimit, nullptr);
        if (t >= 0.0) cands->push_back({t, i, NSEG, TH});
      }
  }
  if (cands->empty()) {
    set_error("tiled kernel: no tile geometry fits shared memory (tile_ic=%d, list piece %d units)",
              f->tile_ic, f->max_list_units);
    return TETRIS_ERR_UNSUPPORTED;
  }
  std::sort(cands->begin(), cands->end(),
            [](const Candidate &a, const Candidate &b) { return a.cost < b.cost; });
  *sm_count_out = sm_count;
  return TETRIS_OK;
}

void fill_plan(const tetris_filter *f, const ConvShape &s, const Candidate &c, int sm_count, Plan *plan) {
  plan_cost(f, s, kInstances[c.instance], c.NSEG, c.TH, sm_count, kSmemLimit, plan);
  plan->instance = c.instance;
}

// Estimated time (SM clocks) of the dense tensor-core variant: 128 x 128 output tiles, one K step
// per (filter tap, 32-channel chunk) at about 1700 clocks (measured: 12 tcgen05.mma of
// 128x128x8 plus operand traffic), plus prologue and epilogue, in waves of one CTA per SM.
double tc_cost(const tetris_filter *f, const ConvShape &s, int sm_count) {
  const double tiles = std::ceil((double)s.N * s.OH * s.OW / 128.0 / 0.9) * ((s.OC + 127) / 128);
  // (up to 4 input channels the variant folds taps and channels into one K axis)
  const double iters = s.IC <= 4 ? (double)((s.KS * s.KS * s.IC + 31) / 32) : (double)s.KS * s.KS * ((s.IC + 31) / 32);
  // measured: ~1100 clocks per K step (conv3_3: 7 tiles x 72 steps in 0.283 ms; conv5: 144 steps in
  // 0.088 ms) and ~3500 per tile (conv1_1 folded: 43 one-step tiles in 0.098 ms)
  return std::ceil(tiles / sm_count) * (iters * 1050.0 + 3000.0);
}

int make_plan(const tetris_filter *f, const ConvShape &s, Plan *plan) {
  std::vector<Candidate> cands;
  int sm_count = 0;
  const int rc = enumerate_plans(f, s, &sm_count, &cands);
  if (rc) return rc;
  fill_plan(f, s, cands[0], sm_count, plan);
  // The list kernel's wavefront model counts issue slots only and comes out 1.2-1.75x below the
  // measured time (1.45x on the layers where the two kernels are close); the tensor-core figure
  // is a measured one.
  // (the split-FP16 variant runs the same contraction at roughly half the clocks per K step)
  if (conv_tc16_supported(f, s) && 0.55 * tc_cost(f, s, sm_count) < 1.45 * cands[0].cost) plan->use_tc = 2;
  else plan->use_tc = conv_tc_supported(f, s) && tc_cost(f, s, sm_count) < 1.45 * cands[0].cost ? 1 : 0;
  return TETRIS_OK;
}

template <int K, int P2, int WARPS, int MINB>
int launch_instance(const Plan &plan, const float *in, float *out, cudaStream_t st) {
  auto kern = conv_tiled_kernel<K, P2, WARPS, MINB>;
  static thread_local bool configured[16] = {false};  // per device: large shared memory opted in
  int dev = 0;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  if (plan.smem_bytes > 48 * 1024 && (dev >= 16 || !configured[dev])) {
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemLimit));
    if (dev < 16) configured[dev] = true;
  }
  TiledParams p = plan.p;
  p.in = in;
  p.out = out;
  kern<<<plan.grid, WARPS * 32, plan.smem_bytes, st>>>(p);
  TETRIS_CUDA_TRY(cudaGetLastError());
  count_launch();
  return TETRIS_OK;
}

struct PlanCache {
  std::mutex mutex;
  Plan last;                 // plan of the most recent shape (a layer keeps one shape)
  std::vector<Plan> tuned;   // plans chosen by timing (tetris_conv2d_tune); they win over `last`
};

bool same_shape(const ConvShape &a, const ConvShape &b) {
  return a.N == b.N && a.H == b.H && a.W == b.W && a.IC == b.IC && a.OC == b.OC && a.KS == b.KS &&
         a.S == b.S && a.P == b.P;
}

}  // namespace

void *tiled_plan_cache_new() { return new (std::nothrow) PlanCache(); }
void tiled_plan_cache_delete(void *c) { delete static_cast<PlanCache *>(c); }

void tiled_plans_export(const tetris_filter *f, std::vector<int32_t> *out) {
  PlanCache *cache = static_cast<PlanCache *>(f->plan_cache);
  if (!cache) return;
  std::lock_guard<std::mutex> lock(cache->mutex);
  for (const Plan &t : cache->tuned) {
    const int32_t rec[kTunedInts] = {t.shape.N, t.shape.H, t.shape.W, t.shape.S, t.shape.P,
                                     t.instance, t.p.NSEG, t.p.TH, t.use_tc};
    out->insert(out->end(), rec, rec + kTunedInts);
  }
}

// Rebuilds each plan from its tile shape; records that do not fit this filter any more (another
// device with less shared memory, a damaged record) are skipped: the launch then plans afresh.
void tiled_plans_import(const tetris_filter *f, const int32_t *plans, int n) {
  PlanCache *cache = static_cast<PlanCache *>(f->plan_cache);
  if (!cache || f->groups != 1) return;
  int dev = 0, sm_count = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return;
  for (int i = 0; i < n; ++i) {
    const int32_t *r = plans + (size_t)i * kTunedInts;
    ConvShape s;
    s.N = r[0]; s.H = r[1]; s.W = r[2]; s.S = r[3]; s.P = r[4];
    s.IC = f->in_channel; s.OC = f->out_channel; s.KS = f->kernel_size;
    if (s.N < 1 || s.H < 1 || s.W < 1 || s.S < 1 || s.P < 0 || s.H + 2 * s.P < s.KS || s.W + 2 * s.P < s.KS) continue;
    s.OH = (s.H + 2 * s.P - s.KS) / s.S + 1;
    s.OW = (s.W + 2 * s.P - s.KS) / s.S + 1;
    const int inst = r[5], NSEG = r[6], TH = r[7];
    if (!conv_tiled_supported(f, s) || inst < 0 || inst >= (int)(sizeof(kInstances) / sizeof(kInstances[0])) ||
        kInstances[inst].K != f->oc_block || NSEG < 1 || TH < 1 || NSEG * TH > 32)
      continue;
    Plan plan;
    if (plan_cost(f, s, kInstances[inst], NSEG, TH, sm_count, kSmemLimit, &plan) < 0.0) continue;
    plan.instance = inst;
    plan.use_tc = r[8] == 2 && conv_tc16_supported(f, s) ? 2 : r[8] != 0 && conv_tc_supported(f, s) ? 1 : 0;
    std::lock_guard<std::mutex> lock(cache->mutex);
    if (cache->tuned.size() < 8) cache->tuned.push_back(plan);
  }
}

bool conv_tiled_supported(const tetris_filter *f, const ConvShape &s) {
  if (f->groups != 1 || !f->d_lists) return false;
  if (s.KS < 1 || s.KS > 8 || s.S < 1 || s.S > 4) return false;
  if (!(f->oc_block == 16 || f->oc_block == 8)) return false;
  const int tic = f->tile_ic;
  if (tic < 4 || tic > 64 || (tic & (tic - 1)) != 0) return false;
  if ((long long)s.N * s.H * s.W * s.IC >= (1ll << 31)) return false;
  if (s.N < 1 || s.OH < 1 || s.OW < 1) return false;
  return true;
}

int launch_plan(const Plan &plan, const float *in, float *out, cudaStream_t st) {
  // Every instance is bound by shared-memory bandwidth; the narrower register blocks fit more
  // resident warps, the P2 = 2 instances trade a little more record traffic for twice the CTAs
  // on small images.
  switch (plan.instance) {
    case 0: return launch_instance<8, 4, 8, 2>(plan, in, out, st);
    case 1: return launch_instance<8, 2, 8, 3>(plan, in, out, st);
    case 2: return launch_instance<16, 4, 4, 3>(plan, in, out, st);
    default: return launch_instance<16, 2, 4, 4>(plan, in, out, st);
  }
}

// Times the `max_candidates` plans the model ranks best (a few launches each, events on `st`),
// keeps the fastest with the filter and reports its time.  The counterpart of the reference's
// exhaustive tile search (Tetris/spconv2d.cc:285-311), without rebuilding the filter per tile.
int tune_conv_tiled(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                    cudaStream_t st, int max_candidates, float *best_ms) {
  if (!conv_tiled_supported(f, s)) {
    set_error("tiled kernel does not cover this filter/shape");
    return TETRIS_ERR_UNSUPPORTED;
  }
  std::vector<Candidate> cands;
  int sm_count = 0;
  int rc = enumerate_plans(f, s, &sm_count, &cands);
  if (rc) return rc;
  if ((int)cands.size() > max_candidates) cands.resize(max_candidates);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  TETRIS_CUDA_TRY(cudaEventCreate(&e0));
  if (cudaEventCreate(&e1) != cudaSuccess) { cudaEventDestroy(e0); set_error("cudaEventCreate failed"); return TETRIS_ERR_CUDA; }
  Plan best_plan;
  float best = -1.f;
  const int reps = 5;
  const bool debug = getenv("TETRIS_DEBUG_PLAN") != nullptr;  // prints every timed candidate
  for (const Candidate &c : cands) {
    Plan plan;
    fill_plan(f, s, c, sm_count, &plan);
    rc = launch_plan(plan, in, out, st);  // warm-up (also opts in to large shared memory)
    if (rc) break;
    cudaEventRecord(e0, st);
    for (int i = 0; i < reps && !rc; ++i) rc = launch_plan(plan, in, out, st);
    cudaEventRecord(e1, st);
    if (rc) break;
    if (cudaEventSynchronize(e1) != cudaSuccess) {
      set_error("tuning launch failed: %s", cudaGetErrorString(cudaGetLastError()));
      rc = TETRIS_ERR_CUDA;
      break;
    }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    ms /= reps;
    if (debug)
      fprintf(stderr, "[tetris tune] K=%d P2=%d warps=%d NSEG=%d TH=%d grid=%ux%u smem=%zu model=%.0f clk -> %.4f ms\n",
              kInstances[c.instance].K, kInstances[c.instance].P2, kInstances[c.instance].WARPS, c.NSEG,
              c.TH, plan.grid.x, plan.grid.y, plan.smem_bytes, c.cost, ms);
    if (best < 0.f || ms < best) { best = ms; best_plan = plan; }
  }
  // the dense tensor-core variant competes too, when it covers the shape
  if (!rc && conv_tc_supported(f, s) && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
    rc = launch_conv_tc(f, in, out, s, st);
    cudaEventRecord(e0, st);
    for (int i = 0; i < reps && !rc; ++i) rc = launch_conv_tc(f, in, out, s, st);
    cudaEventRecord(e1, st);
    if (!rc && cudaEventSynchronize(e1) != cudaSuccess) {
      set_error("tuning launch failed: %s", cudaGetErrorString(cudaGetLastError()));
      rc = TETRIS_ERR_CUDA;
    }
    if (!rc && !conv_tc_check_error(f)) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      ms /= reps;
      if (debug) fprintf(stderr, "[tetris tune] tensor-core variant -> %.4f ms\n", ms);
      if (ms < best) { best = ms; best_plan.use_tc = 1; }
    }
  }
  // ... and the split-FP16 variant (its launch includes the guard kernel queued behind it)
  if (!rc && conv_tc16_supported(f, s) && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
    rc = launch_conv_tc16(f, in, out, s, st);
    cudaEventRecord(e0, st);
    for (int i = 0; i < reps && !rc; ++i) rc = launch_conv_tc16(f, in, out, s, st);
    cudaEventRecord(e1, st);
    if (!rc && cudaEventSynchronize(e1) != cudaSuccess) {
      set_error("tuning launch failed: %s", cudaGetErrorString(cudaGetLastError()));
      rc = TETRIS_ERR_CUDA;
    }
    if (!rc && !conv_tc16_check_error(f)) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      ms /= reps;
      if (debug) fprintf(stderr, "[tetris tune] split-FP16 tensor-core variant -> %.4f ms\n", ms);
      if (ms < best) { best = ms; best_plan.use_tc = 2; }
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc) return rc;
  PlanCache *cache = static_cast<PlanCache *>(f->plan_cache);
  if (cache) {
    std::lock_guard<std::mutex> lock(cache->mutex);
    bool replaced = false;
    for (Plan &t : cache->tuned)
      if (same_shape(t.shape, s)) { t = best_plan; replaced = true; }
    if (!replaced) {
      if (cache->tuned.size() >= 8) cache->tuned.erase(cache->tuned.begin());
      cache->tuned.push_back(best_plan);
    }
  }
  if (best_ms) *best_ms = best;
  return TETRIS_OK;
}

// Which variant an automatic launch of this shape would use right now (tuned plan if there is one,
// else the cost models): TETRIS_VARIANT_TILED or TETRIS_VARIANT_TENSOR.
int conv_auto_choice(const tetris_filter *f, const ConvShape &s, int *variant) {
  Plan plan;
  PlanCache *cache = static_cast<PlanCache *>(f->plan_cache);
  bool hit = false;
  if (cache) {
    std::lock_guard<std::mutex> lock(cache->mutex);
    for (const Plan &t : cache->tuned)
      if (same_shape(t.shape, s)) { plan = t; hit = true; break; }
    if (!hit && cache->last.valid && same_shape(cache->last.shape, s)) { plan = cache->last; hit = true; }
  }
  if (!hit) {
    const int rc = make_plan(f, s, &plan);
    if (rc) return rc;
  }
  *variant = plan.use_tc == 2 ? TETRIS_VARIANT_TENSOR16 : plan.use_tc ? TETRIS_VARIANT_TENSOR : TETRIS_VARIANT_TILED;
  return TETRIS_OK;
}

int launch_conv_tiled(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                      cudaStream_t st, bool allow_tc) {
  if (!conv_tiled_supported(f, s)) {
    set_error("tiled kernel does not cover KS=%d stride=%d oc_block=%d tile_ic=%d", s.KS, s.S,
              f->oc_block, f->tile_ic);
    return TETRIS_ERR_UNSUPPORTED;
  }
  // The tile shape and the kernel instance depend on the filter and the conv shape only; they
  // are worked out once and kept with the filter.
  Plan plan;
  PlanCache *cache = static_cast<PlanCache *>(f->plan_cache);
  bool hit = false;
  if (cache) {
    std::lock_guard<std::mutex> lock(cache->mutex);
    for (const Plan &t : cache->tuned)
      if (same_shape(t.shape, s)) { plan = t; hit = true; break; }
    if (!hit && cache->last.valid && same_shape(cache->last.shape, s)) { plan = cache->last; hit = true; }
  }
  if (!hit) {
    const int rc = make_plan(f, s, &plan);
    if (rc) return rc;
    if (cache) {
      std::lock_guard<std::mutex> lock(cache->mutex);
      cache->last = plan;
    }
  }
  if (allow_tc && plan.use_tc && (reinterpret_cast<uintptr_t>(in) & 15) == 0)
    return plan.use_tc == 2 ? launch_conv_tc16(f, in, out, s, st) : launch_conv_tc(f, in, out, s, st);
  return launch_plan(plan, in, out, st);
}

}  // namespace tetris
