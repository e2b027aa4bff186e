// Tiled sparse-filter convolution for sm_100a: the hot kernel.
//
// Role of the reference's SparseConv2dKernel + LoadImg2SharedMem
// (Tetris/spconv2d_kernel.cu:13-160), designed differently:
//
//  * lanes are output PIXELS, not output channels.  A lane owns P2 neighbouring output columns of
//    one tile row in two "planes" (two images of the batch, or the upper and lower half of a
//    tile when the batch is odd) and K output channels: K*P2 float2 accumulators in registers.
//    Packing the two planes into one float2 lets every multiply-add be one packed FP32 FMA
//    (fma.rn.f32x2), which halves the issue slots the arithmetic needs.
//  * the weight stream of a warp is warp-uniform: all 32 lanes execute the same compressed
//    PROGRAM (format.h).  A GROUP record loads the input window of one (input channel, filter
//    row) from shared memory into registers once; every following FMA record -- any of the K
//    channels, any filter column -- reuses it from registers.  The record's code selects, by a
//    jump table, the straight-line block that updates accumulator row k with column shift s, so
//    no register is ever indexed dynamically.  Shared memory traffic per multiply-add drops by
//    the number of nonzero weights that share an input offset, which is what lifts the kernel
//    above the one-shared-load-per-FMA ceiling of the reference design.
//  * the input tile (with halo) is staged per input-channel stage with cp.async into a
//    double-buffered shared tile whose layout makes the window loads conflict-free 16-byte
//    loads: per channel, [chunk plane j][input row][segment] chunks of {col0.p0, col0.p1,
//    col1.p0, col1.p1}, plus a small side region for the right-hand halo of each row.
//    (TMA tiled loads do not fit: the source is channel-innermost NHWC while the tile needs the
//    channel outermost and two planes interleaved, so the copy is an element-wise gather.)
//
// NHWC in, NHWC out, FP32, output fully overwritten -- the contract of the reference launcher
// (Tetris/spconv2d_kernel.cu:163-188).
#include "internal.h"
#include "interp_gen.h"

namespace tetris {
namespace {

constexpr int kWarps = 4;  // warps per CTA; each warp runs one output-channel block

template <int KS, int S, int P2>
struct WinCfg {
  static constexpr int WIN = (P2 - 1) * S + KS;            // float2 window entries a lane reads
  static constexpr int OWN = P2 * S / 2;                   // 16-byte chunks of its own columns
  static constexpr int HALO = (KS > S) ? (KS - S + 1) / 2 : 0;  // chunks borrowed from the right
  static constexpr int NCH = OWN + HALO;
  static_assert(P2 % 2 == 0, "P2 must be even");
  static_assert(2 * NCH >= WIN, "window must be covered by the chunks");
  static_assert(HALO <= OWN, "halo chunks come from one neighbouring segment");
};

struct TiledParams {
  const float *in;
  float *out;
  const uint2 *ops;
  const int32_t *prog_offsets;
  int N, H, W, IC, OC, OH, OW, P;
  int TS, TH;            // segments per tile row, tile rows; TS*TH lanes are in use
  int tiles_w, tiles_h;  // tiles along OW and along OH
  int pair_mode;         // 0: planes are images 2j and 2j+1; 1: upper/lower TH rows of one image
  int ROWS, CIN2;        // staged input rows / columns per plane
  int cp16;              // bytes between chunk planes  (ROWS*TS*16)
  int hbase;             // byte offset of the halo region inside a channel slab (OWN*cp16)
  int icpitch;           // bytes per channel slab
  int stage_bytes;       // TIC * icpitch
  int n_entries;         // staging table entries: 2*ROWS*CIN2
  int prog_bytes;        // shared bytes reserved per warp and buffer for its staged program
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

template <int KS, int S, int K, int P2, int MINB>
__global__ void __launch_bounds__(kWarps * 32, MINB) conv_interp_kernel(const TiledParams p) {
  using C = WinCfg<KS, S, P2>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(smem_raw);
  // layout: [input tile 0][input tile 1][programs 0: kWarps x prog_bytes][programs 1]
  //         [staging table: n_entries x {goff, soff}]
  const uint32_t prog0 = smem0 + 2 * p.stage_bytes;
  int2 *tab = reinterpret_cast<int2 *>(smem_raw + 2 * p.stage_bytes + 2 * kWarps * p.prog_bytes);

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
  const int w0 = tw * p.TS * P2;

  // ---- staging table: for every (plane, input row, input column) of the tile, where it comes
  //      from in global memory and where it goes inside a channel slab ----
  for (int e = tid; e < p.n_entries; e += kWarps * 32) {
    const int ci = e % p.CIN2;
    const int ri = (e / p.CIN2) % p.ROWS;
    const int pl = e / (p.CIN2 * p.ROWS);
    const int n = pl ? n1 : n0;
    const int ih = (pl ? h1 : h0) * S + ri - p.P;
    const int iw = w0 * S + ci - p.P;
    const bool ok = (pl == 0 || v1) && ih >= 0 && ih < p.H && iw >= 0 && iw < p.W;
    const int q = ci >> 1, slot = q / C::OWN, jj = q - slot * C::OWN;
    const int chunk = slot < p.TS ? jj * p.cp16 + (ri * p.TS + slot) * 16
                                  : p.hbase + (ri * C::HALO + jj) * 16;
    tab[e] = make_int2(ok ? (int)((((long long)n * p.H + ih) * p.W + iw) * p.IC) : -1,
                       chunk + (ci & 1) * 8 + pl * 4);
  }
  __syncthreads();

  const int b = blockIdx.y * kWarps + warp;  // output-channel block of this warp
  const bool warp_on = b < p.B;

  const int icl_s = tid & (p.TIC - 1);  // this thread's channel inside a stage (staging role)
  const int pe0 = tid >> p.tic_shift, pe_step = (kWarps * 32) >> p.tic_shift;
  auto issue_stage = [&](int t, int buf) {
    const uint32_t dst_base = smem0 + buf * p.stage_bytes;
    if (warp_on) {  // this warp's program of the stage, 16 bytes (two records) per copy
      const int po = p.prog_offsets[b * p.T + t], pn = p.prog_offsets[b * p.T + t + 1];
      const uint32_t dst_p = prog0 + (buf * kWarps + warp) * p.prog_bytes;
      for (int i = lane; 2 * i < pn - po; i += 32) cp_async16(dst_p + i * 16, p.ops + po + 2 * i);
    }
    const int ic = t * p.TIC + icl_s;
    if (ic < p.IC) {
      const float *src_c = p.in + ic;
      const uint32_t dst_c = dst_base + icl_s * p.icpitch;
      for (int e = pe0; e < p.n_entries; e += pe_step) {
        const int2 ent = tab[e];
        cp_async4(dst_c + ent.y, src_c + (ent.x >= 0 ? ent.x : 0), ent.x >= 0 ? 4 : 0);
      }
    }
    cp_async_commit();
  };

  // ---- this lane's pixels (compute role) ----
  const bool lane_on = lane < p.TS * p.TH;
  const int row = lane_on ? lane / p.TS : 0;
  const int seg = lane_on ? lane % p.TS : 0;
  const uint32_t rp = p.TS * 16;
  const uint32_t own_base = ((row * S) * p.TS + seg) * 16;
  uint32_t halo_base = 0, halo_rp = 0, halo_js = 0;
  if constexpr (C::HALO > 0) {
    const bool inner = seg + 1 < p.TS;
    halo_base = inner ? own_base + 16 : p.hbase + (row * S) * C::HALO * 16;
    halo_rp = inner ? rp : C::HALO * 16;
    halo_js = inner ? (uint32_t)p.cp16 : 16u;
  }

  using I = Interp<KS, S, K, P2>;
  I::init();  // K*P2 packed accumulators, zeroed, in registers the interpreter names statically

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
      I::run(prog0 + ((t & 1) * kWarps + warp) * p.prog_bytes, sbase + own_base, sbase + halo_base,
             (uint32_t)p.icpitch, rp, halo_rp, (uint32_t)p.cp16, halo_js);
    }
    __syncthreads();
  }

  // ---- epilogue: NHWC stores, K consecutive channels per pixel ----
  float2 acc[K][P2];
  I::read(acc);
  if (!warp_on || !lane_on) return;
  const int oc0 = b * K;
  const int kn = min(K, p.OC - oc0);
  const bool vec = (p.OC & 3) == 0 && kn == K;
#pragma unroll
  for (int pl = 0; pl < 2; ++pl) {
    const int n = pl ? n1 : n0;
    const int oh = (pl ? h1 : h0) + row;
    if ((pl == 1 && !v1) || oh >= p.OH) continue;
#pragma unroll
    for (int q = 0; q < P2; ++q) {
      const int ow = w0 + seg * P2 + q;
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
struct Geometry {
  int TS, TH, tiles_w, tiles_h, pair_mode, n_pairs;
  int ROWS, CIN2, cp16, hbase, icpitch, n_entries;
  size_t smem_bytes;
};

template <int KS, int S, int P2>
bool choose_geometry(const ConvShape &s, int TIC, size_t smem_limit, size_t prog_total, Geometry *g) {
  using C = WinCfg<KS, S, P2>;
  const int pair_mode = (s.N % 2 == 0) ? 0 : 1;
  double best = 1e300;
  bool found = false;
  for (int TS = 1; TS <= 32; ++TS) {
    for (int TH = 1; TS * TH <= 32; ++TH) {
      const int rows_per_tile = pair_mode ? 2 * TH : TH;
      const int tiles_w = (s.OW + TS * P2 - 1) / (TS * P2);
      const int tiles_h = (s.OH + rows_per_tile - 1) / rows_per_tile;
      const int ROWS = (TH - 1) * S + KS;
      const int CIN2 = 2 * (TS * C::OWN + C::HALO);
      int icpitch = (C::OWN * ROWS * TS + ROWS * C::HALO) * 16;
      if (((icpitch / 16) & 1) == 0) icpitch += 16;  // odd chunk pitch: fewer staging conflicts
      const int n_entries = 2 * ROWS * CIN2;
      const size_t smem = 2 * (size_t)TIC * icpitch + (size_t)n_entries * sizeof(int2) + prog_total;
      if (smem > smem_limit) continue;
      // cost model: every tile runs one full warp program per stage whatever its lane use;
      // staging grows with the staged area.
      const double cost = (double)tiles_w * tiles_h * (2300.0 + 1.2 * ROWS * CIN2);
      if (cost < best) {
        best = cost;
        found = true;
        g->TS = TS; g->TH = TH; g->tiles_w = tiles_w; g->tiles_h = tiles_h;
        g->pair_mode = pair_mode;
        g->n_pairs = pair_mode ? s.N : s.N / 2;
        g->ROWS = ROWS; g->CIN2 = CIN2;
        g->cp16 = ROWS * TS * 16;
        g->hbase = C::OWN * ROWS * TS * 16;
        g->icpitch = icpitch;
        g->n_entries = n_entries;
        g->smem_bytes = smem;
      }
    }
  }
  return found;
}

template <int KS, int S, int K, int P2, int MINB>
int launch_instance(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                    cudaStream_t st) {
  Geometry g;
  const size_t smem_limit = 200 * 1024 / MINB;
  // one record of slack: the interpreter prefetches one record past END
  const int prog_bytes = ((f->max_prog_ops + 2) * 8 + 15) / 16 * 16;
  if (!choose_geometry<KS, S, P2>(s, f->tile_ic, smem_limit, (size_t)2 * kWarps * prog_bytes, &g)) {
    set_error("interpreter kernel: no tile geometry fits shared memory");
    return TETRIS_ERR_UNSUPPORTED;
  }
  TiledParams p;
  p.in = in; p.out = out;
  p.ops = reinterpret_cast<const uint2 *>(f->d_ops);
  p.prog_offsets = f->d_prog_offsets;
  p.N = s.N; p.H = s.H; p.W = s.W; p.IC = s.IC; p.OC = s.OC; p.OH = s.OH; p.OW = s.OW; p.P = s.P;
  p.TS = g.TS; p.TH = g.TH; p.tiles_w = g.tiles_w; p.tiles_h = g.tiles_h;
  p.pair_mode = g.pair_mode;
  p.ROWS = g.ROWS; p.CIN2 = g.CIN2; p.cp16 = g.cp16; p.hbase = g.hbase; p.icpitch = g.icpitch;
  p.stage_bytes = f->tile_ic * g.icpitch;
  p.n_entries = g.n_entries;
  p.prog_bytes = prog_bytes;
  p.T = f->n_stages; p.B = f->n_oc_blocks; p.TIC = f->tile_ic;
  p.tic_shift = 0;
  while ((1 << p.tic_shift) < f->tile_ic) ++p.tic_shift;

  auto kern = conv_interp_kernel<KS, S, K, P2, MINB>;
  static thread_local size_t configured[16] = {0};  // per device: largest smem size opted into
  int dev = 0;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  if (g.smem_bytes > 48 * 1024 && (dev >= 16 || configured[dev] < g.smem_bytes)) {
    TETRIS_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(200 * 1024 / MINB)));
    if (dev < 16) configured[dev] = 200 * 1024 / MINB;
  }
  dim3 grid((unsigned)(g.tiles_w * g.tiles_h * g.n_pairs),
            (unsigned)((f->n_oc_blocks + kWarps - 1) / kWarps));
  kern<<<grid, kWarps * 32, g.smem_bytes, st>>>(p);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

}  // namespace

bool conv_interp_supported(const tetris_filter *f, const ConvShape &s) {
  if (f->groups != 1) return false;
  if (!(s.KS == 1 || s.KS == 3) || !(s.S == 1 || s.S == 2)) return false;
  if (!(f->oc_block == 16 || f->oc_block == 8)) return false;
  const int tic = f->tile_ic;
  if (tic < 4 || tic > 32 || (tic & (tic - 1)) != 0) return false;
  if ((long long)s.N * s.H * s.W * s.IC >= (1ll << 31)) return false;
  if (s.N < 1 || s.OH < 1 || s.OW < 1) return false;
  return true;
}

int launch_conv_interp(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                      cudaStream_t st) {
  if (!conv_interp_supported(f, s)) {
    set_error("interpreter kernel does not cover KS=%d stride=%d oc_block=%d tile_ic=%d", s.KS, s.S,
              f->oc_block, f->tile_ic);
    return TETRIS_ERR_UNSUPPORTED;
  }
  const int K = f->oc_block;
#define T_LAUNCH(KS_, S_, K_, MINB_)                                         \
  if (s.KS == KS_ && s.S == S_ && K == K_)                                   \
    return launch_instance<KS_, S_, K_, 4, MINB_>(f, in, out, s, st);
  T_LAUNCH(3, 1, 16, 3)
  T_LAUNCH(3, 2, 16, 3)
  T_LAUNCH(1, 1, 16, 3)
  T_LAUNCH(1, 2, 16, 3)
  T_LAUNCH(3, 1, 8, 4)
  T_LAUNCH(3, 2, 8, 4)
  T_LAUNCH(1, 1, 8, 4)
  T_LAUNCH(1, 2, 8, 4)
#undef T_LAUNCH
  set_error("interpreter kernel: no instance");
  return TETRIS_ERR_UNSUPPORTED;
}

}  // namespace tetris
