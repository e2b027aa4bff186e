// Weight compressor: dense OIHW filter (already on the device) -> program stream (format.h).
//
// Replaces the host-side SparseFilter constructor of the reference
// (Tetris/spconv2d_utils.h:25-245: per-stage gather, bank-aware reorder, pad-and-interleave).
// Three kernels: count (one warp per program measures its record count with ballots), scan
// (exclusive prefix sum of the counts -> program offsets) and fill (the same walk again, this
// time writing records at ballot-ranked positions).  The walk order fixes the record order, so
// the stream is a pure function of the filter: count and fill cannot disagree.
#include "internal.h"

namespace tetris {

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxRounds = (kMaxOcBlock * 8 + 31) / 32;  // K*KS entries of a group, 32 per round

// One group = the K x KS weights {oc in block b} x {filter column s} at (ic, r).
// Entry e = k*KS + s is tested by lane (e % 32) in round (e / 32).
struct GroupScan {
  unsigned mask[kMaxRounds];
  float val[kMaxRounds];
  int count;
};

__device__ __forceinline__ GroupScan scan_group(const float *__restrict__ filt, int IC, int OC,
                                                int KS, int K, int b, int ic, int r, int lane) {
  GroupScan g;
  g.count = 0;
  const int E = K * KS;
#pragma unroll
  for (int round = 0; round < kMaxRounds; ++round) {
    const int e = round * 32 + lane;
    float v = 0.f;
    if (e < E) {
      const int k = e / KS, s = e - k * KS;
      const int oc = b * K + k;
      if (oc < OC && ic < IC) v = filt[(((size_t)oc * IC + ic) * KS + r) * KS + s];
    }
    g.val[round] = v;
    g.mask[round] = __ballot_sync(0xffffffffu, v != 0.f);
    g.count += __popc(g.mask[round]);
  }
  return g;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
count_kernel(const float *__restrict__ filt, int IC, int OC, int KS, int K, int TIC, int B, int T,
             int32_t *__restrict__ lens, unsigned long long *__restrict__ nnz_total) {
  const int p = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (p >= B * T) return;
  const int b = p / T, t = p - b * T;
  int len = 0, nnz = 0;
  for (int g = 0; g < TIC * KS; ++g) {
    const int icl = g / KS, r = g - icl * KS;
    const GroupScan gs = scan_group(filt, IC, OC, KS, K, b, t * TIC + icl, r, lane);
    len += gs.count + (gs.count > 0 ? 1 : 0);
    nnz += gs.count;
  }
  len += 1;  // END
  len = (len + kProgAlignOps - 1) / kProgAlignOps * kProgAlignOps;
  if (lane == 0) {
    lens[p] = len;
    atomicAdd(nnz_total, (unsigned long long)nnz);
  }
}

// Exclusive scan of n ints by one block; offsets[n] = total.
__global__ void __launch_bounds__(1024)
scan_kernel(const int32_t *__restrict__ lens, int32_t *__restrict__ offsets, int n) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < n ? lens[i] : 0;
    int x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int before = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + x - v;
    if (i < n) offsets[i] = before;
    __syncthreads();
    if (threadIdx.x == 1023) carry = before + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[n] = carry;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
fill_kernel(const float *__restrict__ filt, int IC, int OC, int KS, int K, int TIC, int B, int T,
            const int32_t *__restrict__ offsets, uint64_t *__restrict__ ops, long long n_ops) {
  const int p = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int P = B * T;
  if (p >= P) return;
  const int b = p / T, t = p - b * T;
  const uint32_t c_group = code_group(K, KS), c_end = code_end(K, KS);
  long long pos = offsets[p];
  for (int g = 0; g < TIC * KS; ++g) {
    const int icl = g / KS, r = g - icl * KS;
    const GroupScan gs = scan_group(filt, IC, OC, KS, K, b, t * TIC + icl, r, lane);
    if (gs.count == 0) continue;
    if (lane == 0) ops[pos] = make_op(((uint32_t)icl << 8) | (uint32_t)r, c_group);
    pos += 1;
#pragma unroll
    for (int round = 0; round < kMaxRounds; ++round) {
      const unsigned m = gs.mask[round];
      if (m & (1u << lane)) {
        const int rank = __popc(m & ((1u << lane) - 1u));
        ops[pos + rank] = make_op(__float_as_uint(gs.val[round]), (uint32_t)(round * 32 + lane));
      }
      pos += __popc(m);
    }
  }
  // END, then END padding up to the next program (or through the tail after the last one).
  const long long stop = (p + 1 < P) ? (long long)offsets[p + 1] : n_ops;
  for (long long i = pos + lane; i < stop; i += 32) ops[i] = make_op(0u, c_end);
}

// ---- LIST form ------------------------------------------------------------------------------
// One warp per piece.  The weights of one output channel and one stage are TIC*KS*KS contiguous
// floats, scanned 32 at a time; a ballot gives each nonzero its rank in the list.
__device__ __forceinline__ int list_row_len(int IC, int KS, int TIC, int t) {
  const int ics = min(TIC, IC - t * TIC);
  return ics * KS * KS;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
list_count_kernel(const float *__restrict__ filt, int IC, int OC, int KS, int K, int TIC, int B,
                  int T, int32_t *__restrict__ lens) {
  const int p = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (p >= B * T) return;
  const int b = p / T, t = p - b * T;
  const int row_len = list_row_len(IC, KS, TIC, t);
  int total = 0;
  for (int k = 0; k < K; ++k) {
    const int oc = b * K + k;
    if (oc >= OC) break;
    const float *row = filt + ((size_t)oc * IC + (size_t)t * TIC) * KS * KS;
    int n_k = 0;
    for (int e0 = 0; e0 < row_len; e0 += 32) {
      const int e = e0 + lane;
      const bool nz = e < row_len && row[e] != 0.f;
      n_k += __popc(__ballot_sync(0xffffffffu, nz));
    }
    total += (n_k + 1) & ~1;  // lists are padded to an even length
  }
  int len = list_header_units(K) + total + 2;  // header, records, two sentinels
  len = (len + kProgAlignOps - 1) / kProgAlignOps * kProgAlignOps;
  if (lane == 0) lens[p] = len;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
list_fill_kernel(const float *__restrict__ filt, int IC, int OC, int KS, int K, int TIC, int B,
                 int T, const int32_t *__restrict__ offsets, uint64_t *__restrict__ units,
                 long long n_units) {
  const int p = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int P = B * T;
  if (p >= P) return;
  const int b = p / T, t = p - b * T;
  const int row_len = list_row_len(IC, KS, TIC, t);
  const int KK = KS * KS;
  uint32_t *hdr = reinterpret_cast<uint32_t *>(units + offsets[p]);
  long long pos = (long long)offsets[p] + list_header_units(K);
  int total = 0;
  for (int k = 0; k < K; ++k) {
    const int oc = b * K + k;
    int n_k = 0;
    if (oc < OC) {
      const float *row = filt + ((size_t)oc * IC + (size_t)t * TIC) * KK;
      for (int e0 = 0; e0 < row_len; e0 += 32) {
        const int e = e0 + lane;
        const float v = e < row_len ? row[e] : 0.f;
        const unsigned m = __ballot_sync(0xffffffffu, v != 0.f);
        if (v != 0.f) {
          const int icl = e / KK, rs = e - icl * KK, r = rs / KS, s = rs - r * KS;
          units[pos + n_k + __popc(m & ((1u << lane) - 1u))] =
              make_op(__float_as_uint(v), ((uint32_t)icl << 8) | ((uint32_t)r << 4) | (uint32_t)s);
        }
        n_k += __popc(m);
      }
    }
    const uint64_t pad = make_op(0u, (uint32_t)TIC << 8);
    if ((n_k & 1) && lane == 0) units[pos + n_k] = pad;
    n_k = (n_k + 1) & ~1;
    if (lane == 0) hdr[k] = (uint32_t)n_k;
    pos += n_k;
    total += n_k;
  }
  if (lane < kListHeaderWords) hdr[K + lane] = lane == 0 ? (uint32_t)total : 0u;
  // sentinels, then the same padding record up to the next piece (or through the tail)
  const long long stop = (p + 1 < P) ? (long long)offsets[p + 1] : n_units;
  for (long long i = pos + lane; i < stop; i += 32) units[i] = make_op(0u, (uint32_t)TIC << 8);
}

}  // namespace

int list_count(const float *d_filter, int IC, int OC, int KS, int K, int TIC, int B, int T,
               int32_t *d_lens, cudaStream_t st) {
  const int P = B * T;
  list_count_kernel<<<(P + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, st>>>(
      d_filter, IC, OC, KS, K, TIC, B, T, d_lens);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

int list_fill(const float *d_filter, int IC, int OC, int KS, int K, int TIC, int B, int T,
              const int32_t *d_offsets, uint64_t *d_units, int64_t n_units, cudaStream_t st) {
  const int P = B * T;
  list_fill_kernel<<<(P + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, st>>>(
      d_filter, IC, OC, KS, K, TIC, B, T, d_offsets, d_units, (long long)n_units);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

size_t compress_scratch_bytes(int n_programs) {
  // program lengths, then one 64-bit nonzero counter (8-byte aligned)
  return ((size_t)n_programs * sizeof(int32_t) + 7) / 8 * 8 + sizeof(unsigned long long);
}

static unsigned long long *nnz_slot(int32_t *d_scratch, int n_programs) {
  return reinterpret_cast<unsigned long long *>(reinterpret_cast<char *>(d_scratch) +
                                                ((size_t)n_programs * sizeof(int32_t) + 7) / 8 * 8);
}

// lens -> d_scratch[0..n), nnz -> the counter behind them; offsets -> d_offsets[0..n].
int compress_count(const float *d_filter, int IC, int OC, int KS, int K, int TIC, int B, int T,
                   int32_t *d_scratch, cudaStream_t st) {
  const int P = B * T;
  unsigned long long *d_nnz = nnz_slot(d_scratch, P);
  TETRIS_CUDA_TRY(cudaMemsetAsync(d_nnz, 0, sizeof(unsigned long long), st));
  count_kernel<<<(P + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, st>>>(
      d_filter, IC, OC, KS, K, TIC, B, T, d_scratch, d_nnz);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

int compress_scan(const int32_t *d_scratch, int32_t *d_offsets, int n_programs, cudaStream_t st) {
  scan_kernel<<<1, 1024, 0, st>>>(d_scratch, d_offsets, n_programs);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

const unsigned long long *compress_nnz_ptr(const int32_t *d_scratch, int n_programs) {
  return nnz_slot(const_cast<int32_t *>(d_scratch), n_programs);
}

int compress_fill(const float *d_filter, int IC, int OC, int KS, int K, int TIC, int B, int T,
                  const int32_t *d_offsets, uint64_t *d_ops, int64_t n_ops, cudaStream_t st) {
  const int P = B * T;
  fill_kernel<<<(P + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, st>>>(
      d_filter, IC, OC, KS, K, TIC, B, T, d_offsets, d_ops, (long long)n_ops);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

}  // namespace tetris
