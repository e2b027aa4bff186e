// Compressed sparse-filter format shared by the compressor and the convolution kernels.
//
// The filter (dense OIHW, OC x IC x KS x KS) is cut into PROGRAMS.  Program (b, t) covers the
// output channels of block b (oc in [b*K, b*K+K)) and the input channels of stage t
// (ic in [t*TIC, t*TIC+TIC)).  A program is a stream of 8-byte records {payload:u32, code:u32}:
//
//   code <  K*KS   FMA    k = code / KS (output channel inside the block), s = code % KS (filter
//                         column); payload = the FP32 weight.  Applies to the current group.
//   code == K*KS   GROUP  payload = (ic_local << 8) | r: the following FMA records read input
//                         channel t*TIC + ic_local, filter row r.  A group is emitted only when
//                         at least one of its K*KS weights is nonzero.
//   code == K*KS+1 END    end of program.
//
// Groups appear in (ic_local, r) order and the FMA records of a group in (k, s) order, so for
// every output element the taps are accumulated in (ic, r, s) order -- the order of the
// reference's CPU loop nest (Tetris/tensor_utils.cc:151-153).  This replaces the reference's
// per-lane padded value/position arrays (Tetris/spconv2d_utils.h:206-244): weights that share an
// input offset (same ic and r, any k, neighbouring s) sit next to each other, so one staged input
// window feeds all of them from registers.
//
// Programs start on 16-byte boundaries (even record index) and the stream ends with
// kTailPadOps END records so that a reader may prefetch a few records past any END.
#pragma once
#include <stdint.h>

//
// ---- the LIST form (consumed by the tiled kernel) ------------------------------------------
// Same cut into (b, t) pieces, different order inside a piece: one list per output channel of
// the block, each list in (ic, r, s) order -- again the reference's accumulation order.  Piece
// layout, in 32-bit words:
//
//   [0 .. K)      n_k   records in the list of channel k, padding included (always even)
//   [K]           total = sum of n_k
//   [K+1 .. K+4)  zero
//   then `total` 8-byte records {weight:f32, pos:u32}, lists back to back, k = 0 first,
//   pos = (ic_local << 8) | (r << 4) | s; a list with an odd number of nonzeros is padded with
//   one record {0.0f, TIC << 8}: weight zero, position in the all-zero channel slab the kernel
//   keeps behind the TIC staged ones, so the padded multiply-add adds exactly 0;
//   then two such padding records as sentinels, so a reader may always fetch "the next pair".
//
// Pieces start on 16-byte boundaries; offsets are counted in 8-byte units.  Nothing depends on
// the image size: the kernel turns `pos` into a shared-memory byte offset once per staged piece.
namespace tetris {

constexpr int kListHeaderWords = 4;  // words after the K counts: total + 3 zero words
__host__ __device__ inline int list_header_units(int K) { return (K + kListHeaderWords) / 2; }

constexpr int kProgAlignOps = 2;  // programs start at even record indices (16 bytes)
constexpr int kTailPadOps = 16;   // END records after the last program
constexpr int kMaxOcBlock = 16;
constexpr int kMaxTileIc = 64;

__host__ __device__ inline uint32_t code_group(int K, int KS) { return (uint32_t)(K * KS); }
__host__ __device__ inline uint32_t code_end(int K, int KS) { return (uint32_t)(K * KS + 1); }
__host__ __device__ inline uint64_t make_op(uint32_t payload, uint32_t code) {
  return ((uint64_t)code << 32) | payload;
}

}  // namespace tetris
