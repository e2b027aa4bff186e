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

namespace tetris {

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
