// tetris_list_offsets_noalloc: the piece offsets of the LIST form without a single allocation.
//
// For callers that may not allocate device memory where they call us: a serving process that
// hands all of its device memory to one pool at start-up and forbids cudaMalloc on the request
// path (it synchronises the whole device, and it can fail once the pool owns the memory), or a
// plugin that runs inside somebody else's stream-ordered pipeline and must not stall it.  Such a
// caller brings the dense filter and the output array; the one thing the computation needs
// beyond them -- the per-piece record counts that the scan turns into offsets -- lives in a
// fixed array that is part of the library image on every GPU that loads it.
#include <mutex>

#include "internal.h"

namespace tetris {
namespace {

// Scratch of the entry point: one count per piece.  kNoAllocMaxPieces * 4 bytes = 64 KiB are
// held on every device that loads the library, until the process exits.
constexpr int kNoAllocMaxPieces = 16384;
static __device__ __align__(256) int32_t g_piece_counts[kNoAllocMaxPieces];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
int32_t *g_piece_counts_addr[kMaxDevices] = {nullptr};

// In host code `g_piece_counts` is only a handle for the runtime, not an address a kernel may
// use; the device address is asked for once per device, with that device current.
int scratch_for_current_device(int32_t **out) {
  int dev = -1;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("device index %d outside the supported range", dev);
    return TETRIS_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_piece_counts_addr[dev]) {
    void *p = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&p, g_piece_counts);
    if (err != cudaSuccess || !p) {
      set_error("cudaGetSymbolAddress of the scratch array failed on device %d: %s", dev,
                cudaGetErrorString(err));
      return TETRIS_ERR_CUDA;
    }
    g_piece_counts_addr[dev] = static_cast<int32_t *>(p);
  }
  *out = g_piece_counts_addr[dev];
  return TETRIS_OK;
}

}  // namespace
}  // namespace tetris

using namespace tetris;

extern "C" int tetris_list_offsets_noalloc(const float *d_filter_oihw, int in_channel,
                                           int out_channel, int kernel_size, int oc_block,
                                           int tile_ic, int32_t *d_list_offsets, void *stream) {
  if (!d_filter_oihw || !d_list_offsets) {
    set_error("filter or output pointer is NULL");
    return TETRIS_ERR_INVALID;
  }
  if (in_channel < 1 || out_channel < 1 || kernel_size < 1 || kernel_size > 8 ||
      !(oc_block == 8 || oc_block == 16) || tile_ic < 4 || tile_ic > kMaxTileIc || (tile_ic & 3)) {
    set_error("bad arguments: ic=%d oc=%d ks=%d oc_block=%d tile_ic=%d", in_channel, out_channel,
              kernel_size, oc_block, tile_ic);
    return TETRIS_ERR_INVALID;
  }
  const int B = (out_channel + oc_block - 1) / oc_block, T = (in_channel + tile_ic - 1) / tile_ic;
  const long long pieces = (long long)B * T;
  if (pieces > kNoAllocMaxPieces) {
    set_error("%lld pieces (%d channel blocks x %d stages) exceed the %d this entry point has "
              "scratch for; use tetris_filter_create, or larger oc_block / tile_ic",
              pieces, B, T, kNoAllocMaxPieces);
    return TETRIS_ERR_UNSUPPORTED;
  }
  // Both arrays have to be device memory of the CURRENT device: the scratch array used below is
  // the current device's copy, and a host pointer handed to the kernels would fault.  (A query,
  // not an allocation.)
  int dev = -1;
  TETRIS_CUDA_TRY(cudaGetDevice(&dev));
  const void *ptrs[2] = {d_filter_oihw, d_list_offsets};
  for (const void *ptr : ptrs) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess ||
        !(attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) ||
        (attr.type == cudaMemoryTypeDevice && attr.device != dev)) {
      cudaGetLastError();
      set_error("the %s is not device memory of the current device %d",
                ptr == d_filter_oihw ? "filter" : "offsets array", dev);
      return TETRIS_ERR_INVALID;
    }
  }
  int32_t *d_counts = nullptr;
  int rc = scratch_for_current_device(&d_counts);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // Every count in [0, pieces) is rewritten by the count kernel before the scan reads it, so
  // nothing of an earlier call has to be cleared.
  if ((rc = list_count(d_filter_oihw, in_channel, out_channel, kernel_size, oc_block, tile_ic, B, T,
                       d_counts, st)))
    return rc;
  return compress_scan(d_counts, d_list_offsets, (int)pieces, st);
}
