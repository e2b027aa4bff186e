// SparseFilter with the reference's constructor, getters and public fields
// (Tetris/spconv2d_utils.h:23-27, 495-514), implemented over the engine's C ABI.
//
// The constructor compresses the dense OIHW filter on the current device; the destructor frees
// it.  The compressed layout is the engine's own, so the five device getters do not return
// arrays a caller could read: they all return the same opaque token, which the SparseConv2d<>
// launcher in spconv2d_kernel.cuh turns back into the filter handle.  Host code that only passes
// the getters through to the launcher -- which is all the reference does with them
// (Tetris/spconv2d.cc:294-304) -- keeps working unchanged.  Like the reference class the object
// must not be copied (it owns device memory); here copying is deleted rather than left to
// double-free.
#ifndef TETRIS_B200_HOST_SPCONV2D_UTILS_H_
#define TETRIS_B200_HOST_SPCONV2D_UTILS_H_

#include <cuda_runtime.h>

#include <vector>

#include "cuda_utils.h"
#include "tetris_b200.h"

#define WARP_SIZE 32

template <typename ValueType, typename OffsetType, typename PositionType>
struct SparseFilter {
  SparseFilter(float *filter, int in_channel, int out_channel, int kernel_size, int TILE_IC = 32,
               bool apply_reorder = false, bool apply_vectorize = true)
      : in_channel_(in_channel), out_channel_(out_channel), kernel_size_(kernel_size), nnz_(0),
        TILE_IC_(TILE_IC), handle_(nullptr) {
    (void)apply_reorder;    // the engine always groups weights by output channel and input offset
    (void)apply_vectorize;  // ... and always streams them with vector loads
    int device = 0;
    checkCudaErrors(cudaGetDevice(&device));
    // TILE_IC of the reference is a tile-table entry chosen per timed candidate
    // (Tetris/spconv2d.cc:90-275).  Its default argument, 32, selects the engine's own stage
    // size (chosen from the kernel size and the longest list piece); any other value the engine
    // accepts as a stage size (4, 8, 16, 64) is forwarded; a value it cannot use (e.g. 24) also
    // falls back to the engine's choice, and GetTileIC() / TILE_IC_ report what was used.
    tetris_filter_opts_t opts = {};
    if (TILE_IC != 32 && TILE_IC >= 4 && TILE_IC <= 64 && (TILE_IC & (TILE_IC - 1)) == 0) opts.tile_ic = TILE_IC;
    checkTetris(tetris_filter_create_ex(filter, in_channel, out_channel, kernel_size, 1, device, &opts, &handle_));
    tetris_filter_info_t info;
    checkTetris(tetris_filter_info(handle_, &info));
    nnz_ = (int)info.nnz;
    TILE_IC_ = info.tile_ic;
    oc_permutation_.resize(out_channel);
    for (int o = 0; o < out_channel; ++o) oc_permutation_[o] = o;  // the engine does not permute
  }
  ~SparseFilter() { tetris_filter_destroy(handle_); }
  SparseFilter(const SparseFilter &) = delete;
  SparseFilter &operator=(const SparseFilter &) = delete;

  OffsetType *GetDeviceOffsets() { return reinterpret_cast<OffsetType *>(handle_); }
  OffsetType *GetDeviceStageLen() { return reinterpret_cast<OffsetType *>(handle_); }
  ValueType *GetDeviceValues() { return reinterpret_cast<ValueType *>(handle_); }
  PositionType *GetDevicePosition() { return reinterpret_cast<PositionType *>(handle_); }
  PositionType *GetDeviceOCPermutation() { return reinterpret_cast<PositionType *>(handle_); }
  int GetTileIC() { return TILE_IC_; }
  tetris_filter_t *GetHandle() { return handle_; }

  int in_channel_, out_channel_, kernel_size_;
  int nnz_;
  int TILE_IC_;
  std::vector<OffsetType> oc_permutation_;
  // The reference keeps host copies of its device arrays in these four public fields
  // (Tetris/spconv2d_utils.h:505-514).  The engine compresses on the device into a layout of
  // its own, so they stay EMPTY here; tetris_filter_download / tetris_filter_download_lists
  // return the engine's forms for a host that wants to look at them.
  std::vector<OffsetType> stage_len_;
  std::vector<OffsetType> offsets_;
  std::vector<PositionType> position_;
  std::vector<ValueType> values_;

 private:
  tetris_filter_t *handle_;
};

#endif  // TETRIS_B200_HOST_SPCONV2D_UTILS_H_
