// Error-check macros with the reference's names (Tetris/cuda_utils.h:9-27).  The engine itself
// reports errors as status codes; these are for host programs that keep the reference's
// print-and-exit style.
#ifndef TETRIS_B200_HOST_CUDA_UTILS_H_
#define TETRIS_B200_HOST_CUDA_UTILS_H_

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "tetris_b200.h"

#define checkCudaErrors(call)                                                              \
  do {                                                                                     \
    const cudaError_t status_ = (call);                                                    \
    if (status_ != cudaSuccess) {                                                          \
      std::printf("CUDA error at %s %d: %s\n", __FILE__, __LINE__, cudaGetErrorString(status_)); \
      std::exit(EXIT_FAILURE);                                                             \
    }                                                                                      \
  } while (0)

// Same style for the engine's own status codes.
#define checkTetris(call)                                                                  \
  do {                                                                                     \
    const int status_ = (call);                                                            \
    if (status_ != TETRIS_OK) {                                                            \
      std::printf("tetris_b200 error %d at %s %d: %s\n", status_, __FILE__, __LINE__,      \
                  tetris_last_error());                                                    \
      std::exit(EXIT_FAILURE);                                                             \
    }                                                                                      \
  } while (0)

#endif  // TETRIS_B200_HOST_CUDA_UTILS_H_
