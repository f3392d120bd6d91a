// tcgen05 tensor-core kernels (placeholder while the SIMT path is brought up).
#pragma once
#include <cuda_runtime.h>
#include "../../include/na2d.h"
#include "na2d_index.cuh"

namespace na2d_tc {
__device__ unsigned int g_error_word = 0;

inline bool supported(int, int, int) { return false; }
inline int forward(const Na2dGeom&, int, const void*, const void*, const void*, void*, float*, int, cudaStream_t, int*) { return NA2D_ERR_UNSUPPORTED; }
inline int backward_dq(const Na2dGeom&, int, const void*, const void*, const void*, const void*, const float*, const void*, void*, float*, int, cudaStream_t, int*) { return NA2D_ERR_UNSUPPORTED; }
inline int backward_dkdv(const Na2dGeom&, int, const void*, const void*, const void*, const float*, const void*, const float*, void*, void*, int, cudaStream_t, int*) { return NA2D_ERR_UNSUPPORTED; }
inline int read_and_clear_error(unsigned int* word, cudaStream_t st) {
    if (cudaMemcpyFromSymbolAsync(word, g_error_word, sizeof(unsigned int), 0, cudaMemcpyDeviceToHost, st) != cudaSuccess) return NA2D_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return NA2D_ERR_CUDA;
    unsigned int zero = 0;
    if (cudaMemcpyToSymbolAsync(g_error_word, &zero, sizeof(unsigned int), 0, cudaMemcpyHostToDevice, st) != cudaSuccess) return NA2D_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return NA2D_ERR_CUDA;
    return NA2D_OK;
}
}  // namespace na2d_tc
