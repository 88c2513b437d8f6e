// Cluster-per-row softmax for rows wider than one block's registers
// (softmax_wide.cu). Each call sets *handled; when false nothing was launched
// and the caller falls back to its generic kernel.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace evg {
int softmax_wide_fwd(int dtype, const void* x, void* y, int64_t rows, int64_t cols,
                     cudaStream_t stream, bool* handled);
int softmax_wide_bwd(int dtype, const void* y, const void* dy, void* dx, int64_t rows,
                     int64_t cols, cudaStream_t stream, bool* handled);
}  // namespace evg
