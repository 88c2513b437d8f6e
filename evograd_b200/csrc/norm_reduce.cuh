// Pieces shared by the normalisation backward kernels: the cap on per-block
// partial rows and the second stage of the atomic-free column reduction.
#pragma once
#include "evg_common.cuh"

namespace evg {

#ifdef __CUDACC__
// Stage 2: out[c] = sum_p partial[p][c]. Block = 32 columns x 32 row slices;
// a slice adds its rows p = y, y+32, ... with four independent accumulators
// (so four loads are in flight per thread), the slices are then added in
// order. Fixed order throughout: bit-reproducible. gridDim.y = dweight / dbias.
template <typename T>
__global__ void __launch_bounds__(1024)
colreduce_kernel(const float* __restrict__ partial, int blocks, int64_t cols, T* out_w, T* out_b,
                 float* out_f32) {
  __shared__ float tile[32][33];
  const int which = blockIdx.y;
  const float* src = partial + (size_t)which * blocks * cols;
  const int64_t col = (int64_t)blockIdx.x * 32 + threadIdx.x;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (col < cols) {
    int p = threadIdx.y;
    for (; p + 96 < blocks; p += 128) {
      s0 += src[(size_t)p * cols + col];
      s1 += src[(size_t)(p + 32) * cols + col];
      s2 += src[(size_t)(p + 64) * cols + col];
      s3 += src[(size_t)(p + 96) * cols + col];
    }
    for (; p < blocks; p += 32) s0 += src[(size_t)p * cols + col];
  }
  tile[threadIdx.y][threadIdx.x] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (threadIdx.y == 0 && col < cols) {
    float t = tile[0][threadIdx.x];
#pragma unroll
    for (int i = 1; i < 32; ++i) t += tile[i][threadIdx.x];
    T* out = which == 0 ? out_w : out_b;
    if (out) out[col] = from_f32<T>(t);
    if (out_f32) out_f32[(size_t)which * cols + col] = t;
  }
}
#endif  // __CUDACC__

// Persistent blocks (= partial rows of the column reduction) the backward
// kernels may launch: SMs x `norm_bwd.blocks_per_sm` (default 2).
inline int max_partial_blocks() {
  int per_sm = tune("norm_bwd.blocks_per_sm");
  if (per_sm <= 0) per_sm = 2;
  return device_info().sm_count * per_sm;
}

}  // namespace evg
