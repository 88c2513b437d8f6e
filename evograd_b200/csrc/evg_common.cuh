// Shared device/host helpers for the evg_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "evg_b200.h"

namespace evg {

// ----------------------------------------------------------------- host side
// Records a message for evg_last_error() on the calling thread; returns `code`.
int fail(int code, const char* fmt, ...);
// Checks cudaGetLastError()/cudaPeekAtLastError after a launch.
int check_launch(const char* what);
// Tunable lookup (0 = not set).
int tune(const char* key);
// Kernels with bounded device-side waits keep a sticky status word per source
// file; each file registers a reader (returns the word, optionally clearing
// it) that evg_device_status() polls after synchronising.
using StatusReader = int (*)(int reset);
void register_device_status(StatusReader reader);
// Cached properties of the current device.
struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int max_smem_optin = 0;
  size_t l2_bytes = 0;
};
const DeviceInfo& device_info();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T> struct DtypeOf;
template <> struct DtypeOf<float> { static constexpr int value = EVG_F32; };
template <> struct DtypeOf<__half> { static constexpr int value = EVG_F16; };
template <> struct DtypeOf<__nv_bfloat16> { static constexpr int value = EVG_BF16; };

inline size_t dtype_size(int dtype) { return dtype == EVG_F32 ? 4 : 2; }

// Calls f.template operator()<T>() with T chosen from the dtype enum.
#define EVG_DISPATCH_DTYPE(dtype, ...)                                   \
  [&]() -> int {                                                         \
    switch (dtype) {                                                     \
      case EVG_F32: { using T = float; return __VA_ARGS__(); }           \
      case EVG_F16: { using T = __half; return __VA_ARGS__(); }          \
      case EVG_BF16: { using T = __nv_bfloat16; return __VA_ARGS__(); }  \
      default: return ::evg::fail(EVG_EDTYPE, "unknown dtype %d", (int)(dtype)); \
    }                                                                    \
  }()

// --------------------------------------------------------------- device side
#ifdef __CUDACC__

template <typename T> struct Vec {
  static constexpr int N = 16 / sizeof(T);  // elements per 128-bit access
};

// 128-bit global accesses. Inputs are read once per kernel, so loads go
// through the non-coherent path without polluting L1.
__device__ __forceinline__ uint4 ld_vec(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_vec(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Unpack one 128-bit vector into floats / pack floats (round-to-nearest-even).
template <typename T> __device__ __forceinline__ void unpack(const uint4& v, float (&f)[Vec<T>::N]);
template <> __device__ __forceinline__ void unpack<float>(const uint4& v, float (&f)[4]) {
  f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  // bf16 -> f32 is a 16-bit shift: exact and cheaper than the cvt path.
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack<__half>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    float2 p = __half22float2(h);
    f[2 * i] = p.x; f[2 * i + 1] = p.y;
  }
}
template <typename T> __device__ __forceinline__ uint4 pack(const float (&f)[Vec<T>::N]);
template <> __device__ __forceinline__ uint4 pack<float>(const float (&f)[4]) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                    __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 pack<__half>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Packed pairs of float32 in one 64-bit register: sm_100 executes add / mul /
// fma on both halves with a single instruction, which halves the issue cost of
// element-wise float32 arithmetic (these kernels are issue-bound on B200).
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 f2_make(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ f32x2 f2_splat(float v) { return f2_make(v, v); }
__device__ __forceinline__ void f2_split(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// Round a float to T and back (a rounding point the reference has).
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return to_f32<T>(from_f32<T>(v));
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

struct SumOp {
  static __device__ __forceinline__ float identity() { return 0.f; }
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
struct MaxOp {
  static __device__ __forceinline__ float identity() { return -INFINITY; }
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
};

// All-reduce of NV values over a group of G threads (G = 32: one warp, shuffles
// only; G > 32: G/32 warps of one block exchange through shared memory and a
// named barrier private to the group). `scratch` points at the group's
// 2*NV*(G/32) floats; `phase` alternates between the two halves so that one
// barrier per reduction is enough. Every thread returns the same value, summed
// in a fixed order (deterministic).
template <int G, int NV, typename Op>
__device__ __forceinline__ void group_allreduce(float (&v)[NV], float* scratch, int& phase,
                                                int group_id, int lane_in_group) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = Op::apply(v[i], __shfl_xor_sync(0xffffffffu, v[i], off));
  }
  if constexpr (G > 32) {
    constexpr int W = G / 32;
    float* buf = scratch + phase * (NV * W);
    if ((lane_in_group & 31) == 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) buf[i * W + (lane_in_group >> 5)] = v[i];
    }
    named_barrier_sync(1 + group_id, G);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float s = buf[i * W];
#pragma unroll
      for (int w = 1; w < W; ++w) s = Op::apply(s, buf[i * W + w]);
      v[i] = s;
    }
    phase ^= 1;
  }
}

// Whole-block all-reduce for the generic (any width) row kernels.
template <int NV, typename Op>
__device__ __forceinline__ void block_allreduce(float (&v)[NV], float* scratch /* [2][NV][32] */,
                                                int& phase) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = Op::apply(v[i], __shfl_xor_sync(0xffffffffu, v[i], off));
  }
  const int warps = (blockDim.x + 31) >> 5;
  float* buf = scratch + phase * (NV * 32);
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) buf[i * 32 + (threadIdx.x >> 5)] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float s = buf[i * 32];
    for (int w = 1; w < warps; ++w) s = Op::apply(s, buf[i * 32 + w]);
    v[i] = s;
  }
  phase ^= 1;
}

// Block all-reduce (sum) for a block of exactly WARPS warps (a multiple of 4):
// like block_allreduce, but the per-warp partials are read back with 128-bit
// shared loads. `scratch` holds [2][NV][WARPS] floats, 16-byte aligned.
template <int NV, int WARPS>
__device__ __forceinline__ void block_allreduce_sum_fixed(float (&v)[NV], float* scratch,
                                                          int& phase) {
  static_assert(WARPS % 4 == 0, "WARPS must be a multiple of 4");
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], off);
  }
  float* buf = scratch + phase * (NV * WARPS);
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) buf[i * WARPS + (threadIdx.x >> 5)] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < WARPS / 4; ++q) {
      const float4 p = *reinterpret_cast<const float4*>(buf + i * WARPS + 4 * q);
      s += (p.x + p.y) + (p.z + p.w);
    }
    v[i] = s;
  }
  phase ^= 1;
}

#endif  // __CUDACC__

}  // namespace evg
