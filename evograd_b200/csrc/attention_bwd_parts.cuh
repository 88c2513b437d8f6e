// Pieces shared by the causal-attention backward kernels: warp roles, the
// TMEM -> global row store, the delta / log-sum-exp preparation kernel and the
// launch helpers.
#pragma once

#include "attention_common.cuh"

namespace evg {
namespace attn_bwd {

using namespace umma;
using namespace attn;

struct Roles {
  int warp, lane;
  bool is_tma, is_mma, is_compute;
  int quarter;  // TMEM lane quarter this warp may access (warp % 4)
  int half;     // which half of the tile's columns a compute warp handles
  int row;      // row inside the tile owned by a compute thread
};
__device__ __forceinline__ Roles roles() {
  Roles r;
  r.warp = threadIdx.x >> 5;
  r.lane = threadIdx.x & 31;
  r.is_tma = r.warp == 0;
  r.is_mma = r.warp == 1;
  r.is_compute = r.warp >= 2;
  r.quarter = r.warp & 3;
  r.half = r.is_compute ? (r.warp - 2) >> 2 : 0;
  r.row = r.quarter * 32 + r.lane;
  return r;
}

// A warp has finished its TMEM accesses: order them, then one arrival.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// Rows of a [128 x HD] float32 TMEM accumulator -> 16-bit rows of [B*H, S, HD].
// The CG column groups of compute warps take HD / CG columns each.
// heads / token_major: layout of `out` (tensor_row in attention_common.cuh).
template <int HD, int FMT, int CG = 2>
__device__ __forceinline__ void store_rows(uint32_t t_acc, void* out, int bh, int row0, int S,
                                           float scale, const Roles& r, int heads = 1,
                                           int token_major = 0) {
  constexpr int CW = HD / CG;             // columns per warp
  constexpr int PIECE = CW >= 32 ? 32 : 16;  // columns per TMEM read
  const uint32_t lane_base = (uint32_t)(r.quarter * 32) << 16;
  const int row = row0 + r.row;
  const bool ok = row < S;
  uint8_t* dst = reinterpret_cast<uint8_t*>(out) +
                 tensor_row(bh, ok ? row : 0, S, heads, token_major) * HD * 2;
#pragma unroll
  for (int c = 0; c < CW / PIECE; ++c) {
    const int col = r.half * CW + c * PIECE;
    uint32_t acc[PIECE];
    tmem_ld(t_acc + lane_base + col, acc);
    tmem_wait_ld();
    if (ok) {
#pragma unroll
      for (int v = 0; v < PIECE / 8; ++v) {
        uint4 pk;
        pk.x = pack2<FMT>(__uint_as_float(acc[8 * v + 0]) * scale, __uint_as_float(acc[8 * v + 1]) * scale);
        pk.y = pack2<FMT>(__uint_as_float(acc[8 * v + 2]) * scale, __uint_as_float(acc[8 * v + 3]) * scale);
        pk.z = pack2<FMT>(__uint_as_float(acc[8 * v + 4]) * scale, __uint_as_float(acc[8 * v + 5]) * scale);
        pk.w = pack2<FMT>(__uint_as_float(acc[8 * v + 6]) * scale, __uint_as_float(acc[8 * v + 7]) * scale);
        *reinterpret_cast<uint4*>(dst + (col + v * 8) * 2) = pk;
      }
    }
  }
}

// ------------------------------------------------------------------ prepare
// delta = rowsum(dO * O) and the log-sum-exp in log2 units, both written to
// arrays padded to whole 128-row tiles per (batch, head): rows >= S get
// lse2 = +inf (probability 0) and delta = 0. HD/8 threads per row.
template <int HD, int FMT>
__global__ void __launch_bounds__(256)
attn_prepare_kernel(const void* __restrict__ do_ptr, const void* __restrict__ o_ptr,
                    const float* __restrict__ lse, float* __restrict__ lse2_pad,
                    float* __restrict__ delta_pad, int S, int S_pad, int64_t padded_rows, int heads,
                    int o_tm, int do_tm) {
  constexpr int TPR = HD / 8;
  const int64_t prow = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / TPR;
  const int part = threadIdx.x % TPR;
  if (prow >= padded_rows) return;
  const int64_t bh = prow / S_pad;
  const int q = (int)(prow % S_pad);
  const bool ok = q < S;
  float s = 0.f;
  if (ok) {
    const uint4 a = ld_vec(reinterpret_cast<const uint8_t*>(do_ptr) +
                           (tensor_row((int)bh, q, S, heads, do_tm) * HD + part * 8) * 2);
    const uint4 b = ld_vec(reinterpret_cast<const uint8_t*>(o_ptr) +
                           (tensor_row((int)bh, q, S, heads, o_tm) * HD + part * 8) * 2);
    float af[8], bf[8];
    if constexpr (FMT == 1) { unpack<__nv_bfloat16>(a, af); unpack<__nv_bfloat16>(b, bf); }
    else { unpack<__half>(a, af); unpack<__half>(b, bf); }
#pragma unroll
    for (int i = 0; i < 8; ++i) s += af[i] * bf[i];
  }
#pragma unroll
  for (int off = TPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (part == 0) {
    delta_pad[prow] = ok ? s : 0.f;
    lse2_pad[prow] = ok ? lse[bh * S + q] * kLog2e : INFINITY;
  }
}

// ---------------------------------------------------------------- host side
inline long long wait_limit_cycles2() {
  const int t = tune("attention.wait_limit");  // in millions of cycles
  return t > 0 ? (long long)t * 1000000ll : 2000000000ll;
}

template <typename Kernel>
int reserve_smem(Kernel kernel, size_t bytes) {
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) !=
      cudaSuccess) {
    cudaGetLastError();
    return fail(EVG_ELAUNCH, "attention backward: cannot reserve %zu bytes of shared memory", bytes);
  }
  return EVG_OK;
}

// Fused single-pass backward for head size 128 (attention_bwd3.cu). `dq_acc`:
// float32 [B*H, S_pad, 128], zeroed by the launcher.
int launch_bwd3_128(int fmt, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                    const CUtensorMap& mdo, const float* lse2_pad, const float* delta_pad,
                    float* dq_acc, void* dq, void* dk, void* dv, int64_t B, int64_t H, int64_t Hkv,
                    int64_t S, int64_t S_pad, float scale, cudaStream_t stream, Layouts lay);

}  // namespace attn_bwd
}  // namespace evg
