// Pieces of the cross-GPU exchange that more than one source file uses: the
// layout of a rank's buffer, the handle behind evg_exchange and the
// system-scope loads / stores. See exchange.cu for the protocol.
#pragma once

#include "evg_common.cuh"

namespace evg {
namespace xchg {

constexpr int kMaxRanks = 8;
// Blocks of a fused column-reduce + exchange launch (each has its own flags and
// epoch counter): ceil(hidden / 32) x {dweight, dbias}.
constexpr int kMaxBlocks = 2048;

// Layout of a rank's buffer:
//   epoch counter of the one-block kernel, [block] epoch counters of the fused kernel
//   [slot][source rank] areas of (value, epoch) pairs, 8 bytes per value
struct Layout {
  int64_t max_floats;
  __host__ __device__ size_t area_bytes() const { return ((size_t)max_floats * 8 + 255) & ~(size_t)255; }
  __host__ __device__ size_t counter_offset() const { return 0; }
  __host__ __device__ size_t block_counter_offset(int block) const { return 256 + (size_t)block * 4; }
  __host__ __device__ size_t pair_area_offset(int slot, int src) const {
    return block_counter_offset(kMaxBlocks) + 256 + (size_t)(slot * kMaxRanks + src) * area_bytes();
  }
  __host__ __device__ size_t total_bytes() const { return pair_area_offset(2, 0); }
};

struct Peers {
  uint8_t* base[kMaxRanks];
};

#ifdef __CUDACC__
// A value and the epoch it belongs to, as ONE 8-byte access: the reader needs no
// fence and no separate flag, it polls the pair until the epoch is the one it
// waits for (a scalar 64-bit access is single-copy atomic).
__device__ __forceinline__ void st_pair_sys(uint2* p, float value, uint32_t epoch) {
  const unsigned long long w = ((unsigned long long)epoch << 32) | __float_as_uint(value);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_pair_sys(const uint2* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}
#endif  // __CUDACC__

constexpr int kExchangeWaitId = 951;       // the one-block kernel's wait
constexpr int kFusedExchangeWaitId = 952;  // a block of the fused column-reduce kernel

}  // namespace xchg
}  // namespace evg

// The handle behind the C API's opaque evg_exchange.
struct evg_exchange {
  evg::xchg::Layout lay;
  int n_ranks = 0;
  int rank = 0;
  int device = 0;
  bool connected = false;
  void* local = nullptr;                        // cudaMalloc'ed by create
  void* opened[evg::xchg::kMaxRanks] = {};      // cudaIpcOpenMemHandle results (to close)
  evg::xchg::Peers peers{};
  long long wait_limit = 4000000000ll;
};
