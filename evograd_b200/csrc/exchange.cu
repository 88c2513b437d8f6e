// Cross-GPU exchange of the LayerNorm / RMSNorm parameter-gradient partial sums
// (a few thousand float32 per rank and step) over peer memory.
//
// Every rank owns one small buffer in its own device memory that the other ranks
// of the node map through CUDA IPC; it holds, twice (two slots), one area per
// source rank. One single-block kernel per rank and step
//   1. takes the next epoch e from a counter in device memory (so a captured
//      graph that is replayed keeps counting),
//   2. WRITES the rank's float32 partial sums into its area of slot e % 2 in
//      every rank's buffer (plain peer stores, no multicast) and then publishes
//      them with one release store of e per destination,
//   3. waits, with a cycle budget, until all of its OWN flags of slot e % 2 read
//      e: it polls local memory, so no poll and no data read crosses the link,
//   4. adds the areas of all ranks in rank order, so every rank forms the same
//      bits, rounds once to the parameter dtype and writes the result.
// Two slots are enough: rank r overwrites its area of slot e % 2 in rank p's
// buffer at epoch e + 2, which r reaches only after it has seen p's flag e + 1,
// and p sends e + 1 only after its own reads of epoch e have finished.
// A wait that runs out records EVG_ETIMEOUT in the sticky device status and the
// kernel returns (its results are then undefined); nothing spins without a bound.
// Kernels of different ranks wait on one another, so the ranks must be on
// different GPUs.
#include <cstring>

#include "evg_common.cuh"

namespace evg {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kExchangeThreads = 1024;
constexpr int kExchangeWaitId = 951;

__device__ int g_exchange_status = 0;

// Layout of a rank's buffer: [slot][source rank] data areas, then
// [slot][source rank] flags (one 128-byte line each), then the epoch counter.
struct Layout {
  int64_t max_floats;
  __host__ __device__ size_t area_bytes() const { return ((size_t)max_floats * 4 + 255) & ~(size_t)255; }
  __host__ __device__ size_t area_offset(int slot, int src) const {
    return (size_t)(slot * kMaxRanks + src) * area_bytes();
  }
  __host__ __device__ size_t flag_offset(int slot, int src) const {
    return 2 * kMaxRanks * area_bytes() + (size_t)(slot * kMaxRanks + src) * 128;
  }
  __host__ __device__ size_t counter_offset() const {
    return 2 * kMaxRanks * area_bytes() + 2 * kMaxRanks * 128;
  }
  __host__ __device__ size_t total_bytes() const { return counter_offset() + 256; }
};

struct Peers {
  uint8_t* base[kMaxRanks];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_relaxed_sys_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__device__ __forceinline__ void write_sum(T* out, float* out_f32, int64_t i, float v) {
  if (out) out[i] = from_f32<T>(v);
  if (out_f32) out_f32[i] = v;
}

template <typename T>
__global__ void __launch_bounds__(kExchangeThreads)
exchange_sum_round_kernel(Peers peers, Layout lay, int n_ranks, int rank,
                          const float* __restrict__ partial, int64_t count, T* __restrict__ out,
                          float* __restrict__ out_f32, long long wait_limit) {
  __shared__ uint32_t s_epoch;
  uint8_t* mine = peers.base[rank];
  if (threadIdx.x == 0) {
    uint32_t* counter = reinterpret_cast<uint32_t*>(mine + lay.counter_offset());
    s_epoch = ++*counter;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int slot = (int)(epoch & 1u);
  const bool vec = (count & 3) == 0 && (reinterpret_cast<uintptr_t>(partial) & 15u) == 0;
  // 2. this rank's values into its area in every rank's buffer (its own included)
  if (vec) {
    for (int64_t j = threadIdx.x; j < count / 4; j += blockDim.x) {
      const float4 v = reinterpret_cast<const float4*>(partial)[j];
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < n_ranks)
          reinterpret_cast<float4*>(peers.base[p] + lay.area_offset(slot, rank))[j] = v;
    }
  } else {
    for (int64_t i = threadIdx.x; i < count; i += blockDim.x) {
      const float v = partial[i];
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < n_ranks)
          reinterpret_cast<float*>(peers.base[p] + lay.area_offset(slot, rank))[i] = v;
    }
  }
  __syncthreads();
  // One release store at system scope per destination publishes the values: the
  // block barrier orders every thread's writes before it (a system-wide fence in
  // every thread costs tens of microseconds).
  if ((int)threadIdx.x < n_ranks)
    st_release_sys(
        reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + lay.flag_offset(slot, rank)), epoch);
  // 3. wait for every source rank's flag in this rank's own buffer
  if ((int)threadIdx.x < n_ranks) {
    const uint32_t* flag =
        reinterpret_cast<const uint32_t*>(mine + lay.flag_offset(slot, threadIdx.x));
    const long long start = clock64();
    while (ld_acquire_sys(flag) != epoch) {
      if (clock64() - start > wait_limit) {
        atomicCAS(&g_exchange_status, 0, kExchangeWaitId);
        break;
      }
    }
  }
  __syncthreads();
  // 4. After a timeout the sums below read whatever the areas hold; the host learns
  // of it from the status word. The sum runs over the ranks in rank order on
  // every rank.
  if (vec) {
    for (int64_t j = threadIdx.x; j < count / 4; j += blockDim.x) {
      float4 v[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < n_ranks)
          v[r] = ld_relaxed_sys_f32x4(
              reinterpret_cast<const float*>(mine + lay.area_offset(slot, r)) + 4 * j);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < n_ranks) {
          acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
        }
      write_sum<T>(out, out_f32, 4 * j + 0, acc.x);
      write_sum<T>(out, out_f32, 4 * j + 1, acc.y);
      write_sum<T>(out, out_f32, 4 * j + 2, acc.z);
      write_sum<T>(out, out_f32, 4 * j + 3, acc.w);
    }
  } else {
    for (int64_t i = threadIdx.x; i < count; i += blockDim.x) {
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < n_ranks)
          acc += ld_relaxed_sys_f32(reinterpret_cast<const float*>(mine + lay.area_offset(slot, r)) + i);
      write_sum<T>(out, out_f32, i, acc);
    }
  }
}

int read_exchange_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_exchange_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_exchange_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_exchange_registered = (register_device_status(read_exchange_status), true);

}  // namespace
}  // namespace evg

using namespace evg;

struct evg_exchange {
  Layout lay;
  int n_ranks = 0;
  int rank = 0;
  int device = 0;
  bool connected = false;
  void* local = nullptr;             // cudaMalloc'ed by create
  void* opened[kMaxRanks] = {};      // cudaIpcOpenMemHandle results (to close)
  Peers peers{};
  long long wait_limit = 4000000000ll;
};

extern "C" int evg_exchange_create(int64_t max_floats, int n_ranks, int rank, evg_exchange** out,
                                   unsigned char* ipc_handle) {
  if (!out || !ipc_handle) return fail(EVG_ENULL, "exchange_create: null pointer argument");
  if (max_floats <= 0 || max_floats > (1 << 24))
    return fail(EVG_EBADSHAPE, "exchange_create: max_floats=%lld (1 .. 2^24)", (long long)max_floats);
  if (n_ranks < 1 || n_ranks > kMaxRanks || rank < 0 || rank >= n_ranks)
    return fail(EVG_EBADSHAPE, "exchange_create: rank %d of %d (at most %d ranks)", rank, n_ranks,
                kMaxRanks);
  evg_exchange* x = new evg_exchange();
  x->lay.max_floats = max_floats;
  x->n_ranks = n_ranks;
  x->rank = rank;
  cudaError_t err = cudaGetDevice(&x->device);
  if (err == cudaSuccess) err = cudaMalloc(&x->local, x->lay.total_bytes());
  if (err == cudaSuccess) err = cudaMemset(x->local, 0, x->lay.total_bytes());
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, x->local);
  if (err != cudaSuccess) {
    cudaGetLastError();
    if (x->local) cudaFree(x->local);
    delete x;
    return fail(EVG_ELAUNCH, "exchange_create: %s", cudaGetErrorString(err));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  std::memcpy(ipc_handle, &h, 64);
  x->peers.base[rank] = static_cast<uint8_t*>(x->local);
  if (n_ranks == 1) x->connected = true;
  *out = x;
  return EVG_OK;
}

extern "C" int evg_exchange_connect(evg_exchange* x, const unsigned char* all_handles) {
  if (!x || !all_handles) return fail(EVG_ENULL, "exchange_connect: null pointer argument");
  if (x->connected) return EVG_OK;
  for (int r = 0; r < x->n_ranks; ++r) {
    if (r == x->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, all_handles + (size_t)r * 64, 64);
    void* p = nullptr;
    const cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess || !p) {
      cudaGetLastError();
      return fail(EVG_ELAUNCH, "exchange_connect: cannot map rank %d's buffer: %s", r,
                  cudaGetErrorString(err));
    }
    x->opened[r] = p;
    x->peers.base[r] = static_cast<uint8_t*>(p);
  }
  x->connected = true;
  return EVG_OK;
}

extern "C" int evg_exchange_connect_local(evg_exchange* x, void* const* peer_buffers) {
  if (!x || !peer_buffers) return fail(EVG_ENULL, "exchange_connect_local: null pointer argument");
  for (int r = 0; r < x->n_ranks; ++r)
    if (r != x->rank) x->peers.base[r] = static_cast<uint8_t*>(peer_buffers[r]);
  x->connected = true;
  return EVG_OK;
}

extern "C" void* evg_exchange_buffer(evg_exchange* x) { return x ? x->local : nullptr; }

extern "C" int evg_exchange_set_wait_limit(evg_exchange* x, int64_t cycles) {
  if (!x) return fail(EVG_ENULL, "exchange_set_wait_limit: null handle");
  if (cycles <= 0 || cycles > 4000000000ll)
    return fail(EVG_EBADSHAPE, "exchange_set_wait_limit: cycles must be in (0, 4e9]");
  x->wait_limit = cycles;
  return EVG_OK;
}

extern "C" int evg_exchange_sum_round(evg_exchange* x, const float* partial, int64_t count,
                                      void* out, int dtype, float* out_f32, void* stream) {
  if (!x || !partial) return fail(EVG_ENULL, "exchange_sum_round: null pointer argument");
  if (!x->connected) return fail(EVG_EUNSUPPORTED, "exchange_sum_round: peers are not connected");
  if (count <= 0 || count > x->lay.max_floats)
    return fail(EVG_EBADSHAPE, "exchange_sum_round: count=%lld (1 .. %lld)", (long long)count,
                (long long)x->lay.max_floats);
  if (!out && !out_f32) return fail(EVG_ENULL, "exchange_sum_round: no output requested");
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    exchange_sum_round_kernel<T><<<1, kExchangeThreads, 0, (cudaStream_t)stream>>>(
        x->peers, x->lay, x->n_ranks, x->rank, partial, count, (T*)out, out_f32, x->wait_limit);
    return check_launch("exchange_sum_round");
  });
}

extern "C" int evg_exchange_destroy(evg_exchange* x) {
  if (!x) return EVG_OK;
  for (int r = 0; r < kMaxRanks; ++r)
    if (x->opened[r]) cudaIpcCloseMemHandle(x->opened[r]);
  if (x->local) cudaFree(x->local);
  cudaGetLastError();
  delete x;
  return EVG_OK;
}
