// Cross-GPU exchange of the LayerNorm / RMSNorm parameter-gradient partial sums
// (a few thousand float32 per rank and step) over peer memory.
//
// Every rank owns one small buffer in its own device memory that the other ranks
// of the node map through CUDA IPC. One single-block kernel per rank and step
//   1. takes the next epoch e from a counter in device memory (so a captured
//      graph that is replayed keeps counting),
//   2. copies the rank's float32 partial sums into slot e % 2 of its own buffer
//      and publishes the slot with a release store of e to the slot's flag,
//   3. waits, with a cycle budget, until the flag of slot e % 2 of every other
//      rank reads e (plain peer loads with acquire semantics, no multicast),
//   4. adds the slots of all ranks in rank order, so every rank forms the same
//      bits, rounds once to the parameter dtype and writes the result.
// Two slots are enough: a rank overwrites slot e % 2 at epoch e + 2, which it
// reaches only after it has seen every other rank's flag e + 1, and a rank
// publishes e + 1 only after its own reads of epoch e have finished.
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

// Layout of a rank's buffer: [slot 0 data | slot 1 data | flags | counter].
struct Layout {
  int64_t max_floats;
  __host__ __device__ size_t slot_bytes() const { return ((size_t)max_floats * 4 + 255) & ~(size_t)255; }
  __host__ __device__ size_t flag_offset(int slot) const { return 2 * slot_bytes() + (size_t)slot * 128; }
  __host__ __device__ size_t counter_offset() const { return 2 * slot_bytes() + 256; }
  __host__ __device__ size_t total_bytes() const { return 2 * slot_bytes() + 512; }
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

template <typename T>
__global__ void __launch_bounds__(kExchangeThreads)
exchange_sum_round_kernel(Peers peers, Layout lay, int n_ranks, int rank,
                          const float* __restrict__ partial, int64_t count, T* __restrict__ out,
                          float* __restrict__ out_f32, long long wait_limit) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_abort;
  uint8_t* mine = peers.base[rank];
  if (threadIdx.x == 0) {
    uint32_t* counter = reinterpret_cast<uint32_t*>(mine + lay.counter_offset());
    s_epoch = ++*counter;
    s_abort = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int slot = (int)(epoch & 1u);
  float* my_slot = reinterpret_cast<float*>(mine + (size_t)slot * lay.slot_bytes());
  for (int64_t i = threadIdx.x; i < count; i += blockDim.x) my_slot[i] = partial[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0)
    st_release_sys(reinterpret_cast<uint32_t*>(mine + lay.flag_offset(slot)), epoch);
  if ((int)threadIdx.x < n_ranks && (int)threadIdx.x != rank) {
    const uint32_t* flag =
        reinterpret_cast<const uint32_t*>(peers.base[threadIdx.x] + lay.flag_offset(slot));
    const long long start = clock64();
    while (ld_acquire_sys(flag) != epoch) {
      if (clock64() - start > wait_limit) {
        s_abort = 1;
        atomicCAS(&g_exchange_status, 0, kExchangeWaitId);
        break;
      }
    }
  }
  __syncthreads();
  // After a timeout the sums below read whatever the slots hold; the host learns
  // of it from the status word.
  for (int64_t i = threadIdx.x; i < count; i += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < n_ranks; ++r) {
      const float* src =
          reinterpret_cast<const float*>(peers.base[r] + (size_t)slot * lay.slot_bytes());
      // volatile: the values were written by another GPU after this kernel started
      acc += *reinterpret_cast<const volatile float*>(src + i);
    }
    if (out) out[i] = from_f32<T>(acc);
    if (out_f32) out_f32[i] = acc;
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
