// Cross-GPU exchange of the LayerNorm / RMSNorm parameter-gradient partial sums
// (a few thousand float32 per rank and step) over peer memory.
//
// Every rank owns one small buffer in its own device memory that the other ranks
// of the node map through CUDA IPC; it holds, twice (two slots), one area per
// source rank. A step of a rank
//   1. takes the next epoch e from a counter in device memory (so a captured
//      graph that is replayed keeps counting),
//   2. WRITES each of its float32 sums, paired with e in one 64-bit store, into
//      its area of slot e % 2 in every rank's buffer (plain peer stores, no
//      multicast),
//   3. polls, element by element and with a cycle budget, the pairs in its OWN
//      buffer until each source rank's pair carries e: no poll and no data read
//      crosses the link, and there is no fence and no separate flag (a
//      release store at system scope per step cost 10 us more than all the rest),
//   4. adds the values in rank order, so every rank forms the same bits, rounds
//      once to the parameter dtype and writes the result.
// Two slots are enough: a rank overwrites its areas of slot e % 2 at epoch e + 2,
// which it reaches only after it has read every rank's pairs of epoch e + 1, and
// a rank writes e + 1 only after its own reads of epoch e have finished.
// A wait that runs out records EVG_ETIMEOUT in the sticky device status and the
// kernel returns (its results are then undefined); nothing spins without a bound.
// Kernels of different ranks wait on one another, so the ranks must be on
// different GPUs.
// The kernel here handles a whole vector in one block (evg_exchange_sum_round);
// the normalisation backward runs the same protocol inside the second stage of
// its column reduction, block by block (colreduce_exchange_kernel).
#include <cstring>

#include "evg_common.cuh"
#include "exchange.cuh"

namespace evg {
namespace {

using namespace xchg;

constexpr int kExchangeThreads = 1024;

__device__ int g_exchange_status = 0;

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
  for (int64_t i = threadIdx.x; i < count; i += blockDim.x) {
    const float v = partial[i];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < n_ranks)
        st_pair_sys(reinterpret_cast<uint2*>(peers.base[p] + lay.pair_area_offset(slot, rank)) + i, v,
                    epoch);
  }
  const long long start = clock64();
  bool gave_up = false;
  for (int64_t i = threadIdx.x; i < count; i += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < n_ranks; ++r) {
      const uint2* cell = reinterpret_cast<const uint2*>(mine + lay.pair_area_offset(slot, r)) + i;
      uint2 v = ld_pair_sys(cell);
      while (v.y != epoch && !gave_up) {
        if (clock64() - start > wait_limit) {
          atomicCAS(&g_exchange_status, 0, kExchangeWaitId);
          gave_up = true;  // the remaining elements are read as they are
          break;
        }
        v = ld_pair_sys(cell);
      }
      acc += __uint_as_float(v.x);
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
