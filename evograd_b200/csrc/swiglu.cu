// SwiGLU forward/backward for sm_100a: pure element-wise, HBM-bound. Forward
// reads a, b and writes c; backward reads dc, a, b and writes da, db. Every
// thread keeps UNROLL independent 128-bit loads per tensor in flight.
#include "evg_common.cuh"

namespace evg {
namespace {

constexpr int kUnrollFwd = 4;  // two input streams
constexpr int kUnrollBwd = 2;  // three input streams
constexpr int kThreads = 256;

__device__ __forceinline__ float sigmoid_f32(float a) { return 1.0f / (1.0f + __expf(-a)); }

// c = T(silu(float(a))) * b with the product rounded in T: the two rounding
// points of swiglu_forward_ref (ops/level1/swiglu/forward_ref.py:9). The
// product of two 16-bit floats is exact in float32, so rounding it once equals
// the reference's multiply in T.
template <typename T>
__device__ __forceinline__ float swiglu_fwd_elem(float a, float b) {
  const float s = round_to<T>(a * sigmoid_f32(a));
  return __fmul_rn(s, b);
}

// Gradients as autograd produces them for that forward: the multiply node
// hands dc*b and dc*silu(a) back in T, the silu node works in float32.
template <typename T>
__device__ __forceinline__ void swiglu_bwd_elem(float dc, float a, float b, float& da, float& db) {
  const float sg = sigmoid_f32(a);
  const float silu_t = round_to<T>(a * sg);
  db = __fmul_rn(dc, silu_t);
  const float dsilu = round_to<T>(__fmul_rn(dc, b));
  da = dsilu * (sg * (1.0f + a * (1.0f - sg)));
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
                  int64_t nvec) {
  constexpr int N = Vec<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec;
       base += stride * kUnrollFwd) {
    uint4 av[kUnrollFwd], bv[kUnrollFwd];
#pragma unroll
    for (int u = 0; u < kUnrollFwd; ++u) {
      const int64_t v = base + u * stride;
      if (v < nvec) {
        av[u] = ld_vec(a + v * N);
        bv[u] = ld_vec(b + v * N);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnrollFwd; ++u) {
      const int64_t v = base + u * stride;
      if (v < nvec) {
        float af[N], bf[N], o[N];
        unpack<T>(av[u], af);
        unpack<T>(bv[u], bf);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = swiglu_fwd_elem<T>(af[j], bf[j]);
        st_vec(c + v * N, pack<T>(o));
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_bwd_kernel(const T* dc, const T* a, const T* b, T* da, T* db, int64_t nvec) {
  constexpr int N = Vec<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec;
       base += stride * kUnrollBwd) {
    uint4 cv[kUnrollBwd], av[kUnrollBwd], bv[kUnrollBwd];
#pragma unroll
    for (int u = 0; u < kUnrollBwd; ++u) {
      const int64_t v = base + u * stride;
      if (v < nvec) {
        cv[u] = ld_vec(dc + v * N);
        // a and b may be overwritten by da and db through aliases, so they are
        // read with plain (coherent) loads, and strictly before the stores below.
        av[u] = *reinterpret_cast<const uint4*>(a + v * N);
        bv[u] = *reinterpret_cast<const uint4*>(b + v * N);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnrollBwd; ++u) {
      const int64_t v = base + u * stride;
      if (v < nvec) {
        float cf[N], af[N], bf[N], oa[N], ob[N];
        unpack<T>(cv[u], cf);
        unpack<T>(av[u], af);
        unpack<T>(bv[u], bf);
#pragma unroll
        for (int j = 0; j < N; ++j) swiglu_bwd_elem<T>(cf[j], af[j], bf[j], oa[j], ob[j]);
        st_vec(da + v * N, pack<T>(oa));
        st_vec(db + v * N, pack<T>(ob));
      }
    }
  }
}

// Tail / unaligned elements.
template <typename T>
__global__ void swiglu_fwd_scalar_kernel(const T* a, const T* b, T* c, int64_t begin, int64_t n) {
  for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    c[i] = from_f32<T>(swiglu_fwd_elem<T>(to_f32<T>(a[i]), to_f32<T>(b[i])));
}
template <typename T>
__global__ void swiglu_bwd_scalar_kernel(const T* dc, const T* a, const T* b, T* da, T* db,
                                         int64_t begin, int64_t n) {
  for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float oa, ob;
    swiglu_bwd_elem<T>(to_f32<T>(dc[i]), to_f32<T>(a[i]), to_f32<T>(b[i]), oa, ob);
    da[i] = from_f32<T>(oa);
    db[i] = from_f32<T>(ob);
  }
}

int flat_grid(int64_t work_items, int per_sm) {
  int64_t blocks = (work_items + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)device_info().sm_count * per_sm;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_swiglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype,
                              void* stream) {
  if (!a || !b || !c) return fail(EVG_ENULL, "swiglu_fwd: null pointer argument");
  if (n < 0) return fail(EVG_EBADSHAPE, "swiglu_fwd: n=%lld", (long long)n);
  if (n == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    constexpr int N = Vec<T>::N;
    cudaStream_t st = (cudaStream_t)stream;
    int per_sm = tune("swiglu.blocks_per_sm");
    if (per_sm <= 0) per_sm = 32;
    const bool vec_ok = aligned16(a) && aligned16(b) && aligned16(c);
    const int64_t nvec = vec_ok ? n / N : 0;
    if (nvec > 0) {
      swiglu_fwd_kernel<T><<<flat_grid((nvec + kUnrollFwd - 1) / kUnrollFwd, per_sm), kThreads, 0, st>>>(
          (const T*)a, (const T*)b, (T*)c, nvec);
    }
    if (nvec * N < n) {
      swiglu_fwd_scalar_kernel<T><<<flat_grid(n - nvec * N, per_sm), kThreads, 0, st>>>(
          (const T*)a, (const T*)b, (T*)c, nvec * N, n);
    }
    return check_launch("swiglu_fwd");
  });
}

extern "C" int evg_swiglu_bwd(const void* dc, const void* a, const void* b, void* da, void* db,
                              int64_t n, int dtype, void* stream) {
  if (!dc || !a || !b || !da || !db) return fail(EVG_ENULL, "swiglu_bwd: null pointer argument");
  if (n < 0) return fail(EVG_EBADSHAPE, "swiglu_bwd: n=%lld", (long long)n);
  if (n == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    constexpr int N = Vec<T>::N;
    cudaStream_t st = (cudaStream_t)stream;
    int per_sm = tune("swiglu.blocks_per_sm");
    if (per_sm <= 0) per_sm = 32;
    const bool vec_ok = aligned16(dc) && aligned16(a) && aligned16(b) && aligned16(da) && aligned16(db);
    const int64_t nvec = vec_ok ? n / N : 0;
    if (nvec > 0) {
      swiglu_bwd_kernel<T><<<flat_grid((nvec + kUnrollBwd - 1) / kUnrollBwd, per_sm), kThreads, 0, st>>>(
          (const T*)dc, (const T*)a, (const T*)b, (T*)da, (T*)db, nvec);
    }
    if (nvec * N < n) {
      swiglu_bwd_scalar_kernel<T><<<flat_grid(n - nvec * N, per_sm), kThreads, 0, st>>>(
          (const T*)dc, (const T*)a, (const T*)b, (T*)da, (T*)db, nvec * N, n);
    }
    return check_launch("swiglu_bwd");
  });
}
