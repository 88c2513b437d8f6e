// Gated linear units (SwiGLU, tanh-GeGLU) forward/backward for sm_100a: pure
// element-wise, HBM-bound. Forward reads a, b and writes c; backward reads dc,
// a, b and writes da, db. Every thread keeps UNROLL independent 128-bit loads
// per tensor in flight.
#include "evg_common.cuh"

namespace evg {
namespace {

constexpr int kUnrollFwd = 4;  // two input streams
constexpr int kUnrollBwd = 2;  // three input streams
constexpr int kThreads = 256;

// Gate activations: value and derivative in float32.
struct Silu {  // ops/level1/swiglu/forward_ref.py:9
  // (The reciprocal is the fast one, two ulp: an IEEE division costs the forward an
  // eighth of its time, and the result is rounded to 16 bits or compared at 1e-5.)
  template <bool FAST = false>
  __device__ static __forceinline__ float value(float a) {
    return a * __fdividef(1.0f, 1.0f + __expf(-a));
  }
  template <bool FAST = false>
  __device__ static __forceinline__ void both(float a, float& val, float& der) {
    const float sg = __fdividef(1.0f, 1.0f + __expf(-a));
    val = a * sg;
    der = sg * (1.0f + a * (1.0f - sg));
  }
};
struct GeluTanh {  // ops/level1/geglu/forward_ref.py:9, gelu(approximate="tanh")
  static constexpr float kBeta = 0.7978845608028654f;  // sqrt(2/pi)
  static constexpr float kKappa = 0.044715f;
  // tanh(u) = 1 - 2/(1 + e^{2u}); the absolute error (~1e-7) is what counts
  // because the result is used as 1 + tanh(u). Saturates cleanly at +-1.
  // FAST (16-bit tensors): one tanh.approx on the special-function unit instead of an
  // exponential and a reciprocal; its absolute error of 5e-4 in 1 + tanh(u) is a
  // quarter of a bf16 half-ulp.
  template <bool FAST>
  __device__ static __forceinline__ float tanh_f32(float u) {
    if constexpr (FAST) {
      float t;
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
      return t;
    } else {
      return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
    }
  }
  template <bool FAST = false>
  __device__ static __forceinline__ float value(float a) {
    const float inner = kBeta * fmaf(kKappa * a * a, a, a);
    return 0.5f * a * (1.0f + tanh_f32<FAST>(inner));
  }
  template <bool FAST = false>
  __device__ static __forceinline__ void both(float a, float& val, float& der) {
    const float a2 = a * a;
    const float inner = kBeta * fmaf(kKappa * a2, a, a);
    const float t = tanh_f32<FAST>(inner);
    const float right = 1.0f + t;
    val = 0.5f * a * right;
    const float inner_der = kBeta * fmaf(3.0f * kKappa, a2, 1.0f);
    der = fmaf(0.5f * a * (1.0f - t * t), inner_der, 0.5f * right);
  }
};

// c = T(act(float(a))) * b with the product rounded in T: the two rounding
// points of the trusted forwards. The product of two 16-bit floats is exact in
// float32, so rounding it once equals the reference's multiply in T.
template <typename T, typename ACT>
__device__ __forceinline__ float glu_fwd_elem(float a, float b) {
  return __fmul_rn(round_to<T>(ACT::template value<(sizeof(T) == 2)>(a)), b);
}

// Gradients as autograd produces them for that forward: the multiply node
// hands dc*b and dc*act(a) back in T, the activation node works in float32.
template <typename T, typename ACT>
__device__ __forceinline__ void glu_bwd_elem(float dc, float a, float b, float& da, float& db) {
  float val, der;
  ACT::template both<(sizeof(T) == 2)>(a, val, der);
  db = __fmul_rn(dc, round_to<T>(val));
  da = round_to<T>(__fmul_rn(dc, b)) * der;
}

template <typename T, typename ACT>
__global__ void __launch_bounds__(kThreads)
glu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
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
        for (int j = 0; j < N; ++j) o[j] = glu_fwd_elem<T, ACT>(af[j], bf[j]);
        st_vec(c + v * N, pack<T>(o));
      }
    }
  }
}

template <typename T, typename ACT>
__global__ void __launch_bounds__(kThreads)
glu_bwd_kernel(const T* dc, const T* a, const T* b, T* da, T* db, int64_t nvec) {
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
        for (int j = 0; j < N; ++j) glu_bwd_elem<T, ACT>(cf[j], af[j], bf[j], oa[j], ob[j]);
        st_vec(da + v * N, pack<T>(oa));
        st_vec(db + v * N, pack<T>(ob));
      }
    }
  }
}

// Tail / unaligned elements.
template <typename T, typename ACT>
__global__ void glu_fwd_scalar_kernel(const T* a, const T* b, T* c, int64_t begin, int64_t n) {
  for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    c[i] = from_f32<T>(glu_fwd_elem<T, ACT>(to_f32<T>(a[i]), to_f32<T>(b[i])));
}
template <typename T, typename ACT>
__global__ void glu_bwd_scalar_kernel(const T* dc, const T* a, const T* b, T* da, T* db,
                                         int64_t begin, int64_t n) {
  for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float oa, ob;
    glu_bwd_elem<T, ACT>(to_f32<T>(dc[i]), to_f32<T>(a[i]), to_f32<T>(b[i]), oa, ob);
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

template <typename ACT>
int launch_glu_fwd(const char* op, const void* a, const void* b, void* c, int64_t n, int dtype,
                   void* stream) {
  if (!a || !b || !c) return fail(EVG_ENULL, "%s: null pointer argument", op);
  if (n < 0) return fail(EVG_EBADSHAPE, "%s: n=%lld", op, (long long)n);
  if (n == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    constexpr int N = Vec<T>::N;
    cudaStream_t st = (cudaStream_t)stream;
    int per_sm = tune("swiglu.blocks_per_sm");
    if (per_sm <= 0) per_sm = 32;
    const bool vec_ok = aligned16(a) && aligned16(b) && aligned16(c);
    const int64_t nvec = vec_ok ? n / N : 0;
    if (nvec > 0) {
      glu_fwd_kernel<T, ACT>
          <<<flat_grid((nvec + kUnrollFwd - 1) / kUnrollFwd, per_sm), kThreads, 0, st>>>(
              (const T*)a, (const T*)b, (T*)c, nvec);
    }
    if (nvec * N < n) {
      glu_fwd_scalar_kernel<T, ACT><<<flat_grid(n - nvec * N, per_sm), kThreads, 0, st>>>(
          (const T*)a, (const T*)b, (T*)c, nvec * N, n);
    }
    return check_launch(op);
  });
}

template <typename ACT>
int launch_glu_bwd(const char* op, const void* dc, const void* a, const void* b, void* da,
                   void* db, int64_t n, int dtype, void* stream) {
  if (!dc || !a || !b || !da || !db) return fail(EVG_ENULL, "%s: null pointer argument", op);
  if (n < 0) return fail(EVG_EBADSHAPE, "%s: n=%lld", op, (long long)n);
  if (n == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    constexpr int N = Vec<T>::N;
    cudaStream_t st = (cudaStream_t)stream;
    int per_sm = tune("swiglu.blocks_per_sm");
    if (per_sm <= 0) per_sm = 32;
    const bool vec_ok =
        aligned16(dc) && aligned16(a) && aligned16(b) && aligned16(da) && aligned16(db);
    const int64_t nvec = vec_ok ? n / N : 0;
    if (nvec > 0) {
      glu_bwd_kernel<T, ACT>
          <<<flat_grid((nvec + kUnrollBwd - 1) / kUnrollBwd, per_sm), kThreads, 0, st>>>(
              (const T*)dc, (const T*)a, (const T*)b, (T*)da, (T*)db, nvec);
    }
    if (nvec * N < n) {
      glu_bwd_scalar_kernel<T, ACT><<<flat_grid(n - nvec * N, per_sm), kThreads, 0, st>>>(
          (const T*)dc, (const T*)a, (const T*)b, (T*)da, (T*)db, nvec * N, n);
    }
    return check_launch(op);
  });
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_swiglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype,
                              void* stream) {
  return launch_glu_fwd<Silu>("swiglu_fwd", a, b, c, n, dtype, stream);
}
extern "C" int evg_swiglu_bwd(const void* dc, const void* a, const void* b, void* da, void* db,
                              int64_t n, int dtype, void* stream) {
  return launch_glu_bwd<Silu>("swiglu_bwd", dc, a, b, da, db, n, dtype, stream);
}
extern "C" int evg_geglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype,
                             void* stream) {
  return launch_glu_fwd<GeluTanh>("geglu_fwd", a, b, c, n, dtype, stream);
}
extern "C" int evg_geglu_bwd(const void* dc, const void* a, const void* b, void* da, void* db,
                             int64_t n, int dtype, void* stream) {
  return launch_glu_bwd<GeluTanh>("geglu_bwd", dc, a, b, da, db, n, dtype, stream);
}
