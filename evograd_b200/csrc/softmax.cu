// Row softmax forward/backward for sm_100a. HBM-bound: forward reads x and
// writes y; backward reads y and dy and writes dx. The only saved state is y.
#include "rowcfg.cuh"
#include "softmax_wide.cuh"

namespace evg {
namespace {

constexpr float kLog2e = 1.4426950408889634f;

template <typename T, int G, int VPT>
__global__ void __launch_bounds__(rowcfg_max_threads(G))
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols) {
  constexpr int N = Vec<T>::N;
  extern __shared__ float smem[];
  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int groups = blockDim.x / G;
  const int nvec = cols / N;
  float* scratch = smem + gid * (2 * (G / 32));
  int phase = 0;
  for (int64_t row = (int64_t)blockIdx.x * groups + gid; row < rows;
       row += (int64_t)gridDim.x * groups) {
    const T* xr = x + row * cols;
    float f[VPT][N];
    float m[1] = {-INFINITY};
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      if (idx < nvec) {
        unpack<T>(ld_vec(xr + (size_t)idx * N), f[k]);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) f[k][j] = -INFINITY;
      }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
      for (int j = 0; j < N; ++j) m[0] = fmaxf(m[0], f[k][j]);
    group_allreduce<G, 1, MaxOp>(m, scratch, phase, gid, lig);
    // exp(x - max) as 2^((x - max) * log2(e)); padded lanes give 2^-inf = 0.
    float s[1] = {0.f};
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
      for (int j = 0; j < N; ++j) {
        f[k][j] = exp2f((f[k][j] - m[0]) * kLog2e);
        s[0] += f[k][j];
      }
    group_allreduce<G, 1, SumOp>(s, scratch, phase, gid, lig);
    const float inv = 1.0f / s[0];
    T* yr = y + row * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      if (idx < nvec) {
#pragma unroll
        for (int j = 0; j < N; ++j) f[k][j] *= inv;
        st_vec(yr + (size_t)idx * N, pack<T>(f[k]));
      }
    }
  }
}

template <typename T, int G, int VPT>
__global__ void __launch_bounds__(rowcfg_max_threads(G))
softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                   int64_t rows, int cols) {
  constexpr int N = Vec<T>::N;
  extern __shared__ float smem[];
  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int groups = blockDim.x / G;
  const int nvec = cols / N;
  float* scratch = smem + gid * (2 * (G / 32));
  int phase = 0;
  for (int64_t row = (int64_t)blockIdx.x * groups + gid; row < rows;
       row += (int64_t)gridDim.x * groups) {
    const T* yr = y + row * cols;
    const T* gr = dy + row * cols;
    uint4 yv[VPT], gv[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      yv[k] = make_uint4(0, 0, 0, 0);
      gv[k] = make_uint4(0, 0, 0, 0);
      if (idx < nvec) {
        yv[k] = ld_vec(yr + (size_t)idx * N);
        gv[k] = ld_vec(gr + (size_t)idx * N);
      }
    }
    float d[1] = {0.f};
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      float yf[N], gf[N];
      unpack<T>(yv[k], yf);
      unpack<T>(gv[k], gf);
#pragma unroll
      for (int j = 0; j < N; ++j) d[0] += gf[j] * yf[j];
    }
    group_allreduce<G, 1, SumOp>(d, scratch, phase, gid, lig);
    T* dr = dx + row * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      if (idx < nvec) {
        float yf[N], gf[N], o[N];
        unpack<T>(yv[k], yf);
        unpack<T>(gv[k], gf);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = (gf[j] - d[0]) * yf[j];
        st_vec(dr + (size_t)idx * N, pack<T>(o));
      }
    }
  }
}

// Rows of any width or alignment (rows too wide for registers that the cluster
// kernels of softmax_wide.cu do not take either): one block per row, three
// passes (maximum, sum of exponentials, output); passes two and three re-read
// the row from L2.
// VEC selects 128-bit accesses when the row width and pointers allow them.
template <typename T, bool VEC>
__global__ void __launch_bounds__(1024, 1)
softmax_fwd_generic_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows,
                           int64_t cols) {
  constexpr int N = Vec<T>::N;
  __shared__ float scratch[2 * 32];
  int phase = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float m[1] = {-INFINITY};
    if constexpr (VEC) {
      for (int64_t v = threadIdx.x; v < cols / N; v += blockDim.x) {
        float f[N];
        unpack<T>(*reinterpret_cast<const uint4*>(xr + v * N), f);
#pragma unroll
        for (int j = 0; j < N; ++j) m[0] = fmaxf(m[0], f[j]);
      }
    } else {
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) m[0] = fmaxf(m[0], to_f32<T>(xr[c]));
    }
    block_allreduce<1, MaxOp>(m, scratch, phase);
    float s[1] = {0.f};
    if constexpr (VEC) {
      for (int64_t v = threadIdx.x; v < cols / N; v += blockDim.x) {
        float f[N];
        unpack<T>(*reinterpret_cast<const uint4*>(xr + v * N), f);
#pragma unroll
        for (int j = 0; j < N; ++j) s[0] += exp2f((f[j] - m[0]) * kLog2e);
      }
    } else {
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
        s[0] += exp2f((to_f32<T>(xr[c]) - m[0]) * kLog2e);
    }
    block_allreduce<1, SumOp>(s, scratch, phase);
    const float inv = 1.0f / s[0];
    T* yr = y + row * cols;
    if constexpr (VEC) {
      for (int64_t v = threadIdx.x; v < cols / N; v += blockDim.x) {
        float f[N];
        unpack<T>(*reinterpret_cast<const uint4*>(xr + v * N), f);
#pragma unroll
        for (int j = 0; j < N; ++j) f[j] = exp2f((f[j] - m[0]) * kLog2e) * inv;
        st_vec(yr + v * N, pack<T>(f));
      }
    } else {
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
        yr[c] = from_f32<T>(exp2f((to_f32<T>(xr[c]) - m[0]) * kLog2e) * inv);
    }
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(1024, 1)
softmax_bwd_generic_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                           int64_t rows, int64_t cols) {
  constexpr int N = Vec<T>::N;
  __shared__ float scratch[2 * 32];
  int phase = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* yr = y + row * cols;
    const T* gr = dy + row * cols;
    float d[1] = {0.f};
    if constexpr (VEC) {
      for (int64_t v = threadIdx.x; v < cols / N; v += blockDim.x) {
        float yf[N], gf[N];
        unpack<T>(*reinterpret_cast<const uint4*>(yr + v * N), yf);
        unpack<T>(*reinterpret_cast<const uint4*>(gr + v * N), gf);
#pragma unroll
        for (int j = 0; j < N; ++j) d[0] += gf[j] * yf[j];
      }
    } else {
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
        d[0] += to_f32<T>(gr[c]) * to_f32<T>(yr[c]);
    }
    block_allreduce<1, SumOp>(d, scratch, phase);
    T* dr = dx + row * cols;
    if constexpr (VEC) {
      for (int64_t v = threadIdx.x; v < cols / N; v += blockDim.x) {
        float yf[N], gf[N], o[N];
        unpack<T>(*reinterpret_cast<const uint4*>(yr + v * N), yf);
        unpack<T>(*reinterpret_cast<const uint4*>(gr + v * N), gf);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = (gf[j] - d[0]) * yf[j];
        st_vec(dr + v * N, pack<T>(o));
      }
    } else {
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
        dr[c] = from_f32<T>((to_f32<T>(gr[c]) - d[0]) * to_f32<T>(yr[c]));
    }
  }
}

template <typename T>
int launch_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  const bool vec_ok = cols % N == 0 && aligned16(x) && aligned16(y);
  RowCfg cfg;
  if (vec_ok && !tune("rows.force_generic") && pick_rowcfg("softmax_fwd", cols / N, cfg)) {
    const int groups = cfg.threads / cfg.G;
    const size_t smem = (size_t)groups * 2 * (cfg.G / 32) * sizeof(float);
#define EVG_X(g, v)                                                                          \
  if (cfg.G == g && cfg.VPT == v) {                                                          \
    auto kern = softmax_fwd_kernel<T, g, v>;                                                 \
    const int grid = persistent_grid(kern, cfg.threads, smem, rows, groups);                 \
    kern<<<grid, cfg.threads, smem, stream>>>((const T*)x, (T*)y, rows, (int)cols);          \
    return check_launch("softmax_fwd");                                                      \
  }
    EVG_ROWCFG_LIST(EVG_X)
#undef EVG_X
  }
  if (vec_ok && !tune("rows.force_generic")) {  // wider than any register shape
    bool handled = false;
    const int rc = softmax_wide_fwd(DtypeOf<T>::value, x, y, rows, cols, stream, &handled);
    if (rc || handled) return rc;
  }
  const int threads = cols >= 4096 ? 1024 : (cols >= 256 ? 256 : 64);
  if (vec_ok) {
    auto kern = softmax_fwd_generic_kernel<T, true>;
    kern<<<persistent_grid(kern, threads, 0, rows, 1), threads, 0, stream>>>((const T*)x, (T*)y,
                                                                             rows, cols);
  } else {
    auto kern = softmax_fwd_generic_kernel<T, false>;
    kern<<<persistent_grid(kern, threads, 0, rows, 1), threads, 0, stream>>>((const T*)x, (T*)y,
                                                                             rows, cols);
  }
  return check_launch("softmax_fwd");
}

template <typename T>
int launch_softmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t cols,
                       cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  const bool vec_ok = cols % N == 0 && aligned16(y) && aligned16(dy) && aligned16(dx);
  RowCfg cfg;
  if (vec_ok && !tune("rows.force_generic") && pick_rowcfg("softmax_bwd", cols / N, cfg)) {
    const int groups = cfg.threads / cfg.G;
    const size_t smem = (size_t)groups * 2 * (cfg.G / 32) * sizeof(float);
#define EVG_X(g, v)                                                                          \
  if (cfg.G == g && cfg.VPT == v) {                                                          \
    auto kern = softmax_bwd_kernel<T, g, v>;                                                 \
    const int grid = persistent_grid(kern, cfg.threads, smem, rows, groups);                 \
    kern<<<grid, cfg.threads, smem, stream>>>((const T*)y, (const T*)dy, (T*)dx, rows,       \
                                              (int)cols);                                    \
    return check_launch("softmax_bwd");                                                      \
  }
    EVG_ROWCFG_LIST(EVG_X)
#undef EVG_X
  }
  if (vec_ok && !tune("rows.force_generic")) {  // wider than any register shape
    bool handled = false;
    const int rc = softmax_wide_bwd(DtypeOf<T>::value, y, dy, dx, rows, cols, stream, &handled);
    if (rc || handled) return rc;
  }
  const int threads = cols >= 4096 ? 1024 : (cols >= 256 ? 256 : 64);
  if (vec_ok) {
    auto kern = softmax_bwd_generic_kernel<T, true>;
    kern<<<persistent_grid(kern, threads, 0, rows, 1), threads, 0, stream>>>(
        (const T*)y, (const T*)dy, (T*)dx, rows, cols);
  } else {
    auto kern = softmax_bwd_generic_kernel<T, false>;
    kern<<<persistent_grid(kern, threads, 0, rows, 1), threads, 0, stream>>>(
        (const T*)y, (const T*)dy, (T*)dx, rows, cols);
  }
  return check_launch("softmax_bwd");
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, int dtype,
                               void* stream) {
  if (!x || !y) return fail(EVG_ENULL, "softmax_fwd: null pointer argument");
  if (rows < 0 || cols <= 0)
    return fail(EVG_EBADSHAPE, "softmax_fwd: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (rows == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_softmax_fwd<T>(x, y, rows, cols, (cudaStream_t)stream);
  });
}

extern "C" int evg_softmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t cols,
                               int dtype, void* stream) {
  if (!y || !dy || !dx) return fail(EVG_ENULL, "softmax_bwd: null pointer argument");
  if (rows < 0 || cols <= 0)
    return fail(EVG_EBADSHAPE, "softmax_bwd: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (rows == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_softmax_bwd<T>(y, dy, dx, rows, cols, (cudaStream_t)stream);
  });
}
