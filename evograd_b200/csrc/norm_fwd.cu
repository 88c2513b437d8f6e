// LayerNorm / RMSNorm forward for sm_100a.
//
// HBM-bound: one read of x and one write of y per element (plus 4 or 8 bytes
// of statistics per row). The row lives in registers between the reduction
// passes, so x is read from memory exactly once.
#include "rowcfg.cuh"

namespace evg {
namespace {

// LN = true : y = ((x-mean)*rstd)*w + b, two-pass variance (the rounding points
//             of layernorm_forward_ref, ops/level1/layernorm/forward_ref.py:20-23)
// LN = false: y = (x*rstd)*w          (rmsnorm_forward_ref, .../rmsnorm/forward_ref.py:19-21)
// On B200 these kernels are bounded by instruction issue before HBM (about 22
// thread-instructions per element are available at full bandwidth), so the row
// is unpacked to float32 registers ONCE and weight/bias are staged in shared
// memory as float32, laid out so that consecutive threads read consecutive
// float4 (slot q of vector idx lives at [q * nvec + idx]).
// WBP (groups of 512 threads and more, 16-bit LayerNorm): weight and bias stay in
// their 16-bit form in shared memory, because float32 copies of both for a row of
// 8192+ columns leave room for one block per SM only.
template <typename T, int G, int VPT, bool LN, bool WBP = false>
__global__ void __launch_bounds__(G > 256 ? rowcfg_max_threads(G) : 256,
                                  G > 512 ? 1 : (G > 256 ? 2 : 3))
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                int64_t rows, int cols, float eps) {
  constexpr int N = Vec<T>::N;
  constexpr int Q = N / 4;  // float4 slots per 128-bit input vector
  extern __shared__ float4 smem4[];
  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int groups = blockDim.x / G;
  const int nvec = cols / N;
  float4* w4 = smem4;                              // [Q][nvec]
  float4* b4 = smem4 + (size_t)Q * nvec;           // [Q][nvec] (LayerNorm only)
  uint4* wp = reinterpret_cast<uint4*>(smem4);     // WBP: [nvec] packed weight, then bias
  uint4* bp = wp + nvec;
  float* scratch = WBP ? reinterpret_cast<float*>(wp + (size_t)(LN ? 2 : 1) * nvec)
                       : reinterpret_cast<float*>(smem4 + (size_t)(LN ? 2 : 1) * Q * nvec);
  scratch += gid * (2 * (G / 32));
  int phase = 0;
  for (int idx = threadIdx.x; idx < nvec; idx += blockDim.x) {
    if constexpr (WBP) {
      wp[idx] = *reinterpret_cast<const uint4*>(w + (size_t)idx * N);
      if constexpr (LN) bp[idx] = *reinterpret_cast<const uint4*>(b + (size_t)idx * N);
    } else {
      float f[N];
      unpack<T>(*reinterpret_cast<const uint4*>(w + (size_t)idx * N), f);
#pragma unroll
      for (int q = 0; q < Q; ++q)
        w4[q * nvec + idx] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
      if constexpr (LN) {
        unpack<T>(*reinterpret_cast<const uint4*>(b + (size_t)idx * N), f);
#pragma unroll
        for (int q = 0; q < Q; ++q)
          b4[q * nvec + idx] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
      }
    }
  }
  __syncthreads();
  const float inv_cols = 1.0f / (float)cols;

  // The next row of the group is on its way while this one is reduced and written:
  // its vectors are requested before the first reduction and unpacked a row later.
  const int64_t row_step = (int64_t)gridDim.x * groups;
  uint4 nxt[VPT];
  {
    const int64_t row0 = (int64_t)blockIdx.x * groups + gid;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      nxt[k] = make_uint4(0, 0, 0, 0);
      if (row0 < rows && idx < nvec) nxt[k] = ld_vec(x + row0 * cols + (size_t)idx * N);
    }
  }
  for (int64_t row = (int64_t)blockIdx.x * groups + gid; row < rows; row += row_step) {
    float xf[VPT][N];
#pragma unroll
    for (int k = 0; k < VPT; ++k) unpack<T>(nxt[k], xf[k]);  // padded vectors unpack to zeros
    if (row + row_step < rows) {
      const T* xn = x + (row + row_step) * cols;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int idx = lig + k * G;
        if (idx < nvec) nxt[k] = ld_vec(xn + (size_t)idx * N);
      }
    }
    float mu = 0.f;
    if constexpr (LN) {
      float s[1] = {0.f};
#pragma unroll
      for (int k = 0; k < VPT; ++k)
#pragma unroll
        for (int j = 0; j < N; ++j) s[0] += xf[k][j];
      group_allreduce<G, 1, SumOp>(s, scratch, phase, gid, lig);
      mu = s[0] * inv_cols;
    }
    float q[1] = {0.f};
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      if (lig + k * G < nvec) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float d = xf[k][j] - mu;
          q[0] = fmaf(d, d, q[0]);
        }
      }
    }
    group_allreduce<G, 1, SumOp>(q, scratch, phase, gid, lig);
    const float rs = 1.0f / sqrtf(q[0] * inv_cols + eps);
    const float nmr = -mu * rs;
    if (lig == 0) {
      rstd_out[row] = rs;
      if constexpr (LN) mean_out[row] = mu;
    }
    T* yr = y + row * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      if (idx < nvec) {
        float o[N];
        if constexpr (WBP) {
          float wj[N], bj[N];
          unpack<T>(wp[idx], wj);
          if constexpr (LN) unpack<T>(bp[idx], bj);
#pragma unroll
          for (int j = 0; j < N; ++j) {
            if constexpr (LN) o[j] = fmaf(fmaf(xf[k][j], rs, nmr), wj[j], bj[j]);
            else o[j] = (xf[k][j] * rs) * wj[j];
          }
        } else
#pragma unroll
        for (int qq = 0; qq < Q; ++qq) {
          const float4 wv = w4[qq * nvec + idx];
          const float wj[4] = {wv.x, wv.y, wv.z, wv.w};
          if constexpr (LN) {
            const float4 bv = b4[qq * nvec + idx];
            const float bj[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
              o[4 * qq + j] = fmaf(fmaf(xf[k][4 * qq + j], rs, nmr), wj[j], bj[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) o[4 * qq + j] = (xf[k][4 * qq + j] * rs) * wj[j];
          }
        }
        st_vec(yr + (size_t)idx * N, pack<T>(o));
      }
    }
  }
}

// Any width, any alignment: one block per row, three passes (the second and
// third re-read the row, which the first pass left in L2).
template <typename T, bool LN>
__global__ void __launch_bounds__(1024, 1)
norm_fwd_generic_kernel(const T* __restrict__ x, const T* __restrict__ w,
                        const T* __restrict__ b, T* __restrict__ y,
                        float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t rows,
                        int64_t cols, float eps) {
  __shared__ float scratch[2 * 32];
  int phase = 0;
  const float inv_cols = 1.0f / (float)cols;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float mu = 0.f;
    if constexpr (LN) {
      float s[1] = {0.f};
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s[0] += to_f32<T>(xr[c]);
      block_allreduce<1, SumOp>(s, scratch, phase);
      mu = s[0] * inv_cols;
    }
    float q[1] = {0.f};
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float d = to_f32<T>(xr[c]) - mu;
      q[0] += d * d;
    }
    block_allreduce<1, SumOp>(q, scratch, phase);
    const float rs = 1.0f / sqrtf(q[0] * inv_cols + eps);
    if (threadIdx.x == 0) {
      rstd_out[row] = rs;
      if constexpr (LN) mean_out[row] = mu;
    }
    T* yr = y + row * cols;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float xf = to_f32<T>(xr[c]);
      float o = __fmul_rn(__fmul_rn(xf - mu, rs), to_f32<T>(w[c]));
      if constexpr (LN) o = __fadd_rn(o, to_f32<T>(b[c]));
      yr[c] = from_f32<T>(o);
    }
  }
}

template <typename T, bool LN>
int launch_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                    int64_t rows, int64_t hidden, float eps, cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  const char* op = LN ? "layernorm_fwd" : "rmsnorm_fwd";
  const bool vec_ok = hidden % N == 0 && aligned16(x) && aligned16(y) && aligned16(w) &&
                      (!LN || aligned16(b)) && hidden < (int64_t)1 << 31;
  RowCfg cfg;
  if (vec_ok && !tune("rows.force_generic") && pick_rowcfg(op, hidden / N, cfg)) {
    if (cfg.G <= 256 && cfg.threads > 256) cfg.threads = 256;  // the kernel's launch bound
    const int groups = cfg.threads / cfg.G;
    constexpr bool kCanPack = LN && sizeof(T) == 2;
    const bool packed = kCanPack && cfg.G >= 512;
    const size_t smem = (size_t)(LN ? 2 : 1) * hidden * (packed ? sizeof(T) : sizeof(float)) +
                        (size_t)groups * 2 * (cfg.G / 32) * sizeof(float);
#define EVG_X(g, v)                                                                           \
  if (cfg.G == g && cfg.VPT == v && smem <= (size_t)device_info().max_smem_optin) {           \
    auto kern = norm_fwd_kernel<T, g, v, LN, (kCanPack && g >= 512)>;                         \
    if (smem > 48 * 1024)                                                                     \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    const int grid = persistent_grid(kern, cfg.threads, smem, rows, groups);                  \
    kern<<<grid, cfg.threads, smem, stream>>>((const T*)x, (const T*)w, (const T*)b, (T*)y,   \
                                              mean, rstd, rows, (int)hidden, eps);            \
    return check_launch(op);                                                                  \
  }
    EVG_ROWCFG_LIST(EVG_X)
#undef EVG_X
  }
  auto kern = norm_fwd_generic_kernel<T, LN>;
  const int threads = hidden >= 2048 ? 1024 : (hidden >= 256 ? 256 : 64);
  const int grid = persistent_grid(kern, threads, 0, rows, 1);
  kern<<<grid, threads, 0, stream>>>((const T*)x, (const T*)w, (const T*)b, (T*)y, mean, rstd,
                                     rows, hidden, eps);
  return check_launch(op);
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_layernorm_fwd(const void* x, const void* weight, const void* bias, void* y,
                                 float* mean, float* rstd, int64_t rows, int64_t hidden, float eps,
                                 int dtype, void* stream) {
  if (!x || !weight || !bias || !y || !mean || !rstd)
    return fail(EVG_ENULL, "layernorm_fwd: null pointer argument");
  if (rows < 0 || hidden <= 0) return fail(EVG_EBADSHAPE, "layernorm_fwd: rows=%lld hidden=%lld",
                                           (long long)rows, (long long)hidden);
  if (rows == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_norm_fwd<T, true>(x, weight, bias, y, mean, rstd, rows, hidden, eps,
                                    (cudaStream_t)stream);
  });
}

extern "C" int evg_rmsnorm_fwd(const void* x, const void* weight, void* y, float* rstd,
                               int64_t rows, int64_t hidden, float eps, int dtype, void* stream) {
  if (!x || !weight || !y || !rstd) return fail(EVG_ENULL, "rmsnorm_fwd: null pointer argument");
  if (rows < 0 || hidden <= 0) return fail(EVG_EBADSHAPE, "rmsnorm_fwd: rows=%lld hidden=%lld",
                                           (long long)rows, (long long)hidden);
  if (rows == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_norm_fwd<T, false>(x, weight, nullptr, y, nullptr, rstd, rows, hidden, eps,
                                     (cudaStream_t)stream);
  });
}
