// Residual add fused into RMSNorm, forward and backward, for sm_100a.
//
//   s   = T(x + r)                                   (rounded to the input dtype)
//   out = T( T(s * T(rstd)) * w ),  rstd = rsqrt(mean(float(s)^2) + eps)
//
// which are the rounding points of fused_add_rms_norm_forward_ref
// (ops/level2/fused_add_rms_norm/forward_ref.py:6-14): the sum is taken in the
// input dtype, rstd is float32 but is cast to the input dtype before it
// multiplies s, and both products are taken in the input dtype.
//
// Saved state: float32 rstd per row. The sum s is NOT stored: the backward
// re-forms it from x and r (three reads + one write either way, and no
// rows x hidden tensor is kept alive between the passes).
//
// HBM-bound. Forward: reads x, r, writes out. Backward: reads dout, x, r,
// writes dx (= dr: both inputs see the same gradient through s); dweight by the
// same two-stage atomic-free column reduction as the other norm kernels.
#include "norm_reduce.cuh"
#include "rowcfg.cuh"
#include "sm100_umma.cuh"

namespace evg {
namespace {

template <typename T, int G, int VPT>
__global__ void __launch_bounds__(rowcfg_max_threads(G), G > 512 ? 1 : 2)
add_rms_fwd_kernel(const T* __restrict__ x, const T* __restrict__ r, const T* __restrict__ w,
                   T* __restrict__ y, float* __restrict__ rstd_out, int64_t rows, int cols,
                   float eps) {
  constexpr int N = Vec<T>::N;
  constexpr int Q = N / 4;
  extern __shared__ float4 smem4[];
  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int groups = blockDim.x / G;
  const int nvec = cols / N;
  float4* w4 = smem4;  // float32 weight, slot q of vector idx at [q * nvec + idx]
  float* scratch = reinterpret_cast<float*>(smem4 + (size_t)Q * nvec) + gid * (2 * (G / 32));
  int phase = 0;
  for (int idx = threadIdx.x; idx < nvec; idx += blockDim.x) {
    float f[N];
    unpack<T>(*reinterpret_cast<const uint4*>(w + (size_t)idx * N), f);
#pragma unroll
    for (int q = 0; q < Q; ++q)
      w4[q * nvec + idx] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
  }
  __syncthreads();
  const float inv_cols = 1.0f / (float)cols;

  for (int64_t row = (int64_t)blockIdx.x * groups + gid; row < rows;
       row += (int64_t)gridDim.x * groups) {
    const T* xr = x + row * cols;
    const T* rr = r + row * cols;
    float sf[VPT][N];
    float q[1] = {0.f};
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      uint4 xv = make_uint4(0, 0, 0, 0), rv = make_uint4(0, 0, 0, 0);
      if (idx < nvec) {
        xv = ld_vec(xr + (size_t)idx * N);
        rv = ld_vec(rr + (size_t)idx * N);
      }
      float rf[N];
      unpack<T>(xv, sf[k]);
      unpack<T>(rv, rf);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        sf[k][j] = round_to<T>(sf[k][j] + rf[j]);  // padded vectors stay zero
        q[0] = fmaf(sf[k][j], sf[k][j], q[0]);
      }
    }
    group_allreduce<G, 1, SumOp>(q, scratch, phase, gid, lig);
    const float rs = 1.0f / sqrtf(q[0] * inv_cols + eps);
    const float rb = round_to<T>(rs);
    if (lig == 0) rstd_out[row] = rs;
    T* yr = y + row * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      if (idx < nvec) {
        float o[N];
#pragma unroll
        for (int qq = 0; qq < Q; ++qq) {
          const float4 wv = w4[qq * nvec + idx];
          const float wj[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            o[4 * qq + j] = __fmul_rn(round_to<T>(__fmul_rn(sf[k][4 * qq + j], rb)), wj[j]);
        }
        st_vec(yr + (size_t)idx * N, pack<T>(o));
      }
    }
  }
}

// Any width, any alignment: one block per row, two passes (the second re-reads
// the row, which the first pass left in L2).
template <typename T>
__global__ void __launch_bounds__(1024, 1)
add_rms_fwd_generic_kernel(const T* __restrict__ x, const T* __restrict__ r,
                           const T* __restrict__ w, T* __restrict__ y,
                           float* __restrict__ rstd_out, int64_t rows, int64_t cols, float eps) {
  __shared__ float scratch[2 * 32];
  int phase = 0;
  const float inv_cols = 1.0f / (float)cols;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    const T* rr = r + row * cols;
    float q[1] = {0.f};
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float s = round_to<T>(to_f32<T>(xr[c]) + to_f32<T>(rr[c]));
      q[0] = fmaf(s, s, q[0]);
    }
    block_allreduce<1, SumOp>(q, scratch, phase);
    const float rs = 1.0f / sqrtf(q[0] * inv_cols + eps);
    const float rb = round_to<T>(rs);
    if (threadIdx.x == 0) rstd_out[row] = rs;
    T* yr = y + row * cols;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float s = round_to<T>(to_f32<T>(xr[c]) + to_f32<T>(rr[c]));
      yr[c] = from_f32<T>(__fmul_rn(round_to<T>(__fmul_rn(s, rb)), to_f32<T>(w[c])));
    }
  }
}

template <typename T>
int launch_add_rms_fwd(const void* x, const void* r, const void* w, void* y, float* rstd,
                       int64_t rows, int64_t hidden, float eps, cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  const char* op = "fused_add_rmsnorm_fwd";
  const bool vec_ok = hidden % N == 0 && aligned16(x) && aligned16(r) && aligned16(y) &&
                      aligned16(w) && hidden < (int64_t)1 << 31;
  RowCfg cfg;
  if (vec_ok && !tune("rows.force_generic") && pick_rowcfg(op, hidden / N, cfg)) {
    const int groups = cfg.threads / cfg.G;
    const size_t smem =
        (size_t)hidden * sizeof(float) + (size_t)groups * 2 * (cfg.G / 32) * sizeof(float);
#define EVG_X(g, v)                                                                         \
  if (cfg.G == g && cfg.VPT == v && smem <= (size_t)device_info().max_smem_optin) {         \
    auto kern = add_rms_fwd_kernel<T, g, v>;                                                \
    if (smem > 48 * 1024)                                                                   \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    const int grid = persistent_grid(kern, cfg.threads, smem, rows, groups);                \
    kern<<<grid, cfg.threads, smem, stream>>>((const T*)x, (const T*)r, (const T*)w, (T*)y, \
                                              rstd, rows, (int)hidden, eps);                \
    return check_launch(op);                                                                \
  }
    EVG_ROWCFG_LIST(EVG_X)
#undef EVG_X
  }
  auto kern = add_rms_fwd_generic_kernel<T>;
  const int threads = hidden >= 2048 ? 1024 : (hidden >= 256 ? 256 : 64);
  const int grid = persistent_grid(kern, threads, 0, rows, 1);
  kern<<<grid, threads, 0, stream>>>((const T*)x, (const T*)r, (const T*)w, (T*)y, rstd, rows,
                                     hidden, eps);
  return check_launch(op);
}

// Sticky status of the bounded waits in this file (0 = fine).
__device__ int g_addrms_device_status = 0;

// Backward, row-ring variant (the structure of the RMSNorm backward ring): the
// rows of x, r and dout are brought into a shared-memory ring by bulk async
// copies counted by one mbarrier per stage; one block = THREADS threads walking
// rows blockIdx.x, blockIdx.x + gridDim.x, ...; thread t owns vectors
// t, t + THREADS, ... of every row and keeps its float32 dweight sums in
// registers. With g = dout*w and c = sum_cols(g*s):
//   ds = g*T(rstd) - s * rstd^3 * c / cols,   dweight = sum_rows dout * T(s*T(rstd))
// (autograd of the forward above: the casts pass gradients through unchanged).
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS, (THREADS == 256 && VPT <= 2) ? 2 : 1)
add_rms_bwd_ring_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                        const T* __restrict__ r, const T* __restrict__ w,
                        const float* __restrict__ rstd, T* __restrict__ dx,
                        float* __restrict__ partial, int64_t rows, int cols, int stages,
                        long long wait_limit) {
  using namespace umma;
  constexpr int N = Vec<T>::N;
  constexpr int Q = N / 4;
  constexpr int P = N / 2;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  const int tid = threadIdx.x;
  const int nvec = cols / N;
  const uint32_t row_bytes = (uint32_t)cols * sizeof(T);
  // smem: [stages][3][row_bytes] ring | float32 weight [Q][nvec] float4 | mbarriers | scratch
  uint8_t* ring = ring_raw;
  float4* w4 = reinterpret_cast<float4*>(ring + (size_t)stages * 3 * row_bytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(w4 + (size_t)Q * nvec);
  float* scratch = reinterpret_cast<float*>(full + 16);
  int* abort_flag = reinterpret_cast<int*>(scratch + 2 * 32);
  int phase = 0;

  const int64_t first = blockIdx.x;
  const int64_t n_mine = first < rows ? (rows - first + gridDim.x - 1) / gridDim.x : 0;
  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  for (int idx = tid; idx < nvec; idx += THREADS) {
    float f[N];
    unpack<T>(*reinterpret_cast<const uint4*>(w + (size_t)idx * N), f);
#pragma unroll
    for (int q = 0; q < Q; ++q)
      w4[q * nvec + idx] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
  }
  __syncthreads();
  const WaitCtx ctx{abort_flag, &g_addrms_device_status, wait_limit};
  auto issue = [&](int64_t i) {
    const int s = (int)(i % stages);
    const int64_t row = first + i * gridDim.x;
    uint8_t* dst = ring + (size_t)s * 3 * row_bytes;
    mbar_expect_tx(&full[s], 3 * row_bytes);
    bulk_load_1d(dst, x + row * cols, row_bytes, &full[s]);
    bulk_load_1d(dst + row_bytes, r + row * cols, row_bytes, &full[s]);
    bulk_load_1d(dst + 2 * row_bytes, dy + row * cols, row_bytes, &full[s]);
  };
  if (tid == 0)
    for (int64_t i = 0; i < stages && i < n_mine; ++i) issue(i);

  f32x2 acc_w[VPT][P];
#pragma unroll
  for (int k = 0; k < VPT; ++k)
#pragma unroll
    for (int j = 0; j < P; ++j) acc_w[k][j] = 0ull;
  const float inv_cols = 1.0f / (float)cols;
  float rs_next = n_mine > 0 ? rstd[first] : 0.f;

  int s = 0;
  uint32_t parity = 0;
  const size_t row_step = (size_t)gridDim.x * cols;
  T* dr = dx + first * cols;
  const float* rstd_p = rstd + first;
  for (int64_t i = 0; i < n_mine; ++i) {
    const float rs = rs_next;
    if (i + 1 < n_mine) {
      rstd_p += gridDim.x;
      rs_next = *rstd_p;
    }
    const float rb = round_to<T>(rs);
    mbar_wait(&full[s], parity, ctx, 411);
    const uint8_t* sx = ring + (size_t)s * 3 * row_bytes;
    const uint8_t* sr = sx + row_bytes;
    const uint8_t* sg = sr + row_bytes;

    f32x2 sh[VPT][P], gy[VPT][P];
    f32x2 c0 = 0ull;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = tid + k * THREADS;
      const bool ok = idx < nvec;
      const int sidx = ok ? idx : 0;
      uint4 xv = make_uint4(0, 0, 0, 0), rv = xv, gv = xv;
      if (ok) {
        xv = *reinterpret_cast<const uint4*>(sx + (size_t)idx * 16);
        rv = *reinterpret_cast<const uint4*>(sr + (size_t)idx * 16);
        gv = *reinterpret_cast<const uint4*>(sg + (size_t)idx * 16);
      }
      float xf[N], rf[N], gf[N];
      unpack<T>(xv, xf);
      unpack<T>(rv, rf);
      unpack<T>(gv, gf);  // padded vectors have dout = 0 and add nothing below
#pragma unroll
      for (int j = 0; j < N; ++j) xf[j] = round_to<T>(xf[j] + rf[j]);
#pragma unroll
      for (int qq = 0; qq < Q; ++qq) {
        const float4 wv = w4[qq * nvec + sidx];
        const f32x2 wp[2] = {f2_make(wv.x, wv.y), f2_make(wv.z, wv.w)};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int pi = 2 * qq + h;
          sh[k][pi] = f2_make(xf[2 * pi], xf[2 * pi + 1]);
          gy[k][pi] = f2_make(gf[2 * pi], gf[2 * pi + 1]);
          c0 = f2_fma(f2_mul(gy[k][pi], wp[h]), sh[k][pi], c0);
        }
      }
    }
    float c[1];
    {
      float lo, hi;
      f2_split(c0, lo, hi);
      c[0] = lo + hi;
    }
    block_allreduce_sum_fixed<1, THREADS / 32>(c, scratch, phase);  // all done with stage s
    if (tid == 0 && i + stages < n_mine) issue(i + stages);
    const f32x2 a_s = f2_splat(-(rs * rs) * rs * (c[0] * inv_cols));
    const f32x2 rb2 = f2_splat(rb);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = tid + k * THREADS;
      if (idx < nvec) {
        float o[N];
#pragma unroll
        for (int qq = 0; qq < Q; ++qq) {
          const float4 wv = w4[qq * nvec + idx];
          const f32x2 wp[2] = {f2_make(wv.x, wv.y), f2_make(wv.z, wv.w)};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int pi = 2 * qq + h;
            const f32x2 g = f2_mul(gy[k][pi], wp[h]);
            const f32x2 op = f2_fma(sh[k][pi], a_s, f2_mul(g, rb2));
            f2_split(op, o[2 * pi], o[2 * pi + 1]);
            float t0, t1;
            f2_split(f2_mul(sh[k][pi], rb2), t0, t1);
            acc_w[k][pi] = f2_fma(gy[k][pi], f2_make(round_to<T>(t0), round_to<T>(t1)),
                                  acc_w[k][pi]);
          }
        }
        st_vec(dr + (size_t)idx * N, pack<T>(o));
      }
    }
    dr += row_step;
    if (++s == stages) {
      s = 0;
      parity ^= 1;
    }
  }
  // After a timeout every wait above fell through, so the last copies may still be
  // in flight: give them time to land before the block's shared memory is given up.
  grid_dependents_go();  // the column reduce may be launched behind this grid now
  if (tid == 0 && *(volatile int*)abort_flag) settle_after_abort();
  float* pw = partial + (size_t)blockIdx.x * cols;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int idx = tid + k * THREADS;
    if (idx < nvec) {
#pragma unroll
      for (int qq = 0; qq < Q; ++qq) {
        float a0, a1, a2, a3;
        f2_split(acc_w[k][2 * qq], a0, a1);
        f2_split(acc_w[k][2 * qq + 1], a2, a3);
        *reinterpret_cast<float4*>(pw + (size_t)idx * N + 4 * qq) = make_float4(a0, a1, a2, a3);
      }
    }
  }
}

// Backward, group variant for NARROW rows (fewer than 256 vectors): a row is
// handled by a group of G threads that keep it in registers, a block holds
// several groups working on different rows, and the groups' column sums are
// folded through shared memory in group order before the block writes its one
// partial row. (The one-row-per-block ring above would leave most of its threads
// idle on such rows.) Same arithmetic as the ring kernel.
template <typename T, int G, int VPT>
__global__ void __launch_bounds__(rowcfg_max_threads(G))
add_rms_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ r,
                   const T* __restrict__ w, const float* __restrict__ rstd, T* __restrict__ dx,
                   float* __restrict__ partial, int64_t rows, int cols) {
  constexpr int N = Vec<T>::N;
  constexpr int Q = N / 4;
  extern __shared__ float4 smem4[];
  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int groups = blockDim.x / G;
  const int nvec = cols / N;
  // smem: float32 weight [Q][nvec] float4 | [cols] fold buffer | [groups][2][G/32] scratch
  float4* w4 = smem4;
  float* colbuf = reinterpret_cast<float*>(smem4 + (size_t)Q * nvec);
  float* scratch = colbuf + cols + gid * (2 * (G / 32));
  int phase = 0;
  for (int idx = threadIdx.x; idx < nvec; idx += blockDim.x) {
    float f[N];
    unpack<T>(*reinterpret_cast<const uint4*>(w + (size_t)idx * N), f);
#pragma unroll
    for (int q = 0; q < Q; ++q)
      w4[q * nvec + idx] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
  }
  __syncthreads();
  float acc_w[VPT][N];
#pragma unroll
  for (int k = 0; k < VPT; ++k)
#pragma unroll
    for (int j = 0; j < N; ++j) acc_w[k][j] = 0.f;
  const float inv_cols = 1.0f / (float)cols;

  for (int64_t row = (int64_t)blockIdx.x * groups + gid; row < rows;
       row += (int64_t)gridDim.x * groups) {
    const T* xr = x + row * cols;
    const T* rr = r + row * cols;
    const T* gr = dy + row * cols;
    uint4 xv[VPT], rv[VPT], gv[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      xv[k] = rv[k] = gv[k] = make_uint4(0, 0, 0, 0);
      if (idx < nvec) {
        xv[k] = ld_vec(xr + (size_t)idx * N);
        rv[k] = ld_vec(rr + (size_t)idx * N);
        gv[k] = ld_vec(gr + (size_t)idx * N);
      }
    }
    const float rs = rstd[row];
    const float rb = round_to<T>(rs);
    float sv[VPT][N], gy[VPT][N];
    float c[1] = {0.f};
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      float rf[N];
      unpack<T>(xv[k], sv[k]);
      unpack<T>(rv[k], rf);
      unpack<T>(gv[k], gy[k]);  // padded vectors have dout = 0 and add nothing
      const int sidx = idx < nvec ? idx : 0;
#pragma unroll
      for (int qq = 0; qq < Q; ++qq) {
        const float4 wv = w4[qq * nvec + sidx];
        const float wj[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int e = 4 * qq + j;
          sv[k][e] = round_to<T>(sv[k][e] + rf[e]);
          c[0] = fmaf(gy[k][e] * wj[j], sv[k][e], c[0]);
        }
      }
    }
    group_allreduce<G, 1, SumOp>(c, scratch, phase, gid, lig);
    const float a_s = -(rs * rs) * rs * (c[0] * inv_cols);
    T* dr = dx + row * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      if (idx < nvec) {
        float o[N];
#pragma unroll
        for (int qq = 0; qq < Q; ++qq) {
          const float4 wv = w4[qq * nvec + idx];
          const float wj[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e = 4 * qq + j;
            const float g = gy[k][e] * wj[j];
            o[e] = fmaf(sv[k][e], a_s, g * rb);
            acc_w[k][e] = fmaf(gy[k][e], round_to<T>(sv[k][e] * rb), acc_w[k][e]);
          }
        }
        st_vec(dr + (size_t)idx * N, pack<T>(o));
      }
    }
  }
  // Fold the groups of this block in group order, then write one partial row.
  for (int g = 0; g < groups; ++g) {
    if (gid == g) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int idx = lig + k * G;
        if (idx < nvec) {
#pragma unroll
          for (int j = 0; j < N; ++j) {
            const int col = idx * N + j;
            colbuf[col] = g == 0 ? acc_w[k][j] : colbuf[col] + acc_w[k][j];
          }
        }
      }
    }
    __syncthreads();
  }
  float* pw = partial + (size_t)blockIdx.x * cols;
  for (int col = threadIdx.x; col < cols; col += blockDim.x) pw[col] = colbuf[col];
}

// Any width / alignment. One block per row at a time; the block's partial row
// in the workspace is private to it, so plain read-modify-write is race free.
template <typename T>
__global__ void __launch_bounds__(1024, 1)
add_rms_bwd_generic_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                           const T* __restrict__ r, const T* __restrict__ w,
                           const float* __restrict__ rstd, T* __restrict__ dx,
                           float* __restrict__ partial, int64_t rows, int64_t cols) {
  __shared__ float scratch[2 * 32];
  int phase = 0;
  const float inv_cols = 1.0f / (float)cols;
  float* pw = partial + (size_t)blockIdx.x * cols;
  bool first = true;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    const T* rr = r + row * cols;
    const T* gr = dy + row * cols;
    const float rs = rstd[row];
    const float rb = round_to<T>(rs);
    float c[1] = {0.f};
    for (int64_t col = threadIdx.x; col < cols; col += blockDim.x) {
      const float s = round_to<T>(to_f32<T>(xr[col]) + to_f32<T>(rr[col]));
      c[0] = fmaf(to_f32<T>(gr[col]) * to_f32<T>(w[col]), s, c[0]);
    }
    block_allreduce<1, SumOp>(c, scratch, phase);
    const float a_s = -(rs * rs) * rs * (c[0] * inv_cols);
    T* dr = dx + row * cols;
    for (int64_t col = threadIdx.x; col < cols; col += blockDim.x) {
      const float s = round_to<T>(to_f32<T>(xr[col]) + to_f32<T>(rr[col]));
      const float go = to_f32<T>(gr[col]);
      const float g = go * to_f32<T>(w[col]);
      dr[col] = from_f32<T>(fmaf(s, a_s, g * rb));
      const float contrib = go * round_to<T>(s * rb);
      pw[col] = first ? contrib : pw[col] + contrib;
    }
    first = false;
  }
  if (first)  // a block without rows still owns a partial row
    for (int64_t col = threadIdx.x; col < cols; col += blockDim.x) pw[col] = 0.f;
}

int read_addrms_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_addrms_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_addrms_device_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_addrms_status_registered = (register_device_status(read_addrms_status), true);

int64_t add_rms_bwd_workspace(int64_t rows, int64_t hidden) {
  int64_t blocks = max_partial_blocks();
  if (blocks > rows) blocks = rows > 0 ? rows : 1;
  return blocks * hidden * (int64_t)sizeof(float);
}

template <typename T>
int launch_add_rms_bwd(const void* dy, const void* x, const void* r, const void* w,
                       const float* rstd, void* dx, void* dweight, float* out_f32,
                       void* workspace, int64_t workspace_bytes, int64_t rows, int64_t hidden,
                       cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  const char* op = "fused_add_rmsnorm_bwd";
  const int64_t need = add_rms_bwd_workspace(rows, hidden);
  if (!workspace || workspace_bytes < need)
    return fail(EVG_EWORKSPACE, "%s: workspace %lld bytes, need %lld", op,
                (long long)workspace_bytes, (long long)need);
  if (!aligned16(workspace)) return fail(EVG_EALIGN, "%s: workspace not 16-byte aligned", op);
  float* partial = (float*)workspace;
  const int cap = max_partial_blocks();
  int blocks = 0;
  bool launched = false;
  const bool vec_ok = hidden % N == 0 && aligned16(x) && aligned16(r) && aligned16(dy) &&
                      aligned16(dx) && aligned16(w) && hidden < (int64_t)1 << 31;
  const bool narrow_rows = vec_ok && hidden / N < 256;
  RowCfg cfg;
  if (narrow_rows && !tune("rows.force_generic") &&
      pick_rowcfg(op, hidden / N, cfg, 256, false)) {
    const int groups = cfg.threads / cfg.G;
    const size_t smem = ((size_t)groups * 2 * (cfg.G / 32) + (size_t)2 * hidden) * sizeof(float);
#define EVG_X(g, v)                                                                            \
  if (!launched && cfg.G == g && cfg.VPT == v) {                                               \
    auto kern = add_rms_bwd_kernel<T, g, v>;                                                   \
    if (smem > 48 * 1024)                                                                      \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    blocks = persistent_grid(kern, cfg.threads, smem, rows, groups, cap);                      \
    kern<<<blocks, cfg.threads, smem, stream>>>((const T*)dy, (const T*)x, (const T*)r,        \
                                                (const T*)w, rstd, (T*)dx, partial, rows,      \
                                                (int)hidden);                                  \
    launched = true;                                                                           \
  }
    EVG_X(32, 1) EVG_X(32, 2) EVG_X(32, 4) EVG_X(64, 4)
#undef EVG_X
  }
  if (!launched && vec_ok && !tune("rows.force_generic") && !tune("norm_bwd.no_ring")) {
    const int64_t nvec = hidden / N;
    constexpr int kThreads = 256;
    const size_t row_bytes = (size_t)hidden * sizeof(T);
    const size_t fixed = (size_t)hidden * sizeof(float) + 16 * 8 + 2 * 32 * sizeof(float) + 64;
    const size_t budget = (size_t)device_info().max_smem_optin;
    int stages = tune("norm_bwd.stages");
    if (stages <= 0) stages = (int)((72 * 1024) / (3 * row_bytes));  // 3 for 8 KB rows
    if (stages < 2) stages = 2;
    if (stages > 12) stages = 12;
    while (stages > 0 && fixed + (size_t)stages * 3 * row_bytes > budget) --stages;
    const long long wait_limit = 2000000000ll;
    if (stages >= 2 && nvec <= 8 * kThreads) {
      const size_t smem = fixed + (size_t)stages * 3 * row_bytes;
#define EVG_RING(v)                                                                          \
  if (!launched && nvec <= (int64_t)v * kThreads) {                                          \
    auto kern = add_rms_bwd_ring_kernel<T, kThreads, v>;                                     \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    blocks = persistent_grid(kern, kThreads, smem, rows, 1, cap);                            \
    kern<<<blocks, kThreads, smem, stream>>>((const T*)dy, (const T*)x, (const T*)r,         \
                                             (const T*)w, rstd, (T*)dx, partial, rows,       \
                                             (int)hidden, stages, wait_limit);               \
    launched = true;                                                                         \
  }
      EVG_RING(1) EVG_RING(2) EVG_RING(4) EVG_RING(8)
#undef EVG_RING
    }
  }
  if (!launched) {
    auto kern = add_rms_bwd_generic_kernel<T>;
    const int threads = hidden >= 2048 ? 1024 : (hidden >= 256 ? 256 : 64);
    blocks = persistent_grid(kern, threads, 0, rows, 1, cap);
    kern<<<blocks, threads, 0, stream>>>((const T*)dy, (const T*)x, (const T*)r, (const T*)w,
                                         rstd, (T*)dx, partial, rows, hidden);
  }
  int rc = check_launch(op);
  if (rc) return rc;
  if ((int64_t)blocks * hidden * (int64_t)sizeof(float) > workspace_bytes)
    return fail(EVG_EWORKSPACE, "%s: internal: partial rows exceed workspace", op);
  if (dweight || out_f32) {
    launch_colreduce<T>(partial, blocks, hidden, (T*)dweight, (T*)nullptr, out_f32, 1, stream);
    rc = check_launch("fused_add_rmsnorm_bwd colreduce");
  }
  return rc;
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_fused_add_rmsnorm_fwd(const void* x, const void* residual, const void* weight,
                                         void* out, float* rstd, int64_t rows, int64_t hidden,
                                         float eps, int dtype, void* stream) {
  if (!x || !residual || !weight || !out || !rstd)
    return fail(EVG_ENULL, "fused_add_rmsnorm_fwd: null pointer argument");
  if (rows < 0 || hidden <= 0)
    return fail(EVG_EBADSHAPE, "fused_add_rmsnorm_fwd: rows=%lld hidden=%lld", (long long)rows,
                (long long)hidden);
  if (rows == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_add_rms_fwd<T>(x, residual, weight, out, rstd, rows, hidden, eps,
                                 (cudaStream_t)stream);
  });
}

extern "C" int64_t evg_fused_add_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t hidden,
                                                             int dtype) {
  (void)dtype;
  if (rows < 0 || hidden <= 0) return 0;
  return add_rms_bwd_workspace(rows, hidden);
}

extern "C" int evg_fused_add_rmsnorm_bwd(const void* dout, const void* x, const void* residual,
                                         const void* weight, const float* rstd, void* dx,
                                         void* dweight, float* dweight_f32, void* workspace,
                                         int64_t workspace_bytes, int64_t rows, int64_t hidden,
                                         int dtype, void* stream) {
  if (!dout || !x || !residual || !weight || !rstd || !dx)
    return fail(EVG_ENULL, "fused_add_rmsnorm_bwd: null pointer argument");
  if (rows < 0 || hidden <= 0)
    return fail(EVG_EBADSHAPE, "fused_add_rmsnorm_bwd: rows=%lld hidden=%lld", (long long)rows,
                (long long)hidden);
  if (rows == 0) {
    // No rows: the column sums are zero.
    return EVG_DISPATCH_DTYPE(dtype, [&] {
      if (dweight) cudaMemsetAsync(dweight, 0, (size_t)hidden * sizeof(T), (cudaStream_t)stream);
      if (dweight_f32)
        cudaMemsetAsync(dweight_f32, 0, (size_t)hidden * sizeof(float), (cudaStream_t)stream);
      return check_launch("fused_add_rmsnorm_bwd");
    });
  }
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_add_rms_bwd<T>(dout, x, residual, weight, rstd, dx, dweight, dweight_f32,
                                 workspace, workspace_bytes, rows, hidden, (cudaStream_t)stream);
  });
}
