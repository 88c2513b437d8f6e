// LayerNorm / RMSNorm backward for sm_100a.
//
// HBM-bound: reads x and dy once, writes dx once. dweight/dbias are column sums
// over every row; they are formed in two stages without atomics:
//   stage 1  each persistent block keeps float32 column sums of its own rows in
//            registers and writes ONE partial row per block to the workspace;
//   stage 2  a small kernel adds the partial rows in a fixed order and rounds.
// The result is bit-reproducible from run to run for a given launch shape.
#include <mutex>

#include "norm_reduce.cuh"
#include "rowcfg.cuh"
#include "sm100_umma.cuh"

namespace evg {
namespace {

// Workspace layout (float32): [NP][blocks][cols], NP = 2 (dweight, dbias) for
// LayerNorm and 1 (dweight) for RMSNorm.
// Like the forward, this kernel is limited by instruction issue rather than HBM
// on B200: x-hat and dy are unpacked to float32 registers once per row, weight
// is staged in shared memory as float32 ([q * nvec + idx] float4 layout, read
// conflict-free), and every per-element step is a single fused multiply-add.
template <typename T, int G, int VPT, bool LN>
__global__ void __launch_bounds__(rowcfg_max_threads(G))
norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                const float* __restrict__ mean, const float* __restrict__ rstd,
                T* __restrict__ dx, float* __restrict__ partial, int64_t rows, int cols) {
  constexpr int N = Vec<T>::N;
  constexpr int Q = N / 4;
  constexpr int NV = LN ? 2 : 1;
  extern __shared__ float4 smem4[];
  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int groups = blockDim.x / G;
  const int nvec = cols / N;
  // smem: weight as float32 [Q][nvec] float4; then the [NV][cols] column
  // buffer; then [groups][2][NV][G/32] reduction scratch.
  float4* w4 = smem4;
  float* colbuf = reinterpret_cast<float*>(smem4 + (size_t)Q * nvec);
  float* scratch = colbuf + (size_t)NV * cols + gid * (2 * NV * (G / 32));
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
  float acc_b[LN ? VPT : 1][N];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      acc_w[k][j] = 0.f;
      if constexpr (LN) acc_b[k][j] = 0.f;
    }
  }
  const float inv_cols = 1.0f / (float)cols;

  for (int64_t row = (int64_t)blockIdx.x * groups + gid; row < rows;
       row += (int64_t)gridDim.x * groups) {
    const T* xr = x + row * cols;
    const T* gr = dy + row * cols;
    uint4 xv[VPT], gv[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      xv[k] = make_uint4(0, 0, 0, 0);
      gv[k] = make_uint4(0, 0, 0, 0);
      if (idx < nvec) {
        xv[k] = ld_vec(xr + (size_t)idx * N);
        gv[k] = ld_vec(gr + (size_t)idx * N);
      }
    }
    const float rs = rstd[row];
    float nmr = 0.f;
    if constexpr (LN) nmr = -mean[row] * rs;

    // xh = (x - mean) * rstd, gy = dy; c[0] = sum g*xh, c[1] = sum g with g = dy*w.
    // Padded vectors have dy = 0, so they add nothing to any sum.
    float xh[VPT][N], gy[VPT][N];
    float c[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) c[i] = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      unpack<T>(xv[k], xh[k]);
      unpack<T>(gv[k], gy[k]);
      const int sidx = idx < nvec ? idx : 0;
#pragma unroll
      for (int qq = 0; qq < Q; ++qq) {
        const float4 wv = w4[qq * nvec + sidx];
        const float wj[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int e = 4 * qq + j;
          xh[k][e] = LN ? fmaf(xh[k][e], rs, nmr) : xh[k][e] * rs;
          const float g = gy[k][e] * wj[j];
          c[0] = fmaf(g, xh[k][e], c[0]);
          if constexpr (LN) c[1] += g;
        }
      }
    }
    group_allreduce<G, NV, SumOp>(c, scratch, phase, gid, lig);
    // dx = rs*g - rs*mean(g) - rs*mean(g*xh)*xh
    const float a_x = -rs * (c[0] * inv_cols);
    float a_0 = 0.f;
    if constexpr (LN) a_0 = -rs * (c[1] * inv_cols);

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
            o[e] = fmaf(xh[k][e], a_x, fmaf(g, rs, a_0));
            acc_w[k][e] = fmaf(gy[k][e], xh[k][e], acc_w[k][e]);
            if constexpr (LN) acc_b[k][e] += gy[k][e];
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
            if (g == 0) {
              colbuf[col] = acc_w[k][j];
              if constexpr (LN) colbuf[cols + col] = acc_b[k][j];
            } else {
              colbuf[col] += acc_w[k][j];
              if constexpr (LN) colbuf[cols + col] += acc_b[k][j];
            }
          }
        }
      }
    }
    __syncthreads();
  }
  float* pw = partial + (size_t)blockIdx.x * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    pw[c] = colbuf[c];
    if constexpr (LN) pw[(size_t)gridDim.x * cols + c] = colbuf[cols + c];
  }
}

// Sticky status of the bounded waits in this file (0 = fine).
__device__ int g_norm_device_status = 0;

// Row-ring variant: the rows of x and dy are brought into a shared-memory ring
// by bulk async copies (one thread issues them, an mbarrier per stage counts
// the bytes), so the bytes in flight per SM are set by the ring depth and not
// by registers or occupancy. One block = one group of THREADS threads walking
// rows blockIdx.x, blockIdx.x + gridDim.x, ...; thread t owns vectors
// t, t + THREADS, ... of every row, keeps its float32 column sums in registers
// and writes the block's partial row straight from them at the end.
// The block-wide reduction barrier of row i also tells the issuing thread that
// stage i % STAGES has been read by everyone and can be refilled.
template <typename T, int THREADS, int VPT, bool LN>
__global__ void __launch_bounds__(THREADS, THREADS == 128 ? 4 : (THREADS == 256 && VPT <= 3) ? 2 : 1)
norm_bwd_ring_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                     const float* __restrict__ mean, const float* __restrict__ rstd,
                     T* __restrict__ dx, float* __restrict__ partial, int64_t rows, int cols,
                     int stages, long long wait_limit) {
  using namespace umma;
  constexpr int N = Vec<T>::N;
  constexpr int Q = N / 4;
  constexpr int NV = LN ? 2 : 1;
  // LayerNorm with eight vectors per thread: 128 registers of column sums leave no
  // room for x-hat and dy of the whole row (255 registers and spills). The row is
  // then read from the ring twice, once for the row sums and once for dx and the
  // column sums, and the stage is given back after the second pass.
  constexpr bool TWO_PASS = LN && VPT * THREADS >= 2048;
  constexpr int KEEP = TWO_PASS ? 1 : VPT;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  const int tid = threadIdx.x;
  const int nvec = cols / N;
  const uint32_t row_bytes = (uint32_t)cols * sizeof(T);
  // smem: [stages][2][row_bytes] ring | float32 weight [Q][nvec] float4 | mbarriers | scratch
  uint8_t* ring = ring_raw;
  float4* w4 = reinterpret_cast<float4*>(ring + (size_t)stages * 2 * row_bytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(w4 + (size_t)Q * nvec);
  float* scratch = reinterpret_cast<float*>(full + 16);
  int* abort_flag = reinterpret_cast<int*>(scratch + 2 * NV * 32);
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
  const WaitCtx ctx{abort_flag, &g_norm_device_status, wait_limit};
  auto issue = [&](int64_t i) {
    const int s = (int)(i % stages);
    const int64_t row = first + i * gridDim.x;
    uint8_t* dst = ring + (size_t)s * 2 * row_bytes;
    mbar_expect_tx(&full[s], 2 * row_bytes);
    bulk_load_1d(dst, x + row * cols, row_bytes, &full[s]);
    bulk_load_1d(dst + row_bytes, dy + row * cols, row_bytes, &full[s]);
  };
  if (tid == 0)
    for (int64_t i = 0; i < stages && i < n_mine; ++i) issue(i);

  // Element-wise float32 work is done on packed pairs (f32x2): element 2p and
  // 2p+1 of a vector share one instruction.
  constexpr int P = N / 2;  // pairs per 128-bit input vector
  f32x2 acc_w[VPT][P];
  f32x2 acc_b[LN ? VPT : 1][P];
#pragma unroll
  for (int k = 0; k < VPT; ++k)
#pragma unroll
    for (int j = 0; j < P; ++j) {
      acc_w[k][j] = 0ull;
      if constexpr (LN) acc_b[k][j] = 0ull;
    }
  const float inv_cols = 1.0f / (float)cols;
  float rs_next = 0.f, mu_next = 0.f;
  if (n_mine > 0) {
    rs_next = rstd[first];
    if constexpr (LN) mu_next = mean[first];
  }

  // Loop state is carried incrementally (stage, parity, row pointers): at ~16
  // elements per thread and row, a runtime division per row would be a visible
  // share of the instruction budget.
  int s = 0;
  uint32_t parity = 0;
  const size_t row_step = (size_t)gridDim.x * cols;
  T* dr = dx + first * cols;
  const float* rstd_p = rstd + first;
  const float* mean_p = LN ? mean + first : nullptr;
  for (int64_t i = 0; i < n_mine; ++i) {
    const float rs = rs_next;
    const float nmr = LN ? -mu_next * rs : 0.f;
    if (i + 1 < n_mine) {  // statistics of the next row, off the critical path
      rstd_p += gridDim.x;
      rs_next = *rstd_p;
      if constexpr (LN) {
        mean_p += gridDim.x;
        mu_next = *mean_p;
      }
    }
    mbar_wait(&full[s], parity, ctx, 401);
    const uint8_t* sx = ring + (size_t)s * 2 * row_bytes;
    const uint8_t* sg = sx + row_bytes;
    const f32x2 rs2 = f2_splat(rs), nmr2 = f2_splat(nmr);

    f32x2 xh[KEEP][P], gy[KEEP][P];
    // x-hat and dy of vector k of this thread, from the ring stage
    auto fetch = [&](int k, f32x2 (&xo)[P], f32x2 (&go)[P]) {
      const int idx = tid + k * THREADS;
      uint4 xv = make_uint4(0, 0, 0, 0), gv = make_uint4(0, 0, 0, 0);
      if (idx < nvec) {
        xv = *reinterpret_cast<const uint4*>(sx + (size_t)idx * 16);
        gv = *reinterpret_cast<const uint4*>(sg + (size_t)idx * 16);
      }
      float xf[N], gf[N];
      unpack<T>(xv, xf);
      unpack<T>(gv, gf);  // padded vectors have dy = 0 and add nothing below
#pragma unroll
      for (int pi = 0; pi < P; ++pi) {
        const f32x2 xp = f2_make(xf[2 * pi], xf[2 * pi + 1]);
        go[pi] = f2_make(gf[2 * pi], gf[2 * pi + 1]);
        xo[pi] = LN ? f2_fma(xp, rs2, nmr2) : f2_mul(xp, rs2);
      }
    };
    f32x2 c0 = 0ull, c1 = 0ull;  // sum g*xh, sum g (g = dy*w), per pair lane
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = tid + k * THREADS;
      const int sidx = idx < nvec ? idx : 0;
      f32x2(&xk)[P] = xh[TWO_PASS ? 0 : k];
      f32x2(&gk)[P] = gy[TWO_PASS ? 0 : k];
      fetch(k, xk, gk);
#pragma unroll
      for (int qq = 0; qq < Q; ++qq) {
        const float4 wv = w4[qq * nvec + sidx];
        const f32x2 wp[2] = {f2_make(wv.x, wv.y), f2_make(wv.z, wv.w)};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int pi = 2 * qq + h;
          const f32x2 g = f2_mul(gk[pi], wp[h]);
          c0 = f2_fma(g, xk[pi], c0);
          if constexpr (LN) c1 = f2_add(c1, g);
        }
      }
    }
    float c[NV];
    {
      float lo, hi;
      f2_split(c0, lo, hi);
      c[0] = lo + hi;
      if constexpr (LN) {
        f2_split(c1, lo, hi);
        c[1] = lo + hi;
      }
    }
    block_allreduce_sum_fixed<NV, THREADS / 32>(c, scratch, phase);  // all done with stage s
    if constexpr (!TWO_PASS)
      if (tid == 0 && i + stages < n_mine) issue(i + stages);
    // dx = rs*g - rs*mean(g) - rs*mean(g*xh)*xh
    const f32x2 a_x = f2_splat(-rs * (c[0] * inv_cols));
    const f32x2 a_0 = f2_splat(LN ? -rs * (c[1] * inv_cols) : 0.f);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = tid + k * THREADS;
      f32x2(&xk)[P] = xh[TWO_PASS ? 0 : k];
      f32x2(&gk)[P] = gy[TWO_PASS ? 0 : k];
      if constexpr (TWO_PASS) fetch(k, xk, gk);
      if (idx < nvec) {
        float o[N];
#pragma unroll
        for (int qq = 0; qq < Q; ++qq) {
          const float4 wv = w4[qq * nvec + idx];
          const f32x2 wp[2] = {f2_make(wv.x, wv.y), f2_make(wv.z, wv.w)};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int pi = 2 * qq + h;
            const f32x2 g = f2_mul(gk[pi], wp[h]);
            const f32x2 op = f2_fma(xk[pi], a_x, f2_fma(g, rs2, a_0));
            f2_split(op, o[2 * pi], o[2 * pi + 1]);
            acc_w[k][pi] = f2_fma(gk[pi], xk[pi], acc_w[k][pi]);
            if constexpr (LN) acc_b[k][pi] = f2_add(acc_b[k][pi], gk[pi]);
          }
        }
        st_vec(dr + (size_t)idx * N, pack<T>(o));
      }
    }
    if constexpr (TWO_PASS) {
      __syncthreads();  // the second pass has read stage s too
      if (tid == 0 && i + stages < n_mine) issue(i + stages);
    }
    dr += row_step;
    if (++s == stages) {
      s = 0;
      parity ^= 1;
    }
  }
  grid_dependents_go();
  // After a timeout every wait above fell through, so the last copies may still be
  // in flight: give them time to land before the block's shared memory is given up.
  if (tid == 0 && *(volatile int*)abort_flag) settle_after_abort();
  // One group per block: the partial row goes out straight from registers.
  float* pw = partial + (size_t)blockIdx.x * cols;
  float* pb = partial + ((size_t)gridDim.x + blockIdx.x) * cols;
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
        if constexpr (LN) {
          f2_split(acc_b[k][2 * qq], a0, a1);
          f2_split(acc_b[k][2 * qq + 1], a2, a3);
          *reinterpret_cast<float4*>(pb + (size_t)idx * N + 4 * qq) = make_float4(a0, a1, a2, a3);
        }
      }
    }
  }
}

// Tile-ring variant for rows of fewer than 256 vectors: consecutive rows are
// contiguous in memory, so one ring stage holds a TILE of R = 256 / G whole rows
// of x and of dy, brought in by two bulk copies; group g of the block (G threads,
// VPT vectors per thread) works on row g of the tile. The bytes in flight per SM
// are set by the ring depth and not by registers or occupancy, which lets a
// thread own 16 or 24 elements of a row (the per-row reduction, barrier and
// statistics are paid once per thread and row) with two blocks per SM, the shape
// that the one-row ring above runs at for wide rows. A thread's columns never
// change, so its weight vectors stay in registers. The one block barrier per
// tile serves the per-group reductions and releases the stage for refilling.
template <typename T, int G, int VPT, bool LN, int THREADS = 256>
__global__ void __launch_bounds__(THREADS,
                                  VPT > 1 ? 2 : (LN && sizeof(T) == 2) ? 3 : 4)
norm_bwd_tile_ring_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                          const T* __restrict__ w, const float* __restrict__ mean,
                          const float* __restrict__ rstd, T* __restrict__ dx,
                          float* __restrict__ partial, int64_t rows, int cols, int stages,
                          long long wait_limit) {
  using namespace umma;
  static_assert(G % 32 == 0 && THREADS % G == 0, "groups are whole warps, blocks whole groups");
  constexpr int WARPS = THREADS / 32;
  constexpr int R = THREADS / G;  // rows per tile
  constexpr int W = G / 32;       // warps per group
  constexpr int N = Vec<T>::N;
  constexpr int P = N / 2;
  constexpr int NV = LN ? 2 : 1;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  const int tid = threadIdx.x;
  const int gid = tid / G, lig = tid % G;
  const int nvec = cols / N;
  const uint32_t row_bytes = (uint32_t)cols * sizeof(T);
  const uint32_t tile_bytes = R * row_bytes;
  // smem: [stages][2][tile_bytes] ring | mbarriers | [2][NV][WARPS] scratch | abort flag
  uint8_t* ring = ring_raw;
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + (size_t)stages * 2 * tile_bytes);
  float* scratch = reinterpret_cast<float*>(full + 16);
  int* abort_flag = reinterpret_cast<int*>(scratch + 2 * NV * WARPS);
  int phase = 0;

  const int64_t n_tiles = (rows + R - 1) / R;
  const int64_t first = blockIdx.x;
  const int64_t n_mine = first < n_tiles ? (n_tiles - first + gridDim.x - 1) / gridDim.x : 0;
  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx ctx{abort_flag, &g_norm_device_status, wait_limit};
  auto issue = [&](int64_t i) {
    const int s = (int)(i % stages);
    const int64_t row0 = (first + i * gridDim.x) * R;
    const int64_t left = rows - row0;
    const uint32_t bytes = (left < R ? (uint32_t)left : (uint32_t)R) * row_bytes;
    uint8_t* dst = ring + (size_t)s * 2 * tile_bytes;
    mbar_expect_tx(&full[s], 2 * bytes);
    bulk_load_1d(dst, x + row0 * cols, bytes, &full[s]);
    bulk_load_1d(dst + tile_bytes, dy + row0 * cols, bytes, &full[s]);
  };
  if (tid == 0)
    for (int64_t i = 0; i < stages && i < n_mine; ++i) issue(i);

  f32x2 wp[VPT][P], acc_w[VPT][P], acc_b[LN ? VPT : 1][P];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int idx = lig + k * G;
    float f[N];
    uint4 wv = make_uint4(0, 0, 0, 0);
    if (idx < nvec) wv = *reinterpret_cast<const uint4*>(w + (size_t)idx * N);
    unpack<T>(wv, f);
#pragma unroll
    for (int j = 0; j < P; ++j) {
      wp[k][j] = f2_make(f[2 * j], f[2 * j + 1]);
      acc_w[k][j] = 0ull;
      if constexpr (LN) acc_b[k][j] = 0ull;
    }
  }
  const float inv_cols = 1.0f / (float)cols;
  const int64_t row_step = (int64_t)gridDim.x * R;
  int64_t row = first * R + gid;
  float rs_next = 0.f, mu_next = 0.f;
  if (n_mine > 0 && row < rows) {
    rs_next = rstd[row];
    if constexpr (LN) mu_next = mean[row];
  }

  int s = 0;
  uint32_t parity = 0;
  for (int64_t i = 0; i < n_mine; ++i) {
    const float rs = rs_next;
    const float nmr = LN ? -mu_next * rs : 0.f;
    const bool row_ok = row < rows;
    rs_next = 0.f;
    if (i + 1 < n_mine && row + row_step < rows) {  // statistics of the next tile's row
      rs_next = rstd[row + row_step];
      if constexpr (LN) mu_next = mean[row + row_step];
    }
    mbar_wait(&full[s], parity, ctx, 402);
    const uint8_t* sx = ring + (size_t)s * 2 * tile_bytes + (size_t)gid * row_bytes;
    const f32x2 rs2 = f2_splat(rs), nmr2 = f2_splat(nmr);
    f32x2 xh[VPT][P], gy[VPT][P];
    f32x2 c0 = 0ull, c1 = 0ull;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      uint4 xv = make_uint4(0, 0, 0, 0), gv = make_uint4(0, 0, 0, 0);
      if (row_ok && idx < nvec) {  // rows past the end and padded lanes count as dy = 0
        xv = *reinterpret_cast<const uint4*>(sx + (size_t)idx * 16);
        gv = *reinterpret_cast<const uint4*>(sx + tile_bytes + (size_t)idx * 16);
      }
      float xf[N], gf[N];
      unpack<T>(xv, xf);
      unpack<T>(gv, gf);
#pragma unroll
      for (int j = 0; j < P; ++j) {
        const f32x2 xp = f2_make(xf[2 * j], xf[2 * j + 1]);
        gy[k][j] = f2_make(gf[2 * j], gf[2 * j + 1]);
        xh[k][j] = LN ? f2_fma(xp, rs2, nmr2) : f2_mul(xp, rs2);
        const f32x2 g = f2_mul(gy[k][j], wp[k][j]);
        c0 = f2_fma(g, xh[k][j], c0);
        if constexpr (LN) c1 = f2_add(c1, g);
      }
    }
    float c[NV];
    {
      float lo, hi;
      f2_split(c0, lo, hi);
      c[0] = lo + hi;
      if constexpr (LN) {
        f2_split(c1, lo, hi);
        c[1] = lo + hi;
      }
    }
    // Sum over the group: shuffles inside a warp, then the group's W warps in a
    // fixed order. Every thread of the block has read its vectors from stage s
    // before it reaches the barrier, so the barrier also frees the stage.
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int v = 0; v < NV; ++v) c[v] += __shfl_xor_sync(0xffffffffu, c[v], off);
    }
    float* buf = scratch + phase * (NV * WARPS);
    if constexpr (W > 1) {
      if ((tid & 31) == 0) {
#pragma unroll
        for (int v = 0; v < NV; ++v) buf[v * WARPS + (tid >> 5)] = c[v];
      }
    }
    __syncthreads();
    if constexpr (W > 1) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        float sum = buf[v * WARPS + gid * W];
#pragma unroll
        for (int q = 1; q < W; ++q) sum += buf[v * WARPS + gid * W + q];
        c[v] = sum;
      }
      phase ^= 1;
    }
    if (tid == 0 && i + stages < n_mine) issue(i + stages);
    // dx = rs*g - rs*mean(g) - rs*mean(g*xh)*xh
    const f32x2 a_x = f2_splat(-rs * (c[0] * inv_cols));
    const f32x2 a_0 = f2_splat(LN ? -rs * (c[1] * inv_cols) : 0.f);
    T* dr = dx + row * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      float o[N];
#pragma unroll
      for (int j = 0; j < P; ++j) {
        const f32x2 g = f2_mul(gy[k][j], wp[k][j]);
        const f32x2 op = f2_fma(xh[k][j], a_x, f2_fma(g, rs2, a_0));
        f2_split(op, o[2 * j], o[2 * j + 1]);
        acc_w[k][j] = f2_fma(gy[k][j], xh[k][j], acc_w[k][j]);
        if constexpr (LN) acc_b[k][j] = f2_add(acc_b[k][j], gy[k][j]);
      }
      if (row_ok && idx < nvec) st_vec(dr + (size_t)idx * N, pack<T>(o));
    }
    row += row_step;
    if (++s == stages) {
      s = 0;
      parity ^= 1;
    }
  }
  grid_dependents_go();
  if (tid == 0 && *(volatile int*)abort_flag) settle_after_abort();
  __syncthreads();
  // Every copy has landed and been read: the ring now holds the [NV][cols] float32
  // column buffer in which the block's groups are folded in group order.
  float* colbuf = reinterpret_cast<float*>(ring);
  for (int g = 0; g < R; ++g) {
    if (gid == g) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int idx = lig + k * G;
        if (idx < nvec) {
#pragma unroll
          for (int j = 0; j < P; ++j) {
            float a0, a1;
            f2_split(acc_w[k][j], a0, a1);
            float* cw = colbuf + (size_t)idx * N + 2 * j;
            if (g == 0) {
              cw[0] = a0;
              cw[1] = a1;
            } else {
              cw[0] += a0;
              cw[1] += a1;
            }
            if constexpr (LN) {
              f2_split(acc_b[k][j], a0, a1);
              float* cb = cw + cols;
              if (g == 0) {
                cb[0] = a0;
                cb[1] = a1;
              } else {
                cb[0] += a0;
                cb[1] += a1;
              }
            }
          }
        }
      }
    }
    __syncthreads();
  }
  float* pw = partial + (size_t)blockIdx.x * cols;
  for (int c = tid; c < cols; c += THREADS) {
    pw[c] = colbuf[c];
    if constexpr (LN) pw[(size_t)gridDim.x * cols + c] = colbuf[cols + c];
  }
}

// Any width / alignment. One block per row at a time; the block's partial row
// in the workspace is private to it, so plain read-modify-write is race free.
template <typename T, bool LN>
__global__ void __launch_bounds__(1024, 1)
norm_bwd_generic_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                        const T* __restrict__ w, const float* __restrict__ mean,
                        const float* __restrict__ rstd, T* __restrict__ dx,
                        float* __restrict__ partial, int64_t rows, int64_t cols) {
  constexpr int NV = LN ? 2 : 1;
  __shared__ float scratch[2 * NV * 32];
  int phase = 0;
  const float inv_cols = 1.0f / (float)cols;
  float* pw = partial + (size_t)blockIdx.x * cols;
  float* pb = partial + ((size_t)gridDim.x + blockIdx.x) * cols;
  bool first = true;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    const T* gr = dy + row * cols;
    const float rs = rstd[row];
    float mu = 0.f;
    if constexpr (LN) mu = mean[row];
    float c[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) c[i] = 0.f;
    for (int64_t col = threadIdx.x; col < cols; col += blockDim.x) {
      const float xh = (to_f32<T>(xr[col]) - mu) * rs;
      const float g = to_f32<T>(gr[col]) * to_f32<T>(w[col]);
      c[0] += g * xh;
      if constexpr (LN) c[1] += g;
    }
    block_allreduce<NV, SumOp>(c, scratch, phase);
    const float m_gx = c[0] * inv_cols;
    float m_g = 0.f;
    if constexpr (LN) m_g = c[1] * inv_cols;
    T* dr = dx + row * cols;
    for (int64_t col = threadIdx.x; col < cols; col += blockDim.x) {
      const float gy = to_f32<T>(gr[col]);
      const float xh = (to_f32<T>(xr[col]) - mu) * rs;
      const float g = gy * to_f32<T>(w[col]);
      dr[col] = from_f32<T>((g - m_g - xh * m_gx) * rs);
      if (first) {
        pw[col] = gy * xh;
        if constexpr (LN) pb[col] = gy;
      } else {
        pw[col] += gy * xh;
        if constexpr (LN) pb[col] += gy;
      }
    }
    first = false;
  }
}

int read_norm_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_norm_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_norm_device_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_norm_status_registered = (register_device_status(read_norm_status), true);

// The fewest blocks that walk `rows` (in tiles of `per_tile`) in the same number of rounds as
// `blocks` would: every round is then full. Measured on the tile ring ([65536, 1024] bf16:
// RMSNorm backward 65.3 -> 63.1 us, LayerNorm 71.8 -> 71.0 us); on the one-row ring and the
// forward kernels the same choice was neutral or slower, so they keep the full count.
inline int even_rounds(int blocks, int64_t rows, int per_tile) {
  const int64_t tiles = (rows + per_tile - 1) / per_tile;
  if (blocks < 1 || tiles <= blocks) return blocks;
  const int64_t rounds = (tiles + blocks - 1) / blocks;
  return (int)((tiles + rounds - 1) / rounds);
}

struct BwdPlan {
  bool generic = false;
  RowCfg cfg;
  int blocks = 0;
  size_t smem = 0;
};

// `block_limit` > 0 bounds the number of partial rows (callers with a fixed scratch).
template <typename T, bool LN>
int64_t norm_bwd_workspace(int64_t rows, int64_t hidden, int64_t block_limit = 0) {
  int64_t blocks = max_partial_blocks(hidden);
  if (block_limit > 0 && blocks > block_limit) blocks = block_limit;
  if (blocks > rows) blocks = rows > 0 ? rows : 1;
  return blocks * hidden * (LN ? 2 : 1) * (int64_t)sizeof(float);
}

template <typename T, bool LN>
int launch_norm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                    const float* rstd, void* dx, void* dweight, void* dbias, float* out_f32,
                    void* workspace, int64_t workspace_bytes, int64_t rows, int64_t hidden,
                    cudaStream_t stream, int64_t block_limit = 0, evg_exchange* xchg = nullptr) {
  constexpr int N = Vec<T>::N;
  constexpr int NV = LN ? 2 : 1;
  const char* op = LN ? "layernorm_bwd" : "rmsnorm_bwd";
  const int64_t need = norm_bwd_workspace<T, LN>(rows, hidden, block_limit);
  if (!workspace || workspace_bytes < need)
    return fail(EVG_EWORKSPACE, "%s: workspace %lld bytes, need %lld", op,
                (long long)workspace_bytes, (long long)need);
  if (!aligned16(workspace)) return fail(EVG_EALIGN, "%s: workspace not 16-byte aligned", op);
  float* partial = (float*)workspace;
  int cap = max_partial_blocks(hidden);
  if (block_limit > 0 && cap > block_limit) cap = (int)block_limit;
  int blocks = 0;
  const bool vec_ok = hidden % N == 0 && aligned16(x) && aligned16(dy) && aligned16(dx) &&
                      aligned16(w) && hidden < (int64_t)1 << 31;
  RowCfg cfg;
  bool launched = false;
  // Rows of fewer than 256 vectors (under 4 KB) would leave half of a one-row ring
  // block's threads idle and pay its per-row barriers for little data: they go to
  // the tile ring below, several rows per stage.
  const bool narrow_rows = vec_ok && hidden / N < 256;
  if (vec_ok && !narrow_rows && !tune("rows.force_generic") && !tune("norm_bwd.no_ring") &&
      !tune(LN ? "layernorm_bwd.group" : "rmsnorm_bwd.group")) {
    // Row ring: one group of 256 or 512 threads per block, VPT vectors per
    // thread, as many stages as fit (about 48 KB of rows in flight per block).
    const int64_t nvec = hidden / N;
    // Rows of 257 ... 384 vectors would leave a quarter of a 256-thread block's lanes idle:
    // they run on 128-thread blocks with three vectors per thread, four blocks per SM for
    // LayerNorm and three for RMSNorm ([32768, 3072] bf16: LayerNorm backward 109.9 -> 101.5 us,
    // RMSNorm 96.6 -> 94.3 us; the same idea with five vectors per thread at 640 vectors was
    // slower, 54 -> 60 us).
    int ring_threads = tune("norm_bwd.ring_threads");
    if (ring_threads == 0 && nvec > 256 && nvec <= 384) ring_threads = 128;
    if (ring_threads != 128 && ring_threads != 256 && ring_threads != 512) ring_threads = 256;
    const size_t row_bytes = (size_t)hidden * sizeof(T);
    const size_t fixed = (size_t)hidden * sizeof(float) + 16 * 8 + 2 * NV * 32 * sizeof(float) + 64;
    const size_t budget = (size_t)device_info().max_smem_optin;
    int stages = tune("norm_bwd.stages");
    // About 48 KB of rows in flight per block, and three stages where they fit
    // ([4096, 8192] bf16: LayerNorm 46.4 -> 43.7 us, RMSNorm 41.0 -> 37.1 us against two).
    if (stages <= 0) stages = (int)(((ring_threads == 128 ? 24 : 48) * 1024) / (2 * row_bytes));
    if (stages < (ring_threads == 128 ? 2 : 3)) stages = ring_threads == 128 ? 2 : 3;
    if (stages > 12) stages = 12;
    while (stages > 0 && fixed + (size_t)stages * 2 * row_bytes > budget) --stages;
    long long wait_limit = 2000000000ll;
    int ring_cap = cap;
    if (ring_threads == 128 && !LN && ring_cap > 3 * device_info().sm_count)
      ring_cap = 3 * device_info().sm_count;
    if (stages >= 2 && nvec <= 8 * ring_threads) {  // (the budget loop above may leave two)
      const size_t smem = fixed + (size_t)stages * 2 * row_bytes;
#define EVG_RING(t, v)                                                                           \
  if (!launched && ring_threads == t && nvec <= (int64_t)v * t) {                                \
    auto kern = norm_bwd_ring_kernel<T, t, v, LN>;                                               \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    blocks = persistent_grid(kern, t, smem, rows, 1, ring_cap);                                  \
    kern<<<blocks, t, smem, stream>>>((const T*)dy, (const T*)x, (const T*)w, mean, rstd,        \
                                      (T*)dx, partial, rows, (int)hidden, stages, wait_limit);   \
    launched = true;                                                                             \
  }
      EVG_RING(256, 1) EVG_RING(256, 2) EVG_RING(256, 3) EVG_RING(256, 4) EVG_RING(256, 6)
      EVG_RING(256, 8)
      EVG_RING(512, 1) EVG_RING(512, 2) EVG_RING(512, 4) EVG_RING(512, 8)
      EVG_RING(128, 3)
#undef EVG_RING
    }
  }
  // Tile ring for narrow rows (`norm_bwd.tile_ring` = 2 switches it off). Shape: up to 32
  // vectors, one per thread of a warp; above, two (float32: or three) vectors per thread on
  // the smallest group that holds the row. Measured on bf16, fraction of the copy bandwidth,
  // group kernels -> tile ring: [65536, 1024] LayerNorm 0.70 -> 0.85, RMSNorm 0.85 -> 0.92;
  // [49152, 1536] 0.72 -> 0.85, 0.85 -> 0.91; [131072, 512] 0.71 -> 0.83, 0.75 -> 0.91;
  // [32768, 2040] 0.64 -> 0.86, 0.79 -> 0.96.
  if (narrow_rows && !launched && tune("norm_bwd.tile_ring") != 2 &&
      !tune("rows.force_generic") && !tune("norm_bwd.no_ring") &&
      !tune(LN ? "layernorm_bwd.group" : "rmsnorm_bwd.group")) {
    const int nv = (int)(hidden / N);
    int G = 32, V = 1, threads = 256;
    if (nv > 128 && nv <= 192) {  // 96-thread groups, two vectors each: no idle lanes
      G = 96;
      V = 2;
      threads = 192;  // (288 threads would leave 96 registers per thread: spills)
    } else if (nv > 32) {
      int best = 1 << 30;
      for (int v = 2; v <= (sizeof(T) == 4 ? 3 : 2); ++v) {  // three 16-bit vectors spill
        int g = 32;
        while (g * v < nv) g *= 2;
        if (g * v < best) {
          best = g * v;
          G = g;
          V = v;
        }
      }
    }
    const size_t tile_pair = (size_t)2 * (threads / G) * hidden * sizeof(T);
    int stages = tune("norm_bwd.stages");
    // Ring bytes per block: two blocks of 48 KB, four of 40 KB, or three of 56 KB per SM
    // (one 16-bit LayerNorm vector per thread needs ~70 registers).
    const bool three = V == 1 && LN && sizeof(T) == 2;
    if (stages <= 0) stages = (int)(((V > 1 ? 48 : three ? 56 : 40) * 1024) / tile_pair);
    if (stages < 2) stages = 2;
    if (stages > 12) stages = 12;
    const size_t smem = (size_t)stages * tile_pair + 16 * 8 + 2 * NV * 16 * sizeof(float) + 64;
    const long long wait_limit = 2000000000ll;
#define EVG_TR(g, v, t)                                                                        \
  if (!launched && G == g && V == v && threads == t) {                                         \
    auto kern = norm_bwd_tile_ring_kernel<T, g, v, LN, t>;                                     \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
    blocks = even_rounds(persistent_grid(kern, t, smem, rows, t / g, cap), rows, t / g);       \
    kern<<<blocks, t, smem, stream>>>((const T*)dy, (const T*)x, (const T*)w, mean, rstd,      \
                                      (T*)dx, partial, rows, (int)hidden, stages, wait_limit); \
    launched = true;                                                                           \
  }
    EVG_TR(32, 1, 256)
    EVG_TR(32, 2, 256) EVG_TR(64, 2, 256) EVG_TR(128, 2, 256)
    EVG_TR(96, 2, 192)
    if constexpr (sizeof(T) == 4) {
      EVG_TR(32, 3, 256)
    }
#undef EVG_TR
  }
  if (!launched && vec_ok && !tune("rows.force_generic") &&
      pick_rowcfg(op, hidden / N, cfg, narrow_rows ? 256 : 512, LN)) {
    const int groups = cfg.threads / cfg.G;
    const size_t smem =
        ((size_t)groups * 2 * NV * (cfg.G / 32) + (size_t)(NV + 1) * hidden) * sizeof(float);
    if (smem <= (size_t)device_info().max_smem_optin) {
#define EVG_X(g, v)                                                                            \
  if (!launched && cfg.G == g && cfg.VPT == v) {                                               \
    auto kern = norm_bwd_kernel<T, g, v, LN>;                                                  \
    if (smem > 48 * 1024)                                                                      \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    blocks = persistent_grid(kern, cfg.threads, smem, rows, groups, cap);                      \
    kern<<<blocks, cfg.threads, smem, stream>>>((const T*)dy, (const T*)x, (const T*)w, mean,  \
                                                rstd, (T*)dx, partial, rows, (int)hidden);     \
    launched = true;                                                                           \
  }
      EVG_ROWCFG_LIST(EVG_X)
#undef EVG_X
    }
  }
  if (!launched) {
    auto kern = norm_bwd_generic_kernel<T, LN>;
    const int threads = hidden >= 2048 ? 1024 : (hidden >= 256 ? 256 : 64);
    blocks = persistent_grid(kern, threads, 0, rows, 1, cap);
    kern<<<blocks, threads, 0, stream>>>((const T*)dy, (const T*)x, (const T*)w, mean, rstd,
                                         (T*)dx, partial, rows, hidden);
  }
  int rc = check_launch(op);
  if (rc) return rc;
  if ((int64_t)blocks * hidden * NV * (int64_t)sizeof(float) > workspace_bytes)
    return fail(EVG_EWORKSPACE, "%s: internal: partial rows exceed workspace", op);
  if (xchg) {
    // stage 2 and the sum over ranks in one kernel
    dim3 grid((unsigned)((hidden + 31) / 32), NV);
    int* status = nullptr;
    cudaGetSymbolAddress((void**)&status, g_norm_device_status);
    // a programmatic dependent of the row kernel, like the single-GPU stage 2
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(32, 32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tune("norm_bwd.no_pdl") ? 0 : 1;
    cudaLaunchKernelEx(&cfg, colreduce_exchange_kernel<T>, (const float*)partial, blocks,
                       (int64_t)hidden, (T*)dweight, (T*)dbias, xchg->peers, xchg->lay,
                       xchg->n_ranks, xchg->rank, xchg->wait_limit, status);
    return check_launch("norm_bwd colreduce + exchange");
  }
  if (dweight || dbias || out_f32) {
    launch_colreduce<T>(partial, blocks, hidden, (T*)dweight, (T*)dbias, out_f32, NV, stream);
    rc = check_launch("norm_bwd colreduce");
  }
  return rc;
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int64_t evg_layernorm_bwd_workspace_bytes(int64_t rows, int64_t hidden, int dtype) {
  (void)dtype;
  if (rows < 0 || hidden <= 0) return 0;
  return norm_bwd_workspace<float, true>(rows, hidden);
}

extern "C" int64_t evg_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t hidden, int dtype) {
  (void)dtype;
  if (rows < 0 || hidden <= 0) return 0;
  return norm_bwd_workspace<float, false>(rows, hidden);
}

extern "C" int evg_layernorm_bwd(const void* dy, const void* x, const void* weight,
                                 const float* mean, const float* rstd, void* dx, void* dweight,
                                 void* dbias, float* dwdb_f32, void* workspace,
                                 int64_t workspace_bytes, int64_t rows, int64_t hidden, int dtype,
                                 void* stream) {
  if (!dy || !x || !weight || !mean || !rstd || !dx)
    return fail(EVG_ENULL, "layernorm_bwd: null pointer argument");
  if (rows <= 0 || hidden <= 0)
    return fail(EVG_EBADSHAPE, "layernorm_bwd: rows=%lld hidden=%lld (rows must be >= 1)",
                (long long)rows, (long long)hidden);
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_norm_bwd<T, true>(dy, x, weight, mean, rstd, dx, dweight, dbias, dwdb_f32,
                                    workspace, workspace_bytes, rows, hidden,
                                    (cudaStream_t)stream);
  });
}

extern "C" int evg_rmsnorm_bwd(const void* dy, const void* x, const void* weight,
                               const float* rstd, void* dx, void* dweight, float* dweight_f32,
                               void* workspace, int64_t workspace_bytes, int64_t rows,
                               int64_t hidden, int dtype, void* stream) {
  if (!dy || !x || !weight || !rstd || !dx)
    return fail(EVG_ENULL, "rmsnorm_bwd: null pointer argument");
  if (rows <= 0 || hidden <= 0)
    return fail(EVG_EBADSHAPE, "rmsnorm_bwd: rows=%lld hidden=%lld (rows must be >= 1)",
                (long long)rows, (long long)hidden);
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_norm_bwd<T, false>(dy, x, weight, nullptr, rstd, dx, dweight, nullptr,
                                     dweight_f32, workspace, workspace_bytes, rows, hidden,
                                     (cudaStream_t)stream);
  });
}

// ------------------------------------------------------------------------
// Backward over a row shard with the parameter gradients summed over the ranks
// of an exchange (one process per GPU): stage 2 of the column reduction and the
// cross-GPU sum are one kernel.
namespace {
int check_exchange(const char* op, const evg_exchange* x, int64_t hidden, int nv) {
  if (!x) return fail(EVG_ENULL, "%s: null exchange handle", op);
  if (!x->connected) return fail(EVG_EUNSUPPORTED, "%s: the exchange's peers are not connected", op);
  if ((int64_t)nv * hidden > x->lay.max_floats)
    return fail(EVG_EUNSUPPORTED, "%s: %lld values exceed the exchange buffer (%lld)", op,
                (long long)((int64_t)nv * hidden), (long long)x->lay.max_floats);
  if ((hidden + 31) / 32 * nv > xchg::kMaxBlocks)
    return fail(EVG_EUNSUPPORTED, "%s: hidden=%lld needs more than %d exchange blocks", op,
                (long long)hidden, xchg::kMaxBlocks);
  return EVG_OK;
}
}  // namespace

extern "C" int evg_layernorm_bwd_exchange(const void* dy, const void* x, const void* weight,
                                          const float* mean, const float* rstd, void* dx,
                                          void* dweight, void* dbias, void* workspace,
                                          int64_t workspace_bytes, int64_t rows, int64_t hidden,
                                          int dtype, evg_exchange* exchange, void* stream) {
  if (!dy || !x || !weight || !mean || !rstd || !dx || !dweight || !dbias)
    return fail(EVG_ENULL, "layernorm_bwd_exchange: null pointer argument");
  if (rows <= 0 || hidden <= 0)
    return fail(EVG_EBADSHAPE, "layernorm_bwd_exchange: rows=%lld hidden=%lld (rows must be >= 1)",
                (long long)rows, (long long)hidden);
  if (int rc = check_exchange("layernorm_bwd_exchange", exchange, hidden, 2)) return rc;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_norm_bwd<T, true>(dy, x, weight, mean, rstd, dx, dweight, dbias, nullptr,
                                    workspace, workspace_bytes, rows, hidden,
                                    (cudaStream_t)stream, 0, exchange);
  });
}

extern "C" int evg_rmsnorm_bwd_exchange(const void* dy, const void* x, const void* weight,
                                        const float* rstd, void* dx, void* dweight,
                                        void* workspace, int64_t workspace_bytes, int64_t rows,
                                        int64_t hidden, int dtype, evg_exchange* exchange,
                                        void* stream) {
  if (!dy || !x || !weight || !rstd || !dx || !dweight)
    return fail(EVG_ENULL, "rmsnorm_bwd_exchange: null pointer argument");
  if (rows <= 0 || hidden <= 0)
    return fail(EVG_EBADSHAPE, "rmsnorm_bwd_exchange: rows=%lld hidden=%lld (rows must be >= 1)",
                (long long)rows, (long long)hidden);
  if (int rc = check_exchange("rmsnorm_bwd_exchange", exchange, hidden, 1)) return rc;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_norm_bwd<T, false>(dy, x, weight, nullptr, rstd, dx, dweight, nullptr, nullptr,
                                     workspace, workspace_bytes, rows, hidden,
                                     (cudaStream_t)stream, 0, exchange);
  });
}

// ------------------------------------------------------------------------
// RMSNorm backward for callers that cannot obtain device memory.
//
// The partial-sum rows of the two-stage dweight reduction live in a fixed array
// that is part of the library image, so this entry point performs no device
// allocation of any kind. See the header for the limits and the sharing rules.
namespace {

constexpr int64_t kNoAllocMaxHidden = 8192;
constexpr int64_t kNoAllocMaxBlocks = 320;
constexpr int64_t kNoAllocFloats = kNoAllocMaxBlocks * kNoAllocMaxHidden;  // 10 MiB

static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats];

std::mutex g_noalloc_mutex;
float* g_noalloc_ptr[64] = {};  // device address of the array, per device ordinal

// In host code the array's name only stands for the symbol; the address a kernel
// can use has to be asked for, once per device, with that device current.
int noalloc_scratch_address(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(EVG_ELAUNCH, "rmsnorm_bwd_noalloc: cannot identify the current device");
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (err != cudaSuccess || !p) {
      cudaGetLastError();
      return fail(EVG_ELAUNCH, "rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s",
                  cudaGetErrorString(err));
    }
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return EVG_OK;
}

}  // namespace

extern "C" int evg_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* weight,
                                       const float* rstd, void* dx, void* dweight,
                                       float* dweight_f32, int64_t rows, int64_t hidden,
                                       int dtype, void* stream) {
  if (!dy || !x || !weight || !rstd || !dx)
    return fail(EVG_ENULL, "rmsnorm_bwd_noalloc: null pointer argument");
  if (rows <= 0 || hidden <= 0)
    return fail(EVG_EBADSHAPE, "rmsnorm_bwd_noalloc: rows=%lld hidden=%lld (rows must be >= 1)",
                (long long)rows, (long long)hidden);
  if (hidden > kNoAllocMaxHidden)
    return fail(EVG_EUNSUPPORTED,
                "rmsnorm_bwd_noalloc: hidden=%lld exceeds the built-in scratch (max hidden %lld); "
                "use evg_rmsnorm_bwd with a caller-provided workspace",
                (long long)hidden, (long long)kNoAllocMaxHidden);
  const int64_t block_limit = kNoAllocFloats / hidden;  // >= kNoAllocMaxBlocks
  const int64_t need = norm_bwd_workspace<float, false>(rows, hidden, block_limit);
  const int64_t have = kNoAllocFloats * (int64_t)sizeof(float);
  if (need > have)
    return fail(EVG_EUNSUPPORTED,
                "rmsnorm_bwd_noalloc: this launch shape needs %lld bytes of partial sums, the "
                "built-in scratch holds %lld (at most %lld partial rows of %lld floats)",
                (long long)need, (long long)have, (long long)kNoAllocMaxBlocks,
                (long long)kNoAllocMaxHidden);
  float* scratch = nullptr;
  if (int rc = noalloc_scratch_address(&scratch)) return rc;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_norm_bwd<T, false>(dy, x, weight, nullptr, rstd, dx, dweight, nullptr,
                                     dweight_f32, scratch, have, rows, hidden,
                                     (cudaStream_t)stream, block_limit);
  });
}
