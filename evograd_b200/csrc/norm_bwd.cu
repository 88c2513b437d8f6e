// LayerNorm / RMSNorm backward for sm_100a.
//
// HBM-bound: reads x and dy once, writes dx once. dweight/dbias are column sums
// over every row; they are formed in two stages without atomics:
//   stage 1  each persistent block keeps float32 column sums of its own rows in
//            registers and writes ONE partial row per block to the workspace;
//   stage 2  a small kernel adds the partial rows in a fixed order and rounds.
// The result is bit-reproducible from run to run for a given launch shape.
#include "rowcfg.cuh"

namespace evg {
namespace {

// Workspace layout (float32): [NP][blocks][cols], NP = 2 (dweight, dbias) for
// LayerNorm and 1 (dweight) for RMSNorm.
template <typename T, int G, int VPT, bool LN>
__global__ void __launch_bounds__(rowcfg_max_threads(G))
norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                const float* __restrict__ mean, const float* __restrict__ rstd,
                T* __restrict__ dx, float* __restrict__ partial, int64_t rows, int cols) {
  constexpr int N = Vec<T>::N;
  constexpr int NV = LN ? 2 : 1;
  extern __shared__ float smem[];
  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int groups = blockDim.x / G;
  const int nvec = cols / N;
  // smem: [groups][2][NV][G/32] reduction scratch, then [NV][cols] column buffer
  float* scratch = smem + gid * (2 * NV * (G / 32));
  float* colbuf = smem + groups * (2 * NV * (G / 32));
  int phase = 0;

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
  const int64_t stride = (int64_t)gridDim.x * groups;

  // Software pipeline: the loads of the next row are issued before the current
  // row is reduced, so x/dy requests stay in flight through the whole loop body.
  int64_t row = (int64_t)blockIdx.x * groups + gid;
  uint4 xv[VPT], gv[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int idx = lig + k * G;
    xv[k] = make_uint4(0, 0, 0, 0);
    gv[k] = make_uint4(0, 0, 0, 0);
    if (row < rows && idx < nvec) {
      xv[k] = ld_vec(x + row * cols + (size_t)idx * N);
      gv[k] = ld_vec(dy + row * cols + (size_t)idx * N);
    }
  }
  while (row < rows) {
    const int64_t nrow = row + stride;
    uint4 xn[VPT], gn[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      xn[k] = make_uint4(0, 0, 0, 0);
      gn[k] = make_uint4(0, 0, 0, 0);
      if (nrow < rows && idx < nvec) {
        xn[k] = ld_vec(x + nrow * cols + (size_t)idx * N);
        gn[k] = ld_vec(dy + nrow * cols + (size_t)idx * N);
      }
    }
    const float rs = rstd[row];
    float mu = 0.f;
    if constexpr (LN) mu = mean[row];

    // c[0] = sum g*xhat, c[1] = sum g  (g = dy*w; padded vectors contribute 0)
    float c[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) c[i] = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      if (idx < nvec) {
        float xf[N], gf[N], wf[N];
        unpack<T>(xv[k], xf);
        unpack<T>(gv[k], gf);
        unpack<T>(__ldg(reinterpret_cast<const uint4*>(w + (size_t)idx * N)), wf);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float xh = (xf[j] - mu) * rs;
          const float g = gf[j] * wf[j];
          c[0] += g * xh;
          if constexpr (LN) c[1] += g;
        }
      }
    }
    group_allreduce<G, NV, SumOp>(c, scratch, phase, gid, lig);
    const float m_gx = c[0] * inv_cols;
    float m_g = 0.f;
    if constexpr (LN) m_g = c[1] * inv_cols;

    T* dr = dx + row * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = lig + k * G;
      if (idx < nvec) {
        float xf[N], gf[N], wf[N], o[N];
        unpack<T>(xv[k], xf);
        unpack<T>(gv[k], gf);
        unpack<T>(__ldg(reinterpret_cast<const uint4*>(w + (size_t)idx * N)), wf);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float xh = (xf[j] - mu) * rs;
          const float g = gf[j] * wf[j];
          o[j] = (g - m_g - xh * m_gx) * rs;
          acc_w[k][j] += gf[j] * xh;
          if constexpr (LN) acc_b[k][j] += gf[j];
        }
        st_vec(dr + (size_t)idx * N, pack<T>(o));
      }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      xv[k] = xn[k];
      gv[k] = gn[k];
    }
    row = nrow;
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

// Stage 2: out[c] = sum_p partial[p][c], p ascending inside each of 16 strided
// slices, slices then added in order. gridDim.y selects dweight / dbias.
template <typename T>
__global__ void __launch_bounds__(512)
colreduce_kernel(const float* __restrict__ partial, int blocks, int64_t cols, T* out_w, T* out_b,
                 float* out_f32) {
  __shared__ float tile[16][33];
  const int which = blockIdx.y;
  const float* src = partial + (size_t)which * blocks * cols;
  const int64_t col = (int64_t)blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (col < cols) {
    for (int p = threadIdx.y; p < blocks; p += 16) s += src[(size_t)p * cols + col];
  }
  tile[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && col < cols) {
    float t = tile[0][threadIdx.x];
#pragma unroll
    for (int i = 1; i < 16; ++i) t += tile[i][threadIdx.x];
    T* out = which == 0 ? out_w : out_b;
    if (out) out[col] = from_f32<T>(t);
    if (out_f32) out_f32[(size_t)which * cols + col] = t;
  }
}

struct BwdPlan {
  bool generic = false;
  RowCfg cfg;
  int blocks = 0;
  size_t smem = 0;
};

int max_partial_blocks() {
  int per_sm = tune("norm_bwd.blocks_per_sm");
  if (per_sm <= 0) per_sm = 2;
  return device_info().sm_count * per_sm;
}

template <typename T, bool LN>
int64_t norm_bwd_workspace(int64_t rows, int64_t hidden) {
  int64_t blocks = max_partial_blocks();
  if (blocks > rows) blocks = rows > 0 ? rows : 1;
  return blocks * hidden * (LN ? 2 : 1) * (int64_t)sizeof(float);
}

template <typename T, bool LN>
int launch_norm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                    const float* rstd, void* dx, void* dweight, void* dbias, float* out_f32,
                    void* workspace, int64_t workspace_bytes, int64_t rows, int64_t hidden,
                    cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  constexpr int NV = LN ? 2 : 1;
  const char* op = LN ? "layernorm_bwd" : "rmsnorm_bwd";
  const int64_t need = norm_bwd_workspace<T, LN>(rows, hidden);
  if (!workspace || workspace_bytes < need)
    return fail(EVG_EWORKSPACE, "%s: workspace %lld bytes, need %lld", op,
                (long long)workspace_bytes, (long long)need);
  if (!aligned16(workspace)) return fail(EVG_EALIGN, "%s: workspace not 16-byte aligned", op);
  float* partial = (float*)workspace;
  const int cap = max_partial_blocks();
  int blocks = 0;
  const bool vec_ok = hidden % N == 0 && aligned16(x) && aligned16(dy) && aligned16(dx) &&
                      aligned16(w) && hidden < (int64_t)1 << 31;
  RowCfg cfg;
  bool launched = false;
  if (vec_ok && !tune("rows.force_generic") && pick_rowcfg(op, hidden / N, cfg, 512, LN)) {
    const int groups = cfg.threads / cfg.G;
    const size_t smem =
        ((size_t)groups * 2 * NV * (cfg.G / 32) + (size_t)NV * hidden) * sizeof(float);
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
  if (dweight || dbias || out_f32) {
    dim3 grid((unsigned)((hidden + 31) / 32), NV);
    colreduce_kernel<T><<<grid, dim3(32, 16), 0, stream>>>(partial, blocks, hidden, (T*)dweight,
                                                           (T*)dbias, out_f32);
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
