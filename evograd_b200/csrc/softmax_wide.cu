// Row softmax forward/backward for rows too wide for one block's registers
// (vocabulary-sized logits: 128256 columns = 250 KB in bf16), for sm_100a.
//
// One thread-block CLUSTER per row: each of the C blocks (C = 2, 4 or 8) stages
// its slice of the row in shared memory with bulk async copies (an mbarrier
// counts the bytes), reduces its slice, and the blocks exchange their partial
// (max, sum) through distributed shared memory with one cluster barrier per
// row. The row is read from HBM exactly once and written once, independent of
// what L2 keeps. Several blocks of different clusters share an SM, so one
// block's load overlaps another's arithmetic (a second stage per block is
// available through the `softmax.cluster_stages` knob).
//
//   forward : m = max x, S = sum exp(x - m), y = exp(x - m) / S
//             (float32, one cast: ops/level1/softmax/forward_ref.py:6-7)
//   backward: dx = y * (dy - sum(dy * y))      (saved state = y only)
#include <cooperative_groups.h>

#include "evg_common.cuh"
#include "sm100_umma.cuh"
#include "softmax_wide.cuh"

namespace cg = cooperative_groups;

namespace evg {
namespace {

constexpr int kMaxCluster = 8;  // the portable maximum (16 was measured slower)
constexpr float kLog2eW = 1.4426950408889634f;

// Sticky status of the bounded waits in this file (0 = fine).
__device__ int g_softmax_wide_status = 0;

struct WideSmem {
  uint64_t full[2];
  float2 slots[2][kMaxCluster];  // [row parity][source block]: partial (max, sum)
  float scratch[2 * 32];
  int abort_flag;
};

// `a` is x (forward) or y (backward); `b` is dy (backward only).
template <typename T, bool BWD, int kWideThreads>
__global__ void __launch_bounds__(kWideThreads)
softmax_wide_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                    int64_t rows, int64_t cols, int nvec, int vec_per_block, int stages,
                    long long wait_limit) {
  using namespace umma;
  constexpr int N = Vec<T>::N;
  constexpr int NIN = BWD ? 2 : 1;
  extern __shared__ __align__(128) uint8_t wide_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x;
  const int64_t cid = blockIdx.x / C;
  const int64_t n_clusters = gridDim.x / C;

  const int first_vec = rank * vec_per_block;
  int my_nvec = nvec - first_vec;
  if (my_nvec > vec_per_block) my_nvec = vec_per_block;
  if (my_nvec < 0) my_nvec = 0;
  const uint32_t slice_bytes = (uint32_t)my_nvec * 16u;
  const size_t stage_bytes = (size_t)NIN * vec_per_block * 16;
  uint8_t* buf = wide_raw;
  WideSmem* sm = reinterpret_cast<WideSmem*>(wide_raw + (size_t)stages * stage_bytes);
  int phase = 0;

  if (tid == 0) {
    sm->abort_flag = 0;
    for (int s = 0; s < stages; ++s) mbar_init(&sm->full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx ctx{&sm->abort_flag, &g_softmax_wide_status, wait_limit};
  const int64_t n_mine = cid < rows ? (rows - cid + n_clusters - 1) / n_clusters : 0;

  auto issue = [&](int64_t i) {  // thread 0 only
    if (my_nvec == 0) return;
    const int s = (int)(i % stages);
    const int64_t row = cid + i * n_clusters;
    uint8_t* dst = buf + (size_t)s * stage_bytes;
    mbar_expect_tx(&sm->full[s], NIN * slice_bytes);
    // pieces of at most 32 KB
    for (uint32_t off = 0; off < slice_bytes; off += 32768u) {
      const uint32_t n = slice_bytes - off < 32768u ? slice_bytes - off : 32768u;
      bulk_load_1d(dst + off, reinterpret_cast<const uint8_t*>(a + row * cols) +
                                  (size_t)first_vec * 16 + off, n, &sm->full[s]);
      if constexpr (BWD)
        bulk_load_1d(dst + (size_t)vec_per_block * 16 + off,
                     reinterpret_cast<const uint8_t*>(b + row * cols) + (size_t)first_vec * 16 +
                         off, n, &sm->full[s]);
    }
  };
  if (tid == 0)
    for (int64_t i = 0; i < stages && i < n_mine; ++i) issue(i);

  int s = 0;
  uint32_t parity = 0;
  for (int64_t i = 0; i < n_mine; ++i) {
    const int64_t row = cid + i * n_clusters;
    if (my_nvec > 0) mbar_wait(&sm->full[s], parity, ctx, 421);
    const uint4* sa = reinterpret_cast<const uint4*>(buf + (size_t)s * stage_bytes);
    const uint4* sb = sa + vec_per_block;
    const int par = (int)(i & 1);
    T* orow = out + row * cols + (size_t)first_vec * N;

    if constexpr (!BWD) {
      float m[1] = {-INFINITY};
      for (int v = tid; v < my_nvec; v += kWideThreads) {
        float f[N];
        unpack<T>(sa[v], f);
#pragma unroll
        for (int j = 0; j < N; ++j) m[0] = fmaxf(m[0], f[j]);
      }
      block_allreduce<1, MaxOp>(m, sm->scratch, phase);
      // A slice that is all -inf (or empty) contributes nothing.
      const float nm = m[0] == -INFINITY ? 0.f : -m[0] * kLog2eW;
      float sum[1] = {0.f};
      for (int v = tid; v < my_nvec; v += kWideThreads) {
        float f[N];
        unpack<T>(sa[v], f);
#pragma unroll
        for (int j = 0; j < N; ++j) sum[0] += fast_exp2(fmaf(f[j], kLog2eW, nm));
      }
      block_allreduce<1, SumOp>(sum, sm->scratch, phase);
      if (tid < C) *cluster.map_shared_rank(&sm->slots[par][rank], tid) = make_float2(m[0], sum[0]);
      cluster.sync();
      float gm = -INFINITY;
      for (int r = 0; r < C; ++r) gm = fmaxf(gm, sm->slots[par][r].x);
      float total = 0.f;
      for (int r = 0; r < C; ++r) {
        const float2 p = sm->slots[par][r];
        if (p.x != -INFINITY) total += p.y * fast_exp2((p.x - gm) * kLog2eW);
      }
      const float inv = 1.0f / total;
      const float ngm = -gm * kLog2eW;
      for (int v = tid; v < my_nvec; v += kWideThreads) {
        float f[N];
        unpack<T>(sa[v], f);
#pragma unroll
        for (int j = 0; j < N; ++j) f[j] = fast_exp2(fmaf(f[j], kLog2eW, ngm)) * inv;
        st_vec(orow + (size_t)v * N, pack<T>(f));
      }
    } else {
      float d[1] = {0.f};
      for (int v = tid; v < my_nvec; v += kWideThreads) {
        float yf[N], gf[N];
        unpack<T>(sa[v], yf);
        unpack<T>(sb[v], gf);
#pragma unroll
        for (int j = 0; j < N; ++j) d[0] = fmaf(gf[j], yf[j], d[0]);
      }
      block_allreduce<1, SumOp>(d, sm->scratch, phase);
      if (tid < C) *cluster.map_shared_rank(&sm->slots[par][rank], tid) = make_float2(d[0], 0.f);
      cluster.sync();
      float dot = 0.f;
      for (int r = 0; r < C; ++r) dot += sm->slots[par][r].x;
      for (int v = tid; v < my_nvec; v += kWideThreads) {
        float yf[N], gf[N], o[N];
        unpack<T>(sa[v], yf);
        unpack<T>(sb[v], gf);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = (gf[j] - dot) * yf[j];
        st_vec(orow + (size_t)v * N, pack<T>(o));
      }
    }
    __syncthreads();  // every thread has finished reading stage s
    if (tid == 0 && i + stages < n_mine) issue(i + stages);
    if (++s == stages) {
      s = 0;
      parity ^= 1;
    }
  }
  // after a timeout the last copies may still be in flight: give them time to land
  if (tid == 0 && my_nvec > 0 && *(volatile int*)&sm->abort_flag) settle_after_abort();
  // No block may leave while a peer can still write into its slots: the last
  // write to this block happens before the last cluster barrier it passed.
}

int read_softmax_wide_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_softmax_wide_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_softmax_wide_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_softmax_wide_registered = (register_device_status(read_softmax_wide_status), true);

// Launches the cluster kernel if the row shape allows it; *handled says whether
// it did (false: the caller uses its generic kernel).
template <typename T, bool BWD, int kWideThreads>
int launch_wide_threads(const void* a, const void* b, void* out, int64_t rows, int64_t cols,
                cudaStream_t stream, bool* handled) {
  constexpr int N = Vec<T>::N;
  constexpr int NIN = BWD ? 2 : 1;
  *handled = false;
  if (tune("softmax.no_cluster") || cols % N != 0 || cols / N >= ((int64_t)1 << 30)) return EVG_OK;
  if (!aligned16(a) || !aligned16(out) || (BWD && !aligned16(b))) return EVG_OK;
  const int nvec = (int)(cols / N);
  // Smallest cluster whose per-block slice (all inputs) is at most 32 KB, which
  // lets about seven blocks share an SM; 8 blocks at the latest, with slices as
  // large as shared memory allows. One stage: measured on B200, occupancy
  // (blocks at different phases on one SM) hides the load latency better than
  // a second stage per block does (vocabulary rows, bf16: 444 vs 538 us
  // forward), and 8-block clusters beat 4 and 16.
  const size_t budget = 32 * 1024;
  int C = 2;
  while (C < kMaxCluster && (size_t)NIN * ((nvec + C - 1) / C) * 16 > budget) C *= 2;
  const int forced = tune("softmax.cluster");
  if (forced == 2 || forced == 4 || forced == 8) C = forced;
  const int vec_per_block = (nvec + C - 1) / C;
  const size_t stage_bytes = (size_t)NIN * vec_per_block * 16;
  int stages = 1;
  if (tune("softmax.cluster_stages") == 2) stages = 2;
  const size_t smem = (size_t)stages * stage_bytes + sizeof(WideSmem) + 16;
  if (smem > (size_t)device_info().max_smem_optin) return EVG_OK;

  auto kern = softmax_wide_kernel<T, BWD, kWideThreads>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess) {
    cudaGetLastError();
    return EVG_OK;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kWideThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3((unsigned)C);
  int max_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess ||
      max_clusters < 1) {
    cudaGetLastError();
    return EVG_OK;
  }
  int64_t clusters = rows < max_clusters ? rows : max_clusters;
  cfg.gridDim = dim3((unsigned)(clusters * C));
  const long long wait_limit = 2000000000ll;
  const T* ap = (const T*)a;
  const T* bp = (const T*)b;
  T* op = (T*)out;
  if (cudaLaunchKernelEx(&cfg, kern, ap, bp, op, rows, cols, nvec, vec_per_block, stages,
                         wait_limit) != cudaSuccess) {
    cudaGetLastError();  // cluster launch refused: the generic kernel takes over
    return EVG_OK;
  }
  *handled = true;
  return check_launch(BWD ? "softmax_bwd (cluster)" : "softmax_fwd (cluster)");
}

// 256 threads per block; 512 (knob `softmax.cluster_threads`) measured slower
// on B200 for both directions at vocabulary width.
template <typename T, bool BWD>
int launch_wide(const void* a, const void* b, void* out, int64_t rows, int64_t cols,
                cudaStream_t stream, bool* handled) {
  const int threads = tune("softmax.cluster_threads") == 512 ? 512 : 256;
  if (threads == 512)
    return launch_wide_threads<T, BWD, 512>(a, b, out, rows, cols, stream, handled);
  return launch_wide_threads<T, BWD, 256>(a, b, out, rows, cols, stream, handled);
}

}  // namespace

int softmax_wide_fwd(int dtype, const void* x, void* y, int64_t rows, int64_t cols,
                     cudaStream_t stream, bool* handled) {
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_wide<T, false>(x, nullptr, y, rows, cols, stream, handled);
  });
}

int softmax_wide_bwd(int dtype, const void* y, const void* dy, void* dx, int64_t rows,
                     int64_t cols, cudaStream_t stream, bool* handled) {
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    return launch_wide<T, true>(y, dy, dx, rows, cols, stream, handled);
  });
}

}  // namespace evg
