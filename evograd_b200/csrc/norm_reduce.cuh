// Pieces shared by the normalisation backward kernels: the cap on per-block
// partial rows and the second stage of the atomic-free column reduction.
#pragma once
#include "evg_common.cuh"
#include "exchange.cuh"

namespace evg {

#ifdef __CUDACC__
// Programmatic dependent launch of stage 2 behind stage 1: the column-reduce grid
// is launched while the row kernel's last blocks are still running (its blocks
// become resident as the row kernel's blocks leave) and sleeps in
// grid_dependency_wait() until the row kernel has completed and its writes are
// visible; the launch latency between the two kernels is hidden. The row kernels
// call grid_dependents_go() when their row loop is over. Without the launch
// attribute both instructions do nothing.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_dependents_go() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Stage 2: out[c] = sum_p partial[p][c]. Block = 32 column groups x 32 row
// slices; a thread owns CV adjacent columns (one 4-, 8- or 16-byte load per row)
// and its slice adds rows p = y, y+32, ... with four independent accumulators
// per column (so four loads are in flight per thread); the slices are then added
// in order. The order of additions for a column does not depend on CV: fixed
// throughout, bit-reproducible. gridDim.y = dweight / dbias. Wide rows with few
// partial rows take CV = 2 or 4: a quarter of the blocks, each load four times
// as wide ([2048, 16384] LayerNorm: 1024 blocks of 4.6 rows per thread before).
template <typename T, int CV>
__global__ void __launch_bounds__(1024)
colreduce_kernel(const float* __restrict__ partial, int blocks, int64_t cols, T* out_w, T* out_b,
                 float* out_f32) {
  struct __align__(4 * CV) Cols {
    float v[CV];
  };
  __shared__ float tile[32][32 * CV + 1];
  const int which = blockIdx.y;
  const float* src = partial + (size_t)which * blocks * cols;
  const int64_t col0 = ((int64_t)blockIdx.x * 32 + threadIdx.x) * CV;
  float s0[CV], s1[CV], s2[CV], s3[CV];
#pragma unroll
  for (int j = 0; j < CV; ++j) s0[j] = s1[j] = s2[j] = s3[j] = 0.f;
  grid_dependency_wait();
  if (col0 < cols) {  // cols is a multiple of CV: the whole group is inside
    auto row = [&](int p) { return *reinterpret_cast<const Cols*>(src + (size_t)p * cols + col0); };
    int p = threadIdx.y;
    for (; p + 96 < blocks; p += 128) {
      const Cols a = row(p), b = row(p + 32), c = row(p + 64), d = row(p + 96);
#pragma unroll
      for (int j = 0; j < CV; ++j) {
        s0[j] += a.v[j];
        s1[j] += b.v[j];
        s2[j] += c.v[j];
        s3[j] += d.v[j];
      }
    }
    for (; p < blocks; p += 32) {
      const Cols a = row(p);
#pragma unroll
      for (int j = 0; j < CV; ++j) s0[j] += a.v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < CV; ++j)
    tile[threadIdx.y][threadIdx.x * CV + j] = (s0[j] + s1[j]) + (s2[j] + s3[j]);
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;  // one thread per column of the block
  const int64_t col = (int64_t)blockIdx.x * 32 * CV + t;
  if (t < 32 * CV && col < cols) {
    float sum = tile[0][t];
#pragma unroll
    for (int i = 1; i < 32; ++i) sum += tile[i][t];
    T* out = which == 0 ? out_w : out_b;
    if (out) out[col] = from_f32<T>(sum);
    if (out_f32) out_f32[(size_t)which * cols + col] = sum;
  }
}

// Stage 2 fused with the cross-GPU sum. Every block adds the partial rows of its
// 32 columns as above and then, on its own, takes the next epoch e from its own
// counter in the rank's exchange buffer and writes each of its 32 sums, paired
// with e in one 8-byte store, into its area of slot e % 2 in EVERY rank's buffer
// (plain peer stores, no multicast). The thread that owns a column then polls
// the pairs of that column in its OWN rank's buffer until each source rank's
// pair carries e, adds the values in rank order and rounds: no fence, no
// separate flag, no poll across the link, no block waiting for another block of
// its grid, and bit-identical results on every rank. Two slots are enough: a
// block reaches epoch e + 2 only after it has read every rank's pair of epoch
// e + 1, which a rank writes only after its reads of epoch e. A wait that runs
// out records the wait's id in *status and the thread goes on with what it has.
template <typename T>
__global__ void __launch_bounds__(1024)
colreduce_exchange_kernel(const float* __restrict__ partial, int blocks, int64_t cols, T* out_w,
                          T* out_b, xchg::Peers peers, xchg::Layout lay, int n_ranks, int rank,
                          long long wait_limit, int* status) {
  using namespace xchg;
  __shared__ float tile[32][33];
  __shared__ uint32_t s_epoch;
  const int which = blockIdx.y;
  const int bid = blockIdx.y * gridDim.x + blockIdx.x;
  const float* src = partial + (size_t)which * blocks * cols;
  const int64_t col = (int64_t)blockIdx.x * 32 + threadIdx.x;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  grid_dependency_wait();  // the row kernel's partial rows are complete and visible
  if (col < cols) {
    int p = threadIdx.y;
    for (; p + 96 < blocks; p += 128) {
      s0 += src[(size_t)p * cols + col];
      s1 += src[(size_t)(p + 32) * cols + col];
      s2 += src[(size_t)(p + 64) * cols + col];
      s3 += src[(size_t)(p + 96) * cols + col];
    }
    for (; p < blocks; p += 32) s0 += src[(size_t)p * cols + col];
  }
  tile[threadIdx.y][threadIdx.x] = (s0 + s1) + (s2 + s3);
  uint8_t* mine = peers.base[rank];
  if (threadIdx.x == 0 && threadIdx.y == 0) {
    uint32_t* counter = reinterpret_cast<uint32_t*>(mine + lay.block_counter_offset(bid));
    s_epoch = ++*counter;
  }
  __syncthreads();
  if (threadIdx.y != 0 || col >= cols) return;  // warp 0: one thread per column
  const uint32_t epoch = s_epoch;
  const int slot = (int)(epoch & 1u);
  const size_t elem = (size_t)which * cols + (size_t)col;
  float t = tile[0][threadIdx.x];
#pragma unroll
  for (int i = 1; i < 32; ++i) t += tile[i][threadIdx.x];
#pragma unroll
  for (int p = 0; p < kMaxRanks; ++p)
    if (p < n_ranks)
      st_pair_sys(reinterpret_cast<uint2*>(peers.base[p] + lay.pair_area_offset(slot, rank)) + elem, t,
                  epoch);
  float acc = 0.f;
  const long long start = clock64();
  for (int r = 0; r < n_ranks; ++r) {
    const uint2* cell = reinterpret_cast<const uint2*>(mine + lay.pair_area_offset(slot, r)) + elem;
    uint2 v = ld_pair_sys(cell);
    while (v.y != epoch) {
      if (clock64() - start > wait_limit) {
        atomicCAS(status, 0, kFusedExchangeWaitId);
        break;
      }
      v = ld_pair_sys(cell);
    }
    acc += __uint_as_float(v.x);
  }
  T* out = which == 0 ? out_w : out_b;
  if (out) out[col] = from_f32<T>(acc);
}
#endif  // __CUDACC__

// Persistent blocks (= partial rows of the column reduction) the backward
// kernels may launch: SMs x `norm_bwd.blocks_per_sm`; by default 2, and 4 for
// rows of at most 3072 elements, whose kernels keep few values per thread, fit
// four blocks on an SM and need them to hide their load latency (a partial row
// is then at most 12 KB). A bound: kernels that fit fewer blocks launch fewer.
inline int max_partial_blocks(int64_t hidden = (int64_t)1 << 40) {
  int per_sm = tune("norm_bwd.blocks_per_sm");
  if (per_sm <= 0) per_sm = hidden <= 3072 ? 4 : 2;
  return device_info().sm_count * per_sm;
}


#ifdef __CUDACC__
// Launches stage 2 as a programmatic dependent of the kernel before it in `stream`
// (`norm_bwd.no_pdl` = 1: as a plain launch).
template <typename T>
inline void launch_colreduce(const float* partial, int blocks, int64_t cols, T* out_w, T* out_b,
                             float* out_f32, int parts, cudaStream_t stream) {
  // Columns per thread: four while that leaves a block per SM, two while it leaves
  // one and a half (measured on bf16 LayerNorm backward, one column per thread ->
  // this choice: [2048, 16384] 49.4 -> 45.9 us with four, [4096, 8192] 40.9 -> 40.3 us
  // with two; [8192, 5120] with two, 160 blocks, was 0.8 us slower).
  const int sms = device_info().sm_count;
  int cv = 1;
  if (!tune("norm_bwd.narrow_colreduce")) {
    if (cols % 4 == 0 && (cols / 128) * parts >= sms) cv = 4;
    else if (cols % 2 == 0 && 2 * (cols / 64) * parts >= 3 * sms) cv = 2;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((cols + 32 * cv - 1) / (32 * cv)), (unsigned)parts);
  cfg.blockDim = dim3(32, 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tune("norm_bwd.no_pdl") ? 0 : 1;
  auto kern = cv == 4 ? colreduce_kernel<T, 4> : cv == 2 ? colreduce_kernel<T, 2>
                                                         : colreduce_kernel<T, 1>;
  cudaLaunchKernelEx(&cfg, kern, partial, blocks, cols, out_w, out_b, out_f32);
}
#endif

}  // namespace evg
