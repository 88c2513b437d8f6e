// EvoformerAttention on the sm_100a tensor cores (head sizes 32 and 64).
//
//   o = softmax(scale * q k^T + pair_bias + res_mask) v      over the residue axis
//   (ops/level1/evoattention/forward_ref.py:22-49)
//
// q, k, v, o, do are [B, S, N, H, D]: the rows of one (batch, MSA row, head)
// are H*D elements apart, so a TMA descriptor over [B*S, N, H*D] with a
// [rows x 64] box picks the 64 contiguous elements that hold head h (D = 64) or
// the head pair (h & ~1, h | 1) (D = 32) of every residue row, 128-byte
// swizzled as the tcgen05 shared-memory descriptors expect.
//   * Products that contract over the head dimension (q k^T, do v^T) read the
//     tile K-major and simply use the k-steps of their own head.
//   * Products whose output columns are the head dimension (p v, ds k, p^T do,
//     ds^T q) read the tile MN-major over all 64 columns; with D = 32 the other
//     head's 32 output columns are computed and ignored (these shapes are bound
//     by the exponentials, not by the tensor pipe).
// Scores are tiles of 128 rows x 64 columns in TMEM; the 16-bit probabilities /
// dS go back into the columns they came from and are the A operand of the next
// product. With residue counts of a few hundred a block is short, so there is
// no warp specialisation: a block runs  products -> element-wise -> products
// in sequence, warp 0 issues TMA and MMA, and the overlap comes from two to
// four blocks sharing an SM (128 or 256 TMEM columns each).
// pair_bias tiles (float32) also arrive by TMA: as [128 queries x 32 keys] boxes
// with the 128-byte swizzle, so that 32 threads reading 32 different rows hit
// different banks, or, for the kernel whose threads own key rows, as an
// unswizzled [64 queries x 128 keys] box read by column. (Reading the bias rows
// straight from global memory, 1 KB apart per thread, cost six times the rest
// of the forward kernel.) The key mask and the per-query statistics of a chunk
// come by bulk copy.
// Four kernels: forward (thread = query row), dK/dV (thread = key row),
// dQ (thread = query row) and d_pair_bias (a block owns a 128 x 64 tile of the
// bias gradient and walks the MSA rows, summing dS in float32 registers, in
// order: no atomics anywhere).
#include <algorithm>

#include "attention_common.cuh"

namespace evg {

__device__ int g_evo_tc_device_status = 0;

namespace {

using namespace umma;
using namespace attn;

constexpr uint32_t kRowTileBytes = 128 * 128;  // [128 x 64] 16-bit elements
constexpr uint32_t kColTileBytes = 64 * 128;   // [64 x 64]

struct EvoDims {
  int S, N, H;
};

// Which part of a 64-column tile belongs to head h.
template <int HD> __device__ __forceinline__ int tile_x0(int h) { return HD == 32 ? (h >> 1) * 64 : h * 64; }
template <int HD> __device__ __forceinline__ int tile_ks0(int h) { return HD == 32 ? (h & 1) * 2 : 0; }
template <int HD> __device__ __forceinline__ int tile_c0(int h) { return HD == 32 ? (h & 1) * 32 : 0; }

// D[128 x 64] = A[128 x HD] * B[64 x HD]^T, both K-major, the k-steps of head h.
template <int HD>
__device__ __forceinline__ void issue_head_scores(bool lead, uint32_t d_tmem, uint32_t a_saddr,
                                                  uint32_t b_saddr, uint32_t idesc, int ks0) {
  const DescBase a = desc_base_kmajor(a_saddr), b = desc_base_kmajor(b_saddr);
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks)
    if (lead)
      mma_ss(d_tmem, desc_at(a, 2u * (uint32_t)(ks0 + ks)), desc_at(b, 2u * (uint32_t)(ks0 + ks)),
             idesc, ks > 0 ? 1u : 0u);
}
// D[128 x 64] (+)= A_tmem[128 x 64 (16-bit)] * B[64 rows x 64], B read MN-major.
// The packed A columns of k-step kk (16 rows of B) start at a_tmem + a_col(kk).
template <typename ACol>
__device__ __forceinline__ void issue_head_accumulate(bool lead, uint32_t d_tmem, uint32_t a_tmem,
                                                      ACol a_col, uint32_t b_saddr, uint32_t idesc,
                                                      bool accumulate) {
  const DescBase b = desc_base_mnmajor(b_saddr, 64);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    if (lead)
      mma_ts(d_tmem, a_tmem + a_col(kk), desc_at(b, kstep_mnmajor(kk)), idesc,
             (accumulate || kk > 0) ? 1u : 0u);
}

constexpr uint32_t kBiasTileBytes = 128 * 64 * 4;  // [128 x 64] or [64 x 128] float32

// 16-byte chunk j (4 floats) of row r of a [rows x 32] float32 box written by TMA
// with the 128-byte swizzle.
__device__ __forceinline__ float4 swz_row_f32x4(const uint8_t* box, int r, int j) {
  return *reinterpret_cast<const float4*>(box + r * 128 + ((j ^ (r & 7)) << 4));
}
// Bias tile of (query tile q0.., key chunk k0..) as two swizzled boxes + the key
// mask of the chunk (only the valid keys are copied). Thread 0.
__device__ __forceinline__ void load_bias_rows(uint8_t* s_bias, float* s_mask,
                                               const CUtensorMap* map_bias, const float* mrow,
                                               int q0, int k0, int bh, int N, uint64_t* bar) {
  const int valid = N - k0 < 64 ? N - k0 : 64;
  mbar_expect_tx(bar, kBiasTileBytes + (uint32_t)valid * 4u);
  tma_load_3d(s_bias, map_bias, k0, q0, bh, bar);
  tma_load_3d(s_bias + kBiasTileBytes / 2, map_bias, k0 + 32, q0, bh, bar);
  bulk_load_1d(s_mask, mrow + k0, (uint32_t)valid * 4u, bar);
}

struct Setup {
  BlockSetup bs;
  uint32_t tmem;
};
// Barrier initialisation, TMEM allocation (warp 0) and the hand-over of the
// TMEM base address to every thread.
template <typename InitBars>
__device__ __forceinline__ Setup block_setup(uint8_t* raw, size_t tile_bytes_total,
                                             uint32_t tmem_cols, InitBars init_bars) {
  Setup s;
  s.bs = carve(raw, tile_bytes_total);
  if (threadIdx.x == 0) {
    *s.bs.abort_flag = 0;
    init_bars(s.bs.bars);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    tmem_alloc(s.bs.tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  s.tmem = *s.bs.tmem_slot;
  return s;
}

template <int FMT>
__device__ __forceinline__ void store_packed16(uint8_t* dst, const uint32_t* acc, int n, float mul) {
  // n float32 accumulator columns (multiple of 8) -> n 16-bit elements at dst
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    if (v * 8 < n) {
      uint4 pk;
      pk.x = pack2<FMT>(__uint_as_float(acc[8 * v + 0]) * mul, __uint_as_float(acc[8 * v + 1]) * mul);
      pk.y = pack2<FMT>(__uint_as_float(acc[8 * v + 2]) * mul, __uint_as_float(acc[8 * v + 3]) * mul);
      pk.z = pack2<FMT>(__uint_as_float(acc[8 * v + 4]) * mul, __uint_as_float(acc[8 * v + 5]) * mul);
      pk.w = pack2<FMT>(__uint_as_float(acc[8 * v + 6]) * mul, __uint_as_float(acc[8 * v + 7]) * mul);
      *reinterpret_cast<uint4*>(dst + v * 16) = pk;
    }
  }
}

// Rows of a [128 x 64] accumulator -> the HD columns of head h of [B*S, N, H, HD]
// rows row0..row0+127 (< N). 256 threads: (row, half) each store HD/2 columns.
template <int HD, int FMT>
__device__ __forceinline__ void store_head_rows(uint32_t t_acc, void* out, int bs, int row0, int h,
                                                const EvoDims& d, float mul) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quarter = warp & 3, half = warp >> 2;
  const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
  const int row = row0 + quarter * 32 + lane;
  constexpr int W = HD / 2;  // columns per thread
  const int col = tile_c0<HD>(h) + half * W;
  uint32_t acc[W];
  tmem_ld(t_acc + lane_base + col, acc);
  tmem_wait_ld();
  if (row < d.N) {
    uint8_t* dst = reinterpret_cast<uint8_t*>(out) +
                   ((((size_t)bs * d.N + row) * d.H + h) * HD + half * W) * 2;
    store_packed16<FMT>(dst, acc, W, mul);
  }
}

// ------------------------------------------------------------------ forward
// grid = (query tiles of 128, H, B*S), 128 threads: thread = query row, key
// chunks of 64. TMEM (256 columns): two score buffers [0,64), [64,128) (chunk c
// uses buffer c % 2; its P is packed into the buffer's first 32 columns) and
// O [128,192). After the block barrier that ends chunk c, warp 0 first issues the
// scores of chunk c+1 into the other buffer and only then O += P V of chunk c,
// so the other warps wait for two small products, not for the whole issue
// sequence. Online softmax with a lazily moved running maximum.
template <int HD, int FMT>
__global__ void __launch_bounds__(128, 2)
evo_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_bias,
                  const float* __restrict__ res_mask, void* __restrict__ o_ptr,
                  float* __restrict__ lse_ptr, EvoDims d, float scale_log2, long long wait_limit) {
  extern __shared__ uint8_t smem_raw[];
  Setup su = block_setup(smem_raw, kRowTileBytes + 4 * kColTileBytes + kBiasTileBytes + 256, 256,
                         [](uint64_t* bars) {
                           for (int i = 0; i < 6; ++i) mbar_init(bars + i, 1);
                         });
  uint8_t* sQ = su.bs.smem;
  uint8_t* sK = sQ + kRowTileBytes;       // 2 stages
  uint8_t* sV = sK + 2 * kColTileBytes;   // 2 stages
  uint8_t* sB = sV + 2 * kColTileBytes;   // bias tile of the current chunk
  float* sM = reinterpret_cast<float*>(sB + kBiasTileBytes);  // key mask of the current chunk
  uint64_t* q_full = su.bs.bars + 0;
  uint64_t* kv_full = su.bs.bars + 1;  // [2]
  uint64_t* s_done = su.bs.bars + 3;
  uint64_t* bias_full = su.bs.bars + 4;
  uint64_t* pv_done = su.bs.bars + 5;
  const WaitCtx ctx{su.bs.abort_flag, &g_evo_tc_device_status, wait_limit};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, bs = blockIdx.z, b = bs / d.S;
  const int N = d.N;
  const int n_kc = (N + 63) / 64;
  const int x0 = tile_x0<HD>(h), ks0 = tile_ks0<HD>(h), oc0 = tile_c0<HD>(h);
  const uint32_t tO = su.tmem + 128;
  constexpr uint32_t idesc_s = instr_desc_f16(FMT, 128, 64, 0, 0);
  constexpr uint32_t idesc_o = instr_desc_f16(FMT, 128, 64, 0, 1);

  auto load_kv = [&](int c) {  // thread 0
    const int st = c & 1;
    mbar_expect_tx(kv_full + st, 2 * kColTileBytes);
    tma_load_3d(sK + st * kColTileBytes, &map_k, x0, c * 64, bs, kv_full + st);
    tma_load_3d(sV + st * kColTileBytes, &map_v, x0, c * 64, bs, kv_full + st);
  };
  bool lead = false;
  auto issue_s = [&](int c) {  // warp 0, converged
    const int st = c & 1;
    mbar_wait(kv_full + st, (c >> 1) & 1, ctx, 801);
    tc_fence_after_sync();
    issue_head_scores<HD>(lead, su.tmem + st * 64, smem_u32(sQ), smem_u32(sK + st * kColTileBytes),
                          idesc_s, ks0);
    if (lead) mma_commit(s_done);
  };
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v);
    prefetch_tensormap(&map_bias);
    mbar_expect_tx(q_full, kRowTileBytes);
    tma_load_3d(sQ, &map_q, x0, qt * 128, bs, q_full);
    load_kv(0);
    load_bias_rows(sB, sM, &map_bias, res_mask + (size_t)bs * N, qt * 128, 0, b * d.H + h, N,
                   bias_full);
    if (n_kc > 1) load_kv(1);
  }
  __syncwarp();
  if (warp == 0) {
    lead = elect_one();
    mbar_wait(q_full, 0, ctx, 802);
    issue_s(0);
  }
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const int row = warp * 32 + lane;
  const int qg = qt * 128 + row;
  const bool q_ok = qg < N;
  float m_run = -INFINITY, l_run = 0.f;

  for (int c = 0; c < n_kc; ++c) {
    const int st = c & 1;
    const uint32_t tS = su.tmem + st * 64;
    mbar_wait(s_done, c & 1, ctx, 803);
    __syncwarp();
    tc_fence_after_sync();
    uint32_t sr[64];
    tmem_ld32(tS + lane_base, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
    tmem_ld32(tS + lane_base + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
    tmem_wait_ld();
    if (threadIdx.x == 0 && c >= 1 && c + 1 < n_kc) {
      // chunk c+1 takes the K/V stage of chunk c-1 once O += P V (c-1) has read V
      mbar_wait(pv_done, (c - 1) & 1, ctx, 807);
      load_kv(c + 1);
    }
    mbar_wait(bias_full, c & 1, ctx, 805);
    const int k0 = c * 64;
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int g = 0; g < 16; ++g) {
      float z[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (k0 + 4 * g < N) {  // N is a multiple of 4: a group of four keys is valid or not
        const float4 b4 = swz_row_f32x4(sB + (g >> 3) * (kBiasTileBytes / 2), row, g & 7);
        const float4 m4 = reinterpret_cast<const float4*>(sM)[g];
        const float add[4] = {b4.x + m4.x, b4.y + m4.y, b4.z + m4.z, b4.w + m4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          z[e] = fmaf(__uint_as_float(sr[4 * g + e]), scale_log2, add[e] * kLog2e);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        sr[4 * g + e] = __float_as_uint(z[e]);
        mx4[e] = fmaxf(mx4[e], z[e]);
      }
    }
    const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    const bool grow = mx > m_run + kRescaleThreshold;  // always true for the first chunk
    const float m_new = grow ? mx : m_run;
    if (c > 0 && __any_sync(0xffffffffu, grow)) {
      // Rows that did not grow use alpha = 1. O += P V of the previous chunk must
      // have completed before O is touched.
      mbar_wait(pv_done, (c - 1) & 1, ctx, 806);
      __syncwarp();
      tc_fence_after_sync();
      const float alpha = grow ? fast_exp2(m_run - m_new) : 1.0f;
      l_run *= alpha;
#pragma unroll
      for (int cc = 0; cc < HD / 32; ++cc) {
        uint32_t orow[32];
        tmem_ld32(tO + lane_base + oc0 + cc * 32, orow);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
        tmem_st32(tO + lane_base + oc0 + cc * 32, orow);
      }
    }
    m_run = m_new;
    float ls4[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t pr[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float p0 = fast_exp2(__uint_as_float(sr[2 * i]) - m_run);
      const float p1 = fast_exp2(__uint_as_float(sr[2 * i + 1]) - m_run);
      ls4[i & 3] += p0 + p1;
      pr[i] = pack2<FMT>(p0, p1);
    }
    l_run += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
    tmem_st32(tS + lane_base, pr);
    tmem_wait_st();
    tc_fence_before_sync();
    __syncthreads();  // P is in TMEM; every thread is past its bias / mask reads
    if (warp == 0) {
      tc_fence_after_sync();
      if (c + 1 < n_kc) issue_s(c + 1);  // into the other score buffer
      issue_head_accumulate(lead, tO, tS, [](int kk) { return (uint32_t)kk * 8u; },
                            smem_u32(sV + st * kColTileBytes), idesc_o, c > 0);
      if (lead) mma_commit(pv_done);
      __syncwarp();
      if (lane == 0 && c + 1 < n_kc)
        load_bias_rows(sB, sM, &map_bias, res_mask + (size_t)bs * N, qt * 128, (c + 1) * 64,
                       b * d.H + h, N, bias_full);
      __syncwarp();
    }
  }
  mbar_wait(pv_done, (n_kc - 1) & 1, ctx, 804);
  __syncwarp();
  tc_fence_after_sync();
  {
    const float inv_l = 1.0f / l_run;
    uint32_t acc[HD];
#pragma unroll
    for (int cc = 0; cc < HD / 32; ++cc)
      tmem_ld32(tO + lane_base + oc0 + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[cc * 32]));
    tmem_wait_ld();
    if (q_ok) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(o_ptr) + (((size_t)bs * N + qg) * d.H + h) * HD * 2;
#pragma unroll
      for (int cc = 0; cc < HD / 32; ++cc) store_packed16<FMT>(dst + cc * 64, acc + cc * 32, 32, inv_l);
      lse_ptr[((size_t)bs * d.H + h) * N + qg] = (m_run + log2f(l_run)) * kLn2;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(su.tmem, 256);
}

// ------------------------------------------------- backward: shared pieces
// 256 threads: warp w reads TMEM lanes 32*(w&3).. (its rows) and the 32 columns
// 32*(w>>2).. of a 64-column score tile.
struct BwdThread {
  int warp, lane, quarter, half, row;
  uint32_t lane_base;
};
__device__ __forceinline__ BwdThread bwd_thread() {
  BwdThread t;
  t.warp = threadIdx.x >> 5;
  t.lane = threadIdx.x & 31;
  t.quarter = t.warp & 3;
  t.half = t.warp >> 2;
  t.row = t.quarter * 32 + t.lane;
  t.lane_base = (uint32_t)(t.quarter * 32) << 16;
  return t;
}
// packed A columns of k-step kk when each half packed its 32 columns into 16
__device__ __forceinline__ uint32_t packed_col(int kk) { return (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8); }

// ------------------------------------------------------------------------ dQ
// grid = (query tiles of 128, H, B*S). Thread = (query row, half of a 64-key
// chunk). TMEM (256 columns): [0,64) S -> dS packed, [64,128) dP, [128,192) dQ.
template <int HD, int FMT>
__global__ void __launch_bounds__(256, 2)
evo_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                 const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                 const __grid_constant__ CUtensorMap map_bias, const float* __restrict__ res_mask,
                 const float* __restrict__ lse, const float* __restrict__ delta,
                 void* __restrict__ dq_ptr, EvoDims d, float scale, long long wait_limit) {
  extern __shared__ uint8_t smem_raw[];
  Setup su = block_setup(smem_raw, 2 * kRowTileBytes + 4 * kColTileBytes + kBiasTileBytes + 256,
                         256, [](uint64_t* bars) {
                           for (int i = 0; i < 5; ++i) mbar_init(bars + i, 1);
                         });
  uint8_t* sQ = su.bs.smem;
  uint8_t* sDO = sQ + kRowTileBytes;
  uint8_t* sK = sDO + kRowTileBytes;      // 2 stages
  uint8_t* sV = sK + 2 * kColTileBytes;   // 2 stages
  uint8_t* sB = sV + 2 * kColTileBytes;   // bias tile of the current chunk
  float* sM = reinterpret_cast<float*>(sB + kBiasTileBytes);
  uint64_t* qdo_full = su.bs.bars + 0;
  uint64_t* kv_full = su.bs.bars + 1;  // [2]
  uint64_t* sdp_done = su.bs.bars + 3;
  uint64_t* bias_full = su.bs.bars + 4;
  const WaitCtx ctx{su.bs.abort_flag, &g_evo_tc_device_status, wait_limit};
  const BwdThread t = bwd_thread();
  const int qt = blockIdx.x, h = blockIdx.y, bs = blockIdx.z, b = bs / d.S;
  const int N = d.N;
  const int n_kc = (N + 63) / 64;
  const int x0 = tile_x0<HD>(h), ks0 = tile_ks0<HD>(h);
  const uint32_t tS = su.tmem, tDP = su.tmem + 64, tDQ = su.tmem + 128;
  constexpr uint32_t idesc_s = instr_desc_f16(FMT, 128, 64, 0, 0);
  constexpr uint32_t idesc_d = instr_desc_f16(FMT, 128, 64, 0, 1);
  const float scale_log2 = scale * kLog2e;

  auto load_kv = [&](int c) {  // thread 0
    const int st = c & 1;
    mbar_expect_tx(kv_full + st, 2 * kColTileBytes);
    tma_load_3d(sK + st * kColTileBytes, &map_k, x0, c * 64, bs, kv_full + st);
    tma_load_3d(sV + st * kColTileBytes, &map_v, x0, c * 64, bs, kv_full + st);
  };
  bool lead = false;
  auto issue_sdp = [&](int c) {  // warp 0, converged
    const int st = c & 1;
    mbar_wait(kv_full + st, (c >> 1) & 1, ctx, 811);
    tc_fence_after_sync();
    issue_head_scores<HD>(lead, tS, smem_u32(sQ), smem_u32(sK + st * kColTileBytes), idesc_s, ks0);
    issue_head_scores<HD>(lead, tDP, smem_u32(sDO), smem_u32(sV + st * kColTileBytes), idesc_s, ks0);
    if (lead) mma_commit(sdp_done);
  };
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_do);
    prefetch_tensormap(&map_k); prefetch_tensormap(&map_v);
    mbar_expect_tx(qdo_full, 2 * kRowTileBytes);
    tma_load_3d(sQ, &map_q, x0, qt * 128, bs, qdo_full);
    tma_load_3d(sDO, &map_do, x0, qt * 128, bs, qdo_full);
    load_kv(0);
    prefetch_tensormap(&map_bias);
    load_bias_rows(sB, sM, &map_bias, res_mask + (size_t)bs * N, qt * 128, 0, b * d.H + h, N,
                   bias_full);
  }
  __syncwarp();
  if (t.warp == 0) {
    lead = elect_one();
    mbar_wait(qdo_full, 0, ctx, 812);
    issue_sdp(0);
  }
  const int qg = qt * 128 + t.row;
  const int qc = qg < N ? qg : N - 1;
  const uint8_t* bbox = sB + t.half * (kBiasTileBytes / 2);  // this half's 32 key columns
  const float4* m4p = reinterpret_cast<const float4*>(sM + t.half * 32);
  const float nl = -lse[((size_t)bs * d.H + h) * N + qc] * kLog2e;
  const float dl = delta[((size_t)bs * d.H + h) * N + qc];

  for (int c = 0; c < n_kc; ++c) {
    const int st = c & 1;
    mbar_wait(sdp_done, c & 1, ctx, 813);
    __syncwarp();
    tc_fence_after_sync();
    if (threadIdx.x == 0 && c + 1 < n_kc) load_kv(c + 1);
    uint32_t sr[32], dr[32];
    tmem_ld32(tS + t.lane_base + t.half * 32, sr);
    tmem_ld32(tDP + t.lane_base + t.half * 32, dr);
    tmem_wait_ld();
    mbar_wait(bias_full, c & 1, ctx, 815);
    const int k0 = c * 64 + t.half * 32;
    uint32_t dd[16];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float ds[4] = {0.f, 0.f, 0.f, 0.f};
      if (k0 + 4 * g < N) {
        const float4 b4 = swz_row_f32x4(bbox, t.row, g);
        const float4 m4 = m4p[g];
        const float add[4] = {b4.x + m4.x, b4.y + m4.y, b4.z + m4.z, b4.w + m4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = fast_exp2(
              fmaf(__uint_as_float(sr[4 * g + e]), scale_log2, fmaf(add[e], kLog2e, nl)));
          ds[e] = p * (__uint_as_float(dr[4 * g + e]) - dl);
        }
      }
      dd[2 * g] = pack2<FMT>(ds[0], ds[1]);
      dd[2 * g + 1] = pack2<FMT>(ds[2], ds[3]);
    }
    tmem_st16(tS + t.lane_base + t.half * 32, dd);
    tmem_wait_st();
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && c + 1 < n_kc)
      load_bias_rows(sB, sM, &map_bias, res_mask + (size_t)bs * N, qt * 128, (c + 1) * 64,
                     b * d.H + h, N, bias_full);
    if (t.warp == 0) {
      tc_fence_after_sync();
      issue_head_accumulate(lead, tDQ, tS, packed_col, smem_u32(sK + st * kColTileBytes), idesc_d,
                            c > 0);
      if (c + 1 < n_kc) {
        issue_sdp(c + 1);
      } else if (lead) {
        mma_commit(sdp_done);
      }
      __syncwarp();
    }
  }
  mbar_wait(sdp_done, n_kc & 1, ctx, 814);
  __syncwarp();
  tc_fence_after_sync();
  store_head_rows<HD, FMT>(tDQ, dq_ptr, bs, qt * 128, h, d, scale);
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(su.tmem, 256);
}

// -------------------------------------------------------------------- dK, dV
// grid = (key tiles of 128, H, B*S). Thread = (key row, half of a 64-query
// chunk). TMEM (256 columns): [0,64) S^T -> P^T packed, [64,128) dP^T -> dS^T
// packed, [128,192) dV, [192,256) dK.
template <int HD, int FMT>
__global__ void __launch_bounds__(256, 2)
evo_dkdv_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_bias_t, const float* __restrict__ res_mask,
                   const float* __restrict__ lse, const float* __restrict__ delta,
                   void* __restrict__ dk_ptr, void* __restrict__ dv_ptr, EvoDims d, float scale,
                   long long wait_limit) {
  extern __shared__ uint8_t smem_raw[];
  Setup su = block_setup(smem_raw, 2 * kRowTileBytes + 4 * kColTileBytes + kBiasTileBytes + 512,
                         256, [](uint64_t* bars) {
                           for (int i = 0; i < 5; ++i) mbar_init(bars + i, 1);
                         });
  uint8_t* sK = su.bs.smem;
  uint8_t* sV = sK + kRowTileBytes;
  uint8_t* sQ = sV + kRowTileBytes;        // 2 stages of 64 query rows
  uint8_t* sDO = sQ + 2 * kColTileBytes;   // 2 stages
  // bias[q][k] of the current chunk, [64 queries x 128 keys] float32, and the
  // chunk's per-query statistics (64 x lse, 64 x delta)
  const float* sB = reinterpret_cast<const float*>(sDO + 2 * kColTileBytes);
  float* sStat = reinterpret_cast<float*>(sDO + 2 * kColTileBytes + kBiasTileBytes);
  uint64_t* kv_full = su.bs.bars + 0;
  uint64_t* qdo_full = su.bs.bars + 1;  // [2]
  uint64_t* sdp_done = su.bs.bars + 3;
  uint64_t* aux_full = su.bs.bars + 4;
  const WaitCtx ctx{su.bs.abort_flag, &g_evo_tc_device_status, wait_limit};
  const BwdThread t = bwd_thread();
  const int kt = blockIdx.x, h = blockIdx.y, bs = blockIdx.z, b = bs / d.S;
  const int N = d.N;
  const int n_qc = (N + 63) / 64;
  const int x0 = tile_x0<HD>(h), ks0 = tile_ks0<HD>(h);
  const uint32_t tS = su.tmem, tDP = su.tmem + 64, tDV = su.tmem + 128, tDK = su.tmem + 192;
  constexpr uint32_t idesc_s = instr_desc_f16(FMT, 128, 64, 0, 0);
  constexpr uint32_t idesc_d = instr_desc_f16(FMT, 128, 64, 0, 1);
  const float scale_log2 = scale * kLog2e;

  auto load_qdo = [&](int c) {  // thread 0
    const int st = c & 1;
    mbar_expect_tx(qdo_full + st, 2 * kColTileBytes);
    tma_load_3d(sQ + st * kColTileBytes, &map_q, x0, c * 64, bs, qdo_full + st);
    tma_load_3d(sDO + st * kColTileBytes, &map_do, x0, c * 64, bs, qdo_full + st);
  };
  bool lead = false;
  auto issue_sdp = [&](int c) {  // warp 0, converged
    const int st = c & 1;
    mbar_wait(qdo_full + st, (c >> 1) & 1, ctx, 821);
    tc_fence_after_sync();
    issue_head_scores<HD>(lead, tS, smem_u32(sK), smem_u32(sQ + st * kColTileBytes), idesc_s, ks0);
    issue_head_scores<HD>(lead, tDP, smem_u32(sV), smem_u32(sDO + st * kColTileBytes), idesc_s, ks0);
    if (lead) mma_commit(sdp_done);
  };
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_do);
    prefetch_tensormap(&map_k); prefetch_tensormap(&map_v);
    mbar_expect_tx(kv_full, 2 * kRowTileBytes);
    tma_load_3d(sK, &map_k, x0, kt * 128, bs, kv_full);
    tma_load_3d(sV, &map_v, x0, kt * 128, bs, kv_full);
    load_qdo(0);
    prefetch_tensormap(&map_bias_t);
  }
  const float* lrow = lse + ((size_t)bs * d.H + h) * N;
  const float* drow = delta + ((size_t)bs * d.H + h) * N;
  auto load_aux = [&](int c) {  // thread 0: bias tile and statistics of query chunk c
    const int valid = N - c * 64 < 64 ? N - c * 64 : 64;
    mbar_expect_tx(aux_full, kBiasTileBytes + 2u * (uint32_t)valid * 4u);
    tma_load_3d(const_cast<float*>(sB), &map_bias_t, kt * 128, c * 64, b * d.H + h, aux_full);
    bulk_load_1d(sStat, lrow + c * 64, (uint32_t)valid * 4u, aux_full);
    bulk_load_1d(sStat + 64, drow + c * 64, (uint32_t)valid * 4u, aux_full);
  };
  if (threadIdx.x == 0) load_aux(0);
  __syncwarp();
  if (t.warp == 0) {
    lead = elect_one();
    mbar_wait(kv_full, 0, ctx, 822);
    issue_sdp(0);
  }
  const int kg = kt * 128 + t.row;
  const int kc = kg < N ? kg : N - 1;
  const float mk = res_mask[(size_t)bs * N + kc];

  for (int c = 0; c < n_qc; ++c) {
    const int st = c & 1;
    mbar_wait(sdp_done, c & 1, ctx, 823);
    __syncwarp();
    tc_fence_after_sync();
    if (threadIdx.x == 0 && c + 1 < n_qc) load_qdo(c + 1);
    uint32_t sr[32], dr[32];
    tmem_ld32(tS + t.lane_base + t.half * 32, sr);
    tmem_ld32(tDP + t.lane_base + t.half * 32, dr);
    tmem_wait_ld();
    mbar_wait(aux_full, c & 1, ctx, 825);
    const int q0 = c * 64 + t.half * 32;
    // column t.row of the bias tile, rows (queries) half*32 ..: conflict-free
    const float* bcol = sB + (size_t)(t.half * 32) * 128 + t.row;
    const float4* l4p = reinterpret_cast<const float4*>(sStat + t.half * 32);
    const float4* d4p = reinterpret_cast<const float4*>(sStat + 64 + t.half * 32);
    uint32_t pp[16], dd[16];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float p[4] = {0.f, 0.f, 0.f, 0.f}, ds[4] = {0.f, 0.f, 0.f, 0.f};
      if (q0 + 4 * g < N) {
        const float4 l4 = l4p[g];
        const float4 d4 = d4p[g];
        const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float bias = bcol[(4 * g + e) * 128];
          p[e] = fast_exp2(fmaf(__uint_as_float(sr[4 * g + e]), scale_log2,
                                (bias + mk - lv[e]) * kLog2e));
          ds[e] = p[e] * (__uint_as_float(dr[4 * g + e]) - dv[e]);
        }
      }
      pp[2 * g] = pack2<FMT>(p[0], p[1]);
      pp[2 * g + 1] = pack2<FMT>(p[2], p[3]);
      dd[2 * g] = pack2<FMT>(ds[0], ds[1]);
      dd[2 * g + 1] = pack2<FMT>(ds[2], ds[3]);
    }
    tmem_st16(tS + t.lane_base + t.half * 32, pp);
    tmem_st16(tDP + t.lane_base + t.half * 32, dd);
    tmem_wait_st();
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && c + 1 < n_qc) load_aux(c + 1);
    if (t.warp == 0) {
      tc_fence_after_sync();
      issue_head_accumulate(lead, tDV, tS, packed_col, smem_u32(sDO + st * kColTileBytes), idesc_d,
                            c > 0);
      issue_head_accumulate(lead, tDK, tDP, packed_col, smem_u32(sQ + st * kColTileBytes), idesc_d,
                            c > 0);
      if (c + 1 < n_qc) {
        issue_sdp(c + 1);
      } else if (lead) {
        mma_commit(sdp_done);
      }
      __syncwarp();
    }
  }
  mbar_wait(sdp_done, n_qc & 1, ctx, 824);
  __syncwarp();
  tc_fence_after_sync();
  store_head_rows<HD, FMT>(tDV, dv_ptr, bs, kt * 128, h, d, 1.0f);
  store_head_rows<HD, FMT>(tDK, dk_ptr, bs, kt * 128, h, d, scale);
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(su.tmem, 256);
}

// --------------------------------------------------------------- d_pair_bias
// grid = (query tiles of 128, key chunks of 64, B*H*split). The block owns the
// [128 x 64] tile (query tile, key chunk) of d_pair_bias[b, h] and walks the MSA
// rows s of its part in order: S and dP of (s, tile), dS in registers, summed
// in float32. Part `part` writes out[part][b][h][q][k]; the parts are added in a
// fixed order by the caller's reduction kernel (split == 1 writes the result).
// TMEM (128 columns): [0,64) S, [64,128) dP.
template <int HD, int FMT>
__global__ void __launch_bounds__(256, 1)
evo_dbias_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const __grid_constant__ CUtensorMap map_bias, const float* __restrict__ res_mask,
                    const float* __restrict__ lse, const float* __restrict__ delta,
                    float* __restrict__ out, EvoDims d, int B, int split, float scale,
                    long long wait_limit) {
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t kStage = 2 * kRowTileBytes + 2 * kColTileBytes;
  Setup su = block_setup(smem_raw, 2 * kStage + kBiasTileBytes + 512, 128, [](uint64_t* bars) {
    for (int i = 0; i < 4; ++i) mbar_init(bars + i, 1);
  });
  uint8_t* sB = su.bs.smem + 2 * kStage;  // the block's bias tile, loaded once
  float* sM = reinterpret_cast<float*>(sB + kBiasTileBytes);  // [2 stages][64] key mask
  uint64_t* full = su.bs.bars + 0;  // [2]
  uint64_t* sdp_done = su.bs.bars + 2;
  uint64_t* bias_full = su.bs.bars + 3;
  const WaitCtx ctx{su.bs.abort_flag, &g_evo_tc_device_status, wait_limit};
  const BwdThread t = bwd_thread();
  const int qt = blockIdx.x, kc_ = blockIdx.y;
  const int part = blockIdx.z % split, bh = blockIdx.z / split;
  const int b = bh / d.H, h = bh % d.H;
  const int N = d.N;
  const int s_begin = (int)((long long)part * d.S / split);
  const int s_end = (int)((long long)(part + 1) * d.S / split);
  const int n_s = s_end - s_begin;
  const int x0 = tile_x0<HD>(h), ks0 = tile_ks0<HD>(h);
  const uint32_t tS = su.tmem, tDP = su.tmem + 64;
  constexpr uint32_t idesc_s = instr_desc_f16(FMT, 128, 64, 0, 0);
  const float scale_log2 = scale * kLog2e;

  auto stage_ptr = [&](int st) { return su.bs.smem + st * kStage; };
  auto load_s = [&](int i) {  // thread 0: tiles of MSA row s_begin + i
    const int st = i & 1, bs = b * d.S + s_begin + i;
    uint8_t* p = stage_ptr(st);
    const int valid = N - kc_ * 64 < 64 ? N - kc_ * 64 : 64;
    mbar_expect_tx(full + st, kStage + (uint32_t)valid * 4u);
    bulk_load_1d(sM + st * 64, res_mask + (size_t)bs * N + kc_ * 64, (uint32_t)valid * 4u,
                 full + st);
    tma_load_3d(p, &map_q, x0, qt * 128, bs, full + st);
    tma_load_3d(p + kRowTileBytes, &map_do, x0, qt * 128, bs, full + st);
    tma_load_3d(p + 2 * kRowTileBytes, &map_k, x0, kc_ * 64, bs, full + st);
    tma_load_3d(p + 2 * kRowTileBytes + kColTileBytes, &map_v, x0, kc_ * 64, bs, full + st);
  };
  bool lead = false;
  auto issue_sdp = [&](int i) {  // warp 0, converged
    const int st = i & 1;
    const uint32_t p = smem_u32(stage_ptr(st));
    mbar_wait(full + st, (i >> 1) & 1, ctx, 831);
    tc_fence_after_sync();
    issue_head_scores<HD>(lead, tS, p, p + 2 * kRowTileBytes, idesc_s, ks0);
    issue_head_scores<HD>(lead, tDP, p + kRowTileBytes, p + 2 * kRowTileBytes + kColTileBytes,
                          idesc_s, ks0);
    if (lead) mma_commit(sdp_done);
  };
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_do);
    prefetch_tensormap(&map_k); prefetch_tensormap(&map_v);
    prefetch_tensormap(&map_bias);
    mbar_expect_tx(bias_full, kBiasTileBytes);
    tma_load_3d(sB, &map_bias, kc_ * 64, qt * 128, bh, bias_full);
    tma_load_3d(sB + kBiasTileBytes / 2, &map_bias, kc_ * 64 + 32, qt * 128, bh, bias_full);
    if (n_s > 0) load_s(0);
    if (n_s > 1) load_s(1);
  }
  __syncwarp();
  if (t.warp == 0) {
    lead = elect_one();
    if (n_s > 0) issue_sdp(0);
  }
  const int qg = qt * 128 + t.row;
  const int qc = qg < N ? qg : N - 1;
  const int k0 = kc_ * 64 + t.half * 32;
  const uint8_t* bbox = sB + t.half * (kBiasTileBytes / 2);
  float acc[32];
#pragma unroll
  for (int e = 0; e < 32; ++e) acc[e] = 0.f;
  mbar_wait(bias_full, 0, ctx, 833);

  for (int i = 0; i < n_s; ++i) {
    const int bs = b * d.S + s_begin + i;
    mbar_wait(sdp_done, i & 1, ctx, 832);
    __syncwarp();
    tc_fence_after_sync();
    uint32_t sr[32], dr[32];
    tmem_ld32(tS + t.lane_base + t.half * 32, sr);
    tmem_ld32(tDP + t.lane_base + t.half * 32, dr);
    tmem_wait_ld();
    float4 m4v[8];  // the key mask of this MSA row, before its stage is refilled
#pragma unroll
    for (int g = 0; g < 8; ++g)
      m4v[g] = reinterpret_cast<const float4*>(sM + (i & 1) * 64 + t.half * 32)[g];
    tc_fence_before_sync();
    __syncthreads();  // every thread holds its scores: stage i&1 and the TMEM tiles are free
    if (threadIdx.x == 0 && i + 2 < n_s) load_s(i + 2);
    if (t.warp == 0 && i + 1 < n_s) {
      tc_fence_after_sync();
      issue_sdp(i + 1);
      __syncwarp();
    }
    const float nl = -__ldg(lse + ((size_t)bs * d.H + h) * N + qc) * kLog2e;
    const float dl = __ldg(delta + ((size_t)bs * d.H + h) * N + qc);
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (k0 + 4 * g < N) {
        const float4 b4 = swz_row_f32x4(bbox, t.row, g);
        const float4 m4 = m4v[g];
        const float add[4] = {b4.x + m4.x, b4.y + m4.y, b4.z + m4.z, b4.w + m4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = fast_exp2(
              fmaf(__uint_as_float(sr[4 * g + e]), scale_log2, fmaf(add[e], kLog2e, nl)));
          acc[4 * g + e] = fmaf(p, __uint_as_float(dr[4 * g + e]) - dl, acc[4 * g + e]);
        }
      }
    }
  }
  if (qg < N) {
    float* dst = out + (((size_t)part * B + b) * d.H + h) * N * N + (size_t)qg * N + k0;
#pragma unroll
    for (int g = 0; g < 8; ++g)
      if (k0 + 4 * g < N)
        reinterpret_cast<float4*>(dst)[g] =
            make_float4(acc[4 * g], acc[4 * g + 1], acc[4 * g + 2], acc[4 * g + 3]);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(su.tmem, 128);
}

// ---------------------------------------------------------------- host side
int read_evo_tc_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_evo_tc_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_evo_tc_device_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_evo_tc_status_registered = (register_device_status(read_evo_tc_status), true);

long long evo_wait_limit() {
  const int t = tune("attention.wait_limit");  // in millions of cycles
  return t > 0 ? (long long)t * 1000000ll : 2000000000ll;
}

template <typename Kernel>
int evo_reserve(Kernel kernel, size_t bytes) {
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) !=
      cudaSuccess) {
    cudaGetLastError();
    return fail(EVG_ELAUNCH, "evoattention: cannot reserve %zu bytes of shared memory", bytes);
  }
  return EVG_OK;
}

struct EvoMaps {
  CUtensorMap row[4];  // q, k, v, do with 128-row boxes
  CUtensorMap col[4];  // the same tensors with 64-row boxes
  CUtensorMap bias;    // pair_bias as swizzled [128 queries x 32 keys] boxes
  CUtensorMap bias_t;  // pair_bias as unswizzled [64 queries x 128 keys] boxes
};
int encode_maps(EvoMaps* m, int fmt, const void* q, const void* k, const void* v, const void* dout,
                const float* pair_bias, int64_t B, int64_t S, int64_t N, int64_t H, int64_t D) {
  if (!encode_tile_map_f32(&m->bias, pair_bias, (uint64_t)N, (uint64_t)N, (uint64_t)(B * H), 32, 128,
                           true) ||
      !encode_tile_map_f32(&m->bias_t, pair_bias, (uint64_t)N, (uint64_t)N, (uint64_t)(B * H), 128,
                           64, false))
    return fail(EVG_ELAUNCH, "evoattention: cuTensorMapEncodeTiled failed for pair_bias");
  const void* ptr[4] = {q, k, v, dout};
  for (int i = 0; i < 4; ++i) {
    if (!ptr[i]) continue;
    if (!encode_tile_map_16bit(&m->row[i], ptr[i], fmt, (uint64_t)(H * D), (uint64_t)N,
                               (uint64_t)(B * S), 128) ||
        !encode_tile_map_16bit(&m->col[i], ptr[i], fmt, (uint64_t)(H * D), (uint64_t)N,
                               (uint64_t)(B * S), 64))
      return fail(EVG_ELAUNCH, "evoattention: cuTensorMapEncodeTiled failed");
  }
  return EVG_OK;
}

template <int HD, int FMT>
int launch_fwd_tc(const void* q, const void* k, const void* v, const float* res_mask,
                  const float* pair_bias, void* o, float* lse, int64_t B, int64_t S, int64_t N,
                  int64_t H, float scale, cudaStream_t stream) {
  EvoMaps m;
  if (int rc = encode_maps(&m, FMT, q, k, v, nullptr, pair_bias, B, S, N, H, HD)) return rc;
  const size_t smem = kRowTileBytes + 4 * kColTileBytes + kBiasTileBytes + 256 + kControlBytes + 1024;
  auto kern = evo_fwd_tc_kernel<HD, FMT>;
  if (int rc = evo_reserve(kern, smem)) return rc;
  const EvoDims d{(int)S, (int)N, (int)H};
  dim3 grid((unsigned)((N + 127) / 128), (unsigned)H, (unsigned)(B * S));
  kern<<<grid, 128, smem, stream>>>(m.row[0], m.col[1], m.col[2], m.bias, res_mask, o, lse, d,
                                    scale * kLog2e, evo_wait_limit());
  return check_launch("evoattention_fwd");
}

template <int HD, int FMT>
int launch_bwd_tc(const void* dout, const void* q, const void* k, const void* v,
                  const float* res_mask, const float* pair_bias, const float* lse,
                  const float* delta, void* dq, void* dk, void* dv, float* dbias_out, int split,
                  int64_t B, int64_t S, int64_t N, int64_t H, float scale, cudaStream_t stream) {
  EvoMaps m;
  if (int rc = encode_maps(&m, FMT, q, k, v, dout, pair_bias, B, S, N, H, HD)) return rc;
  const EvoDims d{(int)S, (int)N, (int)H};
  const long long limit = evo_wait_limit();
  const unsigned tiles = (unsigned)((N + 127) / 128), chunks = (unsigned)((N + 63) / 64);
  {
    const size_t smem =
        2 * kRowTileBytes + 4 * kColTileBytes + kBiasTileBytes + 512 + kControlBytes + 1024;
    auto kern = evo_dkdv_tc_kernel<HD, FMT>;
    if (int rc = evo_reserve(kern, smem)) return rc;
    kern<<<dim3(tiles, (unsigned)H, (unsigned)(B * S)), 256, smem, stream>>>(
        m.row[1], m.row[2], m.col[0], m.col[3], m.bias_t, res_mask, lse, delta, dk, dv, d, scale,
        limit);
    if (int rc = check_launch("evoattention_bwd dkdv")) return rc;
  }
  {
    const size_t smem =
        2 * kRowTileBytes + 4 * kColTileBytes + kBiasTileBytes + 256 + kControlBytes + 1024;
    auto kern = evo_dq_tc_kernel<HD, FMT>;
    if (int rc = evo_reserve(kern, smem)) return rc;
    kern<<<dim3(tiles, (unsigned)H, (unsigned)(B * S)), 256, smem, stream>>>(
        m.row[0], m.row[3], m.col[1], m.col[2], m.bias, res_mask, lse, delta, dq, d, scale,
        limit);
    if (int rc = check_launch("evoattention_bwd dq")) return rc;
  }
  {
    const size_t smem = 2 * (2 * kRowTileBytes + 2 * kColTileBytes) + kBiasTileBytes + 512 +
                        kControlBytes + 1024;
    auto kern = evo_dbias_tc_kernel<HD, FMT>;
    if (int rc = evo_reserve(kern, smem)) return rc;
    kern<<<dim3(tiles, chunks, (unsigned)(B * H * split)), 256, smem, stream>>>(
        m.row[0], m.row[3], m.col[1], m.col[2], m.bias, res_mask, lse, delta, dbias_out, d,
        (int)B, split, scale, limit);
    if (int rc = check_launch("evoattention_bwd dbias")) return rc;
  }
  return EVG_OK;
}

}  // namespace

namespace attn {

bool evo_tc_shape(int64_t B, int64_t S, int64_t N, int64_t H, int64_t D, int dtype) {
  if (tune("evoattention.no_tc")) return false;
  if (dtype != EVG_BF16 && dtype != EVG_F16) return false;
  if (D != 32 && D != 64) return false;
  if (D == 32 && (H & 1)) return false;  // heads share 64-column tiles in pairs
  if (N % 4 != 0) return false;          // float4 reads of bias / mask / statistics rows
  return H <= 65535 && B * S <= 65535 && B * H * 16 <= 65535;
}

int launch_evo_tc_fwd(int head_dim, int fmt, const void* q, const void* k, const void* v,
                      const float* res_mask, const float* pair_bias, void* o, float* lse,
                      int64_t B, int64_t S, int64_t N, int64_t H, float scale,
                      cudaStream_t stream) {
#define EVG_EVO_TC_FWD(hd, f)                                                                  \
  if (head_dim == hd && fmt == f)                                                              \
    return launch_fwd_tc<hd, f>(q, k, v, res_mask, pair_bias, o, lse, B, S, N, H, scale, stream);
  EVG_EVO_TC_FWD(32, 0) EVG_EVO_TC_FWD(32, 1) EVG_EVO_TC_FWD(64, 0) EVG_EVO_TC_FWD(64, 1)
#undef EVG_EVO_TC_FWD
  return fail(EVG_EUNSUPPORTED, "evoattention_fwd: head_dim %d on the tensor-core path", head_dim);
}

int launch_evo_tc_bwd(int head_dim, int fmt, const void* dout, const void* q, const void* k,
                      const void* v, const float* res_mask, const float* pair_bias,
                      const float* lse, const float* delta, void* dq, void* dk, void* dv,
                      float* dbias_out, int split, int64_t B, int64_t S, int64_t N, int64_t H,
                      float scale, cudaStream_t stream) {
#define EVG_EVO_TC_BWD(hd, f)                                                                  \
  if (head_dim == hd && fmt == f)                                                              \
    return launch_bwd_tc<hd, f>(dout, q, k, v, res_mask, pair_bias, lse, delta, dq, dk, dv,   \
                                dbias_out, split, B, S, N, H, scale, stream);
  EVG_EVO_TC_BWD(32, 0) EVG_EVO_TC_BWD(32, 1) EVG_EVO_TC_BWD(64, 0) EVG_EVO_TC_BWD(64, 1)
#undef EVG_EVO_TC_BWD
  return fail(EVG_EUNSUPPORTED, "evoattention_bwd: head_dim %d on the tensor-core path", head_dim);
}

}  // namespace attn
}  // namespace evg
