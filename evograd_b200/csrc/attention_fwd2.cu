// Causal attention forward, warp-specialised with two query tiles per block
// (sm_100a).
//
// A block of 320 threads owns query tiles 2t (tile A) and 2t+1 (tile B) of one
// (batch, head):
//   warp 0        TMA producer (lane 0): Q_A, Q_B once, then K_j / V_j into
//                 two-stage rings gated by empty/full mbarriers;
//   warp 1        tcgen05.mma issuer (all lanes in step, instruction predicated
//                 by elect.sync), order per key tile j:
//                     O_A += P_A(j) V_j;  S_A(j+1) = Q_A K_{j+1}^T;
//                     O_B += P_B(j) V_j;  S_B(j+1) = Q_B K_{j+1}^T
//                 so one tile's softmax runs while the other tile's products do;
//   warps 2..5    softmax of tile A, one thread per query row (TMEM lane);
//   warps 6..9    softmax of tile B.
// TMEM (512 columns): S_A [0,128) (P_A packed into its first 64), S_B [128,256),
// O_A [256,256+HD), O_B [384,384+HD).
// The running row maximum is moved lazily (only when it would grow by more than
// 2^8), so O is rescaled in TMEM only a few times per row.
#include "attention_common.cuh"

namespace evg {

__device__ int g_attn_fwd2_device_status = 0;

namespace {

using namespace umma;
using namespace attn;

constexpr int kFwd2Threads = 320;

template <int HD, int FMT>
__global__ void __launch_bounds__(kFwd2Threads, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, void* __restrict__ o_ptr,
                 float* __restrict__ lse_ptr, int S, int group, float scale_log2,
                 long long wait_limit, int n_pairs, int n_bh, int head_group, int heads,
                 int o_tm, int v_tm) {
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t TB = tile_bytes<HD>();
  BlockSetup bs = carve(smem_raw, 6 * TB);
  uint8_t* sQ[2] = {bs.smem, bs.smem + TB};
  uint8_t* sK[2] = {bs.smem + 2 * TB, bs.smem + 3 * TB};
  uint8_t* sV[2] = {bs.smem + 4 * TB, bs.smem + 5 * TB};
  uint64_t* q_full = bs.bars + 0;
  uint64_t* k_full = bs.bars + 1;   // [2]
  uint64_t* k_empty = bs.bars + 3;  // [2]
  uint64_t* v_full = bs.bars + 5;   // [2]
  uint64_t* v_empty = bs.bars + 7;  // [2]
  uint64_t* s_full = bs.bars + 9;   // [2] tile A, tile B
  uint64_t* p_full = bs.bars + 11;  // [2]
  uint64_t* o_done = bs.bars + 13;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (S + kTile - 1) / kTile;
  // Heaviest pairs first, for a group of heads at a time (map_block).
  int pair, bh;
  map_block(blockIdx.x, n_pairs, n_bh, head_group, pair, bh);
  pair = n_pairs - 1 - pair;
  const int bh_kv = bh / group;  // grouped-query attention: `group` query heads per k/v head
  const int qt[2] = {2 * pair, 2 * pair + 1};
  const bool b_active = qt[1] < n_tiles;
  const int n_kv[2] = {qt[0] + 1, b_active ? qt[1] + 1 : 0};
  const int n_max = b_active ? n_kv[1] : n_kv[0];

  if (threadIdx.x == 0) {
    *bs.abort_flag = 0;
    mbar_init(q_full, 1); mbar_init(o_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + i, 1); mbar_init(k_empty + i, 1);
      mbar_init(v_full + i, 1); mbar_init(v_empty + i, 1);
      mbar_init(s_full + i, 1); mbar_init(p_full + i, 4);
    }
    fence_mbar_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v);
  }
  __syncthreads();
  if (warp == 1) { tmem_alloc(bs.tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *bs.tmem_slot;
  const WaitCtx ctx{bs.abort_flag, &g_attn_fwd2_device_status, wait_limit};
  constexpr uint32_t idesc_s = instr_desc_f16(FMT, 128, 128, 0, 0);
  constexpr uint32_t idesc_o = instr_desc_f16(FMT, 128, HD, 0, 1);
  const uint32_t tS[2] = {tmem, tmem + 128};
  const uint32_t tO[2] = {tmem + 256, tmem + 384};

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, (b_active ? 2 : 1) * TB);
      load_tile<HD>(sQ[0], &map_q, qt[0] * kTile, bh, q_full);
      if (b_active) load_tile<HD>(sQ[1], &map_q, qt[1] * kTile, bh, q_full);
      for (int j = 0; j < n_max; ++j) {
        const int st = j & 1;
        if (j >= 2) mbar_wait(k_empty + st, ((j >> 1) - 1) & 1, ctx, 701);
        mbar_expect_tx(k_full + st, TB);
        load_tile<HD>(sK[st], &map_k, j * kTile, bh_kv, k_full + st);
        if (j >= 2) mbar_wait(v_empty + st, ((j >> 1) - 1) & 1, ctx, 702);
        mbar_expect_tx(v_full + st, TB);
        load_tile_bh<HD>(sV[st], &map_v, j * kTile, bh_kv, heads / group, v_tm, v_full + st);
      }
    }
  } else if (warp == 1) {
    const bool lead = elect_one();
    mbar_wait(q_full, 0, ctx, 703);
    mbar_wait(k_full + 0, 0, ctx, 704);
    tc_fence_after_sync();
    issue_scores<HD>(lead, tS[0], smem_u32(sQ[0]), smem_u32(sK[0]), idesc_s);
    if (lead) mma_commit(s_full + 0);
    if (b_active) {
      issue_scores<HD>(lead, tS[1], smem_u32(sQ[1]), smem_u32(sK[0]), idesc_s);
      if (lead) mma_commit(s_full + 1);
    }
    if (lead) mma_commit(k_empty + 0);
    for (int j = 0; j < n_max; ++j) {
      const int st = j & 1, st1 = (j + 1) & 1;
      const uint32_t ph = j & 1;
      mbar_wait(v_full + st, (j >> 1) & 1, ctx, 705);
      if (j < n_kv[0]) {
        mbar_wait(p_full + 0, ph, ctx, 706);
        tc_fence_after_sync();
        issue_accumulate(lead, tO[0], tS[0], smem_u32(sV[st]), idesc_o, j > 0);
      }
      if (j + 1 < n_max) {
        mbar_wait(k_full + st1, ((j + 1) >> 1) & 1, ctx, 707);
        tc_fence_after_sync();
      }
      if (j + 1 < n_kv[0]) {
        issue_scores<HD>(lead, tS[0], smem_u32(sQ[0]), smem_u32(sK[st1]), idesc_s);
        if (lead) mma_commit(s_full + 0);
      }
      if (b_active) {
        mbar_wait(p_full + 1, ph, ctx, 708);
        tc_fence_after_sync();
        issue_accumulate(lead, tO[1], tS[1], smem_u32(sV[st]), idesc_o, j > 0);
      }
      if (lead) mma_commit(v_empty + st);
      if (b_active && j + 1 < n_kv[1]) {
        issue_scores<HD>(lead, tS[1], smem_u32(sQ[1]), smem_u32(sK[st1]), idesc_s);
        if (lead) mma_commit(s_full + 1);
      }
      if (lead && j + 1 < n_max) mma_commit(k_empty + st1);
      __syncwarp();
    }
    if (lead) mma_commit(o_done);
  } else {
    // ---- softmax warps: one query row per thread
    const int wg = (warp - 2) >> 2;  // 0: tile A, 1: tile B
    const int quarter = warp & 3;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int row = quarter * 32 + lane;
    const int q_glob = qt[wg] * kTile + row;
    const int n_mine = n_kv[wg];
    const uint32_t tSw = tS[wg], tOw = tO[wg];
    float m_run = -INFINITY, l_run = 0.f;
    for (int j = 0; j < n_mine; ++j) {
      mbar_wait(s_full + wg, j & 1, ctx, 709);
      __syncwarp();
      tc_fence_after_sync();
      // Pass 1: row maximum. Score columns [0, 64) stay in registers for pass 2;
      // [64, 96) arrive in the same round trip to tensor memory and [96, 128) while
      // the first maxima are being formed: two load latencies per tile are exposed
      // instead of the eight of a chunk-by-chunk walk in both passes (there are only
      // two softmax warps per scheduler to hide them). Four independent partial
      // maxima keep the comparisons from forming one long dependent chain.
      const int kv0 = j * kTile;
      const bool diag = (j == qt[wg]);
      uint32_t keep[64], tmp[32];
      tmem_ld32(tSw + lane_base, *reinterpret_cast<uint32_t(*)[32]>(&keep[0]));
      tmem_ld32(tSw + lane_base + 32, *reinterpret_cast<uint32_t(*)[32]>(&keep[32]));
      tmem_ld32(tSw + lane_base + 64, tmp);
      tmem_wait_ld();
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      auto fold = [&](const uint32_t* v, int col0, int n) {
        if (diag) {
#pragma unroll
          for (int i = 0; i < n; ++i) {
            float t = __uint_as_float(v[i]);
            if (kv0 + col0 + i > q_glob) t = -INFINITY;
            mx4[i & 3] = fmaxf(mx4[i & 3], t);
          }
        } else {
#pragma unroll
          for (int i = 0; i < n; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        }
      };
      fold(tmp, 64, 32);
      tmem_ld32(tSw + lane_base + 96, tmp);
      fold(keep, 0, 64);
      tmem_wait_ld();
      fold(tmp, 96, 32);
      // scale_log2 > 0, so scaling commutes with the maximum
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      const bool grow = mx > m_run + kRescaleThreshold;  // always true on the first tile
      const float m_new = grow ? mx : m_run;
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // Rescale this warp's rows of O (rows that did not grow use alpha = 1). The
        // previous O += P V has completed: the scores just read were issued after it.
        const float alpha = grow ? fast_exp2(m_run - m_new) : 1.0f;
        l_run *= alpha;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t orow[32];
          tmem_ld32(tOw + lane_base + c * 32, orow);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
          tmem_st32(tOw + lane_base + c * 32, orow);
        }
      }
      m_run = m_new;
      // Pass 2: probabilities. The packed P of chunk c (16 columns) lands in
      // columns [16c, 16c+16), which belong to score chunks already consumed.
      const float neg_m = -m_run;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
      // 32 score columns -> 16 packed probability columns at [16 c, 16 c + 16)
      auto probs = [&](const uint32_t* v, int c) {
        uint32_t pr[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = fast_exp2(fmaf(__uint_as_float(v[2 * i]), scale_log2, neg_m));
          float p1 = fast_exp2(fmaf(__uint_as_float(v[2 * i + 1]), scale_log2, neg_m));
          if (diag) {
            if (kv0 + c * 32 + 2 * i > q_glob) p0 = 0.f;
            if (kv0 + c * 32 + 2 * i + 1 > q_glob) p1 = 0.f;
          }
          ls4[i & 3] += p0 + p1;
          pr[i] = pack2<FMT>(p0, p1);
        }
        tmem_st16(tSw + lane_base + c * 16, pr);
      };
      // columns [64, 128) come back from tensor memory under the exponentials of [0, 64)
      uint32_t late[32];
      tmem_ld32(tSw + lane_base + 64, late);
      probs(&keep[0], 0);
      tmem_ld32(tSw + lane_base + 96, tmp);
      probs(&keep[32], 1);
      tmem_wait_ld();
      probs(late, 2);
      probs(tmp, 3);
      const float lsum = (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      l_run += lsum;
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + wg);
    }
    if (n_mine > 0) {
      mbar_wait(o_done, 0, ctx, 710);
      __syncwarp();
      tc_fence_after_sync();
      const float inv_l = 1.0f / l_run;
      const bool row_ok = q_glob < S;
      uint8_t* orow_g = reinterpret_cast<uint8_t*>(o_ptr) +
                        tensor_row(bh, row_ok ? q_glob : 0, S, heads, o_tm) * HD * 2;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t orow[32];
        tmem_ld32(tOw + lane_base + c * 32, orow);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 pk;
            pk.x = pack2<FMT>(__uint_as_float(orow[8 * v + 0]) * inv_l, __uint_as_float(orow[8 * v + 1]) * inv_l);
            pk.y = pack2<FMT>(__uint_as_float(orow[8 * v + 2]) * inv_l, __uint_as_float(orow[8 * v + 3]) * inv_l);
            pk.z = pack2<FMT>(__uint_as_float(orow[8 * v + 4]) * inv_l, __uint_as_float(orow[8 * v + 5]) * inv_l);
            pk.w = pack2<FMT>(__uint_as_float(orow[8 * v + 6]) * inv_l, __uint_as_float(orow[8 * v + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow_g + (c * 32 + v * 8) * 2) = pk;
          }
        }
      }
      if (row_ok) lse_ptr[(size_t)bh * S + q_glob] = (m_run + log2f(l_run)) * kLn2;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

int read_fwd2_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_attn_fwd2_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attn_fwd2_device_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_fwd2_status_registered = (register_device_status(read_fwd2_status), true);

template <int HD, int FMT>
int launch_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, int64_t B,
                int64_t H, int64_t Hkv, int64_t S, float scale, cudaStream_t stream, Layouts lay) {
  CUtensorMap mq, mk, mv;
  if (!encode_tile_map_16bit(&mq, q, FMT, HD, S, B * H, kTile) ||
      !encode_tile_map_16bit(&mk, k, FMT, HD, S, B * Hkv, kTile) ||
      !encode_bh_map(&mv, v, FMT, HD, S, Hkv, B, lay.v_token_major))
    return fail(EVG_ELAUNCH, "causal_attention_fwd: cuTensorMapEncodeTiled failed");
  const size_t smem = 6 * tile_bytes<HD>() + kControlBytes + 1024;
  auto kern = attn_fwd2_kernel<HD, FMT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess) {
    cudaGetLastError();
    return fail(EVG_ELAUNCH, "causal_attention_fwd: cannot reserve %zu bytes of shared memory", smem);
  }
  const int64_t n_tiles = (S + kTile - 1) / kTile;
  const int64_t n_pairs = (n_tiles + 1) / 2;
  dim3 grid((unsigned)(n_pairs * B * H));
  const int t = tune("attention.wait_limit");
  const long long limit = t > 0 ? (long long)t * 1000000ll : 2000000000ll;
  kern<<<grid, kFwd2Threads, smem, stream>>>(mq, mk, mv, o, lse, (int)S, (int)(H / Hkv),
                                             scale * kLog2e, limit, (int)n_pairs, (int)(B * H),
                                             head_group_for(n_pairs * B * H, B * H), (int)H,
                                             lay.o_token_major, lay.v_token_major);
  return check_launch("causal_attention_fwd");
}

}  // namespace

namespace attn {

int launch_fwd2_any(int head_dim, int fmt, const void* q, const void* k, const void* v, void* o,
                    float* lse, int64_t B, int64_t H, int64_t Hkv, int64_t S, float scale,
                    cudaStream_t stream, Layouts lay) {
  if (head_dim == 128)
    return fmt == 1 ? launch_fwd2<128, 1>(q, k, v, o, lse, B, H, Hkv, S, scale, stream, lay)
                    : launch_fwd2<128, 0>(q, k, v, o, lse, B, H, Hkv, S, scale, stream, lay);
  return fmt == 1 ? launch_fwd2<64, 1>(q, k, v, o, lse, B, H, Hkv, S, scale, stream, lay)
                  : launch_fwd2<64, 0>(q, k, v, o, lse, B, H, Hkv, S, scale, stream, lay);
}

}  // namespace attn
}  // namespace evg
