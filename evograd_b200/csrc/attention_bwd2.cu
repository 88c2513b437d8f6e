// Causal attention backward, warp-specialised and pipelined (sm_100a).
//
// Roles inside a block:
//   warp 0, lane 0   TMA producer: tiles of Q/K/V/dO (+ row statistics) into
//                    shared-memory rings, completion on "full" mbarriers, refills
//                    gated by "empty" mbarriers that the MMA thread commits;
//   warp 1           tcgen05.mma issuer: every product of the kernel, in an
//                    order that keeps the tensor pipe fed while the compute
//                    warps work on the previous tile;
//   warps 2..        compute threads: thread = one TMEM lane (score row) and one
//                    group of the tile's columns (8 warps in the dQ kernel,
//                    16 in the dK/dV kernel).
// A compute warp writes its 16-bit results only into TMEM columns it read
// itself, so no block-wide barrier is needed between reading scores and writing
// dS: the A operand of the following product is addressed k-step by k-step and
// need not be contiguous.
//
// dK/dV belong to the block that owns a key tile and dQ to the block that owns
// a query tile: deterministic, no atomics, at the price of 7 tile products
// where a fused backward with a float32 dQ reduction needs 5. On a B200 both
// kernels run into the board's power limit (sw_power_cap active, SM clock near
// 1.55 GHz); their time per tile product is within a few percent of what a
// library bf16 GEMM sustains under the same limit, so the number of tile
// products, not idle cycles between them, is what sets the time.
#include "attention_bwd_parts.cuh"

namespace evg {

__device__ int g_attn2_device_status = 0;

namespace {

using namespace umma;
using namespace attn;
using namespace attn_bwd;

constexpr int kThreads2 = 320;

// ------------------------------------------------------------------------ dQ
// grid = (query tiles, B*H). The block owns query tile `qtile` and walks key
// tiles j = 0..qtile:  S = Q K_j^T, dP = dO V_j^T, dS = exp2(S*c - lse2)*(dP - delta),
// dQ += dS K_j.
// TMEM (512 columns): [0,128) and [128,256) two score buffers (tile j uses
// buffer j%2; its dS goes back into the same buffer), [256,384) dP,
// [384,384+HD) dQ.
// Issue order of the MMA thread for tile j:  S(j+1), dP(j+1) [after the compute
// warps have pulled dP(j) into registers], dQ(j) [after dS(j) is in TMEM].
template <int HD, int FMT>
__global__ void __launch_bounds__(kThreads2, 1)
attn_bwd2_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                    const float* __restrict__ lse2_pad, const float* __restrict__ delta_pad,
                    void* __restrict__ dq_ptr, int S, int S_pad, int group, float scale,
                    long long wait_limit, int n_bh, int head_group, int heads, int v_tm,
                    int do_tm) {
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t TB = tile_bytes<HD>();
  BlockSetup bs = carve(smem_raw, 7 * TB);
  uint8_t* sQ = bs.smem;
  uint8_t* sDO = sQ + TB;
  // K is needed twice per tile (scores at the start, dQ at the end), V once:
  // three K stages and two V stages keep the TMA latency off the MMA thread.
  uint8_t* sK[3] = {sDO + TB, sDO + 2 * TB, sDO + 3 * TB};
  uint8_t* sV[2] = {sDO + 4 * TB, sDO + 5 * TB};
  uint64_t* qdo_full = bs.bars + 0;
  uint64_t* k_full = bs.bars + 1;    // [3]
  uint64_t* k_empty = bs.bars + 4;   // [3]
  uint64_t* v_full = bs.bars + 7;    // [2]
  uint64_t* v_empty = bs.bars + 9;   // [2]
  uint64_t* s_full = bs.bars + 11;   // [2]
  uint64_t* dp_full = bs.bars + 13;
  uint64_t* dp_free = bs.bars + 14;
  uint64_t* ds_full = bs.bars + 15;  // [2]
  uint64_t* done = bs.bars + 17;
  const Roles r = roles();
  int qtile, bh;  // heaviest tiles first (map_block)
  map_block(blockIdx.x, S_pad / kTile, n_bh, head_group, qtile, bh);
  qtile = S_pad / kTile - 1 - qtile;
  const int bh_kv = bh / group;  // `group` query heads share one k/v head
  const int q0 = qtile * kTile;
  const int n_it = qtile + 1;
  const float scale_log2 = scale * kLog2e;

  if (threadIdx.x == 0) {
    *bs.abort_flag = 0;
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(k_full + i, 1); mbar_init(k_empty + i, 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(v_full + i, 1); mbar_init(v_empty + i, 1);
      mbar_init(s_full + i, 1); mbar_init(ds_full + i, 8);
    }
    mbar_init(dp_full, 1); mbar_init(dp_free, 8); mbar_init(done, 1);
    fence_mbar_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v); prefetch_tensormap(&map_do);
  }
  __syncthreads();
  if (r.warp == 1) { tmem_alloc(bs.tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *bs.tmem_slot;
  const WaitCtx ctx{bs.abort_flag, &g_attn2_device_status, wait_limit};
  constexpr uint32_t idesc_s = instr_desc_f16(FMT, 128, 128, 0, 0);
  constexpr uint32_t idesc_d = instr_desc_f16(FMT, 128, HD, 0, 1);
  const uint32_t tSb[2] = {tmem, tmem + 128};
  const uint32_t tDP = tmem + 256, tDQ = tmem + 384;

  if (r.is_tma && r.lane == 0) {
    mbar_expect_tx(qdo_full, 2 * TB);
    load_tile<HD>(sQ, &map_q, q0, bh, qdo_full);
    load_tile_bh<HD>(sDO, &map_do, q0, bh, heads, do_tm, qdo_full);
    for (int j = 0; j < n_it; ++j) {
      const int ks = j % 3, vs = j & 1;
      if (j >= 3) mbar_wait(k_empty + ks, ((j / 3) - 1) & 1, ctx, 501);
      mbar_expect_tx(k_full + ks, TB);
      load_tile<HD>(sK[ks], &map_k, j * kTile, bh_kv, k_full + ks);
      if (j >= 2) mbar_wait(v_empty + vs, ((j >> 1) - 1) & 1, ctx, 510);
      mbar_expect_tx(v_full + vs, TB);
      load_tile_bh<HD>(sV[vs], &map_v, j * kTile, bh_kv, heads / group, v_tm, v_full + vs);
    }
  } else if (r.is_mma) {
    // All 32 lanes run this program; `lead` predicates the tcgen05 instructions.
    const bool lead = elect_one();
    mbar_wait(qdo_full, 0, ctx, 502);
    mbar_wait(k_full + 0, 0, ctx, 503);
    tc_fence_after_sync();
    issue_scores<HD>(lead, tSb[0], smem_u32(sQ), smem_u32(sK[0]), idesc_s);
    if (lead) mma_commit(s_full + 0);
    mbar_wait(v_full + 0, 0, ctx, 511);
    tc_fence_after_sync();
    issue_scores<HD>(lead, tDP, smem_u32(sDO), smem_u32(sV[0]), idesc_s);
    if (lead) { mma_commit(dp_full); mma_commit(v_empty + 0); }
    for (int j = 0; j < n_it; ++j) {
      const int b = j & 1;
      if (j + 1 < n_it) {
        const int b1 = (j + 1) & 1, k1 = (j + 1) % 3;
        mbar_wait(k_full + k1, ((j + 1) / 3) & 1, ctx, 504);
        tc_fence_after_sync();
        issue_scores<HD>(lead, tSb[b1], smem_u32(sQ), smem_u32(sK[k1]), idesc_s);
        if (lead) mma_commit(s_full + b1);
        mbar_wait(v_full + b1, ((j + 1) >> 1) & 1, ctx, 512);
        mbar_wait(dp_free, j & 1, ctx, 505);
        tc_fence_after_sync();
        issue_scores<HD>(lead, tDP, smem_u32(sDO), smem_u32(sV[b1]), idesc_s);
        if (lead) { mma_commit(dp_full); mma_commit(v_empty + b1); }
      }
      mbar_wait(ds_full + b, (j >> 1) & 1, ctx, 506);
      tc_fence_after_sync();
      // dS is stored as two 32-column halves at buffer columns 0 and 64.
      const DescBase kb = desc_base_mnmajor(smem_u32(sK[j % 3]), kTile);
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks)
        if (lead)
          mma_ts(tDQ, tSb[b] + (ks >> 2) * 64 + (ks & 3) * 8, desc_at(kb, kstep_mnmajor(ks)),
                 idesc_d, (j > 0 || ks > 0) ? 1u : 0u);
      if (lead) mma_commit(k_empty + (j % 3));
      __syncwarp();
    }
    if (lead) mma_commit(done);
  } else if (r.is_compute) {
    const uint32_t lane_base = (uint32_t)(r.quarter * 32) << 16;
    const int q_glob = q0 + r.row;
    const float lse2 = lse2_pad[(size_t)bh * S_pad + q_glob];
    const float delta = delta_pad[(size_t)bh * S_pad + q_glob];
    for (int j = 0; j < n_it; ++j) {
      const int b = j & 1;
      mbar_wait(s_full + b, (j >> 1) & 1, ctx, 507);
      mbar_wait(dp_full, j & 1, ctx, 508);
      __syncwarp();
      tc_fence_after_sync();
      uint32_t sr[64], dr[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tmem_ld32(tSb[b] + lane_base + r.half * 64 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[c * 32]));
        tmem_ld32(tDP + lane_base + r.half * 64 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&dr[c * 32]));
      }
      tmem_wait_ld();
      warp_arrive(dp_free, r.lane);
      const int kv0 = j * kTile + r.half * 64;
      const float nlse = -lse2;
      uint32_t dd[32];
      if (j == qtile) {  // diagonal tile: keys after the query are masked
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float d[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float pe = fast_exp2(fmaf(__uint_as_float(sr[2 * i + e]), scale_log2, nlse));
            if (kv0 + 2 * i + e > q_glob) pe = 0.f;
            d[e] = pe * (__uint_as_float(dr[2 * i + e]) - delta);
          }
          dd[i] = pack2<FMT>(d[0], d[1]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(sr[2 * i]), scale_log2, nlse));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sr[2 * i + 1]), scale_log2, nlse));
          dd[i] = pack2<FMT>(p0 * (__uint_as_float(dr[2 * i]) - delta),
                             p1 * (__uint_as_float(dr[2 * i + 1]) - delta));
        }
      }
      tmem_st32(tSb[b] + lane_base + r.half * 64, dd);
      tmem_wait_st();
      warp_arrive(ds_full + b, r.lane);
    }
    mbar_wait(done, 0, ctx, 509);
    __syncwarp();
    tc_fence_after_sync();
    store_rows<HD, FMT>(tDQ, dq_ptr, bh, q0, S, scale, r);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (r.warp == 1) tmem_dealloc(tmem, 512);
}

// -------------------------------------------------------------------- dK, dV
// grid = (key tiles, B*Hkv). The block owns key tile `kvt` and walks whole
// 128-row query tiles i >= kvt:
//   S^T = K Q_i^T                                 [128 keys x 128 queries]
//   dP^T = V dO_i^T                               two chunks of 64 queries
//   P^T = exp2(S^T*c - lse2_q), dS^T = P^T*(dP^T - delta_q)
//   dV += P^T dO_i, dK += dS^T Q_i                (A from TMEM, k-steps of 16 queries)
// TMEM: X [0,128) S^T; Y0 [128,192), Y1 [192,256) dP^T of query chunk 0 / 1,
// replaced in place by the 16-bit P^T / dS^T; [256,256+HD) dV; [384,384+HD) dK.
// The S^T product has N = 128, so its two shared-memory operands stay within the
// SM's 128 bytes per clock (a 64-column product needs 192). Program of the MMA
// warp for tile i:
//     S^T(i+1) -> X       as soon as the compute warps have pulled S^T(i) into registers
//     dV, dK (i, chunk 0) -> dP^T(i+1, chunk 0) -> Y0
//     dV, dK (i, chunk 1) -> dP^T(i+1, chunk 1) -> Y1
// The tensor pipe runs its instructions in order, so dP^T(i+1, ch) lands in Y_ch
// right behind the products that read it. The exponentials of tile i+1 run under
// the products of tile i, and the dS step of one chunk runs under the products of
// the other chunk, so no step of the chain  dP^T -> dS^T -> dV/dK -> dP^T  waits
// for the compute warps as long as they keep up.
// Q tiles sit in a ring of QST stages and dO tiles (with the row statistics) in
// a ring of two, each with its own full/empty barriers: Q(i+1) is wanted soon
// after dK(i-1) has released a stage, so with QST = 3 its load is already a tile
// ahead; dO(i+1) is only wanted after dV/dK(i, chunk 0).
// 4 * CG compute warps: warp (TMEM lane quarter q, column group g) handles
// CPW = 64 / CG query columns of each chunk and writes CPW/2 columns of P^T
// followed by CPW/2 of dS^T into the same CPW columns of Y_ch: it only ever
// overwrites what it has read itself. CG = 4 (16 warps, 32 elements per thread
// and tile) keeps the SM's issue slots and its special-function unit busier than
// CG = 2 does, with half the registers per thread.
template <int HD, int FMT, int QST, int CG>
__global__ void __launch_bounds__(64 + 128 * CG, 1)
attn_bwd2_dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                      const float* __restrict__ lse2_pad, const float* __restrict__ delta_pad,
                      void* __restrict__ dk_ptr, void* __restrict__ dv_ptr, int S, int S_pad,
                      int group, float scale, long long wait_limit, uint32_t smem_bytes, int n_bh,
                      int head_group, int heads_kv, int dv_tm, int v_tm, int do_tm) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t TB = tile_bytes<HD>();
  constexpr uint32_t kTiles = 4 + QST;
  BlockSetup bs = carve(smem_raw, kTiles * TB + 2048);
  // The launch reserves little more than the tiles themselves: if the dynamic
  // shared memory did not start on a 1024-byte boundary the carve-up would not
  // fit, which is reported instead of run.
  if ((uint32_t)(bs.smem - smem_raw) + kTiles * TB + 2048 + (uint32_t)kControlBytes > smem_bytes) {
    if (threadIdx.x == 0) atomicCAS(&g_attn2_device_status, 0, 699);
    return;
  }
  uint8_t* sK = bs.smem;
  uint8_t* sV = sK + TB;
  uint8_t* sDO0 = sV + TB;        // 2 stages
  uint8_t* sQ0 = sDO0 + 2 * TB;   // QST stages
  float* s_stat = reinterpret_cast<float*>(sQ0 + QST * TB);  // [stage][lse2 | delta][128]
  uint64_t* kv_full = bs.bars + 0;
  uint64_t* q_full = bs.bars + 1;    // [QST]
  uint64_t* q_empty = bs.bars + 4;   // [QST]
  uint64_t* do_full = bs.bars + 7;   // [2]
  uint64_t* do_empty = bs.bars + 9;  // [2]
  uint64_t* s_full = bs.bars + 11;
  uint64_t* x_free = bs.bars + 12;
  uint64_t* dp_full = bs.bars + 13;   // [2] per query chunk
  uint64_t* pds_full = bs.bars + 15;  // [2]
  uint64_t* done = bs.bars + 17;
  constexpr int CPW = 64 / CG;  // query columns of a chunk per compute warp
  // First packed P^T column (inside Y_ch) of the chunk's query k-step kk.
  auto p_col = [](int kk) { return (kk * 16 / CPW) * CPW + (kk * 16 % CPW) / 2; };
  const Roles r = roles();  // r.half is the warp's column group, 0 .. CG-1
  int kvt, bh;  // key tile 0 meets the most query tiles: heaviest first (map_block)
  map_block(blockIdx.x, S_pad / kTile, n_bh, head_group, kvt, bh);
  const int kv0 = kvt * kTile;
  const int n_it = S_pad / kTile - kvt;
  // Grouped-query attention: the query tiles of each of the `group` query heads
  // bh*group + hh in turn (iteration git = hh * n_it + it), accumulating in TMEM.
  const int n_git = group * n_it;
  const float scale_log2 = scale * kLog2e;

  if (threadIdx.x == 0) {
    *bs.abort_flag = 0;
    mbar_init(kv_full, 1); mbar_init(done, 1);
    for (int i = 0; i < QST; ++i) { mbar_init(q_full + i, 1); mbar_init(q_empty + i, 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(do_full + i, 1); mbar_init(do_empty + i, 1);
      mbar_init(dp_full + i, 1); mbar_init(pds_full + i, 4 * CG);
    }
    mbar_init(s_full, 1); mbar_init(x_free, 4 * CG);
    fence_mbar_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v); prefetch_tensormap(&map_do);
  }
  __syncthreads();
  if (r.warp == 1) { tmem_alloc(bs.tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *bs.tmem_slot;
  const WaitCtx ctx{bs.abort_flag, &g_attn2_device_status, wait_limit};
  constexpr uint32_t idesc_s = instr_desc_f16(FMT, 128, 128, 0, 0);
  constexpr uint32_t idesc_p = instr_desc_f16(FMT, 128, 64, 0, 0);
  constexpr uint32_t idesc_d = instr_desc_f16(FMT, 128, HD, 0, 1);
  const uint32_t tX = tmem;
  const uint32_t tY[2] = {tmem + 128, tmem + 192};
  const uint32_t tDV = tmem + 256, tDK = tmem + 384;

  if (r.is_tma && r.lane == 0) {
    mbar_expect_tx(kv_full, 2 * TB);
    load_tile<HD>(sK, &map_k, kv0, bh, kv_full);
    load_tile_bh<HD>(sV, &map_v, kv0, bh, heads_kv, v_tm, kv_full);
    int it = 0, bhq = bh * group, git = 0;
    int qs = 0, q_round = 0;  // Q stage of tile git and how often the ring has wrapped
    for (; git < n_git; ++git) {
      const int ds = git & 1;
      const int q0 = (kvt + it) * kTile;
      if (q_round > 0) mbar_wait(q_empty + qs, (q_round - 1) & 1, ctx, 621);
      if (*ctx.abort_flag) break;  // no new copies after a timeout
      mbar_expect_tx(q_full + qs, TB);
      load_tile<HD>(sQ0 + qs * TB, &map_q, q0, bhq, q_full + qs);
      if (git >= 2) mbar_wait(do_empty + ds, ((git >> 1) - 1) & 1, ctx, 631);
      if (!*ctx.abort_flag) {
        mbar_expect_tx(do_full + ds, TB + 1024);
        load_tile_bh<HD>(sDO0 + ds * TB, &map_do, q0, bhq, heads_kv * group, do_tm, do_full + ds);
        bulk_load_1d(s_stat + ds * 256, lse2_pad + (size_t)bhq * S_pad + q0, 512, do_full + ds);
        bulk_load_1d(s_stat + ds * 256 + 128, delta_pad + (size_t)bhq * S_pad + q0, 512,
                     do_full + ds);
      }
      if (++qs == QST) { qs = 0; ++q_round; }
      if (++it == n_it) { it = 0; ++bhq; }
    }
    if (*ctx.abort_flag) {
      // Let the copies still in flight land before the block returns: each of
      // these waits gives up after the same cycle budget.
      mbar_drain(kv_full, 0, wait_limit);
      for (int g = git > QST ? git - QST : 0; g < git; ++g)
        mbar_drain(q_full + g % QST, (uint32_t)((g / QST) & 1), wait_limit);
      for (int g = git > 2 ? git - 2 : 0; g < git; ++g)
        mbar_drain(do_full + (g & 1), (uint32_t)((g >> 1) & 1), wait_limit);
    }
  } else if (r.is_mma) {
    const bool lead = elect_one();
    const DescBase v_base = desc_base_kmajor(smem_u32(sV));
    // dP^T of query chunk ch: B operand = rows [64 ch, 64 ch + 64) of a dO tile.
    auto issue_dp = [&](int ch, uint32_t do_saddr) {
      const DescBase da = desc_base_kmajor(do_saddr + ch * 64 * 128);
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        if (lead)
          mma_ss(tY[ch], desc_at(v_base, kstep_kmajor(kTile, ks)),
                 desc_at(da, kstep_kmajor(kTile, ks)), idesc_p, ks > 0 ? 1u : 0u);
      if (lead) mma_commit(dp_full + ch);
    };
    mbar_wait(kv_full, 0, ctx, 622);
    mbar_wait(q_full + 0, 0, ctx, 623);
    tc_fence_after_sync();
    issue_scores<HD>(lead, tX, smem_u32(sK), smem_u32(sQ0), idesc_s);
    if (lead) mma_commit(s_full);
    mbar_wait(do_full + 0, 0, ctx, 632);
    tc_fence_after_sync();
    issue_dp(0, smem_u32(sDO0));
    issue_dp(1, smem_u32(sDO0));
    int qs = 0, q_par = 0;  // Q stage of tile c and the parity of its full barrier
    for (int c = 0; c < n_git; ++c) {
      const int ds = c & 1, ds1 = ds ^ 1;
      const bool more = c + 1 < n_git;
      int qs1 = qs + 1, q_par1 = q_par;
      if (qs1 == QST) { qs1 = 0; q_par1 ^= 1; }
      if (more) {
        mbar_wait(q_full + qs1, q_par1, ctx, 624);
        mbar_wait(x_free, c & 1, ctx, 625);
        tc_fence_after_sync();
        issue_scores<HD>(lead, tX, smem_u32(sK), smem_u32(sQ0 + qs1 * TB), idesc_s);
        if (lead) mma_commit(s_full);
      }
      const uint32_t do_saddr = smem_u32(sDO0 + ds * TB), q_saddr = smem_u32(sQ0 + qs * TB);
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        mbar_wait(pds_full + ch, c & 1, ctx, 626);
        tc_fence_after_sync();
        // Query k-step kk of the chunk (16 queries = 8 packed columns): its P^T
        // columns start at p_col(kk), dS^T sits CPW/2 columns after P^T.
        const DescBase dob = desc_base_mnmajor(do_saddr + ch * 64 * 128, kTile);
        const DescBase qb = desc_base_mnmajor(q_saddr + ch * 64 * 128, kTile);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          if (lead)
            mma_ts(tDV, tY[ch] + p_col(kk), desc_at(dob, kstep_mnmajor(kk)), idesc_d,
                   (c > 0 || ch > 0 || kk > 0) ? 1u : 0u);
        if (lead && ch == 1) mma_commit(do_empty + ds);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          if (lead)
            mma_ts(tDK, tY[ch] + p_col(kk) + CPW / 2, desc_at(qb, kstep_mnmajor(kk)), idesc_d,
                   (c > 0 || ch > 0 || kk > 0) ? 1u : 0u);
        if (lead && ch == 1) mma_commit(q_empty + qs);
        if (more) {
          if (ch == 0) {
            mbar_wait(do_full + ds1, ((c + 1) >> 1) & 1, ctx, 633);
            tc_fence_after_sync();
          }
          issue_dp(ch, smem_u32(sDO0 + ds1 * TB));
        }
      }
      qs = qs1;
      q_par = q_par1;
      __syncwarp();
    }
    if (lead) mma_commit(done);
  } else if (r.is_compute) {
    const uint32_t lane_base = (uint32_t)(r.quarter * 32) << 16;
    const int kv_glob = kv0 + r.row;
    const int col0 = r.half * CPW;  // first query column inside a chunk of this warp
    int it = 0;                     // query-tile index within the current query head
    for (int c = 0; c < n_git; ++c) {
      const int ds = c & 1;
      mbar_wait(do_full + ds, (c >> 1) & 1, ctx, 627);  // row statistics landed
      mbar_wait(s_full, c & 1, ctx, 628);
      __syncwarp();
      tc_fence_after_sync();
      uint32_t sr[2][CPW];  // [chunk][columns]
      tmem_ld(tX + lane_base + col0, sr[0]);
      tmem_ld(tX + lane_base + 64 + col0, sr[1]);
      tmem_wait_ld();
      warp_arrive(x_free, r.lane);
      const float* stat = s_stat + ds * 256;
      float p[2][CPW];
      uint32_t pp[2][CPW / 2];
      if (it == 0) {  // diagonal tile: queries before the key are masked
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const float4* lse4 = reinterpret_cast<const float4*>(stat + ch * 64 + col0);
          const int q_first = kvt * kTile + ch * 64 + col0;
#pragma unroll
          for (int g = 0; g < CPW / 4; ++g) {
            const float4 l4 = lse4[g];
            const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float pe =
                  fast_exp2(fmaf(__uint_as_float(sr[ch][4 * g + e]), scale_log2, -lv[e]));
              p[ch][4 * g + e] = (q_first + 4 * g + e < kv_glob) ? 0.f : pe;
            }
          }
        }
      } else {
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const float4* lse4 = reinterpret_cast<const float4*>(stat + ch * 64 + col0);
#pragma unroll
          for (int g = 0; g < CPW / 4; ++g) {
            const float4 l4 = lse4[g];
            const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              p[ch][4 * g + e] =
                  fast_exp2(fmaf(__uint_as_float(sr[ch][4 * g + e]), scale_log2, -lv[e]));
          }
        }
      }
#pragma unroll
      for (int ch = 0; ch < 2; ++ch)
#pragma unroll
        for (int g = 0; g < CPW / 2; ++g) pp[ch][g] = pack2<FMT>(p[ch][2 * g], p[ch][2 * g + 1]);
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        mbar_wait(dp_full + ch, c & 1, ctx, 629);
        __syncwarp();
        tc_fence_after_sync();
        uint32_t dr[CPW];
        tmem_ld(tY[ch] + lane_base + col0, dr);
        tmem_wait_ld();
        const float4* del4 = reinterpret_cast<const float4*>(stat + 128 + ch * 64 + col0);
        uint32_t dd[CPW / 2];
#pragma unroll
        for (int g = 0; g < CPW / 4; ++g) {
          const float4 d4 = del4[g];
          const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
          float d[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            d[e] = p[ch][4 * g + e] * (__uint_as_float(dr[4 * g + e]) - dv[e]);
          dd[2 * g] = pack2<FMT>(d[0], d[1]);
          dd[2 * g + 1] = pack2<FMT>(d[2], d[3]);
        }
        tmem_st(tY[ch] + lane_base + col0, pp[ch]);
        tmem_st(tY[ch] + lane_base + col0 + CPW / 2, dd);
        tmem_wait_st();
        warp_arrive(pds_full + ch, r.lane);
      }
      if (++it == n_it) it = 0;
    }
    mbar_wait(done, 0, ctx, 630);
    __syncwarp();
    tc_fence_after_sync();
    store_rows<HD, FMT, CG>(tDV, dv_ptr, bh, kv0, S, 1.0f, r, heads_kv, dv_tm);
    store_rows<HD, FMT, CG>(tDK, dk_ptr, bh, kv0, S, scale, r);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (r.warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------- host side
template <int HD, int FMT>
int launch_bwd2(const void* dout, const void* q, const void* k, const void* v, const void* o,
                const float* lse, void* dq, void* dk, void* dv, float* workspace, int64_t B,
                int64_t H, int64_t Hkv, int64_t S, float scale, cudaStream_t stream, Layouts lay) {
  CUtensorMap mq, mk, mv, mdo;
  const int group = (int)(H / Hkv);
  if (!encode_tile_map_16bit(&mq, q, FMT, HD, S, B * H, kTile) ||
      !encode_tile_map_16bit(&mk, k, FMT, HD, S, B * Hkv, kTile) ||
      !encode_bh_map(&mv, v, FMT, HD, S, Hkv, B, lay.v_token_major) ||
      !encode_bh_map(&mdo, dout, FMT, HD, S, H, B, lay.do_token_major))
    return fail(EVG_ELAUNCH, "causal_attention_bwd: cuTensorMapEncodeTiled failed");
  const int64_t n_q = (S + kTile - 1) / kTile;
  const int64_t S_pad = n_q * kTile;
  const int64_t padded_rows = B * H * S_pad;
  float* lse2_pad = workspace;
  float* delta_pad = workspace + padded_rows;
  {
    constexpr int TPR = HD / 8;
    const int64_t threads = padded_rows * TPR;  // a multiple of 256
    attn_prepare_kernel<HD, FMT><<<(unsigned)(threads / 256), 256, 0, stream>>>(
        dout, o, lse, lse2_pad, delta_pad, (int)S, (int)S_pad, padded_rows, (int)H,
        lay.o_token_major, lay.do_token_major);
    if (int rc = check_launch("causal_attention_bwd prepare")) return rc;
  }
  // Head size 128: one fused pass with a float32 dQ copy (behind the two arrays
  // above in the scratch) unless bit-reproducible results are asked for.
  if constexpr (HD == 128) {
    if (!tune("attention.two_kernel_bwd"))
      return launch_bwd3_128(FMT, mq, mk, mv, mdo, lse2_pad, delta_pad, workspace + 2 * padded_rows,
                             dq, dk, dv, B, H, Hkv, S, S_pad, scale, stream, lay);
  }
  dim3 grid((unsigned)(n_q * B * H));
  const long long limit = wait_limit_cycles2();
  {
    // 7 tiles of 32 KB at head size 128 leave 768 bytes of the 227 KB for alignment.
    size_t smem = 7 * tile_bytes<HD>() + 2048 + kControlBytes + 1024;
    const size_t most = (size_t)device_info().max_smem_optin;
    if (smem > most) smem = most;
    constexpr int CG = 4;  // 16 compute warps
    auto kern = attn_bwd2_dkdv_kernel<HD, FMT, 3, CG>;
    if (int rc = reserve_smem(kern, smem)) return rc;
    dim3 grid_kv((unsigned)(n_q * B * Hkv));
    kern<<<grid_kv, 64 + 128 * CG, smem, stream>>>(mq, mk, mv, mdo, lse2_pad, delta_pad, dk, dv,
                                                   (int)S, (int)S_pad, group, scale, limit,
                                                   (uint32_t)smem, (int)(B * Hkv),
                                                   head_group_for(n_q * B * Hkv, B * Hkv), (int)Hkv,
                                                   lay.dv_token_major, lay.v_token_major,
                                                   lay.do_token_major);
    if (int rc = check_launch("causal_attention_bwd dkdv")) return rc;
  }
  {
    const size_t smem = 7 * tile_bytes<HD>() + kControlBytes + 1024;
    auto kern = attn_bwd2_dq_kernel<HD, FMT>;
    if (int rc = reserve_smem(kern, smem)) return rc;
    kern<<<grid, kThreads2, smem, stream>>>(mq, mk, mv, mdo, lse2_pad, delta_pad, dq, (int)S,
                                            (int)S_pad, group, scale, limit, (int)(B * H),
                                            head_group_for(n_q * B * H, B * H), (int)H,
                                            lay.v_token_major, lay.do_token_major);
    if (int rc = check_launch("causal_attention_bwd dq")) return rc;
  }
  return EVG_OK;
}

int read_attention2_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_attn2_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attn2_device_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_attention2_status_registered =
    (register_device_status(read_attention2_status), true);

}  // namespace

namespace attn {

int64_t bwd2_workspace_bytes(int64_t B, int64_t H, int64_t S, int64_t D) {
  const int64_t S_pad = (S + kTile - 1) / kTile * kTile;
  const int64_t rows = B * H * S_pad;
  // two statistics per padded row; head size 128 adds the float32 dQ copy
  return (2 * rows + (D == 128 ? rows * 128 : 0)) * (int64_t)sizeof(float);
}

int launch_bwd2_any(int head_dim, int fmt, const void* dout, const void* q, const void* k,
                    const void* v, const void* o, const float* lse, void* dq, void* dk, void* dv,
                    float* workspace, int64_t B, int64_t H, int64_t Hkv, int64_t S, float scale,
                    cudaStream_t stream, Layouts lay) {
  if (head_dim == 128)
    return fmt == 1 ? launch_bwd2<128, 1>(dout, q, k, v, o, lse, dq, dk, dv, workspace, B, H, Hkv,
                                          S, scale, stream, lay)
                    : launch_bwd2<128, 0>(dout, q, k, v, o, lse, dq, dk, dv, workspace, B, H, Hkv,
                                          S, scale, stream, lay);
  return fmt == 1 ? launch_bwd2<64, 1>(dout, q, k, v, o, lse, dq, dk, dv, workspace, B, H, Hkv, S,
                                       scale, stream, lay)
                  : launch_bwd2<64, 0>(dout, q, k, v, o, lse, dq, dk, dv, workspace, B, H, Hkv, S,
                                       scale, stream, lay);
}

}  // namespace attn
}  // namespace evg
