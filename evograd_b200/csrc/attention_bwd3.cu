// Causal attention backward in ONE pass over the score tiles, head size 128
// (sm_100a): dQ, dK and dV from five tile products per (key tile, query tile)
// pair, where the split into a dK/dV kernel and a dQ kernel needs seven.
//
// grid = (key tiles, B*Hkv). The block owns key tile `kvt`, keeps K and V in
// shared memory and dV, dK in tensor memory, and walks the query tiles i >= kvt
// in chunks of 64 queries (two per tile):
//   S^T   = K Q_i^T                       [128 keys x 128 queries], once per tile
//   dP^T  = V dO^T                        [128 keys x 64 queries]
//   P^T   = exp2(S^T c - lse2_q),  dS^T = P^T (dP^T - delta_q)
//   dV   += P^T dO,   dK += dS^T Q        (A from tensor memory)
//   dQ^T  = K^T dS^T                      [128 head columns x 64 queries]
// dQ^T is the only product whose result belongs to another block's rows too: the
// compute warps take it out of tensor memory and add it to a float32 copy of dQ
// with red.global.add (one 128-byte line per warp instruction); a last small
// kernel scales and rounds that copy to the 16-bit dQ. The order of the float32
// additions is not fixed, so dQ can differ in the last bit from run to run; the
// two-kernel backward (attention_bwd2.cu) stays available for bit-reproducible
// results.
//
// Tensor memory (512 columns): X [0,128) S^T; Y [128,192) dP^T of the current
// chunk, replaced in place by the 16-bit P^T and dS^T; D [192,256) dQ^T of the
// current chunk; [256,384) dV; [384,512) dK. dS^T is also written to shared
// memory (16 KB per chunk, two buffers, 128-byte swizzle) as the B operand of
// the dQ^T product, whose A operand is the K tile read MN-major.
//
// Shared memory: K, V, two dO stages, two Q stages, two dS^T chunks: 7 x 32 KB
// plus the row statistics.
//
// Program of the MMA warp for tile c (chunks h = 2c, 2c+1):
//   dV,dK(2c)   -> dP^T(2c+1) -> dQ^T(2c)   -> S^T(c+1)
//   dV,dK(2c+1) -> dP^T(2c+2) -> dQ^T(2c+1)
// The tensor pipe runs in order, so dP^T(h+1) lands in Y right behind the
// products that read P^T/dS^T(h) from it. The compute warps work one chunk
// ahead with the exponentials: while the products of chunk h run they turn
// S^T of chunk h+1 into P^T (in registers) and take dQ^T(h-1) out of D.
#include "attention_bwd_parts.cuh"

namespace evg {

__device__ int g_attn3_device_status = 0;

namespace {

using namespace umma;
using namespace attn;
using namespace attn_bwd;

constexpr int kCG3 = 4;                       // column groups of compute warps
// TMA warp, MMA warp, 16 compute warps, 4 warps that take dQ^T out of tensor memory
constexpr int kThreads3 = 64 + 128 * kCG3 + 128;
constexpr uint32_t kChunkBytes = 64 * 128 * 2;  // 64 queries x 128 keys of 16-bit dS^T

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void red_add_f32(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

template <int FMT>
__global__ void __launch_bounds__(kThreads3, 1)
attn_bwd3_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                 const float* __restrict__ lse2_pad, const float* __restrict__ delta_pad,
                 float* __restrict__ dq_acc, void* __restrict__ dk_ptr, void* __restrict__ dv_ptr,
                 int S, int S_pad, int group, float scale, long long wait_limit,
                 uint32_t smem_bytes, int n_bh, int head_group, int heads_kv, int dv_tm,
                 int v_tm, int do_tm) {
  constexpr int HD = 128;
  constexpr int CG = kCG3;
  constexpr int CPW = 64 / CG;  // query columns of a chunk per compute warp (16)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t TB = tile_bytes<HD>();
  constexpr uint32_t kTiles = 7;
  BlockSetup bs = carve(smem_raw, kTiles * TB + 2048);
  if ((uint32_t)(bs.smem - smem_raw) + kTiles * TB + 2048 + (uint32_t)kControlBytes > smem_bytes) {
    if (threadIdx.x == 0) atomicCAS(&g_attn3_device_status, 0, 799);
    return;
  }
  uint8_t* sK = bs.smem;
  uint8_t* sV = sK + TB;
  uint8_t* sDO0 = sV + TB;       // 2 stages
  uint8_t* sQ0 = sDO0 + 2 * TB;  // 2 stages
  uint8_t* sDS = sQ0 + 2 * TB;   // 2 chunks of dS^T
  float* s_stat = reinterpret_cast<float*>(sDS + TB);  // [stage][lse2 | delta][128]
  uint64_t* kv_full = bs.bars + 0;
  uint64_t* q_full = bs.bars + 1;    // [2]
  uint64_t* q_empty = bs.bars + 3;   // [2]
  uint64_t* do_full = bs.bars + 5;   // [2]
  uint64_t* do_empty = bs.bars + 7;  // [2]
  uint64_t* s_full = bs.bars + 9;
  uint64_t* x_free = bs.bars + 10;
  uint64_t* dp_full = bs.bars + 11;   // [2] by chunk parity
  uint64_t* pds_full = bs.bars + 13;  // [2] P^T / dS^T of the chunk are in Y
  uint64_t* ds_full = bs.bars + 15;   // [2] dS^T of the chunk is in shared memory
  uint64_t* dq_full = bs.bars + 17;   // [2] dQ^T of the chunk is in D
  uint64_t* d_free = bs.bars + 19;    // [2] D has been read
  uint64_t* done = bs.bars + 21;
  const Roles r = roles();  // r.half is the warp's column group, 0 .. CG-1
  // Key tile 0 meets the most query tiles: the heaviest blocks of a group of heads
  // start first (map_block).
  int kvt, bh;
  map_block(blockIdx.x, S_pad / kTile, n_bh, head_group, kvt, bh);
  const int kv0 = kvt * kTile;
  const int n_it = S_pad / kTile - kvt;
  // Grouped-query attention: the query tiles of each of the `group` query heads
  // bh*group + hh in turn (iteration c = hh * n_it + it), accumulating dK/dV.
  const int n_git = group * n_it;
  const float scale_log2 = scale * kLog2e;

  if (threadIdx.x == 0) {
    *bs.abort_flag = 0;
    mbar_init(kv_full, 1); mbar_init(done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full + i, 1); mbar_init(q_empty + i, 1);
      mbar_init(do_full + i, 1); mbar_init(do_empty + i, 1);
      mbar_init(dp_full + i, 1); mbar_init(pds_full + i, 4 * CG);
      mbar_init(ds_full + i, 4 * CG); mbar_init(dq_full + i, 1); mbar_init(d_free + i, 4);
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
  const WaitCtx ctx{bs.abort_flag, &g_attn3_device_status, wait_limit};
  constexpr uint32_t idesc_s = instr_desc_f16(FMT, 128, 128, 0, 0);
  constexpr uint32_t idesc_p = instr_desc_f16(FMT, 128, 64, 0, 0);
  constexpr uint32_t idesc_d = instr_desc_f16(FMT, 128, HD, 0, 1);
  constexpr uint32_t idesc_q = instr_desc_f16(FMT, 128, 64, 1, 1);
  const uint32_t tX = tmem, tY = tmem + 128, tD = tmem + 192;
  const uint32_t tDV = tmem + 256, tDK = tmem + 384;

  if (r.is_tma && r.lane == 0) {
    mbar_expect_tx(kv_full, 2 * TB);
    load_tile<HD>(sK, &map_k, kv0, bh, kv_full);
    load_tile_bh<HD>(sV, &map_v, kv0, bh, heads_kv, v_tm, kv_full);
    int it = 0, bhq = bh * group, git = 0;
    for (; git < n_git; ++git) {
      const int st = git & 1;
      const int q0 = (kvt + it) * kTile;
      if (git >= 2) mbar_wait(q_empty + st, ((git >> 1) - 1) & 1, ctx, 721);
      if (*ctx.abort_flag) break;  // no new copies after a timeout
      mbar_expect_tx(q_full + st, TB);
      load_tile<HD>(sQ0 + st * TB, &map_q, q0, bhq, q_full + st);
      if (git >= 2) mbar_wait(do_empty + st, ((git >> 1) - 1) & 1, ctx, 731);
      if (!*ctx.abort_flag) {
        mbar_expect_tx(do_full + st, TB + 1024);
        load_tile_bh<HD>(sDO0 + st * TB, &map_do, q0, bhq, heads_kv * group, do_tm, do_full + st);
        bulk_load_1d(s_stat + st * 256, lse2_pad + (size_t)bhq * S_pad + q0, 512, do_full + st);
        bulk_load_1d(s_stat + st * 256 + 128, delta_pad + (size_t)bhq * S_pad + q0, 512,
                     do_full + st);
      }
      if (++it == n_it) { it = 0; ++bhq; }
    }
    if (*ctx.abort_flag) {
      // Let the copies still in flight land before the block returns: each of
      // these waits gives up after the same cycle budget.
      mbar_drain(kv_full, 0, wait_limit);
      for (int g = git > 2 ? git - 2 : 0; g < git; ++g) {
        mbar_drain(q_full + (g & 1), (uint32_t)((g >> 1) & 1), wait_limit);
        mbar_drain(do_full + (g & 1), (uint32_t)((g >> 1) & 1), wait_limit);
      }
    }
  } else if (r.is_mma) {
    const bool lead = elect_one();
    const DescBase v_base = desc_base_kmajor(smem_u32(sV));
    const DescBase kt_base = desc_base_mnmajor(smem_u32(sK), kTile);
    // dP^T of query chunk ch: B operand = rows [64 ch, 64 ch + 64) of a dO tile.
    auto issue_dp = [&](int ch, uint32_t do_saddr) {
      const DescBase da = desc_base_kmajor(do_saddr + ch * 64 * 128);
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        if (lead)
          mma_ss(tY, desc_at(v_base, kstep_kmajor(kTile, ks)), desc_at(da, kstep_kmajor(kTile, ks)),
                 idesc_p, ks > 0 ? 1u : 0u);
      if (lead) mma_commit(dp_full + ch);
    };
    // Query k-step kk of the chunk (16 queries): P^T in Y columns [16 kk, 16 kk + 8),
    // dS^T in the 8 columns behind it (the layout the compute warps write).
    auto issue_dv = [&](int ch, uint32_t do_saddr, bool first) {
      const DescBase dob = desc_base_mnmajor(do_saddr + ch * 64 * 128, kTile);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        if (lead)
          mma_ts(tDV, tY + kk * CPW, desc_at(dob, kstep_mnmajor(kk)), idesc_d,
                 (first && kk == 0) ? 0u : 1u);
    };
    auto issue_dk = [&](int ch, uint32_t q_saddr, bool first) {
      const DescBase qb = desc_base_mnmajor(q_saddr + ch * 64 * 128, kTile);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        if (lead)
          mma_ts(tDK, tY + kk * CPW + CPW / 2, desc_at(qb, kstep_mnmajor(kk)), idesc_d,
                 (first && kk == 0) ? 0u : 1u);
    };
    // dQ^T of chunk ch: A = K^T (the K tile read MN-major), B = dS^T chunk.
    auto issue_dq = [&](int ch) {
      const DescBase dsb = desc_base_mnmajor(smem_u32(sDS) + ch * kChunkBytes, kTile);
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks)
        if (lead)
          mma_ss(tD, desc_at(kt_base, kstep_mnmajor(ks)), desc_at(dsb, kstep_mnmajor(ks)), idesc_q,
                 ks > 0 ? 1u : 0u);
      if (lead) mma_commit(dq_full + ch);
    };
    mbar_wait(kv_full, 0, ctx, 722);
    mbar_wait(q_full + 0, 0, ctx, 723);
    tc_fence_after_sync();
    issue_scores<HD>(lead, tX, smem_u32(sK), smem_u32(sQ0), idesc_s);
    if (lead) mma_commit(s_full);
    mbar_wait(do_full + 0, 0, ctx, 732);
    tc_fence_after_sync();
    issue_dp(0, smem_u32(sDO0));
    for (int c = 0; c < n_git; ++c) {
      const int st = c & 1, st1 = st ^ 1;
      const uint32_t par = (uint32_t)(c & 1), par1 = (uint32_t)(((c + 1) >> 1) & 1);
      const bool more = c + 1 < n_git;
      const uint32_t do_saddr = smem_u32(sDO0 + st * TB), q_saddr = smem_u32(sQ0 + st * TB);
      // One wait on the critical path per chunk (P^T / dS^T are ready), with the
      // waits that are normally satisfied long before taken care of ahead of it:
      // every wait, satisfied or not, costs this warp about a hundred cycles, and
      // the tensor pipe's queue is only a few instructions deep. dQ^T runs one
      // chunk behind, so its operand in shared memory and its place in D are
      // ready by the time it is issued.
      // chunk 0
      if (c > 0) {
        mbar_wait(d_free + 0, par ^ 1u, ctx, 726);
        mbar_wait(ds_full + 1, par ^ 1u, ctx, 725);
      }
      mbar_wait(pds_full + 0, par, ctx, 724);
      tc_fence_after_sync();
      issue_dv(0, do_saddr, c == 0);
      issue_dk(0, q_saddr, c == 0);
      issue_dp(1, do_saddr);
      if (c > 0) issue_dq(1);  // of tile c - 1
      if (more) {
        mbar_wait(q_full + st1, par1, ctx, 727);
        mbar_wait(x_free, par, ctx, 728);
        tc_fence_after_sync();
        issue_scores<HD>(lead, tX, smem_u32(sK), smem_u32(sQ0 + st1 * TB), idesc_s);
        if (lead) mma_commit(s_full);
      }
      // chunk 1
      if (c > 0) mbar_wait(d_free + 1, par ^ 1u, ctx, 735);
      mbar_wait(ds_full + 0, par, ctx, 734);
      if (more) mbar_wait(do_full + st1, par1, ctx, 733);
      mbar_wait(pds_full + 1, par, ctx, 729);
      tc_fence_after_sync();
      issue_dv(1, do_saddr, false);
      if (lead) mma_commit(do_empty + st);
      issue_dk(1, q_saddr, false);
      if (lead) mma_commit(q_empty + st);
      if (more) issue_dp(0, smem_u32(sDO0 + st1 * TB));
      issue_dq(0);
      __syncwarp();
    }
    {
      const uint32_t last = (uint32_t)((n_git - 1) & 1);
      mbar_wait(d_free + 0, last, ctx, 736);
      mbar_wait(ds_full + 1, last, ctx, 737);
      tc_fence_after_sync();
      issue_dq(1);
    }
    if (lead) mma_commit(done);
  } else if (r.warp >= 2 + 4 * CG) {
    // dQ^T of every chunk: this warp's 32 lanes (head columns) x 64 query columns
    // of D, one 128-byte line of the float32 dQ copy per warp instruction. The
    // additions queue up behind the L2's float32 adders, which is why they have
    // warps of their own: nothing else waits for them.
    const uint32_t lane_base = (uint32_t)(r.quarter * 32) << 16;
    int it = 0, bhq = bh * group;
    for (int c = 0; c < n_git; ++c) {
      const uint32_t par = (uint32_t)(c & 1);
      float* tile_dst = dq_acc + ((size_t)bhq * S_pad + (size_t)(kvt + it) * kTile) * HD + r.row;
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        mbar_wait(dq_full + ch, par, ctx, 741);
        __syncwarp();
        tc_fence_after_sync();
        uint32_t acc[2][32];
        tmem_ld(tD + lane_base, acc[0]);
        tmem_ld(tD + lane_base + 32, acc[1]);
        tmem_wait_ld();
        warp_arrive(d_free + ch, r.lane);
        float* dst = tile_dst + ch * 64 * HD;
#pragma unroll
        for (int j = 0; j < 64; ++j) red_add_f32(dst + j * HD, __uint_as_float(acc[j >> 5][j & 31]));
      }
      if (++it == n_it) { it = 0; ++bhq; }
    }
  } else if (r.is_compute) {
    const uint32_t lane_base = (uint32_t)(r.quarter * 32) << 16;
    const int kv_glob = kv0 + r.row;
    const int col0 = r.half * CPW;  // first query column inside a chunk of this warp
    f32x2 p2[CPW / 2];  // P^T of the chunk that comes next, two query columns per element
    uint32_t pp[CPW / 2];
    const f32x2 neg_scale2 = f2_splat(-scale_log2);
    // P^T of one chunk from 16 columns of X, two columns per packed instruction:
    // t = lse2 - s c, p = 2^-t. `diag`: queries before the key are masked. When
    // `release` is set, X is handed back as soon as its columns are in registers.
    auto exp_chunk = [&](uint32_t x_col, const float* lse_ptr, bool diag, int q_first, bool release) {
      uint32_t sr[CPW];
      tmem_ld(tX + lane_base + x_col, sr);
      tmem_wait_ld();
      if (release) warp_arrive(x_free, r.lane);
      const float4* lse4 = reinterpret_cast<const float4*>(lse_ptr);
#pragma unroll
      for (int g = 0; g < CPW / 4; ++g) {
        const float4 l4 = lse4[g];
        const f32x2 t01 = f2_fma(f2_make(__uint_as_float(sr[4 * g]), __uint_as_float(sr[4 * g + 1])),
                                 neg_scale2, f2_make(l4.x, l4.y));
        const f32x2 t23 = f2_fma(f2_make(__uint_as_float(sr[4 * g + 2]), __uint_as_float(sr[4 * g + 3])),
                                 neg_scale2, f2_make(l4.z, l4.w));
        float t[4];
        f2_split(t01, t[0], t[1]);
        f2_split(t23, t[2], t[3]);
        float pe[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) pe[e] = fast_exp2(-t[e]);
        if (diag) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (q_first + 4 * g + e < kv_glob) pe[e] = 0.f;
        }
        p2[2 * g] = f2_make(pe[0], pe[1]);
        p2[2 * g + 1] = f2_make(pe[2], pe[3]);
        pp[2 * g] = pack2<FMT>(pe[0], pe[1]);
        pp[2 * g + 1] = pack2<FMT>(pe[2], pe[3]);
      }
    };
    int it = 0;
    // P^T of the very first chunk
    mbar_wait(do_full + 0, 0, ctx, 742);
    mbar_wait(s_full, 0, ctx, 743);
    __syncwarp();
    tc_fence_after_sync();
    exp_chunk(col0, s_stat + col0, true, kvt * kTile + col0, false);
    for (int c = 0; c < n_git; ++c) {
      const int st = c & 1;
      const uint32_t par = (uint32_t)(c & 1);
      const float* stat = s_stat + st * 256;
      const int q0 = (kvt + it) * kTile;
      const int it1 = it + 1 == n_it ? 0 : it + 1;
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        // dS^T of chunk (c, ch): into Y behind P^T, and into shared memory
        mbar_wait(dp_full + ch, par, ctx, 744);
        __syncwarp();
        tc_fence_after_sync();
        uint32_t dr[CPW];
        tmem_ld(tY + lane_base + col0, dr);
        tmem_wait_ld();
        const float4* del4 = reinterpret_cast<const float4*>(stat + 128 + ch * 64 + col0);
        uint32_t dd[CPW / 2];
        const f32x2 minus_one2 = f2_splat(-1.0f);
#pragma unroll
        for (int g = 0; g < CPW / 4; ++g) {
          const float4 d4 = del4[g];
          // dS = P (dP - delta), two columns at a time
          const f32x2 a01 = f2_fma(f2_make(d4.x, d4.y), minus_one2,
                                   f2_make(__uint_as_float(dr[4 * g]), __uint_as_float(dr[4 * g + 1])));
          const f32x2 a23 = f2_fma(f2_make(d4.z, d4.w), minus_one2,
                                   f2_make(__uint_as_float(dr[4 * g + 2]), __uint_as_float(dr[4 * g + 3])));
          float d[4];
          f2_split(f2_mul(p2[2 * g], a01), d[0], d[1]);
          f2_split(f2_mul(p2[2 * g + 1], a23), d[2], d[3]);
          dd[2 * g] = pack2<FMT>(d[0], d[1]);
          dd[2 * g + 1] = pack2<FMT>(d[2], d[3]);
        }
        // P^T / dS^T into Y first: the products that wait for them are the critical path.
        tmem_st(tY + lane_base + col0, pp);
        tmem_st(tY + lane_base + col0 + CPW / 2, dd);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (r.lane == 0) mbar_arrive(pds_full + ch);
        if (c > 0) mbar_wait(dq_full + ch, par ^ 1u, ctx, 748);  // the buffer's last reader is done
        {
          // dS^T for the dQ^T product: row r.row (a key) of the chunk's [128 keys x 64
          // queries] tile, 16-byte pieces 2g and 2g+1 of its 128 bytes, at their
          // swizzled places.
          uint8_t* row_ptr = sDS + ch * kChunkBytes + r.row * 128;
          const int sw = r.row & 7;
          *reinterpret_cast<uint4*>(row_ptr + (((2 * r.half) ^ sw) << 4)) =
              make_uint4(dd[0], dd[1], dd[2], dd[3]);
          *reinterpret_cast<uint4*>(row_ptr + (((2 * r.half + 1) ^ sw) << 4)) =
              make_uint4(dd[4], dd[5], dd[6], dd[7]);
        }
        // P^T of the chunk after this one
        if (ch == 0) {
          exp_chunk(64 + col0, stat + 64 + col0, it == 0, q0 + 64 + col0, true);
        } else if (c + 1 < n_git) {
          mbar_wait(do_full + (st ^ 1), (uint32_t)(((c + 1) >> 1) & 1), ctx, 745);
          mbar_wait(s_full, par ^ 1u, ctx, 746);
          __syncwarp();
          tc_fence_after_sync();
          exp_chunk(col0, s_stat + (st ^ 1) * 256 + col0, it1 == 0, (kvt + it1) * kTile + col0, false);
        }
        // The tensor pipe reads the shared-memory copy of dS^T a whole chunk later:
        // its proxy fence waits here, behind the exponentials, where the stores have
        // long landed.
        fence_proxy_async_smem();
        __syncwarp();
        if (r.lane == 0) mbar_arrive(ds_full + ch);
      }
      it = it1;
    }
    mbar_wait(done, 0, ctx, 747);
    __syncwarp();
    tc_fence_after_sync();
    store_rows<HD, FMT, CG>(tDV, dv_ptr, bh, kv0, S, 1.0f, r, heads_kv, dv_tm);
    store_rows<HD, FMT, CG>(tDK, dk_ptr, bh, kv0, S, scale, r);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (r.warp == 1) tmem_dealloc(tmem, 512);
}

// dq[bh, s, :] = round(scale * dq_acc[bh, s (padded rows), :]); 8 elements per thread.
template <int FMT>
__global__ void __launch_bounds__(256)
attn_bwd3_finish_kernel(const float* __restrict__ dq_acc, void* __restrict__ dq, int S, int S_pad,
                        int64_t vectors, float scale) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= vectors) return;
  const int64_t row = i >> 4;  // 16 vectors of 8 per 128-wide row
  const int part = (int)(i & 15);
  const int64_t bh = row / S, s = row % S;
  const float4* src = reinterpret_cast<const float4*>(dq_acc + ((size_t)bh * S_pad + s) * 128 + part * 8);
  const float4 a = src[0], b = src[1];
  uint4 pk;
  pk.x = pack2<FMT>(a.x * scale, a.y * scale);
  pk.y = pack2<FMT>(a.z * scale, a.w * scale);
  pk.z = pack2<FMT>(b.x * scale, b.y * scale);
  pk.w = pack2<FMT>(b.z * scale, b.w * scale);
  reinterpret_cast<uint4*>(dq)[i] = pk;
}

template <int FMT>
int launch3(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
            const CUtensorMap& mdo, const float* lse2_pad, const float* delta_pad, float* dq_acc,
            void* dq, void* dk, void* dv, int64_t B, int64_t H, int64_t Hkv, int64_t S,
            int64_t S_pad, float scale, cudaStream_t stream, Layouts lay) {
  const size_t acc_bytes = (size_t)B * H * S_pad * 128 * sizeof(float);
  if (cudaMemsetAsync(dq_acc, 0, acc_bytes, stream) != cudaSuccess) {
    cudaGetLastError();
    return fail(EVG_ELAUNCH, "causal_attention_bwd: clearing the float32 dQ copy failed");
  }
  size_t smem = 7 * tile_bytes<128>() + 2048 + kControlBytes + 1024;
  const size_t most = (size_t)device_info().max_smem_optin;
  if (smem > most) smem = most;
  auto kern = attn_bwd3_kernel<FMT>;
  if (int rc = reserve_smem(kern, smem)) return rc;
  dim3 grid((unsigned)((S_pad / kTile) * B * Hkv));
  kern<<<grid, kThreads3, smem, stream>>>(mq, mk, mv, mdo, lse2_pad, delta_pad, dq_acc, dk, dv,
                                          (int)S, (int)S_pad, (int)(H / Hkv), scale,
                                          wait_limit_cycles2(), (uint32_t)smem, (int)(B * Hkv),
                                          head_group_for((S_pad / kTile) * B * Hkv, B * Hkv), (int)Hkv,
                                          lay.dv_token_major, lay.v_token_major, lay.do_token_major);
  if (int rc = check_launch("causal_attention_bwd fused")) return rc;
  const int64_t vectors = B * H * S * 16;
  attn_bwd3_finish_kernel<FMT><<<(unsigned)((vectors + 255) / 256), 256, 0, stream>>>(
      dq_acc, dq, (int)S, (int)S_pad, vectors, scale);
  return check_launch("causal_attention_bwd finish");
}

int read_attention3_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_attn3_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attn3_device_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_attention3_status_registered =
    (register_device_status(read_attention3_status), true);

}  // namespace

namespace attn_bwd {

int launch_bwd3_128(int fmt, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                    const CUtensorMap& mdo, const float* lse2_pad, const float* delta_pad,
                    float* dq_acc, void* dq, void* dk, void* dv, int64_t B, int64_t H, int64_t Hkv,
                    int64_t S, int64_t S_pad, float scale, cudaStream_t stream, Layouts lay) {
  return fmt == 1 ? launch3<1>(mq, mk, mv, mdo, lse2_pad, delta_pad, dq_acc, dq, dk, dv, B, H, Hkv,
                               S, S_pad, scale, stream, lay)
                  : launch3<0>(mq, mk, mv, mdo, lse2_pad, delta_pad, dq_acc, dq, dk, dv, B, H, Hkv,
                               S, S_pad, scale, stream, lay);
}

}  // namespace attn_bwd
}  // namespace evg
