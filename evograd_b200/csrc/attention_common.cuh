// Building blocks shared by the attention kernels: tile geometry, TMA tile
// loads, tcgen05 issue helpers for the two product shapes, 16-bit packing and
// the shared-memory carve-up.
#pragma once

#include "evg_common.cuh"
#include "sm100_umma.cuh"

namespace evg {
namespace attn {

using namespace umma;

constexpr int kTile = 128;  // rows of every tile (queries and keys alike)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// The running maximum of a query row is only moved when it would grow by more
// than this many powers of two; until then probabilities may exceed 1 (by at
// most 2^8), which float32 sums and 16-bit P absorb, and O needs no rescaling.
constexpr float kRescaleThreshold = 8.0f;

template <int HD> __host__ __device__ constexpr uint32_t tile_bytes() { return kTile * HD * 2; }

// One 128-row tile = HD/64 TMA boxes of [128 x 64].
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* smem_tile, const CUtensorMap* map, int row0,
                                          int outer, uint64_t* bar) {
#pragma unroll
  for (int a = 0; a < HD / 64; ++a)
    tma_load_3d(smem_tile + a * (kTile * 128), map, a * 64, row0, outer, bar);
}

// v and dO, which may be token-major: then the map is 4-D with coordinates (column,
// position, head, batch) of a tensor with `heads` heads per batch; head-major tensors
// keep the 3-D map (measured 1-2 % faster than a 4-D map of the same memory).
template <int HD>
__device__ __forceinline__ void load_tile_bh(uint8_t* smem_tile, const CUtensorMap* map, int row0,
                                             int bh, int heads, int token_major, uint64_t* bar) {
  if (!token_major) {
    load_tile<HD>(smem_tile, map, row0, bh, bar);
    return;
  }
#pragma unroll
  for (int a = 0; a < HD / 64; ++a)
    tma_load_4d(smem_tile + a * (kTile * 128), map, a * 64, row0, bh % heads, bh / heads, bar);
}
// Host side: the map that load_tile_bh expects for a [B, H, S, D] / [B, S, H, D] tensor.
inline bool encode_bh_map(CUtensorMap* map, const void* base, int fmt, int64_t D, int64_t S,
                          int64_t H, int64_t B, int token_major) {
  return token_major ? encode_tile_map_16bit_4d(map, base, fmt, D, S, H, B, kTile, true)
                     : encode_tile_map_16bit(map, base, fmt, D, S, B * H, kTile);
}

// S[128xN] = A[128xHD] * B[NxHD]^T, both tiles K-major (N from the descriptor).
template <int HD>
__device__ __forceinline__ void issue_scores(bool lead, uint32_t d_tmem, uint32_t a_saddr,
                                             uint32_t b_saddr, uint32_t idesc) {
  const DescBase a = desc_base_kmajor(a_saddr), b = desc_base_kmajor(b_saddr);
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks)
    if (lead)
      mma_ss(d_tmem, desc_at(a, kstep_kmajor(kTile, ks)), desc_at(b, kstep_kmajor(kTile, ks)),
             idesc, ks > 0 ? 1u : 0u);
}
template <int HD>
__device__ __forceinline__ void issue_scores(uint32_t d_tmem, uint32_t a_saddr, uint32_t b_saddr,
                                             uint32_t idesc) {
  issue_scores<HD>(true, d_tmem, a_saddr, b_saddr, idesc);
}
// D[128xHD] (+)= A_tmem[128x128 (16-bit)] * B[128 rows x HD], B read MN-major.
__device__ __forceinline__ void issue_accumulate(bool lead, uint32_t d_tmem, uint32_t a_tmem,
                                                 uint32_t b_saddr, uint32_t idesc,
                                                 bool accumulate) {
  const DescBase b = desc_base_mnmajor(b_saddr, kTile);
#pragma unroll
  for (int ks = 0; ks < kTile / 16; ++ks)
    if (lead)
      mma_ts(d_tmem, a_tmem + ks * 8, desc_at(b, kstep_mnmajor(ks)), idesc,
             (accumulate || ks > 0) ? 1u : 0u);
}
__device__ __forceinline__ void issue_accumulate(uint32_t d_tmem, uint32_t a_tmem,
                                                 uint32_t b_saddr, uint32_t idesc,
                                                 bool accumulate) {
  issue_accumulate(true, d_tmem, a_tmem, b_saddr, idesc, accumulate);
}

template <int FMT> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (FMT == 1) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// Order in which the blocks of a causal kernel start: `n_x` work items per head
// (item 0 = the heaviest), `n_bh` heads, 1-D grid of n_x * n_bh blocks. Heads are
// taken in groups of `head_group`: within a group ALL heads' item 0 come first, then
// all item 1, ... A grid of a few waves uses one group (no heavy block starts when
// most SMs have nothing left to do: at 32 query / 8 k/v heads and 4096 tokens the
// forward went from 178 to 144 us); a large grid uses groups of four heads, so that
// the blocks that run together read the same few heads' tiles from L2 (one head per
// group leaves the last head's heaviest block for the end: 0.5-1.5 % slower).
__device__ __forceinline__ void map_block(int64_t id, int n_x, int n_bh, int head_group, int& x,
                                          int& bh) {
  const int64_t per_group = (int64_t)head_group * n_x;
  const int g = (int)(id / per_group);
  const int r = (int)(id % per_group);
  const int first = g * head_group;
  const int in_group = n_bh - first < head_group ? n_bh - first : head_group;
  x = r / in_group;
  bh = first + r % in_group;
}
// One group of all heads for grids of up to six waves, four heads per group beyond.
inline int head_group_for(int64_t n_blocks, int64_t n_bh) {
  return n_blocks <= 6 * (int64_t)device_info().sm_count ? (int)n_bh : 4;
}

struct BlockSetup {
  uint8_t* smem;        // 1024-byte aligned dynamic shared memory
  uint64_t* bars;       // mbarriers
  uint32_t* tmem_slot;  // where tcgen05.alloc writes the base address
  int* abort_flag;
};

__device__ __forceinline__ BlockSetup carve(uint8_t* raw, size_t tile_region_bytes) {
  BlockSetup b;
  b.smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  b.bars = reinterpret_cast<uint64_t*>(b.smem + tile_region_bytes);
  b.tmem_slot = reinterpret_cast<uint32_t*>(b.bars + 24);
  b.abort_flag = reinterpret_cast<int*>(b.tmem_slot + 1);
  return b;
}
constexpr size_t kControlBytes = 24 * 8 + 64;

// Optional token-major tensors of the tensor-core kernels: v, o, dO as [B, S, H, D] and
// dv as [B, S, Hkv, D], which is how the
// projections around the attention of a decoder layer want them (no transposing
// copies). Everything else is [B, H, S, D].
struct Layouts {
  int o_token_major = 0;
  int dv_token_major = 0;
  int v_token_major = 0;   // v and dO are read through 4-D TMA maps when token-major
  int do_token_major = 0;
};
// Row of a [B, H, S, D] (or, token-major, [B, S, H, D]) tensor that holds position s of
// (batch, head) pair bh.
__host__ __device__ __forceinline__ size_t tensor_row(int bh, int s, int S, int heads,
                                                       int token_major) {
  return token_major ? ((size_t)(bh / heads) * S + s) * heads + bh % heads : (size_t)bh * S + s;
}

// Two-tile warp-specialised forward (attention_fwd2.cu).
// H query heads share Hkv key/value heads (H % Hkv == 0; Hkv == H is plain
// multi-head attention): query head h reads k/v head h / (H / Hkv).
int launch_fwd2_any(int head_dim, int fmt, const void* q, const void* k, const void* v, void* o,
                    float* lse, int64_t B, int64_t H, int64_t Hkv, int64_t S, float scale,
                    cudaStream_t stream, Layouts lay = Layouts());
// Pipelined backward (attention_bwd2.cu, attention_bwd3.cu): scratch = two float32
// arrays padded to whole tiles per (batch, head), plus, at head size 128, a
// float32 copy of dQ with the same padding. fmt: 0 float16, 1 bfloat16.
int64_t bwd2_workspace_bytes(int64_t B, int64_t H, int64_t S, int64_t D);
int launch_bwd2_any(int head_dim, int fmt, const void* dout, const void* q, const void* k,
                    const void* v, const void* o, const float* lse, void* dq, void* dk, void* dv,
                    float* workspace, int64_t B, int64_t H, int64_t Hkv, int64_t S, float scale,
                    cudaStream_t stream, Layouts lay = Layouts());
// CUDA-core kernels for float32 and head sizes other than 64 / 128
// (attention_generic.cu). Scratch: one float32 per query row.
int64_t generic_bwd_workspace_bytes(int64_t B, int64_t Hq, int64_t S);
int launch_generic_fwd(int dtype, const void* q, const void* k, const void* v, void* o,
                       float* lse, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                       float scale, cudaStream_t stream);
int launch_generic_bwd(int dtype, const void* dout, const void* q, const void* k, const void* v,
                       const void* o, const float* lse, void* dq, void* dk, void* dv,
                       void* workspace, int64_t workspace_bytes, int64_t B, int64_t Hq,
                       int64_t Hkv, int64_t S, int64_t D, float scale, cudaStream_t stream);


// EvoformerAttention on the tensor cores (attention_evo_tc.cu): head sizes 32 and
// 64, 16-bit inputs, residue counts that are a multiple of 4.
bool evo_tc_shape(int64_t B, int64_t S, int64_t N, int64_t H, int64_t D, int dtype);
int launch_evo_tc_fwd(int head_dim, int fmt, const void* q, const void* k, const void* v,
                      const float* res_mask, const float* pair_bias, void* o, float* lse,
                      int64_t B, int64_t S, int64_t N, int64_t H, float scale,
                      cudaStream_t stream);
// delta = rowsum(do * o) as float32 [B, S, H, N] comes from the caller; dbias_out
// receives `split` partial d_pair_bias arrays [split][B][H][N][N] (MSA rows cut
// into `split` parts), which the caller adds up when split > 1.
int launch_evo_tc_bwd(int head_dim, int fmt, const void* dout, const void* q, const void* k,
                      const void* v, const float* res_mask, const float* pair_bias,
                      const float* lse, const float* delta, void* dq, void* dk, void* dv,
                      float* dbias_out, int split, int64_t B, int64_t S, int64_t N, int64_t H,
                      float scale, cudaStream_t stream);

}  // namespace attn
}  // namespace evg
