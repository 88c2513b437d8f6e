// EvoformerAttention (AlphaFold-3 style) forward/backward on the CUDA cores:
//
//   o = softmax(scale * q k^T + pair_bias + res_mask) v      over the residue axis
//   (ops/level1/evoattention/forward_ref.py:22-49)
//
//   q, k, v, o, do : [B, S, N, H, D]   (S = MSA rows, N = residues, H heads)
//   res_mask       : [B, S, N] float32, additive per key (the reference's
//                    [B, S, 1, 1, N])
//   pair_bias      : [B, H, N, N] float32, shared by all S rows, trainable
//   d_pair_bias    : sum over S of dS, float32
//
// The residue counts are small (128-384, head sizes 8-128), so these are
// one-warp-per-row kernels on the CUDA cores: a block first stages the K and V
// (or Q and dO) rows of its (batch, MSA row, head) in shared memory, padded so
// that 32 lanes reading 32 different rows hit 32 different banks, and every warp
// then walks several rows against them. (If the rows do not fit shared memory
// the same code reads them from global memory.) Every sum has a fixed order:
// d_pair_bias is accumulated over the MSA rows inside the warp that owns a
// (batch, head, query) row, without atomics. Saved state: o and the float32
// log-sum-exp [B, S, H, N].
#include <algorithm>
#include <initializer_list>
#include <type_traits>

#include "attention_common.cuh"
#include "evg_common.cuh"

// 16-bit element types only (the reference declares float16 | bfloat16).
#define EVG_DISPATCH_DTYPE_16(dtype, ...)                               \
  [&]() -> int {                                                        \
    if ((dtype) == EVG_F16) { using T = __half; return __VA_ARGS__(); } \
    using T = __nv_bfloat16;                                            \
    return __VA_ARGS__();                                               \
  }()

namespace evg {
namespace {

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 4;  // forward and dK/dV: rows a warp walks per block
constexpr int kMaxDT = 8;     // head_dim <= 256
constexpr int kMaxChunks = 32;  // residues <= 1024 (d_pair_bias row kept in registers)

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// dot(a, b_row): a is float32 in shared memory (broadcast reads, 16-byte aligned),
// b_row a row of T in shared or global memory. 16-bit rows are read as 32-bit
// words when D is a multiple of 4 (rows then start on 4-byte boundaries in
// every layout used).
template <typename T>
__device__ __forceinline__ void unpack_word(uint32_t u, float& lo, float& hi) {
  T a, b;
  const uint32_t uh = u >> 16;
  memcpy(&a, &u, 2);
  memcpy(&b, &uh, 2);
  lo = to_f32<T>(a);
  hi = to_f32<T>(b);
}
template <typename T>
__device__ __forceinline__ float dot_row(const float* a_smem, const T* b_row, int D) {
  float s = 0.f;
  if constexpr (sizeof(T) == 2) {
    if ((D & 3) == 0) {  // four elements per step: one float4 of a, two words of b
      const uint32_t* w = reinterpret_cast<const uint32_t*>(b_row);
      const float4* a4 = reinterpret_cast<const float4*>(a_smem);
      float s1 = 0.f;
      for (int d = 0; d < D / 4; ++d) {
        const float4 a = a4[d];
        float b0, b1, b2, b3;
        unpack_word<T>(w[2 * d], b0, b1);
        unpack_word<T>(w[2 * d + 1], b2, b3);
        s = fmaf(a.x, b0, s);
        s1 = fmaf(a.y, b1, s1);
        s = fmaf(a.z, b2, s);
        s1 = fmaf(a.w, b3, s1);
      }
      return s + s1;
    }
  }
  for (int d = 0; d < D; ++d) s = fmaf(a_smem[d], to_f32<T>(b_row[d]), s);
  return s;
}

// Row pitch (elements) of a staged [N, D] matrix: D + 2 puts consecutive rows
// an odd number of 32-bit words apart whenever D is a multiple of 4.
__host__ __device__ __forceinline__ int staged_pitch(int D) { return D + 2; }

// All threads of the block copy N rows of D elements (row stride src_rs) into
// shared memory with pitch staged_pitch(D): 16-byte global loads and 4-byte
// shared stores when a row is a whole number of 16-byte vectors (the padded
// pitch keeps rows 4-byte aligned only), element by element otherwise.
template <typename T>
__device__ __forceinline__ void stage_rows(T* dst, const T* src, int N, int D, size_t src_rs) {
  const int P = staged_pitch(D);
  constexpr int EPV = 16 / (int)sizeof(T);  // elements per 16-byte vector
  if (D % EPV == 0 && src_rs % EPV == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const int vpr = D / EPV;  // vectors per row
    int n = threadIdx.x / vpr, c = threadIdx.x - n * vpr;
    const int dn = blockDim.x / vpr, dc = blockDim.x - dn * vpr;
    while (n < N) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + (size_t)n * src_rs + c * EPV);
      uint32_t* w = reinterpret_cast<uint32_t*>(dst + (size_t)n * P + c * EPV);
      w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w;
      n += dn;
      c += dc;
      if (c >= vpr) { c -= vpr; ++n; }
    }
    return;
  }
  for (int e = threadIdx.x; e < N * D; e += blockDim.x) {
    const int n = e / D, d = e - n * D;
    dst[n * P + d] = src[(size_t)n * src_rs + d];
  }
}

struct EvoShape {
  int B, S, N, H, D;
  float scale;
};
// element offset of row n of (b, s, h) in a [B, S, N, H, D] tensor
__device__ __forceinline__ size_t row_off(const EvoShape& sh, int b, int s, int n, int h) {
  return ((((size_t)b * sh.S + s) * sh.N + n) * sh.H + h) * sh.D;
}

// DT = ceil(head_dim / 32) accumulators per lane (1, 2, 4 or 8).
// `staged` != 0: the K and V rows of this (batch, MSA row, head) are first copied
// into shared memory (after the per-warp float32 row buffers).
template <typename T, int DT>
__global__ void __launch_bounds__(kWarps * 32)
evo_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
               const float* __restrict__ mask, const float* __restrict__ bias,
               T* __restrict__ o, float* __restrict__ lse, EvoShape sh, int staged) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, bs = blockIdx.z, b = bs / sh.S, s = bs % sh.S;
  const int N = sh.N, D = sh.D;
  float* qs = smem + warp * D;
  size_t rs = (size_t)sh.H * D;  // stride between residues
  const T* kb = k + row_off(sh, b, s, 0, h);
  const T* vb = v + row_off(sh, b, s, 0, h);
  if (staged) {
    T* sk = reinterpret_cast<T*>(smem + kWarps * D);
    T* sv = sk + (size_t)N * staged_pitch(D);
    stage_rows<T>(sk, kb, N, D, rs);
    stage_rows<T>(sv, vb, N, D, rs);
    __syncthreads();
    kb = sk;
    vb = sv;
    rs = staged_pitch(D);
  }
  const float* mrow = mask + (size_t)bs * N;
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int i = (blockIdx.x * kWarps + warp) * kRowsPerWarp + r;
    if (i >= N) break;
    const T* qr = q + row_off(sh, b, s, i, h);
    const float* brow = bias + (((size_t)b * sh.H + h) * N + i) * N;
    __syncwarp();
    for (int d = lane; d < D; d += 32) qs[d] = to_f32<T>(qr[d]);
    __syncwarp();
    float m = -INFINITY, l = 0.f;
    float acc[DT];
#pragma unroll
    for (int t = 0; t < DT; ++t) acc[t] = 0.f;
    for (int j0 = 0; j0 < N; j0 += 32) {
      const int j = j0 + lane;
      const float sc = j < N ? sh.scale * dot_row<T>(qs, kb + j * rs, D) + brow[j] + mrow[j]
                             : -INFINITY;
      const float m_new = fmaxf(m, warp_max(sc));
      const float corr = expf(m - m_new);
      const float p = expf(sc - m_new);
      l = l * corr + warp_sum(p);
      const float pr = round_to<T>(p);  // probabilities enter P V in the input dtype
#pragma unroll
      for (int t = 0; t < DT; ++t) acc[t] *= corr;
      const int n = min(32, N - j0);
      for (int jj = 0; jj < n; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pr, jj);
        const T* vr = vb + (size_t)(j0 + jj) * rs;
#pragma unroll
        for (int t = 0; t < DT; ++t) {
          const int d = lane + 32 * t;
          if (d < D) acc[t] = fmaf(pj, to_f32<T>(vr[d]), acc[t]);
        }
      }
      m = m_new;
    }
    T* orow = o + row_off(sh, b, s, i, h);
    const float inv = 1.0f / l;
#pragma unroll
    for (int t = 0; t < DT; ++t) {
      const int d = lane + 32 * t;
      if (d < D) orow[d] = from_f32<T>(acc[t] * inv);
    }
    if (lane == 0) lse[((size_t)bs * sh.H + h) * N + i] = m + logf(l);
  }
}

// delta[b,s,h,i] = sum_d do * o
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
evo_delta_kernel(const T* __restrict__ dout, const T* __restrict__ o, float* __restrict__ delta,
                 EvoShape sh) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * kWarps + warp;
  const int h = blockIdx.y, bs = blockIdx.z, b = bs / sh.S, s = bs % sh.S;
  if (i >= sh.N) return;
  const size_t off = row_off(sh, b, s, i, h);
  float a = 0.f;
  for (int d = lane; d < sh.D; d += 32) a = fmaf(to_f32<T>(dout[off + d]), to_f32<T>(o[off + d]), a);
  a = warp_sum(a);
  if (lane == 0) delta[((size_t)bs * sh.H + h) * sh.N + i] = a;
}

// The same with D / 8 threads per row and 16-byte loads (D a power of two, 8..256,
// 16-bit elements, rows 16-byte aligned): row r of the [B*S*N*H, D] view.
template <typename T>
__global__ void __launch_bounds__(256)
evo_delta_vec_kernel(const T* __restrict__ dout, const T* __restrict__ o, float* __restrict__ delta,
                     int64_t rows, int N, int H, int D) {
  const int tpr = D / 8;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid / tpr;
  const int part = (int)(gid - row * tpr);
  float a = 0.f;
  if (row < rows) {
    const uint4 x = ld_vec(dout + row * D + part * 8);
    const uint4 y = ld_vec(o + row * D + part * 8);
    float xf[8], yf[8];
    unpack<T>(x, xf);
    unpack<T>(y, yf);
#pragma unroll
    for (int i = 0; i < 8; ++i) a = fmaf(xf[i], yf[i], a);
  }
  for (int off = tpr >> 1; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
  if (row < rows && part == 0) {
    const int64_t h = row % H, n = (row / H) % N, bs = row / ((int64_t)H * N);
    delta[(bs * H + h) * N + n] = a;
  }
}

// One warp per (batch, head, query row): walks the MSA rows, writes dq for each
// and keeps the row of d_pair_bias (lane = key index mod 32) in registers. With
// `staged`, the block re-stages K and V for every MSA row.
template <typename T, int DT, int MAXC>
__global__ void __launch_bounds__(kWarps * 32)
evo_dq_dbias_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k,
                    const T* __restrict__ v, const float* __restrict__ mask,
                    const float* __restrict__ bias, const float* __restrict__ lse,
                    const float* __restrict__ delta, T* __restrict__ dq,
                    float* __restrict__ dbias, EvoShape sh, int staged, int split) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * kWarps + warp;
  // blockIdx.z = b * split + part: the MSA rows are cut into `split` contiguous
  // parts so that enough blocks exist; part p writes its own d_pair_bias slab
  // (dbias + p * B*H*N*N), added up afterwards in part order.
  const int h = blockIdx.y, b = blockIdx.z / split, part = blockIdx.z % split;
  const int N = sh.N, D = sh.D;
  const int s_lo = (int)((long long)sh.S * part / split);
  const int s_hi = (int)((long long)sh.S * (part + 1) / split);
  float* qs = smem + warp * 2 * D;
  float* gs = qs + D;
  T* sk = reinterpret_cast<T*>(smem + kWarps * 2 * D);
  T* sv = sk + (size_t)N * staged_pitch(D);
  const bool active = i < N;  // idle warps still take part in the block barriers
  const float* brow = bias + (((size_t)b * sh.H + h) * N + (active ? i : 0)) * N;
  float db[MAXC];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) db[c] = 0.f;
  for (int s = s_lo; s < s_hi; ++s) {
    const int bs = b * sh.S + s;
    size_t rs = (size_t)sh.H * D;
    const T* kb = k + row_off(sh, b, s, 0, h);
    const T* vb = v + row_off(sh, b, s, 0, h);
    if (staged) {
      __syncthreads();  // every warp is done with the previous MSA row's K and V
      stage_rows<T>(sk, kb, N, D, rs);
      stage_rows<T>(sv, vb, N, D, rs);
      __syncthreads();
      kb = sk;
      vb = sv;
      rs = staged_pitch(D);
    }
    if (!active) continue;
    const size_t off = row_off(sh, b, s, i, h);
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      qs[d] = to_f32<T>(q[off + d]);
      gs[d] = to_f32<T>(dout[off + d]);
    }
    __syncwarp();
    const float* mrow = mask + (size_t)bs * N;
    const size_t stat = ((size_t)bs * sh.H + h) * N + i;
    const float lse_i = lse[stat], delta_i = delta[stat];
    float acc[DT];
#pragma unroll
    for (int t = 0; t < DT; ++t) acc[t] = 0.f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int j0 = c * 32;
      if (j0 < N) {
        const int j = j0 + lane;
        float ds = 0.f;
        if (j < N) {
          const float p = expf(sh.scale * dot_row<T>(qs, kb + j * rs, D) + brow[j] + mrow[j] - lse_i);
          ds = p * (dot_row<T>(gs, vb + j * rs, D) - delta_i);
        }
        db[c] += ds;
        const int n = min(32, N - j0);
        for (int jj = 0; jj < n; ++jj) {
          const float dj = __shfl_sync(0xffffffffu, ds, jj);
          const T* kr = kb + (size_t)(j0 + jj) * rs;
#pragma unroll
          for (int t = 0; t < DT; ++t) {
            const int d = lane + 32 * t;
            if (d < D) acc[t] = fmaf(dj, to_f32<T>(kr[d]), acc[t]);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < DT; ++t) {
      const int d = lane + 32 * t;
      if (d < D) dq[off + d] = from_f32<T>(sh.scale * acc[t]);
    }
  }
  if (!active) return;
  float* drow = dbias + ((((size_t)part * sh.B + b) * sh.H + h) * N + i) * N;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int j = c * 32 + lane;
    if (j < N) drow[j] = db[c];
  }
}

// One warp per key row of (batch, MSA row, head); with `staged` the block first
// copies the Q and dO rows into shared memory.
template <typename T, int DT>
__global__ void __launch_bounds__(kWarps * 32)
evo_dkdv_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k,
                const T* __restrict__ v, const float* __restrict__ mask,
                const float* __restrict__ bias, const float* __restrict__ lse,
                const float* __restrict__ delta, T* __restrict__ dk, T* __restrict__ dv,
                EvoShape sh, int staged) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, bs = blockIdx.z, b = bs / sh.S, s = bs % sh.S;
  const int N = sh.N, D = sh.D;
  float* ks = smem + warp * 2 * D;
  float* vs = ks + D;
  size_t rs = (size_t)sh.H * D;
  const T* qb = q + row_off(sh, b, s, 0, h);
  const T* gb = dout + row_off(sh, b, s, 0, h);
  if (staged) {
    T* sq = reinterpret_cast<T*>(smem + kWarps * 2 * D);
    T* sg = sq + (size_t)N * staged_pitch(D);
    stage_rows<T>(sq, qb, N, D, rs);
    stage_rows<T>(sg, gb, N, D, rs);
    __syncthreads();
    qb = sq;
    gb = sg;
    rs = staged_pitch(D);
  }
  const float* lrow = lse + ((size_t)bs * sh.H + h) * N;
  const float* drow = delta + ((size_t)bs * sh.H + h) * N;
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int j = (blockIdx.x * kWarps + warp) * kRowsPerWarp + r;
    if (j >= N) break;
    const size_t koff = row_off(sh, b, s, j, h);
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      ks[d] = to_f32<T>(k[koff + d]);
      vs[d] = to_f32<T>(v[koff + d]);
    }
    __syncwarp();
    const float* bcol = bias + ((size_t)b * sh.H + h) * N * N + j;  // + i * N
    const float mj = mask[(size_t)bs * N + j];
    float acc_k[DT], acc_v[DT];
#pragma unroll
    for (int t = 0; t < DT; ++t) acc_k[t] = acc_v[t] = 0.f;
    for (int i0 = 0; i0 < N; i0 += 32) {
      const int i = i0 + lane;
      float p = 0.f, ds = 0.f;
      if (i < N) {
        p = expf(sh.scale * dot_row<T>(ks, qb + i * rs, D) + bcol[(size_t)i * N] + mj - lrow[i]);
        ds = p * (dot_row<T>(vs, gb + i * rs, D) - drow[i]);
        p = round_to<T>(p);  // P^T dO takes P in the input dtype, as P V does
      }
      const int n = min(32, N - i0);
      for (int ii = 0; ii < n; ++ii) {
        const float pi = __shfl_sync(0xffffffffu, p, ii);
        const float di = __shfl_sync(0xffffffffu, ds, ii);
        const T* qr = qb + (size_t)(i0 + ii) * rs;
        const T* gr = gb + (size_t)(i0 + ii) * rs;
#pragma unroll
        for (int t = 0; t < DT; ++t) {
          const int d = lane + 32 * t;
          if (d < D) {
            acc_v[t] = fmaf(pi, to_f32<T>(gr[d]), acc_v[t]);
            acc_k[t] = fmaf(di, to_f32<T>(qr[d]), acc_k[t]);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < DT; ++t) {
      const int d = lane + 32 * t;
      if (d < D) {
        dk[koff + d] = from_f32<T>(sh.scale * acc_k[t]);
        dv[koff + d] = from_f32<T>(acc_v[t]);
      }
    }
  }
}

// d_pair_bias = sum over the `split` slabs, in slab order.
__global__ void evo_dbias_reduce_kernel(const float* __restrict__ slabs, float* __restrict__ out,
                                        int64_t n, int split) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n;
       e += (int64_t)gridDim.x * blockDim.x) {
    float a = slabs[e];
    for (int p = 1; p < split; ++p) a += slabs[(size_t)p * n + e];
    out[e] = a;
  }
}

// Parts the MSA axis is cut into for the dq / d_pair_bias kernel: enough for
// about four blocks per SM, at most 16 and at most S.
int evo_split(int64_t B, int64_t S, int64_t N, int64_t H) {
  const int64_t blocks = ((N + kWarps - 1) / kWarps) * H * B;
  int64_t split = (4 * (int64_t)device_info().sm_count + blocks - 1) / blocks;
  if (split > 16) split = 16;
  if (split > S) split = S;
  return split < 1 ? 1 : (int)split;
}

// The same for the tensor-core d_pair_bias kernel, whose blocks own a
// [128 x 64] tile of the gradient: about four blocks per SM, at most 32 parts.
int evo_tc_split(int64_t B, int64_t S, int64_t N, int64_t H) {
  const int64_t blocks = ((N + 127) / 128) * ((N + 63) / 64) * H * B;
  int64_t split = (4 * (int64_t)device_info().sm_count + blocks - 1) / blocks;
  if (split > 32) split = 32;
  if (split > S) split = S;
  while (split > 1 && B * H * split > 65535) --split;
  return split < 1 ? 1 : (int)split;
}

bool evo_use_tc(int64_t B, int64_t S, int64_t N, int64_t H, int64_t D, int dtype,
                std::initializer_list<const void*> ptrs) {
  if (!attn::evo_tc_shape(B, S, N, H, D, dtype)) return false;
  for (const void* p : ptrs)
    if (!aligned16(p)) return false;
  return true;
}

// Dynamic shared memory of a kernel with `bufs` float32 row buffers per warp
// and (when it fits) two staged [N, D] matrices of T; *staged says which.
template <typename T, typename Kernel>
size_t evo_smem(Kernel kernel, int bufs, int64_t N, int64_t D, int* staged) {
  const size_t base = (size_t)kWarps * bufs * D * sizeof(float);
  const size_t want = base + 2 * (size_t)N * staged_pitch((int)D) * sizeof(T);
  *staged = 0;
  if (!tune("evoattention.no_stage") && want <= (size_t)device_info().max_smem_optin &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)want) ==
          cudaSuccess) {
    *staged = 1;
    return want;
  }
  cudaGetLastError();
  return base;
}

int check_evo(const char* what, int64_t B, int64_t S, int64_t N, int64_t H, int64_t D, int dtype) {
  if (B <= 0 || S <= 0 || N <= 0 || H <= 0 || D <= 0)
    return fail(EVG_EBADSHAPE, "%s: B=%lld S=%lld N=%lld H=%lld D=%lld must be positive", what,
                (long long)B, (long long)S, (long long)N, (long long)H, (long long)D);
  if (dtype != EVG_BF16 && dtype != EVG_F16)  // the declaration's dtypes (float16|bfloat16)
    return fail(EVG_EDTYPE, "%s: dtype %d (supported: float16, bfloat16)", what, dtype);
  if (D > 32 * kMaxDT || N > 32 * kMaxChunks)
    return fail(EVG_EUNSUPPORTED, "%s: head_dim %lld (max 256) or residues %lld (max 1024)", what,
                (long long)D, (long long)N);
  if (H > 65535 || B * S > 65535)
    return fail(EVG_EUNSUPPORTED, "%s: H=%lld or B*S=%lld above 65535", what, (long long)H,
                (long long)(B * S));
  return EVG_OK;
}

inline int evo_dt(int D) { return D <= 32 ? 1 : D <= 64 ? 2 : D <= 128 ? 4 : 8; }

template <typename T>
int launch_evo_fwd(const void* q, const void* k, const void* v, const float* res_mask,
                   const float* pair_bias, void* o, float* lse, const EvoShape& sh,
                   cudaStream_t stream) {
  const int N = sh.N, D = sh.D, dt = evo_dt(D);
  const int rows_per_block = kWarps * kRowsPerWarp;
  dim3 grid((unsigned)((N + rows_per_block - 1) / rows_per_block), (unsigned)sh.H,
            (unsigned)(sh.B * sh.S));
#define EVG_EVO_FWD(DT_)                                                                     \
  if (dt == DT_) {                                                                           \
    int staged = 0;                                                                          \
    auto kern = evo_fwd_kernel<T, DT_>;                                                      \
    const size_t smem = evo_smem<T>(kern, 1, N, D, &staged);                                 \
    kern<<<grid, kWarps * 32, smem, stream>>>((const T*)q, (const T*)k, (const T*)v,         \
                                              res_mask, pair_bias, (T*)o, lse, sh, staged);  \
  }
  EVG_EVO_FWD(1) EVG_EVO_FWD(2) EVG_EVO_FWD(4) EVG_EVO_FWD(8)
#undef EVG_EVO_FWD
  return check_launch("evoattention_fwd");
}

template <typename T>
int launch_evo_bwd(const void* dout, const void* q, const void* k, const void* v,
                   const float* res_mask, const float* pair_bias, const void* o,
                   const float* lse, void* dq, void* dk, void* dv, float* d_pair_bias,
                   float* workspace, const EvoShape& sh, bool use_tc, cudaStream_t st) {
  const int64_t B = sh.B, S = sh.S, N = sh.N, H = sh.H, D = sh.D;
  float* delta = workspace;
  const int split = use_tc ? evo_tc_split(B, S, N, H) : evo_split(B, S, N, H);
  float* slabs = split > 1 ? delta + B * S * H * N : d_pair_bias;
  const int dt = evo_dt((int)D);
  const bool few_chunks = N <= 384;
  const unsigned tiles = (unsigned)((N + kWarps - 1) / kWarps);
  const int rows_per_block = kWarps * kRowsPerWarp;
  const unsigned wide_tiles = (unsigned)((N + rows_per_block - 1) / rows_per_block);
  if (use_tc) {  // head sizes 32 / 64, aligned tensors
    const int64_t rows = B * S * N * H, threads = rows * (D / 8);
    evo_delta_vec_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(
        (const T*)dout, (const T*)o, delta, rows, (int)N, (int)H, (int)D);
  } else {
    evo_delta_kernel<T><<<dim3(tiles, (unsigned)H, (unsigned)(B * S)), kWarps * 32, 0, st>>>(
        (const T*)dout, (const T*)o, delta, sh);
  }
  if (use_tc) {
    if (int rc = check_launch("evoattention_bwd delta")) return rc;
    if (int rc = attn::launch_evo_tc_bwd((int)D, sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0,
                                         dout, q, k, v, res_mask, pair_bias, lse, delta, dq, dk,
                                         dv, slabs, split, B, S, N, H, sh.scale, st))
      return rc;
    if (split > 1) {
      const int64_t n = B * H * N * N;
      evo_dbias_reduce_kernel<<<(unsigned)std::min<int64_t>((n + 255) / 256, 4096), 256, 0, st>>>(
          slabs, d_pair_bias, n, split);
    }
    return check_launch("evoattention_bwd");
  }
#define EVG_EVO_DQ(DT_, MAXC_)                                                                   \
  if (dt == DT_ && few_chunks == (MAXC_ == 12)) {                                                \
    int staged = 0;                                                                              \
    auto kern = evo_dq_dbias_kernel<T, DT_, MAXC_>;                                              \
    const size_t smem = evo_smem<T>(kern, 2, N, D, &staged);                                     \
    kern<<<dim3(tiles, (unsigned)H, (unsigned)(B * split)), kWarps * 32, smem, st>>>(            \
        (const T*)dout, (const T*)q, (const T*)k, (const T*)v, res_mask, pair_bias, lse, delta,  \
        (T*)dq, slabs, sh, staged, split);                                                       \
  }
  EVG_EVO_DQ(1, 12) EVG_EVO_DQ(2, 12) EVG_EVO_DQ(4, 12) EVG_EVO_DQ(8, 12)
  EVG_EVO_DQ(1, 32) EVG_EVO_DQ(2, 32) EVG_EVO_DQ(4, 32) EVG_EVO_DQ(8, 32)
#undef EVG_EVO_DQ
  if (split > 1) {
    const int64_t n = B * H * N * N;
    evo_dbias_reduce_kernel<<<(unsigned)std::min<int64_t>((n + 255) / 256, 4096), 256, 0, st>>>(
        slabs, d_pair_bias, n, split);
  }
#define EVG_EVO_DKDV(DT_)                                                                        \
  if (dt == DT_) {                                                                               \
    int staged = 0;                                                                              \
    auto kern = evo_dkdv_kernel<T, DT_>;                                                         \
    const size_t smem = evo_smem<T>(kern, 2, N, D, &staged);                                     \
    kern<<<dim3(wide_tiles, (unsigned)H, (unsigned)(B * S)), kWarps * 32, smem, st>>>(           \
        (const T*)dout, (const T*)q, (const T*)k, (const T*)v, res_mask, pair_bias, lse, delta,  \
        (T*)dk, (T*)dv, sh, staged);                                                             \
  }
  EVG_EVO_DKDV(1) EVG_EVO_DKDV(2) EVG_EVO_DKDV(4) EVG_EVO_DKDV(8)
#undef EVG_EVO_DKDV
  return check_launch("evoattention_bwd");
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_evoattention_fwd(const void* q, const void* k, const void* v,
                                    const float* res_mask, const float* pair_bias, void* o,
                                    float* lse, int64_t B, int64_t S, int64_t N, int64_t H,
                                    int64_t D, float scale, int dtype, void* stream) {
  if (!q || !k || !v || !res_mask || !pair_bias || !o || !lse)
    return fail(EVG_ENULL, "evoattention_fwd: null pointer argument");
  if (int rc = check_evo("evoattention_fwd", B, S, N, H, D, dtype)) return rc;
  const EvoShape sh{(int)B, (int)S, (int)N, (int)H, (int)D, scale};
  if (evo_use_tc(B, S, N, H, D, dtype, {q, k, v, res_mask, pair_bias, o, lse}))
    return attn::launch_evo_tc_fwd((int)D, dtype == EVG_BF16 ? 1 : 0, q, k, v, res_mask, pair_bias,
                                   o, lse, B, S, N, H, scale, (cudaStream_t)stream);
  return EVG_DISPATCH_DTYPE_16(dtype, [&] {
    return launch_evo_fwd<T>(q, k, v, res_mask, pair_bias, o, lse, sh, (cudaStream_t)stream);
  });
}

extern "C" int64_t evg_evoattention_bwd_workspace_bytes(int64_t B, int64_t S, int64_t N,
                                                        int64_t H, int64_t D, int dtype) {
  (void)D; (void)dtype;
  if (B <= 0 || S <= 0 || N <= 0 || H <= 0) return 0;
  // delta [B,S,H,N] + (split > 1: one d_pair_bias slab per part); enough for
  // whichever of the two kernel families the call ends up on
  const int split = std::max(evo_split(B, S, N, H), evo_tc_split(B, S, N, H));
  return (B * S * H * N + (split > 1 ? (int64_t)split * B * H * N * N : 0)) *
         (int64_t)sizeof(float);
}

extern "C" int evg_evoattention_bwd(const void* dout, const void* q, const void* k, const void* v,
                                    const float* res_mask, const float* pair_bias, const void* o,
                                    const float* lse, void* dq, void* dk, void* dv,
                                    float* d_pair_bias, void* workspace, int64_t workspace_bytes,
                                    int64_t B, int64_t S, int64_t N, int64_t H, int64_t D,
                                    float scale, int dtype, void* stream) {
  if (!dout || !q || !k || !v || !res_mask || !pair_bias || !o || !lse || !dq || !dk || !dv ||
      !d_pair_bias)
    return fail(EVG_ENULL, "evoattention_bwd: null pointer argument");
  if (int rc = check_evo("evoattention_bwd", B, S, N, H, D, dtype)) return rc;
  const int64_t need = evg_evoattention_bwd_workspace_bytes(B, S, N, H, D, dtype);
  if (!workspace || workspace_bytes < need)
    return fail(EVG_EWORKSPACE, "evoattention_bwd: workspace %lld bytes, need %lld",
                (long long)workspace_bytes, (long long)need);
  const EvoShape sh{(int)B, (int)S, (int)N, (int)H, (int)D, scale};
  const bool use_tc = evo_use_tc(B, S, N, H, D, dtype,
                                 {dout, q, k, v, res_mask, pair_bias, o, lse, (const void*)dq,
                                  (const void*)dk, (const void*)dv, (const void*)d_pair_bias,
                                  (const void*)workspace});
  return EVG_DISPATCH_DTYPE_16(dtype, [&] {
    return launch_evo_bwd<T>(dout, q, k, v, res_mask, pair_bias, o, lse, dq, dk, dv, d_pair_bias,
                             (float*)workspace, sh, use_tc, (cudaStream_t)stream);
  });
}
