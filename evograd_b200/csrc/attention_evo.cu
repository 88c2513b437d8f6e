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
// The residue counts are small (128-384, head sizes 8-128), so these are the
// plain one-warp-per-row kernels of attention_generic.cu with the bias and mask
// added to the scores; nothing here is tuned for speed. Every sum has a fixed
// order: d_pair_bias is accumulated over the MSA rows inside the warp that owns
// a (batch, head, query) row, without atomics. Saved state: o and the float32
// log-sum-exp [B, S, H, N].
#include "evg_common.cuh"

namespace evg {
namespace {

constexpr int kWarps = 4;
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
template <typename T>
__device__ __forceinline__ float dot_row(const float* a_smem, const T* b_row, int D) {
  float s = 0.f;
  for (int d = 0; d < D; ++d) s = fmaf(a_smem[d], to_f32<T>(b_row[d]), s);
  return s;
}

struct EvoShape {
  int B, S, N, H, D;
  float scale;
};
// element offset of row n of (b, s, h) in a [B, S, N, H, D] tensor
__device__ __forceinline__ size_t row_off(const EvoShape& sh, int b, int s, int n, int h) {
  return ((((size_t)b * sh.S + s) * sh.N + n) * sh.H + h) * sh.D;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
evo_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
               const float* __restrict__ mask, const float* __restrict__ bias,
               T* __restrict__ o, float* __restrict__ lse, EvoShape sh) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * kWarps + warp;
  const int h = blockIdx.y, bs = blockIdx.z, b = bs / sh.S, s = bs % sh.S;
  const int N = sh.N, D = sh.D;
  float* qs = smem + warp * D;
  if (i >= N) return;
  const size_t rs = (size_t)sh.H * D;  // stride between residues
  const T* qr = q + row_off(sh, b, s, i, h);
  const T* kb = k + row_off(sh, b, s, 0, h);
  const T* vb = v + row_off(sh, b, s, 0, h);
  const float* brow = bias + (((size_t)b * sh.H + h) * N + i) * N;
  const float* mrow = mask + (size_t)bs * N;
  for (int d = lane; d < D; d += 32) qs[d] = to_f32<T>(qr[d]);
  __syncwarp();
  float m = -INFINITY, l = 0.f;
  float acc[kMaxDT];
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) acc[t] = 0.f;
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
    for (int t = 0; t < kMaxDT; ++t) acc[t] *= corr;
    const int n = min(32, N - j0);
    for (int jj = 0; jj < n; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pr, jj);
      const T* vr = vb + (size_t)(j0 + jj) * rs;
#pragma unroll
      for (int t = 0; t < kMaxDT; ++t) {
        const int d = lane + 32 * t;
        if (d < D) acc[t] = fmaf(pj, to_f32<T>(vr[d]), acc[t]);
      }
    }
    m = m_new;
  }
  T* orow = o + row_off(sh, b, s, i, h);
  const float inv = 1.0f / l;
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) {
    const int d = lane + 32 * t;
    if (d < D) orow[d] = from_f32<T>(acc[t] * inv);
  }
  if (lane == 0) lse[((size_t)bs * sh.H + h) * N + i] = m + logf(l);
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

// One warp per (batch, head, query row): walks the MSA rows, writes dq for each
// and keeps the row of d_pair_bias (lane = key index mod 32) in registers.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
evo_dq_dbias_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k,
                    const T* __restrict__ v, const float* __restrict__ mask,
                    const float* __restrict__ bias, const float* __restrict__ lse,
                    const float* __restrict__ delta, T* __restrict__ dq,
                    float* __restrict__ dbias, EvoShape sh) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * kWarps + warp;
  const int h = blockIdx.y, b = blockIdx.z;
  const int N = sh.N, D = sh.D;
  float* qs = smem + warp * 2 * D;
  float* gs = qs + D;
  if (i >= N) return;
  const size_t rs = (size_t)sh.H * D;
  const float* brow = bias + (((size_t)b * sh.H + h) * N + i) * N;
  float db[kMaxChunks];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) db[c] = 0.f;
  for (int s = 0; s < sh.S; ++s) {
    const int bs = b * sh.S + s;
    const size_t off = row_off(sh, b, s, i, h);
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      qs[d] = to_f32<T>(q[off + d]);
      gs[d] = to_f32<T>(dout[off + d]);
    }
    __syncwarp();
    const T* kb = k + row_off(sh, b, s, 0, h);
    const T* vb = v + row_off(sh, b, s, 0, h);
    const float* mrow = mask + (size_t)bs * N;
    const size_t stat = ((size_t)bs * sh.H + h) * N + i;
    const float lse_i = lse[stat], delta_i = delta[stat];
    float acc[kMaxDT];
#pragma unroll
    for (int t = 0; t < kMaxDT; ++t) acc[t] = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
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
          for (int t = 0; t < kMaxDT; ++t) {
            const int d = lane + 32 * t;
            if (d < D) acc[t] = fmaf(dj, to_f32<T>(kr[d]), acc[t]);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < kMaxDT; ++t) {
      const int d = lane + 32 * t;
      if (d < D) dq[off + d] = from_f32<T>(sh.scale * acc[t]);
    }
  }
  float* drow = dbias + (((size_t)b * sh.H + h) * N + i) * N;
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int j = c * 32 + lane;
    if (j < N) drow[j] = db[c];
  }
}

// One warp per key row of (batch, MSA row, head).
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
evo_dkdv_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k,
                const T* __restrict__ v, const float* __restrict__ mask,
                const float* __restrict__ bias, const float* __restrict__ lse,
                const float* __restrict__ delta, T* __restrict__ dk, T* __restrict__ dv,
                EvoShape sh) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * kWarps + warp;
  const int h = blockIdx.y, bs = blockIdx.z, b = bs / sh.S, s = bs % sh.S;
  const int N = sh.N, D = sh.D;
  float* ks = smem + warp * 2 * D;
  float* vs = ks + D;
  if (j >= N) return;
  const size_t rs = (size_t)sh.H * D;
  const size_t koff = row_off(sh, b, s, j, h);
  for (int d = lane; d < D; d += 32) {
    ks[d] = to_f32<T>(k[koff + d]);
    vs[d] = to_f32<T>(v[koff + d]);
  }
  __syncwarp();
  const T* qb = q + row_off(sh, b, s, 0, h);
  const T* gb = dout + row_off(sh, b, s, 0, h);
  const float* bcol = bias + ((size_t)b * sh.H + h) * N * N + j;  // + i * N
  const float mj = mask[(size_t)bs * N + j];
  const float* lrow = lse + ((size_t)bs * sh.H + h) * N;
  const float* drow = delta + ((size_t)bs * sh.H + h) * N;
  float acc_k[kMaxDT], acc_v[kMaxDT];
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) acc_k[t] = acc_v[t] = 0.f;
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
      for (int t = 0; t < kMaxDT; ++t) {
        const int d = lane + 32 * t;
        if (d < D) {
          acc_v[t] = fmaf(pi, to_f32<T>(gr[d]), acc_v[t]);
          acc_k[t] = fmaf(di, to_f32<T>(qr[d]), acc_k[t]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) {
    const int d = lane + 32 * t;
    if (d < D) {
      dk[koff + d] = from_f32<T>(sh.scale * acc_k[t]);
      dv[koff + d] = from_f32<T>(acc_v[t]);
    }
  }
}

int check_evo(const char* what, int64_t B, int64_t S, int64_t N, int64_t H, int64_t D, int dtype) {
  if (B <= 0 || S <= 0 || N <= 0 || H <= 0 || D <= 0)
    return fail(EVG_EBADSHAPE, "%s: B=%lld S=%lld N=%lld H=%lld D=%lld must be positive", what,
                (long long)B, (long long)S, (long long)N, (long long)H, (long long)D);
  if (dtype != EVG_BF16 && dtype != EVG_F16 && dtype != EVG_F32)
    return fail(EVG_EDTYPE, "%s: dtype %d", what, dtype);
  if (D > 32 * kMaxDT || N > 32 * kMaxChunks)
    return fail(EVG_EUNSUPPORTED, "%s: head_dim %lld (max 256) or residues %lld (max 1024)", what,
                (long long)D, (long long)N);
  if (H > 65535 || B * S > 65535)
    return fail(EVG_EUNSUPPORTED, "%s: H=%lld or B*S=%lld above 65535", what, (long long)H,
                (long long)(B * S));
  return EVG_OK;
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
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    dim3 grid((unsigned)((N + kWarps - 1) / kWarps), (unsigned)H, (unsigned)(B * S));
    evo_fwd_kernel<T><<<grid, kWarps * 32, kWarps * D * sizeof(float), (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k, (const T*)v, res_mask, pair_bias, (T*)o, lse, sh);
    return check_launch("evoattention_fwd");
  });
}

extern "C" int64_t evg_evoattention_bwd_workspace_bytes(int64_t B, int64_t S, int64_t N,
                                                        int64_t H, int64_t D, int dtype) {
  (void)D; (void)dtype;
  if (B <= 0 || S <= 0 || N <= 0 || H <= 0) return 0;
  return B * S * H * N * (int64_t)sizeof(float);
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
  float* delta = (float*)workspace;
  cudaStream_t st = (cudaStream_t)stream;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    const unsigned tiles = (unsigned)((N + kWarps - 1) / kWarps);
    const size_t smem = (size_t)kWarps * 2 * D * sizeof(float);
    evo_delta_kernel<T><<<dim3(tiles, (unsigned)H, (unsigned)(B * S)), kWarps * 32, 0, st>>>(
        (const T*)dout, (const T*)o, delta, sh);
    evo_dq_dbias_kernel<T><<<dim3(tiles, (unsigned)H, (unsigned)B), kWarps * 32, smem, st>>>(
        (const T*)dout, (const T*)q, (const T*)k, (const T*)v, res_mask, pair_bias, lse, delta,
        (T*)dq, d_pair_bias, sh);
    evo_dkdv_kernel<T><<<dim3(tiles, (unsigned)H, (unsigned)(B * S)), kWarps * 32, smem, st>>>(
        (const T*)dout, (const T*)q, (const T*)k, (const T*)v, res_mask, pair_bias, lse, delta,
        (T*)dk, (T*)dv, sh);
    return check_launch("evoattention_bwd");
  });
}
