// Causal (grouped-query) attention forward/backward on the CUDA cores, for the
// shapes the tensor-core kernels do not take: float32 inputs and head sizes
// other than 64 / 128 (any D <= 256). These are the small correctness shapes of
// a decoder block (head_dim 16 / 32, float32); nothing here is tuned for speed.
//
// One warp owns one row: a query row in the forward and in dQ, a key row in
// dK/dV. Lanes take 32 consecutive rows of the other side at a time, and the
// rank-1 updates are spread over lanes by head-dimension index. Every sum has a
// fixed order, so results are bit-reproducible. Query head h reads key/value
// head h / (Hq / Hkv); dK/dV add up the query heads of the group in head order.
#include "attention_common.cuh"
#include "evg_common.cuh"

namespace evg {
namespace attn {
namespace {

constexpr int kWarps = 4;
constexpr int kMaxDT = 8;  // head_dim <= 256

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

// o[i] = sum_j softmax_j(scale q_i.k_j) v_j, lse[i] = log sum_j exp(scale q_i.k_j)
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
generic_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   T* __restrict__ o, float* __restrict__ lse, int Hq, int Hkv, int S, int D,
                   float scale) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * kWarps + warp;
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (Hq / Hkv);
  float* qs = smem + warp * D;
  if (i >= S) return;
  const T* qr = q + (((size_t)b * Hq + h) * S + i) * D;
  const T* kb = k + ((size_t)b * Hkv + g) * S * D;
  const T* vb = v + ((size_t)b * Hkv + g) * S * D;
  for (int d = lane; d < D; d += 32) qs[d] = to_f32<T>(qr[d]);
  __syncwarp();
  float m = -INFINITY, l = 0.f;
  float acc[kMaxDT];
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) acc[t] = 0.f;
  for (int j0 = 0; j0 <= i; j0 += 32) {
    const int j = j0 + lane;
    const float s = j <= i ? scale * dot_row<T>(qs, kb + (size_t)j * D, D) : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // 0 on the first chunk (m = -inf)
    const float p = expf(s - m_new);     // 0 for masked lanes
    l = l * corr + warp_sum(p);
    const float pr = round_to<T>(p);  // probabilities enter P V in the input dtype
#pragma unroll
    for (int t = 0; t < kMaxDT; ++t) acc[t] *= corr;
    const int n = min(32, i - j0 + 1);
    for (int jj = 0; jj < n; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pr, jj);
      const T* vr = vb + (size_t)(j0 + jj) * D;
#pragma unroll
      for (int t = 0; t < kMaxDT; ++t) {
        const int d = lane + 32 * t;
        if (d < D) acc[t] = fmaf(pj, to_f32<T>(vr[d]), acc[t]);
      }
    }
    m = m_new;
  }
  T* orow = o + (((size_t)b * Hq + h) * S + i) * D;
  const float inv = 1.0f / l;
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) {
    const int d = lane + 32 * t;
    if (d < D) orow[d] = from_f32<T>(acc[t] * inv);
  }
  if (lane == 0) lse[((size_t)b * Hq + h) * S + i] = m + logf(l);
}

// delta[i] = sum_d do[i][d] * o[i][d]
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
generic_delta_kernel(const T* __restrict__ dout, const T* __restrict__ o,
                     float* __restrict__ delta, int64_t rows, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * kWarps + warp;
  if (r >= rows) return;
  float s = 0.f;
  for (int d = lane; d < D; d += 32)
    s = fmaf(to_f32<T>(dout[r * D + d]), to_f32<T>(o[r * D + d]), s);
  s = warp_sum(s);
  if (lane == 0) delta[r] = s;
}

// dq_i = scale * sum_{j<=i} ds_ij k_j,  ds_ij = p_ij (do_i.v_j - delta_i)
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
generic_dq_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k,
                  const T* __restrict__ v, const float* __restrict__ lse,
                  const float* __restrict__ delta, T* __restrict__ dq, int Hq, int Hkv, int S,
                  int D, float scale) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * kWarps + warp;
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (Hq / Hkv);
  float* qs = smem + warp * 2 * D;
  float* gs = qs + D;
  if (i >= S) return;
  const size_t row = ((size_t)b * Hq + h) * S + i;
  const T* kb = k + ((size_t)b * Hkv + g) * S * D;
  const T* vb = v + ((size_t)b * Hkv + g) * S * D;
  for (int d = lane; d < D; d += 32) {
    qs[d] = to_f32<T>(q[row * D + d]);
    gs[d] = to_f32<T>(dout[row * D + d]);
  }
  __syncwarp();
  const float lse_i = lse[row], delta_i = delta[row];
  float acc[kMaxDT];
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) acc[t] = 0.f;
  for (int j0 = 0; j0 <= i; j0 += 32) {
    const int j = j0 + lane;
    float ds = 0.f;
    if (j <= i) {
      const float p = expf(scale * dot_row<T>(qs, kb + (size_t)j * D, D) - lse_i);
      ds = p * (dot_row<T>(gs, vb + (size_t)j * D, D) - delta_i);
    }
    const int n = min(32, i - j0 + 1);
    for (int jj = 0; jj < n; ++jj) {
      const float dj = __shfl_sync(0xffffffffu, ds, jj);
      const T* kr = kb + (size_t)(j0 + jj) * D;
#pragma unroll
      for (int t = 0; t < kMaxDT; ++t) {
        const int d = lane + 32 * t;
        if (d < D) acc[t] = fmaf(dj, to_f32<T>(kr[d]), acc[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) {
    const int d = lane + 32 * t;
    if (d < D) dq[row * D + d] = from_f32<T>(scale * acc[t]);
  }
}

// dv_j = sum_{heads of the group} sum_{i>=j} p_ij do_i ; dk_j = scale * sum ds_ij q_i
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
generic_dkdv_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k,
                    const T* __restrict__ v, const float* __restrict__ lse,
                    const float* __restrict__ delta, T* __restrict__ dk, T* __restrict__ dv,
                    int Hq, int Hkv, int S, int D, float scale) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * kWarps + warp;
  const int g = blockIdx.y, b = blockIdx.z;
  const int group = Hq / Hkv;
  float* ks = smem + warp * 2 * D;
  float* vs = ks + D;
  if (j >= S) return;
  const size_t krow = ((size_t)b * Hkv + g) * S + j;
  for (int d = lane; d < D; d += 32) {
    ks[d] = to_f32<T>(k[krow * D + d]);
    vs[d] = to_f32<T>(v[krow * D + d]);
  }
  __syncwarp();
  float acc_k[kMaxDT], acc_v[kMaxDT];
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) acc_k[t] = acc_v[t] = 0.f;
  for (int hh = 0; hh < group; ++hh) {
    const int h = g * group + hh;
    const size_t base = ((size_t)b * Hq + h) * S;
    for (int i0 = j; i0 < S; i0 += 32) {
      const int i = i0 + lane;
      float p = 0.f, ds = 0.f;
      if (i < S) {
        const T* qr = q + (base + i) * D;
        const T* gr = dout + (base + i) * D;
        p = expf(scale * dot_row<T>(ks, qr, D) - lse[base + i]);
        ds = p * (dot_row<T>(vs, gr, D) - delta[base + i]);
        p = round_to<T>(p);  // P^T dO takes P in the input dtype, as P V does
      }
      const int n = min(32, S - i0);
      for (int ii = 0; ii < n; ++ii) {
        const float pi = __shfl_sync(0xffffffffu, p, ii);
        const float di = __shfl_sync(0xffffffffu, ds, ii);
        const T* qr = q + (base + i0 + ii) * D;
        const T* gr = dout + (base + i0 + ii) * D;
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
  }
#pragma unroll
  for (int t = 0; t < kMaxDT; ++t) {
    const int d = lane + 32 * t;
    if (d < D) {
      dk[krow * D + d] = from_f32<T>(scale * acc_k[t]);
      dv[krow * D + d] = from_f32<T>(acc_v[t]);
    }
  }
}

}  // namespace

int64_t generic_bwd_workspace_bytes(int64_t B, int64_t Hq, int64_t S) {
  return B * Hq * S * (int64_t)sizeof(float);
}

int launch_generic_fwd(int dtype, const void* q, const void* k, const void* v, void* o,
                       float* lse, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                       float scale, cudaStream_t stream) {
  if (D > 32 * kMaxDT) return fail(EVG_EUNSUPPORTED, "causal attention: head_dim %lld > 256",
                                   (long long)D);
  if (Hq > 65535 || B > 65535)
    return fail(EVG_EUNSUPPORTED, "causal attention (generic): more than 65535 heads or batches");
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    dim3 grid((unsigned)((S + kWarps - 1) / kWarps), (unsigned)Hq, (unsigned)B);
    generic_fwd_kernel<T><<<grid, kWarps * 32, kWarps * D * sizeof(float), stream>>>(
        (const T*)q, (const T*)k, (const T*)v, (T*)o, lse, (int)Hq, (int)Hkv, (int)S, (int)D,
        scale);
    return check_launch("causal_attention_fwd (generic)");
  });
}

int launch_generic_bwd(int dtype, const void* dout, const void* q, const void* k, const void* v,
                       const void* o, const float* lse, void* dq, void* dk, void* dv,
                       void* workspace, int64_t workspace_bytes, int64_t B, int64_t Hq,
                       int64_t Hkv, int64_t S, int64_t D, float scale, cudaStream_t stream) {
  if (D > 32 * kMaxDT) return fail(EVG_EUNSUPPORTED, "causal attention: head_dim %lld > 256",
                                   (long long)D);
  if (Hq > 65535 || B > 65535)
    return fail(EVG_EUNSUPPORTED, "causal attention (generic): more than 65535 heads or batches");
  if (!workspace || workspace_bytes < generic_bwd_workspace_bytes(B, Hq, S))
    return fail(EVG_EWORKSPACE, "causal_attention_bwd: workspace %lld bytes, need %lld",
                (long long)workspace_bytes, (long long)generic_bwd_workspace_bytes(B, Hq, S));
  float* delta = (float*)workspace;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    const int64_t rows = B * Hq * S;
    generic_delta_kernel<T><<<(unsigned)((rows + kWarps - 1) / kWarps), kWarps * 32, 0, stream>>>(
        (const T*)dout, (const T*)o, delta, rows, (int)D);
    const size_t smem = (size_t)kWarps * 2 * D * sizeof(float);
    dim3 gq((unsigned)((S + kWarps - 1) / kWarps), (unsigned)Hq, (unsigned)B);
    generic_dq_kernel<T><<<gq, kWarps * 32, smem, stream>>>(
        (const T*)dout, (const T*)q, (const T*)k, (const T*)v, lse, delta, (T*)dq, (int)Hq,
        (int)Hkv, (int)S, (int)D, scale);
    dim3 gk((unsigned)((S + kWarps - 1) / kWarps), (unsigned)Hkv, (unsigned)B);
    generic_dkdv_kernel<T><<<gk, kWarps * 32, smem, stream>>>(
        (const T*)dout, (const T*)q, (const T*)k, (const T*)v, lse, delta, (T*)dk, (T*)dv,
        (int)Hq, (int)Hkv, (int)S, (int)D, scale);
    return check_launch("causal_attention_bwd (generic)");
  });
}

}  // namespace attn
}  // namespace evg
