// Rotary position embedding (rotate-half convention) for sm_100a, forward and
// backward in one kernel family: the backward is the transposed rotation.
// HBM-bound: one read and one write per element; the cos/sin tables are a few
// MB and stay in L2. One launch can rotate two tensors (q and k).
#include "evg_common.cuh"

namespace evg {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxTensors = 2;

struct RopeTensor {
  const void* x;
  void* y;
  int64_t heads;
  int64_t xs_b, xs_h, xs_t;
  int64_t ys_b, ys_h, ys_t;
  int64_t items;  // batch * heads * tokens * (units per row)
};
struct RopeArgs {
  RopeTensor t[kMaxTensors];
  int count;
  const void* cos;
  const void* sin;
  int64_t batch, tokens;
  int head_dim, table_cols;
  int inverse;
};

// Forward:  y1 = x1*c1 - x2*s1 ; y2 = x2*c2 + x1*s2   (rope_forward_ref,
//           ops/level1/rope/forward_ref.py:44-47: separate float32 products, one add)
// Backward: dx1 = dy1*c1 + dy2*s2 ; dx2 = dy2*c2 - dy1*s1  (what autograd returns
//           for that forward; equals the declared "sine negated" rule when the
//           two table halves are equal).
__device__ __forceinline__ void rotate(float x1, float x2, float c1, float s1, float c2, float s2,
                                       bool inverse, float& y1, float& y2) {
  if (!inverse) {
    y1 = __fadd_rn(__fmul_rn(x1, c1), __fmul_rn(-x2, s1));
    y2 = __fadd_rn(__fmul_rn(x2, c2), __fmul_rn(x1, s2));
  } else {
    y1 = __fadd_rn(__fmul_rn(x1, c1), __fmul_rn(x2, s2));
    y2 = __fadd_rn(__fmul_rn(x2, c2), -__fmul_rn(x1, s1));
  }
}

template <typename TT, int N>
__device__ __forceinline__ void load_table(const TT* p, float (&f)[N]) {
  if constexpr (sizeof(TT) == 4) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const uint4 v = *reinterpret_cast<const uint4*>(p + 4 * i);
      f[4 * i + 0] = __uint_as_float(v.x); f[4 * i + 1] = __uint_as_float(v.y);
      f[4 * i + 2] = __uint_as_float(v.z); f[4 * i + 3] = __uint_as_float(v.w);
    }
  } else {
    static_assert(N == 8, "16-bit tables pair with 16-bit activations");
    unpack<TT>(*reinterpret_cast<const uint4*>(p), f);
  }
}

// Vector path: a work item is one 128-bit vector of the first half of a row
// together with the matching vector of the second half.
template <typename T, typename TT>
__global__ void __launch_bounds__(kThreads)
rope_vec_kernel(const RopeArgs args) {
  constexpr int N = Vec<T>::N;
  constexpr int U = 2;  // independent work items in flight per thread
  const RopeTensor& tz = args.t[blockIdx.y];
  const int half = args.head_dim / 2;
  const int hv = half / N;  // vectors per half row
  const T* x = (const T*)tz.x;
  T* y = (T*)tz.y;
  const TT* ct = (const TT*)args.cos;
  const TT* st = (const TT*)args.sin;
  const bool full = args.table_cols == args.head_dim;
  // Walk the faster-varying of (head, token) first so neighbouring threads
  // touch neighbouring memory whichever layout the caller uses.
  const bool head_inner = tz.xs_h < tz.xs_t;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < tz.items;
       base += stride * U) {
    uint4 v1[U], v2[U];
    int64_t yoff[U], trow[U];
    int iv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t item = base + u * stride;
      if (item < tz.items) {
        const int i = (int)(item % hv);
        int64_t r = item / hv;
        int64_t h, t;
        if (head_inner) { h = r % tz.heads; r /= tz.heads; t = r % args.tokens; r /= args.tokens; }
        else { t = r % args.tokens; r /= args.tokens; h = r % tz.heads; r /= tz.heads; }
        const int64_t b = r;
        const T* xr = x + b * tz.xs_b + h * tz.xs_h + t * tz.xs_t + i * N;
        v1[u] = ld_vec(xr);
        v2[u] = ld_vec(xr + half);
        yoff[u] = b * tz.ys_b + h * tz.ys_h + t * tz.ys_t + i * N;
        trow[u] = t * args.table_cols + i * N;
        iv[u] = i;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t item = base + u * stride;
      if (item < tz.items) {
        float c1[N], s1[N], c2[N], s2[N];
        load_table<TT, N>(ct + trow[u], c1);
        load_table<TT, N>(st + trow[u], s1);
        if (full) {
          load_table<TT, N>(ct + trow[u] + half, c2);
          load_table<TT, N>(st + trow[u] + half, s2);
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j) { c2[j] = c1[j]; s2[j] = s1[j]; }
        }
        float x1[N], x2[N], o1[N], o2[N];
        unpack<T>(v1[u], x1);
        unpack<T>(v2[u], x2);
#pragma unroll
        for (int j = 0; j < N; ++j)
          rotate(x1[j], x2[j], c1[j], s1[j], c2[j], s2[j], args.inverse != 0, o1[j], o2[j]);
        T* yr = y + yoff[u];
        st_vec(yr, pack<T>(o1));
        st_vec(yr + half, pack<T>(o2));
      }
    }
    (void)iv;
  }
}

// Fast path when a half row is a power-of-two number of vectors: a thread owns
// one (token, vector) position, loads its cos/sin values ONCE and then walks
// over (batch, head) pairs, so the table traffic and its unpacking are amortised
// over every pair the thread visits and no per-element index division is left.
// grid = (token tiles, chunks of (batch, head) pairs, tensors).
template <typename T, typename TT>
__global__ void __launch_bounds__(kThreads)
rope_tile_kernel(const RopeArgs args, int hv_log2, int pairs_per_chunk) {
  constexpr int N = Vec<T>::N;
  constexpr int U = 4;  // (batch, head) pairs in flight per thread
  const RopeTensor& tz = args.t[blockIdx.z];
  const int half = args.head_dim / 2;
  const int hv = 1 << hv_log2;
  const int i = threadIdx.x & (hv - 1);
  const int64_t t = (int64_t)blockIdx.x * (kThreads >> hv_log2) + (threadIdx.x >> hv_log2);
  if (t >= args.tokens) return;
  const int64_t pairs = args.batch * tz.heads;
  int64_t n = (int64_t)blockIdx.y * pairs_per_chunk;
  const int64_t n_end = min(n + (int64_t)pairs_per_chunk, pairs);
  if (n >= n_end) return;

  float c1[N], s1[N], c2[N], s2[N];
  {
    const TT* crow = (const TT*)args.cos + t * args.table_cols + i * N;
    const TT* srow = (const TT*)args.sin + t * args.table_cols + i * N;
    load_table<TT, N>(crow, c1);
    load_table<TT, N>(srow, s1);
    if (args.table_cols == args.head_dim) {
      load_table<TT, N>(crow + half, c2);
      load_table<TT, N>(srow + half, s2);
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) { c2[j] = c1[j]; s2[j] = s1[j]; }
    }
  }
  const T* x = (const T*)tz.x + t * tz.xs_t + i * N;
  T* y = (T*)tz.y + t * tz.ys_t + i * N;
  const bool inverse = args.inverse != 0;
  int64_t b = n / tz.heads, h = n % tz.heads;
  for (; n < n_end; n += U) {
    uint4 v1[U], v2[U];
    int64_t yo[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (n + u < n_end) {
        const T* xr = x + b * tz.xs_b + h * tz.xs_h;
        v1[u] = ld_vec(xr);
        v2[u] = ld_vec(xr + half);
        yo[u] = b * tz.ys_b + h * tz.ys_h;
        if (++h == tz.heads) { h = 0; ++b; }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (n + u < n_end) {
        float x1[N], x2[N], o1[N], o2[N];
        unpack<T>(v1[u], x1);
        unpack<T>(v2[u], x2);
#pragma unroll
        for (int j = 0; j < N; ++j)
          rotate(x1[j], x2[j], c1[j], s1[j], c2[j], s2[j], inverse, o1[j], o2[j]);
        st_vec(y + yo[u], pack<T>(o1));
        st_vec(y + yo[u] + half, pack<T>(o2));
      }
    }
  }
}

// Scalar path for head sizes or alignments the vector path does not cover.
template <typename T, typename TT>
__global__ void __launch_bounds__(kThreads)
rope_scalar_kernel(const RopeArgs args) {
  const RopeTensor& tz = args.t[blockIdx.y];
  const int half = args.head_dim / 2;
  const T* x = (const T*)tz.x;
  T* y = (T*)tz.y;
  const TT* ct = (const TT*)args.cos;
  const TT* st = (const TT*)args.sin;
  const bool full = args.table_cols == args.head_dim;
  for (int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; item < tz.items;
       item += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(item % half);
    int64_t r = item / half;
    const int64_t t = r % args.tokens; r /= args.tokens;
    const int64_t h = r % tz.heads;
    const int64_t b = r / tz.heads;
    const T* xr = x + b * tz.xs_b + h * tz.xs_h + t * tz.xs_t + i;
    const float c1 = to_f32<TT>(ct[t * args.table_cols + i]);
    const float s1 = to_f32<TT>(st[t * args.table_cols + i]);
    const float c2 = full ? to_f32<TT>(ct[t * args.table_cols + half + i]) : c1;
    const float s2 = full ? to_f32<TT>(st[t * args.table_cols + half + i]) : s1;
    float o1, o2;
    rotate(to_f32<T>(xr[0]), to_f32<T>(xr[half]), c1, s1, c2, s2, args.inverse != 0, o1, o2);
    T* yr = y + b * tz.ys_b + h * tz.ys_h + t * tz.ys_t + i;
    yr[0] = from_f32<T>(o1);
    yr[half] = from_f32<T>(o2);
  }
}

template <typename T, typename TT>
int launch_rope(RopeArgs& args, cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  const int half = args.head_dim / 2;
  bool vec_ok = half % N == 0 && aligned16(args.cos) && aligned16(args.sin) &&
                (args.table_cols * sizeof(TT)) % 16 == 0 && (half * sizeof(TT)) % 16 == 0;
  for (int i = 0; i < args.count; ++i) {
    const RopeTensor& t = args.t[i];
    vec_ok = vec_ok && aligned16(t.x) && aligned16(t.y) && t.xs_b % N == 0 && t.xs_h % N == 0 &&
             t.xs_t % N == 0 && t.ys_b % N == 0 && t.ys_h % N == 0 && t.ys_t % N == 0;
  }
  int per_sm = tune("rope.blocks_per_sm");
  if (per_sm <= 0) per_sm = 27;
  const int64_t cap = (int64_t)device_info().sm_count * per_sm;
  const int hv = vec_ok ? half / N : 0;
  if (vec_ok && hv >= 1 && hv <= 64 && (hv & (hv - 1)) == 0 && !tune("rope.generic")) {
    int hv_log2 = 0;
    while ((1 << hv_log2) < hv) ++hv_log2;
    const int tokens_per_block = kThreads >> hv_log2;
    const int64_t tiles = (args.tokens + tokens_per_block - 1) / tokens_per_block;
    int64_t max_pairs = 0;
    for (int i = 0; i < args.count; ++i)
      max_pairs = args.batch * args.t[i].heads > max_pairs ? args.batch * args.t[i].heads : max_pairs;
    if (tiles == 0 || max_pairs == 0) return EVG_OK;
    // enough chunks to fill the machine, but at least 4 pairs per thread
    int64_t chunks = (cap + tiles * args.count - 1) / (tiles * args.count);
    if (chunks > (max_pairs + 3) / 4) chunks = (max_pairs + 3) / 4;
    if (chunks < 1) chunks = 1;
    if (chunks > 65535) chunks = 65535;
    // A thread takes its pairs four at a time: a chunk that is not a multiple of four ends in
    // a round of loads that is partly empty (q, k [8, 4096, 32, 128] bf16: 26 pairs per chunk
    // 183.8 us, 16 pairs per chunk 177.2 us).
    int pairs_per_chunk = (int)((max_pairs + chunks - 1) / chunks);
    if (pairs_per_chunk > 4) pairs_per_chunk = (pairs_per_chunk + 3) / 4 * 4;
    chunks = (max_pairs + pairs_per_chunk - 1) / pairs_per_chunk;
    if (tiles <= 0x7fffffff) {
      dim3 grid((unsigned)tiles, (unsigned)chunks, (unsigned)args.count);
      rope_tile_kernel<T, TT><<<grid, kThreads, 0, stream>>>(args, hv_log2, pairs_per_chunk);
      return check_launch("rope");
    }
  }
  const int unit = vec_ok ? N : 1;
  int64_t max_items = 0;
  for (int i = 0; i < args.count; ++i) {
    args.t[i].items = args.batch * args.t[i].heads * args.tokens * (half / unit);
    if (args.t[i].items > max_items) max_items = args.t[i].items;
  }
  if (max_items == 0) return EVG_OK;
  int64_t blocks = (max_items + 2 * kThreads - 1) / (2 * kThreads);
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks, (unsigned)args.count);
  if (vec_ok) rope_vec_kernel<T, TT><<<grid, kThreads, 0, stream>>>(args);
  else rope_scalar_kernel<T, TT><<<grid, kThreads, 0, stream>>>(args);
  return check_launch("rope");
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_rope(const evg_rope_tensor* tensors, int count, const void* cos_table,
                        const void* sin_table, int64_t batch, int64_t tokens, int64_t head_dim,
                        int64_t table_cols, int table_dtype, int dtype, int inverse,
                        void* stream) {
  if (!tensors || !cos_table || !sin_table) return fail(EVG_ENULL, "rope: null pointer argument");
  if (count < 1 || count > kMaxTensors)
    return fail(EVG_EBADSHAPE, "rope: count=%d (1 or 2 tensors per launch)", count);
  if (batch < 0 || tokens < 0 || head_dim <= 0 || head_dim % 2 || head_dim > (1 << 20))
    return fail(EVG_EBADSHAPE, "rope: batch=%lld tokens=%lld head_dim=%lld (head_dim must be even)",
                (long long)batch, (long long)tokens, (long long)head_dim);
  if (table_cols != head_dim && table_cols != head_dim / 2)
    return fail(EVG_EBADSHAPE, "rope: table_cols=%lld must be head_dim or head_dim/2",
                (long long)table_cols);
  if (table_dtype != dtype && table_dtype != EVG_F32)
    return fail(EVG_EDTYPE, "rope: table dtype %d must equal dtype %d or be float32", table_dtype,
                dtype);
  RopeArgs args{};
  args.count = count;
  for (int i = 0; i < count; ++i) {
    if (!tensors[i].x || !tensors[i].y) return fail(EVG_ENULL, "rope: tensor %d has a null pointer", i);
    if (tensors[i].heads < 0) return fail(EVG_EBADSHAPE, "rope: tensor %d heads < 0", i);
    args.t[i] = RopeTensor{tensors[i].x, tensors[i].y, tensors[i].heads, tensors[i].x_stride_b,
                           tensors[i].x_stride_h, tensors[i].x_stride_t, tensors[i].y_stride_b,
                           tensors[i].y_stride_h, tensors[i].y_stride_t, 0};
  }
  args.cos = cos_table; args.sin = sin_table;
  args.batch = batch; args.tokens = tokens;
  args.head_dim = (int)head_dim; args.table_cols = (int)table_cols;
  args.inverse = inverse;
  cudaStream_t st = (cudaStream_t)stream;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    if (table_dtype == EVG_F32) return launch_rope<T, float>(args, st);
    return launch_rope<T, T>(args, st);
  });
}
