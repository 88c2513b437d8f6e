// Causal attention: the C entry points and what the tensor-core kernels share
// on the host side (argument checks, TMA descriptor encoding).
//
// The kernels live in attention_fwd2.cu / attention_bwd2.cu (tcgen05 + TMEM,
// head sizes 64 / 128, 16-bit inputs) and attention_generic.cu (CUDA cores,
// float32 and other head sizes). Work decomposition is deterministic: forward
// and the dQ kernel own a query tile, the dK/dV kernel owns a key tile.
#include <cmath>
#include <cstdio>
#include <mutex>

#include "attention_common.cuh"

namespace evg {

namespace umma {

bool encode_tile_map_16bit(CUtensorMap* map, const void* base, int fmt, uint64_t cols,
                           uint64_t rows, uint64_t outer, uint32_t box_rows) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      encode = (EncodeFn)fn;
  });
  if (!encode) return false;
  const cuuint64_t dims[3] = {cols, rows, outer};
  const cuuint64_t strides[2] = {cols * 2, cols * rows * 2};  // bytes, dims 1 and 2
  const cuuint32_t box[3] = {64, box_rows, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult rc = encode(
      map, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
      const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}


bool encode_tile_map_16bit_4d(CUtensorMap* map, const void* base, int fmt, uint64_t D, uint64_t S,
                              uint64_t H, uint64_t B, uint32_t box_rows, bool token_major) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      encode = (EncodeFn)fn;
  });
  if (!encode) return false;
  const cuuint64_t dims[4] = {D, S, H, B};
  // byte strides of positions, heads and batches
  const cuuint64_t strides[3] = {token_major ? H * D * 2 : D * 2, token_major ? D * 2 : S * D * 2,
                                 H * S * D * 2};
  const cuuint32_t box[4] = {64, box_rows, 1, 1};
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  const CUresult rc = encode(
      map, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
      const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

bool encode_tile_map_f32(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                         uint64_t outer, uint32_t box_cols, uint32_t box_rows, bool swizzle128) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      encode = (EncodeFn)fn;
  });
  if (!encode) return false;
  const cuuint64_t dims[3] = {cols, rows, outer};
  const cuuint64_t strides[2] = {cols * 4, cols * rows * 4};  // bytes, dims 1 and 2
  const cuuint32_t box[3] = {box_cols, box_rows, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult rc =
      encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box,
             elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
             swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

}  // namespace umma

namespace {

using namespace umma;
using namespace attn;


// The kernels take the row maximum on raw scores and scale afterwards, which is
// only the same thing for a positive, finite scale.
int check_scale(const char* what, float scale) {
  if (!(scale > 0.f) || !std::isfinite(scale))
    return fail(EVG_EUNSUPPORTED, "%s: scale %g (must be positive and finite)", what,
                (double)scale);
  return EVG_OK;
}

int check_attention_args(const char* what, int64_t B, int64_t H, int64_t S, int64_t D, int dtype,
                         float scale) {
  if (int rc = check_scale(what, scale)) return rc;
  if (B <= 0 || H <= 0 || S <= 0)
    return fail(EVG_EBADSHAPE, "%s: B=%lld H=%lld S=%lld must be positive", what, (long long)B,
                (long long)H, (long long)S);
  if (D != 64 && D != 128)
    return fail(EVG_EUNSUPPORTED, "%s: head_dim %lld (supported: 64, 128)", what, (long long)D);
  if (dtype != EVG_BF16 && dtype != EVG_F16)
    return fail(EVG_EDTYPE, "%s: dtype %d (supported: float16, bfloat16)", what, dtype);
  if (B * H > 65535 || S > (1 << 24))
    return fail(EVG_EUNSUPPORTED, "%s: B*H=%lld (max 65535) or S=%lld too large", what,
                (long long)(B * H), (long long)S);
  return EVG_OK;
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_causal_attention_fwd(const void* q, const void* k, const void* v, void* o,
                                        float* lse, int64_t B, int64_t H, int64_t S, int64_t D,
                                        float scale, int dtype, void* stream) {
  if (!q || !k || !v || !o || !lse) return fail(EVG_ENULL, "causal_attention_fwd: null pointer argument");
  if (int rc = check_attention_args("causal_attention_fwd", B, H, S, D, dtype, scale)) return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(EVG_EALIGN, "causal_attention_fwd: q/k/v/o must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  return attn::launch_fwd2_any((int)D, dtype == EVG_BF16 ? 1 : 0, q, k, v, o, lse, B, H, H, S,
                               scale, st);
}

extern "C" int64_t evg_causal_attention_bwd_workspace_bytes(int64_t B, int64_t H, int64_t S,
                                                            int64_t D, int dtype) {
  (void)dtype;
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  return attn::bwd2_workspace_bytes(B, H, S, D);
}

extern "C" int evg_causal_attention_bwd(const void* dout, const void* q, const void* k,
                                        const void* v, const void* o, const float* lse, void* dq,
                                        void* dk, void* dv, void* workspace,
                                        int64_t workspace_bytes, int64_t B, int64_t H, int64_t S,
                                        int64_t D, float scale, int dtype, void* stream) {
  if (!dout || !q || !k || !v || !o || !lse || !dq || !dk || !dv)
    return fail(EVG_ENULL, "causal_attention_bwd: null pointer argument");
  if (int rc = check_attention_args("causal_attention_bwd", B, H, S, D, dtype, scale)) return rc;
  const int64_t need = evg_causal_attention_bwd_workspace_bytes(B, H, S, D, dtype);
  if (!workspace || workspace_bytes < need)
    return fail(EVG_EWORKSPACE, "causal_attention_bwd: workspace %lld bytes, need %lld",
                (long long)workspace_bytes, (long long)need);
  for (const void* p : {dout, q, k, v, o, (const void*)dq, (const void*)dk, (const void*)dv, (const void*)workspace})
    if (!aligned16(p)) return fail(EVG_EALIGN, "causal_attention_bwd: tensors must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  return attn::launch_bwd2_any((int)D, dtype == EVG_BF16 ? 1 : 0, dout, q, k, v, o, lse, dq, dk,
                               dv, (float*)workspace, B, H, H, S, scale, st);
}


// ---------------------------------------------------- grouped-query attention
namespace {
bool tensor_core_shape(int64_t D, int dtype) {
  return (D == 64 || D == 128) && (dtype == EVG_BF16 || dtype == EVG_F16);
}
int check_gqa_args(const char* what, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                   int dtype, float scale) {
  if (int rc = check_scale(what, scale)) return rc;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || D <= 0)
    return fail(EVG_EBADSHAPE, "%s: B=%lld Hq=%lld Hkv=%lld S=%lld D=%lld must be positive", what,
                (long long)B, (long long)Hq, (long long)Hkv, (long long)S, (long long)D);
  if (Hq % Hkv != 0)
    return fail(EVG_EBADSHAPE, "%s: %lld query heads are not a multiple of %lld k/v heads", what,
                (long long)Hq, (long long)Hkv);
  if (dtype != EVG_BF16 && dtype != EVG_F16 && dtype != EVG_F32)
    return fail(EVG_EDTYPE, "%s: dtype %d", what, dtype);
  if (D > 256) return fail(EVG_EUNSUPPORTED, "%s: head_dim %lld > 256", what, (long long)D);
  if (B * Hq > 65535 || S > (1 << 24))
    return fail(EVG_EUNSUPPORTED, "%s: B*Hq=%lld (max 65535) or S=%lld too large", what,
                (long long)(B * Hq), (long long)S);
  return EVG_OK;
}
}  // namespace

extern "C" int evg_causal_gqa_attention_fwd(const void* q, const void* k, const void* v, void* o,
                                            float* lse, int64_t B, int64_t Hq, int64_t Hkv,
                                            int64_t S, int64_t D, float scale, int dtype,
                                            void* stream) {
  if (!q || !k || !v || !o || !lse)
    return fail(EVG_ENULL, "causal_gqa_attention_fwd: null pointer argument");
  if (int rc = check_gqa_args("causal_gqa_attention_fwd", B, Hq, Hkv, S, D, dtype, scale)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (tensor_core_shape(D, dtype) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o))
    return attn::launch_fwd2_any((int)D, dtype == EVG_BF16 ? 1 : 0, q, k, v, o, lse, B, Hq, Hkv, S,
                                 scale, st);
  return attn::launch_generic_fwd(dtype, q, k, v, o, lse, B, Hq, Hkv, S, D, scale, st);
}

extern "C" int64_t evg_causal_gqa_attention_bwd_workspace_bytes(int64_t B, int64_t Hq,
                                                                int64_t Hkv, int64_t S, int64_t D,
                                                                int dtype) {
  (void)Hkv;
  if (B <= 0 || Hq <= 0 || S <= 0) return 0;
  // the tensor-core path needs the larger scratch; it also covers the generic one
  (void)dtype;
  return attn::bwd2_workspace_bytes(B, Hq, S, D);
}

extern "C" int evg_causal_gqa_attention_bwd(const void* dout, const void* q, const void* k,
                                            const void* v, const void* o, const float* lse,
                                            void* dq, void* dk, void* dv, void* workspace,
                                            int64_t workspace_bytes, int64_t B, int64_t Hq,
                                            int64_t Hkv, int64_t S, int64_t D, float scale,
                                            int dtype, void* stream) {
  if (!dout || !q || !k || !v || !o || !lse || !dq || !dk || !dv)
    return fail(EVG_ENULL, "causal_gqa_attention_bwd: null pointer argument");
  if (int rc = check_gqa_args("causal_gqa_attention_bwd", B, Hq, Hkv, S, D, dtype, scale)) return rc;
  const int64_t need = evg_causal_gqa_attention_bwd_workspace_bytes(B, Hq, Hkv, S, D, dtype);
  if (!workspace || workspace_bytes < need)
    return fail(EVG_EWORKSPACE, "causal_gqa_attention_bwd: workspace %lld bytes, need %lld",
                (long long)workspace_bytes, (long long)need);
  cudaStream_t st = (cudaStream_t)stream;
  bool aligned = aligned16(workspace);
  for (const void* p : {dout, q, k, v, o, (const void*)dq, (const void*)dk, (const void*)dv})
    aligned = aligned && aligned16(p);
  if (tensor_core_shape(D, dtype) && aligned)
    return attn::launch_bwd2_any((int)D, dtype == EVG_BF16 ? 1 : 0, dout, q, k, v, o, lse, dq, dk,
                                 dv, (float*)workspace, B, Hq, Hkv, S, scale, st);
  return attn::launch_generic_bwd(dtype, dout, q, k, v, o, lse, dq, dk, dv, workspace,
                                  workspace_bytes, B, Hq, Hkv, S, D, scale, st);
}

extern "C" int evg_causal_gqa_attention_fwd_tm(const void* q, const void* k, const void* v,
                                               void* o_token_major, float* lse, int64_t B,
                                               int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                                               float scale, int dtype, void* stream) {
  if (!q || !k || !v || !o_token_major || !lse)
    return fail(EVG_ENULL, "causal_gqa_attention_fwd_tm: null pointer argument");
  if (int rc = check_gqa_args("causal_gqa_attention_fwd_tm", B, Hq, Hkv, S, D, dtype, scale))
    return rc;
  if (!tensor_core_shape(D, dtype) || !aligned16(q) || !aligned16(k) || !aligned16(v) ||
      !aligned16(o_token_major))
    return fail(EVG_EUNSUPPORTED,
                "causal_gqa_attention_fwd_tm: 16-bit, head size 64 / 128, 16-byte aligned only");
  attn::Layouts lay;
  lay.o_token_major = 1;
  lay.v_token_major = 1;
  return attn::launch_fwd2_any((int)D, dtype == EVG_BF16 ? 1 : 0, q, k, v, o_token_major, lse, B,
                               Hq, Hkv, S, scale, (cudaStream_t)stream, lay);
}

extern "C" int evg_causal_gqa_attention_bwd_tm(const void* dout, const void* q, const void* k,
                                               const void* v, const void* o_token_major,
                                               const float* lse, void* dq, void* dk,
                                               void* dv_token_major, void* workspace,
                                               int64_t workspace_bytes, int64_t B, int64_t Hq,
                                               int64_t Hkv, int64_t S, int64_t D, float scale,
                                               int dtype, void* stream) {
  if (!dout || !q || !k || !v || !o_token_major || !lse || !dq || !dk || !dv_token_major)
    return fail(EVG_ENULL, "causal_gqa_attention_bwd_tm: null pointer argument");
  if (int rc = check_gqa_args("causal_gqa_attention_bwd_tm", B, Hq, Hkv, S, D, dtype, scale))
    return rc;
  const int64_t need = evg_causal_gqa_attention_bwd_workspace_bytes(B, Hq, Hkv, S, D, dtype);
  if (!workspace || workspace_bytes < need)
    return fail(EVG_EWORKSPACE, "causal_gqa_attention_bwd_tm: workspace %lld bytes, need %lld",
                (long long)workspace_bytes, (long long)need);
  bool aligned = aligned16(workspace);
  for (const void* p : {dout, q, k, v, o_token_major, (const void*)dq, (const void*)dk,
                        (const void*)dv_token_major})
    aligned = aligned && aligned16(p);
  if (!tensor_core_shape(D, dtype) || !aligned)
    return fail(EVG_EUNSUPPORTED,
                "causal_gqa_attention_bwd_tm: 16-bit, head size 64 / 128, 16-byte aligned only");
  attn::Layouts lay;
  lay.o_token_major = 1;
  lay.dv_token_major = 1;
  lay.v_token_major = 1;
  lay.do_token_major = 1;
  return attn::launch_bwd2_any((int)D, dtype == EVG_BF16 ? 1 : 0, dout, q, k, v, o_token_major, lse,
                               dq, dk, dv_token_major, (float*)workspace, B, Hq, Hkv, S, scale,
                               (cudaStream_t)stream, lay);
}
