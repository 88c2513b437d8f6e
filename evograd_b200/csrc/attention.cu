// Placeholder entry points; replaced by the tcgen05 implementation.
#include "evg_common.cuh"
using namespace evg;
extern "C" int evg_causal_attention_fwd(const void*, const void*, const void*, void*, float*,
                                        int64_t, int64_t, int64_t, int64_t, float, int, void*) {
  return fail(EVG_EUNSUPPORTED, "causal_attention_fwd: not built yet");
}
extern "C" int64_t evg_causal_attention_bwd_workspace_bytes(int64_t B, int64_t H, int64_t S,
                                                            int64_t, int) {
  return B * H * S * 4;
}
extern "C" int evg_causal_attention_bwd(const void*, const void*, const void*, const void*,
                                        const void*, const float*, void*, void*, void*, void*,
                                        int64_t, int64_t, int64_t, int64_t, int64_t, float, int,
                                        void*) {
  return fail(EVG_EUNSUPPORTED, "causal_attention_bwd: not built yet");
}
