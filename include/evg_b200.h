/*
 * evg_b200.h - C ABI of libevg_b200.so: hand-written sm_100a kernels for the
 * forward/backward ("autograd pair") hot path of evograd's softmax, LayerNorm,
 * RMSNorm, SwiGLU, RoPE and causal attention operators.
 *
 * Conventions shared by every entry point
 *   - All pointers are DEVICE pointers unless the comment says otherwise.
 *   - Tensors are dense row-major ("contiguous") unless strides are arguments.
 *   - `dtype` is one of EVG_F32 / EVG_F16 / EVG_BF16 and names the element type
 *     of the activations, parameters and gradients; statistics (mean, rstd,
 *     logsumexp) and partial sums are always float32.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *   - Nothing here allocates, frees or synchronises unless the comment says so.
 *     Kernels are only enqueued; scratch memory is passed in by the caller.
 *   - Return value: EVG_OK (0) or a negative EVG_E* code; the text of the last
 *     failure on the calling thread is available from evg_last_error().
 *   - Inputs are never written, with the one exception documented at
 *     evg_swiglu_bwd (outputs may alias inputs there).
 *
 * "replaces:" lines cite the reference (akumdam2/evograd) interface, by path
 * inside that project, whose device work the entry point takes over.
 */
#ifndef EVG_B200_H
#define EVG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 2: added geglu, fused add + rmsnorm, grouped-query attention, evoattention,
 *    the no-allocation rmsnorm backward and the bounded-wait self-test; every
 *    version-1 entry point is unchanged.
 * 3: added the evg_exchange_* calls (cross-GPU sum of parameter-gradient
 *    partial sums over peer memory); evoattention head sizes 32 / 64 run on the
 *    tensor cores; attention entry points reject a scale that is not positive
 *    and finite. */
#define EVG_ABI_VERSION 4

enum evg_dtype { EVG_F32 = 0, EVG_F16 = 1, EVG_BF16 = 2 };

enum evg_status {
  EVG_OK = 0,
  EVG_EBADSHAPE = -1,    /* a size is zero/negative or inconsistent          */
  EVG_EALIGN = -2,       /* a pointer is not aligned as the kernel requires  */
  EVG_EDTYPE = -3,       /* dtype enum out of range / unsupported for the op */
  EVG_ELAUNCH = -4,      /* CUDA reported an error when enqueuing            */
  EVG_ETIMEOUT = -5,     /* a bounded device-side wait gave up               */
  EVG_ENULL = -6,        /* a required pointer is NULL                       */
  EVG_EWORKSPACE = -7,   /* scratch buffer missing or too small              */
  EVG_EUNSUPPORTED = -8  /* shape outside what the kernel family covers      */
};

/* Library identity and diagnostics. */
int evg_abi_version(void);
const char* evg_last_error(void);
/* Name the compute capability the kernels were built for (returns 100). */
int evg_built_for_sm(void);

/*
 * Launch-shape override for experiments: key is "<op>.<knob>" (for example
 * "rmsnorm_bwd.group", "layernorm_fwd.vpt", "rows.threads"); value 0 restores
 * the built-in choice. Unknown keys return EVG_EUNSUPPORTED. Results never
 * depend on these knobs beyond floating-point summation order.
 */
int evg_tune_set(const char* key, int value);
int evg_tune_get(const char* key);

/* ------------------------------------------------------------------ softmax
 * y = softmax(x, dim=-1) evaluated in float32 and rounded once to dtype.
 * replaces: softmax_forward_ref, src/evograd/ops/level1/softmax/forward_ref.py:6-7;
 *           candidate forward for declaration ops/level1/softmax/__init__.py:69-92.
 * Saved state for the backward is y only.
 */
int evg_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols,
                    int dtype, void* stream);
/*
 * dx = y * (dy - sum(dy * y, dim=-1)), float32 arithmetic, one rounding.
 * replaces: backward semantics of ops/level1/softmax/__init__.py:78 (the
 *           gradient torch.autograd.grad returns in opdecl/oracle.py:103).
 */
int evg_softmax_bwd(const void* y, const void* dy, void* dx, int64_t rows,
                    int64_t cols, int dtype, void* stream);

/* ---------------------------------------------------------------- layernorm
 * mean/var over the last dimension in float32 with the two-pass variance
 * mean((x-mean)^2); y = ((x-mean)*rstd)*weight + bias, rounded once.
 * Writes mean[rows], rstd[rows] (float32): the only new saved state.
 * replaces: layernorm_forward_ref, ops/level1/layernorm/forward_ref.py:6-23;
 *           candidate forward for ops/level1/layernorm/__init__.py:124-171.
 */
int evg_layernorm_fwd(const void* x, const void* weight, const void* bias,
                      void* y, float* mean, float* rstd, int64_t rows,
                      int64_t hidden, float eps, int dtype, void* stream);
/* Bytes of scratch evg_layernorm_bwd needs for this shape on the current device. */
int64_t evg_layernorm_bwd_workspace_bytes(int64_t rows, int64_t hidden, int dtype);
/*
 * dx = rstd*(g - mean(g) - xhat*mean(g*xhat)), g = dy*weight;
 * dweight = sum_rows dy*xhat; dbias = sum_rows dy. The column sums are
 * two-stage and atomic-free: every thread block writes one float32 partial row
 * into `workspace`, a second kernel adds the partial rows in a fixed order.
 * Outputs of the column sums (each may be NULL):
 *   dweight, dbias : [hidden] in `dtype`
 *   dwdb_f32       : [2, hidden] float32 (row 0 dweight, row 1 dbias), for callers
 *                    that all-reduce partial sums across GPUs before rounding.
 * replaces: the gradients of opdecl/oracle.py:103 for the layernorm declaration
 *           (backward semantics ops/level1/layernorm/__init__.py:139).
 */
int evg_layernorm_bwd(const void* dy, const void* x, const void* weight,
                      const float* mean, const float* rstd, void* dx,
                      void* dweight, void* dbias, float* dwdb_f32,
                      void* workspace, int64_t workspace_bytes, int64_t rows,
                      int64_t hidden, int dtype, void* stream);

/* ------------------------------------------------------------------ rmsnorm
 * rstd = 1/sqrt(mean(x^2)+eps) in float32; y = (x*rstd)*weight rounded once.
 * Writes rstd[rows] float32 (the only new saved state).
 * replaces: rmsnorm_forward_ref, ops/level1/rmsnorm/forward_ref.py:6-21;
 *           candidate forward for ops/level1/rmsnorm/__init__.py:72-130.
 */
int evg_rmsnorm_fwd(const void* x, const void* weight, void* y, float* rstd,
                    int64_t rows, int64_t hidden, float eps, int dtype,
                    void* stream);
int64_t evg_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t hidden, int dtype);
/*
 * dx = (g - xhat*mean(g*xhat))*rstd with xhat = x*rstd, g = dy*weight;
 * dweight = sum_rows dy*xhat (two-stage, atomic-free, as for layernorm).
 * dweight ([hidden], dtype) and dweight_f32 ([hidden], float32) may each be NULL.
 * replaces: backward semantics ops/level1/rmsnorm/__init__.py:86.
 */
int evg_rmsnorm_bwd(const void* dy, const void* x, const void* weight,
                    const float* rstd, void* dx, void* dweight,
                    float* dweight_f32, void* workspace, int64_t workspace_bytes,
                    int64_t rows, int64_t hidden, int dtype, void* stream);

/*
 * RMSNorm backward without any allocation: same arguments and results as
 * evg_rmsnorm_bwd minus the workspace. It has no counterpart in the reference.
 *
 * Who needs it: code that cannot get device memory at the moment it must run
 * the backward - for instance a plug-in inside a host process that has already
 * given every byte of GPU memory to its own pool and offers no allocator to its
 * guests, or a step of a latency-bound loop where a cudaMalloc (which may
 * synchronise the whole device) is not acceptable. Such a caller has the
 * tensors it was handed and nothing else, so the float32 partial sums of the
 * two-stage dweight reduction are kept in an array that is compiled into the
 * library (10 MiB, resident on every GPU that loads the library until the
 * process exits) instead of a caller-provided workspace. The call performs no
 * cudaMalloc / cudaFree and calls no allocating library routine.
 *
 * Limits: hidden <= 8192. The launch is shaped so that its partial rows fit the
 * array (at least 320 rows of 8192 floats, more for narrower rows); a request
 * that cannot be made to fit returns EVG_EUNSUPPORTED with a message and
 * enqueues nothing.
 * First call on a device: looks up the array's device address (once per
 * device, under a lock, with that device current). Make that first call before
 * starting any stream capture.
 * Sharing: every call on a device uses the same array. Nothing in it has to
 * start at zero - each launch overwrites the rows it later reads - so stale
 * contents from an earlier call are harmless, but two of these calls whose
 * kernels overlap on the GPU (different streams, no ordering between them)
 * race on it. Calls on one stream are safe.
 */
int evg_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* weight,
                            const float* rstd, void* dx, void* dweight,
                            float* dweight_f32, int64_t rows, int64_t hidden,
                            int dtype, void* stream);

/* ------------------------------------------------------- fused add + rmsnorm
 * s = dtype(x + residual); rstd = rsqrt(mean(float(s)^2) + eps);
 * out = dtype(dtype(s * dtype(rstd)) * weight): the rounding points of
 * fused_add_rms_norm_forward_ref,
 * ops/level2/fused_add_rms_norm/forward_ref.py:6-14. Saved state is float32
 * rstd[rows] only; s is re-formed from x and residual by the backward.
 * replaces: the fused_add_rms_norm candidate pair derived from
 * ops/level2/fused_add_rms_norm/__init__.py:76-122 (forward_with_saved).
 */
int evg_fused_add_rmsnorm_fwd(const void* x, const void* residual,
                              const void* weight, void* out, float* rstd,
                              int64_t rows, int64_t hidden, float eps,
                              int dtype, void* stream);
/* Bytes of scratch evg_fused_add_rmsnorm_bwd needs (partial dweight rows). */
int64_t evg_fused_add_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t hidden,
                                                  int dtype);
/*
 * dx (which is also the gradient of residual: both reach the output through
 * s) and dweight [hidden]; `dweight_f32` (optional, [hidden]) receives the
 * unrounded float32 column sums for a caller that all-reduces before rounding.
 * replaces: backward_from_saved of the same declaration (returns dx, dr,
 * dweight with dx == dr, __init__.py:96-99).
 */
int evg_fused_add_rmsnorm_bwd(const void* dout, const void* x,
                              const void* residual, const void* weight,
                              const float* rstd, void* dx, void* dweight,
                              float* dweight_f32, void* workspace,
                              int64_t workspace_bytes, int64_t rows,
                              int64_t hidden, int dtype, void* stream);

/* ------------------------------------------------------------------- swiglu
 * c = round(silu(float(a))) * b  with the product taken in dtype, exactly the
 * rounding points of swiglu_forward_ref, ops/level1/swiglu/forward_ref.py:6-9.
 * `n` is the total element count (rows*cols). No saved state beyond a, b.
 */
int evg_swiglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype,
                   void* stream);
/*
 * s = sigmoid(a): db = dc*silu(a); da = dc*b*(s*(1 + a*(1-s))).
 * da may alias a and db may alias b (the declaration allows the backward to
 * overwrite them: ops/level1/swiglu/__init__.py:89-96).
 */
int evg_swiglu_bwd(const void* dc, const void* a, const void* b, void* da,
                   void* db, int64_t n, int dtype, void* stream);

/* -------------------------------------------------------------------- geglu
 * c = round(gelu_tanh(float(a))) * b, the rounding points of
 * geglu_forward_ref, ops/level1/geglu/forward_ref.py:6-9
 * (gelu_tanh(a) = a/2 * (1 + tanh(sqrt(2/pi) * (a + 0.044715 a^3)))).
 * Same calling convention as the swiglu pair; da/db may alias a/b.
 * replaces: the geglu candidate pair derived from
 * ops/level1/geglu/__init__.py:52-84.
 */
int evg_geglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype,
                  void* stream);
int evg_geglu_bwd(const void* dc, const void* a, const void* b, void* da,
                  void* db, int64_t n, int dtype, void* stream);

/* --------------------------------------------------------------------- rope
 * Rotate-half (GPT-NeoX / Llama) rotary embedding of a 4-D tensor whose last
 * dimension (head_dim, even) is contiguous:
 *   y[..., :h] = x1*cos1 - x2*sin1 ;  y[..., h:] = x2*cos2 + x1*sin2
 * with products and the sum in float32 and one rounding. `inverse` != 0 negates
 * the sine, which is the backward (dx from dy). Strides are in ELEMENTS for the
 * batch, head and token axes of x and y. The tables are [T, table_cols] with
 * table_cols == head_dim (both halves stored, cos1/cos2 read separately) or
 * head_dim/2 (one half stored), of element type `table_dtype`.
 * replaces: rope_forward_ref, ops/level1/rope/forward_ref.py:28-47 and the
 *           backward semantics ops/level1/rope/__init__.py:124-130.
 */
typedef struct evg_rope_tensor {
  const void* x;
  void* y;
  int64_t heads;
  int64_t x_stride_b, x_stride_h, x_stride_t;
  int64_t y_stride_b, y_stride_h, y_stride_t;
} evg_rope_tensor;

/* Rotates `count` (1 or 2) tensors sharing batch, T, head_dim and the tables
 * in ONE launch (for example q and k of one layer). */
int evg_rope(const evg_rope_tensor* tensors /* HOST pointer */, int count,
             const void* cos_table, const void* sin_table, int64_t batch,
             int64_t tokens, int64_t head_dim, int64_t table_cols,
             int table_dtype, int dtype, int inverse, void* stream);

/* --------------------------------------------------------- causal attention
 * o = softmax(scale * q k^T + causal_mask) v for q,k,v,o of shape [B,H,S,D]
 * (contiguous, D in {64,128}, dtype EVG_BF16 or EVG_F16), logits and softmax in
 * float32, probabilities rounded to dtype before the second product (the
 * rounding point of ops/level1/evoattention/forward_ref.py:44-47). Writes
 * lse[B,H,S] = log(sum exp(scale*s - max)) + max in float32 (natural log).
 * Runs on the tcgen05 tensor cores with TMEM accumulators and TMA-staged tiles.
 * replaces: F.scaled_dot_product_attention(q,k,v,is_causal=True) as called at
 *           ops/level3/llama3_decoder_layer/forward_ref.py:107 (there is no
 *           standalone causal-attention declaration in the reference).
 * Saved state: o and lse (q, k, v are kept by reference).
 */
int evg_causal_attention_fwd(const void* q, const void* k, const void* v,
                             void* o, float* lse, int64_t B, int64_t H,
                             int64_t S, int64_t D, float scale, int dtype,
                             void* stream);
int64_t evg_causal_attention_bwd_workspace_bytes(int64_t B, int64_t H, int64_t S,
                                                 int64_t D, int dtype);
/*
 * delta = rowsum(do*o); P = exp(scale*s - lse); dV = P^T dO; dP = dO V^T;
 * dS = P*(dP - delta); dQ = scale*dS K; dK = scale*dS^T Q.
 * dK/dV are accumulated in a fixed order by the block that owns a key tile:
 * same bits on every run. At head size 128 the same block also forms its part
 * of dQ and adds it to a float32 copy with global float32 adds, so dq can
 * differ in the last bit between runs; the tunable "attention.two_kernel_bwd"
 * = 1 (and head size 64) uses a second kernel that owns a query tile instead:
 * no atomics, bit-reproducible dq, about 10 % slower.
 * workspace holds two float32 arrays padded to whole 128-row tiles per (batch,
 * head), delta and the log-sum-exp in log2 units, and at head size 128 the
 * float32 dQ copy [B*H, padded S, 128] (ask the _workspace_bytes function).
 */
int evg_causal_attention_bwd(const void* dout, const void* q, const void* k,
                             const void* v, const void* o, const float* lse,
                             void* dq, void* dk, void* dv, void* workspace,
                             int64_t workspace_bytes, int64_t B, int64_t H,
                             int64_t S, int64_t D, float scale, int dtype,
                             void* stream);

/* ------------------------------------------- causal grouped-query attention
 * The same attention with Hq query heads sharing Hkv key/value heads
 * (Hq % Hkv == 0): q, o, dout, dq are [B,Hq,S,D]; k, v, dk, dv are [B,Hkv,S,D];
 * query head h reads k/v head h / (Hq/Hkv); dk/dv sum over the query heads of
 * a group inside one block (deterministic, no atomics). Equivalent to
 * repeat_interleave of k and v followed by scaled_dot_product_attention, as at
 * ops/level3/llama3_decoder_layer/forward_ref.py:100-107, without materialising
 * the repeated tensors. 16-bit inputs with D in {64,128} run on the tensor-core
 * kernels; float32 inputs and other head sizes (D <= 256; the decoder block's
 * small correctness shapes, __init__.py:52-61) run on plain CUDA-core kernels.
 */
int evg_causal_gqa_attention_fwd(const void* q, const void* k, const void* v,
                                 void* o, float* lse, int64_t B, int64_t Hq,
                                 int64_t Hkv, int64_t S, int64_t D, float scale,
                                 int dtype, void* stream);
int64_t evg_causal_gqa_attention_bwd_workspace_bytes(int64_t B, int64_t Hq,
                                                     int64_t Hkv, int64_t S,
                                                     int64_t D, int dtype);
int evg_causal_gqa_attention_bwd(const void* dout, const void* q, const void* k,
                                 const void* v, const void* o, const float* lse,
                                 void* dq, void* dk, void* dv, void* workspace,
                                 int64_t workspace_bytes, int64_t B, int64_t Hq,
                                 int64_t Hkv, int64_t S, int64_t D, float scale,
                                 int dtype, void* stream);

/*
 * The same two calls for a caller whose projections produce and consume
 * token-major tensors (the decoder layer at
 * ops/level3/llama3_decoder_layer/forward_ref.py:100-110 transposes o back to
 * [B,S,H*D] before the output projection, v comes out of its projection as
 * [B,S,Hkv*D], and their gradients likewise): v, o and dout are read / written
 * as [B,S,H,D] and dv is written as [B,S,Hkv,D]; q, k, dq, dk (which pass
 * through RoPE, which changes layout on the way) and lse keep the [B,H,S,D] /
 * [B,H,S] layout. Tensor-core shapes only (16-bit, D in {64,128}, 16-byte
 * aligned); EVG_EUNSUPPORTED otherwise.
 */
int evg_causal_gqa_attention_fwd_tm(const void* q, const void* k,
                                    const void* v_token_major,
                                    void* o_token_major, float* lse, int64_t B,
                                    int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                                    float scale, int dtype, void* stream);
int evg_causal_gqa_attention_bwd_tm(const void* dout_token_major, const void* q,
                                    const void* k, const void* v_token_major,
                                    const void* o_token_major,
                                    const float* lse, void* dq, void* dk,
                                    void* dv_token_major, void* workspace,
                                    int64_t workspace_bytes, int64_t B, int64_t Hq,
                                    int64_t Hkv, int64_t S, int64_t D, float scale,
                                    int dtype, void* stream);

/* ------------------------------------------------------------ evoattention
 * AlphaFold-3 style EvoformerAttention over [B, S, N, H, D] tensors (S = MSA
 * rows, N = residues): o = softmax(scale*q k^T + pair_bias + res_mask) v along
 * the residue axis, ops/level1/evoattention/forward_ref.py:22-49. res_mask is
 * float32 [B,S,N] (the reference's [B,S,1,1,N], additive per key), pair_bias
 * float32 [B,H,N,N] (the reference's [B,1,H,N,N], shared by all MSA rows).
 * lse is float32 [B,S,H,N]. Any of float32/float16/bfloat16, D <= 256,
 * N <= 1024; plain CUDA-core kernels (residue counts are a few hundred).
 * replaces: the evoattention candidate pair derived from
 * ops/level1/evoattention/__init__.py:80-137.
 */
int evg_evoattention_fwd(const void* q, const void* k, const void* v,
                         const float* res_mask, const float* pair_bias, void* o,
                         float* lse, int64_t B, int64_t S, int64_t N, int64_t H,
                         int64_t D, float scale, int dtype, void* stream);
int64_t evg_evoattention_bwd_workspace_bytes(int64_t B, int64_t S, int64_t N,
                                             int64_t H, int64_t D, int dtype);
/* dq, dk, dv in the input layout and dtype; d_pair_bias float32 [B,H,N,N] =
 * sum over the S axis of dS, accumulated in a fixed order without atomics. */
int evg_evoattention_bwd(const void* dout, const void* q, const void* k,
                         const void* v, const float* res_mask,
                         const float* pair_bias, const void* o, const float* lse,
                         void* dq, void* dk, void* dv, float* d_pair_bias,
                         void* workspace, int64_t workspace_bytes, int64_t B,
                         int64_t S, int64_t N, int64_t H, int64_t D, float scale,
                         int dtype, void* stream);

/*
 * Synchronises the current device (the one exception to "nothing synchronises")
 * and reports the sticky device-side status of the kernels that wait on
 * mbarriers (attention, the norm backward rings, wide softmax): every wait
 * inside them is bounded, and a wait that gives up records its identity,
 * lets the kernel finish and is reported here as EVG_ETIMEOUT. Results of that
 * launch are then undefined, and so is everything enqueued on the device
 * between that launch and this call (it may have consumed the bad results).
 * reset != 0 clears the status after reading it.
 */
int evg_device_status(int reset);

/*
 * Self-test of the bounded-wait protocol: launches one small block that waits
 * (through the same helper as the product kernels) for a barrier phase nothing
 * completes, gives up after `limit_cycles` SM cycles (0 < limit <= 4e8) and
 * returns normally. `observed_abort_word` (device pointer, optional) receives
 * the block's abort word (the id of the wait that gave up, 901). Afterwards
 * evg_device_status() reports EVG_ETIMEOUT once; the context stays usable.
 * No reference counterpart: the reference has no device-side waits.
 */
int evg_selftest_bounded_wait(int64_t limit_cycles, int* observed_abort_word,
                              void* stream);

/* ------------------------------------------------- cross-GPU parameter sums
 * One process per GPU; LayerNorm / RMSNorm over a row shard leave every rank
 * with float32 partial sums of dweight (and dbias) over its own rows. These
 * calls add the partial sums of all ranks of ONE node and round once: a rank
 * writes each sum, paired with a step counter in one 64-bit store, into the
 * other ranks' buffers through peer memory (CUDA IPC mappings, plain stores,
 * no multicast) and then adds what arrived in its own; every rank adds in
 * rank order and therefore obtains the same bits. They replace an
 * all_reduce(SUM) of the float32 sums followed by evg_cast_from_f32.
 * No counterpart in the reference (its --gpus option runs independent
 * searches; nothing there shards an operator).
 *
 * evg_exchange_create    allocates this rank's buffer (the only allocation;
 *                        room for max_floats values per step), writes the 64
 *                        byte IPC handle other ranks need to ipc_handle.
 * evg_exchange_connect   all_handles = the n_ranks handles in rank order (the
 *                        caller gathers them with its own collective); maps
 *                        the other ranks' buffers.
 * evg_exchange_connect_local   same-process wiring for tests: peer_buffers[r]
 *                        is the device address of rank r's buffer
 *                        (evg_exchange_buffer of its handle).
 * evg_exchange_sum_round enqueues the step's kernel on `stream`: partial is
 *                        this rank's float32 sums (count values), out
 *                        (optional) receives the sum over ranks rounded to
 *                        dtype, out_f32 (optional) the float32 sum. Every rank
 *                        must make the same sequence of calls; the kernels of
 *                        the ranks wait for one another, so each rank needs
 *                        its own GPU. The waits are bounded
 *                        (evg_exchange_set_wait_limit, SM cycles, default
 *                        4e9): a rank whose peers do not arrive gives up, and
 *                        evg_device_status() then reports EVG_ETIMEOUT.
 *                        Safe to capture in a CUDA graph and replay (the step
 *                        counter lives in device memory).
 */
typedef struct evg_exchange evg_exchange;
int evg_exchange_create(int64_t max_floats, int n_ranks, int rank,
                        evg_exchange** out, unsigned char* ipc_handle);
int evg_exchange_connect(evg_exchange* x, const unsigned char* all_handles);
int evg_exchange_connect_local(evg_exchange* x, void* const* peer_buffers);
void* evg_exchange_buffer(evg_exchange* x);
int evg_exchange_set_wait_limit(evg_exchange* x, int64_t cycles);
int evg_exchange_sum_round(evg_exchange* x, const float* partial, int64_t count,
                           void* out, int dtype, float* out_f32, void* stream);
int evg_exchange_destroy(evg_exchange* x);
/*
 * LayerNorm / RMSNorm backward over this rank's row shard with dweight (and
 * dbias) summed over the ranks of `exchange`: as evg_layernorm_bwd /
 * evg_rmsnorm_bwd, but the second stage of the column reduction also does the
 * cross-GPU sum, block by block (every block of 32 columns exchanges its own
 * sums; no extra launch). dweight / dbias receive the sums over ALL ranks'
 * rows, rounded once, identical on every rank. Every rank must make the same
 * sequence of calls on the exchange; workspace as for the plain entry points.
 * No counterpart in the reference.
 */
int evg_layernorm_bwd_exchange(const void* dy, const void* x, const void* weight,
                               const float* mean, const float* rstd, void* dx,
                               void* dweight, void* dbias, void* workspace,
                               int64_t workspace_bytes, int64_t rows,
                               int64_t hidden, int dtype, evg_exchange* exchange,
                               void* stream);
int evg_rmsnorm_bwd_exchange(const void* dy, const void* x, const void* weight,
                             const float* rstd, void* dx, void* dweight,
                             void* workspace, int64_t workspace_bytes,
                             int64_t rows, int64_t hidden, int dtype,
                             evg_exchange* exchange, void* stream);

/* ------------------------------------------------------------------ helpers
 * dst[i] = round_to_dtype(src[i]) for float32 src; used after the cross-GPU
 * all-reduce of float32 dweight/dbias partial sums.
 */
int evg_cast_from_f32(const float* src, void* dst, int64_t n, int dtype,
                      void* stream);
/* Writes `bytes` of a repeating pattern; the benchmark driver uses it on a
 * buffer larger than L2 to evict cached lines between timed iterations. */
int evg_flush_l2(void* buffer, int64_t bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EVG_B200_H */
