/*
 * ttb.h -- C ABI of the B200-native transformer-layer kernels (libttb.so).
 *
 * This is the boundary the C++ layer classes (and any other host language, through its FFI) call.
 * Plain pointers and sizes only; every function returns a ttb_status and never throws, traps or exits.
 * All pointers named "device" are CUDA device pointers valid on the context's device; work is queued
 * on the context's stream and is asynchronous unless stated otherwise.
 *
 * Each entry point names the interface of the reference project (Tencent/TurboTransformers, paths
 * relative to its root) that it replaces.
 */
#ifndef TTB_H_
#define TTB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ttb_ctx ttb_ctx;

typedef enum {
  TTB_OK = 0,
  TTB_ERR_INVALID = 1,      /* bad argument: null pointer, negative size, unsupported shape            */
  TTB_ERR_CUDA = 2,         /* a CUDA runtime/driver call failed; see ttb_last_error                   */
  TTB_ERR_UNSUPPORTED = 3,  /* dtype / shape combination has no kernel                                 */
  TTB_ERR_OOM = 4,          /* the device pool could not satisfy an allocation                         */
  TTB_ERR_DEVICE_WAIT = 5,  /* a bounded device-side wait (mbarrier) expired; results are undefined    */
  TTB_ERR_BAD_INDEX = 6     /* an embedding id was outside its table (it was clamped, not trapped on)  */
} ttb_status;

typedef enum { TTB_F32 = 0, TTB_F16 = 1, TTB_BF16 = 2, TTB_I8 = 3 } ttb_dtype;
typedef enum { TTB_ACT_GELU = 0, TTB_ACT_TANH = 1, TTB_ACT_RELU = 2 } ttb_act;
typedef enum { TTB_POOL_FIRST = 0, TTB_POOL_LAST = 1, TTB_POOL_MEAN = 2, TTB_POOL_MAX = 3 } ttb_pool;

/* Epilogues of ttb_linear / ttb_linear_int8 (what happens to the accumulator before it is stored). */
typedef enum {
  TTB_EPI_NONE = 0,          /* out = acc                                   (kernels::MatMul alone)       */
  TTB_EPI_BIAS = 1,          /* out = acc + bias                            (MatMul + AddBias)            */
  TTB_EPI_BIAS_GELU = 2,     /* out = gelu_tanh(acc + bias)                 (MatMul + AddBiasAct<Gelu>)   */
  TTB_EPI_BIAS_RESIDUAL = 3, /* out = acc + bias + residual                 (MatMul + AddInputBias)       */
  TTB_EPI_BIAS_TANH = 4      /* out = tanh(acc + bias)                      (MatMul + AddBiasAct<Tanh>)   */
} ttb_epilogue;
/* May be OR-ed into ttb_linear's `epilogue` when N is not a multiple of 8 and ldo is: declares columns
 * [N, round_up(N, 8)) of every output row scratch (the fast store path overwrites them with zeros). Without it
 * such an output takes a slower element-wise store that leaves those columns untouched. */
#define TTB_EPI_FLAG_ROW_PADDING_IS_SCRATCH 0x100

/* ---- context: replaces core::CUDADeviceContext (turbo_transformers/core/cuda_device_context.cpp:23-60),
 * one per device (and per host thread, if callers want concurrency) instead of one global singleton. ---- */
int ttb_ctx_create(int device, void* cuda_stream /* cudaStream_t; NULL = the legacy default stream */,
                   ttb_ctx** out);
int ttb_ctx_destroy(ttb_ctx* ctx);
/* Work queued after the call runs on `cuda_stream`, ordered after everything queued through the context before it (the new
 * stream waits for an event on the old one). A context serves one stream at a time: host threads that want different streams
 * at the same time use one context each. */
int ttb_ctx_set_stream(ttb_ctx* ctx, void* cuda_stream);
void* ttb_ctx_stream(ttb_ctx* ctx);
int ttb_ctx_device(ttb_ctx* ctx);
int ttb_ctx_sync(ttb_ctx* ctx);
/* Text of the last failure seen on this context ("" if none). Valid until the next call on the context. */
const char* ttb_last_error(ttb_ctx* ctx);
/* Synchronises the stream, then reads and clears the device-side status word that kernels set instead of
 * trapping (TTB_ERR_DEVICE_WAIT, TTB_ERR_BAD_INDEX). Replaces the `asm("trap;")` of
 * turbo_transformers/layers/kernels/gpu_embedding_kernel.cu:32-34 and the exit(0) of core/cuda_enforce.cuh:50-65. */
int ttb_device_status(ttb_ctx* ctx);
/* Number of kernel launches issued through this context since creation (for benchmarks). */
uint64_t ttb_launch_count(ttb_ctx* ctx);
const char* ttb_version(void);

/* ---- allocator: replaces core::allocator::Allocator / NaiveAllocator (cub caching allocator),
 * turbo_transformers/core/allocator/allocator_api.cpp:26-125 and naive_allocator.h:39-66, with a
 * stream-ordered CUDA memory pool. `name` keeps the reference's name-keyed contract (it is recorded for
 * statistics only). ---- */
int ttb_alloc(ttb_ctx* ctx, size_t bytes, const char* name, void** out_device_ptr);
int ttb_free(ttb_ctx* ctx, void* device_ptr, const char* name);
/* bytes currently handed out, high-water mark, and number of ttb_alloc calls */
int ttb_pool_stats(ttb_ctx* ctx, size_t* in_use, size_t* high_water, uint64_t* n_allocs);
/* Caps the bytes the pool may hand out (0 = no cap); a request beyond it returns TTB_ERR_OOM. */
int ttb_pool_set_limit(ttb_ctx* ctx, size_t bytes);
/* Arena mode: between ttb_arena_begin and ttb_arena_end every ttb_alloc is served from one buffer reserved up front, at
 * increasing 256-byte-aligned offsets, without any driver call; ttb_free of such a pointer does nothing, then or later. A
 * forward pass run this way places every temporary and its outputs at fixed addresses, which is what capturing that pass into
 * a CUDA graph needs (the graph's kernels keep using the arena at every replay, so outputs are valid until the next replay).
 * Every ttb_arena_begin reserves a buffer of its own, so graphs captured earlier keep theirs. ttb_arena_end hands the buffer
 * to the caller (*arena_out, may be NULL to leave it with the context until ttb_ctx_destroy); ttb_arena_release frees it once
 * nothing replays over it any more (it waits for the device first). No reference counterpart: the reference's model-aware
 * allocator (allocator_api.cpp:112-125) served the same purpose of a driver-call-free forward.
 * ttb_bytes_allocated_total: sum of all ttb_alloc sizes so far; its increase over one forward pass sizes the arena. */
int ttb_arena_begin(ttb_ctx* ctx, size_t bytes);
int ttb_arena_end(ttb_ctx* ctx, size_t* bytes_used, void** arena_out);
int ttb_arena_release(ttb_ctx* ctx, void* arena);
int ttb_bytes_allocated_total(ttb_ctx* ctx, uint64_t* bytes);
/* Model-aware plan: replaces bert_opt_mem_allocate_api (core/allocator/allocator_api.cpp:112-125,
 * bert_config.cpp:43-94): computes one arena size for a BERT forward of this shape and reserves it in the
 * pool so steady-state forwards make no driver calls. Returns the arena bytes. */
int ttb_plan_activations(ttb_ctx* ctx, int64_t batch, int64_t tokens, int64_t heads, int64_t hidden,
                         int64_t ffn, int64_t layers, int dtype, size_t* arena_bytes);

/* Synchronous host<->device copies on the context's stream: core::Memcpy (turbo_transformers/core/memory.cpp:40-50). */
int ttb_memcpy_h2d(ttb_ctx* ctx, void* device_dst, const void* host_src, size_t bytes);
int ttb_memcpy_d2h(ttb_ctx* ctx, void* host_dst, const void* device_src, size_t bytes);

/* Device-to-device copy of `rows` rows of `width_bytes` between pitched buffers, on the context's stream (asynchronous). */
int ttb_copy_2d(ttb_ctx* ctx, void* dst, size_t dst_pitch_bytes, const void* src, size_t src_pitch_bytes, size_t width_bytes,
                size_t rows);

/* ---- A1: kernels::MatMul (turbo_transformers/layers/kernels/mat_mul.cpp:30-118).
 * C[M,N] = alpha * op(A) * op(B) + beta * C, row-major; op = transpose when the flag is non-zero.
 * A is [M,K] (or [K,M] if a_trans), B is [K,N] (or [N,K] if b_trans). Exact-precision SIMT path,
 * any dtype in {F32,F16,BF16} with fp32 accumulation. ---- */
int ttb_matmul(ttb_ctx* ctx, int dtype, const void* A, int a_trans, const void* B, int b_trans, int64_t M,
               int64_t N, int64_t K, float alpha, float beta, void* C);
/* ---- A2: kernels::BatchMatMul (mat_mul.cpp:119-213): `batch` independent GEMMs, operands contiguous
 * with strides M*K, K*N, M*N. ---- */
int ttb_batch_matmul(ttb_ctx* ctx, int dtype, const void* A, int a_trans, const void* B, int b_trans,
                     int64_t batch, int64_t M, int64_t N, int64_t K, float alpha, float beta, void* C);

/* ---- A3: kernels::SplitAddBiasTransposeForScore, 3-output form (transpose.cpp:310-406;
 * gpu_transpose_kernel.cu:80-120,184-197): qkv [B,L,3,heads,d] + bias [3,heads,d] -> q,k,v [B,heads,L,d]. ---- */
int ttb_split_add_bias_transpose(ttb_ctx* ctx, int dtype, const void* qkv, const void* bias, int64_t B,
                                 int64_t L, int64_t heads, int64_t d, void* q, void* k, void* v);
/* ---- A5: kernels::TransposeForScore (transpose.cpp:158-191): [B,heads,L,d] -> [B,L,heads*d]. ---- */
int ttb_transpose_for_score(ttb_ctx* ctx, int dtype, const void* in, int64_t B, int64_t heads, int64_t L,
                            int64_t d, void* out);
/* kernels::AddBiasTransposeForScore (transpose.cpp:193-240): [B,L,heads,d] + bias -> [B,heads,L,d]. */
int ttb_add_bias_transpose_for_score(ttb_ctx* ctx, int dtype, const void* in, const void* bias, int64_t B,
                                     int64_t L, int64_t heads, int64_t d, void* out);
/* ---- S1: the *Pad family (transpose.cpp:409-623; gpu_transpose_kernel.cu:127-182,264-322,355-398).
 * Packed tokens [sumL, ...] <-> zero-padded [B,heads,maxL,d]. `cu_seqlens` is a DEVICE int32 array of
 * B+1 prefix sums (the reference passed a host vector and did malloc+memcpy+free per call). ---- */
int ttb_split_add_bias_transpose_pad(ttb_ctx* ctx, int dtype, const void* qkv, const void* bias,
                                     const int32_t* cu_seqlens, int64_t B, int64_t maxL, int64_t heads,
                                     int64_t d, void* q, void* k, void* v);
int ttb_transpose_for_score_pad(ttb_ctx* ctx, int dtype, const void* in, const int32_t* cu_seqlens, int64_t B,
                                int64_t maxL, int64_t heads, int64_t d, void* out);
int ttb_add_bias_transpose_for_score_pad(ttb_ctx* ctx, int dtype, const void* in, const void* bias,
                                         const int32_t* cu_seqlens, int64_t B, int64_t maxL, int64_t heads,
                                         int64_t d, void* out);

/* ---- A4: kernels::ApplyMaskAndSoftmax (softmax.cpp:28-125; gpu_softmax_kernel.cu:61-202): in-place
 * softmax(scores*scale + mask) over the last dim of [B,heads,Lq,Lk]. mask is fp32, NULL, one row per
 * batch ([B,Lk], mask_is_2d != 0) or one row per query ([B,Lq,Lk]). No length limit, no +1e-6. ---- */
int ttb_mask_softmax(ttb_ctx* ctx, int dtype, void* scores, const float* mask, int64_t B, int64_t heads,
                     int64_t Lq, int64_t Lk, float scale, int mask_is_2d);

/* ---- A6: kernels::AddBiasLayerNorm (layer_norm.cpp:98-180): out = LN(out + input + bias)*gamma + beta.
 * `eps` is honoured (the reference GPU kernel ignored it, gpu_layer_norm_kernel.cu:48,98). ---- */
int ttb_add_bias_layernorm(ttb_ctx* ctx, int dtype, void* out, const void* input, const void* bias,
                           const void* gamma, const void* beta, int64_t M, int64_t N, float eps);
/* ---- A7: kernels::LayerNorm (layer_norm.cpp:32-91): in place. `in` may equal `out`. ---- */
int ttb_layernorm(ttb_ctx* ctx, int dtype, const void* in, void* out, const void* gamma, const void* beta,
                  int64_t M, int64_t N, float eps);
/* LayerNorm for models that keep more precision between layers than their 16-bit dtype holds (no reference counterpart:
 * the reference is fp32 throughout). `in` is of out_dtype or F32 (an fp32 residual stream); out (out_dtype) is the
 * operand of the next GEMM; out_lo (out_dtype, may be NULL) receives y - round(y), the second activation plane of
 * ttb_linear_ex; out_f32 (may be NULL) the unrounded value, the residual of the next block. */
int ttb_layernorm_planes(ttb_ctx* ctx, int in_dtype, int out_dtype, const void* in, void* out, void* out_lo, float* out_f32,
                         const void* gamma, const void* beta, int64_t M, int64_t N, float eps);
/* ---- A8: kernels::AddBiasAct (activation.cpp:90-119): in-place act(out + bias). ---- */
int ttb_add_bias_act(ttb_ctx* ctx, int dtype, void* out, const void* bias, int64_t M, int64_t N, int act);
/* ---- A9: kernels::LookupEmbedding (embedding.cpp:28-85): out[i,:] (=|+=) table[ids[i],:]. An id outside
 * [0,vocab) is clamped and TTB_ERR_BAD_INDEX is recorded in the device status word. ---- */
int ttb_lookup_embedding(ttb_ctx* ctx, int dtype, void* out, const void* table, const int64_t* ids,
                         int64_t n_ids, int64_t hidden, int64_t vocab, int add);
/* ---- A10: kernels::AddBias / AddInputBias (utils.cpp:103-169). ---- */
int ttb_add_bias(ttb_ctx* ctx, int dtype, void* out, const void* bias, int64_t M, int64_t N);
int ttb_add_input_bias(ttb_ctx* ctx, int dtype, const void* in1, const void* in2, const void* bias, int64_t M,
                       int64_t N, void* out);
/* ---- A11: kernels::SeqPool (seq_pool.cpp:124-155): [B,L,H] -> [B,H]. ---- */
int ttb_seq_pool(ttb_ctx* ctx, int dtype, const void* in, int64_t B, int64_t L, int64_t H, int pool_type,
                 void* out);
/* Var-length First/Last pooling over packed tokens: out[b,:] = in[cu_seqlens[b] (or cu_seqlens[b+1]-1), :]. */
int ttb_seq_pool_varlen(ttb_ctx* ctx, int dtype, const void* in, const int32_t* cu_seqlens, int64_t B,
                        int64_t H, int pool_type, void* out);
/* ---- A12: PrepareBertMasks (layers/prepare_bert_masks.cpp:24-66; kernels/common.cpp:37-90). Any output
 * pointer may be NULL to skip it. position_ids[b,l] = l; token_type = 0; att_mask = 1 (int64 each);
 * extended[b,l] = -10000*(1 - att_mask_in[b,l]) as fp32 (att_mask_in NULL means all ones). ---- */
int ttb_prepare_bert_masks(ttb_ctx* ctx, int64_t B, int64_t L, const int64_t* att_mask_in, int64_t* att_mask_out,
                           int64_t* token_type_out, int64_t* position_ids_out, float* extended_out);

/* ================= fused entry points the layer classes use for F16 / BF16 / INT8 ================= */

/* Re-lays a Linear weight out for the tensor-core GEMM: K-major [N,K] in `dst_dtype`.
 * src is [K,N] row-major (the reference's default "[in,out]" packing, modeling_bert.py:88-95) or, when
 * src_is_nk != 0, already [N,K] (the reference's is_trans_weight=True). The layer owns dst; the source,
 * which may alias torch storage, is never modified. */
int ttb_prepack_weight(ttb_ctx* ctx, int src_dtype, const void* src, int src_is_nk, int64_t K, int64_t N,
                       int dst_dtype, void* dst);
/* Same, to int8 with one symmetric scale for the tensor: *scale_out (device fp32) = max|W|/127. */
int ttb_prepack_weight_int8(ttb_ctx* ctx, int src_dtype, const void* src, int src_is_nk, int64_t K, int64_t N,
                            int8_t* dst, float* scale_out);

/* out[M,N] = epilogue(A[M,K] . Wp[N,K]^T): kernels::MatMul + the elementwise kernel that followed it in
 * the reference (mat_mul.cpp:30-118 with activation.cpp:90-119 / utils.cpp:103-169), as ONE tcgen05/TMEM
 * GEMM fed by TMA. dtype in {F16,BF16}; A, out, residual row-major with leading dimensions lda/ldo/ldr
 * (elements); K % 8 == 0 and lda % 8 == 0 (16-byte TMA rows). bias/residual may be NULL if unused. */
int ttb_linear(ttb_ctx* ctx, int dtype, const void* A, int64_t lda, const void* Wp, const void* bias,
               const void* residual, int64_t ldr, int64_t M, int64_t N, int64_t K, int epilogue, void* out,
               int64_t ldo);
/* The general form of ttb_linear: operands that carry more precision than one tensor-core format are given as two planes,
 * and the kernel accumulates one product per pair of planes into the same accumulator:
 *   dtype F16 / BF16, A2 == NULL           out = epilogue(A . W^T)                                   (what ttb_linear computes)
 *   dtype F16 / BF16, A2 != NULL           out = epilogue(A . W^T + A2 . W^T): activations kept as a rounded value plus what
 *                                          the rounding dropped (see out_lo), so a bf16 model's GEMMs see 16 significant bits
 *   dtype F32 (A, A2, W, W2 all given)     out = epilogue(A . W^T + A2 . W^T + A . W2^T) on tf32 tensor cores: A/A2 and W/W2
 *                                          are the hi/lo planes ttb_split_tf32 makes; the sum has fp32-level accuracy. This is
 *                                          the tensor-core route of kernels::MatMul for fp32 models (mat_mul.cpp:81-96, where
 *                                          the reference selects CUBLAS_GEMM_DEFAULT_TENSOR_OP)
 * out_dtype is dtype, or F32 for 16-bit operands (an fp32 residual stream); bias and residual are of out_dtype. out_lo
 * (BF16 outputs only, may be NULL) receives v - round(v) for every output value v, with out's pitch. W and W2 are
 * K-major [N, K] (ttb_prepack_weight). K % 8 == 0 (16-bit) or K % 4 == 0 (F32); lda likewise. */
typedef struct ttb_linear_args {
  int dtype, out_dtype;
  const void* A;
  const void* A2;
  int64_t lda;
  const void* W;
  const void* W2;
  const void* bias;
  const void* residual;
  int64_t ldr;
  int64_t M, N, K;
  int epilogue;
  void* out;
  void* out_lo;
  int64_t ldo;
} ttb_linear_args;
int ttb_linear_ex(ttb_ctx* ctx, const ttb_linear_args* args);
/* out = LayerNorm(A . Wp^T + bias + residual) * gamma + beta over rows of N: the attention output projection and the FFN
 * output Linear of a post-LN encoder layer together with the AddBiasLayerNorm that follows them
 * (turbo_transformers/layers/bert_output.cpp:40-56, kernels/layer_norm.cpp:30-75). By default ttb_linear and
 * ttb_layernorm run in sequence. With TTB_GEMM_LN=1 in the environment, N a multiple of 256 up to 1024, M >= 1024 and
 * K >= 2048 (TTB_GEMM_LN=2: any K), one kernel does all of it: the CTAs holding a row block's N-tiles exchange row sums
 * through a workspace the context owns. That form needs its whole grid resident, so use it with one context per device.
 * The LayerNorm sees the sum rounded to `dtype` either way. F16/BF16, dense output rows, 16-byte aligned pointers. */
int ttb_linear_layernorm(ttb_ctx* ctx, int dtype, const void* A, int64_t lda, const void* Wp, const void* bias,
                         const void* residual, int64_t ldr, const void* gamma, const void* beta, float eps, int64_t M,
                         int64_t N, int64_t K, void* out, int64_t ldo);
/* hi[i] = x[i] rounded to tf32 (10 mantissa bits), lo[i] = x[i] - hi[i] rounded likewise; x may be hi (in place).
 * The operand planes of the F32 form of ttb_linear_ex. 16-byte aligned pointers. */
int ttb_split_tf32(ttb_ctx* ctx, const float* x, int64_t n, float* hi, float* lo);

/* int8 x int8 -> int32 (tcgen05 kind::i8), out = epilogue(acc * row_scale[m] * *w_scale + bias), out dtype
 * F16/BF16. Replaces the torch dynamic-quantised Linear + FusedAddBiasGELU / FusedAddBiasLayerNorm glue of
 * python/turbo_transformers/layers/qmodeling_bert.py:13-45. K % 16 == 0. */
int ttb_linear_int8(ttb_ctx* ctx, int out_dtype, const int8_t* Aq, const float* row_scale, const int8_t* Wq,
                    const float* w_scale, const void* bias, const void* residual, int64_t ldr, int64_t M,
                    int64_t N, int64_t K, int epilogue, void* out, int64_t ldo);
/* ttb_linear_int8 that also gathers, in its epilogue, what a per-row int8 quantiser of `out` needs: row_absmax[m] (fp32,
 * [M], overwritten) = max |out[m, :]| of the values as stored in out_dtype. With ttb_quantize_rows_int8_given_max the
 * output of one int8 Linear (the FFN's bias + GELU) becomes the int8 input of the next in one read of it instead of two. */
int ttb_linear_int8_rowmax(ttb_ctx* ctx, int out_dtype, const int8_t* Aq, const float* row_scale, const int8_t* Wq,
                           const float* w_scale, const void* bias, const void* residual, int64_t ldr, int64_t M,
                           int64_t N, int64_t K, int epilogue, void* out, int64_t ldo, float* row_absmax);
/* The reference's own int8 recipe, python/turbo_transformers/layers/qmodeling_bert.py:13-45: torch dynamic quantisation
 * (torch.quantization.quantize_dynamic, qint8) of a Linear. Weights: per-tensor symmetric, scale = max|W| / 127.5,
 * q = clamp(rint(W / scale), -128, 127), plus their per-output-row sums. Activations: per-tensor affine over the whole
 * [M, K] tensor with the range widened to contain 0, 7-bit levels 0..127 (the x86 engines' reduce_range), zero point from
 * the end of the range with the smaller rounding error. out = epilogue((sum_k (xq - zp) * wq) * x_scale * w_scale + bias).
 *   ttb_prepack_weight_int8_affine : dst int8 [N, K], *scale_out (device fp32), col_sum_out int32 [N]
 *   ttb_quantize_tensor_affine     : xq int8 [M, K] (values 0..127); qparams = device fp32 [4]: scale, zero point, and two
 *                                    words of scratch (the running minimum and maximum)
 *   ttb_linear_int8_affine         : the GEMM (tcgen05 kind::i8) with the zero-point correction in its epilogue */
int ttb_prepack_weight_int8_affine(ttb_ctx* ctx, int src_dtype, const void* src, int src_is_nk, int64_t K, int64_t N,
                                   int8_t* dst, float* scale_out, int32_t* col_sum_out);
int ttb_quantize_tensor_affine(ttb_ctx* ctx, int dtype, const void* x, int64_t M, int64_t K, int8_t* xq, float* qparams);
int ttb_linear_int8_affine(ttb_ctx* ctx, int out_dtype, const int8_t* Aq, const float* act_qparams, const int8_t* Wq,
                           const float* w_scale, const int32_t* col_sum, const void* bias, const void* residual, int64_t ldr,
                           int64_t M, int64_t N, int64_t K, int epilogue, void* out, int64_t ldo);
/* int8 Linear with the activations quantised on the fly, for callers that cannot allocate device memory.
 * This entry point has no counterpart in the reference. It exists for hosts that pass the library only their
 * inputs and outputs: a server whose arena already owns all device memory, code inside a region where the CUDA
 * allocator must not be entered, or a foreign runtime whose FFI cannot own device buffers. It computes
 *   out = epilogue(quantize_rows(x) . Wq^T * row_scale * *w_scale + bias)        (x: [M,K] F16/BF16, out likewise)
 * exactly like ttb_quantize_rows_int8 followed by ttb_linear_int8, but keeps the quantised activations and their
 * row scales in a fixed 8.25 MiB array inside the library image, which every GPU that loads the library holds
 * until the process exits. Limits: M <= 65536 and M*K <= 8388608; larger problems get TTB_ERR_INVALID and a
 * message that names the two-call path. It calls no allocator of any kind. The first call on each device looks
 * the array's address up (one runtime query); make that call before starting any stream capture. All calls on a
 * device share the one array and nothing in it carries over between calls, but two calls whose kernels overlap
 * on the GPU (different streams, or graphs replayed concurrently) would race on it: serialise them. */
int ttb_linear_int8_dynamic_noalloc(ttb_ctx* ctx, int dtype, const void* x, const int8_t* Wq, const float* w_scale,
                                    const void* bias, const void* residual, int64_t ldr, int64_t M, int64_t N,
                                    int64_t K, int epilogue, void* out, int64_t ldo);

/* Per-row dynamic symmetric int8 quantisation: scale[m] = max|x[m,:]|/127, xq = clamp(rint(x * (1/scale)), -127, 127)
 * with the reciprocal rounded to fp32. */
int ttb_quantize_rows_int8(ttb_ctx* ctx, int dtype, const void* x, int64_t M, int64_t K, int8_t* xq,
                           float* row_scale);

/* ttb_quantize_rows_int8 for rows whose maxima are known (row_absmax[m] = max|x[m,:]|): one streaming pass, results
 * identical to ttb_quantize_rows_int8. x F16/BF16, K % 8 == 0, 16-byte aligned x and xq. */
int ttb_quantize_rows_int8_given_max(ttb_ctx* ctx, int dtype, const void* x, int64_t M, int64_t K, const float* row_absmax,
                                     int8_t* xq, float* row_scale);

/* ttb_layernorm followed by ttb_quantize_rows_int8 of its output, in one pass: out (16-bit, may be `in`) is the layer
 * norm, xq / row_scale its per-row int8 form. For int8 models, whose Linears take the normalised activations as int8 and
 * whose residual path takes them in 16 bits (no reference counterpart: the reference quantises inside torch). */
int ttb_layernorm_quant_int8(ttb_ctx* ctx, int dtype, const void* in, void* out, int8_t* xq, float* row_scale, const void* gamma,
                             const void* beta, int64_t M, int64_t N, float eps);

/* Self-attention over packed tokens, replacing BatchMatMul + ApplyMaskAndSoftmax + BatchMatMul +
 * TransposeForScore and all *Pad kernels (multi_headed_attention.cpp:320-354,
 * multi_headed_attention_smart_batch.cpp:362-393) with one kernel that never writes the score matrix.
 *   qkv   : [T, 3*heads*d] rows = tokens, columns q|k|v (bias already added), dtype F16/BF16, d == 64
 *   total_tokens : T = cu_seqlens[B], the number of rows of qkv (known to the host; bounds the tile loads)
 *   cu_seqlens : device int32 [B+1]; sequence b owns token rows [cu[b], cu[b+1])
 *   mask  : optional fp32 additive mask, element (b, i, j) at mask[b*mask_batch_stride + i*mask_row_stride + j]
 *           (mask_row_stride = 0 for a per-key mask); NULL for none
 *   causal: non-zero masks keys j > i
 *   out   : [T, heads*d]
 */
int ttb_attention_fwd(ttb_ctx* ctx, int dtype, const void* qkv, int64_t total_tokens, const int32_t* cu_seqlens, int64_t B,
                      int64_t max_seqlen, int64_t heads, int64_t d, const float* mask,
                      int64_t mask_batch_stride, int64_t mask_row_stride, int causal, float scale, void* out);

/* Decoder step with a key/value cache: replaces the per-step Concat of the whole cache and the padded attention sequence
 * of `layer_cache` self-attention (multi_headed_attention.cpp:207-231, 320-354; Concat: kernels/utils.cpp:32-97).
 *   qkv      : [B * n_new, 3*heads*d], row b*n_new + t, columns q|k|v (bias already added), dtype F16/BF16, d == 64
 *   k_cache, v_cache : paged [pages, B, 16, heads*d]: token j of sequence b is row (j / 16, b, j % 16); tokens [0, past_len)
 *              are cached so far. Appending is in place and growth adds pages at the end.
 * ttb_kv_cache_append files the new keys/values as tokens [past_len, past_len + n_new) (after a prompt that went through
 * ttb_attention_fwd). ttb_attention_decode does the same append and then attends: query t sees tokens [0, past_len + t].
 * n_new <= 64 there; out is [B * n_new, heads*d]. Capacity is the caller's business: pages up to token past_len + n_new - 1
 * are written (ceil((past_len + n_new) / 16) pages). */
int ttb_kv_cache_append(ttb_ctx* ctx, int dtype, const void* qkv, int64_t B, int64_t n_new, int64_t heads, int64_t d,
                        void* k_cache, void* v_cache, int64_t past_len);
int ttb_attention_decode(ttb_ctx* ctx, int dtype, const void* qkv, int64_t B, int64_t n_new, int64_t heads, int64_t d,
                         void* k_cache, void* v_cache, int64_t past_len, float scale, void* out);

/* BERTEmbedding::operator() (layers/bert_embedding.cpp:24-65) in one pass: three gathers + LayerNorm.
 * ids is [n_tokens]. token_type_ids may be NULL (all 0). position_ids may be NULL: the position of token t is
 * then t - cu_seqlens[b] for the sequence b that owns it (packed batches, B+1 prefix sums), or t % seq_len
 * when cu_seqlens is NULL too (a [B, seq_len] batch). Ids outside a table are clamped and flagged. */
int ttb_embedding_ln(ttb_ctx* ctx, int dtype, const int64_t* ids, const int64_t* position_ids,
                     const int64_t* token_type_ids, const int32_t* cu_seqlens, int64_t B, int64_t seq_len,
                     int64_t n_tokens, const void* word, const void* position, const void* token_type,
                     const void* gamma, const void* beta, int64_t hidden, int64_t vocab, int64_t n_positions,
                     int64_t n_types, float eps, void* out);

/* ttb_embedding_ln with the two extra outputs of ttb_layernorm_planes (either may be NULL). */
int ttb_embedding_ln_planes(ttb_ctx* ctx, int dtype, const int64_t* ids, const int64_t* position_ids,
                            const int64_t* token_type_ids, const int32_t* cu_seqlens, int64_t B, int64_t seq_len,
                            int64_t n_tokens, const void* word, const void* position, const void* token_type,
                            const void* gamma, const void* beta, int64_t hidden, int64_t vocab, int64_t n_positions,
                            int64_t n_types, float eps, void* out, void* out_lo, float* out_f32);

/* cu_seqlens (device int32 [B+1]) from host sequence lengths; a helper for callers that hold the
 * reference's `query_seq_len_list` host vector (multi_headed_attention_smart_batch.h:60-75). Asynchronous on the
 * context's stream for B <= 960 (the lengths ride in the kernel's parameters); larger batches take a staging copy that the
 * call waits for. */
int ttb_build_cu_seqlens(ttb_ctx* ctx, const int64_t* host_seq_lens, int64_t B, int32_t* cu_seqlens_device);

/* Self-test of the bounded device-side waits that every tensor-core kernel's hang safety rests on (no reference
 * counterpart). Launches one small kernel in which a thread waits, for at most `limit_cycles` SM cycles (<= 1e8, a
 * twentieth of a second), on a barrier that nothing arrives at. The wait gives up by itself; the kernel then records
 * TTB_ERR_DEVICE_WAIT in the status word, which the next ttb_device_status returns (and clears).
 * observed (device int32 [3]): whether the wait reported completion (0 expected), the abort flag (1 expected), and the
 * time the wait took in units of 1024 cycles. */
int ttb_selftest_bounded_wait(ttb_ctx* ctx, int64_t limit_cycles, int32_t* observed_device);

#ifdef __cplusplus
}
#endif
#endif /* TTB_H_ */
