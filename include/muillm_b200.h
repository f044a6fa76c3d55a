/*
 * muillm_b200 — C ABI of the B200 (sm_100a) decode hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, i.e. a
 * cudaStream_t / CUstream; NULL = the legacy default stream) and returns a mui_status_t. Nothing
 * here allocates device memory unless its comment says so; outputs and scratch are caller-owned.
 * Launches are asynchronous on the given stream. A non-zero status leaves a message that
 * mui_last_error() returns (thread-local).
 *
 * Citations name the file:line of the Epliz/muiLLM interface each entry point stands in for.
 */
#ifndef MUILLM_B200_H_
#define MUILLM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MUI_API __attribute__((visibility("default")))

typedef enum {
  MUI_OK = 0,
  MUI_ERR_INVALID_ARG = 1,  /* null pointer, bad size, misaligned pointer */
  MUI_ERR_UNSUPPORTED = 2,  /* shape/dtype outside what the kernels cover */
  MUI_ERR_CUDA = 3,         /* a CUDA runtime call failed */
  MUI_ERR_DEVICE = 4,       /* a kernel recorded a device-side status (timeout of a bounded wait) */
  MUI_ERR_COMM = 5          /* communicator bootstrap or peer mapping failed */
} mui_status_t;

/* 16-bit element type of activations, weights and outputs.                              */
/* Mirrors the fp16/bf16 twin kernels of the reference (csrc/linear/linear.cu:40-70).    */
typedef enum { MUI_F16 = 0, MUI_BF16 = 1 } mui_dtype_t;

/* Activation applied to the accumulator before biases (csrc/linear/activation.h:4-7).   */
typedef enum { MUI_ACT_IDENTITY = 0, MUI_ACT_SILU = 1 } mui_activation_t;

/* Weight-only 8-bit formats.
 *  MUI_W8_SYM_ROW   : int8, symmetric, one fp16/bf16 scale per output row  (w = s[n] * q)
 *  MUI_W8_GROUP_MIN : uint8, asymmetric, per (row, group) {scale, min} pairs stored [N*G, 2] in the
 *                     activation dtype (w = q * scale + min) — the layout produced by
 *                     muillm/quantization/rtnquantizer.py:49-88 and consumed by
 *                     csrc/int8_linear_kernels.cu:238-249. */
typedef enum { MUI_W8_SYM_ROW = 0, MUI_W8_GROUP_MIN = 1 } mui_w8_format_t;

/* Launch flags (bit set). */
#define MUI_FLAG_PDL 1u          /* launch with programmatic stream serialization (overlaps the weight prefetch
                                    of this kernel with the tail of the previous kernel on the stream) */
#define MUI_FLAG_FORCE_GENERIC 2u /* use the plain-load kernel even where the bulk-copy pipeline applies */
#define MUI_FLAG_FORCE_PIPELINE 4u /* fail with MUI_ERR_UNSUPPORTED instead of falling back to the plain-load kernel */
#define MUI_FLAG_SPLIT_CONTEXT 32u  /* fused decode attention with a workspace: the tokens in view are split over several
                                      CTAs per KV head (about 256 each), each running the tensor-core kernel of
                                      MUI_FLAG_SHORT_CONTEXT on its part; the last one to arrive merges the parts */
#define MUI_FLAG_SHORT_CONTEXT 16u  /* mui_rope_flash_decode / decode stack: at most a few hundred tokens are attended;
                                      one CTA per KV head stages the whole K/V history in shared memory (up to 384 rows
                                      per round) before the QKV projection has finished. Correct for any length. */

MUI_API const char* mui_status_string(mui_status_t s);
MUI_API const char* mui_last_error(void);
MUI_API int mui_version(void);

/* ---- engine: per-device properties (csrc/engine.cpp:3-25, csrc/gpu_info.cpp) -------------------- */
typedef struct mui_device_props {
  int device;
  int sm_count;
  int cc_major, cc_minor;
  int smem_per_block_optin;
  int l2_bytes;
  size_t total_mem;
} mui_device_props_t;
MUI_API mui_status_t mui_device_props(int device, mui_device_props_t* out);

/* Reads (and clears when `clear` != 0) the device status word that kernels set when a bounded wait
 * ran out. Synchronises the device. *code == 0 means no kernel reported anything. */
MUI_API mui_status_t mui_device_status(unsigned* code, int clear);

/* ---- launch tracing (the reference has none built in; its examples wrap generate() in torch.profiler,
 * examples/llama3_8b.py:61-67) ------------------------------------------------------------------------------
 * After mui_trace_enable(stream, buf, n) the calling thread's next n launches of the GEMV, gate/up, flash-decoding,
 * RoPE and all-reduce kernels each fill one record of eight uint64 words in the device buffer `buf` (n * 64 bytes,
 * filled with 0xFF by this call on `stream`). Words are %globaltimer values in ns; "~" marks words stored
 * complemented (so that one atomicMin serves minima and maxima alike):
 *   [0] first CTA start          [1] ~last CTA end
 *   [2] first CTA past its wait for the previous kernel      [3] ~last CTA with its activations staged
 *   [4] ~last CTA done pushing its partial sums to the peers  [5] ~last CTA that has seen every peer's partials
 *   [6] first CTA that has seen every peer's partials         [7] unused
 * [2]-[3] are written by the pipeline GEMV only, [4]-[6] by tensor-parallel launches only. Records are bound at
 * launch (or capture) time, so a captured graph keeps writing its records on every replay. mui_trace_enable(…, NULL,
 * 0) switches tracing off. mui_trace_count returns how many records were handed out and their kernel tags
 * (1 linear GEMV, 2 gate/up GEMV, 3 flash decoding, 4 RoPE, 5 stand-alone all-reduce). */
MUI_API mui_status_t mui_trace_enable(void* stream, void* device_buffer, int max_records);
MUI_API int mui_trace_count(int* tags_out, int max_tags);

/* ---- (a1) linear / GEMV --------------------------------------------------------------------------
 * y[b, n] = act( sum_k W[n,k] * xn[b,k] ) * mul_bias[n] + add_bias[n] + residual[b, n]
 * xn = x                                   when norm_weights == NULL
 * xn = round16(round16(x * rsqrt(mean(x^2) + eps)) * norm_weights)   otherwise (HF RMSNorm rounding)
 * W is row-major [N, K]; x [B, K]; y, residual [B, N]; 1 <= B <= 8. fp32 accumulation, one rounding.
 * Replaces muillm_linear_activ_forward_{fp16,bf16} (csrc/linear/linear.cu:40-70, kernels at
 * csrc/linear/linear_fp16_kernels.cu:164,359). */
MUI_API mui_status_t mui_linear_forward(void* stream, mui_dtype_t dtype, int B, int N, int K,
                                        const void* norm_weights, float epsilon, const void* weights,
                                        mui_activation_t activ, const void* mul_bias, const void* add_bias,
                                        const void* residual, const void* x, void* y, unsigned flags);

/* ---- (a4) fused gate/up + SiLU -------------------------------------------------------------------
 * t[b, i] = silu(sum_k G[i,k] xn[b,k]) * (sum_k U[i,k] xn[b,k]);  G,U row-major [I, H]; x [B,H]; t [B,I].
 * Replaces muillm_gateupsilu_gemv[_norm_inputs]_{fp16,bf16}_kernel launches
 * (csrc/ffn/gateup_fp16_kernels.cu:161,345,859-956). */
MUI_API mui_status_t mui_gateup_silu_forward(void* stream, mui_dtype_t dtype, int B, int I, int H,
                                             const void* norm_weights, float epsilon, const void* gate_weights,
                                             const void* up_weights, const void* x, void* t, unsigned flags);

/* Whole MLP: t = gateup_silu(x) into `scratch_t` ([B,I] elements of dtype), then
 * y = D t + residual with D row-major [H, I]. Replaces muillm_gateupsilu_forward
 * (csrc/ffn/gateup.cu:176-219). */
MUI_API mui_status_t mui_gateupdown_forward(void* stream, mui_dtype_t dtype, int B, int I, int H,
                                            const void* norm_weights, float epsilon, const void* gate_weights,
                                            const void* up_weights, const void* down_weights, const void* residual,
                                            const void* x, void* scratch_t, void* y, unsigned flags);

/* ---- prefill / batched rows (more than 8) on the tcgen05 tensor cores --------------------------------
 * Same math as mui_linear_forward (without the fused norm: normalise with mui_rmsnorm_forward first) and
 * mui_gateup_silu_forward for M rows of x [M, K] (prompt tokens): one kernel, weights streamed once per 256 rows,
 * TMA tile loads into 128-byte-swizzled shared-memory stages, tcgen05.mma with fp32 accumulators in tensor memory.
 * K % 8 == 0; weights, x 16-byte aligned. The call builds the tensor maps of its operands on the host (a few
 * microseconds). Stands where the reference falls back to at::linear for more than one token
 * (csrc/modules/linear_module.cpp:61-77, csrc/modules/parallel_linear_module.cpp:73-83). */
MUI_API mui_status_t mui_prefill_linear_forward(void* stream, mui_dtype_t dtype, int M, int N, int K,
                                                const void* weights, mui_activation_t activ, const void* mul_bias,
                                                const void* add_bias, const void* residual, const void* x, void* y,
                                                unsigned flags);
MUI_API mui_status_t mui_prefill_gateup_silu_forward(void* stream, mui_dtype_t dtype, int M, int I, int H,
                                                     const void* gate_weights, const void* up_weights, const void* x,
                                                     void* t, unsigned flags);

/* ---- (a3/a5) weight-only 8-bit GEMV and gate/up ---------------------------------------------------
 * Same math as mui_linear_forward / mui_gateup_silu_forward on de-quantised weights.
 * scales: SYM_ROW -> [N] of dtype; GROUP_MIN -> [N * (K >> group_shift), 2] of dtype (scale, min).
 * Replaces muillm_int8_linear_activ_forward (csrc/int8_linear_kernels.cu:703-784) and
 * muillm_int8_gateupsilu_forward (csrc/int8_gateup_kernels.cu:871-940). mui_gateup_silu_w8_forward takes gate and
 * up as separate [I, H] matrices with separate scale arrays; mui_gateup_silu_w8_packed_forward takes the reference's
 * own layout, the element-interleaved [I, H, 2] pack (gate, up) with [I, G, 2, 2] {scale, min} pairs
 * (muillm/modules/quantized/int8gateupdownmlp.py:211-230), and splits the bytes in registers; it returns
 * MUI_ERR_UNSUPPORTED for shapes the pipeline kernel does not serve (H % 16 != 0, groups outside 32..2048, or a
 * batch whose staged activations leave no room for two weight stages). Both formats run on the bulk-copy pipeline
 * when K % 32 == 0 (GROUP_MIN: groups of 32..2048) and the pointers are 16-byte aligned, else on the plain-load
 * kernel. */
MUI_API mui_status_t mui_linear_w8_forward(void* stream, mui_dtype_t dtype, mui_w8_format_t fmt, int group_shift,
                                           int B, int N, int K, const void* norm_weights, float epsilon,
                                           const void* qweights, const void* scales, mui_activation_t activ,
                                           const void* mul_bias, const void* add_bias, const void* residual,
                                           const void* x, void* y, unsigned flags);
MUI_API mui_status_t mui_gateup_silu_w8_forward(void* stream, mui_dtype_t dtype, mui_w8_format_t fmt,
                                                int group_shift, int B, int I, int H, const void* norm_weights,
                                                float epsilon, const void* gate_q, const void* gate_scales,
                                                const void* up_q, const void* up_scales, const void* x, void* t,
                                                unsigned flags);
MUI_API mui_status_t mui_gateup_silu_w8_packed_forward(void* stream, mui_dtype_t dtype, int group_shift, int B, int I,
                                                       int H, const void* norm_weights, float epsilon,
                                                       const void* gate_up_q, const void* gate_up_scales_min,
                                                       const void* x, void* t, unsigned flags);
/* Full de-quantisation to [N,K] of dtype (batched fallback of the reference,
 * csrc/int8_dequantization_kernel.cu:74). */
MUI_API mui_status_t mui_w8_dequantize(void* stream, mui_dtype_t dtype, mui_w8_format_t fmt, int group_shift, int N,
                                       int K, const void* qweights, const void* scales, void* out);

/* ---- (a14) RMSNorm / L2 norm ----------------------------------------------------------------------
 * y[r,:] = round16(round16(x[r,:] * rsqrt(mean(x[r,:]^2) + eps)) * w) ; w == NULL -> no weight (L2 norm of
 * Llama-4, csrc/norm/l2norm_fp16_kernels.cu:35). Replaces muillm_rmsnorm_forward (csrc/norm/rmsnorm.cu:31-84). */
MUI_API mui_status_t mui_rmsnorm_forward(void* stream, mui_dtype_t dtype, int rows, int K, const void* w,
                                         float epsilon, const void* x, void* y, unsigned flags);

/* ---- (a8) rotary embedding + static-cache write-out ----------------------------------------------
 * q_out[b,h,t,:] = rope(q_in[b,h,t,:]);  K[b,h,cache_position[t],:] = rope(k_in[b,h,t,:]);
 * V[b,h,cache_position[t],:] = v_in[b,h,t,:].  rope(x) = x*cos + rotate_half(x)*sin evaluated in fp32 and
 * rounded once. q/k/v are [B,H*,T,D] views given by element strides (innermost stride 1); caches are
 * contiguous [B,Hkv,MAX_T,D]; cos/sin tables are [S, D] indexed by position_ids[b,t] (layout 0) or
 * [B,T,D] indexed by (b,t) (layout 1); position_ids [B,T] and cache_position [T] are int64.
 * k_cache/v_cache may be NULL (no cache: k_out receives rope(k), contiguous [B,Hkv,T,D]).
 * Replaces muillm_apply_rope_forward_{fp16,bf16}_static_cache / _no_cache
 * (csrc/rope/rotary.cu:603-756, csrc/rope/rotary_fp16_kernels.cu:95,575). */
typedef struct mui_strides3 { int64_t batch, head, tok; } mui_strides3_t;
MUI_API mui_status_t mui_rope_forward(void* stream, mui_dtype_t dtype, int B, int T, int max_T, int Hq, int Hkv,
                                      int D, int table_layout, const int64_t* position_ids, const void* cos_table,
                                      const void* sin_table, const void* q_in, mui_strides3_t q_strides,
                                      const void* k_in, mui_strides3_t k_strides, const void* v_in,
                                      mui_strides3_t v_strides, void* q_out, void* k_out, void* k_cache,
                                      void* v_cache, const int64_t* cache_position, unsigned flags);

/* Static-cache scatter only (csrc/kvcaches/static_kvcache.cpp:35-120). */
MUI_API mui_status_t mui_static_kvcache_update(void* stream, mui_dtype_t dtype, int B, int T, int max_T, int Hkv,
                                               int D, const void* k_in, mui_strides3_t k_strides, const void* v_in,
                                               mui_strides3_t v_strides, void* k_cache, void* v_cache,
                                               const int64_t* cache_position, unsigned flags);

/* ---- (a10) flash decoding -------------------------------------------------------------------------
 * out[b, 0, h*D:(h+1)*D] = softmax_s( q[b,h,:]·K[b,h/(Hq/Hkv),s,:] * scale + mask[b,s] ) · V[b,..,s,:]
 * for one query token. q contiguous [B,Hq,1,D]; K,V given by element strides (batch, head, token;
 * innermost 1); out contiguous [B,1,Hq*D]. S tokens are attended; when seq_len_dev != NULL the device
 * int32 it points to replaces S at run time (must be <= S; makes the launch replayable in a CUDA graph).
 * mask: NULL or additive [B,S] of dtype, a position is kept iff its mask value == 0
 * (csrc/attention/flash_decoding_fp16_kernels.cu:386-393). Split-KV with fp32 (m, l, acc) partials in
 * `workspace` (mui_flash_decode_workspace_bytes bytes, 256-byte aligned). The first 4 KiB of the
 * workspace hold arrival counters that must be zero before the first call; every call leaves them zero.
 * Replaces flash_decode_no_mask / flash_decode_masked (csrc/attention/flash_decoding.cu:288-325). */
MUI_API size_t mui_flash_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_S);
MUI_API mui_status_t mui_flash_decode(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D, int S,
                                      const int32_t* seq_len_dev, float scale, const void* q, const void* k,
                                      const void* v, mui_strides3_t kv_strides, const void* mask, void* out,
                                      void* workspace, size_t workspace_bytes, unsigned flags);

/* Fused decode attention: RoPE on q and on the new k, write of rope(k) and v into the static caches at
 * cache_position, and attention of the one new token over the S = *seq_len_dev cached-plus-new tokens, in ONE launch
 * (thread-block cluster of 8 CTAs per (KV head, sequence), partials merged through distributed shared memory: no
 * global scratch). qkv is the packed output of the QKV projection [B, (Hq + 2*Hkv) * D] (q rows, then k, then v);
 * position_ids [B] (int64, RoPE position per sequence), cache_position [1] (int64, row written) and seq_len_dev
 * (int32) live on the device; out is [B, Hq * D]. D == 128, Hq / Hkv <= 8. cos/sin tables hold at least max_seq
 * rows; a cache_position or position id outside [0, max_seq) records MUI_DEV_BAD_LENGTH in the device status word
 * and the launch writes nothing (a replayed graph cannot run past the cache). Replaces the pair
 * muillm_rope_forward_static_cache + flash_decode_no_mask on the decode path (csrc/rope/rotary.cu:603-756,
 * csrc/attention/flash_decoding.cu:288-305; MuiLLMParallelAttention::forward chains them,
 * csrc/modules/parallel_attention_module.cpp:45-90). */
MUI_API mui_status_t mui_rope_flash_decode(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D, int max_seq,
                                           const void* qkv, const void* cos_table, const void* sin_table,
                                           const int64_t* position_ids, const int64_t* cache_position,
                                           const int32_t* seq_len_dev, float scale, void* k_cache, void* v_cache,
                                           void* out, unsigned flags);

/* mui_rope_flash_decode with a workspace (mui_flash_decode_workspace_bytes bytes, first 4 KiB zero before the first
 * call) and an upper bound `max_attended` of the tokens the launch (or every replay of it in a CUDA graph) will
 * attend. With MUI_FLAG_SPLIT_CONTEXT the tokens are split over ceil(max_attended / 256) CTAs per (KV head, sequence)
 * (at most 64, i.e. 16384 tokens; beyond that the cluster kernel runs): each stages its tokens in shared memory and
 * runs QK^T and PV on the tensor cores, the last one to arrive merges the partial (max, denominator, output) triples
 * by log-sum-exp. For a few thousand tokens this is three to four times faster than the cluster kernel, which keeps
 * one cluster per KV head whatever the length. */
MUI_API mui_status_t mui_rope_flash_decode_ws(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D,
                                              int max_seq, const void* qkv, const void* cos_table,
                                              const void* sin_table, const int64_t* position_ids,
                                              const int64_t* cache_position, const int32_t* seq_len_dev, float scale,
                                              void* k_cache, void* v_cache, void* out, void* workspace,
                                              size_t workspace_bytes, int max_attended, unsigned flags);

/* The same fused launch for a Llama-4 attention layer: instead of the rotate-half RoPE, q and the new k go through
 * the Llama-4 prologue — interleaved-pair rotation by freqs[position] ([max_pos, D/2, 2] fp32 (cos, sin); use_rope),
 * L2 norm over the head dim (use_qk_norm, norm_eps), and for q the temperature scale
 * log1p(floor((cache_position + 1) / floor_scale)) * attn_scale + 1 (temperature_tuning) — each stage rounded to the
 * 16-bit type exactly like mui_llama4_qk_prologue; then the new row is written and the token attends. With chunk > 0
 * the layer's caches [B, Hkv, cache_rows, D] are a ring indexed by cache_position % chunk and the token attends the
 * rows of its own chunk, rows 0 .. cache_position % chunk (chunked attention; cache_rows >= min(chunk, longest
 * sequence)); with chunk == 0 the cache is plain and rows 0 .. cache_position are attended. cache_position [1] is the
 * absolute position of the new token. D == 128, Hq / Hkv <= 8. workspace / workspace_bytes / max_attended as in
 * mui_rope_flash_decode_ws (workspace may be NULL without MUI_FLAG_SPLIT_CONTEXT). One launch where the reference's
 * MuiLLMParallelLlama4Attention::forward chains rope, QK norm, temperature tuning, the hybrid chunked cache update and
 * flash decoding (csrc/modules/parallel_llama4_attention_module.cpp:66-147,
 * csrc/modules/hybrid_chunked_kvcache.cpp:23-77). */
MUI_API mui_status_t mui_llama4_rope_flash_decode(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D,
                                                  int cache_rows, int max_pos, const void* qkv, const float* freqs,
                                                  const int64_t* position_ids, const int64_t* cache_position,
                                                  int use_rope, int use_qk_norm, float norm_eps,
                                                  int temperature_tuning, float attn_scale, float floor_scale,
                                                  int chunk, float scale, void* k_cache, void* v_cache, void* out,
                                                  void* workspace, size_t workspace_bytes, int max_attended,
                                                  unsigned flags);

/* Flash decoding for callers that may not allocate device memory. No counterpart in the reference (there,
 * torch allocates the partial buffers on every call, csrc/attention/flash_decoding.cu:154-158). Meant for hosts
 * that pass this library nothing but input and output buffers because all device memory is already carved up by
 * their own arena, and for loops that must not reach cudaMalloc since it synchronises the whole device. Same
 * arguments and results as mui_flash_decode minus the workspace: the split-KV partials and arrival counters live
 * in a static __device__ array inside the library (about 2.04 MiB that every GPU loading the library holds until
 * the process exits), which limits the problem to B * Hq * (D + 2) <= MUI_FD_STATIC_MAX_ROW_FLOATS (e.g. 64 heads
 * of head dim 128 in total); larger problems are rejected with MUI_ERR_UNSUPPORTED. It calls no cudaMalloc,
 * cudaFree or other allocating routine. The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and clears the counters on `stream`; make that first call
 * outside any stream capture. All calls share the one array and it keeps the previous call's partials, so two
 * calls that overlap on the GPU (different streams, or different threads on one device) race; calls ordered on
 * one stream are safe. */
#define MUI_FD_STATIC_MAX_ROW_FLOATS (64 * 130)
MUI_API mui_status_t mui_flash_decode_static_scratch(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D,
                                                     int S, const int32_t* seq_len_dev, float scale, const void* q,
                                                     const void* k, const void* v, mui_strides3_t kv_strides,
                                                     const void* mask, void* out, unsigned flags);

/* ---- (a15) Llama-4 attention prologue, windowed cache, small bookkeeping ops ------------------------
 * q/k are [B,H,T,D] views given by element strides (innermost stride 1, D even, D <= 256); outputs are contiguous
 * [B,H,T,D]. Every stage computes in fp32 and rounds once to dtype.
 *
 * mui_complex_rope_forward: (x[2i] + j·x[2i+1]) · (cos_i + j·sin_i) with position_embeds fp32 [B,T,D/2,2].
 *   Replaces muillm_complex_rope_forward_no_cache (csrc/rope/rotary.cu:798-915).
 * mui_qkl2norm_forward: x · rsqrt(mean(x²) + eps) on rows_q rows of q and rows_k rows of k (contiguous rows of D).
 *   Replaces muillm_qkl2norm_forward (csrc/norm/qkl2norm.cu:38-100); with rows_k = 0 also muillm_l2norm_forward
 *   for rows of at most 256 elements. eps is added to the mean (HF Llama4TextL2Norm), not to the sum as the
 *   reference kernel does (csrc/norm/qkl2norm_fp16_kernels.cu:66,117).
 * mui_temperature_tuning_forward: q · (log1p(floor((cache_position[t] + 1) / floor_scale)) · attn_scale + 1).
 *   Replaces muillm_apply_temperature_tuning (csrc/temperaturetuning/temperature_tuning.cu).
 * mui_llama4_qk_prologue: the three above in one launch, in that order; a stage is skipped when its input is
 *   absent (position_embeds NULL: no rope; use_qk_norm 0: no norm; cache_position NULL: no temperature scale, which
 *   applies to q only). Bit-identical to the three separate calls. */
MUI_API mui_status_t mui_complex_rope_forward(void* stream, mui_dtype_t dtype, int B, int T, int Hq, int Hk, int D,
                                              const float* position_embeds, const void* q_in,
                                              mui_strides3_t q_strides, const void* k_in, mui_strides3_t k_strides,
                                              void* q_out, void* k_out, unsigned flags);
MUI_API mui_status_t mui_qkl2norm_forward(void* stream, mui_dtype_t dtype, long long rows_q, long long rows_k, int D,
                                          const void* q, const void* k, void* q_out, void* k_out, float eps,
                                          unsigned flags);
MUI_API mui_status_t mui_temperature_tuning_forward(void* stream, mui_dtype_t dtype, int B, int T, int H, int D,
                                                    const void* q_in, mui_strides3_t q_strides,
                                                    const int64_t* cache_position, void* q_out, float attn_scale,
                                                    float floor_scale, unsigned flags);
MUI_API mui_status_t mui_llama4_qk_prologue(void* stream, mui_dtype_t dtype, int B, int T, int Hq, int Hk, int D,
                                            const float* position_embeds, int use_qk_norm, float norm_eps,
                                            const int64_t* cache_position, float attn_scale, float floor_scale,
                                            const void* q_in, mui_strides3_t q_strides, const void* k_in,
                                            mui_strides3_t k_strides, void* q_out, void* k_out, unsigned flags);

/* Sliding-window cache update, rows kept in chronological order (csrc/kvcaches/sliding_kvcache.cpp:87-246).
 * seen_tokens counts the T new tokens. *mode_out (host int, may be NULL) tells what happened:
 *   0  seen_tokens == T: first fill; the last min(T, max_T) new rows go to cache rows 0..; attend k_in / v_in.
 *   1  seen_tokens > max_T: the window is full; k_cache_out / v_cache_out (second buffers, required) receive the
 *      old rows shifted down by min(T, max_T) followed by the new rows; attend all max_T rows of the new buffers.
 *   2  otherwise: new rows are scattered in place at cache_position[t]; attend the first seen_tokens rows. */
MUI_API mui_status_t mui_sliding_kvcache_update(void* stream, mui_dtype_t dtype, int B, int T, int max_T, int Hk,
                                                int Hv, int D, const void* k_in, mui_strides3_t k_strides,
                                                const void* v_in, mui_strides3_t v_strides, void* k_cache,
                                                void* v_cache, void* k_cache_out, void* v_cache_out,
                                                const int64_t* cache_position, long long seen_tokens, int* mode_out,
                                                unsigned flags);

/* y[b, n] = sum_m x[b, m, n], fp32 accumulation (N == 1 sums the last dimension of [B, M]).
 * Replaces muillm_reduce_sum_forward (csrc/reduce/reduce.cu:33-108). */
MUI_API mui_status_t mui_reduce_sum_forward(void* stream, mui_dtype_t dtype, long long B, int M, long long N,
                                            const void* x, void* y, unsigned flags);

/* One step of a generation loop's bookkeeping: next_input_ids [B,T+1] = input_ids [B,T] with the next token
 * appended (pad_token_id for sequences already finished when the eos criterion is on); next_unfinished[b] =
 * unfinished[b] and not (token is one of eos_token_ids) and not (T + 1 >= max_length), each criterion only if
 * enabled. next_tokens is int32, the rest int64. Follows the generation loop of HF `GenerationMixin._sample`
 * that the reference's muillm_add_tokens_check_finished fuses (csrc/generation/generation.cu:30-213); the
 * reference kernel's extra store to next_input_ids[b] and its `T <= max_length` test are not reproduced. */
MUI_API mui_status_t mui_add_tokens_check_finished(void* stream, int B, int T, const int64_t* input_ids,
                                                   const int32_t* next_tokens, const int64_t* unfinished_sequences,
                                                   int has_eos_stopping_criteria, long long pad_token_id,
                                                   const int64_t* eos_token_ids, int num_eos_tokens,
                                                   int has_max_length_stopping_criteria, long long max_length,
                                                   int64_t* next_input_ids, int64_t* next_unfinished_sequences,
                                                   unsigned flags);

/* ---- (a6) router top-k + sigmoid -------------------------------------------------------------------
 * For each of `rows` rows of logits [rows, M] (M <= 4096): the k largest values (ties -> lowest index, as a
 * stable descending sort orders them), sigmoid in fp32, rounded to dtype; indices int64.
 * Replaces muillm_topk_sigmoid_forward (csrc/topk/topk.cu:34-93). */
MUI_API mui_status_t mui_topk_sigmoid_forward(void* stream, mui_dtype_t dtype, int rows, int M, int k,
                                              const void* logits, void* values, int64_t* indices, unsigned flags);
/* Router of one token in one launch: logits[e] = router_weights[e, :] . rmsnorm(x) (E x H weights, fused norm as in
 * mui_linear_forward, each logit rounded to the 16-bit type), then the top k of them with their sigmoid, as
 * mui_topk_sigmoid_forward gives. logits_scratch: E floats; counter: one zero-initialised uint32 that every call
 * leaves at zero. E <= 1024. Replaces the router GEMV + muillm_topk_sigmoid_forward pair of
 * MuiLLMParallelGateUpDownMLPMoE::forward (csrc/modules/parallel_gateupmoe_module.cpp:45-77). */
MUI_API mui_status_t mui_router_topk_sigmoid_forward(void* stream, mui_dtype_t dtype, int E, int H, int k,
                                                     const void* norm_weights, float epsilon,
                                                     const void* router_weights, const void* x, float* logits_scratch,
                                                     unsigned int* counter, void* values, int64_t* indices,
                                                     unsigned flags);

/* ---- (a7) MoE MLP for one token -------------------------------------------------------------------
 * Computed experts = the num_shared shared ones (score 1) followed by the top_k routed ones named by
 * router_indices[top_k] (int64, device; expert e of the routed set uses rows num_shared + e of the packs) with
 * router_scores[top_k] (dtype, device). gate/up packs are [(num_shared + num_routed) * I, H], the down pack is
 * [(num_shared + num_routed) * H, I].
 *   t[s, :] = silu(score_s * G_e xn) * (score_s * U_e xn)        (the score scales the pre-activations,
 *                                                                  csrc/moeffn/gateupmoe_fp16_kernels.cu:355-360)
 *   y = sum_s D_e t[s, :] + residual                              (summed inside the down kernel in fp32; the
 *                                                                  reference writes per-expert rows and reduces,
 *                                                                  csrc/moeffn/moelinear_fp16_kernels.cu:363-375,
 *                                                                  csrc/reduce/reduce_fp16_kernels.cu:32)
 * t is [num_shared + top_k, I] of dtype. mui_moe_down_forward can also leave fp32 sums in y_f32 (tensor-parallel
 * partials). Replaces muillm_gateupsilumoe_forward (csrc/moeffn/gateupmoe.cu:115-290). */
MUI_API mui_status_t mui_moe_gateup_silu_forward(void* stream, mui_dtype_t dtype, int num_shared, int num_routed,
                                                 int top_k, int I, int H, const void* norm_weights, float epsilon,
                                                 const void* gate_weights, const void* up_weights, const void* x,
                                                 const void* router_scores, const int64_t* router_indices, void* t,
                                                 unsigned flags);
MUI_API mui_status_t mui_moe_down_forward(void* stream, mui_dtype_t dtype, int num_shared, int num_routed, int top_k,
                                          int H, int I, const void* down_weights, const void* residual,
                                          const void* t, const int64_t* router_indices, void* y, float* y_f32,
                                          unsigned flags);
MUI_API mui_status_t mui_moe_mlp_forward(void* stream, mui_dtype_t dtype, int num_shared, int num_routed, int top_k,
                                         int I, int H, const void* norm_weights, float epsilon,
                                         const void* gate_weights, const void* up_weights, const void* down_weights,
                                         const void* residual, const void* x, const void* router_scores,
                                         const int64_t* router_indices, void* scratch_t, void* y, unsigned flags);

/* ---- (a11/a12) tensor-parallel communicator, one node, one process per GPU ------------------------------
 * Stands in for muillm_comm_* (csrc/comms/comm.h:12-56, csrc/comms/comm_p2p.cu). Each rank owns a device segment
 * (allocated by mui_comm_create with cudaMalloc — the only allocation in this library besides the static
 * scratch above) of 2 generations x world slots x capacity fp32 elements plus per-rank flags; peers map it with
 * CUDA IPC. Collectives are one-shot: every rank stores its fp32 partials into its slot of every rank's segment
 * over NVLink, publishes a flag, waits (bounded, 2 s) for all flags and sums the slots of its own segment in rank
 * order — bit-identical results on all ranks, one rounding. All ranks must issue collectives in the same order
 * (one host thread per rank), like the reference (csrc/comms/comm_p2p.cu:178-184,1033-1035).
 * mui_comm_init_local = create + handle exchange over a UNIX socket in /tmp keyed by `key` (rank 0 listens; every
 * socket wait is bounded by timeout_s, default 60) + open. The three-step form lets the caller move the 64-byte
 * handles over any transport it has (e.g. torch.distributed). */
typedef struct mui_comm mui_comm_t;
#define MUI_COMM_F32 2 /* dtype code of fp32 payloads for mui_comm_all_reduce_sum (besides MUI_F16 / MUI_BF16) */
MUI_API mui_status_t mui_bootstrap_allgather(int rank, int world, const char* key, const void* blob,
                                             size_t blob_bytes, void* out, double timeout_s);
MUI_API size_t mui_comm_ipc_handle_bytes(void);
MUI_API mui_status_t mui_comm_create(int rank, int world, size_t capacity_elems, mui_comm_t** out);
MUI_API mui_status_t mui_comm_ipc_handle(mui_comm_t* comm, void* handle_out);
MUI_API mui_status_t mui_comm_open_peers(mui_comm_t* comm, const void* handles /* world x handle bytes */);
MUI_API mui_status_t mui_comm_init_local(int rank, int world, const char* key, size_t capacity_elems,
                                         double timeout_s, mui_comm_t** out);
MUI_API mui_status_t mui_comm_destroy(mui_comm_t* comm);
MUI_API mui_status_t mui_comm_info(mui_comm_t* comm, int* rank, int* world, size_t* capacity_elems);
/* dst = sum over ranks of src, `count` elements of dtype (MUI_F16, MUI_BF16 or MUI_COMM_F32); in place allowed.
 * Replaces muillm_comm_all_reduce_sum (csrc/comms/comm_p2p.cu:1494-1526). */
MUI_API mui_status_t mui_comm_all_reduce_sum(mui_comm_t* comm, void* stream, int dtype, const void* src, void* dst,
                                             size_t count, unsigned flags);
/* dst (all ranks) = src of rank `root`; bytes a multiple of 4. Replaces muillm_comm_broadcast
 * (csrc/comms/comm_p2p.cu:1571-1615). */
MUI_API mui_status_t mui_comm_broadcast(mui_comm_t* comm, void* stream, int root, const void* src, void* dst,
                                        size_t bytes, unsigned flags);
/* K-sharded linear with the all-reduce fused into the GEMV kernel: every rank multiplies its [N, K_local] weight
 * shard with its slice of x, pushes the fp32 partial rows straight from the GEMV epilogue into all ranks' slots,
 * and the same kernel's tail reduces them into y [B, N] (identical on all ranks). mul_bias applies to every
 * partial; add_bias and residual enter once, on rank 0 (csrc/parallel_linear_kernels.cu:131-133). Replaces
 * muillm_parallel_linear_activ_forward with sharding_dim == 1 (csrc/parallel_linear_kernels.cu:50-173). */
MUI_API mui_status_t mui_parallel_linear_forward(mui_comm_t* comm, void* stream, mui_dtype_t dtype, int B, int N,
                                                 int K_local, const void* norm_weights, float epsilon,
                                                 const void* weights, const void* mul_bias, const void* add_bias,
                                                 const void* residual, const void* x, void* y, unsigned flags);
/* Sharded MLP: gate/up row-sharded [I_local, H] (no collective), down K-sharded [H, I_local] + fused all-reduce.
 * Replaces muillm_parallel_gateupsilu_forward (csrc/parallel_gateup_kernels.cu:6-112). */
MUI_API mui_status_t mui_parallel_gateupdown_forward(mui_comm_t* comm, void* stream, mui_dtype_t dtype, int B,
                                                     int I_local, int H, const void* norm_weights, float epsilon,
                                                     const void* gate_weights, const void* up_weights,
                                                     const void* down_weights, const void* residual, const void* x,
                                                     void* scratch_t, void* y, unsigned flags);

/* Sharded MoE MLP: every expert's gate/up rows and down columns are split across ranks ([(shared + routed)·I_local, H]
 * and [(shared + routed)·H, I_local]); the router outputs are replicated. Gate/up is local; the down kernel sums the
 * computed experts and all-reduces across ranks in the same launch; the residual enters on rank 0. scratch_t holds
 * [num_shared + top_k, I_local] elements. Replaces muillm_parallel_gateupsilumoe_forward
 * (csrc/parallel_gateupmoe_kernels.cu:6-125). */
MUI_API mui_status_t mui_parallel_moe_mlp_forward(mui_comm_t* comm, void* stream, mui_dtype_t dtype, int num_shared,
                                                  int num_routed, int top_k, int I_local, int H,
                                                  const void* norm_weights, float epsilon, const void* gate_weights,
                                                  const void* up_weights, const void* down_weights,
                                                  const void* residual, const void* x, const void* router_scores,
                                                  const int64_t* router_indices, void* scratch_t, void* y,
                                                  unsigned flags);

/* ---- embedding row gather (csrc/embedding/embedding_xx16_kernels.cu:26,74) ------------------------
 * out[i, :] = table[token_ids[i], :] for 16-bit tables [vocab, H]; token ids are int64 on the device and
 * are clamped to [0, vocab). */
MUI_API mui_status_t mui_embedding_forward(void* stream, mui_dtype_t dtype, int num_tokens, int H, int vocab,
                                           const void* table, const int64_t* token_ids, void* out, unsigned flags);

/* ---- decode stack ----------------------------------------------------------------------------------
 * One call launches every kernel of a decode step of a Llama-architecture model for `batch` sequences:
 * embedding, per layer {fused-norm QKV GEMV, RoPE + static-cache write, flash decoding, o_proj + residual,
 * fused-norm gate/up + SiLU, down + residual}, final-norm lm_head GEMV, greedy arg-max. The step's token,
 * position ids, cache position and attended length live in device memory and are advanced by the step
 * itself, so consecutive steps need no host round trip and a step can be captured once in a CUDA graph
 * and replayed. The reference has this level for tensor-parallel runs only
 * (MuiLLMParallelDecoderStack::forward, csrc/modules/parallel_decoder_stack.cpp:22-45); its single-GPU
 * decode returns to Python between layers (muillm/modules/decoder/decoder.py:95-165).
 * All device memory is caller-owned: weights, per-layer KV caches [batch, kv_heads, max_seq, head_dim],
 * cos/sin tables [max_seq, head_dim] and one scratch block of mui_llama_stack_scratch_bytes() bytes
 * (256-byte aligned). create/destroy only manage a small host object (and the captured graph). */
typedef struct mui_llama_config {
  mui_dtype_t dtype;
  int layers, hidden, intermediate, heads, kv_heads, head_dim, vocab;
  int max_seq;      /* static KV-cache length */
  int batch;        /* 1..8 sequences decoded together */
  float rms_eps;
  float attn_scale; /* softmax scale, normally 1/sqrt(head_dim) */
  /* Tensor parallelism (both 0 on one GPU): heads, kv_heads, intermediate and vocab above are then this rank's
   * shard sizes; embed_vocab = rows of the (replicated) embedding table; vocab_offset = first token id of this
   * rank's lm_head rows. */
  int embed_vocab;
  int vocab_offset;
} mui_llama_config_t;

typedef struct mui_llama_weights {
  const void* embed;            /* [vocab, hidden] */
  const void* final_norm;       /* [hidden] */
  const void* lm_head;          /* [vocab, hidden] */
  const void* cos_table;        /* [max_seq, head_dim] */
  const void* sin_table;        /* [max_seq, head_dim] */
  const void* const* qkv;       /* per layer [(heads + 2*kv_heads)*head_dim, hidden]: q rows, then k, then v */
  const void* const* o;         /* per layer [hidden, heads*head_dim] */
  const void* const* gate;      /* per layer [intermediate, hidden] */
  const void* const* up;        /* per layer [intermediate, hidden] */
  const void* const* down;      /* per layer [hidden, intermediate] */
  const void* const* ln1;       /* per layer input RMSNorm weight [hidden] */
  const void* const* ln2;       /* per layer post-attention RMSNorm weight [hidden] */
  void* const* k_cache;         /* per layer [batch, kv_heads, max_seq, head_dim] */
  void* const* v_cache;
} mui_llama_weights_t;

typedef struct mui_llama_stack mui_llama_stack_t;

MUI_API size_t mui_llama_stack_scratch_bytes(const mui_llama_config_t* cfg);
MUI_API mui_status_t mui_llama_stack_create(const mui_llama_config_t* cfg, const mui_llama_weights_t* weights,
                                            void* scratch, size_t scratch_bytes, mui_llama_stack_t** out);
MUI_API mui_status_t mui_llama_stack_destroy(mui_llama_stack_t* stack);
/* The same decode stack for a Llama-4 text model, batch 1: per layer {fused-norm QKV GEMV, the fused Llama-4
 * attention launch (mui_llama4_rope_flash_decode; layers with use_rope[l] != 0 are chunked-attention layers with rope
 * and, if use_qk_norm, the QK L2 norm, the others attend everything and get the temperature scale if
 * temperature_tuning), o_proj + residual, router + top-k sigmoid, gate/up + SiLU of the shared and the selected
 * experts, expert down projections summed + residual}: six launches per layer, where the reference's
 * MuiLLMParallelLlama4DecoderStack chains about a dozen (csrc/modules/parallel_llama4_decoder_stack.cpp:18-60,
 * parallel_llama4_decoder_module.cpp:25-66). Rope layers keep ring caches of min(max_seq, chunk) rows, the others
 * plain caches of max_seq rows (the hybrid chunked cache, csrc/modules/hybrid_chunked_kvcache.cpp:23-77). Expert
 * weights are packed shared-first: gate/up [(num_shared + num_experts) * expert_intermediate, hidden], down
 * [(num_shared + num_experts) * hidden, expert_intermediate]. Head dims other than 128 run the prologue, the cache
 * write and flash decoding as separate launches. The handle is a mui_llama_stack_t: reset, set_tokens, step,
 * capture, replay, logits, set_comm (expert intermediate, heads and lm_head rows sharded; router replicated) and
 * destroy are the functions below and above. */
typedef struct mui_llama4_config {
  mui_dtype_t dtype;
  int layers, hidden, expert_intermediate, heads, kv_heads, head_dim, vocab;
  int max_seq;             /* longest sequence: rows of the full-attention caches and of the rotary table */
  int chunk;               /* attention chunk of the rope layers; 0 = they attend everything too */
  int num_experts, top_k, num_shared;
  float rms_eps;
  float softmax_scale;     /* normally 1/sqrt(head_dim) */
  int use_qk_norm, temperature_tuning;
  float attn_scale, floor_scale;
  int embed_vocab, vocab_offset; /* tensor parallelism, as in mui_llama_config_t */
} mui_llama4_config_t;

typedef struct mui_llama4_weights {
  const void* embed;
  const void* final_norm;
  const void* lm_head;
  const float* freqs;           /* [max_seq, head_dim/2, 2] fp32 (cos, sin) of the interleaved rotation */
  const int* use_rope;          /* host array [layers] */
  const void* const* qkv;
  const void* const* o;
  const void* const* router;    /* per layer [num_experts, hidden] */
  const void* const* gate;
  const void* const* up;
  const void* const* down;
  const void* const* ln1;
  const void* const* ln2;
  void* const* k_cache;         /* per layer [1, kv_heads, rows, head_dim], rows = mui_llama4_stack_cache_rows() */
  void* const* v_cache;
} mui_llama4_weights_t;

MUI_API int mui_llama4_stack_cache_rows(const mui_llama4_config_t* cfg, int use_rope);
MUI_API size_t mui_llama4_stack_scratch_bytes(const mui_llama4_config_t* cfg);
MUI_API mui_status_t mui_llama4_stack_create(const mui_llama4_config_t* cfg, const mui_llama4_weights_t* weights,
                                             void* scratch, size_t scratch_bytes, mui_llama_stack_t** out);
/* Device pointers of the last step's router outputs: logits [layers, num_experts] (fp32, rounded to the model
 * dtype) and the chosen experts [layers, 8] (int64, the first top_k of each row). Routing is the one discontinuous
 * step of the model; two runs whose tokens differ can be compared layer by layer with these. */
MUI_API mui_status_t mui_llama4_stack_router_state(mui_llama_stack_t* stack, float** logits_dev,
                                                   int64_t** indices_dev);
/* Tensor-parallel decode: with a communicator of world > 1 attached, the weights are this rank's shards — QKV and
 * gate/up by output rows (whole heads per rank), o_proj and down by input columns with the all-reduce fused into
 * their GEMV (residual on rank 0), lm_head by rows with the arg-max finished by exchanging each rank's best
 * (value, token) pair — the sharding of muillm/modules/parallelmultilinear.py:323-387,
 * parallelgateupdownmlp.py:88-117, except the lm_head, which the reference shards by columns and all-reduces
 * (muillm/modules/models/llama/model.py:655-664). All ranks must step together. */
MUI_API mui_status_t mui_llama_stack_set_comm(mui_llama_stack_t* stack, mui_comm_t* comm);
/* Sets the device-side state: `position` tokens are already in the cache (the next step writes row `position`),
 * per-sequence RoPE positions (host array of `batch` int64, NULL = position for all), and the device buffer
 * [out_capacity, batch] int64 that receives each step's arg-max token (may be NULL). Drops a captured graph. */
MUI_API mui_status_t mui_llama_stack_reset(mui_llama_stack_t* stack, void* stream, int position,
                                           const int64_t* position_ids_host, int64_t* out_tokens_dev,
                                           int out_capacity);
/* Token ids (int64, `batch` of them) fed to the next step; host or device pointer. */
MUI_API mui_status_t mui_llama_stack_set_tokens(mui_llama_stack_t* stack, void* stream, const int64_t* tokens,
                                                int on_device);
/* Batches of sequences with different lengths, left-padded to a common length the way the reference's generation
 * loop receives them from the HF tokenizer (attention_mask + position_ids, muillm/modules/models/llama/model.py:437-615,
 * masked attention csrc/attention/flash_decoding.cu:307-325): all sequences share the cache row and the attended
 * length, every sequence has its own RoPE position, and `mask_dev` ([batch, max_seq] of the model dtype, additive:
 * 0 keeps a cache row, anything else drops it, e.g. the rows of a sequence's padding) is applied by every layer's
 * attention. With a mask set, a step runs RoPE + cache write and masked split-KV flash decoding as two launches
 * instead of the fused attention kernel. NULL clears the mask. Changing the mask drops a captured graph; its
 * CONTENTS may change between replays. mui_llama_stack_set_position_ids overwrites the per-sequence positions the
 * next step uses (host or device array of `batch` int64); every step then advances them by one. */
MUI_API mui_status_t mui_llama_stack_set_attention_mask(mui_llama_stack_t* stack, const void* mask_dev);
MUI_API mui_status_t mui_llama_stack_set_position_ids(mui_llama_stack_t* stack, void* stream,
                                                      const int64_t* position_ids, int on_device);
MUI_API mui_status_t mui_llama_stack_step(mui_llama_stack_t* stack, void* stream, unsigned flags);
/* Captures one step on `stream` (must not be the default stream) into a graph; replay launches it `steps` times. */
MUI_API mui_status_t mui_llama_stack_capture(mui_llama_stack_t* stack, void* stream, unsigned flags);
MUI_API mui_status_t mui_llama_stack_replay(mui_llama_stack_t* stack, void* stream, int steps);
/* The decoder layers only, for callers that keep the final norm, lm_head and sampling outside — what the reference's
 * MuiLLMParallelDecoderStack::forward does for one new token (csrc/modules/parallel_decoder_stack.cpp:22-45): from
 * token ids [batch] (embedding lookup) or from hidden states h_in [batch, hidden], with RoPE positions
 * position_ids [batch] and the cache row cache_position [1] (int64, device); the new token attends
 * cache_position + 1 rows, which the caller also passes as the host integer seen_tokens (it picks the attention
 * variant). h_out [batch, hidden] receives the last layer's output. The device-side decode state of the stack is
 * overwritten; a captured graph of mui_llama_stack_step is unaffected. */
MUI_API mui_status_t mui_llama_stack_forward_hidden(mui_llama_stack_t* stack, void* stream,
                                                    const int64_t* token_ids_dev, const void* h_in,
                                                    const int64_t* position_ids_dev,
                                                    const int64_t* cache_position_dev, int seen_tokens, void* h_out,
                                                    unsigned flags);
/* Device pointers of the last step's logits [batch, vocab] (dtype) and of the int64 state words
 * {step, tokens in cache, cache position, position_ids[batch], next tokens[batch]}. */
MUI_API mui_status_t mui_llama_stack_logits(mui_llama_stack_t* stack, void** logits_dev, int64_t** state_dev);

#ifdef __cplusplus
}
#endif
#endif /* MUILLM_B200_H_ */
