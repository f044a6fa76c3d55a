// Llama-architecture decode stack: one call launches every kernel of a decode step (embedding, per layer
// fused-norm QKV GEMV -> RoPE + cache write -> flash decoding -> o_proj + residual -> fused-norm gate/up
// + SiLU -> down + residual, then final-norm lm_head GEMV and greedy arg-max). Positions, sequence length
// and the token fed to the next step live in device memory, so a step is replayable from a CUDA graph
// and consecutive steps need no host round trip. Host-side C++ only; all kernels are reached through
// the same entry points the C ABI exports.
//
// The reference has this level only for tensor-parallel runs (MuiLLMParallelDecoderStack::forward,
// csrc/modules/parallel_decoder_stack.cpp:22-45, MuiLLMParallelDecoder::forward,
// csrc/modules/parallel_decoder_module.cpp:22-62); single-GPU decode goes through Python per layer there
// (muillm/modules/decoder/decoder.py:95-165).
#include "gemv_common.cuh"

#include <algorithm>
#include <cstring>
#include <new>
#include <vector>

mui_status_t mui_launch_embedding(cudaStream_t stream, const void* table, const int64_t* tokens, void* out, int B,
                                  int H, int vocab, int pdl);
mui_status_t mui_launch_argmax_advance(cudaStream_t stream, mui_dtype_t dtype, const void* logits, int V, int B,
                                       long long* state, int32_t* seq_len32, long long* out_tokens, int out_capacity,
                                       void* work, int pdl, const CommDev* comm, int index_offset);
mui_status_t mui_comm_device_view(mui_comm_t* c, CommDev* out);
size_t mui_argmax_work_bytes(int B);
mui_status_t mui_linear_forward_hinted(void* stream, mui_dtype_t dtype, int B, int N, int K,
                                       const void* norm_weights, float epsilon, const void* weights,
                                       mui_activation_t activ, const void* mul_bias, const void* add_bias,
                                       const void* residual, const void* x, void* y, unsigned flags,
                                       const GemvHints* hints);
mui_status_t mui_gateup_silu_forward_hinted(void* stream, mui_dtype_t dtype, int B, int I, int H,
                                            const void* norm_weights, float epsilon, const void* gate_weights,
                                            const void* up_weights, const void* x, void* t, unsigned flags,
                                            const GemvHints* hints);
mui_status_t mui_parallel_linear_forward_hinted(mui_comm_t* c, void* stream, mui_dtype_t dtype, int B, int N, int K,
                                                const void* norm_weights, float epsilon, const void* weights,
                                                const void* mul_bias, const void* add_bias, const void* residual,
                                                const void* x, void* y, unsigned flags, const GemvHints* hints);
mui_status_t mui_llama4_qk_prologue_indexed(cudaStream_t stream, mui_dtype_t dtype, int B, int T, int Hq, int Hk, int D,
                                            const float* freqs_table, const int64_t* position_ids, int use_rope,
                                            int use_qk_norm, float norm_eps, const int64_t* cache_position,
                                            float attn_scale, float floor_scale, const void* q_in,
                                            mui_strides3_t q_strides, const void* k_in, mui_strides3_t k_strides,
                                            void* q_out, void* k_out, unsigned flags);

struct WeightRef {
  const void* ptr;
  int rows, row_bytes;
};

struct mui_llama_stack {
  mui_llama_config_t cfg;
  std::vector<const void*> qkv, o, gate, up, down, ln1, ln2;
  std::vector<void*> k_cache, v_cache;
  const void *embed, *final_norm, *lm_head, *cos_t, *sin_t;
  // scratch carve-up (device)
  unsigned char* scratch;
  long long* state;      // [3 + 2B] int64: step, tokens in cache, cache_position, position_ids[B], tokens[B]
  int32_t* seq_len32;    // tokens attended by the current step (= tokens in cache + 1)
  void *h, *qkv_out, *q_rot, *k_rot, *attn, *t, *logits;
  void* fd_ws;
  size_t fd_ws_bytes;
  void* argmax_work;
  long long* out_tokens;
  int out_capacity;
  int s_upper;           // upper bound of the attended length until the next reset (picks the attention variant)
  int host_pos;          // tokens in the cache as far as the host has launched steps
  bool capturing;        // launch_step runs under stream capture
  bool graph_short;      // the captured step uses the short-context attention kernel
  bool layers_only;      // launch_step stops after the last decoder layer (mui_llama_stack_forward_hidden)
  bool skip_embedding;   // launch_step starts from the hidden states already in `h`
  cudaGraphExec_t graph_exec;
  unsigned graph_flags;
  mui_comm_t* comm;  // tensor-parallel communicator (null on a single GPU)
  const void* attn_mask;  // additive [B, max_seq] of the model dtype (left-padded batches), or null
  CommDev comm_dev;
  std::vector<WeightRef> order;  // weight matrices in execution order: per layer qkv, o, gate, up, down; then lm_head
  size_t prefetch_window;
  // Llama-4 (MoE, chunked / full attention layers); `cfg` then carries the common sizes with intermediate =
  // expert_intermediate and batch = 1
  bool l4;
  mui_llama4_config_t l4cfg;
  std::vector<const void*> router;
  std::vector<int> use_rope, cache_rows;
  const float* freqs;
  // router outputs of the last step, kept per layer (the caller can read them back, mui_llama4_stack_router_state)
  float* router_logits;           // [layers][num_experts]
  unsigned int* router_counter;   // arrival counter of the router kernel (zero between launches)
  unsigned char* router_scores;   // [layers][8] 16-bit
  long long* router_idx;          // [layers][8]
  long long* chunk_row;           // separate-launch attention path: cache row and attended length of the chunked
  int32_t* chunk_len32;           //   layers for the current step
};

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct ScratchLayout {
  size_t state, seq_len, h, qkv, q_rot, attn, t, logits, fd_ws, fd_ws_bytes, argmax_work, router, k_rot, total;
};

// t_rows: rows of the MLP intermediate (1 for a dense MLP, computed experts for MoE); router_experts > 0 adds the
// router scratch and the rotated-key row of the separate-launch Llama-4 attention path
ScratchLayout scratch_layout(const mui_llama_config_t& c, int t_rows = 1, int router_experts = 0) {
  const size_t L = c.layers;
  ScratchLayout l;
  const size_t B = c.batch, e = 2;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off = align_up(off + bytes, 256);
    return at;
  };
  l.state = take((3 + 2 * B) * sizeof(long long));
  l.seq_len = take(sizeof(int32_t));
  l.h = take(B * c.hidden * e);
  l.qkv = take(B * (size_t)(c.heads + 2 * c.kv_heads) * c.head_dim * e);
  l.q_rot = take(B * (size_t)c.heads * c.head_dim * e);
  l.attn = take(B * (size_t)c.heads * c.head_dim * e);
  l.t = take(B * (size_t)t_rows * c.intermediate * e);
  l.logits = take(B * (size_t)c.vocab * e);
  l.fd_ws_bytes = mui_flash_decode_workspace_bytes(c.batch, c.heads, c.kv_heads, c.head_dim, c.max_seq);
  l.fd_ws = take(l.fd_ws_bytes);
  l.argmax_work = take(mui_argmax_work_bytes(c.batch));
  l.router = l.k_rot = 0;
  if (router_experts > 0) {
    // [0,64): counter; [64,128): chunk row (int64) + chunk length (int32); [256, ...): per layer 8 indices (int64),
    // then per layer 8 scores (16 bytes), then per layer the logits (fp32)
    l.router = take(256 + L * 64 + L * 16 + L * (size_t)router_experts * 4);
    l.k_rot = take(B * (size_t)c.kv_heads * c.head_dim * e);
  }
  l.total = off;
  return l;
}

mui_llama_config_t common_cfg(const mui_llama4_config_t& c) {
  mui_llama_config_t o;
  memset(&o, 0, sizeof(o));
  o.dtype = c.dtype;
  o.layers = c.layers;
  o.hidden = c.hidden;
  o.intermediate = c.expert_intermediate;
  o.heads = c.heads;
  o.kv_heads = c.kv_heads;
  o.head_dim = c.head_dim;
  o.vocab = c.vocab;
  o.max_seq = c.max_seq;
  o.batch = 1;
  o.rms_eps = c.rms_eps;
  o.attn_scale = c.softmax_scale;
  o.embed_vocab = c.embed_vocab;
  o.vocab_offset = c.vocab_offset;
  return o;
}

mui_status_t validate_cfg_l4(const mui_llama4_config_t* c) {
  MUI_REQUIRE(c != nullptr, MUI_ERR_INVALID_ARG, "config is null");
  MUI_REQUIRE(c->num_experts >= 1 && c->num_experts <= 1024 && c->top_k >= 1 && c->top_k <= c->num_experts &&
                  c->num_shared >= 0 && c->num_shared + c->top_k <= 8,
              MUI_ERR_UNSUPPORTED, "experts=%d top_k=%d shared=%d (at most 8 experts are computed per token)",
              c->num_experts, c->top_k, c->num_shared);
  MUI_REQUIRE(c->chunk >= 0, MUI_ERR_INVALID_ARG, "chunk must not be negative");
  MUI_REQUIRE(!c->temperature_tuning || c->floor_scale > 0.f, MUI_ERR_INVALID_ARG, "floor_scale must be positive");
  MUI_REQUIRE((c->head_dim & 1) == 0, MUI_ERR_UNSUPPORTED, "head_dim must be even");
  return MUI_OK;
}

int l4_cache_rows(const mui_llama4_config_t& c, int use_rope) {
  return (use_rope && c.chunk > 0) ? std::min(c.max_seq, c.chunk) : c.max_seq;
}

// Separate-launch Llama-4 attention path: row and attended length of the chunked layers for this step
__global__ void l4_chunk_state_kernel(const long long* state, long long* chunk_row, int32_t* chunk_len32, int chunk) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const long long pos = __ldcg(state + 2);
  const long long row = chunk > 0 ? pos % chunk : pos;
  *chunk_row = row;
  *chunk_len32 = static_cast<int32_t>(row + 1);
}

mui_status_t validate_cfg(const mui_llama_config_t* c) {
  MUI_REQUIRE(c != nullptr, MUI_ERR_INVALID_ARG, "config is null");
  MUI_REQUIRE(c->dtype == MUI_F16 || c->dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)c->dtype);
  MUI_REQUIRE(c->layers >= 1 && c->hidden >= 8 && c->intermediate >= 8 && c->vocab >= 1, MUI_ERR_INVALID_ARG,
              "bad model sizes");
  MUI_REQUIRE(c->heads >= 1 && c->kv_heads >= 1 && c->heads % c->kv_heads == 0, MUI_ERR_INVALID_ARG,
              "heads=%d kv_heads=%d", c->heads, c->kv_heads);
  MUI_REQUIRE(c->head_dim == 64 || c->head_dim == 128, MUI_ERR_UNSUPPORTED, "head_dim %d unsupported", c->head_dim);
  MUI_REQUIRE(c->batch >= 1 && c->batch <= 8, MUI_ERR_UNSUPPORTED, "batch %d outside 1..8", c->batch);
  MUI_REQUIRE(c->max_seq >= 1, MUI_ERR_INVALID_ARG, "max_seq must be positive");
  return MUI_OK;
}

// Decode state from caller-owned device tensors (mui_llama_stack_forward_hidden): tokens in cache = cache position,
// attended length = cache position + 1; the step counter is left alone.
__global__ void set_decode_state_kernel(long long* state, int32_t* seq_len32, const long long* tokens,
                                        const long long* position_ids, const long long* cache_position, int B) {
  const int t = threadIdx.x;
  const long long cp = cache_position[0];
  if (t == 0) {
    state[1] = cp;
    state[2] = cp;
    *seq_len32 = static_cast<int32_t>(cp + 1);
  }
  if (t < B) {
    state[3 + t] = position_ids[t];
    if (tokens) state[3 + B + t] = tokens[t];
  }
}

// Hints for the GEMV about to be launched: the weight matrices that follow it in execution order, up to `window`
// bytes in total (a gate/up pair shares its part of the window evenly, since the kernel consumes both in step), and
// the SMs it leaves free. 24 MB measured best on the 8B decode step (8-48 MB within 1 %, none -2 %, 96 MB -3 %).
constexpr size_t PREFETCH_WINDOW_BYTES = (size_t)24 << 20;

GemvHints make_hints(const std::vector<WeightRef>& order, size_t first, size_t window, int reserve_sms) {
  GemvHints h;
  memset(&h, 0, sizeof(h));
  h.reserve_sms = reserve_sms;
  int n = 0;
  for (size_t i = first; i < order.size() && n < 3 && window > 0; ++i) {
    const size_t full = (size_t)order[i].rows * order[i].row_bytes;
    const bool pair = (i % 5 == 2) && i + 1 < order.size() && n < 2;  // gate followed by up
    if (pair) {
      const size_t take = std::min(2 * full, window);
      const int f = (int)std::min<size_t>(1024, take * 1024 / (2 * full));
      for (int j = 0; j < 2; ++j) {
        h.pf_ptr[n] = order[i + j].ptr;
        h.pf_rows[n] = order[i + j].rows;
        h.pf_row_bytes[n] = order[i + j].row_bytes;
        h.pf_frac[n] = f;
        ++n;
      }
      window -= take;
      ++i;
    } else {
      const size_t take = std::min(full, window);
      h.pf_ptr[n] = order[i].ptr;
      h.pf_rows[n] = order[i].rows;
      h.pf_row_bytes[n] = order[i].row_bytes;
      h.pf_frac[n] = (int)std::min<size_t>(1024, take * 1024 / full);
      window -= take;
      ++n;
    }
  }
  return h;
}

// One decode step of a Llama-4 text model (batch 1): six launches per layer on the fused path.
mui_status_t launch_step_l4(mui_llama_stack* s, cudaStream_t stream, unsigned flags) {
  const mui_llama_config_t& c = s->cfg;
  const mui_llama4_config_t& c4 = s->l4cfg;
  const int H = c.hidden, Hq = c.heads, Hkv = c.kv_heads, D = c.head_dim, I = c.intermediate;
  const int qkv_n = (Hq + 2 * Hkv) * D;
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  const long long* tokens = s->state + 4;
  const int64_t* position_ids = reinterpret_cast<const int64_t*>(s->state + 3);
  const int64_t* cache_position = reinterpret_cast<const int64_t*>(s->state + 2);
  const bool tp = s->comm != nullptr;
  const int embed_rows = c.embed_vocab > 0 ? c.embed_vocab : c.vocab;
  mui_status_t st;
  if (!s->skip_embedding) {
    st = mui_launch_embedding(stream, s->embed, (const int64_t*)tokens, s->h, 1, H, embed_rows, pdl);
    if (st != MUI_OK) return st;
  }
  const bool fused_attn = D == 128 && Hq / Hkv <= 8 && !(flags & MUI_FLAG_FORCE_GENERIC);
  const int attended = s->capturing ? s->s_upper : s->host_pos + 1;
  if (!fused_attn && c4.chunk > 0) {
    MUI_CUDA_CHECK(mui_launch(l4_chunk_state_kernel, dim3(1), dim3(1), 0, stream, pdl, (const long long*)s->state,
                              s->chunk_row, s->chunk_len32, c4.chunk));
  }
  const mui_strides3_t qs = {(int64_t)qkv_n, (int64_t)D, (int64_t)qkv_n};
  const mui_strides3_t krs = {(int64_t)Hkv * D, (int64_t)D, (int64_t)D};
  const size_t e = 2;
  for (int l = 0; l < c.layers; ++l) {
    const int rope = s->use_rope[l];
    const int rows = s->cache_rows[l];
    const int norm = (c4.use_qk_norm && rope) ? 1 : 0;
    const int tune = (c4.temperature_tuning && !rope) ? 1 : 0;
    const int chunk = (rope && c4.chunk > 0) ? c4.chunk : 0;
    // the one-CTA-per-KV-head attention kernel serves up to 384 attended rows: always enough for a short chunk
    const int layer_attended = chunk > 0 ? std::min(attended, chunk) : attended;
    const bool short_ctx = fused_attn && pdl && layer_attended <= 384 && Hkv <= 16;
    if (s->capturing && short_ctx && !(chunk > 0 && chunk <= 384)) s->graph_short = true;
    // the attention CTAs (one per KV head) move in beside the QKV projection and are still there when o_proj starts
    GemvHints reserve;
    memset(&reserve, 0, sizeof(reserve));
    reserve.reserve_sms = short_ctx ? Hkv : 0;
    st = mui_linear_forward_hinted(stream, c.dtype, 1, qkv_n, H, s->ln1[l], c.rms_eps, s->qkv[l], MUI_ACT_IDENTITY,
                                   nullptr, nullptr, nullptr, s->h, s->qkv_out, flags, &reserve);
    if (st != MUI_OK) return st;
    if (fused_attn) {
      st = mui_llama4_rope_flash_decode(stream, c.dtype, 1, Hq, Hkv, D, rows, c.max_seq, s->qkv_out, s->freqs,
                                        position_ids, cache_position, rope, norm, c.rms_eps, tune, c4.attn_scale,
                                        c4.floor_scale, chunk, c.attn_scale, s->k_cache[l], s->v_cache[l], s->attn,
                                        s->fd_ws, s->fd_ws_bytes, layer_attended,
                                        flags | (short_ctx ? MUI_FLAG_SHORT_CONTEXT : MUI_FLAG_SPLIT_CONTEXT));
      if (st != MUI_OK) return st;
    } else {
      const unsigned char* qp = (const unsigned char*)s->qkv_out;
      const int64_t* row_ptr = chunk > 0 ? reinterpret_cast<const int64_t*>(s->chunk_row) : cache_position;
      const int32_t* len_ptr = chunk > 0 ? s->chunk_len32 : s->seq_len32;
      const void* q_for_attn = s->q_rot;
      const void* k_for_cache = s->k_rot;
      if (rope || norm || tune) {
        st = mui_llama4_qk_prologue_indexed(stream, c.dtype, 1, 1, Hq, Hkv, D, s->freqs, position_ids, rope, norm,
                                            c.rms_eps, tune ? cache_position : nullptr, c4.attn_scale, c4.floor_scale,
                                            qp, qs, qp + (size_t)Hq * D * e, qs, s->q_rot, s->k_rot, flags);
        if (st != MUI_OK) return st;
      } else {
        // nothing to do to q and k: q must still be contiguous for flash decoding (it is: one token), k is read
        // through its strides
        q_for_attn = qp;
        k_for_cache = nullptr;
      }
      st = mui_static_kvcache_update(stream, c.dtype, 1, 1, rows, Hkv, D,
                                     k_for_cache ? k_for_cache : (const void*)(qp + (size_t)Hq * D * e),
                                     k_for_cache ? krs : qs, qp + (size_t)(Hq + Hkv) * D * e, qs, s->k_cache[l],
                                     s->v_cache[l], row_ptr, flags);
      if (st != MUI_OK) return st;
      const mui_strides3_t kvs = {(int64_t)Hkv * rows * D, (int64_t)rows * D, (int64_t)D};
      st = mui_flash_decode(stream, c.dtype, 1, Hq, Hkv, D, rows, len_ptr, c.attn_scale, q_for_attn, s->k_cache[l],
                            s->v_cache[l], kvs, nullptr, s->attn, s->fd_ws, s->fd_ws_bytes, flags);
      if (st != MUI_OK) return st;
    }
    if (tp)
      st = mui_parallel_linear_forward_hinted(s->comm, stream, c.dtype, 1, H, Hq * D, nullptr, 0.f, s->o[l], nullptr,
                                              nullptr, s->h, s->attn, s->h, flags, &reserve);
    else
      st = mui_linear_forward_hinted(stream, c.dtype, 1, H, Hq * D, nullptr, 0.f, s->o[l], MUI_ACT_IDENTITY, nullptr,
                                     nullptr, s->h, s->attn, s->h, flags, &reserve);
    if (st != MUI_OK) return st;
    float* r_logits = s->router_logits + (size_t)l * c4.num_experts;
    void* r_scores = s->router_scores + (size_t)l * 16;
    int64_t* r_idx = reinterpret_cast<int64_t*>(s->router_idx + (size_t)l * 8);
    st = mui_router_topk_sigmoid_forward(stream, c.dtype, c4.num_experts, H, c4.top_k, s->ln2[l], c.rms_eps,
                                         s->router[l], s->h, r_logits, s->router_counter, r_scores, r_idx, flags);
    if (st != MUI_OK) return st;
    if (tp)
      st = mui_parallel_moe_mlp_forward(s->comm, stream, c.dtype, c4.num_shared, c4.num_experts, c4.top_k, I, H,
                                        s->ln2[l], c.rms_eps, s->gate[l], s->up[l], s->down[l], s->h, s->h,
                                        r_scores, r_idx, s->t, s->h,
                                        flags);
    else
      st = mui_moe_mlp_forward(stream, c.dtype, c4.num_shared, c4.num_experts, c4.top_k, I, H, s->ln2[l], c.rms_eps,
                               s->gate[l], s->up[l], s->down[l], s->h, s->h, r_scores, r_idx, s->t, s->h, flags);
    if (st != MUI_OK) return st;
  }
  if (s->layers_only) return MUI_OK;
  st = mui_linear_forward(stream, c.dtype, 1, c.vocab, H, s->final_norm, c.rms_eps, s->lm_head, MUI_ACT_IDENTITY,
                          nullptr, nullptr, nullptr, s->h, s->logits, flags);
  if (st != MUI_OK) return st;
  return mui_launch_argmax_advance(stream, c.dtype, s->logits, c.vocab, 1, s->state, s->seq_len32, s->out_tokens,
                                   s->out_capacity, s->argmax_work, pdl, tp ? &s->comm_dev : nullptr, c.vocab_offset);
}

mui_status_t launch_step(mui_llama_stack* s, cudaStream_t stream, unsigned flags) {
  if (s->l4) return launch_step_l4(s, stream, flags);
  const mui_llama_config_t& c = s->cfg;
  const int B = c.batch, H = c.hidden, Hq = c.heads, Hkv = c.kv_heads, D = c.head_dim;
  const int qkv_n = (Hq + 2 * Hkv) * D;
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  const long long* tokens = s->state + 3 + B;
  const long long* position_ids = s->state + 3;
  const long long* cache_position = s->state + 2;
  mui_status_t st;
  const bool tp = s->comm != nullptr;
  const bool pf = s->prefetch_window > 0;
  const int embed_rows = c.embed_vocab > 0 ? c.embed_vocab : c.vocab;
  if (!s->skip_embedding) {
    st = mui_launch_embedding(stream, s->embed, (const int64_t*)tokens, s->h, B, H, embed_rows, pdl);
    if (st != MUI_OK) return st;
  }
  // q,k,v are slices of the packed qkv row: [B, 1, (Hq+2Hkv)*D] viewed as [B, H*, 1, D]
  const mui_strides3_t qs = {(int64_t)qkv_n, (int64_t)D, (int64_t)qkv_n};
  const mui_strides3_t kvs = {(int64_t)Hkv * c.max_seq * D, (int64_t)c.max_seq * D, (int64_t)D};
  const size_t e = 2;
  const size_t win = pf ? s->prefetch_window : 0;
  for (int l = 0; l < c.layers; ++l) {
    // a masked (left-padded) batch takes RoPE + cache write and split-KV flash decoding as two launches
    const bool fused_attn = D == 128 && Hq / Hkv <= 8 && !(flags & MUI_FLAG_FORCE_GENERIC) && s->attn_mask == nullptr;
    // short histories: one CTA per KV head that moves in beside the QKV projection (which leaves it the SMs) and
    // has the K/V rows in shared memory by the time q arrives
    const int attended = s->capturing ? s->s_upper : s->host_pos + 1;
    const bool short_ctx = fused_attn && pdl && attended <= 384 && Hkv * B <= 16;
    if (s->capturing) s->graph_short = short_ctx;
    const int reserve = short_ctx ? Hkv * B : 0;
    GemvHints hints = make_hints(s->order, 5 * (size_t)l + 1, win, reserve);
    st = mui_linear_forward_hinted(stream, c.dtype, B, qkv_n, H, s->ln1[l], c.rms_eps, s->qkv[l], MUI_ACT_IDENTITY,
                                   nullptr, nullptr, nullptr, s->h, s->qkv_out, flags, &hints);
    if (st != MUI_OK) return st;
    if (fused_attn) {
      // one launch: RoPE + cache write + attention. Up to 384 tokens one CTA per KV head (resident beside the QKV
      // projection); beyond, the same tensor-core kernel with the tokens split over several CTAs per KV head
      st = mui_rope_flash_decode_ws(stream, c.dtype, B, Hq, Hkv, D, c.max_seq, s->qkv_out, s->cos_t, s->sin_t,
                                    (const int64_t*)position_ids, (const int64_t*)cache_position, s->seq_len32,
                                    c.attn_scale, s->k_cache[l], s->v_cache[l], s->attn, s->fd_ws, s->fd_ws_bytes,
                                    attended,
                                    flags | (short_ctx ? MUI_FLAG_SHORT_CONTEXT : MUI_FLAG_SPLIT_CONTEXT));
      if (st != MUI_OK) return st;
    } else {
      const unsigned char* qp = (const unsigned char*)s->qkv_out;
      st = mui_rope_forward(stream, c.dtype, B, 1, c.max_seq, Hq, Hkv, D, 0, (const int64_t*)position_ids, s->cos_t,
                            s->sin_t, qp, qs, qp + (size_t)Hq * D * e, qs, qp + (size_t)(Hq + Hkv) * D * e, qs,
                            s->q_rot, nullptr, s->k_cache[l], s->v_cache[l], (const int64_t*)cache_position, flags);
      if (st != MUI_OK) return st;
      st = mui_flash_decode(stream, c.dtype, B, Hq, Hkv, D, c.max_seq, s->seq_len32, c.attn_scale, s->q_rot,
                            s->k_cache[l], s->v_cache[l], kvs, s->attn_mask, s->attn, s->fd_ws, s->fd_ws_bytes, flags);
      if (st != MUI_OK) return st;
    }
    // the attention CTAs still hold their SMs when o_proj's CTAs are placed: a full-width grid would leave its last
    // CTAs waiting for them (measured on the 8B decode step: +1.6 % tokens/s)
    hints = make_hints(s->order, 5 * (size_t)l + 2, win, reserve);
    if (tp)
      st = mui_parallel_linear_forward_hinted(s->comm, stream, c.dtype, B, H, Hq * D, nullptr, 0.f, s->o[l], nullptr,
                                              nullptr, s->h, s->attn, s->h, flags, &hints);
    else
      st = mui_linear_forward_hinted(stream, c.dtype, B, H, Hq * D, nullptr, 0.f, s->o[l], MUI_ACT_IDENTITY, nullptr,
                                     nullptr, s->h, s->attn, s->h, flags, &hints);
    if (st != MUI_OK) return st;
    hints = make_hints(s->order, 5 * (size_t)l + 4, win, 0);
    st = mui_gateup_silu_forward_hinted(stream, c.dtype, B, c.intermediate, H, s->ln2[l], c.rms_eps, s->gate[l],
                                        s->up[l], s->h, s->t, flags, &hints);
    if (st != MUI_OK) return st;
    hints = make_hints(s->order, 5 * (size_t)l + 5, win, 0);
    if (tp)
      st = mui_parallel_linear_forward_hinted(s->comm, stream, c.dtype, B, H, c.intermediate, nullptr, 0.f, s->down[l],
                                              nullptr, nullptr, s->h, s->t, s->h, flags, &hints);
    else
      st = mui_linear_forward_hinted(stream, c.dtype, B, H, c.intermediate, nullptr, 0.f, s->down[l],
                                     MUI_ACT_IDENTITY, nullptr, nullptr, s->h, s->t, s->h, flags, &hints);
    if (st != MUI_OK) return st;
  }
  if (s->layers_only) return MUI_OK;
  st = mui_linear_forward(stream, c.dtype, B, c.vocab, H, s->final_norm, c.rms_eps, s->lm_head, MUI_ACT_IDENTITY,
                          nullptr, nullptr, nullptr, s->h, s->logits, flags);
  if (st != MUI_OK) return st;
  return mui_launch_argmax_advance(stream, c.dtype, s->logits, c.vocab, B, s->state, s->seq_len32, s->out_tokens,
                                   s->out_capacity, s->argmax_work, pdl, tp ? &s->comm_dev : nullptr,
                                   c.vocab_offset);
}

}  // namespace

extern "C" {

size_t mui_llama_stack_scratch_bytes(const mui_llama_config_t* cfg) {
  if (validate_cfg(cfg) != MUI_OK) return 0;
  return scratch_layout(*cfg).total;
}

mui_status_t mui_llama_stack_create(const mui_llama_config_t* cfg, const mui_llama_weights_t* w, void* scratch,
                                    size_t scratch_bytes, mui_llama_stack_t** out) {
  if (mui_status_t s = validate_cfg(cfg)) return s;
  MUI_REQUIRE(w && scratch && out, MUI_ERR_INVALID_ARG, "weights, scratch and out must be non-null");
  MUI_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255) == 0, MUI_ERR_INVALID_ARG, "scratch must be 256-byte aligned");
  const ScratchLayout lay = scratch_layout(*cfg);
  MUI_REQUIRE(scratch_bytes >= lay.total, MUI_ERR_INVALID_ARG, "scratch too small: %zu < %zu", scratch_bytes, lay.total);
  MUI_REQUIRE(w->embed && w->final_norm && w->lm_head && w->cos_table && w->sin_table, MUI_ERR_INVALID_ARG,
              "embed, final_norm, lm_head, cos_table and sin_table must be non-null");
  MUI_REQUIRE(w->qkv && w->o && w->gate && w->up && w->down && w->ln1 && w->ln2 && w->k_cache && w->v_cache,
              MUI_ERR_INVALID_ARG, "per-layer pointer arrays must be non-null");
  mui_llama_stack* s = new (std::nothrow) mui_llama_stack();
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "out of host memory");
  s->cfg = *cfg;
  for (int l = 0; l < cfg->layers; ++l) {
    const void* ptrs[] = {w->qkv[l], w->o[l], w->gate[l], w->up[l], w->down[l], w->ln1[l], w->ln2[l],
                          w->k_cache[l], w->v_cache[l]};
    for (const void* p : ptrs) {
      if (p == nullptr) {
        delete s;
        mui_set_error("layer %d has a null weight or cache pointer", l);
        return MUI_ERR_INVALID_ARG;
      }
    }
    s->qkv.push_back(w->qkv[l]);
    s->o.push_back(w->o[l]);
    s->gate.push_back(w->gate[l]);
    s->up.push_back(w->up[l]);
    s->down.push_back(w->down[l]);
    s->ln1.push_back(w->ln1[l]);
    s->ln2.push_back(w->ln2[l]);
    s->k_cache.push_back(w->k_cache[l]);
    s->v_cache.push_back(w->v_cache[l]);
  }
  s->embed = w->embed;
  s->final_norm = w->final_norm;
  s->lm_head = w->lm_head;
  s->cos_t = w->cos_table;
  s->sin_t = w->sin_table;
  unsigned char* base = reinterpret_cast<unsigned char*>(scratch);
  s->scratch = base;
  s->state = reinterpret_cast<long long*>(base + lay.state);
  s->seq_len32 = reinterpret_cast<int32_t*>(base + lay.seq_len);
  s->h = base + lay.h;
  s->qkv_out = base + lay.qkv;
  s->q_rot = base + lay.q_rot;
  s->attn = base + lay.attn;
  s->t = base + lay.t;
  s->logits = base + lay.logits;
  s->fd_ws = base + lay.fd_ws;
  s->fd_ws_bytes = lay.fd_ws_bytes;
  s->argmax_work = base + lay.argmax_work;
  s->out_tokens = nullptr;
  s->out_capacity = 0;
  s->s_upper = cfg->max_seq;
  s->host_pos = 0;
  s->capturing = false;
  s->graph_short = false;
  s->layers_only = false;
  s->skip_embedding = false;
  s->graph_exec = nullptr;
  s->graph_flags = 0;
  s->comm = nullptr;
  s->attn_mask = nullptr;
  s->l4 = false;
  s->k_rot = nullptr;
  s->freqs = nullptr;
  s->router_logits = nullptr;
  s->router_counter = nullptr;
  s->router_scores = nullptr;
  s->router_idx = nullptr;
  s->chunk_row = nullptr;
  s->chunk_len32 = nullptr;
  {
    const int qkv_rows = (cfg->heads + 2 * cfg->kv_heads) * cfg->head_dim;
    const int od = cfg->heads * cfg->head_dim;
    for (int l = 0; l < cfg->layers; ++l) {
      s->order.push_back(WeightRef{w->qkv[l], qkv_rows, cfg->hidden * 2});
      s->order.push_back(WeightRef{w->o[l], cfg->hidden, od * 2});
      s->order.push_back(WeightRef{w->gate[l], cfg->intermediate, cfg->hidden * 2});
      s->order.push_back(WeightRef{w->up[l], cfg->intermediate, cfg->hidden * 2});
      s->order.push_back(WeightRef{w->down[l], cfg->hidden, cfg->intermediate * 2});
    }
    s->order.push_back(WeightRef{w->lm_head, cfg->vocab, cfg->hidden * 2});
    s->prefetch_window = PREFETCH_WINDOW_BYTES;
  }
  *out = s;
  return MUI_OK;
}

int mui_llama4_stack_cache_rows(const mui_llama4_config_t* cfg, int use_rope) {
  if (cfg == nullptr) return 0;
  return l4_cache_rows(*cfg, use_rope);
}

size_t mui_llama4_stack_scratch_bytes(const mui_llama4_config_t* cfg) {
  if (validate_cfg_l4(cfg) != MUI_OK) return 0;
  const mui_llama_config_t c = common_cfg(*cfg);
  if (validate_cfg(&c) != MUI_OK) return 0;
  return scratch_layout(c, cfg->num_shared + cfg->top_k, cfg->num_experts).total;
}

mui_status_t mui_llama4_stack_create(const mui_llama4_config_t* cfg4, const mui_llama4_weights_t* w, void* scratch,
                                     size_t scratch_bytes, mui_llama_stack_t** out) {
  if (mui_status_t st = validate_cfg_l4(cfg4)) return st;
  const mui_llama_config_t cfg = common_cfg(*cfg4);
  if (mui_status_t st = validate_cfg(&cfg)) return st;
  MUI_REQUIRE(w && scratch && out, MUI_ERR_INVALID_ARG, "weights, scratch and out must be non-null");
  MUI_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255) == 0, MUI_ERR_INVALID_ARG, "scratch must be 256-byte aligned");
  const ScratchLayout lay = scratch_layout(cfg, cfg4->num_shared + cfg4->top_k, cfg4->num_experts);
  MUI_REQUIRE(scratch_bytes >= lay.total, MUI_ERR_INVALID_ARG, "scratch too small: %zu < %zu", scratch_bytes, lay.total);
  MUI_REQUIRE(w->embed && w->final_norm && w->lm_head && w->freqs && w->use_rope, MUI_ERR_INVALID_ARG,
              "embed, final_norm, lm_head, freqs and use_rope must be non-null");
  MUI_REQUIRE(w->qkv && w->o && w->router && w->gate && w->up && w->down && w->ln1 && w->ln2 && w->k_cache &&
                  w->v_cache,
              MUI_ERR_INVALID_ARG, "per-layer pointer arrays must be non-null");
  MUI_REQUIRE((reinterpret_cast<uintptr_t>(w->freqs) & 15) == 0, MUI_ERR_INVALID_ARG, "freqs must be 16-byte aligned");
  mui_llama_stack* s = new (std::nothrow) mui_llama_stack();
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "out of host memory");
  s->cfg = cfg;
  s->l4 = true;
  s->l4cfg = *cfg4;
  for (int l = 0; l < cfg.layers; ++l) {
    const void* ptrs[] = {w->qkv[l], w->o[l], w->router[l], w->gate[l], w->up[l], w->down[l], w->ln1[l], w->ln2[l],
                          w->k_cache[l], w->v_cache[l]};
    for (const void* p : ptrs) {
      if (p == nullptr) {
        delete s;
        mui_set_error("layer %d has a null weight or cache pointer", l);
        return MUI_ERR_INVALID_ARG;
      }
    }
    s->qkv.push_back(w->qkv[l]);
    s->o.push_back(w->o[l]);
    s->router.push_back(w->router[l]);
    s->gate.push_back(w->gate[l]);
    s->up.push_back(w->up[l]);
    s->down.push_back(w->down[l]);
    s->ln1.push_back(w->ln1[l]);
    s->ln2.push_back(w->ln2[l]);
    s->k_cache.push_back(w->k_cache[l]);
    s->v_cache.push_back(w->v_cache[l]);
    s->use_rope.push_back(w->use_rope[l] ? 1 : 0);
    s->cache_rows.push_back(l4_cache_rows(*cfg4, w->use_rope[l]));
  }
  s->embed = w->embed;
  s->final_norm = w->final_norm;
  s->lm_head = w->lm_head;
  s->cos_t = s->sin_t = nullptr;
  s->freqs = w->freqs;
  unsigned char* base = reinterpret_cast<unsigned char*>(scratch);
  s->scratch = base;
  s->state = reinterpret_cast<long long*>(base + lay.state);
  s->seq_len32 = reinterpret_cast<int32_t*>(base + lay.seq_len);
  s->h = base + lay.h;
  s->qkv_out = base + lay.qkv;
  s->q_rot = base + lay.q_rot;
  s->k_rot = base + lay.k_rot;
  s->attn = base + lay.attn;
  s->t = base + lay.t;
  s->logits = base + lay.logits;
  s->fd_ws = base + lay.fd_ws;
  s->fd_ws_bytes = lay.fd_ws_bytes;
  s->argmax_work = base + lay.argmax_work;
  s->router_counter = reinterpret_cast<unsigned int*>(base + lay.router);
  s->chunk_row = reinterpret_cast<long long*>(base + lay.router + 64);
  s->chunk_len32 = reinterpret_cast<int32_t*>(base + lay.router + 72);
  s->router_idx = reinterpret_cast<long long*>(base + lay.router + 256);
  s->router_scores = base + lay.router + 256 + (size_t)cfg.layers * 64;
  s->router_logits = reinterpret_cast<float*>(base + lay.router + 256 + (size_t)cfg.layers * 80);
  s->out_tokens = nullptr;
  s->out_capacity = 0;
  s->s_upper = cfg.max_seq;
  s->host_pos = 0;
  s->capturing = false;
  s->graph_short = false;
  s->layers_only = false;
  s->skip_embedding = false;
  s->graph_exec = nullptr;
  s->graph_flags = 0;
  s->comm = nullptr;
  s->attn_mask = nullptr;
  s->prefetch_window = 0;
  *out = s;
  return MUI_OK;
}

mui_status_t mui_llama4_stack_router_state(mui_llama_stack_t* s, float** logits_dev, int64_t** indices_dev) {
  MUI_REQUIRE(s != nullptr && s->l4, MUI_ERR_INVALID_ARG, "not a Llama-4 stack");
  if (logits_dev) *logits_dev = s->router_logits;
  if (indices_dev) *indices_dev = reinterpret_cast<int64_t*>(s->router_idx);
  return MUI_OK;
}

mui_status_t mui_llama_stack_set_comm(mui_llama_stack_t* s, mui_comm_t* comm) {
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "stack is null");
  if (comm == nullptr) {
    s->comm = nullptr;
    return MUI_OK;
  }
  int world = 1;
  size_t cap = 0;
  if (mui_status_t st = mui_comm_info(comm, nullptr, &world, &cap)) return st;
  if (world <= 1) {
    s->comm = nullptr;
    return MUI_OK;
  }
  MUI_REQUIRE(cap >= (size_t)s->cfg.batch * s->cfg.hidden, MUI_ERR_UNSUPPORTED,
              "communicator capacity %zu below batch*hidden = %zu", cap, (size_t)s->cfg.batch * s->cfg.hidden);
  if (mui_status_t st = mui_comm_device_view(comm, &s->comm_dev)) return st;
  s->comm = comm;
  if (s->graph_exec) {
    cudaGraphExecDestroy(s->graph_exec);
    s->graph_exec = nullptr;
  }
  return MUI_OK;
}

mui_status_t mui_llama_stack_destroy(mui_llama_stack_t* s) {
  if (s == nullptr) return MUI_OK;
  if (s->graph_exec) cudaGraphExecDestroy(s->graph_exec);
  delete s;
  return MUI_OK;
}

mui_status_t mui_llama_stack_reset(mui_llama_stack_t* s, void* stream, int position, const int64_t* position_ids_host,
                                   int64_t* out_tokens_dev, int out_capacity) {
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "stack is null");
  MUI_REQUIRE(position >= 0 && position < s->cfg.max_seq, MUI_ERR_INVALID_ARG, "position %d outside the cache (%d)",
              position, s->cfg.max_seq);
  const int B = s->cfg.batch;
  std::vector<long long> st(3 + 2 * B, 0);
  st[0] = 0;
  st[1] = position;
  st[2] = position;
  for (int b = 0; b < B; ++b) st[3 + b] = position_ids_host ? position_ids_host[b] : position;
  cudaStream_t cs = (cudaStream_t)stream;
  // pageable host memory: the runtime stages the copy before returning, the vector may go out of scope
  MUI_CUDA_CHECK(cudaMemcpyAsync(s->state, st.data(), st.size() * sizeof(long long), cudaMemcpyHostToDevice, cs));
  const int32_t sl = position + 1;
  MUI_CUDA_CHECK(cudaMemcpyAsync(s->seq_len32, &sl, sizeof(sl), cudaMemcpyHostToDevice, cs));
  // flash-decoding and arg-max arrival counters start at zero
  MUI_CUDA_CHECK(cudaMemsetAsync(s->fd_ws, 0, 4096, cs));
  MUI_CUDA_CHECK(cudaMemsetAsync(s->argmax_work, 0, 64, cs));
  if (s->l4) MUI_CUDA_CHECK(cudaMemsetAsync(s->router_counter, 0, 64, cs));
  s->out_tokens = reinterpret_cast<long long*>(out_tokens_dev);
  s->out_capacity = out_tokens_dev ? out_capacity : 0;
  // the caller's token buffer bounds how far this run decodes; without one assume the whole cache
  s->s_upper = out_tokens_dev ? std::min(s->cfg.max_seq, position + out_capacity + 1) : s->cfg.max_seq;
  s->host_pos = position;
  if (s->graph_exec) {  // the captured argmax node holds the old output pointer
    cudaGraphExecDestroy(s->graph_exec);
    s->graph_exec = nullptr;
  }
  return MUI_OK;
}

mui_status_t mui_llama_stack_set_tokens(mui_llama_stack_t* s, void* stream, const int64_t* tokens, int on_device) {
  MUI_REQUIRE(s && tokens, MUI_ERR_INVALID_ARG, "null pointer");
  const int B = s->cfg.batch;
  MUI_CUDA_CHECK(cudaMemcpyAsync(s->state + 3 + B, tokens, B * sizeof(long long),
                                 on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return MUI_OK;
}

mui_status_t mui_llama_stack_set_position_ids(mui_llama_stack_t* s, void* stream, const int64_t* position_ids,
                                              int on_device) {
  MUI_REQUIRE(s && position_ids, MUI_ERR_INVALID_ARG, "null pointer");
  MUI_CUDA_CHECK(cudaMemcpyAsync(s->state + 3, position_ids, s->cfg.batch * sizeof(long long),
                                 on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return MUI_OK;
}

mui_status_t mui_llama_stack_set_attention_mask(mui_llama_stack_t* s, const void* mask_dev) {
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "stack is null");
  MUI_REQUIRE(!s->l4 || mask_dev == nullptr, MUI_ERR_UNSUPPORTED, "the Llama-4 stack decodes one sequence: no mask");
  if (mask_dev != s->attn_mask && s->graph_exec) {  // a captured step holds the old attention launches
    cudaGraphExecDestroy(s->graph_exec);
    s->graph_exec = nullptr;
  }
  s->attn_mask = mask_dev;
  return MUI_OK;
}

mui_status_t mui_llama_stack_step(mui_llama_stack_t* s, void* stream, unsigned flags) {
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "stack is null");
  // a step writes cache row host_pos and reads row host_pos of the rotary tables: both end at max_seq
  MUI_REQUIRE(s->host_pos < s->cfg.max_seq, MUI_ERR_UNSUPPORTED,
              "the KV cache is full: %d tokens cached, max_seq %d (reset the stack or build it with a longer cache)",
              s->host_pos, s->cfg.max_seq);
  s->capturing = false;
  const mui_status_t st = launch_step(s, (cudaStream_t)stream, flags);
  if (st == MUI_OK) s->host_pos += 1;
  return st;
}

mui_status_t mui_llama_stack_capture(mui_llama_stack_t* s, void* stream, unsigned flags) {
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "stack is null");
  MUI_REQUIRE(stream != nullptr, MUI_ERR_INVALID_ARG, "capture needs a non-default stream");
  cudaStream_t cs = (cudaStream_t)stream;
  if (s->graph_exec) {
    cudaGraphExecDestroy(s->graph_exec);
    s->graph_exec = nullptr;
  }
  MUI_CUDA_CHECK(cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal));
  s->capturing = true;
  s->graph_short = false;
  mui_status_t st = launch_step(s, cs, flags);
  s->capturing = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(cs, &graph);
  if (st != MUI_OK) {
    if (graph) cudaGraphDestroy(graph);
    return st;
  }
  if (e != cudaSuccess) {
    mui_set_error("cudaStreamEndCapture failed: %s", cudaGetErrorString(e));
    return MUI_ERR_CUDA;
  }
  e = cudaGraphInstantiate(&s->graph_exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    s->graph_exec = nullptr;
    mui_set_error("cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    return MUI_ERR_CUDA;
  }
  s->graph_flags = flags;
  return MUI_OK;
}

mui_status_t mui_llama_stack_replay(mui_llama_stack_t* s, void* stream, int steps) {
  MUI_REQUIRE(s != nullptr && s->graph_exec != nullptr, MUI_ERR_INVALID_ARG, "no captured graph (call capture first)");
  MUI_REQUIRE(steps >= 0 && s->host_pos + steps <= s->cfg.max_seq, MUI_ERR_UNSUPPORTED,
              "%d more steps do not fit the KV cache: %d tokens cached, max_seq %d", steps, s->host_pos,
              s->cfg.max_seq);
  MUI_REQUIRE(!s->graph_short || s->host_pos + steps <= 384, MUI_ERR_UNSUPPORTED,
              "the captured step uses the short-context attention kernel (384 tokens); %d tokens are cached and %d "
              "more steps were asked for: reset with a larger token buffer and capture again", s->host_pos, steps);
  s->host_pos += steps;
  for (int i = 0; i < steps; ++i) MUI_CUDA_CHECK(cudaGraphLaunch(s->graph_exec, (cudaStream_t)stream));
  return MUI_OK;
}

mui_status_t mui_llama_stack_forward_hidden(mui_llama_stack_t* s, void* stream, const int64_t* token_ids_dev,
                                            const void* h_in, const int64_t* position_ids_dev,
                                            const int64_t* cache_position_dev, int seen_tokens, void* h_out,
                                            unsigned flags) {
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "stack is null");
  MUI_REQUIRE((token_ids_dev != nullptr) != (h_in != nullptr), MUI_ERR_INVALID_ARG,
              "give either token ids or hidden states");
  MUI_REQUIRE(position_ids_dev && cache_position_dev && h_out, MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(seen_tokens >= 1 && seen_tokens <= s->cfg.max_seq, MUI_ERR_INVALID_ARG,
              "seen_tokens %d outside 1..%d", seen_tokens, s->cfg.max_seq);
  cudaStream_t cs = (cudaStream_t)stream;
  const int B = s->cfg.batch;
  const size_t hbytes = (size_t)B * s->cfg.hidden * 2;
  set_decode_state_kernel<<<1, 32, 0, cs>>>(s->state, s->seq_len32, reinterpret_cast<const long long*>(token_ids_dev),
                                            reinterpret_cast<const long long*>(position_ids_dev),
                                            reinterpret_cast<const long long*>(cache_position_dev), B);
  MUI_CUDA_CHECK(cudaGetLastError());
  if (h_in) MUI_CUDA_CHECK(cudaMemcpyAsync(s->h, h_in, hbytes, cudaMemcpyDeviceToDevice, cs));
  s->capturing = false;
  s->host_pos = seen_tokens - 1;
  s->layers_only = true;
  s->skip_embedding = h_in != nullptr;
  const mui_status_t st = launch_step(s, cs, flags);
  s->layers_only = false;
  s->skip_embedding = false;
  if (st != MUI_OK) return st;
  s->host_pos = seen_tokens;
  MUI_CUDA_CHECK(cudaMemcpyAsync(h_out, s->h, hbytes, cudaMemcpyDeviceToDevice, cs));
  return MUI_OK;
}

mui_status_t mui_llama_stack_logits(mui_llama_stack_t* s, void** logits_dev, int64_t** state_dev) {
  MUI_REQUIRE(s != nullptr, MUI_ERR_INVALID_ARG, "stack is null");
  if (logits_dev) *logits_dev = s->logits;
  if (state_dev) *state_dev = reinterpret_cast<int64_t*>(s->state);
  return MUI_OK;
}

}  // extern "C"
