// Llama-4 attention prologue and windowed cache, plus two small bookkeeping kernels:
//   * q/k prologue: interleaved ("complex") rotary embedding -> L2 norm over the head dim -> temperature scale,
//     any subset, one warp per (head, token, batch) row, one launch. Each stage is evaluated in fp32 and rounded
//     to the 16-bit type, so the fused launch gives the same bits as the three stages launched one after another.
//       complex rope : (x[2i] + j x[2i+1]) * (c_i + j s_i), c/s fp32 pairs per position   (q and k)
//       L2 norm      : x * rsqrt(mean(x^2) + eps)                                          (q and k)
//       temperature  : q * (log1p(floor((pos + 1) / floor_scale)) * attn_scale + 1)        (q only)
//   * sliding-window KV cache update in the three modes of the reference (first fill, in-place scatter while the
//     window is not full, shift-by-new-rows into a second buffer once it is), rows kept in chronological order.
//   * sum over one dimension ([B, M, N] -> [B, N]), fp32 accumulation.
//   * append-next-token + stopping criteria on int64 token buffers.
// All of it is launch-latency work: a few KiB per call.
#include "common.cuh"

MUI_STATUS_ACCESSOR(llama4)

namespace {

constexpr int PRO_WARPS = 4;

struct PrologueArgs {
  const void *q_in, *k_in;
  void *q_out, *k_out;
  const float* pos_embeds;        // [B, T, D/2, 2] (cos, sin) or null
  const int64_t* pos_index;       // optional [B, T]: pos_embeds is then a table [positions, D/2, 2] indexed by it
  const int64_t* cache_position;  // [T] or null
  mui_strides3_t qs, ks;
  int B, T, Hq, Hk, D;
  int do_rope, do_norm, do_temp;
  float eps, attn_scale, floor_scale;
};

// D <= 256: every lane holds up to 4 (even, odd) pairs
template <typename T>
__global__ void __launch_bounds__(PRO_WARPS * 32) qk_prologue_kernel(const PrologueArgs a) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = a.Hq + a.Hk;
  const long long row = (long long)blockIdx.x * PRO_WARPS + warp;
  if (row >= (long long)heads_total * a.T * a.B) return;
  int head = static_cast<int>(row % heads_total);
  const long long bt = row / heads_total;
  const int t = static_cast<int>(bt % a.T), b = static_cast<int>(bt / a.T);
  const int D = a.D, pairs = D >> 1;
  const bool is_q = head < a.Hq;
  const T* in;
  T* out;
  if (is_q) {
    in = reinterpret_cast<const T*>(a.q_in) + b * a.qs.batch + head * a.qs.head + t * a.qs.tok;
    out = reinterpret_cast<T*>(a.q_out) + (((size_t)b * a.Hq + head) * a.T + t) * D;
  } else {
    head -= a.Hq;
    in = reinterpret_cast<const T*>(a.k_in) + b * a.ks.batch + head * a.ks.head + t * a.ks.tok;
    out = reinterpret_cast<T*>(a.k_out) + (((size_t)b * a.Hk + head) * a.T + t) * D;
  }
  float re[4], im[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = lane + 32 * j;
    re[j] = im[j] = 0.f;
    if (p < pairs) {
      re[j] = ld_act_f32<T>(in + 2 * p);
      im[j] = ld_act_f32<T>(in + 2 * p + 1);
    }
  }
  if (a.do_rope) {
    const size_t prow = a.pos_index ? static_cast<size_t>(__ldcg(a.pos_index + (size_t)b * a.T + t))
                                    : ((size_t)b * a.T + t);
    const float2* cs = reinterpret_cast<const float2*>(a.pos_embeds) + prow * pairs;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = lane + 32 * j;
      if (p < pairs) {
        const float2 c = cs[p];
        const float r = re[j] * c.x - im[j] * c.y;
        const float i = re[j] * c.y + im[j] * c.x;
        re[j] = Elt<T>::to_f32(Elt<T>::from_f32(r));
        im[j] = Elt<T>::to_f32(Elt<T>::from_f32(i));
      }
    }
  }
  if (a.do_norm) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += re[j] * re[j] + im[j] * im[j];
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / static_cast<float>(D) + a.eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      re[j] = Elt<T>::to_f32(Elt<T>::from_f32(re[j] * r));
      im[j] = Elt<T>::to_f32(Elt<T>::from_f32(im[j] * r));
    }
  }
  if (a.do_temp && is_q) {
    const float pos = static_cast<float>(__ldcg(a.cache_position + t));
    const float s = log1pf(floorf((pos + 1.0f) / a.floor_scale)) * a.attn_scale + 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      re[j] *= s;
      im[j] *= s;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = lane + 32 * j;
    if (p < pairs) {
      out[2 * p] = Elt<T>::from_f32(re[j]);
      out[2 * p + 1] = Elt<T>::from_f32(im[j]);
    }
  }
}

mui_status_t launch_prologue(cudaStream_t stream, mui_dtype_t dtype, const PrologueArgs& a, unsigned flags) {
  const long long rows = (long long)(a.Hq + a.Hk) * a.T * a.B;
  if (rows == 0) return MUI_OK;
  const int grid = static_cast<int>((rows + PRO_WARPS - 1) / PRO_WARPS);
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(qk_prologue_kernel<__half>, dim3(grid), dim3(PRO_WARPS * 32), 0, stream, pdl, a));
  } else {
    MUI_CUDA_CHECK(mui_launch(qk_prologue_kernel<__nv_bfloat16>, dim3(grid), dim3(PRO_WARPS * 32), 0, stream, pdl, a));
  }
  return MUI_OK;
}

mui_status_t check_prologue_sizes(mui_dtype_t dtype, int B, int T, int Hq, int Hk, int D) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(B >= 0 && T >= 0 && Hq >= 0 && Hk >= 0, MUI_ERR_INVALID_ARG, "bad sizes B=%d T=%d Hq=%d Hk=%d", B, T, Hq,
              Hk);
  MUI_REQUIRE(D >= 2 && (D & 1) == 0 && D <= 256, MUI_ERR_UNSUPPORTED, "head dim %d must be even and at most 256", D);
  return MUI_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// sliding-window cache

struct SlideArgs {
  const uint16_t *k_in, *v_in, *k_cache_in, *v_cache_in;
  uint16_t *k_cache_out, *v_cache_out;
  const int64_t* cache_position;
  mui_strides3_t ks, vs;
  int B, T, max_T, Hk, Hv, D;
  int mode;      // 0 first fill, 1 shift into the second buffer, 2 scatter in place
  int start_t;   // first copied new token (T - min(T, max_T))
  int rows_out;  // rows written per (batch, head)
};

// one warp per output row (head, row, batch); 16-bit elements moved as raw bits
__global__ void __launch_bounds__(PRO_WARPS * 32) sliding_cache_kernel(const SlideArgs a) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = a.Hk + a.Hv;
  const long long row = (long long)blockIdx.x * PRO_WARPS + warp;
  if (row >= (long long)heads_total * a.rows_out * a.B) return;
  int head = static_cast<int>(row % heads_total);
  const long long br = row / heads_total;
  const int r = static_cast<int>(br % a.rows_out), b = static_cast<int>(br / a.rows_out);
  const bool is_k = head < a.Hk;
  const int H = is_k ? a.Hk : a.Hv;
  if (!is_k) head -= a.Hk;
  const uint16_t* in_new = is_k ? a.k_in : a.v_in;
  const mui_strides3_t st = is_k ? a.ks : a.vs;
  const uint16_t* cache_in = is_k ? a.k_cache_in : a.v_cache_in;
  uint16_t* cache_out = is_k ? a.k_cache_out : a.v_cache_out;
  const size_t cache_row0 = ((size_t)b * H + head) * a.max_T;
  const uint16_t* src;
  size_t dst_row;
  if (a.mode == 0) {
    src = in_new + b * st.batch + head * st.head + (long long)(r + a.start_t) * st.tok;
    dst_row = cache_row0 + r;
  } else if (a.mode == 1) {
    const int n_new = a.T - a.start_t, n_old = a.max_T - n_new;
    if (r >= n_old) {
      src = in_new + b * st.batch + head * st.head + (long long)(r - n_old + a.start_t) * st.tok;
    } else {
      src = cache_in + (cache_row0 + r + n_new) * a.D;
    }
    dst_row = cache_row0 + r;
  } else {
    src = in_new + b * st.batch + head * st.head + (long long)r * st.tok;
    dst_row = cache_row0 + static_cast<size_t>(__ldcg(a.cache_position + r));
  }
  uint16_t* dst = cache_out + dst_row * a.D;
  for (int i = lane; i < a.D; i += 32) dst[i] = __ldcg(src + i);
}

// ---------------------------------------------------------------------------------------------------------------
// sum over the middle dimension of [B, M, N]

template <typename T>
__global__ void __launch_bounds__(256) reduce_sum_kernel(const T* __restrict__ x, T* __restrict__ y, int M,
                                                         long long N, long long total) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long b = i / N, n = i % N;
  const T* p = x + (size_t)b * M * N + n;
  float acc = 0.f;
  for (int m = 0; m < M; ++m) acc += ld_act_f32<T>(p + (size_t)m * N);
  y[i] = Elt<T>::from_f32(acc);
}

// sum over the last dimension: one warp per row of [R, M]
template <typename T>
__global__ void __launch_bounds__(128) reduce_sum_last_kernel(const T* __restrict__ x, T* __restrict__ y, int M,
                                                              long long R) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const long long r = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= R) return;
  const int lane = threadIdx.x & 31;
  float acc = 0.f;
  for (int m = lane; m < M; m += 32) acc += ld_act_f32<T>(x + (size_t)r * M + m);
  acc = warp_sum(acc);
  if (lane == 0) y[r] = Elt<T>::from_f32(acc);
}

// ---------------------------------------------------------------------------------------------------------------
// token bookkeeping of a generation loop

struct AddTokArgs {
  const int64_t* input_ids;     // [B, T]
  const int32_t* next_tokens;   // [B]
  const int64_t* unfinished;    // [B]
  const int64_t* eos_ids;       // [n_eos]
  int64_t* next_input_ids;      // [B, T + 1]
  int64_t* next_unfinished;     // [B]
  long long max_length, pad_token_id;
  int B, T, n_eos, has_eos, has_max_length;
};

__global__ void __launch_bounds__(256) add_tokens_kernel(const AddTokArgs a) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int64_t* src = a.input_ids + (size_t)b * a.T;
  int64_t* dst = a.next_input_ids + (size_t)b * (a.T + 1);
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < a.T; t += gridDim.x * blockDim.x) dst[t] = __ldcg(src + t);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const bool prev = __ldcg(a.unfinished + b) != 0;
    long long tok = __ldcg(a.next_tokens + b);
    if (a.has_eos && !prev) tok = a.pad_token_id;
    dst[a.T] = tok;
    bool unfinished = prev;
    if (a.has_max_length) unfinished = unfinished && (a.T + 1 < a.max_length);
    if (a.has_eos) {
      bool is_eos = false;
      for (int i = 0; i < a.n_eos; ++i) is_eos = is_eos || (tok == a.eos_ids[i]);
      unfinished = unfinished && !is_eos;
    }
    a.next_unfinished[b] = unfinished ? 1 : 0;
  }
}

}  // namespace

extern "C" {

mui_status_t mui_complex_rope_forward(void* stream, mui_dtype_t dtype, int B, int T, int Hq, int Hk, int D,
                                      const float* position_embeds, const void* q_in, mui_strides3_t q_strides,
                                      const void* k_in, mui_strides3_t k_strides, void* q_out, void* k_out,
                                      unsigned flags) {
  if (mui_status_t s = check_prologue_sizes(dtype, B, T, Hq, Hk, D)) return s;
  MUI_REQUIRE(position_embeds, MUI_ERR_INVALID_ARG, "position_embeds must be non-null");
  MUI_REQUIRE((Hq == 0 || (q_in && q_out)) && (Hk == 0 || (k_in && k_out)), MUI_ERR_INVALID_ARG,
              "q/k inputs and outputs must be non-null");
  PrologueArgs a{};
  a.q_in = q_in; a.k_in = k_in; a.q_out = q_out; a.k_out = k_out;
  a.pos_embeds = position_embeds;
  a.qs = q_strides; a.ks = k_strides;
  a.B = B; a.T = T; a.Hq = Hq; a.Hk = Hk; a.D = D;
  a.do_rope = 1;
  return launch_prologue(static_cast<cudaStream_t>(stream), dtype, a, flags);
}

mui_status_t mui_qkl2norm_forward(void* stream, mui_dtype_t dtype, long long rows_q, long long rows_k, int D,
                                  const void* q, const void* k, void* q_out, void* k_out, float eps,
                                  unsigned flags) {
  if (mui_status_t s = check_prologue_sizes(dtype, 1, 1, 0, 0, D)) return s;
  MUI_REQUIRE(rows_q >= 0 && rows_k >= 0 && rows_q + rows_k < (1ll << 31), MUI_ERR_INVALID_ARG, "bad row counts");
  MUI_REQUIRE((rows_q == 0 || (q && q_out)) && (rows_k == 0 || (k && k_out)), MUI_ERR_INVALID_ARG,
              "inputs and outputs must be non-null");
  // contiguous rows: treat every row as one head of a single (batch, token)
  PrologueArgs a{};
  a.q_in = q; a.k_in = k; a.q_out = q_out; a.k_out = k_out;
  a.qs = mui_strides3_t{0, D, 0};
  a.ks = mui_strides3_t{0, D, 0};
  a.B = 1; a.T = 1; a.Hq = static_cast<int>(rows_q); a.Hk = static_cast<int>(rows_k); a.D = D;
  a.do_norm = 1; a.eps = eps;
  return launch_prologue(static_cast<cudaStream_t>(stream), dtype, a, flags);
}

mui_status_t mui_temperature_tuning_forward(void* stream, mui_dtype_t dtype, int B, int T, int H, int D,
                                            const void* q_in, mui_strides3_t q_strides,
                                            const int64_t* cache_position, void* q_out, float attn_scale,
                                            float floor_scale, unsigned flags) {
  if (mui_status_t s = check_prologue_sizes(dtype, B, T, H, 0, D)) return s;
  MUI_REQUIRE(H == 0 || (q_in && q_out), MUI_ERR_INVALID_ARG, "q_in and q_out must be non-null");
  MUI_REQUIRE(cache_position, MUI_ERR_INVALID_ARG, "cache_position must be non-null");
  MUI_REQUIRE(floor_scale > 0.f, MUI_ERR_INVALID_ARG, "floor_scale must be positive");
  PrologueArgs a{};
  a.q_in = q_in; a.q_out = q_out; a.qs = q_strides;
  a.cache_position = cache_position;
  a.B = B; a.T = T; a.Hq = H; a.Hk = 0; a.D = D;
  a.do_temp = 1; a.attn_scale = attn_scale; a.floor_scale = floor_scale;
  return launch_prologue(static_cast<cudaStream_t>(stream), dtype, a, flags);
}

mui_status_t mui_llama4_qk_prologue(void* stream, mui_dtype_t dtype, int B, int T, int Hq, int Hk, int D,
                                    const float* position_embeds, int use_qk_norm, float norm_eps,
                                    const int64_t* cache_position, float attn_scale, float floor_scale,
                                    const void* q_in, mui_strides3_t q_strides, const void* k_in,
                                    mui_strides3_t k_strides, void* q_out, void* k_out, unsigned flags) {
  if (mui_status_t s = check_prologue_sizes(dtype, B, T, Hq, Hk, D)) return s;
  MUI_REQUIRE((Hq == 0 || (q_in && q_out)) && (Hk == 0 || (k_in && k_out)), MUI_ERR_INVALID_ARG,
              "q/k inputs and outputs must be non-null");
  MUI_REQUIRE(!cache_position || floor_scale > 0.f, MUI_ERR_INVALID_ARG, "floor_scale must be positive");
  PrologueArgs a{};
  a.q_in = q_in; a.k_in = k_in; a.q_out = q_out; a.k_out = k_out;
  a.pos_embeds = position_embeds; a.cache_position = cache_position;
  a.qs = q_strides; a.ks = k_strides;
  a.B = B; a.T = T; a.Hq = Hq; a.Hk = Hk; a.D = D;
  a.do_rope = position_embeds ? 1 : 0;
  a.do_norm = use_qk_norm ? 1 : 0;
  a.do_temp = cache_position ? 1 : 0;
  a.eps = norm_eps; a.attn_scale = attn_scale; a.floor_scale = floor_scale;
  return launch_prologue(static_cast<cudaStream_t>(stream), dtype, a, flags);
}

}  // extern "C"

// Decode-stack use: the rotation angles come from the table row position_ids[b * T + t] (device side), so the launch
// can be captured and replayed.
mui_status_t mui_llama4_qk_prologue_indexed(cudaStream_t stream, mui_dtype_t dtype, int B, int T, int Hq, int Hk, int D,
                                            const float* freqs_table, const int64_t* position_ids, int use_rope,
                                            int use_qk_norm, float norm_eps, const int64_t* cache_position,
                                            float attn_scale, float floor_scale, const void* q_in,
                                            mui_strides3_t q_strides, const void* k_in, mui_strides3_t k_strides,
                                            void* q_out, void* k_out, unsigned flags) {
  if (mui_status_t s = check_prologue_sizes(dtype, B, T, Hq, Hk, D)) return s;
  PrologueArgs a{};
  a.q_in = q_in; a.k_in = k_in; a.q_out = q_out; a.k_out = k_out;
  a.pos_embeds = use_rope ? freqs_table : nullptr;
  a.pos_index = position_ids;
  a.cache_position = cache_position;
  a.qs = q_strides; a.ks = k_strides;
  a.B = B; a.T = T; a.Hq = Hq; a.Hk = Hk; a.D = D;
  a.do_rope = use_rope ? 1 : 0;
  a.do_norm = use_qk_norm ? 1 : 0;
  a.do_temp = cache_position ? 1 : 0;
  a.eps = norm_eps; a.attn_scale = attn_scale; a.floor_scale = floor_scale;
  return launch_prologue(stream, dtype, a, flags);
}

extern "C" {

mui_status_t mui_sliding_kvcache_update(void* stream, mui_dtype_t dtype, int B, int T, int max_T, int Hk, int Hv,
                                        int D, const void* k_in, mui_strides3_t k_strides, const void* v_in,
                                        mui_strides3_t v_strides, void* k_cache, void* v_cache, void* k_cache_out,
                                        void* v_cache_out, const int64_t* cache_position, long long seen_tokens,
                                        int* mode_out, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(B >= 0 && T >= 0 && max_T >= 1 && Hk >= 0 && Hv >= 0 && D >= 1, MUI_ERR_INVALID_ARG,
              "bad sizes B=%d T=%d max_T=%d Hk=%d Hv=%d D=%d", B, T, max_T, Hk, Hv, D);
  MUI_REQUIRE(seen_tokens >= T, MUI_ERR_INVALID_ARG, "seen_tokens (%lld) counts the %d new tokens too", seen_tokens, T);
  MUI_REQUIRE(k_in && v_in && k_cache && v_cache, MUI_ERR_INVALID_ARG, "k/v inputs and caches must be non-null");
  SlideArgs a{};
  a.k_in = static_cast<const uint16_t*>(k_in); a.v_in = static_cast<const uint16_t*>(v_in);
  a.ks = k_strides; a.vs = v_strides;
  a.B = B; a.T = T; a.max_T = max_T; a.Hk = Hk; a.Hv = Hv; a.D = D;
  a.start_t = T < max_T ? 0 : T - max_T;
  a.cache_position = cache_position;
  if (seen_tokens == T) {
    a.mode = 0;
    a.k_cache_out = static_cast<uint16_t*>(k_cache); a.v_cache_out = static_cast<uint16_t*>(v_cache);
    a.rows_out = T < max_T ? T : max_T;
  } else if (seen_tokens > max_T) {
    MUI_REQUIRE(k_cache_out && v_cache_out && k_cache_out != k_cache && v_cache_out != v_cache, MUI_ERR_INVALID_ARG,
                "a full window shifts into a second pair of buffers: k_cache_out / v_cache_out must be given");
    a.mode = 1;
    a.k_cache_in = static_cast<const uint16_t*>(k_cache); a.v_cache_in = static_cast<const uint16_t*>(v_cache);
    a.k_cache_out = static_cast<uint16_t*>(k_cache_out); a.v_cache_out = static_cast<uint16_t*>(v_cache_out);
    a.rows_out = max_T;
  } else {
    MUI_REQUIRE(cache_position, MUI_ERR_INVALID_ARG, "cache_position must be non-null");
    a.mode = 2;
    a.k_cache_out = static_cast<uint16_t*>(k_cache); a.v_cache_out = static_cast<uint16_t*>(v_cache);
    a.rows_out = T;
  }
  if (mode_out) *mode_out = a.mode;
  const long long rows = (long long)(Hk + Hv) * a.rows_out * B;
  if (rows == 0) return MUI_OK;
  const int grid = static_cast<int>((rows + PRO_WARPS - 1) / PRO_WARPS);
  MUI_CUDA_CHECK(mui_launch(sliding_cache_kernel, dim3(grid), dim3(PRO_WARPS * 32), 0,
                            static_cast<cudaStream_t>(stream), (flags & MUI_FLAG_PDL) ? 1 : 0, a));
  return MUI_OK;
}

mui_status_t mui_reduce_sum_forward(void* stream, mui_dtype_t dtype, long long B, int M, long long N, const void* x,
                                    void* y, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(B >= 0 && M >= 0 && N >= 0, MUI_ERR_INVALID_ARG, "bad sizes");
  const long long total = B * N;
  if (total == 0) return MUI_OK;
  MUI_REQUIRE(x && y, MUI_ERR_INVALID_ARG, "x and y must be non-null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  if (N == 1) {
    const int grid = static_cast<int>((B + 3) / 4);
    if (dtype == MUI_F16) {
      MUI_CUDA_CHECK(mui_launch(reduce_sum_last_kernel<__half>, dim3(grid), dim3(128), 0, st, pdl,
                                static_cast<const __half*>(x), static_cast<__half*>(y), M, B));
    } else {
      MUI_CUDA_CHECK(mui_launch(reduce_sum_last_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, st, pdl,
                                static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), M, B));
    }
    return MUI_OK;
  }
  const int grid = static_cast<int>((total + 255) / 256);
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(reduce_sum_kernel<__half>, dim3(grid), dim3(256), 0, st, pdl,
                              static_cast<const __half*>(x), static_cast<__half*>(y), M, N, total));
  } else {
    MUI_CUDA_CHECK(mui_launch(reduce_sum_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, pdl,
                              static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), M, N, total));
  }
  return MUI_OK;
}

mui_status_t mui_add_tokens_check_finished(void* stream, int B, int T, const int64_t* input_ids,
                                           const int32_t* next_tokens, const int64_t* unfinished_sequences,
                                           int has_eos_stopping_criteria, long long pad_token_id,
                                           const int64_t* eos_token_ids, int num_eos_tokens,
                                           int has_max_length_stopping_criteria, long long max_length,
                                           int64_t* next_input_ids, int64_t* next_unfinished_sequences,
                                           unsigned flags) {
  MUI_REQUIRE(B >= 0 && T >= 0 && num_eos_tokens >= 0, MUI_ERR_INVALID_ARG, "bad sizes B=%d T=%d", B, T);
  if (B == 0) return MUI_OK;
  MUI_REQUIRE((T == 0 || input_ids) && next_tokens && unfinished_sequences && next_input_ids &&
                  next_unfinished_sequences, MUI_ERR_INVALID_ARG, "token buffers must be non-null");
  MUI_REQUIRE(!has_eos_stopping_criteria || num_eos_tokens == 0 || eos_token_ids, MUI_ERR_INVALID_ARG,
              "eos_token_ids must be non-null");
  AddTokArgs a{};
  a.input_ids = input_ids; a.next_tokens = next_tokens; a.unfinished = unfinished_sequences; a.eos_ids = eos_token_ids;
  a.next_input_ids = next_input_ids; a.next_unfinished = next_unfinished_sequences;
  a.max_length = max_length; a.pad_token_id = pad_token_id;
  a.B = B; a.T = T; a.n_eos = num_eos_tokens;
  a.has_eos = has_eos_stopping_criteria ? 1 : 0;
  a.has_max_length = has_max_length_stopping_criteria ? 1 : 0;
  int gx = (T + 255) / 256;
  gx = gx < 1 ? 1 : (gx > 64 ? 64 : gx);
  MUI_CUDA_CHECK(mui_launch(add_tokens_kernel, dim3(gx, B), dim3(256), 0, static_cast<cudaStream_t>(stream),
                            (flags & MUI_FLAG_PDL) ? 1 : 0, a));
  return MUI_OK;
}

}  // extern "C"
