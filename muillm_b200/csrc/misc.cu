// Small kernels around the decode step: embedding row gather, greedy arg-max with the device-side
// bookkeeping that lets a whole decode step replay from a CUDA graph (positions, sequence length and the
// token fed to the next step all live in device memory).
#include "common.cuh"

MUI_STATUS_ACCESSOR(misc)

namespace {

// one CTA copies one embedding row of 16-bit elements (csrc/embedding/embedding_xx16_kernels.cu:26,74)
__global__ void __launch_bounds__(256) embedding_kernel(const uint16_t* __restrict__ table,
                                                        const int64_t* __restrict__ tokens,
                                                        uint16_t* __restrict__ out, int H, int vocab) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  long long tok = __ldcg(tokens + blockIdx.x);
  if (tok < 0) tok = 0;
  if (tok >= vocab) tok = vocab - 1;
  const uint16_t* src = table + (size_t)tok * H;
  uint16_t* dst = out + (size_t)blockIdx.x * H;
  const bool vec_ok = ((H & 7) == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
  if (vec_ok) {
    for (int i = threadIdx.x * 8; i < H; i += 256 * 8)
      *reinterpret_cast<uint4*>(dst + i) = ld_cached16(src + i);
  } else {
    for (int i = threadIdx.x; i < H; i += 256) dst[i] = src[i];
  }
}

constexpr int ARGMAX_THREADS = 1024;

// One CTA per row: arg-max over V 16-bit logits, lowest index wins ties. Then (thread 0 of row 0) advances
// the decode state. state layout (int64 words): [0] step, [1] tokens in the cache before the step,
// [2] cache_position (row this step wrote), [3..3+B) position_ids, [3+B..3+2B) tokens fed to the step.
template <typename T>
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_advance_kernel(const T* __restrict__ logits, int V, int B,
                                                                        long long* __restrict__ state,
                                                                        int32_t* __restrict__ seq_len32,
                                                                        long long* __restrict__ out_tokens,
                                                                        int out_capacity) {
  __shared__ float s_val[ARGMAX_THREADS / 32];
  __shared__ int s_idx[ARGMAX_THREADS / 32];
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* row = logits + (size_t)b * V;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < V; i += ARGMAX_THREADS) {
    const float v = ld_act_f32<T>(row + i);
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(MUI_FULL_MASK, best, o);
    const int oi = __shfl_xor_sync(MUI_FULL_MASK, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < ARGMAX_THREADS / 32; ++w) {
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) {
        best = s_val[w];
        best_i = s_idx[w];
      }
    }
    if (best_i == 0x7fffffff) best_i = 0;  // all NaN / empty
    const long long step = __ldcg(state);
    state[3 + B + b] = best_i;  // token fed to the next step
    if (out_tokens != nullptr && step < out_capacity) out_tokens[step * B + b] = best_i;
    state[3 + b] = __ldcg(state + 3 + b) + 1;  // position id of this sequence
    if (b == 0) {
      const long long in_cache = __ldcg(state + 1) + 1;
      state[0] = step + 1;
      state[1] = in_cache;
      state[2] = __ldcg(state + 2) + 1;
      *seq_len32 = static_cast<int32_t>(in_cache + 1);  // the next step attends its own new token too
    }
  }
}

}  // namespace

mui_status_t mui_launch_embedding(cudaStream_t stream, const void* table, const int64_t* tokens, void* out, int B,
                                  int H, int vocab, int pdl) {
  MUI_CUDA_CHECK(mui_launch(embedding_kernel, dim3(B), dim3(256), 0, stream, pdl, (const uint16_t*)table, tokens,
                            (uint16_t*)out, H, vocab));
  return MUI_OK;
}

mui_status_t mui_launch_argmax_advance(cudaStream_t stream, mui_dtype_t dtype, const void* logits, int V, int B,
                                       long long* state, int32_t* seq_len32, long long* out_tokens, int out_capacity,
                                       int pdl) {
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(argmax_advance_kernel<__half>, dim3(B), dim3(ARGMAX_THREADS), 0, stream, pdl,
                              (const __half*)logits, V, B, state, seq_len32, out_tokens, out_capacity));
  } else {
    MUI_CUDA_CHECK(mui_launch(argmax_advance_kernel<__nv_bfloat16>, dim3(B), dim3(ARGMAX_THREADS), 0, stream, pdl,
                              (const __nv_bfloat16*)logits, V, B, state, seq_len32, out_tokens, out_capacity));
  }
  return MUI_OK;
}

extern "C" mui_status_t mui_embedding_forward(void* stream, mui_dtype_t dtype, int num_tokens, int H, int vocab,
                                              const void* table, const int64_t* token_ids, void* out,
                                              unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(num_tokens >= 0 && H >= 1 && vocab >= 1, MUI_ERR_INVALID_ARG, "bad sizes");
  if (num_tokens == 0) return MUI_OK;
  MUI_REQUIRE(table && token_ids && out, MUI_ERR_INVALID_ARG, "null pointer");
  return mui_launch_embedding((cudaStream_t)stream, table, token_ids, out, num_tokens, H, vocab,
                              (flags & MUI_FLAG_PDL) ? 1 : 0);
}
