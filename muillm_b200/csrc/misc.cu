// Small kernels around the decode step: embedding row gather, greedy arg-max with the device-side
// bookkeeping that lets a whole decode step replay from a CUDA graph (positions, sequence length and the
// token fed to the next step all live in device memory).
#include "comm_dev.cuh"

#include <cstring>

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

constexpr int ARGMAX_THREADS = 256;
constexpr int ARGMAX_CTAS = 32;  // CTAs per row

__device__ __forceinline__ bool argmax_better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

// ARGMAX_CTAS CTAs per row scan slices of the V 16-bit logits (16-byte loads); lowest index wins ties. Each
// CTA leaves its (value, index) in `partials`; the last CTA of the launch to arrive (arrival counter in
// `counters[0]`, left at zero again) picks every row's winner and advances the decode state.
// state layout (int64 words): [0] step, [1] tokens in the cache before the step, [2] cache_position (row this
// step wrote), [3..3+B) position_ids, [3+B..3+2B) tokens fed to the step.
template <typename T>
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_advance_kernel(const T* logits, int V, int B,
                                                                        long long* state, int32_t* seq_len32,
                                                                        long long* out_tokens, int out_capacity,
                                                                        float* partial_val, int* partial_idx,
                                                                        unsigned int* counters, int use_comm,
                                                                        int index_offset, const CommDev comm) {
  __shared__ float s_val[ARGMAX_THREADS / 32];
  __shared__ int s_idx[ARGMAX_THREADS / 32];
  __shared__ int s_last;
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* row = logits + (size_t)b * V;
  // slice of this CTA, in units of 8 elements
  const int vec_total = V >> 3;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  if (vec_ok) {
    const int v_begin = static_cast<int>((long long)vec_total * blockIdx.x / gridDim.x);
    const int v_end = static_cast<int>((long long)vec_total * (blockIdx.x + 1) / gridDim.x);
    for (int v = v_begin + tid; v < v_end; v += ARGMAX_THREADS) {
      float f[8];
      unpack8<T>(ld_act16(row + (size_t)v * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (argmax_better(f[i], v * 8 + i, best, best_i)) {
          best = f[i];
          best_i = v * 8 + i;
        }
    }
    if (blockIdx.x == gridDim.x - 1)  // tail elements
      for (int i = vec_total * 8 + tid; i < V; i += ARGMAX_THREADS) {
        const float v = ld_act_f32<T>(row + i);
        if (argmax_better(v, i, best, best_i)) {
          best = v;
          best_i = i;
        }
      }
  } else {
    const int e_begin = static_cast<int>((long long)V * blockIdx.x / gridDim.x);
    const int e_end = static_cast<int>((long long)V * (blockIdx.x + 1) / gridDim.x);
    for (int i = e_begin + tid; i < e_end; i += ARGMAX_THREADS) {
      const float v = ld_act_f32<T>(row + i);
      if (argmax_better(v, i, best, best_i)) {
        best = v;
        best_i = i;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(MUI_FULL_MASK, best, o);
    const int oi = __shfl_xor_sync(MUI_FULL_MASK, best_i, o);
    if (argmax_better(ov, oi, best, best_i)) {
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
    for (int w = 1; w < ARGMAX_THREADS / 32; ++w)
      if (argmax_better(s_val[w], s_idx[w], best, best_i)) {
        best = s_val[w];
        best_i = s_idx[w];
      }
    partial_val[b * gridDim.x + blockIdx.x] = best;
    partial_idx[b * gridDim.x + blockIdx.x] = best_i;
    __threadfence();
    const unsigned prev = atomicAdd(&counters[0], 1u);
    s_last = (prev == gridDim.x * gridDim.y - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  // the last CTA of the whole launch finishes every row (warp w takes row w; B <= 8 warps)
  __threadfence();
  const long long step = __ldcg(state);
  const unsigned long long comm_seq = use_comm ? comm_begin(comm) : 0ull;
  if (warp < B) {
    const int r = warp;
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (int c = lane; c < (int)gridDim.x; c += 32) {
      const float v = __ldcg(partial_val + r * gridDim.x + c);
      const int i = __ldcg(partial_idx + r * gridDim.x + c);
      if (argmax_better(v, i, best, best_i)) {
        best = v;
        best_i = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(MUI_FULL_MASK, best, o);
      const int oi = __shfl_xor_sync(MUI_FULL_MASK, best_i, o);
      if (argmax_better(ov, oi, best, best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (best_i == 0x7fffffff) best_i = 0;  // all NaN / empty
    best_i += index_offset;                // rows of a vocabulary shard -> global token id
    if (use_comm) {
      // tensor-parallel lm_head sharded by rows: exchange each rank's (value, token) pair and keep the best
      // (lowest token id on ties) — every rank picks the same winner
      if (lane == 0) {
        comm_push(comm, comm_seq, 2 * r, best);
        comm_push(comm, comm_seq, 2 * r + 1, __int_as_float(best_i));
      }
      float gv = -INFINITY;
      int gi = 0x7fffffff;
      if (lane < comm.world) {
        float v = -INFINITY, fi = 0.f;
        if (comm_take(comm, comm_seq, lane, 2 * r, &v) && comm_take(comm, comm_seq, lane, 2 * r + 1, &fi)) {
          gv = v;
          gi = __float_as_int(fi);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(MUI_FULL_MASK, gv, o);
        const int oi = __shfl_xor_sync(MUI_FULL_MASK, gi, o);
        if (argmax_better(ov, oi, gv, gi)) {
          gv = ov;
          gi = oi;
        }
      }
      best_i = (gi == 0x7fffffff) ? 0 : gi;
    }
    if (lane == 0) {
      state[3 + B + r] = best_i;             // token fed to the next step
      if (out_tokens != nullptr && step < out_capacity) out_tokens[step * B + r] = best_i;
      state[3 + r] = __ldcg(state + 3 + r) + 1;  // position id of this sequence
    }
  }
  __syncthreads();  // every warp has read `step` before it moves
  if (tid == 0) {
    counters[0] = 0u;
    if (use_comm) comm_cta_done(comm, comm_seq, 1);
    const long long in_cache = __ldcg(state + 1) + 1;
    state[0] = step + 1;
    state[1] = in_cache;
    state[2] = __ldcg(state + 2) + 1;
    *seq_len32 = static_cast<int32_t>(in_cache + 1);  // the next step attends its own new token too
  }
}

}  // namespace

mui_status_t mui_launch_embedding(cudaStream_t stream, const void* table, const int64_t* tokens, void* out, int B,
                                  int H, int vocab, int pdl) {
  MUI_CUDA_CHECK(mui_launch(embedding_kernel, dim3(B), dim3(256), 0, stream, pdl, (const uint16_t*)table, tokens,
                            (uint16_t*)out, H, vocab));
  return MUI_OK;
}

// `work`: device scratch of mui_argmax_work_bytes(B) bytes whose first 64 bytes (arrival counters) are zero
// before the first call; every call leaves them zero.
size_t mui_argmax_work_bytes(int B) { return 64 + (size_t)B * ARGMAX_CTAS * 8; }

mui_status_t mui_launch_argmax_advance(cudaStream_t stream, mui_dtype_t dtype, const void* logits, int V, int B,
                                       long long* state, int32_t* seq_len32, long long* out_tokens, int out_capacity,
                                       void* work, int pdl, const CommDev* comm, int index_offset) {
  unsigned int* counters = reinterpret_cast<unsigned int*>(work);
  float* pval = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(work) + 64);
  int* pidx = reinterpret_cast<int*>(pval + (size_t)B * ARGMAX_CTAS);
  const dim3 grid(ARGMAX_CTAS, B);
  CommDev cd;
  memset(&cd, 0, sizeof(cd));
  const int use_comm = (comm != nullptr && comm->world > 1) ? 1 : 0;
  if (use_comm) cd = *comm;
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(argmax_advance_kernel<__half>, grid, dim3(ARGMAX_THREADS), 0, stream, pdl,
                              (const __half*)logits, V, B, state, seq_len32, out_tokens, out_capacity, pval, pidx,
                              counters, use_comm, index_offset, cd));
  } else {
    MUI_CUDA_CHECK(mui_launch(argmax_advance_kernel<__nv_bfloat16>, grid, dim3(ARGMAX_THREADS), 0, stream, pdl,
                              (const __nv_bfloat16*)logits, V, B, state, seq_len32, out_tokens, out_capacity, pval,
                              pidx, counters, use_comm, index_offset, cd));
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
