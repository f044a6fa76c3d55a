// Router top-k + sigmoid, and the MoE MLP entry point built on the GEMV kernels' device-side expert
// addressing (shared experts first, then the routed ones picked by router_indices).
#include "gemv_common.cuh"

#include <cstring>

MUI_STATUS_ACCESSOR(moe)

mui_status_t mui_launch_gemv16(cudaStream_t stream, mui_dtype_t dtype, int mode, const GemvArgs& a, unsigned flags);

namespace {

constexpr int TOPK_THREADS = 256;
constexpr int TOPK_MAX_M = 4096;
constexpr int TOPK_MAX_K = 32;

// One CTA per row of logits [rows, M]: k rounds of a block-wide arg-max over the not-yet-taken entries
// (lowest index wins ties, like a stable descending sort), sigmoid of the winners in fp32.
// Replaces muillm_max_sigmoid_fp16_kernel / muillm_topk_sigmoid_fp16_kernel (csrc/topk/topk_fp16_kernels.cu:60,95);
// unlike the reference's k == 1 kernel it is correct for any M <= 4096, not only M <= warp size.
template <typename T>
__global__ void __launch_bounds__(TOPK_THREADS) topk_sigmoid_kernel(const T* logits, T* values, long long* indices,
                                                                    int M, int k) {
  __shared__ float s_logit[TOPK_MAX_M];
  __shared__ float s_val[TOPK_THREADS / 32];
  __shared__ int s_idx[TOPK_THREADS / 32];
  __shared__ int s_winner;
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* row = logits + (size_t)blockIdx.x * M;
  for (int i = tid; i < M; i += TOPK_THREADS) s_logit[i] = ld_act_f32<T>(row + i);
  __syncthreads();
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < M; i += TOPK_THREADS) {
      const float v = s_logit[i];
      // taken entries are marked NaN; NaN never compares greater
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
      for (int w = 1; w < TOPK_THREADS / 32; ++w)
        if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) {
          best = s_val[w];
          best_i = s_idx[w];
        }
      if (best_i == 0x7fffffff) {  // only -inf / NaN left: take the lowest untaken index
        best_i = 0;
        for (int i = 0; i < M; ++i)
          if (!(s_logit[i] != s_logit[i])) {
            best_i = i;
            break;
          }
        best = s_logit[best_i];
      }
      const float sg = 1.f / (1.f + expf(-best));
      values[(size_t)blockIdx.x * k + r] = Elt<T>::from_f32(sg);
      indices[(size_t)blockIdx.x * k + r] = best_i;
      s_logit[best_i] = __int_as_float(0x7fc00000);  // NaN: out of the running
      s_winner = best_i;
    }
    __syncthreads();
  }
}

// Router of one token in ONE launch: CTA e computes logit e = W[e,:] . rmsnorm(x) (fp32 accumulation, the norm with
// the two roundings of the GEMV's fused norm, the logit rounded to the 16-bit type as the GEMV would store it); the
// last CTA to arrive picks the top k (lowest index wins ties) and writes sigmoid(logit) and the indices. Stands where
// the reference chains a GEMV and muillm_topk_sigmoid_forward (csrc/modules/parallel_gateupmoe_module.cpp:45-77).
constexpr int ROUTER_THREADS = 128;
constexpr int ROUTER_MAX_E = 1024;

template <typename T>
__global__ void __launch_bounds__(ROUTER_THREADS) router_topk_kernel(const T* __restrict__ W, const T* x,
                                                                     const T* __restrict__ nw, float eps, int E, int H,
                                                                     int k, float* logits, unsigned int* counter,
                                                                     T* values, long long* indices) {
  __shared__ float s_red[ROUTER_THREADS / 32];
  __shared__ float s_logit[ROUTER_MAX_E];
  __shared__ int s_last;
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e = blockIdx.x;
  const T* w = W + (size_t)e * H;
  float rstd = 1.f;
  float acc = 0.f;
  constexpr int VMAX = 8;  // 16-byte pieces of x a thread keeps in registers: H <= 128 * 8 * 8 = 8192
  const bool vec = ((H & 7) == 0) && H <= ROUTER_THREADS * 8 * VMAX && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(w) & 15) == 0) &&
                   (nw == nullptr || (reinterpret_cast<uintptr_t>(nw) & 15) == 0);
  if (vec) {
    // the row of router weights and the norm weights do not depend on the previous kernel, x does; all loads of a
    // thread are issued before the first use
    uint4 xv[VMAX], wv[VMAX];
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
      const int i = (j * ROUTER_THREADS + tid) * 8;
      xv[j] = (i < H) ? ld_act16(x + i) : make_uint4(0, 0, 0, 0);
      wv[j] = (i < H) ? ld_cached16(w + i) : make_uint4(0, 0, 0, 0);
    }
    if (nw != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VMAX; ++j) {
        float f[8];
        unpack8<T>(xv[j], f);
#pragma unroll
        for (int q = 0; q < 8; ++q) ss = fmaf(f[q], f[q], ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) s_red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < ROUTER_THREADS / 32; ++i) tot += s_red[i];
      rstd = rsqrtf(tot / static_cast<float>(H) + eps);
      __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
      const int i = (j * ROUTER_THREADS + tid) * 8;
      if (i < H) {
        float f[8], g[8], n[8];
        unpack8<T>(xv[j], f);
        unpack8<T>(wv[j], g);
        if (nw != nullptr) {
          unpack8<T>(ld_cached16(nw + i), n);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            f[q] = Elt<T>::to_f32(Elt<T>::from_f32(Elt<T>::to_f32(Elt<T>::from_f32(f[q] * rstd)) * n[q]));
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) acc = fmaf(g[q], f[q], acc);
      }
    }
  } else {
    if (nw != nullptr) {
      float ss = 0.f;
      for (int i = tid; i < H; i += ROUTER_THREADS) {
        const float v = ld_act_f32<T>(x + i);
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) s_red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < ROUTER_THREADS / 32; ++i) tot += s_red[i];
      rstd = rsqrtf(tot / static_cast<float>(H) + eps);
      __syncthreads();
    }
    for (int i = tid; i < H; i += ROUTER_THREADS) {
      float v = ld_act_f32<T>(x + i);
      if (nw != nullptr)
        v = Elt<T>::to_f32(Elt<T>::from_f32(Elt<T>::to_f32(Elt<T>::from_f32(v * rstd)) * Elt<T>::to_f32(nw[i])));
      acc = fmaf(Elt<T>::to_f32(w[i]), v, acc);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) s_red[warp] = acc;
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTER_THREADS / 32; ++i) tot += s_red[i];
    logits[e] = Elt<T>::to_f32(Elt<T>::from_f32(tot));
    __threadfence();
    s_last = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = tid; i < E; i += ROUTER_THREADS) s_logit[i] = __ldcg(logits + i);
  __syncthreads();
  if (warp == 0) {
    for (int r = 0; r < k; ++r) {
      float best = -INFINITY;
      int best_i = 0x7fffffff;
      for (int i = lane; i < E; i += 32) {
        const float v = s_logit[i];  // taken entries are NaN and never compare greater
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
      if (best_i == 0x7fffffff) {  // only -inf / NaN left: the lowest untaken index
        best_i = 0;
        for (int i = 0; i < E; ++i)
          if (!(s_logit[i] != s_logit[i])) {
            best_i = i;
            break;
          }
        best = s_logit[best_i];
      }
      if (lane == 0) {
        values[r] = Elt<T>::from_f32(1.f / (1.f + expf(-best)));
        indices[r] = best_i;
        s_logit[best_i] = __int_as_float(0x7fc00000);
      }
      __syncwarp();
    }
  }
  if (tid == 0) *counter = 0u;
}

}  // namespace

extern "C" {

mui_status_t mui_router_topk_sigmoid_forward(void* stream, mui_dtype_t dtype, int E, int H, int k,
                                             const void* norm_weights, float epsilon, const void* router_weights,
                                             const void* x, float* logits_scratch, unsigned int* counter,
                                             void* values, int64_t* indices, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(E >= 1 && E <= ROUTER_MAX_E && H >= 1, MUI_ERR_UNSUPPORTED, "E=%d (at most %d), H=%d", E, ROUTER_MAX_E, H);
  MUI_REQUIRE(k > 0 && k <= E && k <= TOPK_MAX_K, MUI_ERR_INVALID_ARG, "k=%d outside (0, min(E, %d)]", k, TOPK_MAX_K);
  MUI_REQUIRE(router_weights && x && logits_scratch && counter && values && indices, MUI_ERR_INVALID_ARG,
              "null pointer");
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(router_topk_kernel<__half>, dim3(E), dim3(ROUTER_THREADS), 0, (cudaStream_t)stream, pdl,
                              (const __half*)router_weights, (const __half*)x, (const __half*)norm_weights, epsilon, E,
                              H, k, logits_scratch, counter, (__half*)values, (long long*)indices));
  } else {
    MUI_CUDA_CHECK(mui_launch(router_topk_kernel<__nv_bfloat16>, dim3(E), dim3(ROUTER_THREADS), 0,
                              (cudaStream_t)stream, pdl, (const __nv_bfloat16*)router_weights,
                              (const __nv_bfloat16*)x, (const __nv_bfloat16*)norm_weights, epsilon, E, H, k,
                              logits_scratch, counter, (__nv_bfloat16*)values, (long long*)indices));
  }
  return MUI_OK;
}

mui_status_t mui_topk_sigmoid_forward(void* stream, mui_dtype_t dtype, int rows, int M, int k, const void* logits,
                                      void* values, int64_t* indices, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(rows >= 0 && M >= 1, MUI_ERR_INVALID_ARG, "rows=%d M=%d", rows, M);
  MUI_REQUIRE(k > 0 && k <= M, MUI_ERR_INVALID_ARG, "k must be in the range (0, M] where M is the last dimension of x");
  MUI_REQUIRE(M <= TOPK_MAX_M, MUI_ERR_UNSUPPORTED, "M=%d must not exceed %d", M, TOPK_MAX_M);
  MUI_REQUIRE(k <= TOPK_MAX_K, MUI_ERR_UNSUPPORTED, "k=%d must not exceed %d", k, TOPK_MAX_K);
  if (rows == 0) return MUI_OK;
  MUI_REQUIRE(logits && values && indices, MUI_ERR_INVALID_ARG, "null pointer");
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(topk_sigmoid_kernel<__half>, dim3(rows), dim3(TOPK_THREADS), 0, (cudaStream_t)stream,
                              pdl, (const __half*)logits, (__half*)values, (long long*)indices, M, k));
  } else {
    MUI_CUDA_CHECK(mui_launch(topk_sigmoid_kernel<__nv_bfloat16>, dim3(rows), dim3(TOPK_THREADS), 0,
                              (cudaStream_t)stream, pdl, (const __nv_bfloat16*)logits, (__nv_bfloat16*)values,
                              (long long*)indices, M, k));
  }
  return MUI_OK;
}

mui_status_t mui_moe_gateup_silu_forward(void* stream, mui_dtype_t dtype, int num_shared, int num_routed, int top_k,
                                         int I, int H, const void* norm_weights, float epsilon,
                                         const void* gate_weights, const void* up_weights, const void* x,
                                         const void* router_scores, const int64_t* router_indices, void* t,
                                         unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(num_shared >= 0 && num_routed >= 0 && top_k >= 0 && top_k <= num_routed && num_shared + top_k >= 1,
              MUI_ERR_INVALID_ARG, "num_shared=%d num_routed=%d top_k=%d", num_shared, num_routed, top_k);
  MUI_REQUIRE(num_shared + top_k <= 8, MUI_ERR_UNSUPPORTED, "at most 8 experts are computed per token");
  MUI_REQUIRE(I >= 1 && H >= 1, MUI_ERR_INVALID_ARG, "I=%d H=%d", I, H);
  MUI_REQUIRE(gate_weights && up_weights && x && t, MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(top_k == 0 || (router_scores && router_indices), MUI_ERR_INVALID_ARG, "router outputs are null");
  GemvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = gate_weights;
  a.W2 = up_weights;
  a.x = x;
  a.norm_w = norm_weights;
  a.y = t;
  a.eps = epsilon;
  a.N = I;
  a.K = H;
  a.B = 1;
  a.Kp = (H + 7) & ~7;
  a.moe_mode = GEMV_MOE_ROWS;
  a.slots = num_shared + top_k;
  a.num_shared = num_shared;
  a.router_indices = router_indices;
  a.router_scores = router_scores;
  a.w8_fmt = -1;
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 1, a, flags);
}

mui_status_t mui_moe_down_forward(void* stream, mui_dtype_t dtype, int num_shared, int num_routed, int top_k, int H,
                                  int I, const void* down_weights, const void* residual, const void* t,
                                  const int64_t* router_indices, void* y, float* y_f32, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(num_shared >= 0 && num_routed >= 0 && top_k >= 0 && top_k <= num_routed && num_shared + top_k >= 1,
              MUI_ERR_INVALID_ARG, "num_shared=%d num_routed=%d top_k=%d", num_shared, num_routed, top_k);
  MUI_REQUIRE(num_shared + top_k <= 8, MUI_ERR_UNSUPPORTED, "at most 8 experts are computed per token");
  MUI_REQUIRE(down_weights && t && (y || y_f32), MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(top_k == 0 || router_indices, MUI_ERR_INVALID_ARG, "router_indices is null");
  GemvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = down_weights;
  a.x = t;
  a.residual = residual;
  a.y = y;
  a.y_f32 = y_f32;
  a.N = H;
  a.K = I;
  a.B = 1;
  a.Kp = (I + 7) & ~7;
  a.moe_mode = GEMV_MOE_SEGMENTS;
  a.slots = num_shared + top_k;
  a.num_shared = num_shared;
  a.router_indices = router_indices;
  a.w8_fmt = -1;
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 0, a, flags);
}

mui_status_t mui_moe_mlp_forward(void* stream, mui_dtype_t dtype, int num_shared, int num_routed, int top_k, int I,
                                 int H, const void* norm_weights, float epsilon, const void* gate_weights,
                                 const void* up_weights, const void* down_weights, const void* residual,
                                 const void* x, const void* router_scores, const int64_t* router_indices,
                                 void* scratch_t, void* y, unsigned flags) {
  MUI_REQUIRE(scratch_t != nullptr, MUI_ERR_INVALID_ARG, "scratch_t must be non-null ([num_shared + top_k, I] elements)");
  mui_status_t s = mui_moe_gateup_silu_forward(stream, dtype, num_shared, num_routed, top_k, I, H, norm_weights,
                                               epsilon, gate_weights, up_weights, x, router_scores, router_indices,
                                               scratch_t, flags);
  if (s != MUI_OK) return s;
  return mui_moe_down_forward(stream, dtype, num_shared, num_routed, top_k, H, I, down_weights, residual, scratch_t,
                              router_indices, y, nullptr, flags);
}

}  // extern "C"
