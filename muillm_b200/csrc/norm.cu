// Stand-alone RMSNorm / L2-norm over rows of a [rows, K] matrix (final norm before lm_head, batched
// fallback of the fused GEMV norm, Llama-4 QK L2 norm). One CTA per row, fp32 statistics, roundings
// of the HF modules: y = round16(round16(x * rstd) * w).
#include "common.cuh"

MUI_STATUS_ACCESSOR(norm)

namespace {

constexpr int NORM_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(NORM_THREADS) rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                               T* __restrict__ y, int K, float eps) {
  __shared__ float red[NORM_THREADS / 32];
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* xr = x + (size_t)blockIdx.x * K;
  T* yr = y + (size_t)blockIdx.x * K;
  const bool vec_ok = ((K & 7) == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(yr) & 15) == 0) &&
                      (w == nullptr || (reinterpret_cast<uintptr_t>(w) & 15) == 0);
  float ss = 0.f;
  if (vec_ok) {
    for (int k = tid * 8; k < K; k += NORM_THREADS * 8) {
      float f[8];
      unpack8<T>(ld_act16(xr + k), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
    }
  } else {
    for (int k = tid; k < K; k += NORM_THREADS) {
      const float v = ld_act_f32<T>(xr + k);
      ss = fmaf(v, v, ss);
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_THREADS / 32; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / static_cast<float>(K) + eps);

  if (vec_ok) {
    for (int k = tid * 8; k < K; k += NORM_THREADS * 8) {
      float f[8], wv[8];
      unpack8<T>(ld_act16(xr + k), f);
      if (w != nullptr) unpack8<T>(ld_cached16(w + k), wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float n1 = Elt<T>::to_f32(Elt<T>::from_f32(f[i] * rstd));
        f[i] = (w != nullptr) ? n1 * wv[i] : n1;
      }
      *reinterpret_cast<uint4*>(yr + k) = pack8<T>(f);
    }
  } else {
    for (int k = tid; k < K; k += NORM_THREADS) {
      float n1 = Elt<T>::to_f32(Elt<T>::from_f32(ld_act_f32<T>(xr + k) * rstd));
      if (w != nullptr) n1 *= Elt<T>::to_f32(w[k]);
      yr[k] = Elt<T>::from_f32(n1);
    }
  }
}

}  // namespace

extern "C" mui_status_t mui_rmsnorm_forward(void* stream, mui_dtype_t dtype, int rows, int K, const void* w,
                                            float epsilon, const void* x, void* y, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(rows >= 0 && K >= 1, MUI_ERR_INVALID_ARG, "rows=%d, K=%d", rows, K);
  if (rows == 0) return MUI_OK;
  MUI_REQUIRE(x && y, MUI_ERR_INVALID_ARG, "x and y must be non-null");
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(rmsnorm_kernel<__half>, dim3(rows), dim3(NORM_THREADS), 0, (cudaStream_t)stream, pdl,
                              (const __half*)x, (const __half*)w, (__half*)y, K, epsilon));
  } else {
    MUI_CUDA_CHECK(mui_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(NORM_THREADS), 0,
                              (cudaStream_t)stream, pdl, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                              (__nv_bfloat16*)y, K, epsilon));
  }
  return MUI_OK;
}
