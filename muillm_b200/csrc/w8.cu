// Weight-only 8-bit entry points: linear and gate/up+SiLU on quantised weights (kernels in gemv_kernels.cuh), and the
// full de-quantisation used by batched fallbacks.
#include "gemv_common.cuh"

#include <algorithm>
#include <cstring>

MUI_STATUS_ACCESSOR(w8)

mui_status_t mui_launch_gemv16(cudaStream_t stream, mui_dtype_t dtype, int mode, const GemvArgs& a, unsigned flags);

namespace {

// out[n,k] = q*s[n] (SYM_ROW, q signed) or q*scale[n,g] + min[n,g] (GROUP_MIN, q unsigned); one thread per 16 weights
template <typename T>
__global__ void __launch_bounds__(256) w8_dequantize_kernel(const unsigned char* __restrict__ q,
                                                            const T* __restrict__ scales, T* __restrict__ out,
                                                            long long total, int K, int fmt, int group_shift) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long n = i / K;
    const int k = static_cast<int>(i - n * K);
    float w;
    if (fmt == MUI_W8_SYM_ROW) {
      w = static_cast<float>(static_cast<signed char>(q[i])) * Elt<T>::to_f32(scales[n]);
    } else {
      const long long g = n * (K >> group_shift) + (k >> group_shift);
      w = fmaf(static_cast<float>(q[i]), Elt<T>::to_f32(scales[g * 2]), Elt<T>::to_f32(scales[g * 2 + 1]));
    }
    out[i] = Elt<T>::from_f32(w);
  }
}

mui_status_t check_w8(mui_dtype_t dtype, mui_w8_format_t fmt, int group_shift, int K) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(fmt == MUI_W8_SYM_ROW || fmt == MUI_W8_GROUP_MIN, MUI_ERR_INVALID_ARG, "unknown 8-bit format %d", (int)fmt);
  if (fmt == MUI_W8_GROUP_MIN) {
    MUI_REQUIRE(group_shift >= 0 && group_shift < 31, MUI_ERR_INVALID_ARG, "group_shift %d", group_shift);
    MUI_REQUIRE((K % (1 << group_shift)) == 0, MUI_ERR_INVALID_ARG,
                "groupsize must divide the weight dimension but %d doesn't divide %d", 1 << group_shift, K);
  }
  return MUI_OK;
}

}  // namespace

extern "C" {

mui_status_t mui_linear_w8_forward(void* stream, mui_dtype_t dtype, mui_w8_format_t fmt, int group_shift, int B,
                                   int N, int K, const void* norm_weights, float epsilon, const void* qweights,
                                   const void* scales, mui_activation_t activ, const void* mul_bias,
                                   const void* add_bias, const void* residual, const void* x, void* y,
                                   unsigned flags) {
  if (mui_status_t s = check_w8(dtype, fmt, group_shift, K)) return s;
  MUI_REQUIRE(qweights && scales && x && y, MUI_ERR_INVALID_ARG, "qweights, scales, x and y must be non-null");
  MUI_REQUIRE(B >= 1 && B <= 8, MUI_ERR_UNSUPPORTED, "B=%d outside 1..8 (larger batches de-quantise and use a GEMM)", B);
  MUI_REQUIRE(N >= 1 && K >= 1, MUI_ERR_INVALID_ARG, "N=%d, K=%d must be positive", N, K);
  GemvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = qweights;
  a.scales = scales;
  a.x = x;
  a.norm_w = norm_weights;
  a.mul_bias = mul_bias;
  a.add_bias = add_bias;
  a.residual = residual;
  a.y = y;
  a.eps = epsilon;
  a.N = N;
  a.K = K;
  a.B = B;
  a.activ = (int)activ;
  a.Kp = (K + 7) & ~7;
  a.moe_mode = GEMV_MOE_NONE;
  a.slots = 1;
  a.group_shift = group_shift;
  a.w8_fmt = (int)fmt;
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 0, a, flags);
}

mui_status_t mui_gateup_silu_w8_forward(void* stream, mui_dtype_t dtype, mui_w8_format_t fmt, int group_shift, int B,
                                        int I, int H, const void* norm_weights, float epsilon, const void* gate_q,
                                        const void* gate_scales, const void* up_q, const void* up_scales,
                                        const void* x, void* t, unsigned flags) {
  if (mui_status_t s = check_w8(dtype, fmt, group_shift, H)) return s;
  MUI_REQUIRE(gate_q && gate_scales && up_q && up_scales && x && t, MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(B >= 1 && B <= 8, MUI_ERR_UNSUPPORTED, "B=%d outside 1..8 (larger batches de-quantise and use a GEMM)", B);
  MUI_REQUIRE(I >= 1 && H >= 1, MUI_ERR_INVALID_ARG, "I=%d, H=%d must be positive", I, H);
  GemvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = gate_q;
  a.W2 = up_q;
  a.scales = gate_scales;
  a.scales2 = up_scales;
  a.x = x;
  a.norm_w = norm_weights;
  a.y = t;
  a.eps = epsilon;
  a.N = I;
  a.K = H;
  a.B = B;
  a.Kp = (H + 7) & ~7;
  a.moe_mode = GEMV_MOE_NONE;
  a.slots = 1;
  a.group_shift = group_shift;
  a.w8_fmt = (int)fmt;
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 1, a, flags);
}

mui_status_t mui_gateup_silu_w8_packed_forward(void* stream, mui_dtype_t dtype, int group_shift, int B, int I, int H,
                                               const void* norm_weights, float epsilon, const void* gate_up_q,
                                               const void* gate_up_scales_min, const void* x, void* t,
                                               unsigned flags) {
  if (mui_status_t s = check_w8(dtype, MUI_W8_GROUP_MIN, group_shift, H)) return s;
  MUI_REQUIRE(gate_up_q && gate_up_scales_min && x && t, MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(B >= 1 && B <= 8, MUI_ERR_UNSUPPORTED, "B=%d outside 1..8 (larger batches de-quantise and use a GEMM)", B);
  MUI_REQUIRE(I >= 1 && H >= 1, MUI_ERR_INVALID_ARG, "I=%d, H=%d must be positive", I, H);
  GemvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = gate_up_q;
  a.scales = gate_up_scales_min;
  a.x = x;
  a.norm_w = norm_weights;
  a.y = t;
  a.eps = epsilon;
  a.N = I;
  a.K = H;
  a.B = B;
  a.Kp = (H + 7) & ~7;
  a.moe_mode = GEMV_MOE_NONE;
  a.slots = 1;
  a.group_shift = group_shift;
  a.w8_fmt = (int)MUI_W8_GROUP_MIN;
  a.w8_pack = 1;
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 1, a, flags);
}

mui_status_t mui_w8_dequantize(void* stream, mui_dtype_t dtype, mui_w8_format_t fmt, int group_shift, int N, int K,
                               const void* qweights, const void* scales, void* out) {
  if (mui_status_t s = check_w8(dtype, fmt, group_shift, K)) return s;
  MUI_REQUIRE(N >= 0 && K >= 1, MUI_ERR_INVALID_ARG, "N=%d K=%d", N, K);
  if (N == 0) return MUI_OK;
  MUI_REQUIRE(qweights && scales && out, MUI_ERR_INVALID_ARG, "null pointer");
  const long long total = (long long)N * K;
  const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(w8_dequantize_kernel<__half>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, 0,
                              (const unsigned char*)qweights, (const __half*)scales, (__half*)out, total, K, (int)fmt,
                              group_shift));
  } else {
    MUI_CUDA_CHECK(mui_launch(w8_dequantize_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, 0,
                              (const unsigned char*)qweights, (const __nv_bfloat16*)scales, (__nv_bfloat16*)out,
                              total, K, (int)fmt, group_shift));
  }
  return MUI_OK;
}

}  // extern "C"
