// C-ABI plumbing: status strings, thread-local error text, per-device property cache, the device
// status word, and the argument validation + dispatch of the linear and gate/up entry points.
#include "gemv_common.cuh"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include <vector>

// per-file device status words (see MUI_STATUS_ACCESSOR)
static std::vector<mui_status_accessor_t>& status_accessors() {
  static std::vector<mui_status_accessor_t> v;
  return v;
}
void mui_register_status_accessor(mui_status_accessor_t fn) { status_accessors().push_back(fn); }

static thread_local char tls_error[512] = "";

void mui_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
  va_end(ap);
}

// ---- launch tracing state (per host thread) ----
static thread_local unsigned long long* tls_trace_buf = nullptr;
static thread_local int tls_trace_cap = 0, tls_trace_next = 0;
static thread_local int tls_trace_tags[4096];

unsigned long long* mui_trace_next_record(int kernel_tag) {
  if (tls_trace_buf == nullptr || tls_trace_next >= tls_trace_cap) return nullptr;
  tls_trace_tags[tls_trace_next] = kernel_tag;
  return tls_trace_buf + 8 * (size_t)(tls_trace_next++);
}

const MuiDeviceInfo* mui_current_device_info() {
  static MuiDeviceInfo infos[64];
  static bool valid[64] = {false};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    mui_set_error("cudaGetDevice failed: %s", cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!valid[dev]) {
    MuiDeviceInfo& i = infos[dev];
    i.device = dev;
    int v = 0;
    bool ok = true;
    ok &= cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess;
    i.sm_count = v;
    ok &= cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess;
    i.smem_per_block_optin = v;
    ok &= cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess;
    i.smem_per_sm = v;
    ok &= cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev) == cudaSuccess;
    i.l2_bytes = v;
    if (!ok) {
      mui_set_error("cudaDeviceGetAttribute failed on device %d", dev);
      return nullptr;
    }
    valid[dev] = true;
  }
  return &infos[dev];
}

// defined in gemv.cu
mui_status_t mui_launch_gemv16(cudaStream_t stream, mui_dtype_t dtype, int mode, const GemvArgs& a, unsigned flags);
// the public entry points plus launch hints (decode stack)
mui_status_t mui_linear_forward_hinted(void* stream, mui_dtype_t dtype, int B, int N, int K,
                                       const void* norm_weights, float epsilon, const void* weights,
                                       mui_activation_t activ, const void* mul_bias, const void* add_bias,
                                       const void* residual, const void* x, void* y, unsigned flags,
                                       const GemvHints* hints);
mui_status_t mui_gateup_silu_forward_hinted(void* stream, mui_dtype_t dtype, int B, int I, int H,
                                            const void* norm_weights, float epsilon, const void* gate_weights,
                                            const void* up_weights, const void* x, void* t, unsigned flags,
                                            const GemvHints* hints);

extern "C" {

const char* mui_status_string(mui_status_t s) {
  switch (s) {
    case MUI_OK: return "ok";
    case MUI_ERR_INVALID_ARG: return "invalid argument";
    case MUI_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case MUI_ERR_CUDA: return "CUDA runtime error";
    case MUI_ERR_DEVICE: return "device-side status set (bounded wait ran out)";
    case MUI_ERR_COMM: return "communicator error";
  }
  return "unknown status";
}

const char* mui_last_error(void) { return tls_error; }

int mui_version(void) { return 100; }

mui_status_t mui_device_props(int device, mui_device_props_t* out) {
  MUI_REQUIRE(out != nullptr, MUI_ERR_INVALID_ARG, "out is null");
  cudaDeviceProp p;
  MUI_CUDA_CHECK(cudaGetDeviceProperties(&p, device));
  out->device = device;
  out->sm_count = p.multiProcessorCount;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->smem_per_block_optin = (int)p.sharedMemPerBlockOptin;
  out->l2_bytes = p.l2CacheSize;
  out->total_mem = p.totalGlobalMem;
  return MUI_OK;
}

mui_status_t mui_device_status(unsigned* code, int clear) {
  MUI_REQUIRE(code != nullptr, MUI_ERR_INVALID_ARG, "code is null");
  MUI_CUDA_CHECK(cudaDeviceSynchronize());
  *code = 0;
  for (mui_status_accessor_t acc : status_accessors()) {
    unsigned v = 0;
    MUI_CUDA_CHECK(acc(&v, clear));
    if (v != 0 && *code == 0) *code = v;
  }
  return MUI_OK;
}

mui_status_t mui_trace_enable(void* stream, void* device_buffer, int max_records) {
  if (device_buffer == nullptr || max_records <= 0) {
    tls_trace_buf = nullptr;  // the count and tags of the finished trace stay readable
    tls_trace_cap = 0;
    return MUI_OK;
  }
  MUI_REQUIRE(max_records <= 4096, MUI_ERR_INVALID_ARG, "at most 4096 trace records");
  MUI_CUDA_CHECK(cudaMemsetAsync(device_buffer, 0xFF, (size_t)max_records * 64, (cudaStream_t)stream));
  tls_trace_buf = reinterpret_cast<unsigned long long*>(device_buffer);
  tls_trace_cap = max_records;
  tls_trace_next = 0;
  return MUI_OK;
}

int mui_trace_count(int* tags_out, int max_tags) {
  const int n = tls_trace_next;
  for (int i = 0; i < n && i < max_tags; ++i) tags_out[i] = tls_trace_tags[i];
  return n;
}

static mui_status_t check_dtype(mui_dtype_t d) {
  MUI_REQUIRE(d == MUI_F16 || d == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d is neither MUI_F16 nor MUI_BF16", (int)d);
  return MUI_OK;
}

mui_status_t mui_linear_forward(void* stream, mui_dtype_t dtype, int B, int N, int K, const void* norm_weights,
                                float epsilon, const void* weights, mui_activation_t activ, const void* mul_bias,
                                const void* add_bias, const void* residual, const void* x, void* y, unsigned flags) {
  return mui_linear_forward_hinted(stream, dtype, B, N, K, norm_weights, epsilon, weights, activ, mul_bias, add_bias,
                                   residual, x, y, flags, nullptr);
}

mui_status_t mui_gateup_silu_forward(void* stream, mui_dtype_t dtype, int B, int I, int H, const void* norm_weights,
                                     float epsilon, const void* gate_weights, const void* up_weights, const void* x,
                                     void* t, unsigned flags) {
  return mui_gateup_silu_forward_hinted(stream, dtype, B, I, H, norm_weights, epsilon, gate_weights, up_weights, x, t,
                                        flags, nullptr);
}

}  // extern "C"

mui_status_t mui_linear_forward_hinted(void* stream, mui_dtype_t dtype, int B, int N, int K,
                                       const void* norm_weights, float epsilon, const void* weights,
                                       mui_activation_t activ, const void* mul_bias, const void* add_bias,
                                       const void* residual, const void* x, void* y, unsigned flags,
                                       const GemvHints* hints) {
  if (mui_status_t s = check_dtype(dtype)) return s;
  MUI_REQUIRE(weights && x && y, MUI_ERR_INVALID_ARG, "weights, x and y must be non-null");
  MUI_REQUIRE(B >= 1 && B <= 8, MUI_ERR_UNSUPPORTED, "B=%d outside 1..8 (larger batches belong to a GEMM)", B);
  MUI_REQUIRE(N >= 1 && K >= 1, MUI_ERR_INVALID_ARG, "N=%d, K=%d must be positive", N, K);
  MUI_REQUIRE(activ == MUI_ACT_IDENTITY || activ == MUI_ACT_SILU, MUI_ERR_INVALID_ARG, "unknown activation %d",
              (int)activ);
  GemvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = weights;
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
  a.w8_fmt = -1;
  gemv_apply_hints(a, hints);
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 0, a, flags);
}

mui_status_t mui_gateup_silu_forward_hinted(void* stream, mui_dtype_t dtype, int B, int I, int H,
                                            const void* norm_weights, float epsilon, const void* gate_weights,
                                            const void* up_weights, const void* x, void* t, unsigned flags,
                                            const GemvHints* hints) {
  if (mui_status_t s = check_dtype(dtype)) return s;
  MUI_REQUIRE(gate_weights && up_weights && x && t, MUI_ERR_INVALID_ARG,
              "gate_weights, up_weights, x and t must be non-null");
  MUI_REQUIRE(B >= 1 && B <= 8, MUI_ERR_UNSUPPORTED, "B=%d outside 1..8 (larger batches belong to a GEMM)", B);
  MUI_REQUIRE(I >= 1 && H >= 1, MUI_ERR_INVALID_ARG, "I=%d, H=%d must be positive", I, H);
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
  a.B = B;
  a.Kp = (H + 7) & ~7;
  a.moe_mode = GEMV_MOE_NONE;
  a.slots = 1;
  a.w8_fmt = -1;
  gemv_apply_hints(a, hints);
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 1, a, flags);
}

extern "C" {

mui_status_t mui_gateupdown_forward(void* stream, mui_dtype_t dtype, int B, int I, int H, const void* norm_weights,
                                    float epsilon, const void* gate_weights, const void* up_weights,
                                    const void* down_weights, const void* residual, const void* x, void* scratch_t,
                                    void* y, unsigned flags) {
  MUI_REQUIRE(scratch_t != nullptr, MUI_ERR_INVALID_ARG, "scratch_t must be non-null ([B,I] elements)");
  mui_status_t s = mui_gateup_silu_forward(stream, dtype, B, I, H, norm_weights, epsilon, gate_weights, up_weights,
                                           x, scratch_t, flags);
  if (s != MUI_OK) return s;
  return mui_linear_forward(stream, dtype, B, H, I, nullptr, 0.f, down_weights, MUI_ACT_IDENTITY, nullptr, nullptr,
                            residual, scratch_t, y, flags);
}

}  // extern "C"
