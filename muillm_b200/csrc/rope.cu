// Rotary position embedding (rotate-half form) on q and k of the new tokens, fused with the write of
// rope(k) and v into a static KV cache at cache_position. One warp per (head, token, batch) row.
// rope(x)[i]       = x[i]     * cos[i]       - x[i + D/2] * sin[i]
// rope(x)[i + D/2] = x[i+D/2] * cos[i + D/2] + x[i]       * sin[i + D/2]      evaluated in fp32, rounded once.
// Traffic per call: (Hq + 2*Hkv) * T * B * D * 2 bytes in, the same out, plus one cos/sin row per token.
#include "common.cuh"

MUI_STATUS_ACCESSOR(rope)

namespace {

constexpr int ROPE_WARPS = 4;

struct RopeArgs {
  const void *q_in, *k_in, *v_in;
  void *q_out, *k_out, *k_cache, *v_cache;
  const void *cos_t, *sin_t;
  const int64_t* position_ids;
  const int64_t* cache_position;
  mui_strides3_t qs, ks, vs;
  int B, T, max_T, Hq, Hkv, D, table_layout, apply_rope;
  unsigned long long* trace;
};

template <typename T>
__global__ void __launch_bounds__(ROPE_WARPS * 32) rope_kernel(const RopeArgs a) {
  trace_start(a.trace);
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = a.Hq + 2 * a.Hkv;
  const long long row = (long long)blockIdx.x * ROPE_WARPS + warp;
  const long long rows_total = (long long)heads_total * a.T * a.B;
  if (row >= rows_total) return;
  // row -> (b, t, head) with head fastest
  int head = static_cast<int>(row % heads_total);
  const long long bt = row / heads_total;
  const int t = static_cast<int>(bt % a.T);
  const int b = static_cast<int>(bt / a.T);
  const int D = a.D, half = D >> 1;

  const T* in;
  T* out_plain = nullptr;  // contiguous [B, H, T, D] output
  T* out_cache = nullptr;  // row inside the static cache
  bool rotate;
  if (head < a.Hq) {
    if (a.q_in == nullptr) return;
    in = reinterpret_cast<const T*>(a.q_in) + b * a.qs.batch + head * a.qs.head + t * a.qs.tok;
    out_plain = reinterpret_cast<T*>(a.q_out) + (((size_t)b * a.Hq + head) * a.T + t) * D;
    rotate = a.apply_rope != 0;
  } else if (head < a.Hq + a.Hkv) {
    head -= a.Hq;
    in = reinterpret_cast<const T*>(a.k_in) + b * a.ks.batch + head * a.ks.head + t * a.ks.tok;
    if (a.k_out) out_plain = reinterpret_cast<T*>(a.k_out) + (((size_t)b * a.Hkv + head) * a.T + t) * D;
    if (a.k_cache) {
      // a cache row outside the cache (a replayed graph that ran past the end) is recorded and not written
      const long long cp = __ldcg(a.cache_position + t);
      if (cp < 0 || cp >= a.max_T) {
        if (lane == 0) mui_dev_set_status(MUI_DEV_BAD_LENGTH, static_cast<unsigned>(cp));
        if (!out_plain) return;
      } else {
        out_cache = reinterpret_cast<T*>(a.k_cache) + (((size_t)b * a.Hkv + head) * a.max_T + (size_t)cp) * D;
      }
    }
    rotate = a.apply_rope != 0;
  } else {
    head -= a.Hq + a.Hkv;
    if (a.v_in == nullptr || a.v_cache == nullptr) return;
    in = reinterpret_cast<const T*>(a.v_in) + b * a.vs.batch + head * a.vs.head + t * a.vs.tok;
    const long long cp = __ldcg(a.cache_position + t);
    if (cp < 0 || cp >= a.max_T) {
      if (lane == 0) mui_dev_set_status(MUI_DEV_BAD_LENGTH, static_cast<unsigned>(cp));
      return;
    }
    out_cache = reinterpret_cast<T*>(a.v_cache) + (((size_t)b * a.Hkv + head) * a.max_T + (size_t)cp) * D;
    rotate = false;
  }

  if (!rotate) {
    for (int i = lane; i < D; i += 32) {
      const T v = ld_act<T>(in + i);
      if (out_plain) out_plain[i] = v;
      if (out_cache) out_cache[i] = v;
    }
    return;
  }

  const size_t pos = (a.table_layout == 0) ? static_cast<size_t>(__ldcg(a.position_ids + (size_t)b * a.T + t))
                                           : ((size_t)b * a.T + t);
  const T* cs = reinterpret_cast<const T*>(a.cos_t) + pos * D;
  const T* sn = reinterpret_cast<const T*>(a.sin_t) + pos * D;
  for (int i = lane; i < half; i += 32) {
    const float x1 = ld_act_f32<T>(in + i), x2 = ld_act_f32<T>(in + i + half);
    const float c1 = Elt<T>::to_f32(cs[i]), c2 = Elt<T>::to_f32(cs[i + half]);
    const float s1 = Elt<T>::to_f32(sn[i]), s2 = Elt<T>::to_f32(sn[i + half]);
    const T o1 = Elt<T>::from_f32(fmaf(x1, c1, -x2 * s1));
    const T o2 = Elt<T>::from_f32(fmaf(x2, c2, x1 * s2));
    if (out_plain) {
      out_plain[i] = o1;
      out_plain[i + half] = o2;
    }
    if (out_cache) {
      out_cache[i] = o1;
      out_cache[i + half] = o2;
    }
  }
  if (lane == 0) trace_end(a.trace);
}

mui_status_t launch_rope(cudaStream_t stream, mui_dtype_t dtype, RopeArgs a, unsigned flags) {
  a.trace = mui_trace_next_record(4);
  const long long rows = (long long)(a.Hq + 2 * a.Hkv) * a.T * a.B;
  if (rows == 0) return MUI_OK;
  const int grid = static_cast<int>((rows + ROPE_WARPS - 1) / ROPE_WARPS);
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(rope_kernel<__half>, dim3(grid), dim3(ROPE_WARPS * 32), 0, stream, pdl, a));
  } else {
    MUI_CUDA_CHECK(mui_launch(rope_kernel<__nv_bfloat16>, dim3(grid), dim3(ROPE_WARPS * 32), 0, stream, pdl, a));
  }
  return MUI_OK;
}

}  // namespace

extern "C" {

mui_status_t mui_rope_forward(void* stream, mui_dtype_t dtype, int B, int T, int max_T, int Hq, int Hkv, int D,
                              int table_layout, const int64_t* position_ids, const void* cos_table,
                              const void* sin_table, const void* q_in, mui_strides3_t q_strides, const void* k_in,
                              mui_strides3_t k_strides, const void* v_in, mui_strides3_t v_strides, void* q_out,
                              void* k_out, void* k_cache, void* v_cache, const int64_t* cache_position,
                              unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(B >= 0 && T >= 0 && Hq >= 0 && Hkv >= 0 && D >= 2 && (D & 1) == 0, MUI_ERR_INVALID_ARG,
              "bad sizes B=%d T=%d Hq=%d Hkv=%d D=%d", B, T, Hq, Hkv, D);
  MUI_REQUIRE(cos_table && sin_table, MUI_ERR_INVALID_ARG, "cos/sin tables must be non-null");
  MUI_REQUIRE(table_layout == 0 || table_layout == 1, MUI_ERR_INVALID_ARG, "table_layout must be 0 ([S,D]) or 1 ([B,T,D])");
  MUI_REQUIRE(table_layout == 1 || position_ids, MUI_ERR_INVALID_ARG, "position_ids required for the [S,D] table layout");
  MUI_REQUIRE(Hq == 0 || (q_in && q_out), MUI_ERR_INVALID_ARG, "q_in and q_out must be non-null");
  MUI_REQUIRE(Hkv == 0 || k_in, MUI_ERR_INVALID_ARG, "k_in must be non-null");
  MUI_REQUIRE(Hkv == 0 || k_out || k_cache, MUI_ERR_INVALID_ARG, "k_out or k_cache must be given");
  MUI_REQUIRE(!(k_cache || v_cache) || (k_cache && v_cache && v_in && cache_position && max_T >= 1),
              MUI_ERR_INVALID_ARG, "cache write needs k_cache, v_cache, v_in, cache_position and max_T");
  RopeArgs a;
  a.q_in = q_in; a.k_in = k_in; a.v_in = v_in;
  a.q_out = q_out; a.k_out = k_out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.cos_t = cos_table; a.sin_t = sin_table;
  a.position_ids = position_ids; a.cache_position = cache_position;
  a.qs = q_strides; a.ks = k_strides; a.vs = v_strides;
  a.B = B; a.T = T; a.max_T = max_T; a.Hq = Hq; a.Hkv = Hkv; a.D = D;
  a.table_layout = table_layout; a.apply_rope = 1;
  return launch_rope((cudaStream_t)stream, dtype, a, flags);
}

mui_status_t mui_static_kvcache_update(void* stream, mui_dtype_t dtype, int B, int T, int max_T, int Hkv, int D,
                                       const void* k_in, mui_strides3_t k_strides, const void* v_in,
                                       mui_strides3_t v_strides, void* k_cache, void* v_cache,
                                       const int64_t* cache_position, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(B >= 0 && T >= 0 && Hkv >= 0 && D >= 1 && max_T >= 1, MUI_ERR_INVALID_ARG, "bad sizes");
  MUI_REQUIRE(k_in && v_in && k_cache && v_cache && cache_position, MUI_ERR_INVALID_ARG, "null pointer");
  RopeArgs a;
  a.q_in = nullptr; a.k_in = k_in; a.v_in = v_in;
  a.q_out = nullptr; a.k_out = nullptr; a.k_cache = k_cache; a.v_cache = v_cache;
  a.cos_t = nullptr; a.sin_t = nullptr;
  a.position_ids = nullptr; a.cache_position = cache_position;
  a.qs = k_strides; a.ks = k_strides; a.vs = v_strides;
  a.B = B; a.T = T; a.max_T = max_T; a.Hq = 0; a.Hkv = Hkv; a.D = D;
  a.table_layout = 0; a.apply_rope = 0;
  return launch_rope((cudaStream_t)stream, dtype, a, flags);
}

}  // extern "C"
