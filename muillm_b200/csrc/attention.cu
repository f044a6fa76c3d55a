// Split-KV flash decoding for one query token per sequence.
//
// Grid (splits, kv heads, batch), 256 threads. A CTA owns a contiguous token range of one KV head and
// serves all G = Hq/Hkv query heads of that group, so every K and V row is read from HBM exactly once.
// Inside a warp D/8 lanes share one token row (16 bytes each): per step a warp reads 32/(D/8) tokens of K
// and V, the partial q·k products are finished with xor shuffles, and each lane keeps fp32 online-softmax
// state (m, l, acc[8]) for its 8 output dims of every query head. Warps are merged through shared
// memory. With more than one active split the (m, l, acc) partials go to the fp32 workspace and the last
// CTA to arrive for a (batch, kv head) merges them by log-sum-exp and writes the output — one launch, no
// separate combine kernel. The number of attended tokens may come from device memory, which keeps the
// launch replayable in a CUDA graph while the sequence grows.
//
// Algorithmic bytes: 2 * B * Hkv * S * D * 2 (K and V) + B * Hq * D * 2 * 2 (q in, out) [+ B*S*2 mask].
#include "common.cuh"

#include <algorithm>
#include <cmath>
#include <mutex>

MUI_STATUS_ACCESSOR(attention)

namespace {

constexpr int FD_THREADS = 256;
constexpr int FD_WARPS = 8;
constexpr int FD_MAX_SPLITS = 64;
constexpr int FD_COUNTER_BYTES = 4096;
constexpr int FD_CHUNK_ALIGN = 16;
constexpr int FD_MIN_CHUNK = 64;  // tokens per split at least: one load round of the 8 warps (8 x 2 x 4 tokens at D=128)

struct FdArgs {
  const void *q, *k, *v, *mask;
  void* out;
  unsigned int* counters;  // [B*Hkv]
  float* partials;         // [B, Hq, max_splits, D + 2]
  const int32_t* seq_len_dev;
  mui_strides3_t kvs;
  float scale_log2;  // softmax scale * log2(e)
  int B, Hq, Hkv, D, S, G, max_splits;
  unsigned long long* trace;
};

__device__ __forceinline__ void fd_merge(float& m, float& l, float (&acc)[8], float mo, float lo,
                                         const float (&acco)[8]) {
  const float mn = fmaxf(m, mo);
  const float a = (m == -INFINITY) ? 0.f : exp2f(m - mn);
  const float b = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
  l = l * a + lo * b;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = acc[i] * a + acco[i] * b;
  m = mn;
}

template <typename T, int D, int GP, int U>
__global__ void __launch_bounds__(FD_THREADS) flash_decode_kernel(const FdArgs a) {
  constexpr int LPT = D / 8;    // lanes per token row
  constexpr int TPW = 32 / LPT; // tokens per warp step
  __shared__ float sm_m[FD_WARPS][GP];
  __shared__ float sm_l[FD_WARPS][GP];
  __shared__ float sm_acc[FD_WARPS][GP][D];
  __shared__ int sm_is_last;

  trace_start(a.trace);
  pdl_wait_prior_grid();
  pdl_launch_dependents();

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.G;

  int S = a.S;
  if (a.seq_len_dev != nullptr) S = min(S, max(0, __ldcg(a.seq_len_dev)));
  int chunk = (S + (int)gridDim.x - 1) / (int)gridDim.x;
  chunk = max(FD_MIN_CHUNK, (chunk + FD_CHUNK_ALIGN - 1) / FD_CHUNK_ALIGN * FD_CHUNK_ALIGN);
  const int n_active = max(1, (S + chunk - 1) / chunk);
  if (split >= n_active) return;
  const int t_begin = split * chunk;
  const int t_end = min(S, t_begin + chunk);

  const int sub = lane / LPT;        // which token of the warp step this lane serves
  const int dlane = lane % LPT;      // which 8-dim slice
  const int d0 = dlane * 8;

  // q of the group's heads, pre-multiplied by scale*log2(e)
  float qf[GP][8];
#pragma unroll
  for (int g = 0; g < GP; ++g) {
    if (g < G) {
      const T* qp = reinterpret_cast<const T*>(a.q) + ((size_t)b * a.Hq + (size_t)kvh * G + g) * D + d0;
      unpack8<T>(ld_act16(qp), qf[g]);
#pragma unroll
      for (int i = 0; i < 8; ++i) qf[g][i] *= a.scale_log2;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) qf[g][i] = 0.f;
    }
  }

  float m[GP], l[GP], acc[GP][8];
#pragma unroll
  for (int g = 0; g < GP; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  const T* kbase = reinterpret_cast<const T*>(a.k) + b * a.kvs.batch + kvh * a.kvs.head + d0;
  const T* vbase = reinterpret_cast<const T*>(a.v) + b * a.kvs.batch + kvh * a.kvs.head + d0;
  const T* mrow = (a.mask != nullptr) ? reinterpret_cast<const T*>(a.mask) + (size_t)b * a.S : nullptr;

  // warp w takes tokens t_begin + (i*FD_WARPS + w)*TPW + sub, i = 0,1,...
  for (int t0 = t_begin + warp * TPW; t0 < t_end; t0 += FD_WARPS * TPW * U) {
    uint4 kraw[U], vraw[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u * FD_WARPS * TPW + sub;
      valid[u] = t < t_end;
      if (valid[u] && mrow != nullptr) valid[u] = (ld_act_f32<T>(mrow + t) == 0.f);
      if (valid[u]) {
        kraw[u] = __ldcg(reinterpret_cast<const uint4*>(kbase + (size_t)t * a.kvs.tok));
        vraw[u] = __ldcg(reinterpret_cast<const uint4*>(vbase + (size_t)t * a.kvs.tok));
      } else {
        kraw[u] = make_uint4(0, 0, 0, 0);
        vraw[u] = make_uint4(0, 0, 0, 0);
      }
    }
    float sc[U][GP];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[8];
      unpack8<T>(kraw[u], kf);
#pragma unroll
      for (int g = 0; g < GP; ++g) {
        float p = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) p = fmaf(kf[i], qf[g][i], p);
        sc[u][g] = p;
      }
    }
#pragma unroll
    for (int off = LPT / 2; off > 0; off >>= 1)
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int g = 0; g < GP; ++g) sc[u][g] += __shfl_xor_sync(MUI_FULL_MASK, sc[u][g], off);

#pragma unroll
    for (int g = 0; g < GP; ++g) {
      float mn = m[g];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (valid[u]) mn = fmaxf(mn, sc[u][g]);
      if (mn == -INFINITY) continue;  // nothing valid so far for this lane's stream
      const float corr = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
      m[g] = mn;
      l[g] *= corr;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] *= corr;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (valid[u]) {
          const float p = exp2f(sc[u][g] - mn);
          l[g] += p;
          float vf[8];
          unpack8<T>(vraw[u], vf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i]);
        }
      }
    }
  }

  // merge the token sub-streams of the warp (lanes with the same dlane)
#pragma unroll
  for (int off = LPT; off < 32; off <<= 1) {
#pragma unroll
    for (int g = 0; g < GP; ++g) {
      const float mo = __shfl_xor_sync(MUI_FULL_MASK, m[g], off);
      const float lo = __shfl_xor_sync(MUI_FULL_MASK, l[g], off);
      float ao[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) ao[i] = __shfl_xor_sync(MUI_FULL_MASK, acc[g][i], off);
      fd_merge(m[g], l[g], acc[g], mo, lo, ao);
    }
  }
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < GP; ++g) {
      if (dlane == 0) {
        sm_m[warp][g] = m[g];
        sm_l[warp][g] = l[g];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sm_acc[warp][g][d0 + i] = acc[g][i];
    }
  }
  __syncthreads();

  // merge the warps: thread handles (g, d) pairs
  float* part = a.partials;
  T* out = reinterpret_cast<T*>(a.out);
  for (int idx = tid; idx < G * D; idx += FD_THREADS) {
    const int g = idx / D, d = idx - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < FD_WARPS; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < FD_WARPS; ++w) {
      const float mw = sm_m[w][g];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      ll = fmaf(sm_l[w][g], f, ll);
      aa = fmaf(sm_acc[w][g][d], f, aa);
    }
    const size_t head = (size_t)b * a.Hq + (size_t)kvh * G + g;
    if (n_active == 1) {
      out[head * D + d] = Elt<T>::from_f32(ll > 0.f ? aa / ll : 0.f);
    } else {
      float* p = part + (head * a.max_splits + split) * (D + 2);
      if (d == 0) {
        p[0] = mm;
        p[1] = ll;
      }
      p[2 + d] = aa;
    }
  }
  if (n_active == 1) {
    if (tid == 0) trace_end(a.trace);
    return;
  }

  // last CTA of this (batch, kv head) merges the splits
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(&a.counters[b * a.Hkv + kvh], 1u);
    sm_is_last = (prev == static_cast<unsigned>(n_active - 1)) ? 1 : 0;
  }
  __syncthreads();
  if (!sm_is_last) {
    if (tid == 0) trace_end(a.trace);
    return;
  }
  __threadfence();
  for (int idx = tid; idx < G * D; idx += FD_THREADS) {
    const int g = idx / D, d = idx - g * D;
    const size_t head = (size_t)b * a.Hq + (size_t)kvh * G + g;
    const float* p = part + head * a.max_splits * (D + 2);
    // splits in batches of 8: issue the batch's loads back to back, then fold them (a dependent
    // load-then-max loop would pay one L2 round trip per split)
    float mm = -INFINITY, ll = 0.f, aa = 0.f;
    for (int s0 = 0; s0 < n_active; s0 += 8) {
      float ms[8], ls[8], as[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int s = min(s0 + i, n_active - 1);
        const float* ps = p + (size_t)s * (D + 2);
        ms[i] = __ldcg(ps);
        ls[i] = __ldcg(ps + 1);
        as[i] = __ldcg(ps + 2 + d);
      }
      float bm = mm;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (s0 + i < n_active) bm = fmaxf(bm, ms[i]);
      if (bm == -INFINITY) continue;
      const float c = (mm == -INFINITY) ? 0.f : exp2f(mm - bm);
      ll *= c;
      aa *= c;
      mm = bm;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (s0 + i < n_active && ms[i] != -INFINITY) {
          const float f = exp2f(ms[i] - bm);
          ll = fmaf(ls[i], f, ll);
          aa = fmaf(as[i], f, aa);
        }
      }
    }
    out[head * D + d] = Elt<T>::from_f32(ll > 0.f ? aa / ll : 0.f);
  }
  if (tid == 0) {
    a.counters[b * a.Hkv + kvh] = 0u;  // ready for the next call
    trace_end(a.trace);
  }
}

template <typename T, int D>
mui_status_t launch_fd(cudaStream_t stream, const FdArgs& a, int splits, int pdl) {
  const dim3 grid(splits, a.Hkv, a.B), block(FD_THREADS);
  if (a.G <= 1) {
    MUI_CUDA_CHECK(mui_launch(flash_decode_kernel<T, D, 1, 4>, grid, block, 0, stream, pdl, a));
  } else if (a.G <= 2) {
    MUI_CUDA_CHECK(mui_launch(flash_decode_kernel<T, D, 2, 4>, grid, block, 0, stream, pdl, a));
  } else if (a.G <= 4) {
    MUI_CUDA_CHECK(mui_launch(flash_decode_kernel<T, D, 4, 4>, grid, block, 0, stream, pdl, a));
  } else {
    MUI_CUDA_CHECK(mui_launch(flash_decode_kernel<T, D, 8, 2>, grid, block, 0, stream, pdl, a));
  }
  return MUI_OK;
}

}  // namespace

extern "C" {

size_t mui_flash_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_S) {
  (void)Hkv;
  (void)max_S;
  if (B <= 0 || Hq <= 0 || D <= 0) return FD_COUNTER_BYTES;
  return (size_t)FD_COUNTER_BYTES + (size_t)B * Hq * FD_MAX_SPLITS * (D + 2) * sizeof(float);
}

mui_status_t mui_flash_decode(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D, int S,
                              const int32_t* seq_len_dev, float scale, const void* q, const void* k, const void* v,
                              mui_strides3_t kv_strides, const void* mask, void* out, void* workspace,
                              size_t workspace_bytes, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(B >= 0 && Hq >= 1 && Hkv >= 1 && S >= 0, MUI_ERR_INVALID_ARG, "bad sizes B=%d Hq=%d Hkv=%d S=%d", B,
              Hq, Hkv, S);
  MUI_REQUIRE(D == 64 || D == 128, MUI_ERR_UNSUPPORTED, "head dim %d unsupported (64 or 128)", D);
  MUI_REQUIRE(Hq % Hkv == 0, MUI_ERR_INVALID_ARG, "Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  const int G = Hq / Hkv;
  MUI_REQUIRE(G <= 8, MUI_ERR_UNSUPPORTED, "Hq/Hkv=%d > 8 unsupported", G);
  MUI_REQUIRE(B * Hkv <= FD_COUNTER_BYTES / 4, MUI_ERR_UNSUPPORTED, "B*Hkv=%d exceeds %d", B * Hkv,
              FD_COUNTER_BYTES / 4);
  if (B == 0) return MUI_OK;
  MUI_REQUIRE(q && out && workspace, MUI_ERR_INVALID_ARG, "q, out and workspace must be non-null");
  MUI_REQUIRE(S == 0 || (k && v), MUI_ERR_INVALID_ARG, "k and v must be non-null");
  MUI_REQUIRE(workspace_bytes >= mui_flash_decode_workspace_bytes(B, Hq, Hkv, D, S), MUI_ERR_INVALID_ARG,
              "workspace too small: %zu < %zu", workspace_bytes, mui_flash_decode_workspace_bytes(B, Hq, Hkv, D, S));
  MUI_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, MUI_ERR_INVALID_ARG,
              "workspace must be 256-byte aligned");
  MUI_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) &
               15) == 0,
              MUI_ERR_INVALID_ARG, "q, k, v must be 16-byte aligned");
  MUI_REQUIRE((kv_strides.batch % 8) == 0 && (kv_strides.head % 8) == 0 && (kv_strides.tok % 8) == 0,
              MUI_ERR_INVALID_ARG, "K/V strides must be multiples of 8 elements");

  const MuiDeviceInfo* dev = mui_current_device_info();
  if (!dev) return MUI_ERR_CUDA;
  int splits = (2 * dev->sm_count + B * Hkv - 1) / (B * Hkv);
  splits = std::min(splits, (S + FD_MIN_CHUNK - 1) / FD_MIN_CHUNK);
  splits = std::max(1, std::min(splits, FD_MAX_SPLITS));

  FdArgs a;
  a.q = q; a.k = k; a.v = v; a.mask = mask; a.out = out;
  a.counters = reinterpret_cast<unsigned int*>(workspace);
  a.partials = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + FD_COUNTER_BYTES);
  a.seq_len_dev = seq_len_dev;
  a.kvs = kv_strides;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.S = S; a.G = G; a.max_splits = FD_MAX_SPLITS;
  a.trace = mui_trace_next_record(3);
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == MUI_F16)
    return D == 128 ? launch_fd<__half, 128>(st, a, splits, pdl) : launch_fd<__half, 64>(st, a, splits, pdl);
  return D == 128 ? launch_fd<__nv_bfloat16, 128>(st, a, splits, pdl)
                  : launch_fd<__nv_bfloat16, 64>(st, a, splits, pdl);
}

}  // extern "C"

// =============================================================================================
// Flash decoding without caller-provided scratch
// =============================================================================================
// Same kernel and same results as mui_flash_decode, for callers that cannot hand over a workspace because
// they are not allowed to allocate device memory themselves: a plugin host that gives the library only input
// and output buffers out of an arena it has already carved up completely, or a serving loop that must never
// reach cudaMalloc because that call synchronises the whole device. The split-KV partials and arrival
// counters live in the array below, which every GPU that loads this library keeps until the process exits.
// Its size bounds the problem: B * Hq * (D + 2) <= MUI_FD_STATIC_MAX_ROW_FLOATS (64 heads of head dim 128).
namespace {
constexpr size_t FD_STATIC_BYTES =
    (size_t)FD_COUNTER_BYTES + (size_t)MUI_FD_STATIC_MAX_ROW_FLOATS * FD_MAX_SPLITS * sizeof(float);
}
static __device__ __align__(256) unsigned char g_fd_static_ws[FD_STATIC_BYTES];

extern "C" mui_status_t mui_flash_decode_static_scratch(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv,
                                                        int D, int S, const int32_t* seq_len_dev, float scale,
                                                        const void* q, const void* k, const void* v,
                                                        mui_strides3_t kv_strides, const void* mask, void* out,
                                                        unsigned flags) {
  MUI_REQUIRE(B >= 0 && Hq >= 1 && D >= 1, MUI_ERR_INVALID_ARG, "bad sizes B=%d Hq=%d D=%d", B, Hq, D);
  const long long row_floats = (long long)B * Hq * (D + 2);
  MUI_REQUIRE(row_floats <= MUI_FD_STATIC_MAX_ROW_FLOATS, MUI_ERR_UNSUPPORTED,
              "B*Hq*(D+2) = %lld exceeds the built-in scratch (limit %d, i.e. %zu bytes); use mui_flash_decode with a "
              "caller-provided workspace",
              row_floats, MUI_FD_STATIC_MAX_ROW_FLOATS, FD_STATIC_BYTES);
  // Set-up, once per device and with that device current: `g_fd_static_ws` is a host-side stand-in in this
  // code, the kernel needs the device address behind it. The arrival counters at the front must start at
  // zero; every launch leaves them zero again.
  static void* dev_ptr[64] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  MUI_CUDA_CHECK(cudaGetDevice(&dev));
  MUI_REQUIRE(dev >= 0 && dev < 64, MUI_ERR_UNSUPPORTED, "device ordinal %d outside 0..63", dev);
  void* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev_ptr[dev] == nullptr) {
      void* p = nullptr;
      MUI_CUDA_CHECK(cudaGetSymbolAddress(&p, g_fd_static_ws));
      MUI_CUDA_CHECK(cudaMemsetAsync(p, 0, FD_COUNTER_BYTES, (cudaStream_t)stream));
      dev_ptr[dev] = p;
    }
    ws = dev_ptr[dev];
  }
  return mui_flash_decode(stream, dtype, B, Hq, Hkv, D, S, seq_len_dev, scale, q, k, v, kv_strides, mask, out, ws,
                          FD_STATIC_BYTES, flags);
}
