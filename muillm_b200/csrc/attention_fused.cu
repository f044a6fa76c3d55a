// Fused RoPE + KV-cache write + decode attention for one new token per sequence, as ONE launch with a thread
// block cluster per (KV head, sequence).
//
// The eight CTAs of a cluster share the cached tokens of their KV head (64 tokens per CTA and round: 8 warps x 2
// tokens x 4 loads in flight per lane), so up to 512 tokens cost a single round of K/V loads. Every CTA rotates
// the group's query heads and the new key itself (fp32 math, rounded to the 16-bit type like the stand-alone RoPE
// kernel stores them); cluster rank 0 writes rope(k) and v into the static cache, the last rank attends the new
// token from registers, so nothing is read back that this launch wrote. Each CTA leaves its online-softmax partial
// (m, l, acc[D]) per query head in its own shared memory; after one cluster barrier every CTA merges a slice of the
// output by reading all eight partials through distributed shared memory and writes the final 16-bit values.
// No global scratch, no atomics, no second kernel: the dependent chain is {state + q/k/v} -> {cos/sin + K/V} ->
// cluster barrier -> DSMEM merge.
//
// Replaces the pair muillm_rope_forward_static_cache + flash_decode_no_mask (csrc/rope/rotary.cu:603-756,
// csrc/attention/flash_decoding.cu:288-305) on the decode path; the stand-alone kernels stay for the other uses
// (prefill RoPE, masks, strided views).
#include "common.cuh"

#include <algorithm>

MUI_STATUS_ACCESSOR(attention_fused)

namespace {

constexpr int FA_THREADS = 256;
constexpr int FA_WARPS = 8;
constexpr int FA_CLUSTER = 8;
constexpr int FA_D = 128;

struct FaArgs {
  const void* qkv;            // [B, (Hq + 2 Hkv) * D] packed q rows, k rows, v rows of the new token
  const void *cos_t, *sin_t;  // [max_pos, D]
  const long long* position_ids;    // [B] rope position of the new token
  const long long* cache_position;  // [1] cache row the new token is written to
  const int32_t* seq_len_dev;       // tokens attended including the new one (= cache_position + 1)
  void *k_cache, *v_cache;    // [B, Hkv, max_seq, D]
  void* out;                  // [B, Hq * D]
  float scale_log2;
  int B, Hq, Hkv, max_seq, G;
  unsigned long long* trace;
};

__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(const float* local_ptr, unsigned rank) {
  const uint32_t laddr = smem_u32(local_ptr);
  uint32_t raddr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(laddr), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr) : "memory");
  return v;
}

template <typename T>
__device__ __forceinline__ void fa_rope8(float (&x)[8], const float (&c)[8], const float (&s)[8], bool low_half) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float p = __shfl_xor_sync(MUI_FULL_MASK, x[i], 8);
    const float r = low_half ? fmaf(x[i], c[i], -p * s[i]) : fmaf(x[i], c[i], p * s[i]);
    x[i] = Elt<T>::to_f32(Elt<T>::from_f32(r));
  }
}

__device__ __forceinline__ void fa_merge(float& m, float& l, float (&acc)[8], float mo, float lo,
                                         const float (&acco)[8]) {
  const float mn = fmaxf(m, mo);
  const float fa = (m == -INFINITY) ? 0.f : exp2f(m - mn);
  const float fb = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
  l = l * fa + lo * fb;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = acc[i] * fa + acco[i] * fb;
  m = mn;
}

template <typename T, int GP, int U>
__global__ void __launch_bounds__(FA_THREADS) rope_flash_decode_cluster_kernel(const FaArgs a) {
  constexpr int LPT = FA_D / 8, TPW = 32 / LPT;
  __shared__ float sm_m[FA_WARPS][GP];
  __shared__ float sm_l[FA_WARPS][GP];
  __shared__ float sm_acc[FA_WARPS][GP][FA_D];
  __shared__ float part_m[GP], part_l[GP];
  __shared__ float part_acc[GP][FA_D];

  trace_start(a.trace);
  pdl_wait_prior_grid();
  pdl_launch_dependents();

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned rank = cluster_ctarank();
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.G;
  const int sub = lane / LPT, dlane = lane % LPT, d0 = dlane * 8;
  const bool low = dlane < (LPT / 2);

  // first round of loads: state and the new token's q, k, v (independent of each other)
  const long long pos_id = __ldcg(a.position_ids + b);
  const long long cache_pos = __ldcg(a.cache_position);
  const int S = min(max(__ldcg(a.seq_len_dev), 1), a.max_seq);
  const int cached = S - 1;
  const T* row = reinterpret_cast<const T*>(a.qkv) + (size_t)b * (a.Hq + 2 * a.Hkv) * FA_D;
  uint4 q_raw[GP];
#pragma unroll
  for (int g = 0; g < GP; ++g)
    q_raw[g] = (g < G) ? ld_act16(row + ((size_t)kvh * G + g) * FA_D + d0) : make_uint4(0, 0, 0, 0);
  const uint4 k_raw = ld_act16(row + ((size_t)a.Hq + kvh) * FA_D + d0);
  const uint4 v_new = ld_act16(row + ((size_t)a.Hq + a.Hkv + kvh) * FA_D + d0);

  // second round: cos/sin of the position and the cached K/V rows of this CTA's first tokens
  T* kc = reinterpret_cast<T*>(a.k_cache) + ((size_t)b * a.Hkv + kvh) * a.max_seq * FA_D;
  T* vc = reinterpret_cast<T*>(a.v_cache) + ((size_t)b * a.Hkv + kvh) * a.max_seq * FA_D;
  float cs[8], sn[8];
  unpack8<T>(ld_cached16(reinterpret_cast<const T*>(a.cos_t) + (size_t)pos_id * FA_D + d0), cs);
  unpack8<T>(ld_cached16(reinterpret_cast<const T*>(a.sin_t) + (size_t)pos_id * FA_D + d0), sn);

  float m[GP], l[GP], acc[GP][8];
#pragma unroll
  for (int g = 0; g < GP; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }
  float qf[GP][8];
  bool q_ready = false;
  uint4 k_new = make_uint4(0, 0, 0, 0);

  auto prepare_q = [&]() {
#pragma unroll
    for (int g = 0; g < GP; ++g) {
      unpack8<T>(q_raw[g], qf[g]);
      fa_rope8<T>(qf[g], cs, sn, low);
#pragma unroll
      for (int i = 0; i < 8; ++i) qf[g][i] *= a.scale_log2;
    }
    float kn[8];
    unpack8<T>(k_raw, kn);
    fa_rope8<T>(kn, cs, sn, low);
    k_new = pack8<T>(kn);
    q_ready = true;
  };

  auto fold = [&](const uint4 (&kraw)[U], const uint4 (&vraw)[U], const bool (&valid)[U]) {
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
      if (mn == -INFINITY) continue;
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
  };

  // round i: token = ((i * CLUSTER + rank) * U + u) * (WARPS * TPW) + warp * TPW + sub
  constexpr int PER_CTA_ROUND = FA_WARPS * TPW * U;
  for (int base = (int)rank * PER_CTA_ROUND; base < cached || !q_ready; base += FA_CLUSTER * PER_CTA_ROUND) {
    uint4 kraw[U], vraw[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = base + u * FA_WARPS * TPW + warp * TPW + sub;
      valid[u] = t < cached;
      if (valid[u]) {
        kraw[u] = __ldcg(reinterpret_cast<const uint4*>(kc + (size_t)t * FA_D + d0));
        vraw[u] = __ldcg(reinterpret_cast<const uint4*>(vc + (size_t)t * FA_D + d0));
      } else {
        kraw[u] = make_uint4(0, 0, 0, 0);
        vraw[u] = make_uint4(0, 0, 0, 0);
      }
    }
    if (!q_ready) prepare_q();  // rotates q and the new k while the first K/V loads are in flight
    fold(kraw, vraw, valid);
  }

  // the new token: written to the cache by rank 0, attended from registers by the last rank
  if (rank == 0 && warp == 0 && sub == 0) {
    *reinterpret_cast<uint4*>(kc + (size_t)cache_pos * FA_D + d0) = k_new;
    *reinterpret_cast<uint4*>(vc + (size_t)cache_pos * FA_D + d0) = v_new;
  }
  if (rank == FA_CLUSTER - 1 && warp == 0) {
    uint4 kraw[U], vraw[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      kraw[u] = k_new;
      vraw[u] = v_new;
      valid[u] = (u == 0) && (sub == 0);
    }
    fold(kraw, vraw, valid);
  }

  // warp sub-streams, then warps -> this CTA's partial in shared memory
#pragma unroll
  for (int off = LPT; off < 32; off <<= 1) {
#pragma unroll
    for (int g = 0; g < GP; ++g) {
      const float mo = __shfl_xor_sync(MUI_FULL_MASK, m[g], off);
      const float lo = __shfl_xor_sync(MUI_FULL_MASK, l[g], off);
      float ao[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) ao[i] = __shfl_xor_sync(MUI_FULL_MASK, acc[g][i], off);
      fa_merge(m[g], l[g], acc[g], mo, lo, ao);
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
  for (int idx = tid; idx < GP * FA_D; idx += FA_THREADS) {
    const int g = idx / FA_D, d = idx - g * FA_D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) {
      const float mw = sm_m[w][g];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      ll = fmaf(sm_l[w][g], f, ll);
      aa = fmaf(sm_acc[w][g][d], f, aa);
    }
    if (d == 0) {
      part_m[g] = mm;
      part_l[g] = ll;
    }
    part_acc[g][d] = aa;
  }
  cluster_sync_all();

  // every CTA merges its slice of the G * D outputs over the eight partials (distributed shared memory)
  T* out = reinterpret_cast<T*>(a.out) + ((size_t)b * a.Hq + (size_t)kvh * G) * FA_D;
  const int total = G * FA_D;
  const int e0 = total * (int)rank / FA_CLUSTER, e1 = total * ((int)rank + 1) / FA_CLUSTER;
  for (int e = e0 + tid; e < e1; e += FA_THREADS) {
    const int g = e / FA_D, d = e - g * FA_D;
    float pm[FA_CLUSTER], pl[FA_CLUSTER], pa[FA_CLUSTER];
#pragma unroll
    for (int r = 0; r < FA_CLUSTER; ++r) {
      pm[r] = ld_dsmem_f32(&part_m[g], r);
      pl[r] = ld_dsmem_f32(&part_l[g], r);
      pa[r] = ld_dsmem_f32(&part_acc[g][d], r);
    }
    float mm = -INFINITY;
#pragma unroll
    for (int r = 0; r < FA_CLUSTER; ++r) mm = fmaxf(mm, pm[r]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int r = 0; r < FA_CLUSTER; ++r) {
      const float f = (pm[r] == -INFINITY) ? 0.f : exp2f(pm[r] - mm);
      ll = fmaf(pl[r], f, ll);
      aa = fmaf(pa[r], f, aa);
    }
    out[e] = Elt<T>::from_f32(ll > 0.f ? aa / ll : 0.f);
  }
  // nobody leaves while a peer may still read its shared memory
  cluster_sync_all();
  if (tid == 0) trace_end(a.trace);
}

template <typename T, int GP, int U>
mui_status_t launch_fa(cudaStream_t stream, const FaArgs& a, int pdl) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(FA_CLUSTER, a.Hkv, a.B);
  cfg.blockDim = dim3(FA_THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = FA_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  MUI_CUDA_CHECK(cudaLaunchKernelEx(&cfg, rope_flash_decode_cluster_kernel<T, GP, U>, a));
  return MUI_OK;
}

template <typename T>
mui_status_t launch_fa_g(cudaStream_t stream, const FaArgs& a, int pdl) {
  if (a.G <= 1) return launch_fa<T, 1, 4>(stream, a, pdl);
  if (a.G <= 2) return launch_fa<T, 2, 4>(stream, a, pdl);
  if (a.G <= 4) return launch_fa<T, 4, 4>(stream, a, pdl);
  return launch_fa<T, 8, 2>(stream, a, pdl);
}

}  // namespace

extern "C" mui_status_t mui_rope_flash_decode(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D,
                                              int max_seq, const void* qkv, const void* cos_table,
                                              const void* sin_table, const int64_t* position_ids,
                                              const int64_t* cache_position, const int32_t* seq_len_dev,
                                              float scale, void* k_cache, void* v_cache, void* out, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(D == FA_D, MUI_ERR_UNSUPPORTED, "head dim %d unsupported by the fused kernel (128)", D);
  MUI_REQUIRE(B >= 1 && Hq >= 1 && Hkv >= 1 && Hq % Hkv == 0 && Hq / Hkv <= 8 && max_seq >= 1, MUI_ERR_INVALID_ARG,
              "bad sizes B=%d Hq=%d Hkv=%d max_seq=%d", B, Hq, Hkv, max_seq);
  MUI_REQUIRE(qkv && cos_table && sin_table && position_ids && cache_position && seq_len_dev && k_cache && v_cache &&
                  out,
              MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) |
                reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(cos_table) |
                reinterpret_cast<uintptr_t>(sin_table) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
              MUI_ERR_INVALID_ARG, "pointers must be 16-byte aligned");
  FaArgs a;
  a.qkv = qkv;
  a.cos_t = cos_table;
  a.sin_t = sin_table;
  a.position_ids = reinterpret_cast<const long long*>(position_ids);
  a.cache_position = reinterpret_cast<const long long*>(cache_position);
  a.seq_len_dev = seq_len_dev;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.out = out;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.B = B;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.max_seq = max_seq;
  a.G = Hq / Hkv;
  a.trace = mui_trace_next_record(3);
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  if (dtype == MUI_F16) return launch_fa_g<__half>((cudaStream_t)stream, a, pdl);
  return launch_fa_g<__nv_bfloat16>((cudaStream_t)stream, a, pdl);
}
