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
#include "gemv_common.cuh"

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
  // Llama-4 prologue (l4 != 0) instead of the rotate-half rope: interleaved-pair rotation from an fp32 table, L2
  // norm of q and k over the head dim, temperature scale of q — any subset (FA_L4_* bits), each stage rounded to the
  // 16-bit type like the stand-alone prologue kernel. With chunk > 0 the layer's cache is a ring of `max_seq` rows
  // indexed by position % chunk and the token attends the rows of its own chunk only.
  const float* freqs;  // [max_pos, D/2, 2] (cos, sin)
  int max_pos;         // rows of the rotary table
  // token-split variant of the one-CTA-per-KV-head kernel (gridDim.z > 1): arrival counters [B * Hkv] (zero between
  // launches) and fp32 partials [B, Hq, max_splits, D + 2] = (max, denominator, unnormalised output)
  unsigned int* counters;
  float* partials;
  int max_splits;
  int l4, chunk;
  float eps, attn_scale, floor_scale;
};

constexpr int FA_L4_ON = 1, FA_L4_ROPE = 2, FA_L4_NORM = 4, FA_L4_TEMP = 8;

// Llama-4 prologue on the 8 consecutive head-dim elements a lane holds (4 interleaved pairs); the 16 lanes of a
// half-warp hold one 128-element row, so the L2 norm sums over lane bits 0-3. `temp` applies to queries only.
template <typename T>
__device__ __forceinline__ void fa_l4_prologue8(float (&x)[8], const float2 (&fr)[4], int l4, float eps, bool is_q,
                                                float temp) {
  if (l4 & FA_L4_ROPE) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float re = x[2 * j], im = x[2 * j + 1];
      const float r = re * fr[j].x - im * fr[j].y;
      const float i = re * fr[j].y + im * fr[j].x;
      x[2 * j] = Elt<T>::to_f32(Elt<T>::from_f32(r));
      x[2 * j + 1] = Elt<T>::to_f32(Elt<T>::from_f32(i));
    }
  }
  if (l4 & FA_L4_NORM) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += x[2 * j] * x[2 * j] + x[2 * j + 1] * x[2 * j + 1];
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) ss += __shfl_xor_sync(MUI_FULL_MASK, ss, o);
    const float r = rsqrtf(ss / static_cast<float>(FA_D) + eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = Elt<T>::to_f32(Elt<T>::from_f32(x[i] * r));
  }
  if ((l4 & FA_L4_TEMP) && is_q) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = Elt<T>::to_f32(Elt<T>::from_f32(x[i] * temp));
  }
}
__device__ __forceinline__ float fa_l4_temperature(long long pos, float attn_scale, float floor_scale) {
  return log1pf(floorf((static_cast<float>(pos) + 1.0f) / floor_scale)) * attn_scale + 1.0f;
}

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
  const long long abs_pos = __ldcg(a.cache_position);
  // Llama-4: the row and the attended length follow from the position (ring of `chunk` rows, or a plain cache)
  const long long cache_pos = (a.l4 && a.chunk > 0) ? abs_pos % a.chunk : abs_pos;
  const int S = a.l4 ? static_cast<int>(min(cache_pos + 1, (long long)a.max_seq))
                     : min(max(__ldcg(a.seq_len_dev), 1), a.max_seq);
  // Past the end of the cache or of the rotary tables: record it and leave, writing nothing. The values are the
  // same for every CTA of the cluster, so all of them leave before the first cluster barrier.
  if (abs_pos < 0 || cache_pos >= a.max_seq || pos_id < 0 || pos_id >= a.max_pos) {
    if (tid == 0) mui_dev_set_status(MUI_DEV_BAD_LENGTH, static_cast<unsigned>(abs_pos));
    return;
  }
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
  float2 fr[4];
  float temp = 1.f;
  if (a.l4) {
    float4 f01 = make_float4(1.f, 0.f, 1.f, 0.f), f23 = f01;
    if (a.l4 & FA_L4_ROPE) {
      const float4* f4 = reinterpret_cast<const float4*>(a.freqs + ((size_t)pos_id * (FA_D / 2) + d0 / 2) * 2);
      f01 = __ldg(f4);
      f23 = __ldg(f4 + 1);
    }
    fr[0] = make_float2(f01.x, f01.y);
    fr[1] = make_float2(f01.z, f01.w);
    fr[2] = make_float2(f23.x, f23.y);
    fr[3] = make_float2(f23.z, f23.w);
    if (a.l4 & FA_L4_TEMP) temp = fa_l4_temperature(abs_pos, a.attn_scale, a.floor_scale);
  } else {
    unpack8<T>(ld_cached16(reinterpret_cast<const T*>(a.cos_t) + (size_t)pos_id * FA_D + d0), cs);
    unpack8<T>(ld_cached16(reinterpret_cast<const T*>(a.sin_t) + (size_t)pos_id * FA_D + d0), sn);
  }

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
      if (a.l4) fa_l4_prologue8<T>(qf[g], fr, a.l4, a.eps, true, temp);
      else fa_rope8<T>(qf[g], cs, sn, low);
#pragma unroll
      for (int i = 0; i < 8; ++i) qf[g][i] *= a.scale_log2;
    }
    float kn[8];
    unpack8<T>(k_raw, kn);
    if (a.l4) fa_l4_prologue8<T>(kn, fr, a.l4, a.eps, false, 1.f);
    else fa_rope8<T>(kn, cs, sn, low);
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

// ---------------------------------------------------------------------------------------------------------------
// Short-context variant: ONE CTA per (KV head, sequence), no cluster, so the launch can become resident while the
// QKV projection is still running (that GEMV leaves Hkv*B SMs free for it, see GemvArgs::reserve_sms). Before it
// waits for the projection it reads the decode state (final since the previous step's arg-max, which finished
// before the projection was allowed to start) and pulls the whole K/V history of its head into shared memory with
// 16-byte asynchronous copies into rows padded to 272 bytes (conflict-free ldmatrix); after the wait only the new
// token's q/k/v (one L2 round trip) and the arithmetic are left, and the arithmetic runs on the tensor cores with
// the query heads of the group as the m dimension (padded to 16):
//   pass 1   S^T[head, token] = Q[head, :] . K[token, :]      mma m16n8k16, A = q fragments, B = K rows (ldmatrix)
//   pass 2   O[head, :] = P[head, tokens] . V[tokens, :]       A = exp2(s - max) as a 16-bit value + 16-bit correction,
//                                                              B = V rows through ldmatrix.trans; warps split the
//                                                              tokens and add their partials; denominators in fp32
// At most RA_ROWS tokens (the new one included); a longer history records MUI_DEV_BAD_LENGTH and writes nothing —
// the caller picks this variant (MUI_FLAG_SHORT_CONTEXT) only when it can bound the length.
constexpr int RA_ROWS = 384;
constexpr int RA_PITCH = FA_D + 8;  // elements

template <int GP> constexpr size_t ra_smem_bytes() {
  return (size_t)2 * RA_ROWS * RA_PITCH * 2 + (size_t)GP * FA_D * 2 + (size_t)GP * RA_ROWS * 4 +
         (size_t)2 * FA_WARPS * GP * 4 + 32;
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}

template <typename T, int GP>
__global__ void __launch_bounds__(FA_THREADS) rope_flash_decode_resident_kernel(const FaArgs a) {
  extern __shared__ __align__(128) unsigned char ra_smem[];
  T* Ks = reinterpret_cast<T*>(ra_smem);
  T* Vs = Ks + (size_t)RA_ROWS * RA_PITCH;
  T* Qs = Vs + (size_t)RA_ROWS * RA_PITCH;                         // [GP][D] rotated queries
  float* Sc = reinterpret_cast<float*>(Qs + GP * FA_D);            // [GP][RA_ROWS] scores * scale * log2(e)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int G = a.G;
  trace_start(a.trace);

  // ---- before the dependency wait: decode state + K/V history (nothing the previous kernel writes) ----
  const long long pos_id = __ldcg(a.position_ids + b);
  const long long abs_pos = __ldcg(a.cache_position);
  const long long cache_pos = (a.l4 && a.chunk > 0) ? abs_pos % a.chunk : abs_pos;
  const int S_all = a.l4 ? static_cast<int>(min(cache_pos + 1, (long long)a.max_seq))
                         : min(max(__ldcg(a.seq_len_dev), 1), a.max_seq);
  // Token split (gridDim.z > 1): this CTA attends tokens [tok_begin, tok_begin + S) of the S_all in view; the CTA
  // whose range ends the sequence holds the new token. Chunks are multiples of 16 tokens and at least 64, so short
  // sequences use few of the launched CTAs.
  const int split = blockIdx.z;
  int chunk = S_all, n_active = 1;
  if (gridDim.z > 1) {
    chunk = max(64, ((S_all + (int)gridDim.z - 1) / (int)gridDim.z + 15) & ~15);
    n_active = (S_all + chunk - 1) / chunk;
  }
  if (split >= n_active) return;
  const int tok_begin = split * chunk;
  const int S = min(S_all, tok_begin + chunk) - tok_begin;  // rows of this CTA, the new token included if it owns it
  const bool own_new = (split == n_active - 1);
  if (S > RA_ROWS || abs_pos < 0 || cache_pos >= a.max_seq || pos_id < 0 || pos_id >= a.max_pos) {
    if (tid == 0) mui_dev_set_status(MUI_DEV_BAD_LENGTH, static_cast<unsigned>(S_all));
    return;
  }
  const int cached = own_new ? S - 1 : S;  // rows that come from the cache
  T* kc = reinterpret_cast<T*>(a.k_cache) + ((size_t)b * a.Hkv + kvh) * a.max_seq * FA_D;
  T* vc = reinterpret_cast<T*>(a.v_cache) + ((size_t)b * a.Hkv + kvh) * a.max_seq * FA_D;
  // 16-byte asynchronous copies (cp.async): each lands at its padded position; a bulk copy could not pad, and one
  // bulk copy per row costs the copy engine ~15 ns each
  {
    const uint32_t ks_u = smem_u32(Ks), vs_u = smem_u32(Vs);
    const int pieces = cached * (FA_D / 8);
    for (int i = tid; i < pieces; i += FA_THREADS) {
      const int r = i >> 4, c = (i & 15) * 8;
      const uint32_t so = static_cast<uint32_t>((r * RA_PITCH + c) * 2);
      const size_t go = (size_t)(tok_begin + r) * FA_D + c;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ks_u + so), "l"(kc + go) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vs_u + so), "l"(vc + go) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // rows of the last 16-token slab past the sequence multiply probabilities that are zero: they must be finite
  {
    const int r = S + (tid >> 4);
    if (r < ((S + 15) & ~15)) *reinterpret_cast<uint4*>(Vs + (size_t)r * RA_PITCH + (tid & 15) * 8) = make_uint4(0, 0, 0, 0);
  }
  constexpr int LPT = FA_D / 8;  // 16 lanes hold one 128-element row
  const int sub = lane / LPT, dlane = lane % LPT, d0 = dlane * 8;
  float cs[8], sn[8];
  float2 fr[4];
  float temp = 1.f;
  if (a.l4) {
    float4 f01 = make_float4(1.f, 0.f, 1.f, 0.f), f23 = f01;
    if (a.l4 & FA_L4_ROPE) {
      const float4* f4 = reinterpret_cast<const float4*>(a.freqs + ((size_t)pos_id * (FA_D / 2) + d0 / 2) * 2);
      f01 = __ldg(f4);
      f23 = __ldg(f4 + 1);
    }
    fr[0] = make_float2(f01.x, f01.y);
    fr[1] = make_float2(f01.z, f01.w);
    fr[2] = make_float2(f23.x, f23.y);
    fr[3] = make_float2(f23.z, f23.w);
    if (a.l4 & FA_L4_TEMP) temp = fa_l4_temperature(abs_pos, a.attn_scale, a.floor_scale);
  } else {
    unpack8<T>(ld_cached16(reinterpret_cast<const T*>(a.cos_t) + (size_t)pos_id * FA_D + d0), cs);
    unpack8<T>(ld_cached16(reinterpret_cast<const T*>(a.sin_t) + (size_t)pos_id * FA_D + d0), sn);
  }
  pdl_launch_dependents();
  pdl_wait_prior_grid();
  if (tid == 0) trace_mark(a.trace, 2, false);

  // ---- the new token: half-warp `slot` rotates query head `slot` (< G), the key (== G) or copies the value (== G+1) ----
  {
    const int slot = warp * 2 + sub;
    const T* row = reinterpret_cast<const T*>(a.qkv) + (size_t)b * (a.Hq + 2 * a.Hkv) * FA_D;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (slot < G) raw = ld_act16(row + ((size_t)kvh * G + slot) * FA_D + d0);
    else if (slot == G) raw = ld_act16(row + ((size_t)a.Hq + kvh) * FA_D + d0);
    else if (slot == G + 1) raw = ld_act16(row + ((size_t)a.Hq + a.Hkv + kvh) * FA_D + d0);
    float x[8];
    unpack8<T>(raw, x);
    // every lane takes part in the shuffles
    if (a.l4) fa_l4_prologue8<T>(x, fr, a.l4, a.eps, slot < G, temp);
    else fa_rope8<T>(x, cs, sn, dlane < (LPT / 2));
    const uint4 rot = pack8<T>(x);
    if (slot < G) {
      *reinterpret_cast<uint4*>(Qs + (size_t)slot * FA_D + d0) = rot;
    } else if (slot == G && own_new) {
      *reinterpret_cast<uint4*>(Ks + (size_t)cached * RA_PITCH + d0) = rot;
      *reinterpret_cast<uint4*>(kc + (size_t)cache_pos * FA_D + d0) = rot;
    } else if (slot == G + 1 && own_new) {
      *reinterpret_cast<uint4*>(Vs + (size_t)cached * RA_PITCH + d0) = raw;
      *reinterpret_cast<uint4*>(vc + (size_t)cache_pos * FA_D + d0) = raw;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's pieces of the history have landed
  __syncthreads();

  const int hrow = lane >> 2, cpair = (lane & 3) * 2;  // fragment coordinates of this lane
  const bool real_head = hrow < G;

  // ---- pass 1: scores; warp w takes token tiles w, w + 8, ... and keeps the running maximum of its tiles ----
  float* wmax = Sc + GP * RA_ROWS;         // [WARPS][GP]
  float* wsum = wmax + FA_WARPS * GP;      // [WARPS][GP]
  {
    uint32_t qa[8][2];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qa[kk][0] = real_head ? *reinterpret_cast<const uint32_t*>(Qs + (size_t)hrow * FA_D + kk * 16 + cpair) : 0u;
      qa[kk][1] = real_head ? *reinterpret_cast<const uint32_t*>(Qs + (size_t)hrow * FA_D + kk * 16 + 8 + cpair) : 0u;
    }
    const int ntile = (S + 7) >> 3;
    // ldmatrix: lane gives row (lane % 8) of matrix (lane / 8); matrices = d offsets 0, 8, 16, 24 of a 32-wide k pair
    const uint32_t k_base = smem_u32(Ks) + static_cast<uint32_t>(((lane & 7) * RA_PITCH + (lane >> 3) * 8) * 2);
    float mx = -INFINITY;
    for (int j = warp; j < ntile; j += FA_WARPS) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of four dependent mma
      const uint32_t tile_addr = k_base + static_cast<uint32_t>(j * 8 * RA_PITCH * 2);
#pragma unroll
      for (int k2 = 0; k2 < 4; ++k2) {
        uint32_t r[4];
        ldmatrix_x4(r, tile_addr + k2 * 64);
        const uint32_t a0[4] = {qa[2 * k2][0], 0u, qa[2 * k2][1], 0u};
        const uint32_t a1[4] = {qa[2 * k2 + 1][0], 0u, qa[2 * k2 + 1][1], 0u};
        MmaOp<T>::run(acc, a0, r[0], r[1]);
        MmaOp<T>::run(acc2, a1, r[2], r[3]);
      }
      if (real_head) {
        const int t0 = j * 8 + cpair;
        const float s0 = (acc[0] + acc2[0]) * a.scale_log2, s1 = (acc[1] + acc2[1]) * a.scale_log2;
        if (t0 < S) {
          Sc[hrow * RA_ROWS + t0] = s0;
          mx = fmaxf(mx, s0);
        }
        if (t0 + 1 < S) {
          Sc[hrow * RA_ROWS + t0 + 1] = s1;
          mx = fmaxf(mx, s1);
        }
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(MUI_FULL_MASK, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(MUI_FULL_MASK, mx, 2));
    if (real_head && (lane & 3) == 0) wmax[warp * GP + hrow] = mx;
  }
  __syncthreads();

  // ---- pass 2: O = P V; warp w takes 16-token slabs w, w + 8, ... for all 128 columns (16 independent accumulator
  // tiles), then the warps' partial outputs and denominators are summed through shared memory (the K rows are no
  // longer needed, their space holds the partials). The probabilities enter the tensor cores as a 16-bit value plus
  // a 16-bit correction (two mma per tile), which keeps them at fp32-like accuracy. ----
  float* red = reinterpret_cast<float*>(Ks);  // [WARPS][GP][D]
  {
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const float* sc = Sc + (real_head ? hrow : 0) * RA_ROWS;
    float mh = -INFINITY;
    if (real_head) {
#pragma unroll
      for (int w = 0; w < FA_WARPS; ++w) mh = fmaxf(mh, wmax[w * GP + hrow]);
    }
    // ldmatrix.trans: matrix (lane / 8): bit 0 = token half (+8 rows), bit 1 = column tile (+8 columns)
    const uint32_t v_base = smem_u32(Vs) +
        static_cast<uint32_t>((((lane & 7) + ((lane >> 3) & 1) * 8) * RA_PITCH + (lane >> 4) * 8) * 2);
    const int nslab = (S + 15) >> 4;
    float lsum = 0.f;
    for (int t = warp; t < nslab; t += FA_WARPS) {
      uint32_t ph[4] = {0u, 0u, 0u, 0u}, pl[4] = {0u, 0u, 0u, 0u};
      if (real_head) {
        const int t0 = t * 16 + cpair;
        const float p0 = (t0 < S) ? exp2f(sc[t0] - mh) : 0.f;
        const float p1 = (t0 + 1 < S) ? exp2f(sc[t0 + 1] - mh) : 0.f;
        const float p2 = (t0 + 8 < S) ? exp2f(sc[t0 + 8] - mh) : 0.f;
        const float p3 = (t0 + 9 < S) ? exp2f(sc[t0 + 9] - mh) : 0.f;
        lsum += (p0 + p1) + (p2 + p3);
        ph[0] = Elt<T>::pack2(p0, p1);
        ph[2] = Elt<T>::pack2(p2, p3);
        const float2 h01 = Elt<T>::unpack2(ph[0]), h23 = Elt<T>::unpack2(ph[2]);
        pl[0] = Elt<T>::pack2(p0 - h01.x, p1 - h01.y);
        pl[2] = Elt<T>::pack2(p2 - h23.x, p3 - h23.y);
      }
      const uint32_t slab_addr = v_base + static_cast<uint32_t>(t * 16 * RA_PITCH * 2);
#pragma unroll
      for (int n2 = 0; n2 < 8; ++n2) {
        uint32_t r[4];
        ldmatrix_x4_trans(r, slab_addr + n2 * 32);
        MmaOp<T>::run(o[2 * n2], ph, r[0], r[1]);
        MmaOp<T>::run(o[2 * n2 + 1], ph, r[2], r[3]);
        MmaOp<T>::run(o[2 * n2], pl, r[0], r[1]);
        MmaOp<T>::run(o[2 * n2 + 1], pl, r[2], r[3]);
      }
    }
    lsum += __shfl_xor_sync(MUI_FULL_MASK, lsum, 1);
    lsum += __shfl_xor_sync(MUI_FULL_MASK, lsum, 2);
    if (real_head) {
      if ((lane & 3) == 0) wsum[warp * GP + hrow] = lsum;
      float* dst = red + ((size_t)warp * GP + hrow) * FA_D + cpair;
#pragma unroll
      for (int n = 0; n < 16; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][0], o[n][1]);
    }
  }
  __syncthreads();
  if (tid == 0) trace_mark(a.trace, 3, true);
  T* out = reinterpret_cast<T*>(a.out) + ((size_t)b * a.Hq + (size_t)kvh * G) * FA_D;
  for (int idx = tid; idx < G * FA_D; idx += FA_THREADS) {
    const int g = idx / FA_D, d = idx - g * FA_D;
    float v = 0.f, l = 0.f, mh = -INFINITY;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) {
      v += red[((size_t)w * GP + g) * FA_D + d];
      l += wsum[w * GP + g];
      mh = fmaxf(mh, wmax[w * GP + g]);
    }
    if (n_active == 1) {
      out[idx] = Elt<T>::from_f32(l > 0.f ? v / l : 0.f);
    } else {
      float* p = a.partials + ((((size_t)b * a.Hq + (size_t)kvh * G + g) * a.max_splits) + split) * (FA_D + 2);
      if (d == 0) {
        p[0] = mh;
        p[1] = l;
      }
      p[2 + d] = v;
    }
  }
  if (n_active == 1) {
    if (tid == 0) trace_end(a.trace);
    return;
  }
  // the last CTA of this (sequence, KV head) to arrive merges the splits by log-sum-exp
  __shared__ int is_last_s;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(&a.counters[b * a.Hkv + kvh], 1u);
    is_last_s = (prev == static_cast<unsigned>(n_active - 1)) ? 1 : 0;
  }
  __syncthreads();
  if (!is_last_s) {
    if (tid == 0) trace_end(a.trace);
    return;
  }
  __threadfence();
  for (int idx = tid; idx < G * FA_D; idx += FA_THREADS) {
    const int g = idx / FA_D, d = idx - g * FA_D;
    const float* p = a.partials + (((size_t)b * a.Hq + (size_t)kvh * G + g) * a.max_splits) * (FA_D + 2);
    float mm = -INFINITY, ll = 0.f, aa = 0.f;
    for (int s0 = 0; s0 < n_active; s0 += 8) {  // loads of eight splits back to back, then the fold
      float ms[8], ls[8], as[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float* ps = p + (size_t)min(s0 + i, n_active - 1) * (FA_D + 2);
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
    out[idx] = Elt<T>::from_f32(ll > 0.f ? aa / ll : 0.f);
  }
  if (tid == 0) {
    a.counters[b * a.Hkv + kvh] = 0u;  // ready for the next launch
    trace_end(a.trace);
  }
}

template <typename T, int GP>
mui_status_t launch_ra(cudaStream_t stream, const FaArgs& a, int pdl, int splits) {
  static bool configured = false;  // per instantiation
  auto kern = rope_flash_decode_resident_kernel<T, GP>;
  if (!configured) {
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ra_smem_bytes<GP>()));
    configured = true;
  }
  MUI_CUDA_CHECK(mui_launch(kern, dim3(a.Hkv, a.B, splits), dim3(FA_THREADS), ra_smem_bytes<GP>(), stream, pdl, a));
  return MUI_OK;
}

template <typename T>
mui_status_t launch_ra_g(cudaStream_t stream, const FaArgs& a, int pdl, int splits = 1) {
  if (a.G <= 1) return launch_ra<T, 1>(stream, a, pdl, splits);
  if (a.G <= 2) return launch_ra<T, 2>(stream, a, pdl, splits);
  if (a.G <= 4) return launch_ra<T, 4>(stream, a, pdl, splits);
  return launch_ra<T, 8>(stream, a, pdl, splits);
}

// Workspace of the token-split variant: the layout of mui_flash_decode_workspace_bytes (4 KiB of arrival counters that
// are zero between launches, then fp32 partials [B, Hq, 64, D + 2]).
constexpr int RA_MAX_SPLITS = 64;
constexpr int RA_SPLIT_ROWS = 256;  // tokens per CTA the split count is sized for (a CTA holds up to RA_ROWS)
constexpr size_t RA_COUNTER_BYTES = 4096;

// Picks the kernel variant for `max_attended` tokens: 0 = cluster kernel, 1 = one CTA per KV head, n > 1 = n-way
// token split of the latter (needs the workspace).
int ra_pick_splits(unsigned flags, int max_attended, int B, int Hq, int Hkv, const void* workspace,
                   size_t workspace_bytes) {
  if (flags & MUI_FLAG_SHORT_CONTEXT) return 1;
  if (!(flags & MUI_FLAG_SPLIT_CONTEXT) || workspace == nullptr) return 0;
  const int splits = (max_attended + RA_SPLIT_ROWS - 1) / RA_SPLIT_ROWS;
  const size_t need = RA_COUNTER_BYTES + (size_t)B * Hq * RA_MAX_SPLITS * (FA_D + 2) * sizeof(float);
  if (splits <= 1) return 1;
  if (splits > RA_MAX_SPLITS || workspace_bytes < need || (size_t)B * Hkv * 4 > RA_COUNTER_BYTES) return 0;
  return splits;
}
void ra_bind_workspace(FaArgs& a, void* workspace) {
  a.counters = reinterpret_cast<unsigned int*>(workspace);
  a.partials = workspace ? reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + RA_COUNTER_BYTES)
                         : nullptr;
  a.max_splits = RA_MAX_SPLITS;
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
  return mui_rope_flash_decode_ws(stream, dtype, B, Hq, Hkv, D, max_seq, qkv, cos_table, sin_table, position_ids,
                                  cache_position, seq_len_dev, scale, k_cache, v_cache, out, nullptr, 0, max_seq,
                                  flags & ~MUI_FLAG_SPLIT_CONTEXT);
}

extern "C" mui_status_t mui_rope_flash_decode_ws(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D,
                                                 int max_seq, const void* qkv, const void* cos_table,
                                                 const void* sin_table, const int64_t* position_ids,
                                                 const int64_t* cache_position, const int32_t* seq_len_dev,
                                                 float scale, void* k_cache, void* v_cache, void* out,
                                                 void* workspace, size_t workspace_bytes, int max_attended,
                                                 unsigned flags) {
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
  a.freqs = nullptr;
  a.max_pos = max_seq;
  a.l4 = 0;
  a.chunk = 0;
  a.eps = a.attn_scale = a.floor_scale = 0.f;
  ra_bind_workspace(a, workspace);
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  const int splits = ra_pick_splits(flags, std::min(max_attended, max_seq), B, Hq, Hkv, workspace, workspace_bytes);
  if (splits >= 1) {
    if (dtype == MUI_F16) return launch_ra_g<__half>((cudaStream_t)stream, a, pdl, splits);
    return launch_ra_g<__nv_bfloat16>((cudaStream_t)stream, a, pdl, splits);
  }
  if (dtype == MUI_F16) return launch_fa_g<__half>((cudaStream_t)stream, a, pdl);
  return launch_fa_g<__nv_bfloat16>((cudaStream_t)stream, a, pdl);
}

extern "C" mui_status_t mui_llama4_rope_flash_decode(void* stream, mui_dtype_t dtype, int B, int Hq, int Hkv, int D,
                                                     int cache_rows, int max_pos, const void* qkv,
                                                     const float* freqs, const int64_t* position_ids,
                                                     const int64_t* cache_position, int use_rope, int use_qk_norm,
                                                     float norm_eps, int temperature_tuning, float attn_scale,
                                                     float floor_scale, int chunk, float scale, void* k_cache,
                                                     void* v_cache, void* out, void* workspace,
                                                     size_t workspace_bytes, int max_attended, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(D == FA_D, MUI_ERR_UNSUPPORTED, "head dim %d unsupported by the fused kernel (128)", D);
  MUI_REQUIRE(B >= 1 && Hq >= 1 && Hkv >= 1 && Hq % Hkv == 0 && Hq / Hkv <= 8 && cache_rows >= 1 && max_pos >= 1,
              MUI_ERR_INVALID_ARG, "bad sizes B=%d Hq=%d Hkv=%d cache_rows=%d max_pos=%d", B, Hq, Hkv, cache_rows,
              max_pos);
  MUI_REQUIRE(chunk >= 0, MUI_ERR_INVALID_ARG, "chunk must not be negative");
  MUI_REQUIRE(qkv && position_ids && cache_position && k_cache && v_cache && out && (!use_rope || freqs),
              MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) |
                reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(freqs) |
                reinterpret_cast<uintptr_t>(out)) & 15) == 0,
              MUI_ERR_INVALID_ARG, "pointers must be 16-byte aligned");
  MUI_REQUIRE(!temperature_tuning || floor_scale > 0.f, MUI_ERR_INVALID_ARG, "floor_scale must be positive");
  FaArgs a;
  a.qkv = qkv;
  a.cos_t = a.sin_t = nullptr;
  a.position_ids = reinterpret_cast<const long long*>(position_ids);
  a.cache_position = reinterpret_cast<const long long*>(cache_position);
  a.seq_len_dev = nullptr;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.out = out;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.B = B;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.max_seq = cache_rows;
  a.G = Hq / Hkv;
  a.trace = mui_trace_next_record(3);
  a.freqs = freqs;
  a.max_pos = max_pos;
  a.l4 = FA_L4_ON | (use_rope ? FA_L4_ROPE : 0) | (use_qk_norm ? FA_L4_NORM : 0) |
         (temperature_tuning ? FA_L4_TEMP : 0);
  a.chunk = chunk;
  a.eps = norm_eps;
  a.attn_scale = attn_scale;
  a.floor_scale = floor_scale;
  ra_bind_workspace(a, workspace);
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  const int in_view = std::min(max_attended, chunk > 0 ? std::min(chunk, cache_rows) : cache_rows);
  const int splits = ra_pick_splits(flags, in_view, B, Hq, Hkv, workspace, workspace_bytes);
  if (splits >= 1) {
    if (dtype == MUI_F16) return launch_ra_g<__half>((cudaStream_t)stream, a, pdl, splits);
    return launch_ra_g<__nv_bfloat16>((cudaStream_t)stream, a, pdl, splits);
  }
  if (dtype == MUI_F16) return launch_fa_g<__half>((cudaStream_t)stream, a, pdl);
  return launch_fa_g<__nv_bfloat16>((cudaStream_t)stream, a, pdl);
}
