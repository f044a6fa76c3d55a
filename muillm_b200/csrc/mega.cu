// Whole-step persistent decode kernel ("megakernel") for one sequence of a Llama-architecture model.
//
// One launch = one decode step. One CTA per SM stays resident for the whole step. In each CTA a producer warp
// streams the weight rows this CTA owns of EVERY projection of EVERY layer, in execution order, through one
// shared-memory ring of 1-D bulk async copies (TMA) — it never waits for activations, so the ~190 KiB of copies
// in flight per SM that HBM needs stay in flight across operation boundaries, grid barriers and the attention
// phase. Eight consumer warps run the operations in order: stage the activation vector (RMSNorm fused, the
// embedding row for the first layer, the split-KV merge for o_proj), consume ring stages with ldmatrix +
// mma.sync, write their rows, and meet the other CTAs at a grid barrier (arrival counter in global memory,
// bounded spin). Attention runs between the QKV and o_proj projections on the consumer warps of the first
// kv_heads * splits CTAs: RoPE on q and on the new k, K/V cache write, online softmax over the cached tokens
// plus the new one, fp32 partials per split; meanwhile all producers are already filling their rings with
// o_proj rows. The step ends with the lm_head, a per-CTA arg-max of its logit rows, and CTA 0 picking the token
// and advancing the device-side decode state.
//
// Same math, roundings and memory layout as the kernel-per-operation decode stack (stack.cu); that path remains
// for batches, tensor parallelism and shapes this kernel does not cover.
#include "mega.cuh"

#include <algorithm>
#include <cstring>

MUI_STATUS_ACCESSOR(mega)

namespace {

constexpr int MG_THREADS = GEMV_CONSUMER_THREADS + 32;
constexpr int MG_KC = 2048;
constexpr int MG_ROWS = 16;
constexpr int MG_ROW_PITCH = MG_KC * 2 + 16;
constexpr int MG_STAGE_BYTES = MG_ROWS * MG_ROW_PITCH;
constexpr int MG_STAGES = 3;
constexpr int MG_D = 128;
constexpr int MG_XPAD = 8;
constexpr unsigned long long MG_WAIT_NS = 1000000000ull;

struct MegaSmem {
  int x_off, red_off, merge_off, bar_off, flag_off, total;
};
__host__ __device__ inline MegaSmem mega_smem(int x_elems, int Hq) {
  MegaSmem m;
  m.x_off = MG_STAGES * MG_STAGE_BYTES;
  m.red_off = m.x_off + (((x_elems + MG_XPAD) * 2 + 15) & ~15);
  m.merge_off = m.red_off + 2 * GEMV_CONSUMER_WARPS * MG_ROWS * 4;
  m.bar_off = m.merge_off + ((Hq * (MG_MAX_SPLITS + 1) * 4 + 15) & ~15);
  m.flag_off = m.bar_off + 2 * MG_STAGES * 8;
  m.total = m.flag_off + 16;
  return m;
}

struct MgOp {
  const unsigned char* W;
  const unsigned char* W2;
  int N, K, mode;
};
__device__ __forceinline__ MgOp mg_layer_op(const MegaArgs& a, const MegaLayer& ly, int j) {
  MgOp o;
  o.W2 = nullptr;
  o.mode = 0;
  if (j == 0) {
    o.W = reinterpret_cast<const unsigned char*>(ly.qkv);
    o.N = (a.Hq + 2 * a.Hkv) * MG_D;
    o.K = a.H;
  } else if (j == 1) {
    o.W = reinterpret_cast<const unsigned char*>(ly.o);
    o.N = a.H;
    o.K = a.Hq * MG_D;
  } else if (j == 2) {
    o.W = reinterpret_cast<const unsigned char*>(ly.gate);
    o.W2 = reinterpret_cast<const unsigned char*>(ly.up);
    o.N = a.I;
    o.K = a.H;
    o.mode = 1;
  } else {
    o.W = reinterpret_cast<const unsigned char*>(ly.down);
    o.N = a.H;
    o.K = a.I;
  }
  return o;
}
__device__ __forceinline__ MgOp mg_lm_op(const MegaArgs& a) {
  MgOp o;
  o.W = reinterpret_cast<const unsigned char*>(a.lm_head);
  o.W2 = nullptr;
  o.N = a.V;
  o.K = a.H;
  o.mode = 0;
  return o;
}

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

enum { EPI_STORE = 0, EPI_RESID = 1, EPI_GATEUP = 2, EPI_LOGITS = 3 };

// everything the consumer warps share while walking the step
template <typename T>
struct MgCons {
  const MegaArgs& a;
  unsigned char* stage_mem;
  T* x_s;
  float* red;
  float* merge;
  uint64_t* full_bar;
  uint64_t* empty_bar;
  volatile int* abort_flag;
  int tid, warp, lane;
  int it;        // ring item counter (continues across operations)
  int red_sel;   // which of the two partial-tile buffers the next row block uses
  int bar_j;     // grid barriers passed in this step
  unsigned long long bar_base;
  int num_bars;
  float best_v;  // running arg-max of this thread's logit rows
  int best_i;
  int n_stamps;

  __device__ void stamp(int tag) {
    if (a.op_trace != nullptr && blockIdx.x == 0 && tid == 0 && n_stamps < a.op_trace_cap) {
      a.op_trace[2 * n_stamps] = (unsigned long long)tag;
      a.op_trace[2 * n_stamps + 1] = global_timer_ns();
      n_stamps += 1;
    }
  }

  __device__ MgCons(const MegaArgs& args) : a(args) {}

  // Grid barrier among the consumer warps of all CTAs. Returns false when the step is being abandoned.
  __device__ bool grid_sync() {
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
    if (tid == 0 && !*abort_flag) {
      __threadfence();
      atomicAdd(a.bar, 1ull);
      const unsigned long long target = bar_base + (unsigned long long)(bar_j + 1) * gridDim.x;
      if (ld_acquire_gpu_u64(a.bar) < target) {
        const uint64_t t0 = global_timer_ns();
        unsigned spins = 0;
        while (ld_acquire_gpu_u64(a.bar) < target) {
          if ((++spins & 0x3f) == 0 && global_timer_ns() - t0 > MG_WAIT_NS) {
            mui_dev_set_status(MUI_DEV_TIMEOUT_PEER, 0x800000u | (unsigned)bar_j);
            // hand in this CTA's remaining arrivals so that the others are not held up by it
            atomicAdd(a.bar, (unsigned long long)(num_bars - 1 - bar_j));
            *abort_flag = 1;
            break;
          }
        }
      }
      __threadfence();
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
    bar_j += 1;
    return *abort_flag == 0;
  }

  // x_s = rmsnorm(src) * nw with the roundings of the HF module (nw == nullptr: plain copy). K % 8 == 0.
  __device__ void stage_vec(const T* __restrict__ src, const T* __restrict__ nw, int K, T* copy_out) {
    float rstd = 1.f;
    if (nw != nullptr) {
      float ss = 0.f;
      for (int k = tid * 8; k < K; k += GEMV_CONSUMER_THREADS * 8) {
        float f[8];
        unpack8<T>(ld_act16(src + k), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      named_bar_sync(1, GEMV_CONSUMER_THREADS);
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) tot += red[w];
      rstd = rsqrtf(tot / static_cast<float>(K) + a.eps);
    }
    for (int k = tid * 8; k < K; k += GEMV_CONSUMER_THREADS * 8) {
      const uint4 raw = ld_act16(src + k);
      if (copy_out != nullptr) *reinterpret_cast<uint4*>(copy_out + k) = raw;
      uint4 out = raw;
      if (nw != nullptr) {
        float f[8], wv[8];
        unpack8<T>(raw, f);
        unpack8<T>(ld_cached16(nw + k), wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = Elt<T>::to_f32(Elt<T>::from_f32(f[i] * rstd)) * wv[i];
        out = pack8<T>(f);
      }
      *reinterpret_cast<uint4*>(x_s + k) = out;
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
  }

  // x_s = attention output, merged over the KV splits by log-sum-exp from the fp32 partials, rounded to T.
  __device__ void stage_attention_merge(int nsplit) {
    const int Hq = a.Hq;
    for (int h = tid; h < Hq; h += GEMV_CONSUMER_THREADS) {
      const float* p = a.attn_part + (size_t)h * MG_MAX_SPLITS * (MG_D + 2);
      float ms[MG_MAX_SPLITS], ls[MG_MAX_SPLITS];
#pragma unroll
      for (int s = 0; s < MG_MAX_SPLITS; ++s) {
        ms[s] = (s < nsplit) ? __ldcg(p + (size_t)s * (MG_D + 2)) : -INFINITY;
        ls[s] = (s < nsplit) ? __ldcg(p + (size_t)s * (MG_D + 2) + 1) : 0.f;
      }
      float M = -INFINITY;
#pragma unroll
      for (int s = 0; s < MG_MAX_SPLITS; ++s) M = fmaxf(M, ms[s]);
      float L = 0.f;
#pragma unroll
      for (int s = 0; s < MG_MAX_SPLITS; ++s) {
        const float w = (ms[s] == -INFINITY) ? 0.f : exp2f(ms[s] - M);
        merge[h * (MG_MAX_SPLITS + 1) + s] = w;
        L = fmaf(ls[s], w, L);
      }
      merge[h * (MG_MAX_SPLITS + 1) + MG_MAX_SPLITS] = (L > 0.f) ? 1.f / L : 0.f;
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
    const int groups = Hq * (MG_D / 8);
    for (int e = tid; e < groups; e += GEMV_CONSUMER_THREADS) {
      const int h = e / (MG_D / 8), d0 = (e - h * (MG_D / 8)) * 8;
      const float* p = a.attn_part + (size_t)h * MG_MAX_SPLITS * (MG_D + 2) + 2 + d0;
      const float* w = merge + h * (MG_MAX_SPLITS + 1);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s0 = 0; s0 < nsplit; s0 += 4) {
        float v[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int s = min(s0 + i, nsplit - 1);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __ldcg(p + (size_t)s * (MG_D + 2) + j);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (s0 + i < nsplit) {
            const float ws = w[s0 + i];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(ws, v[i][j], acc[j]);
          }
      }
      const float linv = w[MG_MAX_SPLITS];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= linv;
      *reinterpret_cast<uint4*>(x_s + h * MG_D + d0) = pack8<T>(acc);
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
  }

  // Consume this CTA's rows of one projection from the ring and run the epilogue EPI on each finished row.
  template <int EPI>
  __device__ bool consume(const MgOp& op, T* out) {
    const int rps = op.mode ? 8 : 16;
    const int r0 = static_cast<int>((long long)op.N * blockIdx.x / gridDim.x);
    const int r1 = static_cast<int>((long long)op.N * (blockIdx.x + 1) / gridDim.x);
    const int nblk = (r1 - r0 + rps - 1) / rps;
    const int nchunks = (op.K + MG_KC - 1) / MG_KC;
    const uint32_t a_lane_off =
        static_cast<uint32_t>(((lane & 7) + ((lane >> 3) & 1) * 8) * MG_ROW_PITCH + (lane >> 4) * 16);
    const uint32_t b_lane_off = static_cast<uint32_t>(((lane >> 3) & 1) * 16);
    const uint32_t stage_base = smem_u32(stage_mem);
    const uint32_t x_base = smem_u32(x_s);
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    for (int blk = 0; blk < nblk; ++blk) {
      for (int kc = 0; kc < nchunks; ++kc) {
        const int s = it % MG_STAGES;
        const uint32_t ph = (it / MG_STAGES) & 1;
        if (!mbar_wait_bounded(full_bar + s, ph, abort_flag)) {
          if (lane == 0 && !*abort_flag) {
            mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, s);
            *abort_flag = 1;
          }
          return false;
        }
        const int kc_len = min(MG_KC, op.K - kc * MG_KC);
        const int nsteps = kc_len >> 4;
        const uint32_t a_addr = stage_base + static_cast<uint32_t>(s) * MG_STAGE_BYTES + a_lane_off;
        const uint32_t b_addr = x_base + b_lane_off + static_cast<uint32_t>(kc * MG_KC * 2);
#pragma unroll 4
        for (int j = warp; j < nsteps; j += GEMV_CONSUMER_WARPS) {
          uint32_t af[4], b0, b1;
          ldmatrix_x4(af, a_addr + j * 32);
          ldmatrix_x2(b0, b1, b_addr + j * 32);
          MmaOp<T>::run(d, af, b0, b1);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar + s);
        it += 1;
      }
      // row block complete: sum the eight warps' partial tiles in a fixed order, then the epilogue
      float* rbuf = red + red_sel * (GEMV_CONSUMER_WARPS * MG_ROWS);
      red_sel ^= 1;
      if ((lane & 3) == 0) {
        rbuf[warp * MG_ROWS + (lane >> 2)] = d[0];
        rbuf[warp * MG_ROWS + (lane >> 2) + 8] = d[2];
      }
      d[0] = d[1] = d[2] = d[3] = 0.f;
      named_bar_sync(1, GEMV_CONSUMER_THREADS);
      if (tid < rps) {
        const int row = r0 + blk * rps + tid;
        if (row < r1) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) v += rbuf[w * MG_ROWS + tid];
          if (EPI == EPI_GATEUP) {
            float u = 0.f;
#pragma unroll
            for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) u += rbuf[w * MG_ROWS + tid + 8];
            out[row] = Elt<T>::from_f32(silu_f32(v) * u);
          } else if (EPI == EPI_RESID) {
            out[row] = Elt<T>::from_f32(v + ld_act_f32<T>(out + row));
          } else {
            const T r = Elt<T>::from_f32(v);
            out[row] = r;
            if (EPI == EPI_LOGITS) {
              const float rv = Elt<T>::to_f32(r);
              if (rv > best_v || (rv == best_v && row < best_i)) {
                best_v = rv;
                best_i = row;
              }
            }
          }
        }
      }
    }
    return true;
  }
};

// RoPE of the 8 dims [d0, d0+8) this lane holds of a 128-dim head whose 16 lanes sit side by side: the partner
// dims (d +- 64) are 8 lanes away. Result rounded to T, like the stand-alone RoPE kernel stores it.
template <typename T>
__device__ __forceinline__ void mg_rope8(float (&x)[8], const float (&c)[8], const float (&s)[8], bool low_half) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float p = __shfl_xor_sync(MUI_FULL_MASK, x[i], 8);
    const float r = low_half ? fmaf(x[i], c[i], -p * s[i]) : fmaf(x[i], c[i], p * s[i]);
    x[i] = Elt<T>::to_f32(Elt<T>::from_f32(r));
  }
}

__device__ __forceinline__ void mg_merge_state(float& m, float& l, float (&acc)[8], float mo, float lo,
                                               const float (&acco)[8]) {
  const float mn = fmaxf(m, mo);
  const float fa = (m == -INFINITY) ? 0.f : exp2f(m - mn);
  const float fb = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
  l = l * fa + lo * fb;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = acc[i] * fa + acco[i] * fb;
  m = mn;
}

// Attention phase of one layer on the consumer warps of CTA (kv head, split).
template <typename T, int GP>
__device__ void mg_attention(MgCons<T>& c, const MegaLayer& ly, int cached, int nsplit, long long pos_id,
                             long long cache_pos) {
  const MegaArgs& a = c.a;
  const int kvh = blockIdx.x % a.Hkv, split = blockIdx.x / a.Hkv;
  if (split >= nsplit) return;
  constexpr int LPT = MG_D / 8, TPW = 32 / LPT, U = (GP <= 4) ? 4 : 2;
  const int lane = c.lane, warp = c.warp, tid = c.tid;
  const int sub = lane / LPT, dlane = lane % LPT, d0 = dlane * 8;
  const int G = a.Hq / a.Hkv;
  // scratch aliased on the activation vector (not in use between the QKV projection and the o_proj staging)
  float* sm_m = reinterpret_cast<float*>(c.x_s);
  float* sm_l = sm_m + GEMV_CONSUMER_WARPS * GP;
  float* sm_acc = sm_l + GEMV_CONSUMER_WARPS * GP;

  const T* qkv = reinterpret_cast<const T*>(a.qkv_out);
  float cs[8], sn[8];
  unpack8<T>(ld_cached16(reinterpret_cast<const T*>(a.cos_t) + (size_t)pos_id * MG_D + d0), cs);
  unpack8<T>(ld_cached16(reinterpret_cast<const T*>(a.sin_t) + (size_t)pos_id * MG_D + d0), sn);
  const bool low = dlane < (LPT / 2);

  float qf[GP][8];
#pragma unroll
  for (int g = 0; g < GP; ++g) {
    if (g < G) {
      unpack8<T>(ld_act16(qkv + ((size_t)kvh * G + g) * MG_D + d0), qf[g]);
      mg_rope8<T>(qf[g], cs, sn, low);
#pragma unroll
      for (int i = 0; i < 8; ++i) qf[g][i] *= a.scale_log2;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) qf[g][i] = 0.f;
    }
  }
  // the new token's k (rotated) and v
  float kn[8];
  unpack8<T>(ld_act16(qkv + ((size_t)a.Hq + kvh) * MG_D + d0), kn);
  mg_rope8<T>(kn, cs, sn, low);
  const uint4 k_new = pack8<T>(kn);
  const uint4 v_new = ld_act16(qkv + ((size_t)a.Hq + a.Hkv + kvh) * MG_D + d0);
  T* kc = reinterpret_cast<T*>(ly.k_cache) + (size_t)kvh * a.max_seq * MG_D;
  T* vc = reinterpret_cast<T*>(ly.v_cache) + (size_t)kvh * a.max_seq * MG_D;
  if (split == 0 && warp == 0 && sub == 0) {
    *reinterpret_cast<uint4*>(kc + (size_t)cache_pos * MG_D + d0) = k_new;
    *reinterpret_cast<uint4*>(vc + (size_t)cache_pos * MG_D + d0) = v_new;
  }

  float m[GP], l[GP], acc[GP][8];
#pragma unroll
  for (int g = 0; g < GP; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  int chunk = (cached + nsplit - 1) / nsplit;
  chunk = (chunk + 15) / 16 * 16;
  const int t_begin = split * chunk, t_end = min(cached, t_begin + chunk);

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

  for (int t0 = t_begin + warp * TPW; t0 < t_end; t0 += GEMV_CONSUMER_WARPS * TPW * U) {
    uint4 kraw[U], vraw[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u * GEMV_CONSUMER_WARPS * TPW + sub;
      valid[u] = t < t_end;
      if (valid[u]) {
        kraw[u] = __ldcg(reinterpret_cast<const uint4*>(kc + (size_t)t * MG_D + d0));
        vraw[u] = __ldcg(reinterpret_cast<const uint4*>(vc + (size_t)t * MG_D + d0));
      } else {
        kraw[u] = make_uint4(0, 0, 0, 0);
        vraw[u] = make_uint4(0, 0, 0, 0);
      }
    }
    fold(kraw, vraw, valid);
  }
  // the new token itself: taken from registers by warp 0 of the last split (its cache row is being written by
  // split 0 in this same phase)
  if (warp == 0 && split == nsplit - 1) {
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

  // merge the token sub-streams of the warp, then the warps through shared memory
#pragma unroll
  for (int off = LPT; off < 32; off <<= 1) {
#pragma unroll
    for (int g = 0; g < GP; ++g) {
      const float mo = __shfl_xor_sync(MUI_FULL_MASK, m[g], off);
      const float lo = __shfl_xor_sync(MUI_FULL_MASK, l[g], off);
      float ao[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) ao[i] = __shfl_xor_sync(MUI_FULL_MASK, acc[g][i], off);
      mg_merge_state(m[g], l[g], acc[g], mo, lo, ao);
    }
  }
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < GP; ++g) {
      if (dlane == 0) {
        sm_m[warp * GP + g] = m[g];
        sm_l[warp * GP + g] = l[g];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sm_acc[(warp * GP + g) * MG_D + d0 + i] = acc[g][i];
    }
  }
  named_bar_sync(2, GEMV_CONSUMER_THREADS);
  for (int idx = tid; idx < G * MG_D; idx += GEMV_CONSUMER_THREADS) {
    const int g = idx / MG_D, d = idx - g * MG_D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) mm = fmaxf(mm, sm_m[w * GP + g]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) {
      const float mw = sm_m[w * GP + g];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      ll = fmaf(sm_l[w * GP + g], f, ll);
      aa = fmaf(sm_acc[(w * GP + g) * MG_D + d], f, aa);
    }
    float* p = a.attn_part + (((size_t)kvh * G + g) * MG_MAX_SPLITS + split) * (MG_D + 2);
    if (d == 0) {
      p[0] = mm;
      p[1] = ll;
    }
    p[2 + d] = aa;
  }
}

template <typename T, int GP>
__global__ void __launch_bounds__(MG_THREADS, 1) mega_decode_kernel(const MegaArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const MegaSmem lay = mega_smem(a.x_elems, a.Hq);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw + lay.bar_off);
  uint64_t* empty_bar = full_bar + MG_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + lay.flag_off);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < MG_STAGES; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, GEMV_CONSUMER_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  trace_start(a.trace);
  __syncthreads();
  pdl_launch_dependents();

  if (warp == GEMV_CONSUMER_WARPS) {
    // ------------------------------ producer warp: every projection's rows of this CTA, in order ------------
    const uint64_t policy = l2_policy_evict_first();
    int it = 0;
    bool ok = true;
    auto produce = [&](const MgOp& op) {
      const int rps = op.mode ? 8 : 16;
      const int r0 = static_cast<int>((long long)op.N * blockIdx.x / gridDim.x);
      const int r1 = static_cast<int>((long long)op.N * (blockIdx.x + 1) / gridDim.x);
      const int nblk = (r1 - r0 + rps - 1) / rps;
      const int nchunks = (op.K + MG_KC - 1) / MG_KC;
      for (int blk = 0; blk < nblk && ok; ++blk) {
        const int rb = r0 + blk * rps;
        const int rows_valid = min(rps, r1 - rb);
        for (int kc = 0; kc < nchunks; ++kc) {
          const int s = it % MG_STAGES;
          const uint32_t ph = (it / MG_STAGES) & 1;
          int w_ok = 1;
          if (lane == 0) w_ok = mbar_wait_bounded(empty_bar + s, ph ^ 1u, abort_flag) ? 1 : 0;
          w_ok = __shfl_sync(MUI_FULL_MASK, w_ok, 0);
          if (!w_ok) {
            if (lane == 0 && !*abort_flag) {
              mui_dev_set_status(MUI_DEV_TIMEOUT_EMPTY, s);
              *abort_flag = 1;
            }
            ok = false;
            return;
          }
          const int kc_len = min(MG_KC, op.K - kc * MG_KC);
          const uint32_t bytes = static_cast<uint32_t>(kc_len) * 2u;
          const int ncopies = op.mode ? 2 * rows_valid : rows_valid;
          if (lane == 0) mbar_arrive_expect_tx(full_bar + s, static_cast<uint32_t>(ncopies) * bytes);
          __syncwarp();
          if (lane < MG_ROWS) {
            const int orow = op.mode ? (lane & 7) : lane;
            if (orow < rows_valid) {
              const unsigned char* src = ((op.mode && lane >= 8) ? op.W2 : op.W) +
                                         ((size_t)(rb + orow) * op.K + (size_t)kc * MG_KC) * 2;
              bulk_load_1d(smem_raw + (size_t)s * MG_STAGE_BYTES + (size_t)lane * MG_ROW_PITCH, src, bytes,
                           full_bar + s, policy);
            }
          }
          it += 1;
        }
      }
    };
    for (int l = 0; l < a.L && ok; ++l) {
      const MegaLayer ly = a.layers[l];
      for (int j = 0; j < 4 && ok; ++j) produce(mg_layer_op(a, ly, j));
    }
    if (ok) produce(mg_lm_op(a));
    if (!ok && lane == 0) {
      const int first = max(0, it - MG_STAGES);
      for (int i = first; i < it; ++i) {
        int zero = 0;
        if (!mbar_wait_bounded(full_bar + (i % MG_STAGES), (i / MG_STAGES) & 1, &zero))
          mui_dev_set_status(MUI_DEV_TIMEOUT_DRAIN, i % MG_STAGES);
      }
    }
    return;
  }

  // ------------------------------ consumer warps ------------------------------
  pdl_wait_prior_grid();
  MgCons<T> c(a);
  c.stage_mem = smem_raw;
  c.x_s = reinterpret_cast<T*>(smem_raw + lay.x_off);
  c.red = reinterpret_cast<float*>(smem_raw + lay.red_off);
  c.merge = reinterpret_cast<float*>(smem_raw + lay.merge_off);
  c.full_bar = full_bar;
  c.empty_bar = empty_bar;
  c.abort_flag = abort_flag;
  c.tid = tid;
  c.warp = warp;
  c.lane = lane;
  c.it = 0;
  c.red_sel = 0;
  c.bar_j = 0;
  c.num_bars = 5 * a.L + 1;
  c.best_v = -INFINITY;
  c.best_i = 0x7fffffff;
  c.n_stamps = 0;

  const long long step = __ldcg(a.state);
  const unsigned long long epoch = __ldcg(a.bar + 1);
  const long long cache_pos = __ldcg(a.state + 2);
  const long long pos_id = __ldcg(a.state + 3);
  long long token = __ldcg(a.state + 4);
  token = token < 0 ? 0 : (token >= a.embed_vocab ? a.embed_vocab - 1 : token);
  c.bar_base = epoch * (unsigned long long)c.num_bars * gridDim.x;
  const int cached = static_cast<int>(cache_pos);
  const int max_splits = min(MG_MAX_SPLITS, (int)gridDim.x / a.Hkv);
  const int nsplit = max(1, min(max_splits, (cached + 127) / 128));

  T* h = reinterpret_cast<T*>(a.h);
  T* qkv_out = reinterpret_cast<T*>(a.qkv_out);
  T* t_buf = reinterpret_cast<T*>(a.t);
  bool ok = true;
  for (int l = 0; l < a.L && ok; ++l) {
    const MegaLayer ly = a.layers[l];
    c.stamp(0);
    if (l == 0) {
      // the embedding row is the first layer's input; CTA 0 also leaves it in h for the residual adds
      const T* row = reinterpret_cast<const T*>(a.embed) + (size_t)token * a.H;
      c.stage_vec(row, reinterpret_cast<const T*>(ly.ln1), a.H, blockIdx.x == 0 ? h : nullptr);
    } else {
      if (!(ok = c.grid_sync())) break;
      c.stamp(1);
      c.stage_vec(h, reinterpret_cast<const T*>(ly.ln1), a.H, nullptr);
    }
    c.stamp(2);
    if (!(ok = c.template consume<EPI_STORE>(mg_layer_op(a, ly, 0), qkv_out))) break;
    c.stamp(3);
    if (!(ok = c.grid_sync())) break;
    c.stamp(4);
    mg_attention<T, GP>(c, ly, cached, nsplit, pos_id, cache_pos);
    c.stamp(5);
    if (!(ok = c.grid_sync())) break;
    c.stamp(6);
    c.stage_attention_merge(nsplit);
    c.stamp(7);
    if (!(ok = c.template consume<EPI_RESID>(mg_layer_op(a, ly, 1), h))) break;
    c.stamp(8);
    if (!(ok = c.grid_sync())) break;
    c.stamp(9);
    c.stage_vec(h, reinterpret_cast<const T*>(ly.ln2), a.H, nullptr);
    c.stamp(10);
    if (!(ok = c.template consume<EPI_GATEUP>(mg_layer_op(a, ly, 2), t_buf))) break;
    c.stamp(11);
    if (!(ok = c.grid_sync())) break;
    c.stamp(12);
    c.stage_vec(t_buf, nullptr, a.I, nullptr);
    c.stamp(13);
    if (!(ok = c.template consume<EPI_RESID>(mg_layer_op(a, ly, 3), h))) break;
    c.stamp(14);
  }
  if (ok) ok = c.grid_sync();
  if (ok) {
    c.stage_vec(h, reinterpret_cast<const T*>(a.final_norm), a.H, nullptr);
    ok = c.template consume<EPI_LOGITS>(mg_lm_op(a), reinterpret_cast<T*>(a.logits));
  }
  if (ok) {
    // per-CTA arg-max of its logit rows (threads 0..15 of warp 0 hold candidates)
    float bv = (warp == 0) ? c.best_v : -INFINITY;
    int bi = (warp == 0) ? c.best_i : 0x7fffffff;
    if (warp == 0) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(MUI_FULL_MASK, bv, o);
        const int oi = __shfl_xor_sync(MUI_FULL_MASK, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
          bv = ov;
          bi = oi;
        }
      }
      if (lane == 0) {
        a.argmax_val[blockIdx.x] = bv;
        a.argmax_idx[blockIdx.x] = bi;
      }
    }
    ok = c.grid_sync();
    if (ok && blockIdx.x == 0 && warp == 0) {
      bv = -INFINITY;
      bi = 0x7fffffff;
      for (int i = lane; i < (int)gridDim.x; i += 32) {
        const float v = __ldcg(a.argmax_val + i);
        const int ix = __ldcg(a.argmax_idx + i);
        if (v > bv || (v == bv && ix < bi)) {
          bv = v;
          bi = ix;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(MUI_FULL_MASK, bv, o);
        const int oi = __shfl_xor_sync(MUI_FULL_MASK, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
          bv = ov;
          bi = oi;
        }
      }
      if (lane == 0) {
        if (bi == 0x7fffffff) bi = 0;
        a.state[4] = bi;
        if (a.out_tokens != nullptr && step < a.out_capacity) a.out_tokens[step] = bi;
        a.state[3] = pos_id + 1;
        a.state[0] = step + 1;
        a.state[1] = __ldcg(a.state + 1) + 1;
        a.state[2] = cache_pos + 1;
        *a.seq_len32 = static_cast<int32_t>(cache_pos + 2);
        a.bar[1] = epoch + 1;  // every CTA read the epoch before its first barrier, long ago
      }
    }
  }
  if (tid == 0) trace_end(a.trace);
}

}  // namespace

size_t mui_mega_smem_bytes(int x_elems, int Hq) { return (size_t)mega_smem(x_elems, Hq).total; }

int mui_mega_x_elems(int H, int I, int Hq, int Hkv) {
  const int G = Hq / Hkv;
  const int gp = G <= 1 ? 1 : (G <= 2 ? 2 : (G <= 4 ? 4 : 8));
  const int scratch_elems = (GEMV_CONSUMER_WARPS * gp * (MG_D + 2) * 4 + 1) / 2;  // attention scratch, in 16-bit units
  return std::max(std::max(H, I), std::max(Hq * MG_D, scratch_elems));
}

mui_status_t mui_launch_mega_step(cudaStream_t stream, mui_dtype_t dtype, const MegaArgs& args, int G_ratio,
                                  int grid, int pdl) {
  const size_t smem = mui_mega_smem_bytes(args.x_elems, args.Hq);
  MegaArgs a = args;
  a.trace = mui_trace_next_record(5);
#define MUI_MEGA_LAUNCH(TT, GP)                                                                               \
  do {                                                                                                        \
    auto kern = mega_decode_kernel<TT, GP>;                                                                   \
    static bool configured = false;                                                                           \
    if (!configured) {                                                                                        \
      MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));    \
      MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,               \
                                          cudaSharedmemCarveoutMaxShared));                                   \
      configured = true;                                                                                      \
    }                                                                                                         \
    MUI_CUDA_CHECK(mui_launch(kern, dim3(grid), dim3(MG_THREADS), smem, stream, pdl, a));                     \
  } while (0)
  if (dtype == MUI_F16) {
    if (G_ratio <= 1) MUI_MEGA_LAUNCH(__half, 1);
    else if (G_ratio <= 2) MUI_MEGA_LAUNCH(__half, 2);
    else MUI_MEGA_LAUNCH(__half, 4);
  } else {
    if (G_ratio <= 1) MUI_MEGA_LAUNCH(__nv_bfloat16, 1);
    else if (G_ratio <= 2) MUI_MEGA_LAUNCH(__nv_bfloat16, 2);
    else MUI_MEGA_LAUNCH(__nv_bfloat16, 4);
  }
#undef MUI_MEGA_LAUNCH
  return MUI_OK;
}
