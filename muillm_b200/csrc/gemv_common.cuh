// Argument block, activation staging (with the fused RMSNorm) and epilogues shared by the
// GEMV-shaped kernels (linear, gate/up+SiLU, their weight-only 8-bit and MoE variants).
#pragma once

#include "comm_dev.cuh"

#define GEMV_CONSUMER_THREADS 256
#define GEMV_CONSUMER_WARPS 8

// MoE addressing of the rows / reduction segments (device-side expert selection).
#define GEMV_MOE_NONE 0
#define GEMV_MOE_ROWS 1      // gate/up: output rows span the computed experts, out is [slots, N]
#define GEMV_MOE_SEGMENTS 2  // down: the reduction runs over the computed experts, out is [N]

struct GemvArgs {
  const void* W;         // [N,K] (or [E*N, K] for MoE)
  const void* W2;        // gate/up: the "up" matrix, same shape as W
  const void* scales;    // 8-bit weights: per-row scales or per-group {scale,min} pairs (of W)
  const void* scales2;   // 8-bit gate/up SYM_ROW: scales of W2
  const void* x;         // [B,K] (MoE segments: [slots, K])
  const void* norm_w;    // [K] or null
  const void* mul_bias;  // [N] or null
  const void* add_bias;  // [N] or null
  const void* residual;  // [B,N] or null
  void* y;               // [B,N] 16-bit output (may be null when y_f32 is set)
  float* y_f32;          // optional fp32 output (tensor-parallel partial sums), same indexing as y
  const int64_t* router_indices;  // [slots - num_shared] routed expert ids (device)
  const void* router_scores;      // [slots - num_shared] routed scores, 16-bit (device)
  float eps;
  int N;           // output rows per matrix / expert
  int K;           // reduction length (per segment)
  int B;           // activation rows actually present (<= NB template)
  int activ;       // mui_activation_t
  int Kp;          // smem row stride of the staged activations, K rounded up to 8
  int moe_mode;    // GEMV_MOE_*
  int slots;       // computed experts (shared first, then routed), 1 when not MoE
  int num_shared;  // shared experts among the slots
  int group_shift; // 8-bit GROUP_MIN: log2(group size)
  int w8_fmt;      // -1: 16-bit weights; else mui_w8_format_t of the 8-bit weights
  int w8_pack;     // gate/up GROUP_MIN: W is the element-interleaved pack [N][K][2], scales [N][K/group][2][2]
  unsigned long long* trace;  // launch-trace record or null
  // weights of the kernels that follow on the stream: once its own copies are issued, the producer warp pulls
  // this CTA's slice of them into L2, so that HBM keeps streaming through this kernel's tail, the launch gap and
  // the latency-bound kernels in between
  const void* pf_ptr[3];  // matrices [pf_rows][pf_row_bytes]; CTA c pulls the first pf_frac/1024 of ITS row range
  int pf_rows[3];
  int pf_row_bytes[3];
  int pf_frac[3];
  int pf_skip[3];  // bytes left out at the head of each CTA range (fetched by the consumer kernel's own ring)
  int reserve_sms; // SMs the bulk-copy pipeline leaves without a CTA (a small dependent kernel moves in early)
  int use_comm;    // tensor-parallel: push the fp32 results to every rank, then all-reduce into y
  CommDev comm;
};

// What a caller that knows the rest of the stream (the decode stack) tells one GEMV launch: the weight matrices of
// the kernels that follow (pulled into L2 once the launch's own copies are issued) and how many SMs to leave free
// for a small dependent kernel. Travels in the argument block of that launch only.
struct GemvHints {
  const void* pf_ptr[3];
  int pf_rows[3];
  int pf_row_bytes[3];
  int pf_frac[3];  // of 1024
  int reserve_sms;
};
inline void gemv_apply_hints(GemvArgs& a, const GemvHints* h) {
  if (h == nullptr) return;
  for (int i = 0; i < 3; ++i) {
    const bool on = h->pf_ptr[i] != nullptr && (reinterpret_cast<uintptr_t>(h->pf_ptr[i]) & 15) == 0 &&
                    h->pf_rows[i] > 0 && h->pf_row_bytes[i] > 0 && (h->pf_row_bytes[i] & 15) == 0 && h->pf_frac[i] > 0;
    a.pf_ptr[i] = on ? h->pf_ptr[i] : nullptr;
    a.pf_rows[i] = on ? h->pf_rows[i] : 0;
    a.pf_row_bytes[i] = on ? h->pf_row_bytes[i] : 0;
    a.pf_frac[i] = on ? (h->pf_frac[i] < 1024 ? h->pf_frac[i] : 1024) : 0;
    a.pf_skip[i] = 0;
  }
  a.reserve_sms = h->reserve_sms > 0 ? h->reserve_sms : 0;
}

// expert whose weights serve computed slot `slot`
__device__ __forceinline__ int gemv_slot_expert(const GemvArgs& a, int slot) {
  if (slot < a.num_shared) return slot;
  return a.num_shared + static_cast<int>(__ldcg(a.router_indices + (slot - a.num_shared)));
}
template <typename T>
__device__ __forceinline__ float gemv_slot_score(const GemvArgs& a, int slot) {
  if (slot < a.num_shared) return 1.f;
  return ld_act_f32<T>(reinterpret_cast<const T*>(a.router_scores) + (slot - a.num_shared));
}

// ---------------------------------------------------------------------------------------------
// Stage the activations into shared memory as 16-bit values, applying the RMSNorm with the
// roundings of the HF modules: xn = round16(round16(x * rstd) * w), rstd = rsqrt(mean(x^2) + eps)
// computed in fp32. Rows b >= a.B (template padding) are zero filled. Called by the 256 consumer
// threads; synchronises them on named barrier 1. `red` is NBX*8 floats of shared scratch; `pitch` is the
// element stride between staged rows (>= Kp).
// NBX = number of activation rows staged (batch rows, or MoE segments).
// ---------------------------------------------------------------------------------------------
// Norm weights of the one-row fast path of gemv_stage_x, loaded into registers BEFORE the wait for the previous
// kernel (they are constants, unlike the activations): one L2 round trip less between two dependent kernels.
struct GemvNormPre {
  uint4 w[4];
  bool have;
};
template <typename T, int NBX>
__device__ __forceinline__ bool gemv_stage_fast_path(const GemvArgs& a) {
  const int K = a.K;
  return NBX == 1 && ((K & 7) == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0) && a.norm_w != nullptr &&
         ((reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0) && K <= GEMV_CONSUMER_THREADS * 8 * 4 && a.B >= 1;
}
template <typename T, int NBX>
__device__ __forceinline__ void gemv_prefetch_norm(const GemvArgs& a, int tid, GemvNormPre& pre) {
  pre.have = gemv_stage_fast_path<T, NBX>(a);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = (j * GEMV_CONSUMER_THREADS + tid) * 8;
    pre.w[j] = (pre.have && k < a.K) ? ld_cached16(reinterpret_cast<const T*>(a.norm_w) + k) : make_uint4(0, 0, 0, 0);
  }
}

template <typename T, int NBX>
__device__ __forceinline__ void gemv_stage_x(const GemvArgs& a, int rows_present, T* x_s, int pitch, float* red,
                                             int tid, const GemvNormPre* pre = nullptr) {
  const int K = a.K, Kp = a.Kp;
  const T* __restrict__ x = reinterpret_cast<const T*>(a.x);
  const T* __restrict__ nw = reinterpret_cast<const T*>(a.norm_w);
  const int warp = tid >> 5, lane = tid & 31;
  const bool vec_ok = ((K & 7) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                      (nw == nullptr || (reinterpret_cast<uintptr_t>(nw) & 15) == 0);
  float rstd[NBX];
#pragma unroll
  for (int b = 0; b < NBX; ++b) rstd[b] = 1.f;

  // Fast path (one activation row, K up to 8192, 16-byte aligned): every thread keeps its slices of x in
  // registers between the sum of squares and the scaling, so x is read from L2 once — one dependent round trip
  // less on the critical path between two kernels.
  if (NBX == 1 && vec_ok && nw != nullptr && K <= GEMV_CONSUMER_THREADS * 8 * 4 && rows_present >= 1) {
    uint4 keep[4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = (j * GEMV_CONSUMER_THREADS + tid) * 8;
      keep[j] = (k < K) ? ld_act16(x + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float f[8];
      unpack8<T>(keep[j], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) tot += red[w];
    const float r = rsqrtf(tot / static_cast<float>(K) + a.eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = (j * GEMV_CONSUMER_THREADS + tid) * 8;
      if (k < K) {
        float f[8], wv[8];
        unpack8<T>(keep[j], f);
        unpack8<T>((pre != nullptr && pre->have) ? pre->w[j] : ld_cached16(nw + k), wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = Elt<T>::to_f32(Elt<T>::from_f32(f[i] * r)) * wv[i];
        *reinterpret_cast<uint4*>(x_s + k) = pack8<T>(f);
      }
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
    return;
  }

  if (nw != nullptr) {
    float ss[NBX];
#pragma unroll
    for (int b = 0; b < NBX; ++b) ss[b] = 0.f;
    if (vec_ok) {
      for (int k = tid * 8; k < K; k += GEMV_CONSUMER_THREADS * 8) {
#pragma unroll
        for (int b = 0; b < NBX; ++b) {
          if (b < rows_present) {
            float f[8];
            unpack8<T>(ld_act16(x + (size_t)b * K + k), f);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss[b] = fmaf(f[i], f[i], ss[b]);
          }
        }
      }
    } else {
      for (int k = tid; k < K; k += GEMV_CONSUMER_THREADS) {
#pragma unroll
        for (int b = 0; b < NBX; ++b) {
          if (b < rows_present) {
            float v = ld_act_f32<T>(x + (size_t)b * K + k);
            ss[b] = fmaf(v, v, ss[b]);
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < NBX; ++b) {
      float s = warp_sum(ss[b]);
      if (lane == 0) red[b * GEMV_CONSUMER_WARPS + warp] = s;
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
#pragma unroll
    for (int b = 0; b < NBX; ++b) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) s += red[b * GEMV_CONSUMER_WARPS + w];
      rstd[b] = rsqrtf(s / static_cast<float>(K) + a.eps);
    }
  }

  if (vec_ok) {
    // UNR slices per thread are loaded back to back before any is stored: one L2 round trip per UNR slices instead
    // of one per slice (a row of 14336 elements is seven slices per thread)
    constexpr int UNR = (NBX == 1) ? 8 : (NBX == 2 ? 4 : (NBX <= 4 ? 2 : 1));
    constexpr int STEP = GEMV_CONSUMER_THREADS * 8;
    for (int k0 = tid * 8; k0 < Kp; k0 += STEP * UNR) {
      uint4 raw[UNR][NBX], wraw[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k = k0 + u * STEP;
        wraw[u] = make_uint4(0, 0, 0, 0);
        if (k < Kp && nw != nullptr) wraw[u] = ld_cached16(nw + k);
#pragma unroll
        for (int b = 0; b < NBX; ++b)
          raw[u][b] = (k < Kp && b < rows_present) ? ld_act16(x + (size_t)b * K + k) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k = k0 + u * STEP;
        if (k >= Kp) break;
        float wv[8];
        if (nw != nullptr) unpack8<T>(wraw[u], wv);
#pragma unroll
        for (int b = 0; b < NBX; ++b) {
          uint4 out = raw[u][b];  // zero for the rows past rows_present
          if (b < rows_present && nw != nullptr) {
            float f[8];
            unpack8<T>(raw[u][b], f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float n1 = Elt<T>::to_f32(Elt<T>::from_f32(f[i] * rstd[b]));
              f[i] = n1 * wv[i];
            }
            out = pack8<T>(f);
          }
          *reinterpret_cast<uint4*>(x_s + (size_t)b * pitch + k) = out;
        }
      }
    }
  } else {
    for (int k = tid; k < Kp; k += GEMV_CONSUMER_THREADS) {
#pragma unroll
      for (int b = 0; b < NBX; ++b) {
        T out = Elt<T>::from_f32(0.f);
        if (b < rows_present && k < K) {
          T raw = ld_act<T>(x + (size_t)b * K + k);
          if (nw != nullptr) {
            float n1 = Elt<T>::to_f32(Elt<T>::from_f32(Elt<T>::to_f32(raw) * rstd[b]));
            out = Elt<T>::from_f32(n1 * Elt<T>::to_f32(nw[k]));
          } else {
            out = raw;
          }
        }
        x_s[(size_t)b * pitch + k] = out;
      }
    }
  }
  named_bar_sync(1, GEMV_CONSUMER_THREADS);
}

// Plain staging of `rows` activation rows (no norm): used by the MoE down projection whose
// reduction runs over `rows` = computed experts. Same synchronisation contract as gemv_stage_x.
template <typename T>
__device__ __forceinline__ void gemv_stage_x_plain(const GemvArgs& a, int rows, T* x_s, int pitch, int tid) {
  const int K = a.K, Kp = a.Kp;
  const T* __restrict__ x = reinterpret_cast<const T*>(a.x);
  const bool vec_ok = ((K & 7) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (vec_ok) {
    constexpr int UNR = 4;  // loads of four slices in flight before the first store
    constexpr int STEP = GEMV_CONSUMER_THREADS * 8;
    for (int r = 0; r < rows; ++r)
      for (int k0 = tid * 8; k0 < K; k0 += STEP * UNR) {
        uint4 raw[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u)
          raw[u] = (k0 + u * STEP < K) ? ld_act16(x + (size_t)r * K + k0 + u * STEP) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < UNR; ++u)
          if (k0 + u * STEP < K) *reinterpret_cast<uint4*>(x_s + (size_t)r * pitch + k0 + u * STEP) = raw[u];
      }
  } else {
    for (int r = 0; r < rows; ++r)
      for (int k = tid; k < Kp; k += GEMV_CONSUMER_THREADS)
        x_s[(size_t)r * pitch + k] = (k < K) ? ld_act<T>(x + (size_t)r * K + k) : Elt<T>::from_f32(0.f);
  }
  named_bar_sync(1, GEMV_CONSUMER_THREADS);
}

// weight row that serves output row r (ROWS: r spans slots) / reduction segment seg (SEGMENTS)
__device__ __forceinline__ size_t gemv_weight_row(const GemvArgs& a, int r, int seg) {
  if (a.moe_mode == GEMV_MOE_NONE) return (size_t)r;
  if (a.moe_mode == GEMV_MOE_ROWS) {
    const int slot = r / a.N;
    return (size_t)gemv_slot_expert(a, slot) * a.N + (r - slot * a.N);
  }
  return (size_t)gemv_slot_expert(a, seg) * a.N + r;
}

// ---------------------------------------------------------------------------------------------
// tensor-core helpers of the pipeline kernels (mma.sync m16n8k16, fp32 accumulate) and ldmatrix
// ---------------------------------------------------------------------------------------------
template <typename T> struct MmaOp;
template <> struct MmaOp<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_addr));
}

// ---------------------------------------------------------------------------------------------
// 8-bit weight helpers
// ---------------------------------------------------------------------------------------------
// dot of 16 8-bit weights (signed for SYM_ROW, unsigned for GROUP_MIN) with 16 fp32 activations
template <bool SIGNED>
__device__ __forceinline__ float dot16_w8(const uint4& w, const float (&x)[16]) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t byte = (ww[i] >> (8 * j)) & 0xffu;
      const int q = SIGNED ? static_cast<int>(static_cast<signed char>(byte)) : static_cast<int>(byte);
      acc = fmaf(static_cast<float>(q), x[i * 4 + j], acc);
    }
  return acc;
}

// Four 8-bit integers (one 32-bit register) -> two packed 16-bit pairs {q0,q1}, {q2,q3}, exactly, without
// integer-to-float conversion instructions: the byte is planted in the mantissa of a constant and the
// constant subtracted (fp16: 1024 + u; bf16: through fp32 8388608 + u, then one packing conversion).
// `xmask` flips the sign bits of signed bytes (0x80808080, else 0) and `bias` is the matching constant
// (fp16 pair 1152 / 1024; fp32 8388736 / 8388608 for bf16), both loop-invariant registers, so that one code path
// serves both 8-bit formats without a branch.
template <typename T> struct W8Cvt;
template <> struct W8Cvt<__half> {
  static __device__ __forceinline__ uint32_t bias_for(bool is_signed) {
    const __half2 b = is_signed ? __floats2half2_rn(1152.f, 1152.f) : __floats2half2_rn(1024.f, 1024.f);
    return *reinterpret_cast<const uint32_t*>(&b);
  }
  static __device__ __forceinline__ void cvt4(uint32_t r, uint32_t xmask, uint32_t bias, uint32_t& lo, uint32_t& hi) {
    const uint32_t v = r ^ xmask;
    const uint32_t plo = __byte_perm(v, 0x64646464u, 0x5140);
    const uint32_t phi = __byte_perm(v, 0x64646464u, 0x5342);
    const __half2 b = *reinterpret_cast<const __half2*>(&bias);
    __half2 x = __hsub2(*reinterpret_cast<const __half2*>(&plo), b);
    __half2 y = __hsub2(*reinterpret_cast<const __half2*>(&phi), b);
    lo = *reinterpret_cast<uint32_t*>(&x);
    hi = *reinterpret_cast<uint32_t*>(&y);
  }
  template <bool SIGNED>
  static __device__ __forceinline__ void cvt4(uint32_t r, uint32_t& lo, uint32_t& hi) {
    cvt4(r, SIGNED ? 0x80808080u : 0u, bias_for(SIGNED), lo, hi);
  }
};
template <> struct W8Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t bias_for(bool is_signed) {
    return __float_as_uint(is_signed ? 8388736.f : 8388608.f);
  }
  static __device__ __forceinline__ void cvt4(uint32_t r, uint32_t xmask, uint32_t bias, uint32_t& lo, uint32_t& hi) {
    const uint32_t v = r ^ xmask;
    const float b = __uint_as_float(bias);
    const float f0 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650)) - b;
    const float f1 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7651)) - b;
    const float f2 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7652)) - b;
    const float f3 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7653)) - b;
    lo = Elt<__nv_bfloat16>::pack2(f0, f1);
    hi = Elt<__nv_bfloat16>::pack2(f2, f3);
  }
  template <bool SIGNED>
  static __device__ __forceinline__ void cvt4(uint32_t r, uint32_t& lo, uint32_t& hi) {
    cvt4(r, SIGNED ? 0x80808080u : 0u, bias_for(SIGNED), lo, hi);
  }
};

// ---------------------------------------------------------------------------------------------
// epilogues (one output element). Order follows csrc/linear/linear_fp16_kernels.cu:337-353:
// activation, * mul_bias, + add_bias, + residual; rounded once.
// ---------------------------------------------------------------------------------------------
// `pre`: the per-row scale and the residual value were loaded ahead of time (pre_scale, pre_res) instead of here,
// where a global load would stall the thread — and with it its warp's share of the next tiles — for a round trip.
template <typename T>
__device__ __forceinline__ void gemv_store_linear(const GemvArgs& a, int b, int n, float v,
                                                  unsigned long long comm_seq = 0, bool pre = false,
                                                  float pre_scale = 1.f, float pre_res = 0.f) {
  if (a.w8_fmt == MUI_W8_SYM_ROW) v *= pre ? pre_scale : Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales)[n]);
  if (a.activ == MUI_ACT_SILU) v = silu_f32(v);
  if (a.mul_bias) v *= Elt<T>::to_f32(reinterpret_cast<const T*>(a.mul_bias)[n]);
  if (a.add_bias) v += Elt<T>::to_f32(reinterpret_cast<const T*>(a.add_bias)[n]);
  const size_t o = (size_t)b * a.N + n;
  if (a.residual) v += pre ? pre_res : ld_act_f32<T>(reinterpret_cast<const T*>(a.residual) + o);
  if (a.use_comm) {
    comm_push(a.comm, comm_seq, o, v);
    return;
  }
  if (a.y_f32) a.y_f32[o] = v;
  if (a.y) reinterpret_cast<T*>(a.y)[o] = Elt<T>::from_f32(v);
}

// Tail of a tensor-parallel GEMV: called by all `nthreads` threads that ran the epilogues, after the CTA's last
// push (no CTA-wide barrier is needed: a cell is taken only once it carries this collective's sequence number). The CTA reduces the rows it owns — the same rows the
// same CTA of every other rank pushed — into y, polling its own segment until each rank's cells arrived.
// `row_of(i)` enumerates the CTA's rows.
template <typename T, typename RowFn>
__device__ __forceinline__ void gemv_comm_tail(const GemvArgs& a, unsigned long long seq, int tid, int nthreads,
                                               int bar_id, int num_rows, RowFn row_of) {
  T* y = reinterpret_cast<T*>(a.y);
  const int total = num_rows * a.B;
  unsigned ticket = 0;
  if (tid == 0) {
    trace_mark(a.trace, 4, true);
    ticket = comm_cta_arrive(a.comm);  // result is looked at after the polls below
  }
  for (int i = tid; i < total; i += nthreads) {
    const int b = i / num_rows, n = row_of(i - b * num_rows);
    const size_t o = (size_t)b * a.N + n;
    float v;
    if (comm_reduce_elem(a.comm, seq, o, &v)) y[o] = Elt<T>::from_f32(v);
  }
  if (a.trace != nullptr) {  // tracing only: the stamp below stands for the whole CTA
    named_bar_sync(bar_id, nthreads);
    if (tid == 0) {
      trace_mark(a.trace, 5, true);
      trace_mark(a.trace, 6, false);
    }
  }
  if (tid == 0) comm_cta_finish(a.comm, seq, ticket, gridDim.x);
}

// gate/up: t = silu(s*g) * (s*u); s is the router score of the slot (1 for dense / shared experts),
// applied before the SiLU as csrc/moeffn/gateupmoe_fp16_kernels.cu:355-360 does.
template <typename T>
__device__ __forceinline__ void gemv_store_gateup(const GemvArgs& a, int b, int out_row, int out_rows_total, float g,
                                                  float u, float score, bool pre = false, float pre_scale_g = 1.f,
                                                  float pre_scale_u = 1.f) {
  if (a.w8_fmt == MUI_W8_SYM_ROW) {
    g *= pre ? pre_scale_g : Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales)[out_row]);
    u *= pre ? pre_scale_u : Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales2)[out_row]);
  }
  g *= score;
  u *= score;
  float t = silu_f32(g) * u;
  reinterpret_cast<T*>(a.y)[(size_t)b * out_rows_total + out_row] = Elt<T>::from_f32(t);
}
