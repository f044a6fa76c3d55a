// GEMV-shaped kernels for one to eight activation rows on 16-bit weights, or on 8-bit weight-only
// quantised weights (WB = 8; symmetric per-row int8, or uint8 with per-group scale/min):
//   MODE 0  linear      y = act(W xn) * mul_bias + add_bias + residual
//   MODE 1  gate/up     t = silu(G xn) * (U xn)
// plus MoE addressing of either (device-side expert selection).
//
// Two implementations of the same math:
//  * gemv_pipe_kernel    — persistent, one CTA per SM. A producer warp streams 16-row tiles in 4 KiB row
//                          chunks into a shared-memory ring with 1-D bulk async copies (TMA) completing on
//                          mbarriers; eight consumer warps feed the tiles to mma.sync through ldmatrix
//                          (8-bit weights are widened in registers with a byte-permute + subtract, no
//                          conversion instructions). The weight prefetch does not depend on the previous
//                          kernel, so under programmatic dependent launch it overlaps that kernel's tail.
//  * gemv_generic_kernel — plain 16-byte streaming loads, the 256 threads of a CTA split K, cross-warp
//                          reduction in shared memory. Covers any K / alignment and the per-group format.
//
// HBM traffic per call: N*K*WB/8 (weights, read once) + scales + activations; fp32 accumulation.
// This header holds the kernels and their launchers; gemv_f16.cu and gemv_bf16.cu instantiate them for one element
// type each (two translation units compile side by side), gemv.cu holds the entry point that picks between them.
#pragma once

#include "gemv_common.cuh"

#include <algorithm>

namespace {

// =============================================================================================
// generic kernel
// =============================================================================================
template <typename T, int NB, int MODE, int WB>
__global__ void __launch_bounds__(GEMV_CONSUMER_THREADS) gemv_generic_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* x_s = reinterpret_cast<T*>(smem_raw);
  __shared__ float red[GEMV_CONSUMER_WARPS * 2 * NB];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  trace_start(a.trace);
  pdl_wait_prior_grid();
  pdl_launch_dependents();

  const int nseg = (a.moe_mode == GEMV_MOE_SEGMENTS) ? a.slots : 1;
  const int total_rows = (a.moe_mode == GEMV_MOE_ROWS) ? a.slots * a.N : a.N;
  const unsigned long long comm_seq = (MODE == 0 && a.use_comm) ? comm_begin(a.comm) : 0ull;
  if (a.moe_mode == GEMV_MOE_SEGMENTS)
    gemv_stage_x_plain<T>(a, a.slots, x_s, a.Kp, tid);
  else
    gemv_stage_x<T, NB>(a, a.B, x_s, a.Kp, red, tid);

  const int K = a.K, Kp = a.Kp;
  const unsigned char* __restrict__ W = reinterpret_cast<const unsigned char*>(a.W);
  const unsigned char* __restrict__ W2 = reinterpret_cast<const unsigned char*>(a.W2);
  constexpr int EB = WB / 8;           // bytes per weight
  constexpr int VEC = 16 / EB;         // weights per 16-byte load
  const bool group_fmt = (WB == 8) && (a.w8_fmt == MUI_W8_GROUP_MIN);
  const bool vec_ok = ((K % VEC) == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) &&
                      (MODE == 0 || (reinterpret_cast<uintptr_t>(W2) & 15) == 0) &&
                      (!group_fmt || a.group_shift >= 4);
  const int groups_per_row = group_fmt ? (K >> a.group_shift) : 0;
  const T* __restrict__ SM1 = reinterpret_cast<const T*>(a.scales);
  const T* __restrict__ SM2 = reinterpret_cast<const T*>(MODE == 0 ? a.scales : a.scales2);

  const int num_items = (MODE == 0) ? (total_rows + 1) / 2 : total_rows;
  for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
    const int ra = (MODE == 0) ? 2 * item : item;
    const bool second_valid = (MODE == 0) ? (ra + 1 < total_rows) : true;
    const int rb = (MODE == 0) ? (second_valid ? ra + 1 : ra) : ra;

    float acc[2][NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[0][b] = acc[1][b] = 0.f;

    for (int seg = 0; seg < nseg; ++seg) {
      const size_t wrow_a = gemv_weight_row(a, ra, seg), wrow_b = gemv_weight_row(a, rb, seg);
      const unsigned char* __restrict__ wa = W + wrow_a * (size_t)K * EB;
      const unsigned char* __restrict__ wb = ((MODE == 0) ? W : W2) + wrow_b * (size_t)K * EB;
      const T* xs = x_s + (size_t)seg * Kp;
      if (vec_ok) {
#pragma unroll 2
        for (int k = tid * VEC; k < K; k += GEMV_CONSUMER_THREADS * VEC) {
          const uint4 va = ld_stream16(wa + (size_t)k * EB);
          const uint4 vb = ld_stream16(wb + (size_t)k * EB);
          if (WB == 16) {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              float f[8];
              unpack8<T>(*reinterpret_cast<const uint4*>(xs + (size_t)b * Kp + k), f);
              acc[0][b] = dot8<T>(va, f, acc[0][b]);
              acc[1][b] = dot8<T>(vb, f, acc[1][b]);
            }
          } else {
            float sa = 1.f, ma = 0.f, sb = 1.f, mb = 0.f;
            if (group_fmt) {
              const int g = k >> a.group_shift;
              sa = Elt<T>::to_f32(SM1[(wrow_a * groups_per_row + g) * 2]);
              ma = Elt<T>::to_f32(SM1[(wrow_a * groups_per_row + g) * 2 + 1]);
              sb = Elt<T>::to_f32(SM2[(wrow_b * groups_per_row + g) * 2]);
              mb = Elt<T>::to_f32(SM2[(wrow_b * groups_per_row + g) * 2 + 1]);
            }
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              float f[16];
              {
                float lo[8], hi[8];
                unpack8<T>(*reinterpret_cast<const uint4*>(xs + (size_t)b * Kp + k), lo);
                unpack8<T>(*reinterpret_cast<const uint4*>(xs + (size_t)b * Kp + k + 8), hi);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  f[i] = lo[i];
                  f[8 + i] = hi[i];
                }
              }
              if (group_fmt) {
                // w = q*scale + min inside a group: sum(w x) = scale * sum(q x) + min * sum(x)
                float xsum = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) xsum += f[i];
                acc[0][b] += sa * dot16_w8<false>(va, f) + ma * xsum;
                acc[1][b] += sb * dot16_w8<false>(vb, f) + mb * xsum;
              } else {
                acc[0][b] += dot16_w8<true>(va, f);
                acc[1][b] += dot16_w8<true>(vb, f);
              }
            }
          }
        }
      } else {
        for (int k = tid; k < K; k += GEMV_CONSUMER_THREADS) {
          float fa, fb;
          if (WB == 16) {
            fa = Elt<T>::to_f32(reinterpret_cast<const T*>(wa)[k]);
            fb = Elt<T>::to_f32(reinterpret_cast<const T*>(wb)[k]);
          } else if (group_fmt) {
            const int g = k >> a.group_shift;
            fa = fmaf(static_cast<float>(wa[k]), Elt<T>::to_f32(SM1[(wrow_a * groups_per_row + g) * 2]),
                      Elt<T>::to_f32(SM1[(wrow_a * groups_per_row + g) * 2 + 1]));
            fb = fmaf(static_cast<float>(wb[k]), Elt<T>::to_f32(SM2[(wrow_b * groups_per_row + g) * 2]),
                      Elt<T>::to_f32(SM2[(wrow_b * groups_per_row + g) * 2 + 1]));
          } else {
            fa = static_cast<float>(static_cast<signed char>(wa[k]));
            fb = static_cast<float>(static_cast<signed char>(wb[k]));
          }
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            const float xv = Elt<T>::to_f32(xs[(size_t)b * Kp + k]);
            acc[0][b] = fmaf(fa, xv, acc[0][b]);
            acc[1][b] = fmaf(fb, xv, acc[1][b]);
          }
        }
      }
    }

#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float v = warp_sum(acc[j][b]);
        if (lane == 0) red[(warp * 2 + j) * NB + b] = v;
      }
    __syncthreads();
    if (MODE == 0) {
      if (tid < 2 * NB) {
        const int j = tid / NB, b = tid - j * NB;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) s += red[(w * 2 + j) * NB + b];
        if (b < a.B && (j == 0 || second_valid)) gemv_store_linear<T>(a, b, j == 0 ? ra : rb, s, comm_seq);
      }
    } else {
      if (tid < NB) {
        const int b = tid;
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) {
          g += red[(w * 2 + 0) * NB + b];
          u += red[(w * 2 + 1) * NB + b];
        }
        float score = 1.f;
        if (a.moe_mode == GEMV_MOE_ROWS) score = gemv_slot_score<T>(a, ra / a.N);
        if (b < a.B) gemv_store_gateup<T>(a, b, ra, total_rows, g, u, score);
      }
    }
    __syncthreads();
  }
  if (MODE == 0 && a.use_comm) {
    // rows of this CTA: items blockIdx.x, blockIdx.x + gridDim.x, ... hold rows 2*item and 2*item + 1
    const int my_items = (num_items > (int)blockIdx.x) ? (num_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    int my_rows = 2 * my_items;
    if (my_items > 0 && 2 * ((int)blockIdx.x + (my_items - 1) * (int)gridDim.x) + 1 >= total_rows) my_rows -= 1;
    const int gx = gridDim.x, bx = blockIdx.x;
    gemv_comm_tail<T>(a, comm_seq, tid, GEMV_CONSUMER_THREADS, 1, my_rows,
                      [gx, bx](int i) { return 2 * (bx + (i >> 1) * gx) + (i & 1); });
  }
  if (tid == 0) trace_end(a.trace);
}

// =============================================================================================
// bulk-copy pipeline kernel
// =============================================================================================
// A stage holds one 16-row tile: 16 row chunks of KC elements (one bulk copy each; the copy engine's
// per-copy cost makes copies below ~4 KiB the limiter, so KC is 2048 elements by default), each row padded
// by 16 bytes so that ldmatrix reads of 8 rows x 16 bytes hit distinct banks. MODE 0: 16 consecutive output
// rows. MODE 1: 8 gate rows (tile rows 0-7) and the 8 matching up rows (tile rows 8-15). The eight consumer
// warps split the chunk's K range in steps of 16 and feed mma.sync m16n8k16 (A = weight tile from shared
// memory, B = the staged activations, batch along n, fp32 accumulators) — no per-element conversions, so a
// stage costs each consumer warp a few dozen instructions; at the end of a row block the warps' partial
// tiles are summed through shared memory in a fixed order.
constexpr int PIPE_ROWS = 16;
constexpr int PIPE_MAX_STAGES = 8;
constexpr int PIPE_XPAD = 8;  // elements of padding per staged activation row (bank spread for ldmatrix)

template <int KC, int WB> struct PipeGeom {
  static constexpr int ROW_PITCH = KC * (WB / 8) + 16;        // bytes
  static constexpr int STAGE_BYTES = PIPE_ROWS * ROW_PITCH;   // bytes
};

struct PipeLayout {
  int x_off;      // activations [x_rows][Kp + PIPE_XPAD]
  int bar_off;    // full[stages], empty[stages]
  int red_off;    // floats: stage_x scratch, then 2 x [8 warps][16 rows][NB] partial tiles
  int abort_off;  // int
  int total;
};
__host__ __device__ inline PipeLayout pipe_layout(int stage_bytes, int stages, int x_rows, int Kp, int nb) {
  PipeLayout l;
  l.x_off = stages * stage_bytes;
  int x_bytes = ((x_rows * (Kp + PIPE_XPAD) * 2) + 15) & ~15;
  l.bar_off = l.x_off + x_bytes;
  l.red_off = l.bar_off + (2 * stages + 4) * 8;  // + tile_full[2], tile_free[2] of the asynchronous epilogue
  l.abort_off = l.red_off + 2 * GEMV_CONSUMER_WARPS * PIPE_ROWS * nb * 4;
  l.total = l.abort_off + 16;
  return l;
}

#include "gemv_xchunk.cuh"

// AE = 1 (8-bit weights, and 16-bit linear layers with the fused all-reduce): asynchronous epilogue. The tile loop on 8-bit weights is bound by the mma.sync issue rate
// (one m16n8k16 occupies a sub-partition's tensor pipe for ~34 cycles on this part, and 8-bit weights need as many of
// them per output as 16-bit ones for half the bytes), so every cycle the eight math warps spend at a row block's
// barrier, in its cross-warp sum or in its epilogue is lost. With AE an extra warp owns the cross-warp sum and the
// epilogue: the math warps drop their partial tiles into a double-buffered slot, arrive on an mbarrier and go on.
// With the fused all-reduce the epilogue is where a row block's partial sums are pushed to the peers (eight 64-bit
// system-scope stores per element): on the extra warp those stores no longer hold up warp 0's share of the next
// tiles, and with it every row block's barrier.
template <typename T, int NB, int MODE, int KC, int WB, int NPROD, int AE>
__global__ void __launch_bounds__(GEMV_CONSUMER_THREADS + 32 * (NPROD + AE)) gemv_pipe_kernel(const GemvArgs a,
                                                                                             const int num_stages) {
  using G = PipeGeom<KC, WB>;
  constexpr int MW = GEMV_CONSUMER_WARPS;  // warps in the tile loop
  constexpr int EB = WB / 8;  // bytes per weight
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int x_rows = (a.moe_mode == GEMV_MOE_SEGMENTS) ? a.slots : NB;
  const PipeLayout lay = pipe_layout(G::STAGE_BYTES, num_stages, x_rows, a.Kp, NB);
  unsigned char* stage_mem = smem_raw;
  T* x_s = reinterpret_cast<T*>(smem_raw + lay.x_off);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw + lay.bar_off);
  uint64_t* empty_bar = full_bar + num_stages;
  uint64_t* tile_full = empty_bar + num_stages;  // [2] partial tiles of a row block written (AE)
  uint64_t* tile_free = tile_full + 2;           // [2] slot drained by the epilogue warp (AE)
  float* red = reinterpret_cast<float*>(smem_raw + lay.red_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + lay.abort_off);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(full_bar + s, NPROD);
      mbar_init(empty_bar + s, MW);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tile_full + s, MW);
      mbar_init(tile_free + s, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  trace_start(a.trace);
  __syncthreads();
  pdl_launch_dependents();

  constexpr int ROWS_PER_STAGE = (MODE == 0) ? 16 : 8;  // output rows per stage
  const int K = a.K, Kp = a.Kp;
  const int x_pitch = Kp + PIPE_XPAD;
  const int nseg = (a.moe_mode == GEMV_MOE_SEGMENTS) ? a.slots : 1;
  const int total_rows = (a.moe_mode == GEMV_MOE_ROWS) ? a.slots * a.N : a.N;
  const int r_begin = static_cast<int>((long long)total_rows * blockIdx.x / gridDim.x);
  const int r_end = static_cast<int>((long long)total_rows * (blockIdx.x + 1) / gridDim.x);
  const int nblk = (r_end - r_begin + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE;
  const int nchunks = (K + KC - 1) / KC;
  const int cpb = nseg * nchunks;  // stage items per row block
  const int total_items = nblk * cpb;

  if (warp >= MW && warp < MW + NPROD) {
    // ------------------------------ producer warps ------------------------------
    // each of the NPROD warps issues the copies of its share of the 16 tile rows (the copy engine takes one
    // warp's copies one after the other; two issuing warps double the ingest rate of 4 KiB copies)
    constexpr int ROWS_PER_PROD = PIPE_ROWS / NPROD;
    const int prod = warp - MW;
    if (a.moe_mode != GEMV_MOE_NONE) pdl_wait_prior_grid();  // expert ids come from the previous kernel
    const uint64_t policy = l2_policy_evict_first();
    const unsigned char* __restrict__ W = reinterpret_cast<const unsigned char*>(a.W);
    const unsigned char* __restrict__ W2 = reinterpret_cast<const unsigned char*>(a.W2);
    int issued = 0;
    bool ok = true;
    int blk = 0, c = 0, seg = 0, kc = 0;  // item -> (row block, segment, chunk) without divisions
    int s = -1;         // ring slot and its phase bit, advanced without divisions
    uint32_t ph = 1;
    for (int it = 0; it < total_items; ++it) {
      if (++s == num_stages) s = 0;
      if (s == 0) ph ^= 1u;
      int w_ok = 1;
      if (lane == 0) w_ok = mbar_wait_bounded(empty_bar + s, ph ^ 1u, abort_flag) ? 1 : 0;
      w_ok = __shfl_sync(MUI_FULL_MASK, w_ok, 0);
      if (!w_ok) {
        if (lane == 0 && !*abort_flag) {
          mui_dev_set_status(MUI_DEV_TIMEOUT_EMPTY, s);
          *abort_flag = 1;
        }
        ok = false;
        break;
      }
      const int rb = r_begin + blk * ROWS_PER_STAGE;
      const int kc_len = min(KC, K - kc * KC);
      const uint32_t bytes = static_cast<uint32_t>(kc_len) * EB;
      const int rows_valid = min(ROWS_PER_STAGE, r_end - rb);
      // tile row tr: MODE 0 -> output row rb + tr; MODE 1 -> gate (tr < 8) / up (tr >= 8) row rb + tr%8
      const int tr = prod * ROWS_PER_PROD + lane;
      const int orow = (MODE == 0) ? tr : (tr & 7);
      const bool mine = (lane < ROWS_PER_PROD) && (orow < rows_valid);
      const int ncopies = __popc(__ballot_sync(MUI_FULL_MASK, mine));
      if (lane == 0) mbar_arrive_expect_tx(full_bar + s, static_cast<uint32_t>(ncopies) * bytes);
      __syncwarp();
      if (mine) {
        const unsigned char* src = ((MODE == 1 && tr >= 8) ? W2 : W) +
                                   (gemv_weight_row(a, rb + orow, seg) * (size_t)K + (size_t)kc * KC) * EB;
        bulk_load_1d(stage_mem + (size_t)s * G::STAGE_BYTES + (size_t)tr * G::ROW_PITCH, src, bytes, full_bar + s,
                     policy);
      }
      issued = it + 1;
      if (++kc == nchunks) {
        kc = 0;
        ++seg;
      }
      if (++c == cpb) {
        c = 0;
        seg = 0;
        ++blk;
      }
    }
    if (ok && prod == 0) {
      pipe_prefetch_next(a, lane);
    }
    if (!ok && lane == 0 && prod == 0) {
      // leave no copy in flight behind: wait (bounded) for every stage that was armed
      const int first = max(0, issued - num_stages);
      for (int it = first; it < issued; ++it) {
        int zero = 0;
        if (!mbar_wait_bounded(full_bar + (it % num_stages), (it / num_stages) & 1, &zero))
          mui_dev_set_status(MUI_DEV_TIMEOUT_DRAIN, it % num_stages);
      }
    }
  } else if (AE && warp == MW + NPROD) {
    // ------------------------------ epilogue warp (AE) ------------------------------
    // per row block: the eight warps' partial tiles are summed in a fixed order, then the epilogue; the operands of
    // the epilogue (per-row scales, residual) are fetched before the wait for the tiles
    pdl_wait_prior_grid();
    const unsigned long long eseq = (MODE == 0 && a.use_comm) ? comm_begin(a.comm) : 0ull;
    constexpr int OUTS = ROWS_PER_STAGE * NB;       // outputs per row block
    constexpr int PER_LANE = (OUTS + 31) / 32;
    const bool sym = (WB == 8) && a.w8_fmt == MUI_W8_SYM_ROW && a.moe_mode == GEMV_MOE_NONE;
    for (int blk = 0; blk < nblk; ++blk) {
      const int rb = r_begin + blk * ROWS_PER_STAGE;
      const int slot = blk & 1;
      float pa[PER_LANE], pb[PER_LANE];
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        pa[i] = (MODE == 0) ? 0.f : 1.f;
        pb[i] = 1.f;
        const int o = lane + 32 * i, r = o / NB, b = o - r * NB, row = rb + r;
        if (o < OUTS && row < r_end && b < a.B) {
          if (MODE == 0) {
            if (a.residual) pa[i] = ld_act_f32<T>(reinterpret_cast<const T*>(a.residual) + (size_t)b * a.N + row);
            if (sym) pb[i] = Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales)[row]);
          } else if (sym) {
            pa[i] = Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales)[row]);
            pb[i] = Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales2)[row]);
          }
        }
      }
      if (!mbar_wait_bounded(tile_full + slot, (blk >> 1) & 1, abort_flag)) {
        if (lane == 0 && !*abort_flag) {
          mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, 64 + slot);
          *abort_flag = 1;
        }
        break;
      }
      const float* rbuf = red + slot * (MW * PIPE_ROWS * NB);
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int o = lane + 32 * i, r = o / NB, b = o - r * NB, row = rb + r;
        if (o < OUTS && row < r_end && b < a.B) {
          if (MODE == 0) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < MW; ++w) v += rbuf[(w * PIPE_ROWS + r) * NB + b];
            gemv_store_linear<T>(a, b, row, v, eseq, true, pb[i], pa[i]);
          } else {
            float g = 0.f, u = 0.f;
#pragma unroll
            for (int w = 0; w < MW; ++w) {
              g += rbuf[(w * PIPE_ROWS + r) * NB + b];
              u += rbuf[(w * PIPE_ROWS + r + 8) * NB + b];
            }
            float score = 1.f;
            if (a.moe_mode == GEMV_MOE_ROWS) score = gemv_slot_score<T>(a, row / a.N);
            gemv_store_gateup<T>(a, b, row, total_rows, g, u, score, a.moe_mode == GEMV_MOE_NONE, pa[i], pb[i]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(tile_free + slot);
    }
    if (lane == 0) trace_end(a.trace);
  } else {
    // ------------------------------ consumer warps ------------------------------
    GemvNormPre norm_pre;
    norm_pre.have = false;
    if (a.moe_mode != GEMV_MOE_SEGMENTS) gemv_prefetch_norm<T, NB>(a, tid, norm_pre);
    pdl_wait_prior_grid();
    if (tid == 0) trace_mark(a.trace, 2, false);
    const unsigned long long comm_seq = (MODE == 0 && a.use_comm) ? comm_begin(a.comm) : 0ull;
    // Epilogue operands (residual, per-row 8-bit scales) of every row block this thread will finish, loaded now so
    // that their round trip overlaps the activation staging instead of stalling a row block's epilogue.
    constexpr int EPI_MAX = 16;
    const bool epi_pre = !AE && nblk <= EPI_MAX;
    float epi_a[EPI_MAX], epi_b[EPI_MAX];  // MODE 0: residual, scale; MODE 1: gate scale, up scale
#pragma unroll
    for (int i = 0; i < EPI_MAX; ++i) {
      epi_a[i] = (MODE == 0) ? 0.f : 1.f;
      epi_b[i] = 1.f;
    }
    if (epi_pre && tid < ROWS_PER_STAGE * NB) {
      const int r = tid / NB, b = tid - r * NB;
      const bool sym = (WB == 8) && a.w8_fmt == MUI_W8_SYM_ROW && a.moe_mode == GEMV_MOE_NONE;
#pragma unroll
      for (int i = 0; i < EPI_MAX; ++i) {
        const int row = r_begin + i * ROWS_PER_STAGE + r;
        if (i < nblk && row < r_end && b < a.B) {
          if (MODE == 0) {
            if (a.residual) epi_a[i] = ld_act_f32<T>(reinterpret_cast<const T*>(a.residual) + (size_t)b * a.N + row);
            if (sym) epi_b[i] = Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales)[row]);
          } else if (sym) {
            epi_a[i] = Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales)[row]);
            epi_b[i] = Elt<T>::to_f32(reinterpret_cast<const T*>(a.scales2)[row]);
          }
        }
      }
    }
    if (a.moe_mode == GEMV_MOE_SEGMENTS)
      gemv_stage_x_plain<T>(a, a.slots, x_s, x_pitch, tid);
    else
      gemv_stage_x<T, NB>(a, a.B, x_s, x_pitch, red, tid, &norm_pre);
    if (tid == 0) trace_mark(a.trace, 3, true);

    float d[4] = {0.f, 0.f, 0.f, 0.f};
    float d2[4] = {0.f, 0.f, 0.f, 0.f};  // 8-bit path only
    // ldmatrix sources. A (weight tile, 16 rows x 16 k): lane gives tile row (lane%8) + 8*((lane/8)%2), k offset
    // 8*(lane/16). B (activations, 16 k x 8 batch): lanes 0-15 give staged row min(lane%8, NB-1) (columns past
    // the batch repeat the last row; their results are never read), k offset 8*((lane/8)%2).
    const uint32_t a_lane_off = static_cast<uint32_t>(((lane & 7) + ((lane >> 3) & 1) * 8) * G::ROW_PITCH +
                                                      (lane >> 4) * 16);
    const int b_row = ((lane & 7) < NB) ? (lane & 7) : (NB - 1);
    const uint32_t b_lane_off = static_cast<uint32_t>((b_row * x_pitch + ((lane >> 3) & 1) * 8) * 2);
    const uint32_t stage_base = smem_u32(stage_mem);
    const uint32_t x_base = smem_u32(x_s);

    int blk = 0, c = 0, seg = 0, kc = 0;
    int s = -1;         // ring slot and its phase bit, advanced without divisions
    uint32_t ph = 1;
    for (int it = 0; it < total_items; ++it) {
      if (++s == num_stages) s = 0;
      if (s == 0) ph ^= 1u;
      if (!mbar_wait_bounded(full_bar + s, ph, abort_flag)) {
        if (lane == 0 && !*abort_flag) {
          mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, s);
          *abort_flag = 1;
        }
        break;
      }
      const int kc_len = min(KC, K - kc * KC);
      const uint32_t a_addr = stage_base + static_cast<uint32_t>(s) * G::STAGE_BYTES + a_lane_off;
      if (WB == 16) {
        const int nsteps = kc_len >> 4;
        // MoE segments: segment `seg` multiplies activation row `seg` (NB == 1 there)
        const uint32_t b_addr = x_base + b_lane_off + static_cast<uint32_t>((seg * x_pitch + kc * KC) * 2);
#pragma unroll 4
        for (int j = warp; j < nsteps; j += MW) {
          uint32_t af[4], b0, b1;
          ldmatrix_x4(af, a_addr + j * 32);
          ldmatrix_x2(b0, b1, b_addr + j * 32);
          MmaOp<T>::run(d, af, b0, b1);
        }
      } else {
        // 8-bit weights: one ldmatrix.x4 brings 16 rows x 32 bytes; this thread gets bytes 4q..4q+3 (q = lane%4)
        // of k-blocks [0,16) and [16,32) for tile rows lane/4 and lane/4+8. The four bytes become the k-slots
        // {2q,2q+1} and {2q+8,2q+9} of one mma, so the activations are read as x[4q..4q+3] in the same order.
        const int nsteps = kc_len >> 5;
        const int n_row = ((lane >> 2) < NB) ? (lane >> 2) : (NB - 1);
        const T* xrow = x_s + (size_t)(n_row + seg) * x_pitch + (size_t)kc * KC + (lane & 3) * 4;
        const bool sgn = (a.w8_fmt == MUI_W8_SYM_ROW);
        const uint32_t xmask = sgn ? 0x80808080u : 0u, cbias = W8Cvt<T>::bias_for(sgn);
        const uint32_t x_addr = smem_u32(xrow);
#pragma unroll 4
        for (int j = warp; j < nsteps; j += MW) {
          uint32_t r[4];
          ldmatrix_x4(r, a_addr + j * 32);
          uint32_t xa0, xa1, xb0, xb1;
          lds_v2(x_addr + j * 64, xa0, xa1);
          lds_v2(x_addr + j * 64 + 32, xb0, xb1);
          uint32_t af[4], bf[4];
          W8Cvt<T>::cvt4(r[0], xmask, cbias, af[0], af[2]);
          W8Cvt<T>::cvt4(r[1], xmask, cbias, af[1], af[3]);
          W8Cvt<T>::cvt4(r[2], xmask, cbias, bf[0], bf[2]);
          W8Cvt<T>::cvt4(r[3], xmask, cbias, bf[1], bf[3]);
          MmaOp<T>::run(d, af, xa0, xa1);
          MmaOp<T>::run(d2, bf, xb0, xb1);  // second accumulator: halves the dependent mma chain
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar + s);

      if (++kc == nchunks) {
        kc = 0;
        ++seg;
      }
      if (++c == cpb) {
        // row block complete: sum the eight warps' partial tiles in a fixed order, then the epilogue
        c = 0;
        seg = 0;
        const int rb = r_begin + blk * ROWS_PER_STAGE;
        float* rbuf = red + (blk & 1) * (MW * PIPE_ROWS * NB);
        // this thread holds D[tile row lane/4 (+8)][batch (lane%4)*2 + {0,1}]
        const int trow = lane >> 2, n0 = (lane & 3) * 2;
        if (AE && blk >= 2) {
          // the slot's previous tiles (row block blk - 2) must have been drained by the epilogue warp
          if (!mbar_wait_bounded(tile_free + (blk & 1), ((blk >> 1) - 1) & 1, abort_flag)) {
            if (lane == 0 && !*abort_flag) {
              mui_dev_set_status(MUI_DEV_TIMEOUT_EMPTY, 64 + (blk & 1));
              *abort_flag = 1;
            }
            break;
          }
        }
        if (WB == 8) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            d[q] += d2[q];
            d2[q] = 0.f;
          }
        }
        if (n0 < NB) {
          rbuf[(warp * PIPE_ROWS + trow) * NB + n0] = d[0];
          rbuf[(warp * PIPE_ROWS + trow + 8) * NB + n0] = d[2];
        }
        if (n0 + 1 < NB) {
          rbuf[(warp * PIPE_ROWS + trow) * NB + n0 + 1] = d[1];
          rbuf[(warp * PIPE_ROWS + trow + 8) * NB + n0 + 1] = d[3];
        }
        d[0] = d[1] = d[2] = d[3] = 0.f;
        if (AE) {
          __syncwarp();
          if (lane == 0) mbar_arrive(tile_full + (blk & 1));  // release: the tile stores above are visible to the waiter
          ++blk;
          continue;
        }
        named_bar_sync(1, GEMV_CONSUMER_THREADS);
        if (tid < ROWS_PER_STAGE * NB) {
          const int r = tid / NB, b = tid - r * NB;
          const int row = rb + r;
          if (row < r_end && b < a.B) {
            if (MODE == 0) {
              float v = 0.f;
#pragma unroll
              for (int w = 0; w < MW; ++w) v += rbuf[(w * PIPE_ROWS + r) * NB + b];
              gemv_store_linear<T>(a, b, row, v, comm_seq, epi_pre, epi_b[0], epi_a[0]);
            } else {
              float g = 0.f, u = 0.f;
#pragma unroll
              for (int w = 0; w < MW; ++w) {
                g += rbuf[(w * PIPE_ROWS + r) * NB + b];
                u += rbuf[(w * PIPE_ROWS + r + 8) * NB + b];
              }
              float score = 1.f;
              if (a.moe_mode == GEMV_MOE_ROWS) score = gemv_slot_score<T>(a, row / a.N);
              gemv_store_gateup<T>(a, b, row, total_rows, g, u, score,
                                   epi_pre && a.moe_mode == GEMV_MOE_NONE, epi_a[0], epi_b[0]);
            }
          }
        }
        // next row block's operands move to the front (static register indices)
#pragma unroll
        for (int i = 0; i + 1 < EPI_MAX; ++i) {
          epi_a[i] = epi_a[i + 1];
          epi_b[i] = epi_b[i + 1];
        }
        ++blk;
      }
    }
    if (MODE == 0 && a.use_comm)
      gemv_comm_tail<T>(a, comm_seq, tid, GEMV_CONSUMER_THREADS, 1, r_end - r_begin,
                        [r_begin](int i) { return r_begin + i; });
    if (tid == 0) trace_end(a.trace);  // (the latest stamp of the launch is kept)
  }
}

#include "gemv_w8g.cuh"

// =============================================================================================
// host dispatch
// =============================================================================================
template <typename T, int NB, int MODE, int KC, int WB, int AE>
mui_status_t launch_pipe_ae(cudaStream_t stream, const GemvArgs& a, int pdl, int total_rows, int x_rows,
                            const MuiDeviceInfo* dev, bool* applicable) {
  using G = PipeGeom<KC, WB>;
  // One CTA per SM with (nearly) all of its shared memory: ~190 KiB of copies in flight per SM is what keeps
  // HBM busy; with half of that the kernel runs ~25 % slower.
  // 226 KiB: with K = 14336 the staged activations (28 KiB) and three 64.25 KiB stages need 222.8 KiB
  // (two CTAs per SM with half-size stages measured +5 % on 8-bit weights and -3 % on 16-bit ones: not used)
  const int budget = 226 * 1024;
  const int fixed = pipe_layout(G::STAGE_BYTES, 0, x_rows, a.Kp, NB).total;
  const int stages = std::min((budget - fixed) / G::STAGE_BYTES, PIPE_MAX_STAGES);
  if (stages < 2) {
    *applicable = false;
    return MUI_OK;
  }
  *applicable = true;
  const PipeLayout lay = pipe_layout(G::STAGE_BYTES, stages, x_rows, a.Kp, NB);
  const int units = (total_rows + 7) / 8;  // at least one row block per CTA
  const int sms = std::max(1, dev->sm_count - std::min(a.reserve_sms, dev->sm_count / 4));
  const int grid = std::max(1, std::min(units, sms));
  // one producer warp: a second one doubles the issue rate of 4 KiB copies but measured no faster end to end
  if (WB == 8 && a.use_comm) {
    mui_set_error("8-bit weights with the fused all-reduce are not supported");
    return MUI_ERR_UNSUPPORTED;
  }
  auto kern = gemv_pipe_kernel<T, NB, MODE, KC, WB, 1, AE>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared));
    configured = true;
  }
  MUI_CUDA_CHECK(mui_launch(kern, dim3(grid), dim3(GEMV_CONSUMER_THREADS + 32 * (1 + AE)), (size_t)lay.total, stream, pdl, a,
                            stages));
  return MUI_OK;
}

// Asynchronous epilogue warp: always for 8-bit weights; for 16-bit linear layers where the epilogue pushes to the
// peers or the launch is short.
template <typename T, int NB, int MODE, int KC, int WB>
mui_status_t launch_pipe(cudaStream_t stream, const GemvArgs& a, int pdl, int total_rows, int x_rows,
                         const MuiDeviceInfo* dev, bool* applicable) {
  if constexpr (WB == 8) {
    return launch_pipe_ae<T, NB, MODE, KC, WB, 1>(stream, a, pdl, total_rows, x_rows, dev, applicable);
  } else {
    if constexpr (MODE == 0) {
      // also for short launches (a few row blocks per CTA), where the last row block's barrier, cross-warp sum and
      // epilogue are a visible part of the whole (measured: 4096 x 512: 3.60 -> 3.39 us, 4096 x 1792: 4.82 -> 4.44 us;
      // long launches lose 1 %)
      if (a.use_comm || (size_t)total_rows * a.K * 2 <= ((size_t)24 << 20))
        return launch_pipe_ae<T, NB, MODE, KC, WB, 1>(stream, a, pdl, total_rows, x_rows, dev, applicable);
    }
    return launch_pipe_ae<T, NB, MODE, KC, WB, 0>(stream, a, pdl, total_rows, x_rows, dev, applicable);
  }
}

// Per-group 8-bit format on the bulk-copy pipeline (gemv_w8g.cuh); *applicable = false when the activations leave no
// room for two weight stages.
template <typename T, int NB, int LAYOUT>
mui_status_t launch_gm(cudaStream_t stream, const GemvArgs& a, int pdl, const MuiDeviceInfo* dev, bool* applicable) {
  const int out_tile = (LAYOUT == 2) ? 32 : 16;
  const int ngroups = a.K >> a.group_shift;
  const int budget = 226 * 1024;
  const int fixed = gm_layout(0, NB, a.Kp, ngroups, out_tile).total;
  const int stages = std::min((budget - fixed) / GM_STAGE_BYTES, PIPE_MAX_STAGES);
  *applicable = stages >= 2;
  if (!*applicable) return MUI_OK;
  const GmLayout lay = gm_layout(stages, NB, a.Kp, ngroups, out_tile);
  const int units = (a.N + 7) / 8;
  const int sms = std::max(1, dev->sm_count - std::min(a.reserve_sms, dev->sm_count / 4));
  const int grid = std::max(1, std::min(units, sms));
  auto kern = gemv_pipe_gm_kernel<T, NB, LAYOUT>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared));
    configured = true;
  }
  MUI_CUDA_CHECK(mui_launch(kern, dim3(grid), dim3(32 * (GM_MW + 2)), (size_t)lay.total, stream, pdl, a, stages));
  return MUI_OK;
}

// Chunk-staged batched variant (gemv_xchunk.cuh)
template <typename T, int NB, int MODE, int WB>
mui_status_t launch_xchunk(cudaStream_t stream, const GemvArgs& a, int pdl, const MuiDeviceInfo* dev) {
  using G = XcGeom<WB>;
  const int budget = 226 * 1024;
  const int fixed = xc_layout(G::STAGE_BYTES, 0, NB).total;
  const int stages = std::min((budget - fixed) / G::STAGE_BYTES, PIPE_MAX_STAGES);
  const XcLayout lay = xc_layout(G::STAGE_BYTES, stages, NB);
  const int units = (a.N + 7) / 8;
  const int sms = std::max(1, dev->sm_count - std::min(a.reserve_sms, dev->sm_count / 4));
  const int grid = std::max(1, std::min(units, sms));
  auto kern = gemv_pipe_xchunk_kernel<T, NB, MODE, WB>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared));
    configured = true;
  }
  MUI_CUDA_CHECK(mui_launch(kern, dim3(grid), dim3(GEMV_CONSUMER_THREADS + 32), (size_t)lay.total, stream, pdl, a,
                            stages));
  return MUI_OK;
}

template <typename T, int NB, int MODE, int WB>
mui_status_t launch_gemv_t(cudaStream_t stream, const GemvArgs& a, unsigned flags, const MuiDeviceInfo* dev) {
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  const int total_rows = (a.moe_mode == GEMV_MOE_ROWS) ? a.slots * a.N : a.N;
  const int x_rows = (a.moe_mode == GEMV_MOE_SEGMENTS) ? a.slots : NB;
  const size_t x_bytes = (size_t)x_rows * a.Kp * 2;

  // The pipeline needs 16-byte aligned rows for the bulk copies and whole mma k-steps (16 weights of 16 bits,
  // 32 of 8 bits); the per-group 8-bit format runs on the plain-load kernel.
  const int kstep = (WB == 16) ? 16 : 32;
  const bool aligned = ((a.K % kstep) == 0) && ((reinterpret_cast<uintptr_t>(a.W) & 15) == 0) &&
                       (MODE == 0 || (reinterpret_cast<uintptr_t>(a.W2) & 15) == 0) &&
                       (WB == 16 || a.w8_fmt == MUI_W8_SYM_ROW);
  bool use_pipe = aligned && !(flags & MUI_FLAG_FORCE_GENERIC);
  if constexpr (WB == 8) {
    if (a.w8_fmt == MUI_W8_GROUP_MIN) {
      // groups of 32..2048 weights, whole groups per stage, 16-byte aligned rows and tables
      const bool gm_ok = a.group_shift >= 5 && a.group_shift <= 11 && (a.K % 16) == 0 &&
                         ((reinterpret_cast<uintptr_t>(a.W) & 15) == 0) &&
                         (MODE == 0 || a.w8_pack || (reinterpret_cast<uintptr_t>(a.W2) & 15) == 0) &&
                         ((reinterpret_cast<uintptr_t>(a.scales) & 7) == 0) && a.moe_mode == GEMV_MOE_NONE &&
                         !a.use_comm && !(flags & MUI_FLAG_FORCE_GENERIC);
      if (gm_ok) {
        bool applicable = false;
        mui_status_t st;
        if (MODE == 0) st = launch_gm<T, NB, 0>(stream, a, pdl, dev, &applicable);
        else if (a.w8_pack) st = launch_gm<T, NB, 2>(stream, a, pdl, dev, &applicable);
        else st = launch_gm<T, NB, 1>(stream, a, pdl, dev, &applicable);
        if (st != MUI_OK || applicable) return st;
      }
      if (a.w8_pack) {
        mui_set_error("packed 8-bit gate/up: shape not served by the pipeline kernel (H=%d, group 2^%d, batch %d)",
                      a.K, a.group_shift, a.B);
        return MUI_ERR_UNSUPPORTED;
      }
    }
  }
  if constexpr (NB >= 2) {
    if (use_pipe && a.moe_mode == GEMV_MOE_NONE && ((a.K & 7) == 0) &&
        ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0) &&
        (a.norm_w == nullptr || (reinterpret_cast<uintptr_t>(a.norm_w) & 15) == 0)) {
      // batches: stage the activations chunk by chunk whenever whole rows would leave the weight ring fewer than
      // three full stages (16-bit weights) or fewer than two (8-bit weights: their chunked row copies are 2 KiB,
      // which the copy engine ingests more slowly; measured at the Llama-3-8B MLP shape, two whole-row stages
      // still win there)
      using G = PipeGeom<2048 * (16 / WB), WB>;
      const int fixed = pipe_layout(G::STAGE_BYTES, 0, x_rows, a.Kp, NB).total;
      if ((226 * 1024 - fixed) / G::STAGE_BYTES < (WB == 16 ? 3 : 2))
        return launch_xchunk<T, NB, MODE, WB>(stream, a, pdl, dev);
    }
  }
  if (use_pipe) {
    bool applicable = false;
    mui_status_t st;
    // row chunks of 4 KiB: 2048 16-bit or 4096 8-bit weights
    st = launch_pipe<T, NB, MODE, 2048 * (16 / WB), WB>(stream, a, pdl, total_rows, x_rows, dev, &applicable);
    if (st != MUI_OK || applicable) return st;
    // smaller stages when the staged activations leave no room for two 64 KiB ones
    st = launch_pipe<T, NB, MODE, 1024 * (16 / WB), WB>(stream, a, pdl, total_rows, x_rows, dev, &applicable);
    if (st != MUI_OK || applicable) return st;
  }
  if (flags & MUI_FLAG_FORCE_PIPELINE) {
    mui_set_error("bulk-copy pipeline not applicable (K=%d, alignment or activation size)", a.K);
    return MUI_ERR_UNSUPPORTED;
  }

  // generic
  MUI_REQUIRE(x_bytes <= 200 * 1024, MUI_ERR_UNSUPPORTED,
              "activations (%zu bytes) do not fit the shared-memory staging of the GEMV", x_bytes);
  auto kern = gemv_generic_kernel<T, NB, MODE, WB>;
  static bool configured_g = false;
  if (x_bytes > 48 * 1024 && !configured_g) {
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured_g = true;
  }
  const int num_items = (MODE == 0) ? (total_rows + 1) / 2 : total_rows;
  int per_sm = (int)std::min<size_t>(6, (size_t)(224 * 1024) / (x_bytes + 2048));
  per_sm = std::max(per_sm, 1);
  int grid = std::max(1, std::min(num_items, dev->sm_count * per_sm));
  MUI_CUDA_CHECK(mui_launch(kern, dim3(grid), dim3(GEMV_CONSUMER_THREADS), x_bytes, stream, pdl, a));
  return MUI_OK;
}

template <typename T, int MODE, int WB>
mui_status_t launch_gemv_nb(cudaStream_t stream, const GemvArgs& a, int nb, unsigned flags, const MuiDeviceInfo* dev) {
  switch (nb) {
    case 1: return launch_gemv_t<T, 1, MODE, WB>(stream, a, flags, dev);
    case 2: return launch_gemv_t<T, 2, MODE, WB>(stream, a, flags, dev);
    case 4: return launch_gemv_t<T, 4, MODE, WB>(stream, a, flags, dev);
    default: return launch_gemv_t<T, 8, MODE, WB>(stream, a, flags, dev);
  }
}

template <typename T>
mui_status_t launch_gemv_dt(cudaStream_t stream, int mode, const GemvArgs& a, int nb, unsigned flags,
                            const MuiDeviceInfo* dev) {
  if (a.w8_fmt < 0)
    return mode == 0 ? launch_gemv_nb<T, 0, 16>(stream, a, nb, flags, dev)
                     : launch_gemv_nb<T, 1, 16>(stream, a, nb, flags, dev);
  return mode == 0 ? launch_gemv_nb<T, 0, 8>(stream, a, nb, flags, dev)
                   : launch_gemv_nb<T, 1, 8>(stream, a, nb, flags, dev);
}

}  // namespace
