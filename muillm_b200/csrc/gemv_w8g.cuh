// Bulk-copy pipeline GEMV on the reference's per-group 8-bit format: w = q * scale_g + min_g, q in 0..255, one
// {scale, min} 16-bit pair per `group` consecutive weights of a row (muillm/quantization/rtnquantizer.py:48-88;
// kernels csrc/int8_linear_kernels.cu:212-226, csrc/int8_gateup_kernels.cu:255,522). Included by gemv_kernels.cuh.
//
// Inside one group  sum_k w x = scale * sum_k q x + min * sum_k x:  the first sum runs on the tensor cores with q
// widened to 16 bits (exactly), the second is a per-group sum of the staged activations computed once per CTA.
// Warps take whole groups of a stage, so a warp accumulates one group in a scratch tile and folds it into its
// running tile with the group's scale and min (both fetched one group ahead). As in gemv_pipe_kernel with 8-bit
// weights, the tile loop is bound by the mma.sync issue rate, so the cross-warp sum and the epilogue of a row block
// run on a warp of their own while the math warps go on with the next block.
//
// LAYOUT 0  linear   : tile = 16 rows of W                       (16 output rows per stage, 4096 k)
// LAYOUT 1  gate/up  : tile = 8 gate rows + 8 up rows (two matrices, {scale,min} tables scales / scales2)
// LAYOUT 2  gate/up  : tile = 16 rows of the reference's element-interleaved pack [I][H][2] (gate, up) with
//                      [I][H/group][2][2] (gate {scale,min}, up {scale,min}); the bytes are split in registers
//                      (16 output rows per stage, 2048 k)
#pragma once

constexpr int GM_MW = 16;  // warps in the tile loop (the first eight also stage the activations); then one producer
                           // warp and one epilogue warp. Sixteen measured faster than eight here: the per-group
                           // {scale, min} loads and folds need more warps in flight to hide
constexpr int GM_ROW_BYTES = 4096;
constexpr int GM_ROW_PITCH = GM_ROW_BYTES + 16;
constexpr int GM_STAGE_BYTES = PIPE_ROWS * GM_ROW_PITCH;

struct GmLayout {
  int x_off;     // activations [NB][Kp + PIPE_XPAD]
  int xsum_off;  // floats [K / group][8]: per-group sums of the staged activations
  int bar_off;   // full[stages], empty[stages], tile_full[2], tile_free[2]
  int red_off;   // floats: stage_x scratch, then 2 x [GM_MW][tile rows][NB] partial tiles
  int abort_off;
  int total;
};
__host__ __device__ inline GmLayout gm_layout(int stages, int nb, int Kp, int ngroups, int out_tile_rows) {
  GmLayout l;
  l.x_off = stages * GM_STAGE_BYTES;
  l.xsum_off = l.x_off + (((nb * (Kp + PIPE_XPAD) * 2) + 15) & ~15);
  l.bar_off = l.xsum_off + ngroups * 8 * 4;
  l.red_off = l.bar_off + (2 * stages + 4) * 8;
  l.abort_off = l.red_off + 2 * GM_MW * out_tile_rows * nb * 4;
  l.total = l.abort_off + 16;
  return l;
}

__device__ __forceinline__ uint32_t gm_lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t gm_ldg32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 gm_ldg64(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// Four interleaved bytes (gate k, up k, gate k+1, up k+1) -> the gate pair and the up pair as 16-bit values
// (unsigned bytes; same mantissa planting as W8Cvt::cvt4).
template <typename T> struct W8Split;
template <> struct W8Split<__half> {
  static __device__ __forceinline__ void run(uint32_t v, uint32_t& gate, uint32_t& up) {
    const uint32_t pg = __byte_perm(v, 0x64646464u, 0x5240);
    const uint32_t pu = __byte_perm(v, 0x64646464u, 0x5341);
    const __half2 b = __floats2half2_rn(1024.f, 1024.f);
    __half2 g = __hsub2(*reinterpret_cast<const __half2*>(&pg), b);
    __half2 u = __hsub2(*reinterpret_cast<const __half2*>(&pu), b);
    gate = *reinterpret_cast<uint32_t*>(&g);
    up = *reinterpret_cast<uint32_t*>(&u);
  }
};
template <> struct W8Split<__nv_bfloat16> {
  static __device__ __forceinline__ void run(uint32_t v, uint32_t& gate, uint32_t& up) {
    const float b = 8388608.f;
    const float f0 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650)) - b;
    const float f1 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7651)) - b;
    const float f2 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7652)) - b;
    const float f3 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7653)) - b;
    gate = Elt<__nv_bfloat16>::pack2(f0, f2);
    up = Elt<__nv_bfloat16>::pack2(f1, f3);
  }
};

// {scale, min} pairs of the two tile rows a thread accumulates (LAYOUT 2: gate pair in .x/.z, up pair in .y/.w)
struct GmScales {
  uint32_t a, b, c, d;
};

template <typename T, int NB, int LAYOUT>
__global__ void __launch_bounds__(32 * (GM_MW + 2)) gemv_pipe_gm_kernel(const GemvArgs a, const int num_stages) {
  constexpr int RPS = (LAYOUT == 1) ? 8 : 16;        // output rows per stage
  constexpr int OUT_TILE = (LAYOUT == 2) ? 32 : 16;  // rows of a warp's partial tile
  constexpr int KCK = (LAYOUT == 2) ? 2048 : 4096;   // k per stage
  constexpr int BPK = (LAYOUT == 2) ? 2 : 1;         // tile bytes per k
  constexpr int STEP_K = (LAYOUT == 2) ? 16 : 32;    // k per ldmatrix.x4
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int K = a.K, Kp = a.Kp, gs = a.group_shift;
  const int gpr = K >> gs;  // groups per row
  const GmLayout lay = gm_layout(num_stages, NB, Kp, gpr, OUT_TILE);
  unsigned char* stage_mem = smem_raw;
  T* x_s = reinterpret_cast<T*>(smem_raw + lay.x_off);
  float* xsum = reinterpret_cast<float*>(smem_raw + lay.xsum_off);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw + lay.bar_off);
  uint64_t* empty_bar = full_bar + num_stages;
  uint64_t* tile_full = empty_bar + num_stages;  // [2] partial tiles of a row block written
  uint64_t* tile_free = tile_full + 2;           // [2] slot drained by the epilogue warp
  float* red = reinterpret_cast<float*>(smem_raw + lay.red_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + lay.abort_off);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, GM_MW);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tile_full + s, GM_MW);
      mbar_init(tile_free + s, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  trace_start(a.trace);
  __syncthreads();
  pdl_launch_dependents();

  const int x_pitch = Kp + PIPE_XPAD;
  const int r_begin = static_cast<int>((long long)a.N * blockIdx.x / gridDim.x);
  const int r_end = static_cast<int>((long long)a.N * (blockIdx.x + 1) / gridDim.x);
  const int nblk = (r_end - r_begin + RPS - 1) / RPS;
  const int nchunks = (K + KCK - 1) / KCK;
  const int total_items = nblk * nchunks;

  if (warp == GM_MW) {
    // ------------------------------ producer warp ------------------------------
    const uint64_t policy = l2_policy_evict_first();
    const unsigned char* __restrict__ W = reinterpret_cast<const unsigned char*>(a.W);
    const unsigned char* __restrict__ W2 = reinterpret_cast<const unsigned char*>(a.W2);
    int issued = 0;
    bool ok = true;
    int blk = 0, kc = 0;
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
      const int rb = r_begin + blk * RPS;
      const int kc_len = min(KCK, K - kc * KCK);
      const uint32_t bytes = static_cast<uint32_t>(kc_len) * BPK;
      const int rows_valid = min(RPS, r_end - rb);
      const int tr = lane;
      const int orow = (LAYOUT == 1) ? (tr & 7) : tr;
      const bool mine = (lane < PIPE_ROWS) && (orow < rows_valid);
      const int ncopies = __popc(__ballot_sync(MUI_FULL_MASK, mine));
      if (lane == 0) mbar_arrive_expect_tx(full_bar + s, static_cast<uint32_t>(ncopies) * bytes);
      __syncwarp();
      if (mine) {
        const unsigned char* src = ((LAYOUT == 1 && tr >= 8) ? W2 : W) +
                                   ((size_t)(rb + orow) * (size_t)K + (size_t)kc * KCK) * BPK;
        bulk_load_1d(stage_mem + (size_t)s * GM_STAGE_BYTES + (size_t)tr * GM_ROW_PITCH, src, bytes, full_bar + s,
                     policy);
      }
      issued = it + 1;
      if (++kc == nchunks) {
        kc = 0;
        ++blk;
      }
    }
    if (ok) pipe_prefetch_next(a, lane);
    if (!ok && lane == 0) {
      const int first = max(0, issued - num_stages);
      for (int it = first; it < issued; ++it) {
        int zero = 0;
        if (!mbar_wait_bounded(full_bar + (it % num_stages), (it / num_stages) & 1, &zero))
          mui_dev_set_status(MUI_DEV_TIMEOUT_DRAIN, it % num_stages);
      }
    }
    return;
  }

  if (warp == GM_MW + 1) {
    // ------------------------------ epilogue warp ------------------------------
    pdl_wait_prior_grid();
    constexpr int OUTS = RPS * NB;
    constexpr int UP_OFF = (LAYOUT == 2) ? 16 : 8;
    for (int blk = 0; blk < nblk; ++blk) {
      const int rb = r_begin + blk * RPS;
      const int slot = blk & 1;
      if (!mbar_wait_bounded(tile_full + slot, (blk >> 1) & 1, abort_flag)) {
        if (lane == 0 && !*abort_flag) {
          mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, 64 + slot);
          *abort_flag = 1;
        }
        break;
      }
      const float* rbuf = red + slot * (GM_MW * OUT_TILE * NB);
      for (int o = lane; o < OUTS; o += 32) {
        const int r = o / NB, b = o - r * NB, row = rb + r;
        if (row < r_end && b < a.B) {
          float v = 0.f, u = 0.f;
#pragma unroll
          for (int w = 0; w < GM_MW; ++w) {
            v += rbuf[(w * OUT_TILE + r) * NB + b];
            if (LAYOUT != 0) u += rbuf[(w * OUT_TILE + UP_OFF + r) * NB + b];
          }
          if (LAYOUT == 0) gemv_store_linear<T>(a, b, row, v);
          else gemv_store_gateup<T>(a, b, row, a.N, v, u, 1.f);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(tile_free + slot);
    }
    if (lane == 0) trace_end(a.trace);
    return;
  }

  // ------------------------------ math warps ------------------------------
  const bool stager = warp < GEMV_CONSUMER_WARPS;
  GemvNormPre norm_pre;
  norm_pre.have = false;
  if (stager) gemv_prefetch_norm<T, NB>(a, tid, norm_pre);
  pdl_wait_prior_grid();
  if (tid == 0) trace_mark(a.trace, 2, false);
  if (stager) {
    gemv_stage_x<T, NB>(a, a.B, x_s, x_pitch, red, tid, &norm_pre);
    // per-group sums of the staged (normalised, rounded) activations: four lanes per (group, row)
    const int ntasks = gpr * 8;
    const int part = tid & 3, per_part = (1 << gs) >> 2;
    for (int t0 = 0; t0 < ntasks; t0 += GEMV_CONSUMER_THREADS / 4) {
      const int t = t0 + (tid >> 2);
      const int g = t >> 3, b = t & 7;
      float s = 0.f;
      if (t < ntasks && b < NB) {
        const T* src = x_s + (size_t)b * x_pitch + ((size_t)g << gs) + part * per_part;
        for (int i = 0; i < per_part; i += 8) {
          float f[8];
          unpack8<T>(*reinterpret_cast<const uint4*>(src + i), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) s += f[j];
        }
      }
      s += __shfl_xor_sync(MUI_FULL_MASK, s, 1);
      s += __shfl_xor_sync(MUI_FULL_MASK, s, 2);
      if (t < ntasks && part == 0) xsum[t] = s;
    }
  }
  named_bar_sync(2, GM_MW * 32);  // staged activations and group sums visible to all math warps
  if (tid == 0) trace_mark(a.trace, 3, true);

  float d[4] = {0.f, 0.f, 0.f, 0.f};   // LAYOUT 0/1: the tile; LAYOUT 2: gate
  float du[4] = {0.f, 0.f, 0.f, 0.f};  // LAYOUT 2: up
  const int trow = lane >> 2, n0 = (lane & 3) * 2;
  const uint32_t a_lane_off = static_cast<uint32_t>(((lane & 7) + ((lane >> 3) & 1) * 8) * GM_ROW_PITCH +
                                                    (lane >> 4) * 16);
  const int n_row = (trow < NB) ? trow : (NB - 1);
  const uint32_t stage_base = smem_u32(stage_mem);
  const uint32_t x_lane = smem_u32(x_s + (size_t)n_row * x_pitch + (lane & 3) * (LAYOUT == 2 ? 2 : 4));
  const int spg = (1 << gs) / STEP_K;      // ldmatrix steps per group (a power of two)
  const int gpc_full = KCK >> gs;          // groups per full stage
  const unsigned char* __restrict__ SM1 = reinterpret_cast<const unsigned char*>(a.scales);
  const unsigned char* __restrict__ SM2 = reinterpret_cast<const unsigned char*>(a.scales2);

  // {scale,min} of group G (index along the row) for this thread's two tile rows of row block rb
  auto load_scales = [&](int rb, int G) {
    GmScales r;
    const int ra = min(rb + trow, r_end - 1), rbw = min(rb + trow + 8, r_end - 1);
    if (LAYOUT == 0) {
      r.a = gm_ldg32(SM1 + ((size_t)ra * gpr + G) * 4);
      r.b = gm_ldg32(SM1 + ((size_t)rbw * gpr + G) * 4);
      r.c = r.d = 0;
    } else if (LAYOUT == 1) {
      r.a = gm_ldg32(SM1 + ((size_t)ra * gpr + G) * 4);
      r.b = gm_ldg32(SM2 + ((size_t)ra * gpr + G) * 4);
      r.c = r.d = 0;
    } else {
      const uint2 p = gm_ldg64(SM1 + ((size_t)ra * gpr + G) * 8);
      const uint2 q = gm_ldg64(SM1 + ((size_t)rbw * gpr + G) * 8);
      r.a = p.x;  // gate {scale,min}, row trow
      r.c = p.y;  // up
      r.b = q.x;  // gate, row trow + 8
      r.d = q.y;  // up
    }
    return r;
  };

  int blk = 0, kc = 0;
  int s = -1;         // ring slot and its phase bit, advanced without divisions
  uint32_t ph = 1;
  for (int it = 0; it < total_items; ++it) {
    if (++s == num_stages) s = 0;
    if (s == 0) ph ^= 1u;
    const int rb = r_begin + blk * RPS;
    const int kc_len = min(KCK, K - kc * KCK);
    const int gpc = kc_len >> gs;  // groups in this stage
    const int g_base = kc * gpc_full;
    GmScales cur = {0u, 0u, 0u, 0u};
    if (warp < gpc) cur = load_scales(rb, g_base + warp);  // in flight across the wait below
    if (!mbar_wait_bounded(full_bar + s, ph, abort_flag)) {
      if (lane == 0 && !*abort_flag) {
        mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, s);
        *abort_flag = 1;
      }
      break;
    }
    const uint32_t a_addr = stage_base + static_cast<uint32_t>(s) * GM_STAGE_BYTES + a_lane_off;
    const uint32_t x_addr = x_lane + static_cast<uint32_t>(kc * KCK * 2);
    for (int g = warp; g < gpc; g += GM_MW) {
      GmScales nxt = cur;
      if (g + GM_MW < gpc) nxt = load_scales(rb, g_base + g + GM_MW);
      float t[4] = {0.f, 0.f, 0.f, 0.f}, t2[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t ag = a_addr + static_cast<uint32_t>(g * spg) * 32;
      const uint32_t xg = x_addr + static_cast<uint32_t>(g * spg) * (STEP_K * 2);
      const float2 X = *reinterpret_cast<const float2*>(xsum + (size_t)(g_base + g) * 8 + n0);
      const float2 sa = Elt<T>::unpack2(cur.a), sb = Elt<T>::unpack2(cur.b);
      if (LAYOUT != 2) {
#pragma unroll 4
        for (int j = 0; j < spg; ++j) {
          uint32_t r[4];
          ldmatrix_x4(r, ag + j * 32);
          uint32_t xa0, xa1, xb0, xb1;
          lds_v2(xg + j * 64, xa0, xa1);
          lds_v2(xg + j * 64 + 32, xb0, xb1);
          uint32_t af[4], bf[4];
          W8Cvt<T>::template cvt4<false>(r[0], af[0], af[2]);
          W8Cvt<T>::template cvt4<false>(r[1], af[1], af[3]);
          W8Cvt<T>::template cvt4<false>(r[2], bf[0], bf[2]);
          W8Cvt<T>::template cvt4<false>(r[3], bf[1], bf[3]);
          MmaOp<T>::run(t, af, xa0, xa1);
          MmaOp<T>::run(t2, bf, xb0, xb1);
        }
        d[0] += sa.x * (t[0] + t2[0]) + sa.y * X.x;
        d[1] += sa.x * (t[1] + t2[1]) + sa.y * X.y;
        d[2] += sb.x * (t[2] + t2[2]) + sb.y * X.x;
        d[3] += sb.x * (t[3] + t2[3]) + sb.y * X.y;
      } else {
#pragma unroll 4
        for (int j = 0; j < spg; ++j) {
          uint32_t r[4];
          ldmatrix_x4(r, ag + j * 32);
          const uint32_t b0 = gm_lds32(xg + j * 32), b1 = gm_lds32(xg + j * 32 + 16);
          uint32_t gf[4], uf[4];
          W8Split<T>::run(r[0], gf[0], uf[0]);
          W8Split<T>::run(r[1], gf[1], uf[1]);
          W8Split<T>::run(r[2], gf[2], uf[2]);
          W8Split<T>::run(r[3], gf[3], uf[3]);
          MmaOp<T>::run(t, gf, b0, b1);
          MmaOp<T>::run(t2, uf, b0, b1);
        }
        const float2 ua = Elt<T>::unpack2(cur.c), ub = Elt<T>::unpack2(cur.d);
        d[0] += sa.x * t[0] + sa.y * X.x;
        d[1] += sa.x * t[1] + sa.y * X.y;
        d[2] += sb.x * t[2] + sb.y * X.x;
        d[3] += sb.x * t[3] + sb.y * X.y;
        du[0] += ua.x * t2[0] + ua.y * X.x;
        du[1] += ua.x * t2[1] + ua.y * X.y;
        du[2] += ub.x * t2[2] + ub.y * X.x;
        du[3] += ub.x * t2[3] + ub.y * X.y;
      }
      cur = nxt;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar + s);

    if (++kc == nchunks) {
      // row block complete: the warps' partial tiles are summed in a fixed order
      kc = 0;
      const int slot = blk & 1;
      if (blk >= 2) {
        // the slot's previous tiles (row block blk - 2) must have been drained by the epilogue warp
        if (!mbar_wait_bounded(tile_free + slot, ((blk >> 1) - 1) & 1, abort_flag)) {
          if (lane == 0 && !*abort_flag) {
            mui_dev_set_status(MUI_DEV_TIMEOUT_EMPTY, 64 + slot);
            *abort_flag = 1;
          }
          break;
        }
      }
      float* rbuf = red + slot * (GM_MW * OUT_TILE * NB);
      if (n0 < NB) {
        rbuf[(warp * OUT_TILE + trow) * NB + n0] = d[0];
        rbuf[(warp * OUT_TILE + trow + 8) * NB + n0] = d[2];
        if (LAYOUT == 2) {
          rbuf[(warp * OUT_TILE + 16 + trow) * NB + n0] = du[0];
          rbuf[(warp * OUT_TILE + 24 + trow) * NB + n0] = du[2];
        }
      }
      if (n0 + 1 < NB) {
        rbuf[(warp * OUT_TILE + trow) * NB + n0 + 1] = d[1];
        rbuf[(warp * OUT_TILE + trow + 8) * NB + n0 + 1] = d[3];
        if (LAYOUT == 2) {
          rbuf[(warp * OUT_TILE + 16 + trow) * NB + n0 + 1] = du[1];
          rbuf[(warp * OUT_TILE + 24 + trow) * NB + n0 + 1] = du[3];
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) d[q] = du[q] = 0.f;
      __syncwarp();
      if (lane == 0) mbar_arrive(tile_full + slot);  // release: the tile stores above are visible to the waiter
      ++blk;
    }
  }
}

