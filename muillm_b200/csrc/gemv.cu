// GEMV-shaped kernels on 16-bit weights for one to eight activation rows:
//   MODE 0  linear      y = act(W xn) * mul_bias + add_bias + residual
//   MODE 1  gate/up     t = silu(G xn) * (U xn)
// plus MoE addressing of either (device-side expert selection).
//
// Two implementations of the same math:
//  * gemv_pipe_kernel    — persistent CTAs (two per SM). One producer warp streams 16 row chunks of
//                          512 elements per stage into a shared-memory ring with 1-D bulk async copies
//                          (TMA) completing on mbarriers; eight consumer warps each own two row
//                          streams, multiply against the activations staged in shared memory and
//                          finish their rows with warp shuffles — no cross-warp reduction. The weight
//                          prefetch does not depend on the previous kernel, so under programmatic
//                          dependent launch it overlaps that kernel's tail.
//  * gemv_generic_kernel — plain 16-byte streaming loads, the 256 threads of a CTA split K, cross-warp
//                          reduction in shared memory. Covers any K / alignment.
//
// HBM traffic per call: N*K*2 (weights, read once) + activations; fp32 accumulation.
#include "gemv_common.cuh"

#include <algorithm>

MUI_STATUS_ACCESSOR(gemv)

namespace {

// =============================================================================================
// generic kernel
// =============================================================================================
template <typename T, int NB, int MODE>
__global__ void __launch_bounds__(GEMV_CONSUMER_THREADS) gemv_generic_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* x_s = reinterpret_cast<T*>(smem_raw);
  __shared__ float red[GEMV_CONSUMER_WARPS * 2 * NB];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  pdl_wait_prior_grid();
  pdl_launch_dependents();

  const int nseg = (a.moe_mode == GEMV_MOE_SEGMENTS) ? a.slots : 1;
  const int total_rows = (a.moe_mode == GEMV_MOE_ROWS) ? a.slots * a.N : a.N;
  if (a.moe_mode == GEMV_MOE_SEGMENTS)
    gemv_stage_x_plain<T>(a, a.slots, x_s, tid);
  else
    gemv_stage_x<T, NB>(a, a.B, x_s, red, tid);

  const int K = a.K, Kp = a.Kp;
  const T* __restrict__ W = reinterpret_cast<const T*>(a.W);
  const T* __restrict__ W2 = reinterpret_cast<const T*>(a.W2);
  const bool vec_ok = ((K & 7) == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) &&
                      (MODE == 0 || (reinterpret_cast<uintptr_t>(W2) & 15) == 0);

  const int num_items = (MODE == 0) ? (total_rows + 1) / 2 : total_rows;
  for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
    const int ra = (MODE == 0) ? 2 * item : item;
    const bool second_valid = (MODE == 0) ? (ra + 1 < total_rows) : true;
    const int rb = (MODE == 0) ? (second_valid ? ra + 1 : ra) : ra;

    float acc[2][NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[0][b] = acc[1][b] = 0.f;

    for (int seg = 0; seg < nseg; ++seg) {
      const T* __restrict__ wa = W + gemv_weight_row(a, ra, seg) * (size_t)K;
      const T* __restrict__ wb = ((MODE == 0) ? W : W2) + gemv_weight_row(a, rb, seg) * (size_t)K;
      const T* xs = x_s + (size_t)seg * Kp;
      if (vec_ok) {
#pragma unroll 2
        for (int k = tid * 8; k < K; k += GEMV_CONSUMER_THREADS * 8) {
          const uint4 va = ld_stream16(wa + k);
          const uint4 vb = ld_stream16(wb + k);
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float f[8];
            unpack8<T>(*reinterpret_cast<const uint4*>(xs + (size_t)b * Kp + k), f);
            acc[0][b] = dot8<T>(va, f, acc[0][b]);
            acc[1][b] = dot8<T>(vb, f, acc[1][b]);
          }
        }
      } else {
        for (int k = tid; k < K; k += GEMV_CONSUMER_THREADS) {
          const float fa = Elt<T>::to_f32(wa[k]);
          const float fb = Elt<T>::to_f32(wb[k]);
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
        if (b < a.B && (j == 0 || second_valid)) gemv_store_linear<T>(a, b, j == 0 ? ra : rb, s);
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
}

// =============================================================================================
// bulk-copy pipeline kernel
// =============================================================================================
constexpr int PIPE_KC = 512;                                // elements per row chunk
constexpr int PIPE_SLOTS = 16;                              // row chunks per stage (8 warps x 2 streams)
constexpr int PIPE_STAGE_BYTES = PIPE_SLOTS * PIPE_KC * 2;  // 16 KiB
constexpr int PIPE_THREADS = GEMV_CONSUMER_THREADS + 32;
constexpr int PIPE_MAX_STAGES = 8;

struct PipeLayout {
  int stages;
  int x_off;      // activations
  int bar_off;    // full[stages], empty[stages]
  int red_off;    // floats
  int abort_off;  // int
  int total;
};
__host__ __device__ inline PipeLayout pipe_layout(int stages, int x_rows, int Kp, int nb) {
  PipeLayout l;
  l.stages = stages;
  l.x_off = stages * PIPE_STAGE_BYTES;
  int x_bytes = ((x_rows * Kp * 2) + 15) & ~15;
  l.bar_off = l.x_off + x_bytes;
  l.red_off = l.bar_off + 2 * stages * 8;
  l.abort_off = l.red_off + nb * GEMV_CONSUMER_WARPS * 4;
  l.total = l.abort_off + 16;
  return l;
}

template <typename T, int NB, int MODE>
__global__ void __launch_bounds__(PIPE_THREADS) gemv_pipe_kernel(const GemvArgs a, const int num_stages) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int x_rows = (a.moe_mode == GEMV_MOE_SEGMENTS) ? a.slots : NB;
  const PipeLayout lay = pipe_layout(num_stages, x_rows, a.Kp, NB);
  unsigned char* stage_mem = smem_raw;
  T* x_s = reinterpret_cast<T*>(smem_raw + lay.x_off);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw + lay.bar_off);
  uint64_t* empty_bar = full_bar + num_stages;
  float* red = reinterpret_cast<float*>(smem_raw + lay.red_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + lay.abort_off);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, GEMV_CONSUMER_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  constexpr int ROWS_PER_STAGE = (MODE == 0) ? 16 : 8;
  const int K = a.K, Kp = a.Kp;
  const int nseg = (a.moe_mode == GEMV_MOE_SEGMENTS) ? a.slots : 1;
  const int total_rows = (a.moe_mode == GEMV_MOE_ROWS) ? a.slots * a.N : a.N;
  const int r_begin = static_cast<int>((long long)total_rows * blockIdx.x / gridDim.x);
  const int r_end = static_cast<int>((long long)total_rows * (blockIdx.x + 1) / gridDim.x);
  const int nblk = (r_end - r_begin + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE;
  const int nchunks = (K + PIPE_KC - 1) / PIPE_KC;
  const int cpb = nseg * nchunks;  // stage items per row block
  const int total_items = nblk * cpb;

  if (warp == GEMV_CONSUMER_WARPS) {
    // ------------------------------ producer warp ------------------------------
    if (a.moe_mode != GEMV_MOE_NONE) pdl_wait_prior_grid();  // expert ids come from the previous kernel
    const uint64_t policy = l2_policy_evict_first();
    const T* __restrict__ W = reinterpret_cast<const T*>(a.W);
    const T* __restrict__ W2 = reinterpret_cast<const T*>(a.W2);
    int issued = 0;
    bool ok = true;
    for (int it = 0; it < total_items; ++it) {
      const int s = it % num_stages;
      const uint32_t ph = (it / num_stages) & 1;
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
      const int blk = it / cpb, c = it - blk * cpb;
      const int seg = c / nchunks, kc = c - seg * nchunks;
      const int rb = r_begin + blk * ROWS_PER_STAGE;
      const int kc_len = min(PIPE_KC, K - kc * PIPE_KC);
      const uint32_t bytes = static_cast<uint32_t>(kc_len) * 2u;
      const int rows_valid = min(ROWS_PER_STAGE, r_end - rb);
      const int ncopies = (MODE == 0) ? rows_valid : 2 * rows_valid;
      if (lane == 0) mbar_arrive_expect_tx(full_bar + s, static_cast<uint32_t>(ncopies) * bytes);
      __syncwarp();
      if (lane < PIPE_SLOTS) {
        const int j = lane & 1, w = lane >> 1;
        const int row = (MODE == 0) ? rb + lane : rb + w;
        const bool valid = (MODE == 0) ? (lane < rows_valid) : (w < rows_valid);
        if (valid) {
          const T* src = ((MODE == 1 && j == 1) ? W2 : W) + gemv_weight_row(a, row, seg) * (size_t)K +
                         (size_t)kc * PIPE_KC;
          bulk_load_1d(stage_mem + (size_t)s * PIPE_STAGE_BYTES + (size_t)lane * (PIPE_KC * 2), src, bytes,
                       full_bar + s, policy);
        }
      }
      issued = it + 1;
    }
    if (!ok && lane == 0) {
      // leave no copy in flight behind: wait (bounded) for every stage that was armed
      const int first = max(0, issued - num_stages);
      for (int it = first; it < issued; ++it) {
        int zero = 0;
        if (!mbar_wait_bounded(full_bar + (it % num_stages), (it / num_stages) & 1, &zero))
          mui_dev_set_status(MUI_DEV_TIMEOUT_DRAIN, it % num_stages);
      }
    }
  } else {
    // ------------------------------ consumer warps ------------------------------
    pdl_wait_prior_grid();
    if (a.moe_mode == GEMV_MOE_SEGMENTS)
      gemv_stage_x_plain<T>(a, a.slots, x_s, tid);
    else
      gemv_stage_x<T, NB>(a, a.B, x_s, red, tid);

    float acc[2][NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[0][b] = acc[1][b] = 0.f;

    for (int it = 0; it < total_items; ++it) {
      const int s = it % num_stages;
      const uint32_t ph = (it / num_stages) & 1;
      if (!mbar_wait_bounded(full_bar + s, ph, abort_flag)) {
        if (lane == 0 && !*abort_flag) {
          mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, s);
          *abort_flag = 1;
        }
        break;
      }
      const int blk = it / cpb, c = it - blk * cpb;
      const int seg = c / nchunks, kc = c - seg * nchunks;
      const int rb = r_begin + blk * ROWS_PER_STAGE;
      const int kc_len = min(PIPE_KC, K - kc * PIPE_KC);
      const int row0 = (MODE == 0) ? rb + warp * 2 : rb + warp;
      const bool valid0 = row0 < r_end;
      const bool valid1 = (MODE == 0) ? (row0 + 1 < r_end) : valid0;

      if (valid0) {
        const T* ws0 = reinterpret_cast<const T*>(stage_mem + (size_t)s * PIPE_STAGE_BYTES) +
                       (size_t)(warp * 2) * PIPE_KC;
        const T* ws1 = ws0 + PIPE_KC;
        const T* xs = x_s + (size_t)seg * Kp + (size_t)kc * PIPE_KC;
#pragma unroll
        for (int k = lane * 8; k < PIPE_KC; k += 256) {
          if (k < kc_len) {
            const uint4 v0 = *reinterpret_cast<const uint4*>(ws0 + k);
            const uint4 v1 = valid1 ? *reinterpret_cast<const uint4*>(ws1 + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              float f[8];
              unpack8<T>(*reinterpret_cast<const uint4*>(xs + (size_t)b * Kp + k), f);
              acc[0][b] = dot8<T>(v0, f, acc[0][b]);
              acc[1][b] = dot8<T>(v1, f, acc[1][b]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar + s);

      if (c == cpb - 1) {
        // rows of this block are complete: finish them inside the warp
        if (MODE == 0) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              const float v = warp_sum(acc[j][b]);
              const bool valid = (j == 0) ? valid0 : valid1;
              if (lane == j * NB + b && valid && b < a.B) gemv_store_linear<T>(a, b, row0 + j, v);
            }
        } else {
          float score = 1.f;
          if (a.moe_mode == GEMV_MOE_ROWS && valid0) score = gemv_slot_score<T>(a, row0 / a.N);
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            const float g = warp_sum(acc[0][b]);
            const float u = warp_sum(acc[1][b]);
            if (lane == b && valid0 && b < a.B) gemv_store_gateup<T>(a, b, row0, total_rows, g, u, score);
          }
        }
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[0][b] = acc[1][b] = 0.f;
      }
    }
  }
}

// =============================================================================================
// host dispatch
// =============================================================================================
template <typename T, int NB, int MODE>
mui_status_t launch_gemv_t(cudaStream_t stream, const GemvArgs& a, unsigned flags, const MuiDeviceInfo* dev) {
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  const int total_rows = (a.moe_mode == GEMV_MOE_ROWS) ? a.slots * a.N : a.N;
  const int x_rows = (a.moe_mode == GEMV_MOE_SEGMENTS) ? a.slots : NB;
  const size_t x_bytes = (size_t)x_rows * a.Kp * 2;

  const bool aligned = ((a.K & 7) == 0) && ((reinterpret_cast<uintptr_t>(a.W) & 15) == 0) &&
                       (MODE == 0 || (reinterpret_cast<uintptr_t>(a.W2) & 15) == 0);
  bool use_pipe = aligned && !(flags & MUI_FLAG_FORCE_GENERIC);
  int stages = 0, ctas_per_sm = 2;
  if (use_pipe) {
    // two CTAs per SM when the activations are small enough to leave room for >= 3 stages each
    const int budget2 = 110 * 1024, budget1 = 220 * 1024;
    const int fixed = pipe_layout(0, x_rows, a.Kp, NB).total;
    stages = (budget2 - fixed) / PIPE_STAGE_BYTES;
    if (stages < 3) {
      ctas_per_sm = 1;
      stages = (budget1 - fixed) / PIPE_STAGE_BYTES;
    }
    stages = std::min(stages, PIPE_MAX_STAGES);
    if (stages < 2) use_pipe = false;
  }
  if (!use_pipe && (flags & MUI_FLAG_FORCE_PIPELINE)) {
    mui_set_error("bulk-copy pipeline not applicable (K=%d, alignment or activation size)", a.K);
    return MUI_ERR_UNSUPPORTED;
  }

  if (use_pipe) {
    auto kern = gemv_pipe_kernel<T, NB, MODE>;
    const PipeLayout lay = pipe_layout(stages, x_rows, a.Kp, NB);
    static int configured_smem = 0;  // per instantiation
    if (lay.total > configured_smem) {
      MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 222 * 1024));
      MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
      configured_smem = 222 * 1024;
    }
    const int grid = std::max(1, std::min(total_rows, dev->sm_count * ctas_per_sm));
    MUI_CUDA_CHECK(mui_launch(kern, dim3(grid), dim3(PIPE_THREADS), (size_t)lay.total, stream, pdl, a, stages));
    return MUI_OK;
  }

  // generic
  MUI_REQUIRE(x_bytes <= 200 * 1024, MUI_ERR_UNSUPPORTED,
              "activations (%zu bytes) do not fit the shared-memory staging of the GEMV", x_bytes);
  auto kern = gemv_generic_kernel<T, NB, MODE>;
  static int configured_smem_g = 0;
  if ((int)x_bytes > 48 * 1024 && (int)x_bytes > configured_smem_g) {
    MUI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured_smem_g = 200 * 1024;
  }
  const int num_items = (MODE == 0) ? (total_rows + 1) / 2 : total_rows;
  int per_sm = (int)std::min<size_t>(8, (size_t)(224 * 1024) / (x_bytes + 2048));
  per_sm = std::max(per_sm, 1);
  const int grid = std::max(1, std::min(num_items, dev->sm_count * per_sm));
  MUI_CUDA_CHECK(mui_launch(kern, dim3(grid), dim3(GEMV_CONSUMER_THREADS), x_bytes, stream, pdl, a));
  return MUI_OK;
}

template <typename T, int MODE>
mui_status_t launch_gemv_nb(cudaStream_t stream, const GemvArgs& a, int nb, unsigned flags, const MuiDeviceInfo* dev) {
  switch (nb) {
    case 1: return launch_gemv_t<T, 1, MODE>(stream, a, flags, dev);
    case 2: return launch_gemv_t<T, 2, MODE>(stream, a, flags, dev);
    case 4: return launch_gemv_t<T, 4, MODE>(stream, a, flags, dev);
    default: return launch_gemv_t<T, 8, MODE>(stream, a, flags, dev);
  }
}

}  // namespace

// Launches MODE 0 (linear) or MODE 1 (gate/up) on validated arguments.
mui_status_t mui_launch_gemv16(cudaStream_t stream, mui_dtype_t dtype, int mode, const GemvArgs& a, unsigned flags) {
  const MuiDeviceInfo* dev = mui_current_device_info();
  if (!dev) return MUI_ERR_CUDA;
  const int nb = a.B <= 1 ? 1 : (a.B <= 2 ? 2 : (a.B <= 4 ? 4 : 8));
  if (dtype == MUI_F16) {
    return mode == 0 ? launch_gemv_nb<__half, 0>(stream, a, nb, flags, dev)
                     : launch_gemv_nb<__half, 1>(stream, a, nb, flags, dev);
  } else {
    return mode == 0 ? launch_gemv_nb<__nv_bfloat16, 0>(stream, a, nb, flags, dev)
                     : launch_gemv_nb<__nv_bfloat16, 1>(stream, a, nb, flags, dev);
  }
}
