// Batched variant of the bulk-copy pipeline GEMV (2 to 8 activation rows): the activations are staged in shared
// memory ONE K-CHUNK AT A TIME instead of whole, so that the weight ring keeps (nearly) all of the SM's shared memory
// whatever B*K is. With whole-row staging, 8 rows of K = 14336 do not fit at all (the batch then ran as two passes
// over the weights) and 8 rows of K = 8192 leave room for two small stages only.
//
// Loop order: for each chunk of 2048 activations, for each 16-row block of this CTA's rows. Every consumer thread
// keeps the fp32 accumulators of up to XC_MAX_BLOCKS row blocks in registers across the chunks (a CTA with more row
// blocks runs them in groups; the activations are then re-read from L2, never the weights). The weights are still
// read exactly once, in row chunks of 4 KiB (16-bit) or 2 KiB (8-bit), through the same mbarrier ring. The next
// chunk of activations is loaded into registers while the current one is being multiplied, normalised (fused RMSNorm
// with the HF roundings, from per-row rstd values computed up front) when it is stored to shared memory.
// Included by gemv_kernels.cuh inside its unnamed namespace.
#pragma once

constexpr int XC_KC = 2048;        // activation chunk (elements) = weights per row chunk
constexpr int XC_MAX_BLOCKS = 16;  // row blocks whose accumulators a consumer thread holds at a time

template <int WB> struct XcGeom {
  static constexpr int ROW_PITCH = XC_KC * (WB / 8) + 16;    // bytes
  static constexpr int STAGE_BYTES = PIPE_ROWS * ROW_PITCH;  // bytes
};

struct XcLayout {
  int x_off;     // activations of one chunk [NB][XC_KC + PIPE_XPAD]; reused for the partial tiles at the end
  int bar_off;   // full[stages], empty[stages]
  int misc_off;  // floats: rstd[NB], reduction scratch [NB][8 warps]
  int abort_off;
  int total;
};
__host__ __device__ inline XcLayout xc_layout(int stage_bytes, int stages, int nb) {
  XcLayout l;
  l.x_off = stages * stage_bytes;
  l.bar_off = l.x_off + nb * (XC_KC + PIPE_XPAD) * 2;
  l.misc_off = l.bar_off + 2 * stages * 8;
  l.abort_off = l.misc_off + (nb + nb * GEMV_CONSUMER_WARPS) * 4;
  l.total = l.abort_off + 16;
  return l;
}

// L2 prefetch of the weights that follow on the stream (GemvArgs::pf_*): the head of the row range this CTA index
// owns in the kernel that will consume each hinted matrix, 8 KiB per request. Called by one warp.
__device__ __forceinline__ void pipe_prefetch_next(const GemvArgs& a, int lane) {
#pragma unroll
  for (int sgm = 0; sgm < 3; ++sgm) {
    if (a.pf_ptr[sgm] == nullptr || a.pf_frac[sgm] <= 0) continue;
    const long long rows = a.pf_rows[sgm], rbytes = a.pf_row_bytes[sgm];
    const long long pr0 = rows * blockIdx.x / gridDim.x, pr1 = rows * (blockIdx.x + 1) / gridDim.x;
    const long long total = (pr1 - pr0) * rbytes;
    const long long skip = min(static_cast<long long>(a.pf_skip[sgm]) & ~15ll, total);
    const long long b0 = pr0 * rbytes + skip;
    const long long nb = min((total * a.pf_frac[sgm] / 1024) & ~15ll, total - skip);
    const unsigned char* base = reinterpret_cast<const unsigned char*>(a.pf_ptr[sgm]) + b0;
    for (long long off = (long long)lane * 8192; off < nb; off += 32 * 8192)
      bulk_prefetch_l2(base + off, static_cast<uint32_t>(min(8192ll, nb - off)));
  }
}

template <typename T, int NB, int MODE, int WB>
__global__ void __launch_bounds__(GEMV_CONSUMER_THREADS + 32) gemv_pipe_xchunk_kernel(const GemvArgs a,
                                                                                     const int num_stages) {
  using G = XcGeom<WB>;
  constexpr int EB = WB / 8;
  constexpr int KC = XC_KC;
  constexpr int X_PITCH = KC + PIPE_XPAD;  // elements
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const XcLayout lay = xc_layout(G::STAGE_BYTES, num_stages, NB);
  unsigned char* stage_mem = smem_raw;
  T* x_s = reinterpret_cast<T*>(smem_raw + lay.x_off);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw + lay.bar_off);
  uint64_t* empty_bar = full_bar + num_stages;
  float* rstd_s = reinterpret_cast<float*>(smem_raw + lay.misc_off);
  float* red_s = rstd_s + NB;
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
  trace_start(a.trace);
  __syncthreads();
  pdl_launch_dependents();

  constexpr int ROWS_PER_STAGE = (MODE == 0) ? 16 : 8;  // output rows per stage
  const int K = a.K;
  const int total_rows = a.N;
  const int r_begin = static_cast<int>((long long)total_rows * blockIdx.x / gridDim.x);
  const int r_end = static_cast<int>((long long)total_rows * (blockIdx.x + 1) / gridDim.x);
  const int nblk = (r_end - r_begin + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE;
  const int nchunks = (K + KC - 1) / KC;
  const int ngroups = (nblk + XC_MAX_BLOCKS - 1) / XC_MAX_BLOCKS;

  if (warp >= GEMV_CONSUMER_WARPS) {
    // ------------------------------ producer warp ------------------------------
    const uint64_t policy = l2_policy_evict_first();
    const unsigned char* __restrict__ W = reinterpret_cast<const unsigned char*>(a.W);
    const unsigned char* __restrict__ W2 = reinterpret_cast<const unsigned char*>(a.W2);
    int it = 0;
    bool ok = true;
    for (int gidx = 0; gidx < ngroups && ok; ++gidx) {
      const int blk0 = gidx * XC_MAX_BLOCKS;
      const int nb_g = min(XC_MAX_BLOCKS, nblk - blk0);
      for (int kc = 0; kc < nchunks && ok; ++kc) {
        const int kc_len = min(KC, K - kc * KC);
        const uint32_t bytes = static_cast<uint32_t>(kc_len) * EB;
        for (int bi = 0; bi < nb_g; ++bi, ++it) {
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
          const int rb = r_begin + (blk0 + bi) * ROWS_PER_STAGE;
          const int rows_valid = min(ROWS_PER_STAGE, r_end - rb);
          // tile row tr: MODE 0 -> output row rb + tr; MODE 1 -> gate (tr < 8) / up (tr >= 8) row rb + tr % 8
          const int tr = lane;
          const int orow = (MODE == 0) ? tr : (tr & 7);
          const bool mine = (lane < PIPE_ROWS) && (orow < rows_valid);
          const int ncopies = __popc(__ballot_sync(MUI_FULL_MASK, mine));
          if (lane == 0) mbar_arrive_expect_tx(full_bar + s, static_cast<uint32_t>(ncopies) * bytes);
          __syncwarp();
          if (mine) {
            const unsigned char* src = ((MODE == 1 && tr >= 8) ? W2 : W) +
                                       ((size_t)(rb + orow) * (size_t)K + (size_t)kc * KC) * EB;
            bulk_load_1d(stage_mem + (size_t)s * G::STAGE_BYTES + (size_t)tr * G::ROW_PITCH, src, bytes,
                         full_bar + s, policy);
          }
        }
      }
    }
    if (ok) pipe_prefetch_next(a, lane);
    if (!ok && lane == 0) {
      // leave no copy in flight behind: wait (bounded) for every stage that was armed
      const int first = max(0, it - num_stages);
      for (int i = first; i < it; ++i) {
        int zero = 0;
        if (!mbar_wait_bounded(full_bar + (i % num_stages), (i / num_stages) & 1, &zero))
          mui_dev_set_status(MUI_DEV_TIMEOUT_DRAIN, i % num_stages);
      }
    }
    return;
  }

  // ------------------------------ consumer warps ------------------------------
  pdl_wait_prior_grid();
  if (tid == 0) trace_mark(a.trace, 2, false);
  const unsigned long long comm_seq = (MODE == 0 && a.use_comm) ? comm_begin(a.comm) : 0ull;
  const T* __restrict__ x = reinterpret_cast<const T*>(a.x);
  const T* __restrict__ nw = reinterpret_cast<const T*>(a.norm_w);
  const bool do_norm = nw != nullptr;

  // per-row rstd of the fused RMSNorm: one pass over the activations (L2), thread t owns columns 8t..8t+7 of every
  // chunk — the same columns it stages below
  if (do_norm) {
    float ss[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) ss[b] = 0.f;
    for (int kc = 0; kc < nchunks; ++kc) {
      const int k = kc * KC + tid * 8;
      if (k < K) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          if (b < a.B) {
            float f[8];
            unpack8<T>(ld_act16(x + (size_t)b * K + k), f);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss[b] = fmaf(f[i], f[i], ss[b]);
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const float s = warp_sum(ss[b]);
      if (lane == 0) red_s[b * GEMV_CONSUMER_WARPS + warp] = s;
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
    if (tid < NB) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) s += red_s[tid * GEMV_CONSUMER_WARPS + w];
      rstd_s[tid] = rsqrtf(s / static_cast<float>(K) + a.eps);
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
  }
  float rstd[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) rstd[b] = do_norm ? rstd_s[b] : 1.f;

  // ldmatrix sources (see gemv_pipe_kernel): A = weight tile of the stage, B = the staged chunk of activations
  const uint32_t a_lane_off = static_cast<uint32_t>(((lane & 7) + ((lane >> 3) & 1) * 8) * G::ROW_PITCH +
                                                    (lane >> 4) * 16);
  const int b_row = ((lane & 7) < NB) ? (lane & 7) : (NB - 1);
  const uint32_t b_lane_off = static_cast<uint32_t>((b_row * X_PITCH + ((lane >> 3) & 1) * 8) * 2);
  const uint32_t stage_base = smem_u32(stage_mem);
  const uint32_t x_base = smem_u32(x_s);
  const int n_row8 = ((lane >> 2) < NB) ? (lane >> 2) : (NB - 1);  // 8-bit path: batch row of this lane's B fragment
  const uint32_t x_addr8 = smem_u32(x_s + (size_t)n_row8 * X_PITCH + (lane & 3) * 4);
  const bool sgn = (a.w8_fmt == MUI_W8_SYM_ROW);
  const uint32_t xmask = sgn ? 0x80808080u : 0u, cbias = W8Cvt<T>::bias_for(sgn);

  // chunk loader: this thread's 8 columns of every batch row, and of the norm weights
  uint4 xr[NB], nwr;
  auto load_chunk = [&](int kc) {
    const int k = kc * KC + tid * 8;
    const bool in = k < K;
#pragma unroll
    for (int b = 0; b < NB; ++b)
      xr[b] = (in && b < a.B) ? ld_act16(x + (size_t)b * K + k) : make_uint4(0, 0, 0, 0);
    nwr = (in && do_norm) ? ld_cached16(nw + k) : make_uint4(0, 0, 0, 0);
  };
  auto store_chunk = [&]() {
    float wv[8];
    if (do_norm) unpack8<T>(nwr, wv);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      uint4 out = xr[b];
      if (do_norm) {
        float f[8];
        unpack8<T>(xr[b], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = Elt<T>::to_f32(Elt<T>::from_f32(f[i] * rstd[b])) * wv[i];
        out = pack8<T>(f);
      }
      *reinterpret_cast<uint4*>(x_s + (size_t)b * X_PITCH + tid * 8) = out;
    }
  };

  int it = 0;
  bool ok = true;
  bool first_store = true;
  for (int gidx = 0; gidx < ngroups; ++gidx) {
    const int blk0 = gidx * XC_MAX_BLOCKS;
    const int nb_g = min(XC_MAX_BLOCKS, nblk - blk0);
    float d[XC_MAX_BLOCKS][4];
#pragma unroll
    for (int bi = 0; bi < XC_MAX_BLOCKS; ++bi) d[bi][0] = d[bi][1] = d[bi][2] = d[bi][3] = 0.f;
    load_chunk(0);
    for (int kc = 0; kc < nchunks; ++kc) {
      const int kc_len = min(KC, K - kc * KC);
      // nobody still reads the previous chunk (or the partial tiles of the previous group) from x_s
      if (!first_store) named_bar_sync(1, GEMV_CONSUMER_THREADS);
      first_store = false;
      store_chunk();
      if (kc + 1 < nchunks) load_chunk(kc + 1);  // in flight while this chunk is multiplied
      named_bar_sync(1, GEMV_CONSUMER_THREADS);
      if (tid == 0 && gidx == 0 && kc == 0) trace_mark(a.trace, 3, true);
#pragma unroll
      for (int bi = 0; bi < XC_MAX_BLOCKS; ++bi) {
        if (bi < nb_g && ok) {
          const int s = it % num_stages;
          const uint32_t ph = (it / num_stages) & 1;
          if (!mbar_wait_bounded(full_bar + s, ph, abort_flag)) {
            if (lane == 0 && !*abort_flag) {
              mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, s);
              *abort_flag = 1;
            }
            ok = false;
          } else {
            const uint32_t a_addr = stage_base + static_cast<uint32_t>(s) * G::STAGE_BYTES + a_lane_off;
            if (WB == 16) {
              const int nsteps = kc_len >> 4;
              const uint32_t b_addr = x_base + b_lane_off;
#pragma unroll 4
              for (int j = warp; j < nsteps; j += GEMV_CONSUMER_WARPS) {
                uint32_t af[4], b0, b1;
                ldmatrix_x4(af, a_addr + j * 32);
                ldmatrix_x2(b0, b1, b_addr + j * 32);
                MmaOp<T>::run(d[bi], af, b0, b1);
              }
            } else {
              const int nsteps = kc_len >> 5;
              float d2[4] = {0.f, 0.f, 0.f, 0.f};  // second chain: halves the dependent mma sequence
#pragma unroll 4
              for (int j = warp; j < nsteps; j += GEMV_CONSUMER_WARPS) {
                uint32_t r[4];
                ldmatrix_x4(r, a_addr + j * 32);
                uint32_t xa0, xa1, xb0, xb1;
                lds_v2(x_addr8 + j * 64, xa0, xa1);
                lds_v2(x_addr8 + j * 64 + 32, xb0, xb1);
                uint32_t af[4], bf[4];
                W8Cvt<T>::cvt4(r[0], xmask, cbias, af[0], af[2]);
                W8Cvt<T>::cvt4(r[1], xmask, cbias, af[1], af[3]);
                W8Cvt<T>::cvt4(r[2], xmask, cbias, bf[0], bf[2]);
                W8Cvt<T>::cvt4(r[3], xmask, cbias, bf[1], bf[3]);
                MmaOp<T>::run(d[bi], af, xa0, xa1);
                MmaOp<T>::run(d2, bf, xb0, xb1);
              }
#pragma unroll
              for (int q = 0; q < 4; ++q) d[bi][q] += d2[q];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar + s);
            ++it;
          }
        }
      }
    }

    // the group's row blocks are complete: per block, the eight warps' partial tiles are summed through shared
    // memory (the activation buffer is free now) in a fixed order, then the epilogue
    float* rbuf = reinterpret_cast<float*>(x_s);
    const int trow = lane >> 2, n0 = (lane & 3) * 2;  // this thread holds D[trow (+8)][batch n0, n0 + 1]
#pragma unroll
    for (int bi = 0; bi < XC_MAX_BLOCKS; ++bi) {
      if (bi < nb_g) {
        named_bar_sync(1, GEMV_CONSUMER_THREADS);
        if (n0 < NB) {
          rbuf[(warp * PIPE_ROWS + trow) * NB + n0] = d[bi][0];
          rbuf[(warp * PIPE_ROWS + trow + 8) * NB + n0] = d[bi][2];
        }
        if (n0 + 1 < NB) {
          rbuf[(warp * PIPE_ROWS + trow) * NB + n0 + 1] = d[bi][1];
          rbuf[(warp * PIPE_ROWS + trow + 8) * NB + n0 + 1] = d[bi][3];
        }
        named_bar_sync(1, GEMV_CONSUMER_THREADS);
        if (ok && tid < ROWS_PER_STAGE * NB) {
          const int r = tid / NB, b = tid - r * NB;
          const int row = r_begin + (blk0 + bi) * ROWS_PER_STAGE + r;
          if (row < r_end && b < a.B) {
            if (MODE == 0) {
              float v = 0.f;
#pragma unroll
              for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) v += rbuf[(w * PIPE_ROWS + r) * NB + b];
              gemv_store_linear<T>(a, b, row, v, comm_seq);
            } else {
              float g = 0.f, u = 0.f;
#pragma unroll
              for (int w = 0; w < GEMV_CONSUMER_WARPS; ++w) {
                g += rbuf[(w * PIPE_ROWS + r) * NB + b];
                u += rbuf[(w * PIPE_ROWS + r + 8) * NB + b];
              }
              gemv_store_gateup<T>(a, b, row, total_rows, g, u, 1.f);
            }
          }
        }
      }
    }
  }
  if (MODE == 0 && a.use_comm)
    gemv_comm_tail<T>(a, comm_seq, tid, GEMV_CONSUMER_THREADS, 1, r_end - r_begin,
                      [r_begin](int i) { return r_begin + i; });
  if (tid == 0) trace_end(a.trace);
}
