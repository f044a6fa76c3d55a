// Prefill (more than 8 rows) linear layers on the 5th-generation tensor cores of sm_100a:
//
//   y[m, n] = act( sum_k W[n, k] * x[m, k] ) * mul_bias[n] + add_bias[n] + residual[m, n]        (linear)
//   t[m, i] = silu( sum_k G[i, k] x[m, k] ) * ( sum_k U[i, k] x[m, k] )                           (gate/up)
//
// The reference hands these shapes to at::linear (csrc/modules/linear_module.cpp:61-77,
// csrc/modules/parallel_linear_module.cpp:73-83); the decode GEMV does not apply to them.
//
//  * Operand roles are swapped so that the 128 lanes of tensor memory hold 128 WEIGHT rows and the tokens run along
//    the columns: a CTA owns a [128 weight rows] x [mt tokens] tile (mt = 16..256), so for up to 256 tokens the
//    weights are streamed from HBM exactly once.
//  * One thread issues TMA tile loads (cp.async.bulk.tensor.2d, 128-byte swizzle, K-major, 64 elements of K per
//    stage) of the weight tile(s) and the activation tile into a ring of shared-memory stages completed on
//    mbarriers; rows past the edge of a matrix are zero-filled by the copy engine.
//  * One thread issues tcgen05.mma (kind::f16, M = 128, N = mt, K = 16; fp32 accumulators in tensor memory) and
//    releases each stage with tcgen05.commit.
//  * Four warps read the accumulators back with tcgen05.ld and apply the epilogue.
// Every wait is bounded: a wait that runs out records a device status code, the CTA waits (bounded) for its copies
// and MMAs in flight, frees its tensor memory and returns. No cluster launch, no multicast.
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"

MUI_STATUS_ACCESSOR(prefill)

namespace {

constexpr int PF_TILE_N = 128;                              // weight rows per CTA = UMMA M
constexpr int PF_BLOCK_K = 64;                              // elements of K per stage = one 128-byte swizzle span
constexpr int PF_UMMA_K = 16;                               // K of one tcgen05.mma for 16-bit operands
constexpr int PF_W_TILE_BYTES = PF_TILE_N * PF_BLOCK_K * 2;  // 16 KiB
constexpr int PF_MAX_STAGES = 8;
constexpr int PF_MAX_MT = 256;                              // tokens per CTA tile = UMMA N
// Two warpgroups: warp 0 issues the TMA loads, warp 1 owns the tensor memory and issues the MMAs, warps 2-3 idle,
// warps 4-7 (tensor-memory lanes 32 * (warp % 4)) run the epilogue.
constexpr int PF_THREADS = 256;
constexpr int PF_EPI_WARP0 = 4;

struct PfArgs {
  int M, N, K;
  int mt;         // tokens per CTA tile (multiple of 16)
  int nkb;        // 64-wide K blocks
  int stages;
  int tmem_cols;  // allocated tensor-memory columns (power of two >= 32)
  int activ;
  const void* mul_bias;
  const void* add_bias;
  const void* residual;
  void* y;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
// 2-D tile load global -> this CTA's shared memory; x = element coordinate along K (a multiple of 64 here, so the
// 16-byte rule holds), y = row; completion is counted in bytes on `bar`
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* m, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// whole warp; the base address of `cols` columns is written to *dst_smem
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
// the mbarrier receives one arrival when every tcgen05.mma issued so far by this thread has finished
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, both operands K-major
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 16 consecutive fp32 columns of this thread's tensor-memory lane (lane = 32 * (warp % 4) + lane id)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 16-bit elements) laid out with the
// 128-byte swizzle (what the TMA load above writes): groups of 8 rows are 1024 bytes apart (stride byte offset); the
// leading byte offset is not used by swizzled K-major layouts (set to 1); descriptor version 1 (sm_100); layout type
// 2 (128-byte swizzle). The tile must start on a 1024-byte boundary.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);  // bits [0,14): start address / 16
  d |= static_cast<uint64_t>(1) << 16;                      // bits [16,30): leading byte offset / 16
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // bits [32,46): stride byte offset / 16
  d |= static_cast<uint64_t>(1) << 46;                      // bits [46,48): version
  d |= static_cast<uint64_t>(2) << 61;                      // bits [61,64): SWIZZLE_128B
  return d;
}
// Instruction descriptor of kind::f16: fp32 accumulate, A and B of the same 16-bit format, both K-major.
__device__ __forceinline__ uint32_t make_idesc(int is_bf16, int m, int n) {
  uint32_t d = 0;
  d |= 1u << 4;                                // bits [4,6): accumulator format fp32
  d |= static_cast<uint32_t>(is_bf16) << 7;    // bits [7,10): A format (0 fp16, 1 bf16)
  d |= static_cast<uint32_t>(is_bf16) << 10;   // bits [10,13): B format
  d |= static_cast<uint32_t>(n >> 3) << 17;    // bits [17,23): N / 8
  d |= static_cast<uint32_t>(m >> 4) << 24;    // bits [24,29): M / 16
  return d;
}

template <typename T, int NMAT>
__device__ __forceinline__ void pf_store(const PfArgs& a, int tok, int n, float g, float u) {
  float v = g;
  if (NMAT == 2) {
    v = silu_f32(g) * u;
  } else {
    if (a.activ == MUI_ACT_SILU) v = silu_f32(v);
    // plain loads: the 16-bit __ldg overloads are non-volatile inline asm, which the compiler is free to hoist above
    // the null checks (it did: the first versions of this kernel read address n * 2 when no bias was given)
    if (a.mul_bias != nullptr) v *= Elt<T>::to_f32(reinterpret_cast<const T*>(a.mul_bias)[n]);
    if (a.add_bias != nullptr) v += Elt<T>::to_f32(reinterpret_cast<const T*>(a.add_bias)[n]);
    if (a.residual != nullptr)
      v += ld_act_f32<T>(reinterpret_cast<const T*>(a.residual) + static_cast<size_t>(tok) * a.N + n);
  }
  reinterpret_cast<T*>(a.y)[static_cast<size_t>(tok) * a.N + n] = Elt<T>::from_f32(v);
}

// grid = (weight tiles of 128 rows, token chunks of mt); block = 256 threads
template <typename T, int NMAT>
__global__ void __launch_bounds__(PF_THREADS, 1)
    prefill_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_u,
                        const __grid_constant__ CUtensorMap tm_x, const PfArgs a) {
  extern __shared__ unsigned char pf_smem_raw[];
  __shared__ uint64_t full_bar[PF_MAX_STAGES];   // one arrival (the producer's expect_tx) + the tiles' bytes
  __shared__ uint64_t empty_bar[PF_MAX_STAGES];  // one arrival (tcgen05.commit): the MMAs have read the stage
  __shared__ uint64_t acc_bar;                   // one arrival (tcgen05.commit): the accumulators are complete
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  // the swizzle and the matrix descriptors both assume tiles that start on 1024-byte boundaries
  const uint32_t raw_u = smem_u32(pf_smem_raw);
  const uint32_t tiles_u = (raw_u + 1023u) & ~1023u;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * PF_TILE_N;
  const int tok0 = blockIdx.y * a.mt;
  const int S = a.stages;
  const int nk = a.nkb;
  const uint32_t stage_bytes = static_cast<uint32_t>(NMAT * PF_W_TILE_BYTES + a.mt * PF_BLOCK_K * 2);
  volatile int* abort_flag = &abort_s;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    abort_s = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, static_cast<uint32_t>(a.tmem_cols));
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      pdl_wait_prior_grid();  // the activations are the previous kernel's output
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < nk; ++i) {
        const int s = i % S;
        if (i >= S && !mbar_wait_bounded(&empty_bar[s], ((i / S) - 1) & 1, abort_flag)) {
          if (!*abort_flag) mui_dev_set_status(MUI_DEV_TIMEOUT_EMPTY, 0x700000u | s);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint32_t st = tiles_u + static_cast<uint32_t>(s) * stage_bytes;
        const int k0 = i * PF_BLOCK_K;
        mbar_arrive_expect_tx(&full_bar[s], stage_bytes);
        tma_load_2d(st, &tm_w, k0, n0, &full_bar[s]);
        if (NMAT == 2) tma_load_2d(st + PF_W_TILE_BYTES, &tm_u, k0, n0, &full_bar[s]);
        tma_load_2d(st + NMAT * PF_W_TILE_BYTES, &tm_x, k0, tok0, &full_bar[s]);
        issued = i + 1;
      }
      if (!ok) {
        // leave no copy in flight behind: wait (bounded) for every stage that was armed
        for (int i = max(0, issued - S); i < issued; ++i) {
          int zero = 0;
          if (!mbar_wait_bounded(&full_bar[i % S], (i / S) & 1, &zero)) mui_dev_set_status(MUI_DEV_TIMEOUT_DRAIN, i % S);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(std::is_same<T, __half>::value ? 0 : 1, PF_TILE_N, a.mt);
      bool ok = true;
      for (int i = 0; i < nk && ok; ++i) {
        const int s = i % S;
        if (!mbar_wait_bounded(&full_bar[s], (i / S) & 1, abort_flag)) {
          if (!*abort_flag) mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, 0x700000u | s);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t st = tiles_u + static_cast<uint32_t>(s) * stage_bytes;
        const uint64_t dw = make_kmajor_sw128_desc(st);
        const uint64_t du = make_kmajor_sw128_desc(st + PF_W_TILE_BYTES);
        const uint64_t dx = make_kmajor_sw128_desc(st + NMAT * PF_W_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < PF_BLOCK_K / PF_UMMA_K; ++k) {
          // 16 elements along K = 32 bytes inside the swizzle span = 2 units of the start-address field
          const uint32_t acc = (i | k) != 0;
          umma_f16(tmem_base, dw + 2 * k, dx + 2 * k, idesc, acc);
          if (NMAT == 2) umma_f16(tmem_base + a.mt, du + 2 * k, dx + 2 * k, idesc, acc);
        }
        tc_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
      }
      tc_commit(&acc_bar);  // accumulators complete (on the abort path: whatever was issued has finished)
      if (!ok) {
        int zero = 0;
        if (!mbar_wait_bounded(&acc_bar, 0, &zero)) mui_dev_set_status(MUI_DEV_TIMEOUT_DRAIN, 0x7000ffu);
      }
    }
    __syncwarp();
  } else if (warp >= PF_EPI_WARP0) {
    // ------------------------------ epilogue: warps 4-7 own tensor-memory lanes 32 * (warp % 4) ... ------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;  // weight row inside the tile = tensor-memory lane
    const int n = n0 + row;
    pdl_wait_prior_grid();          // the residual is an earlier kernel's output
    bool ok = mbar_wait_bounded(&acc_bar, 0, abort_flag);
    if (!ok && !*abort_flag) {
      mui_dev_set_status(MUI_DEV_TIMEOUT_FULL, 0x7000ffu);
      *abort_flag = 1;
    }
    ok = ok && (*abort_flag == 0);
    ok = __all_sync(MUI_FULL_MASK, ok);
    tc_fence_after_sync();
    if (ok) {
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      for (int c0 = 0; c0 < a.mt; c0 += 16) {
        if (tok0 + c0 >= a.M) break;  // warp-uniform
        float g[16], u[16];
        tmem_ld16(lane_addr + c0, g);
        if (NMAT == 2) tmem_ld16(lane_addr + a.mt + c0, u);
        if (n < a.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + c0 + j;
            if (tok < a.M) pf_store<T, NMAT>(a, tok, n, g[j], NMAT == 2 ? u[j] : 0.f);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(a.tmem_cols));
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point query (the library links no libcuda)
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Tensor map of a row-major [rows, K] 16-bit matrix, tiles of [box_rows] x [64 elements of K], 128-byte swizzle;
// out-of-range elements read as zero.
mui_status_t make_map(CUtensorMap* m, mui_dtype_t dtype, const void* base, int rows, int K, int box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  MUI_REQUIRE(enc != nullptr, MUI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(PF_BLOCK_K), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estride[2] = {1, 1};
  const CUresult r = enc(m, dtype == MUI_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                         const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MUI_REQUIRE(r == CUDA_SUCCESS, MUI_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (rows=%d K=%d box=%d)",
              static_cast<int>(r), rows, K, box_rows);
  return MUI_OK;
}

int pow2_at_least(int v, int lo) {
  int p = lo;
  while (p < v) p <<= 1;
  return p;
}

template <typename T, int NMAT>
mui_status_t pf_launch(cudaStream_t stream, const CUtensorMap& mw, const CUtensorMap& mu, const CUtensorMap& mx,
                       const PfArgs& a, dim3 grid, size_t smem, int pdl, const MuiDeviceInfo* di) {
  static std::mutex mu_;
  static unsigned long long configured = 0;  // per instantiation: one bit per device
  {
    std::lock_guard<std::mutex> lock(mu_);
    const unsigned long long bit = 1ull << (di->device & 63);
    if (!(configured & bit)) {
      MUI_CUDA_CHECK(cudaFuncSetAttribute(prefill_gemm_kernel<T, NMAT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          di->smem_per_block_optin - 1024));
      configured |= bit;
    }
  }
  MUI_CUDA_CHECK(mui_launch(prefill_gemm_kernel<T, NMAT>, grid, dim3(PF_THREADS), smem, stream, pdl, mw, mu, mx, a));
  return MUI_OK;
}

mui_status_t pf_run(void* stream, mui_dtype_t dtype, int M, int N, int K, int nmat, const void* w, const void* u,
                    mui_activation_t activ, const void* mul_bias, const void* add_bias, const void* residual,
                    const void* x, void* y, unsigned flags) {
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(M >= 1 && N >= 1 && K >= 1, MUI_ERR_INVALID_ARG, "bad sizes M=%d N=%d K=%d", M, N, K);
  MUI_REQUIRE(w && x && y && (nmat == 1 || u), MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(K % 8 == 0, MUI_ERR_UNSUPPORTED, "K=%d: rows must be a multiple of 16 bytes for the tile copies", K);
  MUI_REQUIRE(((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(u)) &
               15) == 0,
              MUI_ERR_INVALID_ARG, "weights and activations must be 16-byte aligned");
  const MuiDeviceInfo* di = mui_current_device_info();
  if (!di) return MUI_ERR_CUDA;
  PfArgs a;
  a.M = M;
  a.N = N;
  a.K = K;
  // token tiles of equal size, a multiple of 16, at most 256
  const int chunks = (M + PF_MAX_MT - 1) / PF_MAX_MT;
  a.mt = ((M + chunks - 1) / chunks + 15) / 16 * 16;
  a.nkb = (K + PF_BLOCK_K - 1) / PF_BLOCK_K;
  const int stage_bytes = nmat * PF_W_TILE_BYTES + a.mt * PF_BLOCK_K * 2;
  int stages = (di->smem_per_block_optin - 3072) / stage_bytes;  // 1 KiB alignment slack, barriers
  stages = stages > PF_MAX_STAGES ? PF_MAX_STAGES : stages;
  stages = stages > a.nkb ? a.nkb : stages;
  MUI_REQUIRE(stages >= 1, MUI_ERR_UNSUPPORTED, "a tile of %d tokens does not fit in shared memory", a.mt);
  a.stages = stages;
  a.tmem_cols = pow2_at_least(nmat * a.mt, 32);
  a.activ = static_cast<int>(activ);
  a.mul_bias = mul_bias;
  a.add_bias = add_bias;
  a.residual = residual;
  a.y = y;
  CUtensorMap mw, mu, mx;
  if (mui_status_t s = make_map(&mw, dtype, w, N, K, PF_TILE_N)) return s;
  if (nmat == 2) {
    if (mui_status_t s = make_map(&mu, dtype, u, N, K, PF_TILE_N)) return s;
  } else {
    mu = mw;
  }
  if (mui_status_t s = make_map(&mx, dtype, x, M, K, a.mt)) return s;
  const dim3 grid((N + PF_TILE_N - 1) / PF_TILE_N, (M + a.mt - 1) / a.mt);
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 1024;
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == MUI_F16)
    return nmat == 1 ? pf_launch<__half, 1>(st, mw, mu, mx, a, grid, smem, pdl, di)
                     : pf_launch<__half, 2>(st, mw, mu, mx, a, grid, smem, pdl, di);
  return nmat == 1 ? pf_launch<__nv_bfloat16, 1>(st, mw, mu, mx, a, grid, smem, pdl, di)
                   : pf_launch<__nv_bfloat16, 2>(st, mw, mu, mx, a, grid, smem, pdl, di);
}

}  // namespace

extern "C" {

mui_status_t mui_prefill_linear_forward(void* stream, mui_dtype_t dtype, int M, int N, int K, const void* weights,
                                        mui_activation_t activ, const void* mul_bias, const void* add_bias,
                                        const void* residual, const void* x, void* y, unsigned flags) {
  return pf_run(stream, dtype, M, N, K, 1, weights, nullptr, activ, mul_bias, add_bias, residual, x, y, flags);
}

mui_status_t mui_prefill_gateup_silu_forward(void* stream, mui_dtype_t dtype, int M, int I, int H,
                                             const void* gate_weights, const void* up_weights, const void* x, void* t,
                                             unsigned flags) {
  return pf_run(stream, dtype, M, I, H, 2, gate_weights, up_weights, MUI_ACT_IDENTITY, nullptr, nullptr, nullptr, x, t,
                flags);
}

}  // extern "C"
