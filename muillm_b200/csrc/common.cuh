// Shared device helpers for the sm_100a decode kernels: 16-bit <-> fp32 packing,
// warp/block reductions, streaming loads, mbarrier + bulk-async-copy (TMA) wrappers
// with bounded waits, programmatic-dependent-launch hooks and the device status word.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "muillm_b200.h"

#define MUI_WARP 32
#define MUI_FULL_MASK 0xffffffffu

// ---------------------------------------------------------------------------------------------
// device status word: kernels never trap; a wait that runs out records a code here and returns.
// ---------------------------------------------------------------------------------------------
// bit layout: [31:24] code, [23:0] detail (kernel specific, e.g. stage index or rank)
#define MUI_DEV_OK 0u
#define MUI_DEV_TIMEOUT_FULL 1u    // consumer gave up waiting for a bulk copy to land
#define MUI_DEV_TIMEOUT_EMPTY 2u   // producer gave up waiting for a stage to be released
#define MUI_DEV_TIMEOUT_PEER 3u    // all-reduce gave up waiting for a peer's flag
#define MUI_DEV_TIMEOUT_DRAIN 4u   // gave up waiting for own copies in flight at exit
#define MUI_DEV_BAD_LENGTH 5u      // a kernel variant with a bounded sequence length was given a longer one

// One status word per translation unit (no relocatable device code is needed that way); each kernel
// file instantiates MUI_STATUS_ACCESSOR(tag) once and mui_device_status() visits all of them.
static __device__ unsigned int g_mui_dev_status = 0;

typedef cudaError_t (*mui_status_accessor_t)(unsigned* v, int clear);
void mui_register_status_accessor(mui_status_accessor_t fn);

#define MUI_STATUS_ACCESSOR(tag)                                                   \
  static cudaError_t mui_status_access_##tag(unsigned* v, int clear) {             \
    cudaError_t e = cudaMemcpyFromSymbol(v, g_mui_dev_status, sizeof(unsigned));   \
    if (e != cudaSuccess) return e;                                                \
    if (clear && *v != 0) {                                                        \
      unsigned z = 0;                                                              \
      e = cudaMemcpyToSymbol(g_mui_dev_status, &z, sizeof(unsigned));              \
    }                                                                              \
    return e;                                                                      \
  }                                                                                \
  static const int mui_status_registered_##tag =                                   \
      (mui_register_status_accessor(mui_status_access_##tag), 0);

__device__ __forceinline__ void mui_dev_set_status(unsigned code, unsigned detail) {
  atomicCAS(&g_mui_dev_status, 0u, (code << 24) | (detail & 0xffffffu));
}

// ---------------------------------------------------------------------------------------------
// programmatic dependent launch (PDL). Both are no-ops when the kernel was launched without the
// programmatic-stream-serialization attribute.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait_prior_grid() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// Launch tracing: when the host has switched tracing on (mui_trace_enable), every traced launch gets a
// record of two 64-bit words in a device buffer pre-filled with 0xFF: the earliest %globaltimer at which any of
// its CTAs started and (stored complemented, so that atomicMin serves both) the latest at which any finished.
// The timeline of a captured, dependently launched step can be read back without a profiler.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void trace_start(unsigned long long* rec) {
  if (rec != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    atomicMin(rec, t);
  }
}
__device__ __forceinline__ void trace_end(unsigned long long* rec) {
  if (rec != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    atomicMin(rec + 1, ~t);
  }
}
// optional extra stamps of a record (words 2 and 3): earliest moment a CTA got past its wait for the previous
// kernel, and (complemented) latest moment a CTA had its activations staged
__device__ __forceinline__ void trace_mark(unsigned long long* rec, int word, bool complement) {
  if (rec != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    atomicMin(rec + word, complement ? ~t : t);
  }
}
// next record of the calling thread's trace (nullptr when tracing is off or the buffer is full)
unsigned long long* mui_trace_next_record(int kernel_tag);

// ---------------------------------------------------------------------------------------------
// 16-bit element traits
// ---------------------------------------------------------------------------------------------
template <typename T> struct Elt;

template <> struct Elt<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
  // unpack two packed elements (low, high) to fp32
  static __device__ __forceinline__ float2 unpack2(uint32_t u) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
  }
  static __device__ __forceinline__ uint32_t pack2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

template <> struct Elt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float2 unpack2(uint32_t u) {
    float2 r;
    r.x = __uint_as_float(u << 16);
    r.y = __uint_as_float(u & 0xffff0000u);
    return r;
  }
  static __device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

// unpack 8 packed 16-bit elements held in a uint4 into 8 floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  float2 a = Elt<T>::unpack2(v.x), b = Elt<T>::unpack2(v.y);
  float2 c = Elt<T>::unpack2(v.z), d = Elt<T>::unpack2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = Elt<T>::pack2(f[0], f[1]);
  v.y = Elt<T>::pack2(f[2], f[3]);
  v.z = Elt<T>::pack2(f[4], f[5]);
  v.w = Elt<T>::pack2(f[6], f[7]);
  return v;
}

// dot of 8 packed weights with 8 fp32 activations, accumulated in fp32
template <typename T>
__device__ __forceinline__ float dot8(const uint4& w, const float (&x)[8], float acc) {
  float f[8];
  unpack8<T>(w, f);
#pragma unroll
  for (int i = 0; i < 8; ++i) acc = fmaf(f[i], x[i], acc);
  return acc;
}

// ---------------------------------------------------------------------------------------------
// loads
// ---------------------------------------------------------------------------------------------
// streaming 16-byte load of read-once data (weights): non-coherent path, do not keep in L1
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// 16-byte load through the read-only path: ONLY for data that no kernel ever writes while this one may be
// resident (weights, norm weights, rotary tables). Under programmatic dependent launch a kernel is resident
// before its predecessor has written the activations, so those must not take this path.
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
// Loads of activations and device-side state produced by earlier kernels: served from L2 (the coherence
// point), never from a possibly stale L1 / read-only cache line.
__device__ __forceinline__ uint4 ld_act16(const void* p) {
  return __ldcg(reinterpret_cast<const uint4*>(p));
}
template <typename T>
__device__ __forceinline__ float ld_act_f32(const T* p) {
  const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return Elt<T>::to_f32(*reinterpret_cast<const T*>(&raw));
}
template <typename T>
__device__ __forceinline__ T ld_act(const T* p) {
  const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return *reinterpret_cast<const T*>(&raw);
}
// 16-byte load with system-scope relaxed semantics (peer memory, never from a stale L1 line)
__device__ __forceinline__ uint4 ld_sys16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(MUI_FULL_MASK, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(MUI_FULL_MASK, v, o));
  return v;
}

__device__ __forceinline__ float silu_f32(float v) { return v / (1.f + __expf(-v)); }

// named barrier over a subset of the CTA's warps (id 1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// mbarrier + bulk async copy (TMA, 1-D form). Waits are bounded: a wait that runs out returns
// false; the caller records a status code and leaves its loop.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void lds_v2(uint32_t addr, uint32_t& a, uint32_t& b) {
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  // make the initialised barriers visible to the async proxy before any copy names them
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~MUI_WAIT_LIMIT_NS of wall time (globaltimer) or as soon as
// *abort_flag becomes non-zero. Returns true when the phase completed.
#define MUI_WAIT_LIMIT_NS 1000000000ull
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  unsigned spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > MUI_WAIT_LIMIT_NS) return false;
    }
  }
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// 1-D bulk copy global -> this CTA's shared memory; completion is counted in bytes on `bar`.
// src and dst must be 16-byte aligned and bytes a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                             uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Bulk prefetch of a global range into L2 (no shared memory involved): src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src_gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------------------------------------
// host helpers
// ---------------------------------------------------------------------------------------------
void mui_set_error(const char* fmt, ...);

#define MUI_REQUIRE(cond, status, ...)  \
  do {                                  \
    if (!(cond)) {                      \
      mui_set_error(__VA_ARGS__);       \
      return (status);                  \
    }                                   \
  } while (0)

#define MUI_CUDA_CHECK(expr)                                                            \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess) {                                                            \
      mui_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return MUI_ERR_CUDA;                                                              \
    }                                                                                   \
  } while (0)

struct MuiDeviceInfo {
  int device;
  int sm_count;
  int smem_per_block_optin;
  int smem_per_sm;
  int l2_bytes;
};
// cached per-device properties of the current device (nullptr + error set on failure)
const MuiDeviceInfo* mui_current_device_info();

// Launch helper: sets the programmatic-stream-serialization attribute when `pdl` is non-zero.
template <typename... KArgs, typename... Args>
static inline cudaError_t mui_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     int pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
