// Device side of the one-shot "push" all-reduce over peer memory (NVLink / NVSwitch), shared by the
// stand-alone collective kernels and the GEMV epilogue.
//
// Every rank owns a segment [2 generations][world][capacity] of fp32 partial sums plus one 64-bit flag per
// source rank. A collective with sequence number s (generation s & 1) runs as:
//   1. each rank stores its fp32 partial for element i into slot [gen][my_rank][i] of EVERY rank's segment
//      (plain 4/16-byte stores to peer pointers; posted writes, nothing is read remotely);
//   2. when all of a rank's stores are issued (all CTAs arrived on a local counter), one thread does
//      __threadfence_system() and writes s into flag[my_rank] of every rank with st.release.sys;
//   3. each rank waits until its local flags of all ranks are >= s (ld.acquire.sys, bounded spin), then sums the
//      world slots of its own segment in rank order 0..P-1 in fp32 and rounds once — every rank gets the same
//      bits. A wait that runs out records MUI_DEV_TIMEOUT_PEER with the late rank and skips the sum.
// A rank may overwrite generation g for collective s+2 only after it left collective s+1, where it saw every
// peer's flag s+1, which a peer publishes only after its own reads of collective s are done: no trailing barrier.
#pragma once

#include "common.cuh"

#define MUI_COMM_MAX_RANKS 8
#define MUI_COMM_WAIT_NS 2000000000ull
#define MUI_COMM_FLAG_STRIDE 16  // u64 words between two ranks' flags (128 bytes)

struct CommDev {
  float* push_dst[MUI_COMM_MAX_RANKS];               // rank p's segment: &data[gen][my_rank][0]
  unsigned long long* flag_dst[MUI_COMM_MAX_RANKS];  // rank p's segment: &flags[my_rank]
  const float* local_slots;                          // my segment: &data[gen][0][0]
  const unsigned long long* local_flags;             // my segment: &flags[0]
  unsigned int* arrive_counter;                      // local, zero between collectives
  unsigned long long seq;
  int world, rank;
  int capacity;  // elements per slot
};

__device__ __forceinline__ void comm_push(const CommDev& c, size_t idx, float v) {
#pragma unroll
  for (int p = 0; p < MUI_COMM_MAX_RANKS; ++p)
    if (p < c.world) c.push_dst[p][idx] = v;
}

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Called by one thread of each CTA after the CTA's pushes are complete (a CTA-wide barrier precedes it).
// The last CTA of the grid publishes the flags.
__device__ __forceinline__ void comm_cta_arrive_and_publish(const CommDev& c, unsigned num_ctas) {
  __threadfence_system();
  const unsigned prev = atomicAdd(c.arrive_counter, 1u);
  if (prev == num_ctas - 1) {
    *c.arrive_counter = 0u;
    __threadfence_system();
    for (int p = 0; p < c.world; ++p) st_release_sys_u64(c.flag_dst[p], c.seq);
  }
}

// Thread r < world waits for rank r's flag. Returns false (and records the status) on timeout.
__device__ __forceinline__ bool comm_wait_rank(const CommDev& c, int r) {
  const unsigned long long* f = c.local_flags + (size_t)r * MUI_COMM_FLAG_STRIDE;
  if (ld_acquire_sys_u64(f) >= c.seq) return true;
  const uint64_t t0 = global_timer_ns();
  unsigned spins = 0;
  while (ld_acquire_sys_u64(f) < c.seq) {
    if ((++spins & 0xff) == 0 && global_timer_ns() - t0 > MUI_COMM_WAIT_NS) {
      mui_dev_set_status(MUI_DEV_TIMEOUT_PEER, static_cast<unsigned>(r));
      return false;
    }
  }
  return true;
}

// Sum of the world slots for element idx, fixed rank order, fp32.
__device__ __forceinline__ float comm_reduce_elem(const CommDev& c, size_t idx) {
  float s = 0.f;
#pragma unroll
  for (int r = 0; r < MUI_COMM_MAX_RANKS; ++r)
    if (r < c.world) s += __ldcg(c.local_slots + (size_t)r * c.capacity + idx);
  return s;
}
