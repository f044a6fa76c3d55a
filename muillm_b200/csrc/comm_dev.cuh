// Device side of the one-shot "push" all-reduce over peer memory (NVLink / NVSwitch), shared by the
// stand-alone collective kernels and the GEMV epilogue.
//
// Every rank owns a segment of 8-byte cells [2 generations][world][capacity] and a device-resident sequence
// counter. A cell carries one fp32 partial sum in its low half and the 32-bit sequence number of the collective
// that wrote it in its high half; the two travel in ONE 64-bit store, so a reader that sees the expected
// sequence number also sees the value — no fence, no separate flag, no remote read:
//   1. the owner of output element i stores {partial, s} into cell [s & 1][my_rank][i] of EVERY rank's segment
//      (plain 64-bit stores to peer pointers; posted writes);
//   2. the same thread block then polls the world cells of element i in its own segment until each shows
//      sequence s (relaxed system-scope loads of local memory, bounded spin) and adds them in rank order 0..P-1
//      in fp32, rounding once — every rank gets the same bits. A wait that runs out records
//      MUI_DEV_TIMEOUT_PEER with the late rank and leaves the output element untouched;
//   3. the last CTA of the grid to finish advances the sequence counter (read from device memory at kernel
//      start, so a launch captured in a CUDA graph replays correctly).
// The in-cell sequence number is the low 32 bits of the 64-bit counter and is compared for equality with the
// expected one. It wraps after 2^32 collectives (about a day of decoding at 50 k collectives per second); a stale
// cell could only be mistaken for a fresh one if it had not been rewritten for exactly 2^32 collectives, i.e. if no
// collective of the same parity had covered its index in all that time. Decode loops repeat their message sizes
// every step, so every cell in use is rewritten every other collective.
// Generation g is overwritten for collective s+2 only after this rank's kernel of collective s+1 completed, in
// which it received every peer's s+1 cells, and a peer writes those only from a kernel that started after its
// own kernel of collective s (which read generation g) completed: no barrier is needed.
#pragma once

#include "common.cuh"

#define MUI_COMM_MAX_RANKS 8
#define MUI_COMM_WAIT_NS 2000000000ull

struct CommDev {
  unsigned long long* peer_cells[MUI_COMM_MAX_RANKS];  // rank p's cell array
  unsigned long long* local_seq;                       // collectives completed on this rank
  unsigned int* arrive_counter;                        // local, zero between collectives
  int world, rank;
  int capacity;  // cells per slot
};

__device__ __forceinline__ unsigned long long comm_begin(const CommDev& c) { return __ldcg(c.local_seq) + 1ull; }

__device__ __forceinline__ void comm_push(const CommDev& c, unsigned long long seq, size_t idx, float v) {
  const size_t off = ((size_t)(seq & 1ull) * c.world + c.rank) * c.capacity + idx;
  const unsigned long long cell = ((seq & 0xffffffffull) << 32) | (unsigned long long)__float_as_uint(v);
#pragma unroll
  for (int p = 0; p < MUI_COMM_MAX_RANKS; ++p)
    if (p < c.world) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(c.peer_cells[p] + off), "l"(cell) : "memory");
}

__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// A peer wait that ran out is sticky: once the status word of this translation unit carries MUI_DEV_TIMEOUT_PEER,
// every later wait (other elements, other ranks, later launches until the host clears the word) gives up at once,
// so a collective with a missing peer ends after ONE wait limit whatever its element count.
__device__ __forceinline__ bool comm_peer_timed_out() {
  return (*reinterpret_cast<volatile unsigned*>(&g_mui_dev_status) >> 24) == MUI_DEV_TIMEOUT_PEER;
}

// Polls rank r's cell of element idx until it carries `seq`; returns false (status recorded) on timeout.
__device__ __forceinline__ bool comm_take(const CommDev& c, unsigned long long seq, int r, size_t idx, float* out) {
  const unsigned long long* cell = c.peer_cells[c.rank] + ((size_t)(seq & 1ull) * c.world + r) * c.capacity + idx;
  const unsigned want = static_cast<unsigned>(seq & 0xffffffffull);
  unsigned long long v = ld_relaxed_sys_u64(cell);
  if (static_cast<unsigned>(v >> 32) != want) {
    if (comm_peer_timed_out()) return false;
    const uint64_t t0 = global_timer_ns();
    unsigned spins = 0;
    while (true) {
      v = ld_relaxed_sys_u64(cell);
      if (static_cast<unsigned>(v >> 32) == want) break;
      if ((++spins & 0xff) == 0) {
        if (comm_peer_timed_out()) return false;
        if (global_timer_ns() - t0 > MUI_COMM_WAIT_NS) {
          mui_dev_set_status(MUI_DEV_TIMEOUT_PEER, static_cast<unsigned>(r));
          return false;
        }
      }
    }
  }
  *out = __uint_as_float(static_cast<unsigned>(v & 0xffffffffull));
  return true;
}

// Sum over ranks of element idx in fixed rank order; false if a rank's cell never arrived. The loads of all ranks'
// cells are issued back to back (one L2 round trip for the common case that everything has landed); only cells
// that still carry an older sequence number are polled.
__device__ __forceinline__ bool comm_reduce_elem(const CommDev& c, unsigned long long seq, size_t idx, float* out) {
  const unsigned long long* base = c.peer_cells[c.rank] + (size_t)(seq & 1ull) * c.world * c.capacity + idx;
  const unsigned want = static_cast<unsigned>(seq & 0xffffffffull);
  unsigned long long v[MUI_COMM_MAX_RANKS];
#pragma unroll
  for (int r = 0; r < MUI_COMM_MAX_RANKS; ++r)
    if (r < c.world) v[r] = ld_relaxed_sys_u64(base + (size_t)r * c.capacity);
  float s = 0.f;
  bool ok = true;
#pragma unroll
  for (int r = 0; r < MUI_COMM_MAX_RANKS; ++r) {
    if (r < c.world) {
      float f = __uint_as_float(static_cast<unsigned>(v[r] & 0xffffffffull));
      if (static_cast<unsigned>(v[r] >> 32) != want) {
        f = 0.f;
        ok = comm_take(c, seq, r, idx, &f) && ok;
      }
      s += f;
    }
  }
  *out = s;
  return ok;
}

// Advancing the sequence counter: every CTA of a collective announces itself once (after it has read the counter
// through comm_begin), and the CTA that finds itself last stores the new value. Split in two so that the round trip
// of the atomic overlaps the wait for the peers' cells: thread 0 calls comm_cta_arrive before it polls and
// comm_cta_finish with the returned ticket afterwards.
__device__ __forceinline__ unsigned comm_cta_arrive(const CommDev& c) { return atomicAdd(c.arrive_counter, 1u); }

__device__ __forceinline__ void comm_cta_finish(const CommDev& c, unsigned long long seq, unsigned ticket,
                                                unsigned num_ctas) {
  if (ticket == num_ctas - 1) {
    *c.arrive_counter = 0u;
    *c.local_seq = seq;
  }
}

__device__ __forceinline__ void comm_cta_done(const CommDev& c, unsigned long long seq, unsigned num_ctas) {
  comm_cta_finish(c, seq, comm_cta_arrive(c), num_ctas);
}
