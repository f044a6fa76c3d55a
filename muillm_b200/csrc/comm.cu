// Tensor-parallel communicator for one node: one process per GPU, symmetric per-rank segments mapped into
// every peer with CUDA IPC, one-shot push all-reduce and broadcast over NVLink / NVSwitch peer stores (see
// comm_dev.cuh for the protocol), and the fused GEMV + all-reduce entry points of the sharded layers.
//
// Stands where the reference has muillm_comm_p2p_t (csrc/comms/comm_p2p.cu: IPC buffer sets, a barrier counter
// in host-pinned memory, a single-CTA read-all-peers reduction in half precision) and its local-socket
// bootstrap (csrc/comms/comm_base.cpp:58-167). Differences by design: flags live in device memory of each rank,
// partial sums travel as fp32 and are added in fixed rank order (bit-identical on all ranks, one rounding),
// every device-side wait is bounded and reports through the device status word, socket waits time out.
#include "gemv_common.cuh"

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <poll.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>
#include <vector>

MUI_STATUS_ACCESSOR(comm)

mui_status_t mui_launch_gemv16(cudaStream_t stream, mui_dtype_t dtype, int mode, const GemvArgs& a, unsigned flags);
mui_status_t mui_parallel_linear_forward_hinted(mui_comm_t* c, void* stream, mui_dtype_t dtype, int B, int N, int K,
                                                const void* norm_weights, float epsilon, const void* weights,
                                                const void* mul_bias, const void* add_bias, const void* residual,
                                                const void* x, void* y, unsigned flags, const GemvHints* hints);

struct mui_comm {
  int rank, world, device;
  size_t capacity;  // fp32 elements per slot
  size_t seg_bytes;
  unsigned char* seg[MUI_COMM_MAX_RANKS];  // seg[rank] is local, the others are IPC mappings
  bool opened[MUI_COMM_MAX_RANKS];
  bool ready;
};

namespace {

constexpr size_t SEG_SEQ_OFF = 0;       // u64 sequence counter (local use only)
constexpr size_t SEG_COUNTER_OFF = 128;  // u32 arrival counter (local use only)
constexpr size_t SEG_DATA_OFF = 4096;    // cells [2][world][capacity] of 8 bytes

size_t seg_size(int world, size_t capacity) { return SEG_DATA_OFF + 2 * (size_t)world * capacity * 8; }

// Device view of the communicator (the same for every collective: the sequence number lives on the device).
void fill_dev(mui_comm* c, CommDev* d) {
  memset(d, 0, sizeof(*d));
  for (int p = 0; p < c->world; ++p)
    d->peer_cells[p] = reinterpret_cast<unsigned long long*>(c->seg[p] + SEG_DATA_OFF);
  unsigned char* me = c->seg[c->rank];
  d->local_seq = reinterpret_cast<unsigned long long*>(me + SEG_SEQ_OFF);
  d->arrive_counter = reinterpret_cast<unsigned int*>(me + SEG_COUNTER_OFF);
  d->world = c->world;
  d->rank = c->rank;
  d->capacity = static_cast<int>(c->capacity);
}

constexpr int AR_THREADS = 256;

template <typename T> struct ArIO {
  static __device__ __forceinline__ float ld(const T* p) { return ld_act_f32<T>(p); }
  static __device__ __forceinline__ void st(T* p, float v) { *p = Elt<T>::from_f32(v); }
};
template <> struct ArIO<float> {
  static __device__ __forceinline__ float ld(const float* p) { return __ldcg(p); }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};

// Stand-alone all-reduce: dst = sum over ranks of src (count elements), same protocol as the fused GEMV tail.
template <typename T>
__global__ void __launch_bounds__(AR_THREADS) allreduce_kernel(const CommDev c, const T* src, T* dst, long long count,
                                                               unsigned long long* trace) {
  trace_start(trace);
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  if (tid == 0) trace_mark(trace, 2, false);
  const unsigned long long seq = comm_begin(c);
  const long long e0 = count * blockIdx.x / gridDim.x, e1 = count * (blockIdx.x + 1) / gridDim.x;
  for (long long i = e0 + tid; i < e1; i += AR_THREADS) comm_push(c, seq, (size_t)i, ArIO<T>::ld(src + i));
  __syncthreads();  // every thread has read the counter before this CTA announces itself
  unsigned ticket = 0;
  if (tid == 0) {
    trace_mark(trace, 4, true);
    ticket = comm_cta_arrive(c);
  }
  for (long long i = e0 + tid; i < e1; i += AR_THREADS) {
    float v;
    if (comm_reduce_elem(c, seq, (size_t)i, &v)) ArIO<T>::st(dst + i, v);
  }
  if (trace != nullptr) {
    __syncthreads();
    if (tid == 0) {
      trace_mark(trace, 5, true);
      trace_mark(trace, 6, false);
      trace_end(trace);
    }
  }
  if (tid == 0) comm_cta_finish(c, seq, ticket, gridDim.x);
}

// Broadcast of `words` 32-bit words from rank `root`: the root pushes the words (as cell payloads), the others
// push one arrival token; every rank polls the root's cells of its own segment and copies them out.
__global__ void __launch_bounds__(AR_THREADS) broadcast_kernel(const CommDev c, int root, const unsigned int* src,
                                                               unsigned int* dst, long long words) {
  pdl_wait_prior_grid();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  const unsigned long long seq = comm_begin(c);
  const long long e0 = words * blockIdx.x / gridDim.x, e1 = words * (blockIdx.x + 1) / gridDim.x;
  if (c.rank == root) {
    for (long long i = e0 + tid; i < e1; i += AR_THREADS)
      comm_push(c, seq, (size_t)i, __uint_as_float(__ldcg(src + i)));
  } else if (blockIdx.x == 0 && tid == 0) {
    comm_push(c, seq, 0, 0.f);  // arrival token in this rank's own slot
  }
  for (long long i = e0 + tid; i < e1; i += AR_THREADS) {
    float v;
    if (comm_take(c, seq, root, (size_t)i, &v)) dst[i] = __float_as_uint(v);
  }
  // every rank also waits for every other rank's token: a rank leaves the collective only when all peers have
  // entered it, which is what lets the next-but-one collective reuse this generation's cells
  if (blockIdx.x == 0 && tid < c.world) {
    float v;
    comm_take(c, seq, tid, 0, &v);
  }
  __syncthreads();
  if (tid == 0) comm_cta_done(c, seq, gridDim.x);
}

}  // namespace

// Device view for other translation units (decode stack).
mui_status_t mui_comm_device_view(mui_comm* c, CommDev* out) {
  MUI_REQUIRE(c != nullptr && out != nullptr, MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(c->ready, MUI_ERR_COMM, "communicator peers are not opened yet");
  fill_dev(c, out);
  return MUI_OK;
}

namespace {

mui_status_t check_ready(mui_comm* c) {
  MUI_REQUIRE(c != nullptr, MUI_ERR_INVALID_ARG, "comm is null");
  MUI_REQUIRE(c->ready, MUI_ERR_COMM, "communicator peers are not opened yet");
  return MUI_OK;
}

// one element per thread up to two CTAs per SM: the collective is a latency chain, not a bandwidth problem
int ar_grid(long long count) {
  return (int)std::max<long long>(1, std::min<long long>(296, (count + AR_THREADS - 1) / AR_THREADS));
}

// ---------------------------------------------------------------------------------------------
// local-socket bootstrap: all-gather of fixed-size blobs between the ranks of one node
// ---------------------------------------------------------------------------------------------
double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

bool io_all(int fd, void* buf, size_t n, bool writing, double deadline) {
  unsigned char* p = reinterpret_cast<unsigned char*>(buf);
  while (n > 0) {
    const double left = deadline - now_s();
    if (left <= 0) return false;
    pollfd pf = {fd, (short)(writing ? POLLOUT : POLLIN), 0};
    const int pr = poll(&pf, 1, (int)(left * 1000) + 1);
    if (pr < 0 && errno == EINTR) continue;
    if (pr <= 0) return false;
    const ssize_t r = writing ? send(fd, p, n, MSG_NOSIGNAL) : recv(fd, p, n, 0);
    if (r < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    if (r <= 0) return false;
    p += r;
    n -= (size_t)r;
  }
  return true;
}

void socket_path(const char* key, sockaddr_un* addr) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  snprintf(addr->sun_path, sizeof(addr->sun_path), "/tmp/muillm_b200_comm_%u_%s", (unsigned)getuid(), key ? key : "0");
}

}  // namespace

extern "C" {

// Rank 0 listens on a UNIX socket derived from `key`; every other rank connects (retrying until the deadline),
// sends {rank, blob}; rank 0 answers each with the table of all blobs. `out` receives world * blob_bytes bytes.
mui_status_t mui_bootstrap_allgather(int rank, int world, const char* key, const void* blob, size_t blob_bytes,
                                     void* out, double timeout_s) {
  MUI_REQUIRE(world >= 1 && world <= 64 && rank >= 0 && rank < world, MUI_ERR_INVALID_ARG, "rank %d of world %d", rank,
              world);
  MUI_REQUIRE(blob && out && blob_bytes > 0 && blob_bytes <= (1u << 20), MUI_ERR_INVALID_ARG, "bad blob");
  unsigned char* table = reinterpret_cast<unsigned char*>(out);
  memcpy(table + (size_t)rank * blob_bytes, blob, blob_bytes);
  if (world == 1) return MUI_OK;
  const double deadline = now_s() + (timeout_s > 0 ? timeout_s : 60.0);
  sockaddr_un addr;
  socket_path(key, &addr);
  if (rank == 0) {
    const int ls = socket(AF_UNIX, SOCK_STREAM, 0);
    MUI_REQUIRE(ls >= 0, MUI_ERR_COMM, "socket() failed: %s", strerror(errno));
    unlink(addr.sun_path);
    if (bind(ls, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || listen(ls, world) != 0) {
      mui_set_error("bind/listen on %s failed: %s", addr.sun_path, strerror(errno));
      close(ls);
      return MUI_ERR_COMM;
    }
    std::vector<int> fds;
    std::vector<bool> seen(world, false);
    bool ok = true;
    while (ok && (int)fds.size() < world - 1) {
      const double left = deadline - now_s();
      pollfd pf = {ls, POLLIN, 0};
      if (left <= 0 || poll(&pf, 1, (int)(left * 1000) + 1) <= 0) {
        mui_set_error("bootstrap: only %zu of %d peers connected before the timeout", fds.size(), world - 1);
        ok = false;
        break;
      }
      const int fd = accept(ls, nullptr, nullptr);
      if (fd < 0) continue;
      int32_t peer = -1;
      if (!io_all(fd, &peer, sizeof(peer), false, deadline) || peer <= 0 || peer >= world || seen[peer] ||
          !io_all(fd, table + (size_t)peer * blob_bytes, blob_bytes, false, deadline)) {
        mui_set_error("bootstrap: bad or truncated hello from a peer (rank field %d)", (int)peer);
        close(fd);
        ok = false;
        break;
      }
      seen[peer] = true;
      fds.push_back(fd);
    }
    for (int fd : fds) {
      if (ok && !io_all(fd, table, (size_t)world * blob_bytes, true, deadline)) {
        mui_set_error("bootstrap: sending the table to a peer failed");
        ok = false;
      }
      close(fd);
    }
    close(ls);
    unlink(addr.sun_path);
    return ok ? MUI_OK : MUI_ERR_COMM;
  }
  // client
  int fd = -1;
  while (true) {
    fd = socket(AF_UNIX, SOCK_STREAM, 0);
    MUI_REQUIRE(fd >= 0, MUI_ERR_COMM, "socket() failed: %s", strerror(errno));
    if (connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) break;
    close(fd);
    if (now_s() > deadline) {
      mui_set_error("bootstrap: rank %d could not reach rank 0 at %s before the timeout", rank, addr.sun_path);
      return MUI_ERR_COMM;
    }
    usleep(20000);
  }
  int32_t me = rank;
  const bool ok = io_all(fd, &me, sizeof(me), true, deadline) &&
                  io_all(fd, const_cast<void*>(blob), blob_bytes, true, deadline) &&
                  io_all(fd, table, (size_t)world * blob_bytes, false, deadline);
  close(fd);
  if (!ok) {
    mui_set_error("bootstrap: rank %d lost the connection to rank 0 or timed out", rank);
    return MUI_ERR_COMM;
  }
  return MUI_OK;
}

size_t mui_comm_ipc_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

mui_status_t mui_comm_create(int rank, int world, size_t capacity_elems, mui_comm_t** out) {
  MUI_REQUIRE(out != nullptr, MUI_ERR_INVALID_ARG, "out is null");
  MUI_REQUIRE(world >= 1 && world <= MUI_COMM_MAX_RANKS && rank >= 0 && rank < world, MUI_ERR_INVALID_ARG,
              "rank %d of world %d (at most %d ranks, one node)", rank, world, MUI_COMM_MAX_RANKS);
  MUI_REQUIRE(capacity_elems >= 1 && capacity_elems <= (1u << 28), MUI_ERR_INVALID_ARG, "capacity %zu", capacity_elems);
  mui_comm* c = new (std::nothrow) mui_comm();
  MUI_REQUIRE(c != nullptr, MUI_ERR_INVALID_ARG, "out of host memory");
  memset(c, 0, sizeof(*c));
  c->rank = rank;
  c->world = world;
  c->capacity = (capacity_elems + 63) & ~(size_t)63;
  c->seg_bytes = seg_size(world, c->capacity);
  cudaError_t e = cudaGetDevice(&c->device);
  void* p = nullptr;
  if (e == cudaSuccess) e = cudaMalloc(&p, c->seg_bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, c->seg_bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    mui_set_error("communicator segment allocation failed: %s", cudaGetErrorString(e));
    if (p) cudaFree(p);
    delete c;
    return MUI_ERR_CUDA;
  }
  c->seg[rank] = reinterpret_cast<unsigned char*>(p);
  c->ready = (world == 1);
  *out = c;
  return MUI_OK;
}

mui_status_t mui_comm_ipc_handle(mui_comm_t* c, void* handle_out) {
  MUI_REQUIRE(c && handle_out, MUI_ERR_INVALID_ARG, "null pointer");
  cudaIpcMemHandle_t h;
  MUI_CUDA_CHECK(cudaIpcGetMemHandle(&h, c->seg[c->rank]));
  memcpy(handle_out, &h, sizeof(h));
  return MUI_OK;
}

mui_status_t mui_comm_open_peers(mui_comm_t* c, const void* handles) {
  MUI_REQUIRE(c && handles, MUI_ERR_INVALID_ARG, "null pointer");
  const unsigned char* hs = reinterpret_cast<const unsigned char*>(handles);
  for (int p = 0; p < c->world; ++p) {
    if (p == c->rank || c->opened[p]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, hs + (size_t)p * sizeof(h), sizeof(h));
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      mui_set_error("cudaIpcOpenMemHandle for rank %d failed: %s", p, cudaGetErrorString(e));
      return MUI_ERR_COMM;
    }
    c->seg[p] = reinterpret_cast<unsigned char*>(ptr);
    c->opened[p] = true;
  }
  c->ready = true;
  return MUI_OK;
}

mui_status_t mui_comm_init_local(int rank, int world, const char* key, size_t capacity_elems, double timeout_s,
                                 mui_comm_t** out) {
  mui_comm_t* c = nullptr;
  mui_status_t s = mui_comm_create(rank, world, capacity_elems, &c);
  if (s != MUI_OK) return s;
  if (world > 1) {
    std::vector<unsigned char> mine(sizeof(cudaIpcMemHandle_t)), all((size_t)world * sizeof(cudaIpcMemHandle_t));
    s = mui_comm_ipc_handle(c, mine.data());
    if (s == MUI_OK) s = mui_bootstrap_allgather(rank, world, key, mine.data(), mine.size(), all.data(), timeout_s);
    if (s == MUI_OK) s = mui_comm_open_peers(c, all.data());
    // second round: nobody starts a collective before every rank has mapped every segment
    unsigned char token = 1;
    std::vector<unsigned char> tokens(world);
    std::string key2 = std::string(key ? key : "0") + "_b";
    if (s == MUI_OK) s = mui_bootstrap_allgather(rank, world, key2.c_str(), &token, 1, tokens.data(), timeout_s);
    if (s != MUI_OK) {
      mui_comm_destroy(c);
      return s;
    }
  }
  *out = c;
  return MUI_OK;
}

mui_status_t mui_comm_destroy(mui_comm_t* c) {
  if (!c) return MUI_OK;
  for (int p = 0; p < c->world; ++p)
    if (p != c->rank && c->opened[p]) cudaIpcCloseMemHandle(c->seg[p]);
  if (c->seg[c->rank]) cudaFree(c->seg[c->rank]);
  delete c;
  return MUI_OK;
}

mui_status_t mui_comm_info(mui_comm_t* c, int* rank, int* world, size_t* capacity_elems) {
  MUI_REQUIRE(c != nullptr, MUI_ERR_INVALID_ARG, "comm is null");
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  if (capacity_elems) *capacity_elems = c->capacity;
  return MUI_OK;
}

mui_status_t mui_comm_all_reduce_sum(mui_comm_t* c, void* stream, int dtype, const void* src, void* dst, size_t count,
                                     unsigned flags) {
  if (mui_status_t s = check_ready(c)) return s;
  MUI_REQUIRE(src && dst, MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE(count <= c->capacity, MUI_ERR_UNSUPPORTED, "count %zu exceeds the communicator capacity %zu", count,
              c->capacity);
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16 || dtype == MUI_COMM_F32, MUI_ERR_UNSUPPORTED, "dtype %d", dtype);
  if (count == 0) return MUI_OK;
  CommDev d;
  fill_dev(c, &d);
  const int pdl = (flags & MUI_FLAG_PDL) ? 1 : 0;
  const dim3 grid(ar_grid((long long)count)), block(AR_THREADS);
  cudaStream_t st = (cudaStream_t)stream;
  unsigned long long* trace = mui_trace_next_record(5);
  if (dtype == MUI_F16) {
    MUI_CUDA_CHECK(mui_launch(allreduce_kernel<__half>, grid, block, 0, st, pdl, d, (const __half*)src, (__half*)dst,
                              (long long)count, trace));
  } else if (dtype == MUI_BF16) {
    MUI_CUDA_CHECK(mui_launch(allreduce_kernel<__nv_bfloat16>, grid, block, 0, st, pdl, d, (const __nv_bfloat16*)src,
                              (__nv_bfloat16*)dst, (long long)count, trace));
  } else {
    MUI_CUDA_CHECK(mui_launch(allreduce_kernel<float>, grid, block, 0, st, pdl, d, (const float*)src, (float*)dst,
                              (long long)count, trace));
  }
  return MUI_OK;
}

mui_status_t mui_comm_broadcast(mui_comm_t* c, void* stream, int root, const void* src, void* dst, size_t bytes,
                                unsigned flags) {
  if (mui_status_t s = check_ready(c)) return s;
  MUI_REQUIRE(root >= 0 && root < c->world, MUI_ERR_INVALID_ARG, "root %d", root);
  MUI_REQUIRE(dst && (c->rank != root || src), MUI_ERR_INVALID_ARG, "null pointer");
  MUI_REQUIRE((bytes & 3) == 0, MUI_ERR_UNSUPPORTED, "broadcast size must be a multiple of 4 bytes");
  MUI_REQUIRE(bytes / 4 <= c->capacity, MUI_ERR_UNSUPPORTED, "broadcast of %zu bytes exceeds the capacity", bytes);
  if (bytes == 0) return MUI_OK;
  CommDev d;
  fill_dev(c, &d);
  const long long words = (long long)(bytes / 4);
  MUI_CUDA_CHECK(mui_launch(broadcast_kernel, dim3(ar_grid(words)), dim3(AR_THREADS), 0, (cudaStream_t)stream,
                            (flags & MUI_FLAG_PDL) ? 1 : 0, d, root, (const unsigned int*)src, (unsigned int*)dst,
                            words));
  return MUI_OK;
}

mui_status_t mui_parallel_linear_forward(mui_comm_t* c, void* stream, mui_dtype_t dtype, int B, int N, int K,
                                         const void* norm_weights, float epsilon, const void* weights,
                                         const void* mul_bias, const void* add_bias, const void* residual,
                                         const void* x, void* y, unsigned flags) {
  return mui_parallel_linear_forward_hinted(c, stream, dtype, B, N, K, norm_weights, epsilon, weights, mul_bias,
                                            add_bias, residual, x, y, flags, nullptr);
}

}  // extern "C"

mui_status_t mui_parallel_linear_forward_hinted(mui_comm_t* c, void* stream, mui_dtype_t dtype, int B, int N, int K,
                                                const void* norm_weights, float epsilon, const void* weights,
                                                const void* mul_bias, const void* add_bias, const void* residual,
                                                const void* x, void* y, unsigned flags, const GemvHints* hints) {
  if (mui_status_t s = check_ready(c)) return s;
  MUI_REQUIRE(dtype == MUI_F16 || dtype == MUI_BF16, MUI_ERR_UNSUPPORTED, "dtype %d unsupported", (int)dtype);
  MUI_REQUIRE(weights && x && y, MUI_ERR_INVALID_ARG, "weights, x and y must be non-null");
  MUI_REQUIRE(B >= 1 && B <= 8, MUI_ERR_UNSUPPORTED, "B=%d outside 1..8", B);
  MUI_REQUIRE(N >= 1 && K >= 1, MUI_ERR_INVALID_ARG, "N=%d, K=%d must be positive", N, K);
  MUI_REQUIRE((size_t)B * N <= c->capacity, MUI_ERR_UNSUPPORTED, "B*N=%zu exceeds the communicator capacity %zu",
              (size_t)B * N, c->capacity);
  MUI_REQUIRE(norm_weights == nullptr, MUI_ERR_UNSUPPORTED,
              "fused normalization is not supported when sharding on dim 1 (K != NORM_K)");
  GemvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = weights;
  a.x = x;
  a.mul_bias = mul_bias;
  // bias and residual enter the sum once: on rank 0 (csrc/parallel_linear_kernels.cu:131-133)
  a.add_bias = (c->rank == 0) ? add_bias : nullptr;
  a.residual = (c->rank == 0) ? residual : nullptr;
  a.y = y;
  a.eps = epsilon;
  a.N = N;
  a.K = K;
  a.B = B;
  a.activ = MUI_ACT_IDENTITY;
  a.Kp = (K + 7) & ~7;
  a.moe_mode = GEMV_MOE_NONE;
  a.slots = 1;
  a.w8_fmt = -1;
  a.use_comm = 1;
  fill_dev(c, &a.comm);
  gemv_apply_hints(a, hints);
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 0, a, flags);
}

extern "C" {

mui_status_t mui_parallel_gateupdown_forward(mui_comm_t* c, void* stream, mui_dtype_t dtype, int B, int I_local, int H,
                                             const void* norm_weights, float epsilon, const void* gate_weights,
                                             const void* up_weights, const void* down_weights, const void* residual,
                                             const void* x, void* scratch_t, void* y, unsigned flags) {
  MUI_REQUIRE(scratch_t != nullptr, MUI_ERR_INVALID_ARG, "scratch_t must be non-null ([B, I_local] elements)");
  mui_status_t s = mui_gateup_silu_forward(stream, dtype, B, I_local, H, norm_weights, epsilon, gate_weights,
                                           up_weights, x, scratch_t, flags);
  if (s != MUI_OK) return s;
  return mui_parallel_linear_forward(c, stream, dtype, B, H, I_local, nullptr, 0.f, down_weights, nullptr, nullptr,
                                     residual, scratch_t, y, flags);
}

mui_status_t mui_parallel_moe_mlp_forward(mui_comm_t* c, void* stream, mui_dtype_t dtype, int num_shared,
                                          int num_routed, int top_k, int I_local, int H, const void* norm_weights,
                                          float epsilon, const void* gate_weights, const void* up_weights,
                                          const void* down_weights, const void* residual, const void* x,
                                          const void* router_scores, const int64_t* router_indices, void* scratch_t,
                                          void* y, unsigned flags) {
  if (mui_status_t s = check_ready(c)) return s;
  MUI_REQUIRE(scratch_t != nullptr, MUI_ERR_INVALID_ARG,
              "scratch_t must be non-null ([num_shared + top_k, I_local] elements)");
  MUI_REQUIRE(down_weights && y, MUI_ERR_INVALID_ARG, "down_weights and y must be non-null");
  MUI_REQUIRE((size_t)H <= c->capacity, MUI_ERR_UNSUPPORTED, "H=%d exceeds the communicator capacity %zu", H,
              c->capacity);
  mui_status_t s = mui_moe_gateup_silu_forward(stream, dtype, num_shared, num_routed, top_k, I_local, H, norm_weights,
                                               epsilon, gate_weights, up_weights, x, router_scores, router_indices,
                                               scratch_t, flags);
  if (s != MUI_OK) return s;
  GemvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = down_weights;
  a.x = scratch_t;
  a.residual = (c->rank == 0) ? residual : nullptr;
  a.y = y;
  a.N = H;
  a.K = I_local;
  a.B = 1;
  a.Kp = (I_local + 7) & ~7;
  a.moe_mode = GEMV_MOE_SEGMENTS;
  a.slots = num_shared + top_k;
  a.num_shared = num_shared;
  a.router_indices = router_indices;
  a.w8_fmt = -1;
  a.use_comm = 1;
  fill_dev(c, &a.comm);
  return mui_launch_gemv16((cudaStream_t)stream, dtype, 0, a, flags);
}

}  // extern "C"
