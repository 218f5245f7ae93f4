// Peer-memory communication runtime for one node of NVLink-connected GPUs (one process per GPU).
//
// Host side: device buffers that every rank of the group can address.  Each rank allocates the
// same layout ("symmetric"), exports a CUDA IPC handle, the handles are exchanged by the Python
// layer over the existing process group, and every rank maps its peers' buffers.  Kernels then
// receive the table of peer base pointers and read/write peers' memory directly over NVLink with
// ordinary global loads/stores (or TMA without cluster qualifiers).
//
// Device side: monotonically increasing 32-bit flags in symmetric memory.
//   producer:  all CTAs of a kernel write their tiles, fence at system scope and bump a local
//              counter; the last CTA adds 1 to the flag word in EVERY rank's memory (release).
//   consumer:  solar_comm_wait enqueues a one-thread kernel that polls the local flag (acquire)
//              until it reaches the expected count, with a wall-clock bound: on timeout it writes a
//              status code and returns, so no stream can hang on a missing peer.
//
// The reference moves the same data with NCCL all_to_all_single / all_gather / all_reduce plus
// packing copies (solar/backends/wan22/runtime/sequence_parallel.py:335-622).
#include "comm.cuh"
#include "host_util.h"
#include "sm100.cuh"

namespace solar {

__global__ void comm_wait_kernel(const unsigned* flag, unsigned expected, int* status, unsigned long long limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    // counters only grow; compare with wrap-around in mind
    if (static_cast<int>(v - expected) >= 0) return;
    if (globaltimer_ns() - t0 > limit_ns) {
      if (status) atomicExch(status, ST_TIMEOUT_PEER);
      return;
    }
    __nanosleep(200);
  }
}

// Round wait whose expected value lives on the device: *epoch += add, then poll until the flag has reached it.
// Nothing in the launch depends on how many rounds came before, so a captured CUDA graph can replay it.
__global__ void comm_wait_round_kernel(const unsigned* flag, unsigned* epoch, unsigned add, int* status,
                                       unsigned long long limit_ns) {
  const unsigned expected = *epoch + add;
  *epoch = expected;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - expected) >= 0) return;
    if (globaltimer_ns() - t0 > limit_ns) {
      if (status) atomicExch(status, ST_TIMEOUT_PEER);
      return;
    }
    __nanosleep(200);
  }
}

// Sum of a few fp32 values over the ranks without a library collective: one CTA stores this rank's `n` values into
// slot `rank` of every peer's [n_ranks, n] table, signals, waits (bounded) for all ranks' signals of this round and
// adds the rows in rank order, so every rank computes the identical sum.  Two tables alternate by round (`parity`
// is read from the epoch word), which keeps a fast rank's next round from overwriting values a slow rank still reads.
__global__ void comm_allsum_kernel(const float* src, int n, PeerTable tables, int rank, PeerFlags flags,
                                   const unsigned* local_flag, unsigned* epoch, float* out, int* status,
                                   unsigned long long limit_ns) {
  __shared__ unsigned s_expected;
  if (threadIdx.x == 0) {
    s_expected = *epoch + static_cast<unsigned>(tables.n);
    *epoch = s_expected;
  }
  __syncthreads();
  const unsigned expected = s_expected;
  const int parity = (expected / static_cast<unsigned>(tables.n)) & 1;
  const long long table_elems = static_cast<long long>(tables.n) * n;
  for (int r = 0; r < tables.n; ++r) {
    float* dst = static_cast<float*>(tables.base[r]) + parity * table_elems + static_cast<long long>(rank) * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    signal_all_peers(flags);
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local_flag) : "memory");
      if (static_cast<int>(v - expected) >= 0) break;
      if (globaltimer_ns() - t0 > limit_ns) {
        if (status) atomicExch(status, ST_TIMEOUT_PEER);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  const volatile float* mine = static_cast<const float*>(tables.base[rank]) + parity * table_elems;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < tables.n; ++r) acc += mine[static_cast<long long>(r) * n + i];
    out[i] = acc;
  }
}

// All-gather by pulling: dst[r * n16 .. (r + 1) * n16) = shard of rank r (16-byte units), read straight from the
// peers' memory over NVLink.  Used to land a block's sharded parameters in local memory ahead of its first GEMM.
__global__ void __launch_bounds__(256) comm_gather_kernel(uint4* __restrict__ dst, PeerTable src, long long n16) {
  const long long total = n16 * src.n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / n16);
    const long long k = i - r * n16;
    dst[i] = static_cast<const uint4*>(src.base[r])[k];
  }
}

// Head exchange of up to three [rows, P * width] matrices (q, k, v after their per-head transforms) as peer stores:
// column block d of every local row goes to rank d, at row `dst_row[t] + r` of that rank's destination t.  The
// destinations may be different buffers with different leading dimensions -- k and v typically land straight in the
// peers' KV caches (an in-place cache append over NVLink), q in an exchange buffer.  The last CTA signals every peer.
struct ScatterColsSeg {
  const uint4* src; long long src_ld16;      // source row stride in 16-byte units
  PeerTable dst; long long dst_ld16; long long dst_row; long long dst_col16;
};
struct ScatterColsParams {
  ScatterColsSeg seg[3];
  int n_seg, n_ranks;
  long long rows;
  int width16;                               // 16-byte units per destination column block
  PeerFlags flags;
};
__global__ void __launch_bounds__(256) comm_scatter_cols_kernel(const __grid_constant__ ScatterColsParams p) {
  const long long per_seg = p.rows * p.n_ranks * p.width16;
  const long long total = per_seg * p.n_seg;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / per_seg);
    long long k = i - t * per_seg;
    const int c = static_cast<int>(k % p.width16);
    k /= p.width16;
    const int d = static_cast<int>(k % p.n_ranks);
    const long long r = k / p.n_ranks;
    const ScatterColsSeg& sg = p.seg[t];
    const uint4 v = sg.src[r * sg.src_ld16 + static_cast<long long>(d) * p.width16 + c];
    static_cast<uint4*>(sg.dst.base[d])[(sg.dst_row + r) * sg.dst_ld16 + sg.dst_col16 + c] = v;
  }
  cta_done_signal_peers(p.flags);
}

__global__ void comm_signal_kernel(PeerFlags flags) {
  if (threadIdx.x == 0 && blockIdx.x == 0) signal_all_peers(flags);
}

// Plain peer copy used by tests and by the all-gather of small vectors: every rank pushes
// `bytes` from src to offset `dst_off` of each peer's buffer, then signals.
__global__ void comm_push_kernel(const uint4* src, PeerTable dst, long long dst_off_bytes, long long n16,
                                 PeerFlags flags) {
  for (int r = 0; r < dst.n; ++r) {
    uint4* out = reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst.base[r]) + dst_off_bytes);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n16;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      out[i] = src[i];
  }
  cta_done_signal_peers(flags);
}

}  // namespace solar

using namespace solar;

extern "C" int solar_comm_alloc(long long bytes, void** out) {
  void* p = nullptr;
  SOLAR_CUDA_OK(cudaMalloc(&p, static_cast<size_t>(bytes)));
  SOLAR_CUDA_OK(cudaMemset(p, 0, static_cast<size_t>(bytes)));
  SOLAR_CUDA_OK(cudaDeviceSynchronize());
  *out = p;
  return 0;
}

extern "C" int solar_comm_free(void* p) {
  SOLAR_CUDA_OK(cudaFree(p));
  return 0;
}

extern "C" int solar_comm_ipc_handle(void* p, unsigned char* out64) {
  cudaIpcMemHandle_t h;
  SOLAR_CUDA_OK(cudaIpcGetMemHandle(&h, p));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out64, &h, 64);
  return 0;
}

extern "C" int solar_comm_ipc_open(const unsigned char* in64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, 64);
  void* p = nullptr;
  SOLAR_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return 0;
}

extern "C" int solar_comm_ipc_close(void* p) {
  SOLAR_CUDA_OK(cudaIpcCloseMemHandle(p));
  return 0;
}

// Same-process peers (tests that drive two GPUs from one process): enable direct access.
extern "C" int solar_comm_enable_peer(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  SOLAR_CUDA_OK(e);
  return 0;
}

extern "C" int solar_comm_wait(const void* flag, unsigned expected, int* status, double limit_seconds, void* stream) {
  const unsigned long long ns = static_cast<unsigned long long>(limit_seconds * 1e9);
  comm_wait_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned*>(flag), expected,
                                                                       status, ns);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// Device-epoch form of solar_comm_wait: `epoch` is a local u32 that the kernel advances by `add` (the number of
// signals one round delivers) before it polls; the launch is replayable inside a CUDA graph.
extern "C" int solar_comm_wait_round(const void* flag, unsigned* epoch, unsigned add, int* status,
                                     double limit_seconds, void* stream) {
  const unsigned long long ns = static_cast<unsigned long long>(limit_seconds * 1e9);
  comm_wait_round_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned*>(flag), epoch,
                                                                             add, status, ns);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

static PeerFlags make_flags(void* const* flag_ptrs, int n, unsigned* counter) {
  PeerFlags f;
  f.n = n;
  for (int i = 0; i < kMaxPeers; ++i) f.flag[i] = i < n ? static_cast<unsigned*>(flag_ptrs[i]) : nullptr;
  f.local_counter = counter;
  return f;
}

extern "C" int solar_comm_signal(void* const* flag_ptrs, int n, void* stream) {
  if (n < 1 || n > kMaxPeers) return fail("comm: peer count out of range%s");
  comm_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_flags(flag_ptrs, n, nullptr));
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// counter: a zero-initialised local u32 the kernel uses to find its last CTA (it resets it).
extern "C" int solar_comm_push(const void* src, void* const* dst_bases, int n, long long dst_off_bytes,
                               long long bytes, void* const* flag_ptrs, unsigned* counter, void* stream) {
  if (n < 1 || n > kMaxPeers) return fail("comm: peer count out of range%s");
  if (bytes % 16 != 0 || dst_off_bytes % 16 != 0) return fail("comm: push size and offset must be multiples of 16%s");
  PeerTable t;
  t.n = n;
  for (int i = 0; i < kMaxPeers; ++i) t.base[i] = i < n ? dst_bases[i] : nullptr;
  const long long n16 = bytes / 16;
  int grid = static_cast<int>((n16 + 255) / 256);
  if (grid > 4 * sm_count()) grid = 4 * sm_count();
  if (grid < 1) grid = 1;
  comm_push_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), t, dst_off_bytes, n16, make_flags(flag_ptrs, n, counter));
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// out[0..n) = sum over ranks of src[0..n) (n <= 256 floats).  table_bases[r]: rank r's [2, n_ranks, n] fp32 table
// in symmetric memory; flag_ptrs[r]: the round's flag word on rank r; epoch: a local u32 (device-side round count).
extern "C" int solar_comm_allsum(const float* src, int n, void* const* table_bases, void* const* flag_ptrs,
                                 int n_ranks, int rank, unsigned* epoch, float* out, int* status,
                                 double limit_seconds, void* stream) {
  if (n_ranks < 1 || n_ranks > kMaxPeers) return fail("comm: peer count out of range%s");
  if (n < 1 || n > 256) return fail("comm allsum: 1..256 values%s");
  if (rank < 0 || rank >= n_ranks) return fail("comm allsum: rank out of range%s");
  PeerTable t;
  t.n = n_ranks;
  for (int i = 0; i < kMaxPeers; ++i) t.base[i] = i < n_ranks ? table_bases[i] : nullptr;
  const unsigned long long ns = static_cast<unsigned long long>(limit_seconds * 1e9);
  comm_allsum_kernel<<<1, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      src, n, t, rank, make_flags(flag_ptrs, n_ranks, nullptr), static_cast<const unsigned*>(flag_ptrs[rank]), epoch,
      out, status, ns);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// dst (local) <- concatenation over ranks of the `shard_bytes` at src_bases[r] (each rank's shard, as mapped here).
extern "C" int solar_comm_gather(void* dst, void* const* src_bases, int n_ranks, long long shard_bytes, int max_ctas,
                                 void* stream) {
  if (n_ranks < 1 || n_ranks > kMaxPeers) return fail("comm: peer count out of range%s");
  if (shard_bytes <= 0 || shard_bytes % 16 != 0) return fail("comm gather: shard size must be a positive multiple of 16%s");
  PeerTable t;
  t.n = n_ranks;
  for (int i = 0; i < kMaxPeers; ++i) t.base[i] = i < n_ranks ? src_bases[i] : nullptr;
  const long long n16 = shard_bytes / 16;
  long long grid = (n16 * n_ranks + 255) / 256;
  const long long cap = max_ctas > 0 ? max_ctas : 4LL * sm_count();
  if (grid > cap) grid = cap;
  comm_gather_kernel<<<(unsigned)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(dst), t, n16);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// n_seg (1..3) matrices src[t] [rows, n_ranks * width] bf16 (row stride src_ld[t] elements): column block d of every
// row is stored at dst_bases[t * n_ranks + d] + ((dst_row[t] + r) * dst_ld[t] + dst_col[t]) elements.  All sizes in
// elements of 2 bytes; width, strides and column offsets must be multiples of 8.  One signal per rank and call.
extern "C" int solar_comm_scatter_cols(int n_seg, const void* const* src, const long long* src_ld, long long rows,
                                       int width, void* const* dst_bases, const long long* dst_ld,
                                       const long long* dst_row, const long long* dst_col, int n_ranks,
                                       void* const* flag_ptrs, unsigned* counter, int max_ctas, void* stream) {
  if (n_seg < 1 || n_seg > 3) return fail("comm scatter: 1..3 matrices%s");
  if (n_ranks < 1 || n_ranks > kMaxPeers) return fail("comm: peer count out of range%s");
  if (rows <= 0 || width <= 0 || width % 8) return fail("comm scatter: width must be a positive multiple of 8%s");
  ScatterColsParams p;
  memset(&p, 0, sizeof(p));
  p.n_seg = n_seg; p.n_ranks = n_ranks; p.rows = rows; p.width16 = width / 8;
  for (int t = 0; t < n_seg; ++t) {
    if (src_ld[t] % 8 || dst_ld[t] % 8 || dst_col[t] % 8 || (reinterpret_cast<uintptr_t>(src[t]) & 15))
      return fail("comm scatter: strides, offsets and pointers must be 16-byte aligned%s");
    p.seg[t].src = static_cast<const uint4*>(src[t]);
    p.seg[t].src_ld16 = src_ld[t] / 8;
    p.seg[t].dst.n = n_ranks;
    for (int d = 0; d < n_ranks; ++d) p.seg[t].dst.base[d] = dst_bases[t * n_ranks + d];
    p.seg[t].dst_ld16 = dst_ld[t] / 8;
    p.seg[t].dst_row = dst_row[t];
    p.seg[t].dst_col16 = dst_col[t] / 8;
  }
  p.flags = make_flags(flag_ptrs, n_ranks, counter);
  const long long total = rows * n_ranks * p.width16 * n_seg;
  long long grid = (total + 255) / 256;
  const long long cap = max_ctas > 0 ? max_ctas : 2LL * sm_count();
  if (grid > cap) grid = cap;
  comm_scatter_cols_kernel<<<(unsigned)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}
