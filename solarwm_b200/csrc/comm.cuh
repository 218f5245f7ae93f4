// Device-side pieces of the peer-memory runtime shared by the fused compute+collective kernels:
// the peer pointer table, the flag table, the "last CTA signals every peer" epilogue and the
// column / row scatter address maps used by the Ulysses exchanges.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace solar {

constexpr int kMaxPeers = 8;

struct PeerTable {
  void* base[kMaxPeers];   // base[r]: the same symmetric buffer as mapped into THIS process for rank r
  int n;
};

struct PeerFlags {
  unsigned* flag[kMaxPeers];   // flag[r]: one u32 in rank r's memory (this rank's slot or a shared counter)
  unsigned* local_counter;     // local u32, zero between kernels; finds the last CTA
  int n;
};

// One thread: add 1 to the flag word on every rank, ordered after all earlier writes of this
// thread and (cumulatively) of every thread it has synchronised with.
__device__ __forceinline__ void signal_all_peers(const PeerFlags& f) {
  __threadfence_system();
  for (int r = 0; r < f.n; ++r)
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(f.flag[r]) : "memory");
}

// Called by every thread of every CTA at the end of a producer kernel.  Each CTA publishes its
// writes (system-scope fence) and bumps the local counter; the CTA that sees the final count
// resets the counter for the next launch and signals all peers once.
__device__ __forceinline__ void cta_done_signal_peers(const PeerFlags& f) {
  if (f.n <= 0) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned prev = atomicAdd(f.local_counter, 1u);
    if (prev == total - 1) {
      __threadfence();
      *f.local_counter = 0;
      signal_all_peers(f);
    }
  }
}

// Column scatter (heads -> ranks): global column `col` of a [rows, groups*group_cols] matrix goes
// to rank (col % group_cols) / cols_per_dest, at local column
// (col / group_cols) * cols_per_dest + (col % group_cols) % cols_per_dest; this rank's rows land
// at row_offset + row in every destination.  With group_cols = dim and cols_per_dest = dim / P a
// fused q|k|v projection arrives as q_local|k_local|v_local per token.
struct ColScatter {
  PeerTable dst;
  PeerFlags flags;
  long long ld;            // destination row stride in elements
  int group_cols;
  int cols_per_dest;
  int row_offset;
  int first_col;           // columns below this one are not scattered (stay local)
  int col_base;            // added to the destination column (separate q / k launches)
  __device__ __forceinline__ bool active() const { return dst.n > 0; }
  __device__ __forceinline__ void* addr(long long row, int col, int elt_bytes) const {
    const int in_group = col % group_cols;
    const int dest = in_group / cols_per_dest;
    const long long lcol = static_cast<long long>(col / group_cols) * cols_per_dest + in_group % cols_per_dest + col_base;
    return static_cast<uint8_t*>(dst.base[dest]) + ((row_offset + row) * ld + lcol) * elt_bytes;
  }
};

// Row scatter (sequence -> ranks): global row `row` of a [S, cols] matrix belongs to the rank whose
// [row_start[r], row_start[r+1]) range contains it and lands at local row row - row_start[r],
// columns shifted by col_offset (this rank's head block inside the full width).
struct RowScatter {
  PeerTable dst;
  PeerFlags flags;
  long long ld;
  int row_start[kMaxPeers + 1];
  int col_offset;
  __device__ __forceinline__ bool active() const { return dst.n > 0; }
  __device__ __forceinline__ int owner(int row) const {
    int r = 0;
#pragma unroll
    for (int i = 1; i < kMaxPeers; ++i)
      if (i < dst.n && row >= row_start[i]) r = i;
    return r;
  }
  __device__ __forceinline__ void* addr(int row, int col, int elt_bytes) const {
    const int r = owner(row);
    return static_cast<uint8_t*>(dst.base[r]) +
           ((static_cast<long long>(row - row_start[r])) * ld + col_offset + col) * elt_bytes;
  }
};

}  // namespace solar
