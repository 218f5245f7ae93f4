// Flash attention backward for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// One kernel template, launched twice:
//
//   MODE_DKV  CTA owns 128 keys (TMEM lane = key).  Stationary tiles K, V; streams 64-query tiles
//             (Q_i, dO_i).   S^T = K Q_i^T,  dP^T = V dO_i^T,
//             P^T = exp2(S^T c - L2[q]),  dS^T = P^T (dP^T - delta[q]) scale,
//             dV += P^T dO_i,  dK += dS^T Q_i.
//   MODE_DQ   CTA owns 128 queries (TMEM lane = query).  Stationary tiles Q, dO; streams 64-key
//             tiles (K_j, V_j).   S = Q K_j^T,  dP = dO V_j^T,  dS as above (L2, delta per lane),
//             dQ += dS K_j.
//
// L2 = log2(e) * logsumexp(scale * scores) and delta = rowsum(O * dO) come from the preprocess
// kernel and are padded to a multiple of 128 rows (L2 = +large, delta = 0 in the padding), which
// together with TMA zero-fill removes every boundary mask from the main loops.
//
// Roles: warp 0 TMA producer (a 5-deep ring of streamed tile pairs), warp 1 TMEM allocation + the score
// MMAs, warp 2 the accumulate MMAs, warps 4..7 / 8..11 two compute warpgroups (thread = TMEM lane; warpgroup g owns columns
// [32g, 32g+32) of every 64-column S / dP tile).
//
// The stationary rows never touch shared memory: the compute warps read them from global memory once
// and store them in TMEM as packed bf16 (64 columns per tensor), where they serve as the A operand of
// the score MMAs.  An MMA whose A operand comes from shared memory re-reads 4 KiB of A per
// instruction, which made the [128 x 64 x 16] score MMAs operand-fetch bound (measured ~84 cycles
// each against 32 cycles of math); from TMEM only the 2 KiB B slice is fetched.  The streamed tile in
// shared memory feeds two MMAs through two descriptors: K-major as B of the score GEMMs and MN-major
// as B of the accumulate GEMMs.  P^T / dS are written back to TMEM as packed bf16 over columns
// [32g, 32g+16) of the S / dP tiles and read from there as the A operand of the accumulate MMAs.
//
// TMEM columns:
//   dQ mode:     Q [0,64)  dO [64,128)  buf0 {S [128,192) dP [192,256)}  buf1 {S [256,320) dP [320,384)}  dQ [384,512)
//   dK/dV mode:  K [0,64)  S0 [64,128)  S1 [128,192)  dP [192,256)  dV [256,384)  dK [384,512); V stays in
//                shared memory (its score MMAs take both operands from there) so that S has two buffers:
//                S_j+1 is computed while the compute warpgroups turn S_j into P_j, which shortens the
//                S_j -> P_j -> dV_j chain that otherwise paces this mode
// Every wait is bounded (sm100.cuh).
//
// Replaces the flash_attn / cuDNN SDPA backward used by the reference
// (solar/backends/wan22/runtime/modeling/attention.py:98-135, solar/backends/minimax_h3/fast_attention.py:103).
#include "attn_mask.cuh"
#include "comm.cuh"
#include "host_util.h"
#include "sm100.cuh"

namespace solar {

constexpr int BW_THREADS = 384;
constexpr int ST_ROWS = 128;   // stationary tile rows
constexpr int SR_ROWS = 64;    // streamed tile rows
constexpr int BW_STAGES = 4;

struct AttnBwdParams {
  int S_stat, S_stream, H, B;
  int S_pad;             // padded length of the L2 / delta rows (multiple of 128)
  float scale, scale_log2;
  const float* L2;       // [B, H, S_pad]
  const float* delta;    // [B, H, S_pad]
  int* status;
  const __nv_bfloat16* stat0; long long stat0_ss, stat0_sb;   // stationary tensors (element strides)
  const __nv_bfloat16* stat1; long long stat1_ss, stat1_sb;
  long long* trace;      // optional cycle counters of CTA (0,0,0): see solar_attn_bwd_trace
  int scat_col[2];       // peer scatter: destination column of head 0 for output 0 (dV / dQ) and output 1 (dK)
  AttnMask mask;         // MASKED instantiations: row_ranges are per QUERY; the tile list is over the streamed operand
};

// trace slots (per mode, 8 each): 0 score-warp loop cycles, 1 score-warp wait strm_full, 2 score-warp
// wait s_free/dp_free, 3 compute loop cycles, 4 compute waits, 5 producer wait strm_empty, 6 tiles,
// 7 accumulate-warp wait p_ready/ds_ready
__device__ long long g_bwd_trace[32];

template <int HD>
struct BwdSmem {
  static constexpr int CHUNKS = HD / 64;
  static constexpr int STAT_CHUNK = ST_ROWS * 128;          // 16 KiB
  static constexpr int STAT_TILE = STAT_CHUNK * CHUNKS;
  static constexpr int STRM_CHUNK = SR_ROWS * 128;          // 8 KiB
  static constexpr int STRM_TILE = STRM_CHUNK * CHUNKS;
  static constexpr int STAT_OFF = 0;                        // stat0 | stat1
  static constexpr int STRM_OFF = 2 * STAT_TILE;            // BW_STAGES x (stream0 | stream1)
  static constexpr int BAR_OFF = STRM_OFF + BW_STAGES * 2 * STRM_TILE;
  static constexpr int VEC_OFF = BAR_OFF + 256;             // per compute warp: 32 L2 + 32 delta floats
  static constexpr int MASK_OFF = VEC_OFF + 8 * 64 * 4;     // per compute warp: key ranges of its 32 streamed queries
  static constexpr int TOTAL = MASK_OFF + 8 * 32 * 6 * 4 + 1024;
};

__device__ __forceinline__ void bw_tma_store_4d(const CUtensorMap* m, const void* src, int c0, int c1, int c2,
                                                int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// fp32 accumulator rows (this thread's TMEM lane) -> bf16 -> 128-byte-swizzled staging chunk(s).
template <int NCOLS>
__device__ __forceinline__ void acc_to_smem(uint32_t t_acc, uint8_t* region, int chunk_bytes, int row) {
#pragma unroll
  for (int cc = 0; cc < NCOLS / 32; ++cc) {
    uint32_t r[32];
    tmem_ld_32x32(t_acc + cc * 32, r);
    tmem_ld_wait();
    uint8_t* dst = region + (cc / 2) * chunk_bytes + row * 128;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint4 o;
      o.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
      o.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
      o.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
      o.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
      const int piece = (cc & 1) * 4 + g;
      *reinterpret_cast<uint4*>(dst + ((piece ^ (row & 7)) << 4)) = o;
    }
  }
}

// fp32 accumulator rows (this thread's TMEM lane) -> bf16 -> 16-byte stores to `dst` (NCOLS * 2 contiguous bytes,
// typically a row of another rank's buffer over NVLink).  `dst` is null for rows past the end; the TMEM loads are
// warp-wide and run regardless.
template <int NCOLS>
__device__ __forceinline__ void acc_to_peer(uint32_t t_acc, uint4* dst) {
#pragma unroll
  for (int cc = 0; cc < NCOLS / 32; ++cc) {
    uint32_t r[32];
    tmem_ld_32x32(t_acc + cc * 32, r);
    tmem_ld_wait();
    if (dst != nullptr) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
        o.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
        o.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
        o.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
        dst[cc * 4 + g] = o;
      }
    }
  }
}

// A load the compiler may not sink to its first use: the prefetch below has to leave a whole tile
// ahead of the values being needed.
__device__ __forceinline__ float4 lds_f4_early(const float* ptr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(ptr)));
  return v;
}
__device__ __forceinline__ float ld_f1_early(const float* ptr) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(ptr));
  return v;
}

// MODE 0 = dK/dV, MODE 1 = dQ.  MASKED: structured key ranges per query (attn_mask.cuh).
template <int HD, int MODE, bool MASKED>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmStat1,
                const __grid_constant__ CUtensorMap tmStrm0, const __grid_constant__ CUtensorMap tmStrm1,
                const __grid_constant__ CUtensorMap tmOut0, const __grid_constant__ CUtensorMap tmOut1,
                const AttnBwdParams p, const __grid_constant__ RowScatter rs) {
  using L = BwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* stat_ready = bars;                       // 1 (256 arrivals)
  uint64_t* strm_full = bars + 1;                    // BW_STAGES
  uint64_t* strm_empty = strm_full + BW_STAGES;      // BW_STAGES
  uint64_t* s_ready = strm_empty + BW_STAGES;        // 2
  uint64_t* p_ready = s_ready + 2;                   // 2 (256 arrivals)
  uint64_t* dp_ready = p_ready + 2;                  // 1 (dK/dV mode)
  uint64_t* ds_ready = dp_ready + 1;                 // 1 (dK/dV mode, 256 arrivals)
  uint64_t* s_free = ds_ready + 1;                   // 2 (commit of the accumulate warp)
  uint64_t* dp_free = s_free + 2;                    // 1 (dK/dV mode)
  uint64_t* acc_done = dp_free + 1;                  // 1
  uint64_t* stat_full = acc_done + 1;                // 1 (dK/dV mode: V tile landed in shared memory)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stat_full + 1);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int st_tile = MASKED ? mask_tile_of_cta(p.mask, blockIdx.x) : static_cast<int>(blockIdx.x);
  const int row0 = st_tile * ST_ROWS;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int n_tiles = MASKED ? p.mask.tile_count[st_tile] : (p.S_stream + SR_ROWS - 1) / SR_ROWS;
  const int* tile_list = MASKED ? p.mask.tile_list + static_cast<long long>(st_tile) * p.mask.stride : nullptr;
  // streamed tile visited by iteration j (every tile in order, or this CTA's list under a structured mask)
  auto tile_of = [&](int j) -> int { return MASKED ? (tile_list[j] & (kMaskPartialBit - 1)) : j; };
  const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;

  if (threadIdx.x == 0) {
    mbar_init(stat_ready, 256);
    for (int s = 0; s < BW_STAGES; ++s) {
      mbar_init(&strm_full[s], 1);
      mbar_init(&strm_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_ready[b], 1);
      mbar_init(&p_ready[b], 256);   // both compute warpgroups arrive
    }
    mbar_init(dp_ready, 1);
    mbar_init(ds_ready, 256);
    mbar_init(&s_free[0], 1);
    mbar_init(&s_free[1], 1);
    mbar_init(dp_free, 1);
    mbar_init(acc_done, 1);
    mbar_init(stat_full, 1);
    *abort_word = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmStat1);
    tma_prefetch_desc(&tmStrm0);
    tma_prefetch_desc(&tmStrm1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base_v = *tmem_slot;
  const uint32_t tmem_base = tmem_base_v;
  // TMEM columns of the working tiles (see the header comment)
  constexpr uint32_t COL_STAT1 = 64;                      // dQ mode only (dK/dV keeps V in shared memory)
  constexpr uint32_t COL_ACC0 = MODE == 0 ? 256 : 384;    // dV or dQ
  constexpr uint32_t COL_ACC1 = 384;                      // dK
  // S tile of buffer b (two buffers in both modes) and the dP tile that goes with it
  auto col_S = [](int b) -> uint32_t { return MODE == 0 ? 64u + 64u * b : 128u + 128u * b; };
  auto col_D = [](int b) -> uint32_t { return MODE == 0 ? 192u : 192u + 128u * b; };

  if (warp == 0) {
    // -------------------------------------------------------------- TMA producer (streamed ring)
    setmaxnreg_dec<72>();
    if (lane == 0) {
      long long w_empty = 0;
      if (MODE == 0) {
        mbar_expect_tx(stat_full, L::STAT_TILE);
#pragma unroll
        for (int c = 0; c < L::CHUNKS; ++c)
          tma_load_4d(smem + L::STAT_OFF + L::STAT_TILE + c * L::STAT_CHUNK, &tmStat1, stat_full, c * 64, head, row0, batch);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % BW_STAGES;
        const uint32_t ph = (j / BW_STAGES) & 1;
        const long long c0 = tracing ? clock64() : 0;
        if (!mbar_wait(&strm_empty[s], ph ^ 1, abort_word, ST_TIMEOUT_EMPTY)) break;
        if (tracing) w_empty += clock64() - c0;
        mbar_expect_tx(&strm_full[s], 2 * L::STRM_TILE);
        uint8_t* base = smem + L::STRM_OFF + s * 2 * L::STRM_TILE;
#pragma unroll
        for (int c = 0; c < L::CHUNKS; ++c) {
          tma_load_4d(base + c * L::STRM_CHUNK, &tmStrm0, &strm_full[s], c * 64, head, tile_of(j) * SR_ROWS, batch);
          tma_load_4d(base + L::STRM_TILE + c * L::STRM_CHUNK, &tmStrm1, &strm_full[s], c * 64, head,
                      tile_of(j) * SR_ROWS, batch);
        }
      }
      if (tracing) p.trace[MODE * 8 + 5] = w_empty;
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- score MMA warp
    // Two warps issue tcgen05.mma: warp 1 the score GEMMs (S, dP), warp 2 the accumulate GEMMs, so a
    // wait of one never delays the other's issue; every cross-warp dependency is an mbarrier fed by
    // tcgen05.commit.  The whole warp runs the loop so that addresses and descriptors stay
    // warp-uniform; one elected lane issues each tcgen05 instruction.
    setmaxnreg_dec<72>();
    {
      const bool leader = elect_one();
      const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_base_v, 0);
      constexpr uint32_t idesc_score = umma_idesc_bf16(128, SR_ROWS, 0, 0);   // [128 x 64], K = HD
      const uint32_t strm = __shfl_sync(0xffffffffu, smem_u32(smem + L::STRM_OFF), 0);
      long long w_full = 0, w_free = 0;
      auto wwait = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_word, code));
      };
      // A = stationary rows held in TMEM (packed bf16, 8 columns per K step of 16),
      // B = streamed tile (K-major in shared memory)
      auto score_mma = [&](uint32_t t_dst, uint32_t t_stat, uint32_t s_tile) {
        const uint64_t d0 = umma_desc_kmajor(s_tile);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t ob = (kk / 4) * L::STRM_CHUNK + (kk % 4) * 32;
          if (leader) umma_ts(t_dst, t_stat + kk * 8, d0 + (ob >> 4), idesc_score, kk != 0);
        }
      };
      // dK/dV mode: dP^T = V dO^T reads V from shared memory (A and B both shared-memory descriptors)
      const uint32_t stat1_smem = __shfl_sync(0xffffffffu, smem_u32(smem + L::STAT_OFF + L::STAT_TILE), 0);
      auto score_mma_ss = [&](uint32_t t_dst, uint32_t a_tile, uint32_t s_tile) {
        const uint64_t a0 = umma_desc_kmajor(a_tile), d0 = umma_desc_kmajor(s_tile);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t oa = (kk / 4) * L::STAT_CHUNK + (kk % 4) * 32;
          const uint32_t ob = (kk / 4) * L::STRM_CHUNK + (kk % 4) * 32;
          if (leader) umma_ss(t_dst, a0 + (oa >> 4), d0 + (ob >> 4), idesc_score, kk != 0);
        }
      };
      bool ok = wwait(stat_ready, 0, ST_TIMEOUT_FULL);
      if (ok && MODE == 0) ok = wwait(stat_full, 0, ST_TIMEOUT_FULL);
      tc_fence_after();
      const long long loop0 = tracing ? clock64() : 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % BW_STAGES;
        const int b = j & 1;
        const uint32_t free_par = ((j >> 1) & 1) ^ 1;
        const uint32_t s0 = strm + s * 2 * L::STRM_TILE;
        const uint32_t tS = tmem_base + col_S(b), tD = tmem_base + col_D(b);
        long long c0 = tracing ? clock64() : 0;
        if (!wwait(&strm_full[s], (j / BW_STAGES) & 1, ST_TIMEOUT_FULL)) { ok = false; break; }
        if (tracing) w_full += clock64() - c0;
        c0 = tracing ? clock64() : 0;
        if (!wwait(&s_free[b], free_par, ST_TIMEOUT_OTHER)) { ok = false; break; }   // readers of the old S / P are done
        if (tracing) w_free += clock64() - c0;
        tc_fence_after();
        score_mma(tS, tmem_base, s0);
        if (MODE == 0) {
          if (elect_one()) umma_commit(&s_ready[b]);
          c0 = tracing ? clock64() : 0;
          if (!wwait(dp_free, (j & 1) ^ 1, ST_TIMEOUT_OTHER)) { ok = false; break; }   // readers of the old dP / dS are done
          if (tracing) w_free += clock64() - c0;
          tc_fence_after();
          score_mma_ss(tD, stat1_smem, s0 + L::STRM_TILE);
          if (elect_one()) umma_commit(dp_ready);
        } else {
          score_mma(tD, tmem_base + COL_STAT1, s0 + L::STRM_TILE);
          if (elect_one()) umma_commit(&s_ready[b]);
        }
      }
      if (tracing && lane == 0) {
        p.trace[MODE * 8 + 0] = clock64() - loop0;
        p.trace[MODE * 8 + 1] = w_full;
        p.trace[MODE * 8 + 2] = w_free;
        p.trace[MODE * 8 + 6] = n_tiles;
      }
    }
  } else if (warp == 2) {
    // -------------------------------------------------------------- accumulate MMA warp
    setmaxnreg_dec<72>();
    {
      const bool leader = elect_one();
      const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_base_v, 0);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, 0, 1);          // [128 x HD], K = 64, B MN-major
      const uint32_t strm = __shfl_sync(0xffffffffu, smem_u32(smem + L::STRM_OFF), 0);
      long long w_p = 0;
      auto wwait = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_word, code));
      };
      // A = packed P / dS in TMEM (two 16-column groups, one per compute warpgroup),
      // B = streamed tile read MN-major
      auto acc_mma = [&](uint32_t t_dst, uint32_t t_a, uint32_t s_tile, int t) {
        const uint64_t d0 = umma_desc_mnmajor(s_tile, L::STRM_CHUNK);
#pragma unroll
        for (int kk = 0; kk < SR_ROWS / 16; ++kk)
          if (leader)
            umma_ts(t_dst, t_a + (kk / 2) * 32 + (kk % 2) * 8, d0 + ((kk * 2048) >> 4), idesc_acc, (t | kk) != 0);
      };
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % BW_STAGES;
        const int b = j & 1;
        const uint32_t par = (j >> 1) & 1;
        const uint32_t s0 = strm + s * 2 * L::STRM_TILE;
        const uint32_t tS = tmem_base + col_S(b), tD = tmem_base + col_D(b);
        // the stage was filled before the score MMAs ran; observing its barrier orders this warp after the copy
        if (!wwait(&strm_full[s], (j / BW_STAGES) & 1, ST_TIMEOUT_FULL)) { ok = false; break; }
        long long c0 = tracing ? clock64() : 0;
        if (!wwait(&p_ready[b], par, ST_TIMEOUT_OTHER)) { ok = false; break; }
        if (tracing) w_p += clock64() - c0;
        tc_fence_after();
        if (MODE == 0) {
          acc_mma(tmem_base + COL_ACC0, tS, s0 + L::STRM_TILE, j);          // dV += P^T dO_j
          if (elect_one()) umma_commit(&s_free[b]);
          c0 = tracing ? clock64() : 0;
          if (!wwait(ds_ready, j & 1, ST_TIMEOUT_OTHER)) { ok = false; break; }
          if (tracing) w_p += clock64() - c0;
          tc_fence_after();
          acc_mma(tmem_base + COL_ACC1, tD, s0, j);                          // dK += dS^T Q_j
          if (elect_one()) umma_commit(dp_free);
        } else {
          acc_mma(tmem_base + COL_ACC0, tD, s0, j);                          // dQ += dS K_j
          if (elect_one()) umma_commit(&s_free[b]);
        }
        if (elect_one()) umma_commit(&strm_empty[s]);
      }
      if (ok && elect_one()) umma_commit(acc_done);
      if (tracing && lane == 0) p.trace[MODE * 8 + 7] = w_p;
    }
  } else if (warp == 3) {
    setmaxnreg_dec<72>();
  } else {
    // -------------------------------------------------------------- compute warpgroups
    setmaxnreg_inc<208>();
    const int wg = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const long long vec_base = (static_cast<long long>(batch) * p.H + head) * p.S_pad;
    const float c = p.scale_log2, sc = p.scale;
    // ---- stationary rows: global -> registers -> TMEM as packed bf16 (warpgroup g loads tensor g).
    // Rows past the end are zero; their results are never stored.
    if (MODE == 1 || wg == 0) {
      const __nv_bfloat16* src = wg == 0 ? p.stat0 : p.stat1;
      const long long ss = wg == 0 ? p.stat0_ss : p.stat1_ss, sb = wg == 0 ? p.stat0_sb : p.stat1_sb;
      const int grow = row0 + row;
      const uint4* g4 = reinterpret_cast<const uint4*>(src + batch * sb + static_cast<long long>(grow) * ss +
                                                       static_cast<long long>(head) * HD);
#pragma unroll
      for (int cc = 0; cc < HD / 32; ++cc) {
        uint32_t r[16];
        if (grow < p.S_stat) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint4 v4 = __ldg(g4 + cc * 4 + q4);
            r[q4 * 4 + 0] = v4.x; r[q4 * 4 + 1] = v4.y; r[q4 * 4 + 2] = v4.z; r[q4 * 4 + 3] = v4.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = 0u;
        }
        tmem_st_32x16(tmem_base + lane_off + wg * COL_STAT1 + cc * 16, r);
      }
      tmem_st_wait();
      tc_fence_before();
    }
    mbar_arrive(stat_ready);
    float my_L2 = 0.f, my_delta = 0.f;
    if (MODE == 1) {
      my_L2 = p.L2[vec_base + row0 + row];
      my_delta = p.delta[vec_base + row0 + row];
    }
    bool ok = true;
    long long w_s = 0;
    long long seg[7] = {0, 0, 0, 0, 0, 0, 0};   // ld S | P math | st P + arrive | ld dP | dS math | st dS + arrive
    const long long cloop0 = tracing ? clock64() : 0;
    const float2 c2 = make_float2(c, c), sc2 = make_float2(sc, sc);
    // dK/dV mode: the per-query L2 / delta values of a tile are the same for every thread and change
    // with the tile.  Lane l of every warp fetches element l of the next tile's two vectors a whole tile
    // ahead (two registers); at the start of a tile the warp parks them in its own 256 bytes of shared
    // memory and reads them back as broadcast float4s, so no global-load latency sits inside a tile.
    float* vec_smem = reinterpret_cast<float*>(smem + L::VEC_OFF) + (warp - 4) * 64;
    float nxtL = 0.f, nxtD = 0.f;
    if (MODE == 0) {
      nxtL = __ldg(p.L2 + vec_base + tile_of(0) * SR_ROWS + wg * 32 + lane);
      nxtD = __ldg(p.delta + vec_base + tile_of(0) * SR_ROWS + wg * 32 + lane);
    }
    // structured mask: in dQ mode the thread's row is a query with its own key ranges; in dK/dV mode the thread's row
    // is a key and the ranges of the tile's 32 queries of this warpgroup are parked per warp in shared memory
    int rg[6] = {0, 0, 0, 0, 0, 0};
    int* mask_smem = reinterpret_cast<int*>(smem + L::MASK_OFF) + (warp - 4) * 32 * 6;
    if (MASKED && MODE == 1 && row0 + row < p.S_stat) {
#pragma unroll
      for (int i = 0; i < 6; ++i) rg[i] = __ldg(p.mask.row_ranges + static_cast<long long>(row0 + row) * 6 + i);
    }
    // Both warpgroups work on every streamed tile: warpgroup g owns columns [32g, 32g+32) of the
    // 64-column S / dP tile and writes its packed bf16 results over columns [32g, 32g+16).
    auto tile = [&](const int j) -> bool {
      const int b = j & 1;
      const uint32_t par = (j >> 1) & 1;
      const uint32_t tS = tmem_base + lane_off + col_S(b) + wg * 32, tD = tmem_base + lane_off + col_D(b) + wg * 32;
      // park this tile's vectors and pull them into registers BEFORE waiting for the S tile: the
      // shared-memory round trip hides in the wait instead of stalling the math loops one load at a time
      float4 cL[8], cD[8];
      if (MODE == 0) {
        __syncwarp();                       // the previous tile's reads of the parking area are done
        vec_smem[lane] = -nxtL;             // both vectors are parked negated: the math below only adds them
        vec_smem[32 + lane] = -nxtD;
        __syncwarp();
        if (j + 1 < n_tiles) {
          nxtL = ld_f1_early(p.L2 + vec_base + tile_of(j + 1) * SR_ROWS + wg * 32 + lane);
          nxtD = ld_f1_early(p.delta + vec_base + tile_of(j + 1) * SR_ROWS + wg * 32 + lane);
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          cL[g] = lds_f4_early(vec_smem + 4 * g);
          cD[g] = lds_f4_early(vec_smem + 32 + 4 * g);
        }
      }
      long long c0 = tracing ? clock64() : 0;
      if (!mbar_wait(&s_ready[b], par, abort_word, ST_TIMEOUT_TMEM_FULL)) return false;
      if (tracing) w_s += clock64() - c0;
      tc_fence_after();
      uint32_t s[32], d[32];
      long long q0 = tracing ? clock64() : 0;
      tmem_ld_32x32(tS, s);
      if (MODE == 1) tmem_ld_32x32(tD, d);
      tmem_ld_wait();
      if (tracing) { const long long q1 = clock64(); seg[0] += q1 - q0; q0 = q1; }
      if (tracing) { const long long q1 = clock64(); seg[6] += q1 - q0; q0 = q1; }
      if (MASKED && (tile_list[j] & kMaskPartialBit)) {
        // masked (query, key) pairs get a score of -inf, hence P = 0 and dS = 0
        const int t0 = tile_of(j) * SR_ROWS + wg * 32;          // first streamed index of this warpgroup's columns
        if (MODE == 1) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (!mask_sees(rg, t0 + e)) s[e] = __float_as_uint(-INFINITY);
        } else {
          __syncwarp();
          const int qi = t0 + lane;
#pragma unroll
          for (int i = 0; i < 6; ++i)
            mask_smem[lane * 6 + i] = qi < p.S_stream ? __ldg(p.mask.row_ranges + static_cast<long long>(qi) * 6 + i) : 0;
          __syncwarp();
          const int key = row0 + row;
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            int qr[6];
#pragma unroll
            for (int i = 0; i < 6; ++i) qr[i] = mask_smem[e * 6 + i];
            if (!mask_sees(qr, key)) s[e] = __float_as_uint(-INFINITY);
          }
        }
      }
      uint32_t pk[16], dk[16];
      // P = exp2(S * c - L2); kept as fp32 in s[] for the dS product
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float2 nL[2];
        if (MODE == 0) {
          const float4 a = cL[g];
          nL[0] = make_float2(a.x, a.y); nL[1] = make_float2(a.z, a.w);
        } else {
          nL[0] = nL[1] = make_float2(-my_L2, -my_L2);
        }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const int e = g * 4 + h2 * 2;
          const float2 tt = __ffma2_rn(make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), c2, nL[h2]);
          const float2 pv = make_float2(exp2_fast(tt.x), exp2_fast(tt.y));
          s[e] = __float_as_uint(pv.x); s[e + 1] = __float_as_uint(pv.y);
          pk[e >> 1] = pack_bf16x2(pv.x, pv.y);
        }
      }
      if (tracing) { const long long q1 = clock64(); seg[1] += q1 - q0; q0 = q1; }
      if (MODE == 0) {
        tmem_st_32x16(tS, pk);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_ready[b]);
        if (tracing) { const long long q1 = clock64(); seg[2] += q1 - q0; q0 = q1; }
        c0 = tracing ? clock64() : 0;
        if (!mbar_wait(dp_ready, j & 1, abort_word, ST_TIMEOUT_TMEM_FULL)) return false;
        if (tracing) w_s += clock64() - c0;
        tc_fence_after();
        q0 = tracing ? clock64() : 0;
        tmem_ld_32x32(tD, d);
        tmem_ld_wait();
        if (tracing) { const long long q1 = clock64(); seg[3] += q1 - q0; q0 = q1; }
      }
      // dS = P * (dP - delta) * scale
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float2 nD[2];                        // minus delta
        if (MODE == 0) {
          const float4 bb = cD[g];
          nD[0] = make_float2(bb.x, bb.y); nD[1] = make_float2(bb.z, bb.w);
        } else {
          nD[0] = nD[1] = make_float2(-my_delta, -my_delta);
        }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const int e = g * 4 + h2 * 2;
          const float2 pv = make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1]));
          float2 dd = __fadd2_rn(make_float2(__uint_as_float(d[e]), __uint_as_float(d[e + 1])), nD[h2]);
          dd = __fmul2_rn(__fmul2_rn(pv, dd), sc2);
          dk[e >> 1] = pack_bf16x2(dd.x, dd.y);
        }
      }
      if (tracing) { const long long q1 = clock64(); seg[4] += q1 - q0; q0 = q1; }
      tmem_st_32x16(tD, dk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(MODE == 0 ? ds_ready : &p_ready[b]);
      if (tracing) { const long long q1 = clock64(); seg[5] += q1 - q0; q0 = q1; }
      return true;
    };
#pragma unroll 1
    for (int j = 0; j < n_tiles && ok; ++j) ok = tile(j);
    if (tracing && threadIdx.x == 128) {
      p.trace[MODE * 8 + 3] = clock64() - cloop0;
      p.trace[MODE * 8 + 4] = w_s;
      for (int i = 0; i < 7; ++i) p.trace[16 + MODE * 8 + i] = seg[i];
    }
    // ---- epilogue: accumulators -> bf16 -> shared memory staging -> TMA store
    if (ok) ok = mbar_wait(acc_done, 0, abort_word, ST_TIMEOUT_OTHER);
    if (ok) {
      tc_fence_after();
      if (rs.active()) {
        // Reverse Ulysses exchange fused into the epilogue: every gradient row goes straight to the rank that owns
        // the token, into that rank's [tokens, dq | dk | dv] buffer at this rank's head columns (peer stores over
        // NVLink); nothing is written locally.
        const int grow = row0 + row;
        if (MODE == 0) {
          uint4* dst = grow < p.S_stat
                           ? reinterpret_cast<uint4*>(rs.addr(grow, p.scat_col[wg] + head * HD, 2)) : nullptr;
          acc_to_peer<HD>(tmem_base + lane_off + (wg == 0 ? COL_ACC0 : COL_ACC1), dst);
        } else if (wg < L::CHUNKS) {
          uint4* dst = grow < p.S_stat
                           ? reinterpret_cast<uint4*>(rs.addr(grow, p.scat_col[0] + head * HD + wg * 64, 2)) : nullptr;
          acc_to_peer<64>(tmem_base + lane_off + COL_ACC0 + wg * 64, dst);
        }
      } else if (MODE == 0) {
        // warpgroup 0 drains dV (acc0), warpgroup 1 drains dK (acc1)
        uint8_t* region = smem + L::STAT_OFF + wg * L::STAT_TILE;
        acc_to_smem<HD>(tmem_base + lane_off + (wg == 0 ? COL_ACC0 : COL_ACC1), region, L::STAT_CHUNK, row);
        fence_proxy_async_smem();
        named_bar_sync(1 + wg, 128);
        if (quarter == 0 && lane == 0) {
          const CUtensorMap* out = wg == 0 ? &tmOut0 : &tmOut1;
#pragma unroll
          for (int ch = 0; ch < L::CHUNKS; ++ch)
            bw_tma_store_4d(out, region + ch * L::STAT_CHUNK, ch * 64, head, row0, batch);
          tma_store_commit();
          tma_store_wait_all<0>();
        }
      } else {
        // dQ (acc0): each warpgroup drains one 64-column chunk
        if (wg < L::CHUNKS) {
          uint8_t* region = smem + L::STAT_OFF + wg * L::STAT_CHUNK;
          acc_to_smem<64>(tmem_base + lane_off + COL_ACC0 + wg * 64, region, L::STAT_CHUNK, row);
          fence_proxy_async_smem();
          named_bar_sync(1 + wg, 128);
          if (quarter == 0 && lane == 0) {
            bw_tma_store_4d(&tmOut0, region, wg * 64, head, row0, batch);
            tma_store_commit();
            tma_store_wait_all<0>();
          }
        }
      }
    }
  }

  if (*abort_word != 0) bounded_drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicExch(p.status, *abort_word);
  if (rs.active()) cta_done_signal_peers(rs.flags);
}

// L2[i] = log2(e) * lse[i], delta[i] = sum_d O[i,d] dO[i,d]; rows >= S get (+1e30, 0).
// One warp per row; grid covers B*H*S_pad rows.
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* o, const __nv_bfloat16* dout, const float* lse,
                                     float* L2, float* delta, int B, int S, int H, int D, int S_pad,
                                     long long o_ss, long long o_sb, long long do_ss, long long do_sb) {
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * H * S_pad;
  if (gw >= total) return;
  const int i = static_cast<int>(gw % S_pad);
  const long long bh = gw / S_pad;
  const int h = static_cast<int>(bh % H);
  const int b = static_cast<int>(bh / H);
  if (i >= S) {
    if (lane == 0) { L2[gw] = 1e30f; delta[gw] = 0.f; }
    return;
  }
  const __nv_bfloat16* po = o + b * o_sb + i * o_ss + static_cast<long long>(h) * D;
  const __nv_bfloat16* pd = dout + b * do_sb + i * do_ss + static_cast<long long>(h) * D;
  float acc = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(po + d));
    const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(pd + d));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    delta[gw] = acc;
    L2[gw] = lse[(static_cast<long long>(b) * H + h) * S + i] * 1.4426950408889634f;
  }
}

static int bshd_map(CUtensorMap* m, const void* ptr, int B, int S, int H, int D, long long ss, long long sb,
                    int box_rows) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)ss * 2, (uint64_t)sb * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tmap_4d(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dims, strides, box);
}

template <int HD, int MODE, bool MASKED = false>
static int launch_bwd(const CUtensorMap* maps, const AttnBwdParams& p, cudaStream_t st, const RowScatter& rs) {
  auto kern = attn_bwd_kernel<HD, MODE, MASKED>;
  static PerDeviceOnce configured;   // the attribute is per device
  if (configured.first()) {
    SOLAR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<HD>::TOTAL));
  }
  dim3 grid((p.S_stat + ST_ROWS - 1) / ST_ROWS, p.H, p.B);
  kern<<<grid, BW_THREADS, BwdSmem<HD>::TOTAL, st>>>(maps[1], maps[2], maps[3], maps[4], maps[5], p, rs);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace solar

using namespace solar;

static int g_trace_enabled = 0;
// Profiling aid: with tracing on, CTA (0,0,0) of each backward kernel records cycle counters of its
// roles (how long each waited on which barrier).  `out16` receives the 16 counters of the last call.
extern "C" int solar_attn_bwd_trace(int enable, long long* out16) {
  g_trace_enabled = enable;
  if (out16 != nullptr) SOLAR_CUDA_OK(cudaMemcpyFromSymbol(out16, g_bwd_trace, 32 * sizeof(long long)));
  return 0;
}

// Tail overlap: the dK/dV kernel and the dQ kernel are independent; with the switch on, the dQ kernel is launched
// on a side stream (forked after the row-statistics kernel, joined before the entry returns control of the
// caller's stream), so its CTAs fill the SMs that the last, partly empty wave of the dK/dV kernel leaves idle.
// It matters when a rank owns few heads (sequence parallelism): 642 + 321 CTAs on 148 SMs run as 7 waves
// instead of 5 + 3; it is applied only while the dK/dV grid is under 8 waves.  Off by default for bare callers of
// the C entry; the framework turns it on.
static int g_bwd_overlap = 0;
namespace {
constexpr int kMaxDev = 64;
cudaStream_t g_side_stream[kMaxDev] = {nullptr};
cudaEvent_t g_fork_ev[kMaxDev] = {nullptr}, g_join_ev[kMaxDev] = {nullptr};
int side_stream_for_device(int* dev_out) {
  int dev = 0;
  SOLAR_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDev) return fail("attention backward: device index out of range%s");
  if (g_side_stream[dev] == nullptr) {
    SOLAR_CUDA_OK(cudaStreamCreateWithFlags(&g_side_stream[dev], cudaStreamNonBlocking));
    SOLAR_CUDA_OK(cudaEventCreateWithFlags(&g_fork_ev[dev], cudaEventDisableTiming));
    SOLAR_CUDA_OK(cudaEventCreateWithFlags(&g_join_ev[dev], cudaEventDisableTiming));
  }
  *dev_out = dev;
  return 0;
}
}  // namespace
extern "C" int solar_attn_bwd_overlap(int enable) {
  const int before = g_bwd_overlap;
  if (enable >= 0) g_bwd_overlap = enable ? 1 : 0;
  return before;
}

// Scatter form of the outputs (B == 1): dq / dk / dv rows leave through `rs` into the token owners' buffers; the two
// kernels signal through separate last-CTA counters because they may run at the same time.
struct BwdScatter {
  RowScatter rs;          // flags.local_counter is filled per kernel from counter_dkv / counter_dq
  unsigned* counter_dkv;
  unsigned* counter_dq;
  int col_dq, col_dk, col_dv;   // destination column of head 0 of each gradient
};

static int attn_bwd_impl(const void* q, const void* k, const void* v, const void* o, const void* dout,
                         const float* lse, void* dq, void* dk, void* dv, float* scratch, int B, int Sq, int Sk, int H,
                         int D, long long q_ss, long long q_sb, long long k_ss, long long k_sb, long long v_ss,
                         long long v_sb, long long o_ss, long long o_sb, long long do_ss, long long do_sb, float scale,
                         int* status, void* stream, int allow_overlap, const BwdScatter* scat,
                         const AttnMask* mask_dkv = nullptr, const AttnMask* mask_dq = nullptr) {
  if (D != 64 && D != 128) return fail("attention backward: head_dim must be 64 or 128%s");
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0) return fail("attention backward: empty problem%s");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int Sq_pad = (Sq + 127) / 128 * 128;
  float* L2 = scratch;
  float* delta = scratch + static_cast<long long>(B) * H * Sq_pad;
  {
    const long long warps = static_cast<long long>(B) * H * Sq_pad;
    const int block = 256;
    const long long blocks = (warps * 32 + block - 1) / block;
    attn_bwd_prep_kernel<<<(unsigned)blocks, block, 0, st>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, L2, delta, B, Sq, H, D, Sq_pad, o_ss, o_sb,
        do_ss, do_sb);
    SOLAR_CUDA_OK(cudaGetLastError());
  }
  AttnBwdParams p;
  p.H = H; p.B = B; p.S_pad = Sq_pad;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.L2 = L2; p.delta = delta; p.status = status;
  p.trace = nullptr;
  p.scat_col[0] = p.scat_col[1] = 0;
  memset(&p.mask, 0, sizeof(p.mask));
  const bool masked = mask_dkv != nullptr && mask_dq != nullptr;
  RowScatter rs;
  memset(&rs, 0, sizeof(rs));
  if (scat != nullptr) {
    rs = scat->rs;
    // with peer scatter nothing is stored locally; the output maps only have to be valid
    dq = const_cast<void*>(q); dk = const_cast<void*>(k); dv = const_cast<void*>(v);
  }
  if (g_trace_enabled) SOLAR_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p.trace), g_bwd_trace));
  const long long c_ss = scat != nullptr ? q_ss : static_cast<long long>(H) * D;   // contiguous outputs
  int rc;
  cudaStream_t st_dq = st;
  int dev = -1;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  // only when the dK/dV grid is a few waves deep: with dozens of waves the partial last one costs nothing and
  // two co-scheduled kernels only disturb each other's L2 reuse
  const long long stat_ctas = static_cast<long long>((Sk + ST_ROWS - 1) / ST_ROWS) * H * B;
  const bool few_waves = stat_ctas < 8LL * sm_count();
  const bool overlap = allow_overlap && few_waves;
  if (overlap) SOLAR_CUDA_OK(cudaStreamIsCapturing(st, &capturing));
  if (overlap && capturing == cudaStreamCaptureStatusNone) {
    if ((rc = side_stream_for_device(&dev))) return rc;
    st_dq = g_side_stream[dev];
    SOLAR_CUDA_OK(cudaEventRecord(g_fork_ev[dev], st));            // after the row statistics
    SOLAR_CUDA_OK(cudaStreamWaitEvent(st_dq, g_fork_ev[dev], 0));
  }
  {
    // dK / dV: stationary K, V (128-row boxes); streamed Q, dO (64-row boxes)
    CUtensorMap m[6];
    p.stat0 = (const __nv_bfloat16*)k; p.stat0_ss = k_ss; p.stat0_sb = k_sb;
    p.stat1 = (const __nv_bfloat16*)v; p.stat1_ss = v_ss; p.stat1_sb = v_sb;
    if ((rc = bshd_map(&m[1], v, B, Sk, H, D, v_ss, v_sb, ST_ROWS))) return rc;     // V stays in shared memory
    if ((rc = bshd_map(&m[2], q, B, Sq, H, D, q_ss, q_sb, SR_ROWS))) return rc;
    if ((rc = bshd_map(&m[3], dout, B, Sq, H, D, do_ss, do_sb, SR_ROWS))) return rc;
    if ((rc = bshd_map(&m[4], dv, B, Sk, H, D, c_ss, c_ss * Sk, ST_ROWS))) return rc;
    if ((rc = bshd_map(&m[5], dk, B, Sk, H, D, c_ss, c_ss * Sk, ST_ROWS))) return rc;
    p.S_stat = Sk; p.S_stream = Sq;
    if (scat != nullptr) {
      rs.flags.local_counter = scat->counter_dkv;
      p.scat_col[0] = scat->col_dv;
      p.scat_col[1] = scat->col_dk;
    }
    if (masked) {
      p.mask = *mask_dkv;
      rc = D == 128 ? launch_bwd<128, 0, true>(m, p, st, rs) : launch_bwd<64, 0, true>(m, p, st, rs);
    } else {
      rc = D == 128 ? launch_bwd<128, 0>(m, p, st, rs) : launch_bwd<64, 0>(m, p, st, rs);
    }
    if (rc) return rc;
  }
  {
    // dQ: stationary Q, dO; streamed K, V
    CUtensorMap m[6];
    p.stat0 = (const __nv_bfloat16*)q; p.stat0_ss = q_ss; p.stat0_sb = q_sb;
    p.stat1 = (const __nv_bfloat16*)dout; p.stat1_ss = do_ss; p.stat1_sb = do_sb;
    if ((rc = bshd_map(&m[2], k, B, Sk, H, D, k_ss, k_sb, SR_ROWS))) return rc;
    if ((rc = bshd_map(&m[3], v, B, Sk, H, D, v_ss, v_sb, SR_ROWS))) return rc;
    if ((rc = bshd_map(&m[4], dq, B, Sq, H, D, c_ss, c_ss * Sq, ST_ROWS))) return rc;
    m[5] = m[4];
    m[1] = m[4];   // the stationary-tile map is unused in dQ mode
    p.S_stat = Sq; p.S_stream = Sk;
    if (scat != nullptr) {
      rs.flags.local_counter = scat->counter_dq;
      p.scat_col[0] = scat->col_dq;
      p.scat_col[1] = scat->col_dq;
    }
    if (masked) {
      p.mask = *mask_dq;
      rc = D == 128 ? launch_bwd<128, 1, true>(m, p, st_dq, rs) : launch_bwd<64, 1, true>(m, p, st_dq, rs);
    } else {
      rc = D == 128 ? launch_bwd<128, 1>(m, p, st_dq, rs) : launch_bwd<64, 1>(m, p, st_dq, rs);
    }
    if (st_dq != st) {                                               // join even when the launch failed
      cudaEventRecord(g_join_ev[dev], st_dq);
      cudaStreamWaitEvent(st, g_join_ev[dev], 0);
    }
    if (rc) return rc;
  }
  return 0;
}

// All tensors are [B, S, H, D] bf16 with unit stride on D and stride D on H; *_ss / *_sb are the
// element strides of the sequence and batch axes.  lse [B,H,Sq] fp32 (natural log, from the
// forward kernel).  scratch: 2 * B*H*Sq_pad fp32 of caller-provided memory, Sq_pad = Sq rounded
// up to 128.  Writes dq [B,Sq,H,D], dk and dv [B,Sk,H,D] (contiguous).
extern "C" int solar_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                              const float* lse, void* dq, void* dk, void* dv, float* scratch, int B, int Sq,
                              int Sk, int H, int D, long long q_ss, long long q_sb, long long k_ss,
                              long long k_sb, long long v_ss, long long v_sb, long long o_ss, long long o_sb,
                              long long do_ss, long long do_sb, float scale, int* status, void* stream) {
  return attn_bwd_impl(q, k, v, o, dout, lse, dq, dk, dv, scratch, B, Sq, Sk, H, D, q_ss, q_sb, k_ss, k_sb, v_ss,
                       v_sb, o_ss, o_sb, do_ss, do_sb, scale, status, stream, g_bwd_overlap, nullptr);
}

// Backward under a structured mask (see solar_attn_fwd_masked): row_ranges [Sq][6] are per query; dkv_* lists, for
// every block of 128 keys, the 64-query tiles that see any of them; dq_* lists, for every block of 128 queries, the
// 64-key tiles they see.  Bit 30 of a list entry marks a tile that contains a masked (query, key) pair.
extern "C" int solar_attn_bwd_masked(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                     const float* lse, void* dq, void* dk, void* dv, float* scratch, int B, int Sq,
                                     int Sk, int H, int D, long long q_ss, long long q_sb, long long k_ss,
                                     long long k_sb, long long v_ss, long long v_sb, long long o_ss, long long o_sb,
                                     long long do_ss, long long do_sb, float scale, int* status, void* stream,
                                     const int* row_ranges, const int* dkv_list, const int* dkv_count, int dkv_stride,
                                     const int* dq_list, const int* dq_count, int dq_stride, const int* dkv_order,
                                     const int* dq_order) {
  if (!row_ranges || !dkv_list || !dkv_count || !dq_list || !dq_count || dkv_stride < 1 || dq_stride < 1)
    return fail("masked attention backward: the mask tables are required%s");
  AttnMask mkv{row_ranges, dkv_list, dkv_count, dkv_stride, dkv_order}, mq{row_ranges, dq_list, dq_count, dq_stride, dq_order};
  return attn_bwd_impl(q, k, v, o, dout, lse, dq, dk, dv, scratch, B, Sq, Sk, H, D, q_ss, q_sb, k_ss, k_sb, v_ss,
                       v_sb, o_ss, o_sb, do_ss, do_sb, scale, status, stream, g_bwd_overlap, nullptr, &mkv, &mq);
}

// The same computation with all three kernels on the caller's stream whatever the tail-overlap switch says: no
// side stream or event is ever created on this path.
extern "C" int solar_attn_bwd_serial(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                     const float* lse, void* dq, void* dk, void* dv, float* scratch, int B, int Sq,
                                     int Sk, int H, int D, long long q_ss, long long q_sb, long long k_ss,
                                     long long k_sb, long long v_ss, long long v_sb, long long o_ss, long long o_sb,
                                     long long do_ss, long long do_sb, float scale, int* status, void* stream) {
  return attn_bwd_impl(q, k, v, o, dout, lse, dq, dk, dv, scratch, B, Sq, Sk, H, D, q_ss, q_sb, k_ss, k_sb, v_ss,
                       v_sb, o_ss, o_sb, do_ss, do_sb, scale, status, stream, 0, nullptr);
}

// Attention backward over this rank's heads and the whole sequence (B == 1, Sq == Sk == S) whose gradients are not
// written locally: row i of dq / dk / dv is stored into the buffer of the rank r that owns token i
// (row_start[r] <= i < row_start[r+1]) at local row i - row_start[r], columns col_dq / col_dk / col_dv + head * D
// of a [*, dst_ld] matrix -- the reverse Ulysses exchange fused into the epilogue.  Each of the two kernels adds 1 to
// the flag word on every rank when its last CTA is done (2 signals per rank and call); counter_dkv / counter_dq are
// two zero-initialised local words.  q, k, v share the sequence stride qkv_ss; o [S, H*D] and dout have their own.
extern "C" int solar_attn_bwd_scatter(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                      const float* lse, float* scratch, int S, int H, int D, long long qkv_ss,
                                      long long o_ss, long long do_ss, float scale, int* status, void* stream,
                                      void* const* dst_bases, void* const* flag_ptrs, unsigned* counter_dkv,
                                      unsigned* counter_dq, int n_ranks, long long dst_ld, long long dst_rows,
                                      const int* row_start, int col_dq, int col_dk, int col_dv) {
  if (n_ranks < 1 || n_ranks > kMaxPeers) return fail("attention backward scatter: rank count out of range%s");
  if ((col_dq | col_dk | col_dv) % 8 != 0 || dst_ld % 8 != 0)
    return fail("attention backward scatter: destination columns must be multiples of 8 elements%s");
  BwdScatter sc;
  memset(&sc, 0, sizeof(sc));
  sc.rs.dst.n = n_ranks;
  sc.rs.flags.n = n_ranks;
  for (int i = 0; i < n_ranks; ++i) {
    sc.rs.dst.base[i] = dst_bases[i];
    sc.rs.flags.flag[i] = static_cast<unsigned*>(flag_ptrs[i]);
    sc.rs.row_start[i] = row_start[i];
    if (row_start[i + 1] - row_start[i] > dst_rows || row_start[i + 1] < row_start[i])
      return fail("attention backward scatter: a rank's rows exceed the destination buffer%s");
  }
  sc.rs.row_start[n_ranks] = row_start[n_ranks];
  if (row_start[n_ranks] != S) return fail("attention backward scatter: row ranges must cover the sequence%s");
  sc.rs.ld = dst_ld;
  sc.rs.col_offset = 0;
  sc.counter_dkv = counter_dkv;
  sc.counter_dq = counter_dq;
  sc.col_dq = col_dq; sc.col_dk = col_dk; sc.col_dv = col_dv;
  return attn_bwd_impl(q, k, v, o, dout, lse, nullptr, nullptr, nullptr, scratch, 1, S, S, H, D, qkv_ss, qkv_ss * S,
                       qkv_ss, qkv_ss * S, qkv_ss, qkv_ss * S, o_ss, o_ss * S, do_ss, do_ss * S, scale, status, stream,
                       g_bwd_overlap, &sc);
}
