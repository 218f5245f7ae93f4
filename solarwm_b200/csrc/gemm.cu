// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma
// with fp32 accumulators in TMEM -> tcgen05.ld epilogue -> TMA store.
//
//   C[M,N] (+)= op(A)[M,K] * op(B)[K,N]   (+ bias[N]) (-> GELU-tanh)
//
// Three operand layouts cover a linear layer's forward, data gradient and weight
// gradient without any transposed copy in global memory:
//   NT : A [M,K] row-major (K-major),  B [N,K] row-major (K-major)   y  = x  W^T
//   NN : A [M,K] row-major (K-major),  B [K,N] row-major (MN-major)  dx = dy W
//   TN : A [K,M] row-major (MN-major), B [K,N] row-major (MN-major)  dW = dy^T x
//
// CTA = 6 warps: warp 0 issues TMA loads, warp 1 allocates TMEM and issues the MMAs
// (one elected thread), warps 2..5 drain TMEM (each warp owns the 32 TMEM lanes its
// rank-in-warpgroup may touch) and store through shared memory with TMA.  Two 256-column
// accumulators double-buffer the epilogue against the next tile's main loop.
//
// Replaces the cuBLAS calls behind every nn.Linear of the reference models
// (reference: solar/backends/wan22/runtime/modeling/model.py:112-147, 230-233).
#include "comm.cuh"
#include "host_util.h"
#include "sm100.cuh"

namespace solar {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;              // 16 KiB
constexpr int B_BYTES = BN * BK * 2;              // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;    // 48 KiB
constexpr int EPI_WARPS = 4;
constexpr int EPI_BUF_BYTES = 32 * 128;           // one warp, 32 rows x 128 B
constexpr int EPI_BYTES = EPI_WARPS * 2 * EPI_BUF_BYTES;  // 32 KiB
constexpr int SMEM_MAIN = STAGES * STAGE_BYTES + EPI_BYTES;
constexpr int SMEM_TOTAL = SMEM_MAIN + 256 + 1024;  // barriers + alignment slack
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;

// Implicit-GEMM convolution on channels-last activations [T, H, W, C]: a 128-row tile of the "A" operand is a
// 16 x 8 pixel box of one frame, fetched by ONE 4-D TMA load per (tap, 64-channel block) at the box origin
// shifted by the tap's (dt, dh, dw); positions outside the tensor read zeros (the spatial "same" padding and
// the causal temporal padding need no padded copy).  The K loop runs over taps x channel blocks against
// weights stored [Cout, taps * kb_per_tap * 64].  The epilogue stores each warp's 2 x 16 pixels with a 4-D TMA
// store, which clips at the frame border.
constexpr int CONV_BOX_W = 16, CONV_BOX_H = 8;
struct ConvPlan {
  int taps;                 // 0: plain GEMM
  int kb_per_tap;
  int tiles_w, tiles_h;
  signed char dt[28], dh[28], dw[28];
};

struct GemmParams {
  ConvPlan conv;
  int ntile;                  // output columns per tile of the single-CTA kernel: BN, or 128 for narrow outputs
  int M, N, K;
  int tiles_m, tiles_n;
  const __nv_bfloat16* bias;  // [N] or null
  int act;                    // 0 none, 1 gelu-tanh
  int accumulate;             // 1: C += result (TMA reduce-add)
  int* status;                // device status word (0 = ok)
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // Groups of 8 M-tiles sweep N together so that the CTAs running at the same time share
  // A and B tiles in L2.
  constexpr int G = 8;
  const int per_group = G * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * G;
  const int rows = min(G, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

// Drain one accumulator tile: this warp's 32 TMEM lanes (rows row0 .. row0+31 of C) x BN columns starting at
// column n0 -> bias / activation -> staged through shared memory -> TMA store, reduce-add or peer scatter.
template <int OUT_F32>
__device__ __forceinline__ void epilogue_tile(const CUtensorMap& tmC, const GemmParams& p, const ColScatter& sc,
                                              uint32_t t_row, int row0, int n0, uint8_t* my_buf, int& buf, int lane,
                                              int cw = 0, int ch = 0, int ct = 0, int ncols = BN) {
  constexpr int CHUNK = OUT_F32 ? 32 : 64;  // columns per 128-byte staged row
  const bool rows_live = (row0) < p.M;
  // act 2 (SwiGLU, bf16 output): the weight rows are interleaved in blocks of 64 (64 gate rows, their 64 up rows,
  // ...), so 128 accumulator columns make 64 output columns = one staged row, stored at half the column offset
  const bool swiglu = !OUT_F32 && p.act == 2;
  const int step = swiglu ? 2 * CHUNK : CHUNK;
#pragma unroll 1
  for (int c0 = 0; c0 < ncols; c0 += step) {
    const int ncol = n0 + c0;
    if (ncol >= p.N) break;
    if (lane == 0) tma_store_wait_read<1>();
    __syncwarp();
    uint8_t* dst = my_buf + buf * EPI_BUF_BYTES + lane * 128;
    if (OUT_F32) {
      uint32_t r[32];
      tmem_ld_32x32(t_row + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = __uint_as_float(r[g * 4 + e]);
        if (p.bias != nullptr && ncol + g * 4 < p.N) {
          const uint2 bb = *reinterpret_cast<const uint2*>(p.bias + ncol + g * 4);
          const float2 b01 = unpack_bf16x2(bb.x), b23 = unpack_bf16x2(bb.y);
          v[0] += b01.x; v[1] += b01.y; v[2] += b23.x; v[3] += b23.y;
        }
        if (p.act == 1) {
#pragma unroll
          for (int e = 0; e < 4; ++e) v[e] = gelu_tanh(v[e]);
        }
        uint4 o = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]),
                             __float_as_uint(v[2]), __float_as_uint(v[3]));
        *reinterpret_cast<uint4*>(dst + ((g ^ (lane & 7)) << 4)) = o;
      }
    } else if (swiglu) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t rg[32], ru[32];
        tmem_ld_32x32(t_row + c0 + 32 * h, rg);          // 32 gate columns
        tmem_ld_32x32(t_row + c0 + 64 + 32 * h, ru);     // their 32 up columns
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float a[8], u[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            a[e] = __uint_as_float(rg[g * 8 + e]);
            u[e] = __uint_as_float(ru[g * 8 + e]);
          }
          if (p.bias != nullptr) {
            const uint4 ba = *reinterpret_cast<const uint4*>(p.bias + ncol + 32 * h + g * 8);
            const uint4 bu = *reinterpret_cast<const uint4*>(p.bias + ncol + 64 + 32 * h + g * 8);
            const uint32_t wa[4] = {ba.x, ba.y, ba.z, ba.w}, wu[4] = {bu.x, bu.y, bu.z, bu.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 fa = unpack_bf16x2(wa[e]), fu = unpack_bf16x2(wu[e]);
              a[2 * e] += fa.x; a[2 * e + 1] += fa.y;
              u[2 * e] += fu.x; u[2 * e + 1] += fu.y;
            }
          }
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = a[e] / (1.f + __expf(-a[e])) * u[e];
          uint4 o = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                               pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
          const int piece = 4 * h + g;
          *reinterpret_cast<uint4*>(dst + ((piece ^ (lane & 7)) << 4)) = o;
        }
      }
    } else {
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(t_row + c0, r0);
      tmem_ld_32x32(t_row + c0 + 32, r1);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
          v[e] = __uint_as_float(g < 4 ? r0[g * 8 + e] : r1[(g - 4) * 8 + e]);
        if (p.bias != nullptr && ncol + g * 8 < p.N) {
          const uint4 bb = *reinterpret_cast<const uint4*>(p.bias + ncol + g * 8);
          const float2 b0 = unpack_bf16x2(bb.x), b1 = unpack_bf16x2(bb.y),
                       b2 = unpack_bf16x2(bb.z), b3 = unpack_bf16x2(bb.w);
          v[0] += b0.x; v[1] += b0.y; v[2] += b1.x; v[3] += b1.y;
          v[4] += b2.x; v[5] += b2.y; v[6] += b3.x; v[7] += b3.y;
        }
        if (p.act == 1) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]);
        }
        uint4 o = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                             pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
        *reinterpret_cast<uint4*>(dst + ((g ^ (lane & 7)) << 4)) = o;
      }
    }
    if (!OUT_F32 && sc.active() && ncol >= sc.first_col) {
      // Ulysses scatter: this 64-column chunk belongs to one head, hence to one rank.  The
      // thread owns one output row; it copies its 128 staged bytes straight into the owning
      // rank's receive buffer over NVLink (the staging pass above already applied the epilogue).
      __syncwarp();
      const int grow = row0 + lane;
      if (grow < p.M) {
        uint4* out = reinterpret_cast<uint4*>(sc.addr(grow, ncol, 2));
#pragma unroll
        for (int g = 0; g < 8; ++g) out[g] = *reinterpret_cast<const uint4*>(dst + ((g ^ (lane & 7)) << 4));
      }
      __syncwarp();
      if (lane == 0) tma_store_commit();   // empty group: keeps the two-deep staging count aligned
      buf ^= 1;
      continue;
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && rows_live) {
      const void* src = my_buf + buf * EPI_BUF_BYTES;
      if (p.conv.taps != 0) {
        tma_store_4d(&tmC, src, ncol, cw, ch, ct);   // this warp's 2 x 16 pixels x 64 channels
      } else if (p.accumulate) {
        asm volatile(
            "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::
                "l"(reinterpret_cast<uint64_t>(&tmC)),
            "r"(smem_u32(src)), "r"(ncol), "r"(row0)
            : "memory");
      } else {
        tma_store_2d(&tmC, src, swiglu ? (ncol >> 1) : ncol, row0);
      }
      tma_store_commit();
    }
    buf ^= 1;
  }
}

template <int A_MN, int B_MN, int OUT_F32>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p,
                 const __grid_constant__ ColScatter sc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SMEM_MAIN);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], EPI_WARPS * 32);
    }
    *abort_word = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * p.ntile;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full_bar[stage], A_BYTES + p.ntile * BK * 2);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (64 * BK * 2), &tmA, &full_bar[stage], m0 + c * 64, k0);
          } else if (p.conv.taps != 0) {
            const int tap = kb / p.conv.kb_per_tap;
            const int tw = tm % p.conv.tiles_w, rest = tm / p.conv.tiles_w;
            const int th = rest % p.conv.tiles_h, tt = rest / p.conv.tiles_h;
            tma_load_4d(sa, &tmA, &full_bar[stage], (kb - tap * p.conv.kb_per_tap) * BK,
                        tw * CONV_BOX_W + p.conv.dw[tap], th * CONV_BOX_H + p.conv.dh[tap], tt + p.conv.dt[tap]);
          } else {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < p.ntile / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &tmB, &full_bar[stage], n0 + c * 64, k0);
          } else {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Every lane runs the loop (warp-uniform addresses and descriptors); one elected lane issues.
    {
      const bool leader = elect_one();   // one lane issues; elected once, not per instruction
      auto wwait = [&](uint64_t* bar, uint32_t parity, volatile int* aw, int code) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, aw, code));
      };
      const uint32_t smem_base = __shfl_sync(0xffffffffu, smem_u32(smem), 0);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t idesc = umma_idesc_bf16(BM, p.ntile, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!wwait(&tempty_bar[acc], acc_phase ^ 1, abort_word, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_u + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wwait(&full_bar[stage], phase, abort_word, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t adesc = A_MN ? umma_desc_mnmajor(sa + kk * 2048, 64 * BK * 2)
                                        : umma_desc_kmajor(sa + kk * 32);
            const uint64_t bdesc = B_MN ? umma_desc_mnmajor(sb + kk * 2048, 64 * BK * 2)
                                        : umma_desc_kmajor(sb + kk * 32);
            if (leader) umma_ss(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0);
          }
          if (elect_one()) umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && elect_one()) umma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint8_t* my_buf = epi_smem + (warp - 2) * 2 * EPI_BUF_BYTES;
    int local = 0;
    int buf = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * BM, n0 = tn * p.ntile;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_word, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (p.conv.taps != 0) {
        const int tw = tm % p.conv.tiles_w, rest = tm / p.conv.tiles_w;
        const int th = rest % p.conv.tiles_h, tt = rest / p.conv.tiles_h;
        epilogue_tile<OUT_F32>(tmC, p, sc, t_row, 0, n0, my_buf, buf, lane, tw * CONV_BOX_W,
                               th * CONV_BOX_H + q * 2, tt, p.ntile);
      } else {
        epilogue_tile<OUT_F32>(tmC, p, sc, t_row, m0 + q * 32, n0, my_buf, buf, lane, 0, 0, 0, p.ntile);
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_word != 0) bounded_drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicExch(p.status, *abort_word);
  if (sc.active()) cta_done_signal_peers(sc.flags);
}

template <int A_MN, int B_MN, int OUT_F32>
static int launch_gemm(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC,
                       const GemmParams& p, int max_ctas, cudaStream_t stream, const ColScatter& sc) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, OUT_F32>;
  static PerDeviceOnce configured;   // the attribute is per device
  if (configured.first()) {
    SOLAR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
  }
  int grid = p.tiles_m * p.tiles_n;
  int cap = max_ctas > 0 ? max_ctas : sm_count();
  if (grid > cap) grid = cap;
  kern<<<grid, GEMM_THREADS, SMEM_TOTAL, stream>>>(tA, tB, tC, p, sc);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}


// ---------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): a cluster of two CTAs computes a 256 x 256 tile.  Each CTA loads
// its own 128 rows of A and only HALF of the B tile (128 of the 256 columns) -- the tensor core of
// either SM reads the other half from the partner's shared memory -- and keeps its 128 x 256 half
// of the accumulator in its own TMEM.  Per MMA step a CTA now stages 32 KiB instead of 48 KiB, which
// lifts the shared-memory operand bandwidth limit of the single-CTA kernel, and one instruction
// issue drives two SMs.  The pair leader (cluster rank 0) issues every MMA; completion is
// committed to the barriers of both CTAs; both CTAs' TMA loads credit the leader's "full" barrier.
// ---------------------------------------------------------------------------------------------
constexpr int P_BN_HALF = BN / 2;                       // B columns staged per CTA
constexpr int P_B_BYTES = P_BN_HALF * BK * 2;           // 16 KiB
constexpr int P_STAGE_BYTES = A_BYTES + P_B_BYTES;      // 32 KiB
constexpr int P_STAGES = 6;
constexpr int P_SMEM_MAIN = P_STAGES * P_STAGE_BYTES + EPI_BYTES;
constexpr int P_SMEM_TOTAL = P_SMEM_MAIN + 256 + 1024;

template <int A_MN, int B_MN, int OUT_F32>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const GemmParams p,
                      const __grid_constant__ ColScatter sc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + P_STAGES * P_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + P_SMEM_MAIN);   // used in the leader only
  uint64_t* empty_bar = full_bar + P_STAGES;                              // one set per CTA
  uint64_t* tfull_bar = empty_bar + P_STAGES;                             // one set per CTA
  uint64_t* tempty_bar = tfull_bar + 2;                                   // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();            // 0 = leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;        // tiles_m counts 256-row tiles here
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * EPI_WARPS * 32);   // the epilogue threads of both CTAs
    }
    *abort_word = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();          // barriers of both CTAs are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM;
        const int half = p.ntile >> 1;                                     // B columns staged per CTA
        const int nb0 = tn * p.ntile + static_cast<int>(rank) * half;      // this CTA's half of the B tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * P_STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t full_leader = mapa_u32(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * (A_BYTES + half * BK * 2));   // both CTAs' bytes
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sa + c * (64 * BK * 2), &tmA, full_leader, m0 + c * 64, k0);
          } else {
            tma_load_2d_pair(sa, &tmA, full_leader, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < half / 64; ++c)
              tma_load_2d_pair(sb + c * (64 * BK * 2), &tmB, full_leader, nb0 + c * 64, k0);
          } else {
            tma_load_2d_pair(sb, &tmB, full_leader, k0, nb0);
          }
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0) {
      const bool leader = elect_one();
      auto wwait = [&](uint64_t* bar, uint32_t parity, volatile int* aw, int code) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, aw, code));
      };
      const uint32_t smem_base = __shfl_sync(0xffffffffu, smem_u32(smem), 0);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t bar_base = __shfl_sync(0xffffffffu, smem_u32(full_bar), 0);
      const uint32_t bar_peer = mapa_u32(bar_base, 1);
      // a barrier of this CTA and the same barrier of the partner
      auto commit_both = [&](uint64_t* bar) {
        const uint32_t off = smem_u32(bar) - bar_base;
        if (leader) {
          umma_commit_pair(bar_base + off);
          umma_commit_pair(bar_peer + off);
        }
      };
      const uint32_t idesc = umma_idesc_bf16(2 * BM, p.ntile, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!wwait(&tempty_bar[acc], acc_phase ^ 1, abort_word, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_u + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wwait(&full_bar[stage], phase, abort_word, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t adesc = A_MN ? umma_desc_mnmajor(sa + kk * 2048, 64 * BK * 2)
                                        : umma_desc_kmajor(sa + kk * 32);
            const uint64_t bdesc = B_MN ? umma_desc_mnmajor(sb + kk * 2048, 64 * BK * 2)
                                        : umma_desc_kmajor(sb + kk * 32);
            if (leader) umma_ss_pair(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0);
          }
          commit_both(&empty_bar[stage]);
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) commit_both(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, both CTAs)
    const int q = warp & 3;
    uint8_t* my_buf = epi_smem + (warp - 2) * 2 * EPI_BUF_BYTES;
    const uint32_t tempty_leader = mapa_u32(smem_u32(tempty_bar), 0);
    int local = 0;
    int buf = 0;
    for (int tile = pair; tile < num_tiles; tile += n_pairs, ++local) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM, n0 = tn * p.ntile;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_word, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      epilogue_tile<OUT_F32>(tmC, p, sc, t_row, m0 + q * 32, n0, my_buf, buf, lane, 0, 0, 0, p.ntile);
      tc_fence_before();
      mbar_arrive_cluster(tempty_leader + acc * 8);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_word != 0) bounded_drain_pause();
  tc_fence_before();
  cluster_sync_all();          // the partner's shared memory and TMEM stay alive until both are done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicExch(p.status, *abort_word);
  if (sc.active()) cta_done_signal_peers(sc.flags);
}

template <int A_MN, int B_MN, int OUT_F32>
static int launch_gemm_pair(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC,
                            const GemmParams& p, int max_ctas, cudaStream_t stream, const ColScatter& sc) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, OUT_F32>;
  static PerDeviceOnce configured;   // the attribute is per device
  if (configured.first()) {
    SOLAR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_TOTAL));
  }
  int pairs = p.tiles_m * p.tiles_n;
  const int cap = (max_ctas > 0 ? max_ctas : sm_count()) / 2;
  if (pairs > cap) pairs = cap;
  if (pairs < 1) pairs = 1;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM_TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  // clusters that cannot be co-resident would start only after others finish and unbalance the persistent loop
  static int max_clusters = 0;
  if (max_clusters == 0) {
    SOLAR_CUDA_OK(cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg));
    if (max_clusters < 1) return fail("gemm pair: no cluster of two CTAs can be resident%s");
  }
  if (pairs > max_clusters) {
    pairs = max_clusters;
    cfg.gridDim = dim3(2 * pairs, 1, 1);
  }
  SOLAR_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tA, tB, tC, p, sc));
  return 0;
}

}  // namespace solar

using namespace solar;

// layout: 0 = NT, 1 = NN, 2 = TN (see the header comment).  lda/ldb/ldc are leading
// dimensions in elements of the row-major arrays as they sit in memory.
// out_f32: C is fp32 instead of bf16.  accumulate: C += (atomic-free TMA reduce-add).
// status: optional device int that receives a non-zero code if a bounded wait gave up.
// -1: choose per problem; 0: single-CTA kernel with 256-column tiles only; 1: CTA-pair kernel whenever legal;
// 2: single-CTA kernel with 192-column tiles, 3: CTA-pair kernel with 128-column tiles (for measurements).
static int g_pair_mode = -1;
extern "C" int solar_gemm_pair_mode(int mode) {
  const int old = g_pair_mode;
  if (mode >= -1 && mode <= 3) g_pair_mode = mode;
  return old;
}

// Tile shape per problem.  Both kernels are persistent with one tile (or CTA-pair tile) in flight per SM, so a
// problem costs ceil(tiles / slots) waves of its tile time.  With few tiles the last wave is mostly empty: a
// [3410 x 3072] product -- the out-projection and FFN-down shapes of 8-way sequence parallelism -- is 168 pair tiles
// over 74 pairs, 2.27 waves that cost 3 (measured: 1,232 TFLOP/s where the same kernel reaches 1,570 on full waves).
// Narrower tiles do NOT recover that; measured on the ten GEMMs of a Wan-5B block at 3,410 / 6,820 / 13,640 rows
// (sum of the ten, ms): pair 256 x 256 1.90 / 3.49 / 6.74; pair 256 x 128 (modes 3) 2.59 / 4.92 / 10.25; one CTA
// 128 x 256 and 128 x 192 (modes 0, 2) 15-25 % behind the pair kernel on every shape.  So the choice is only between
// the pair kernel and, for problems too small to fill the machine with pairs, the single-CTA kernel; the other
// shapes stay selectable for measurements (`kernel_bench tiles`).
struct TileChoice {
  bool pair;
  int ntile;
};
static TileChoice choose_tiles(int M, int N, int act) {
  const int sms = sm_count();
  auto cdiv = [](long long a, long long b) { return (a + b - 1) / b; };
  if (g_pair_mode == 1) return {true, BN};
  if (g_pair_mode == 0) return {false, BN};
  if (g_pair_mode == 2) return {false, act == 2 ? BN : 192};
  if (g_pair_mode == 3) return {true, 128};
  return {cdiv(M, 2 * BM) * cdiv(N, BN) >= sms / 2, BN};
}

static int gemm_entry(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                      long long ldb, long long ldc, int layout, int act, int out_f32, int accumulate, int* status,
                      int max_ctas, void* stream, const ColScatter& sc) {
  if (M <= 0 || N <= 0 || K <= 0) return fail("gemm: empty problem%s");
  if (N % 8 != 0) return fail("gemm: N must be a multiple of 8%s");
  if (layout < 0 || layout > 2) return fail("gemm: bad layout%s");
  if (act == 2 && (out_f32 || accumulate || sc.dst.n != 0 || N % 128 != 0))
    return fail("gemm: the SwiGLU epilogue takes bf16 output, no accumulate, no scatter, N a multiple of 128%s");
  CUtensorMap tA, tB, tC;
  int rc;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (layout == 2) {  // A stored [K, M]
    rc = make_tmap_2d(&tA, A, bf, 2, K, M, lda, BK, 64);
  } else {            // A stored [M, K]
    rc = make_tmap_2d(&tA, A, bf, 2, M, K, lda, BM, BK);
  }
  if (rc) return rc;
  // CTA pairs pay off once there are enough 256-row tiles to fill the machine; small problems stay on the
  // single-CTA kernel.  (The scatter epilogue and its last-CTA signalling are per CTA and work in both.)
  const TileChoice choice = choose_tiles(M, N, act);
  const bool use_pair = choice.pair;
  if (layout == 0) {  // B stored [N, K]
    rc = make_tmap_2d(&tB, B, bf, 2, N, K, ldb, use_pair ? choice.ntile / 2 : choice.ntile, BK);
  } else {            // B stored [K, N]
    rc = make_tmap_2d(&tB, B, bf, 2, K, N, ldb, BK, 64);
  }
  if (rc) return rc;
  if (out_f32) {
    rc = make_tmap_2d(&tC, C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, 32);
  } else {
    rc = make_tmap_2d(&tC, C, bf, 2, M, act == 2 ? N / 2 : N, ldc, 32, 64);
  }
  if (rc) return rc;
  GemmParams p;
  memset(&p.conv, 0, sizeof(p.conv));
  p.ntile = choice.ntile;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = use_pair ? (M + 2 * BM - 1) / (2 * BM) : (M + BM - 1) / BM;
  p.tiles_n = (N + choice.ntile - 1) / choice.ntile;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.act = act;
  p.accumulate = accumulate;
  p.status = status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (use_pair) {
    switch (layout * 2 + (out_f32 ? 1 : 0)) {
      case 0: return launch_gemm_pair<0, 0, 0>(tA, tB, tC, p, max_ctas, st, sc);
      case 1: return launch_gemm_pair<0, 0, 1>(tA, tB, tC, p, max_ctas, st, sc);
      case 2: return launch_gemm_pair<0, 1, 0>(tA, tB, tC, p, max_ctas, st, sc);
      case 3: return launch_gemm_pair<0, 1, 1>(tA, tB, tC, p, max_ctas, st, sc);
      case 4: return launch_gemm_pair<1, 1, 0>(tA, tB, tC, p, max_ctas, st, sc);
      default: return launch_gemm_pair<1, 1, 1>(tA, tB, tC, p, max_ctas, st, sc);
    }
  }
  switch (layout * 2 + (out_f32 ? 1 : 0)) {
    case 0: return launch_gemm<0, 0, 0>(tA, tB, tC, p, max_ctas, st, sc);
    case 1: return launch_gemm<0, 0, 1>(tA, tB, tC, p, max_ctas, st, sc);
    case 2: return launch_gemm<0, 1, 0>(tA, tB, tC, p, max_ctas, st, sc);
    case 3: return launch_gemm<0, 1, 1>(tA, tB, tC, p, max_ctas, st, sc);
    case 4: return launch_gemm<1, 1, 0>(tA, tB, tC, p, max_ctas, st, sc);
    default: return launch_gemm<1, 1, 1>(tA, tB, tC, p, max_ctas, st, sc);
  }
}

extern "C" int solar_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N,
                               int K, long long lda, long long ldb, long long ldc, int layout,
                               int act, int out_f32, int accumulate, int* status, int max_ctas,
                               void* stream) {
  ColScatter none;
  memset(&none, 0, sizeof(none));
  return gemm_entry(A, B, C, bias, M, N, K, lda, ldb, ldc, layout, act, out_f32, accumulate, status, max_ctas,
                    stream, none);
}

// GEMM whose output columns >= first_col leave through the Ulysses column scatter: every
// 64-column chunk is written by the epilogue warps straight into the owning rank's receive
// buffer (peer stores over NVLink), columns below first_col go to C as usual, and the last CTA
// bumps the flag word on every rank.  dst_bases / flag_ptrs: n_ranks pointers each; counter: a
// zeroed local u32.  Destination row stride dst_ld (elements); this rank's rows start at
// row_offset in every destination.
extern "C" int solar_gemm_bf16_scatter(const void* A, const void* B, void* C, const void* bias, int M, int N,
                                       int K, long long lda, long long ldb, long long ldc, int layout, int act,
                                       int* status, int max_ctas, void* stream, void* const* dst_bases,
                                       void* const* flag_ptrs, unsigned* counter, int n_ranks, long long dst_ld,
                                       int group_cols, int cols_per_dest, int row_offset, int first_col,
                                       int col_base) {
  if (n_ranks < 1 || n_ranks > kMaxPeers) return fail("gemm scatter: rank count out of range%s");
  if (cols_per_dest % 64 != 0 || group_cols % cols_per_dest != 0 || first_col % 64 != 0)
    return fail("gemm scatter: column blocks must be multiples of 64%s");
  ColScatter sc;
  memset(&sc, 0, sizeof(sc));
  sc.dst.n = n_ranks;
  sc.flags.n = n_ranks;
  for (int i = 0; i < n_ranks; ++i) {
    sc.dst.base[i] = dst_bases[i];
    sc.flags.flag[i] = static_cast<unsigned*>(flag_ptrs[i]);
  }
  sc.flags.local_counter = counter;
  sc.ld = dst_ld;
  sc.group_cols = group_cols;
  sc.cols_per_dest = cols_per_dest;
  sc.row_offset = row_offset;
  sc.first_col = first_col;
  sc.col_base = col_base;
  return gemm_entry(A, B, C, bias, M, N, K, lda, ldb, ldc, layout, act, 0, 0, status, max_ctas, stream, sc);
}

// Stride-1 convolution over channels-last bf16 activations, "same" padding in H and W, causal in T:
//   x [Tin, H, W, Cin]   w [Cout, taps * kb_per_tap * 64] (tap-major, each tap's Cin zero-padded to 64s)
//   y [Tout, H, W, Cout] = conv(x) + bias;  output frame t reads input frames t + t_shift + (0 .. kt-1)
// (t_shift = -(kt-1) with Tin == Tout: zero history; t_shift = 0 with Tin == Tout + kt - 1: the history frames
// lead the input).  Cin and Cout must be multiples of 8.
extern "C" int solar_conv3d_bf16(const void* x, const void* w, void* y, const void* bias, int Tin, int H, int W,
                                 int Cin, int Tout, int Cout, int kt, int kh, int kw, int t_shift, int* status,
                                 int max_ctas, void* stream) {
  if (Tin <= 0 || Tout <= 0 || H <= 0 || W <= 0) return fail("conv3d: empty problem%s");
  if (Cin % 8 != 0 || Cout % 8 != 0) return fail("conv3d: channel counts must be multiples of 8%s");
  if (kt < 1 || kh < 1 || kw < 1 || kt * kh * kw > 27 || kh % 2 == 0 || kw % 2 == 0)
    return fail("conv3d: kernel must be odd in H / W and have at most 27 taps%s");
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  GemmParams p;
  memset(&p.conv, 0, sizeof(p.conv));
  p.conv.taps = kt * kh * kw;
  p.conv.kb_per_tap = (Cin + BK - 1) / BK;
  p.conv.tiles_w = (W + CONV_BOX_W - 1) / CONV_BOX_W;
  p.conv.tiles_h = (H + CONV_BOX_H - 1) / CONV_BOX_H;
  int tap = 0;
  for (int a = 0; a < kt; ++a)
    for (int b = 0; b < kh; ++b)
      for (int c = 0; c < kw; ++c, ++tap) {
        p.conv.dt[tap] = static_cast<signed char>(a + t_shift);
        p.conv.dh[tap] = static_cast<signed char>(b - kh / 2);
        p.conv.dw[tap] = static_cast<signed char>(c - kw / 2);
      }
  const int K = p.conv.taps * p.conv.kb_per_tap * BK;
  CUtensorMap tA, tB, tC;
  const uint64_t da[4] = {(uint64_t)Cin, (uint64_t)W, (uint64_t)H, (uint64_t)Tin};
  const uint64_t sa[3] = {(uint64_t)Cin * 2, (uint64_t)W * Cin * 2, (uint64_t)H * W * Cin * 2};
  const uint32_t ba[4] = {BK, CONV_BOX_W, CONV_BOX_H, 1};
  int rc = make_tmap_4d(&tA, x, bf, da, sa, ba);
  if (rc) return rc;
  p.ntile = Cout <= 128 ? 128 : BN;      // narrow outputs: a 128-column tile wastes no MMA columns
  rc = make_tmap_2d(&tB, w, bf, 2, Cout, K, K, p.ntile, BK);
  if (rc) return rc;
  const uint64_t dc[4] = {(uint64_t)Cout, (uint64_t)W, (uint64_t)H, (uint64_t)Tout};
  const uint64_t sc4[3] = {(uint64_t)Cout * 2, (uint64_t)W * Cout * 2, (uint64_t)H * W * Cout * 2};
  const uint32_t bc[4] = {64, CONV_BOX_W, 2, 1};
  rc = make_tmap_4d(&tC, y, bf, dc, sc4, bc);
  if (rc) return rc;
  p.tiles_m = Tout * p.conv.tiles_h * p.conv.tiles_w;
  p.tiles_n = (Cout + p.ntile - 1) / p.ntile;
  p.M = p.tiles_m * BM; p.N = Cout; p.K = K;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.act = 0; p.accumulate = 0; p.status = status;
  ColScatter none;
  memset(&none, 0, sizeof(none));
  return launch_gemm<0, 0, 0>(tA, tB, tC, p, max_ctas, reinterpret_cast<cudaStream_t>(stream), none);
}

extern "C" const char* solar_last_error() { return last_error_buf(); }
