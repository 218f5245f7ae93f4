// Flash attention forward for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
//   O[b, i, h, :] = softmax_j(scale * Q[b,i,h,:] . K[b,j,h,:]) V[b,j,h,:]      (bidirectional)
//
// One CTA owns 256 consecutive queries of one (batch, head): two 128-row Q tiles that
// ping-pong so the tensor pipe works on one tile while the softmax warps work on the other.
//
//   warp 0        TMA producer: Q tiles once, then a 2-deep ring of K tiles and a 2-deep ring of
//                 V tiles (128 keys x head_dim each, 128-byte swizzle, no cluster qualifiers)
//   warp 1        allocates TMEM and issues every tcgen05.mma:
//                   S_t = Q_t K_j^T   (both operands from shared memory, K-major)
//                   O_t += P_t V_j    (P from TMEM as bf16, V from shared memory, MN-major)
//   warps 4..7    softmax for Q tile 0 (one thread per query row, TMEM lane = row)
//   warps 8..11   softmax for Q tile 1
//
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t overwrites the
// first 64 columns of S_t as packed bf16 pairs.  The running maximum is only raised (and O
// rescaled in TMEM by the softmax warps) when it would grow by more than 2^8, so the rescale is
// rare; the final O / l division makes the result exact either way.
//
// Every wait is bounded (sm100.cuh); on a timeout the CTA drains, frees TMEM, reports a status.
//
// Replaces flash_attn_varlen_func / SDPA on the reference's attention path
// (solar/backends/wan22/runtime/modeling/attention.py:34-188).
#include "attn_mask.cuh"
#include "comm.cuh"
#include "host_util.h"
#include "sm100.cuh"

namespace solar {

constexpr int ATT_THREADS = 384;
constexpr int QT = 128;    // rows per Q tile
constexpr int KT = 128;    // keys per KV tile
constexpr int KV_STAGES = 2;

struct AttnParams {
  int Sq, Sk, H, B;
  float scale_log2;   // scale * log2(e)
  float scale;
  float* lse;         // [B, H, Sq] natural-log sum-exp of the scaled scores (may be null)
  int* status;
  AttnMask mask;      // used by the MASKED instantiation only
};

template <int HD>
struct AttnSmem {
  static constexpr int CHUNKS = HD / 64;                 // 64-element (128-byte) column chunks
  static constexpr int TILE_BYTES = 128 * HD * 2;        // one Q / K / V tile
  static constexpr int CHUNK_BYTES = 128 * 128;          // 128 rows x 128 bytes
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = 2 * TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int BAR_OFF = V_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int HD, bool MASKED>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                const AttnParams p, const __grid_constant__ RowScatter rs) {
  using L = AttnSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // KV_STAGES
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_ready = v_empty + KV_STAGES; // 2
  uint64_t* p_ready = s_ready + 2;         // 2
  uint64_t* o_done = p_ready + 2;          // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_tile = MASKED ? mask_tile_of_cta(p.mask, blockIdx.x) : static_cast<int>(blockIdx.x);
  const int q0 = q_tile * (2 * QT);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int n_kv = MASKED ? p.mask.tile_count[q_tile] : (p.Sk + KT - 1) / KT;
  const int* kv_list = MASKED ? p.mask.tile_list + static_cast<long long>(q_tile) * p.mask.stride : nullptr;
  // KV tile visited by iteration j (all tiles in order, or the CTA's list under a structured mask)
  auto kv_tile = [&](int j) -> int { return MASKED ? (kv_list[j] & (kMaskPartialBit - 1)) : j; };
  // the second Q tile may be entirely past the end of the sequence
  const bool tile1_live = (q0 + QT) < p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_ready[t], 1);
      mbar_init(&p_ready[t], 128);
      mbar_init(&o_done[t], 1);
    }
    *abort_word = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t TS[2] = {tmem_base + 0, tmem_base + 128};
  const uint32_t TO[2] = {tmem_base + 256, tmem_base + 384};

  if (warp == 0) {
    // -------------------------------------------------------------- TMA producer
    setmaxnreg_dec<72>();
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * L::TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < L::CHUNKS; ++c)
          tma_load_4d(smem + L::Q_OFF + t * L::TILE_BYTES + c * L::CHUNK_BYTES, &tmQ, q_full, c * 64, head,
                      q0 + t * QT, batch);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_word, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&k_full[s], L::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < L::CHUNKS; ++c)
          tma_load_4d(smem + L::K_OFF + s * L::TILE_BYTES + c * L::CHUNK_BYTES, &tmK, &k_full[s], c * 64, head,
                      kv_tile(j) * KT, batch);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_word, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&v_full[s], L::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < L::CHUNKS; ++c)
          tma_load_4d(smem + L::V_OFF + s * L::TILE_BYTES + c * L::CHUNK_BYTES, &tmV, &v_full[s], c * 64, head,
                      kv_tile(j) * KT, batch);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop so that addresses and descriptors stay warp-uniform (an issue loop
    // confined to one lane computes them per thread and pays a register-file crossing per operand,
    // which made instruction issue the bottleneck); one elected lane issues each tcgen05 instruction.
    setmaxnreg_dec<72>();
    {
      const bool leader = elect_one();   // one lane issues; elected once, not per instruction
      auto wwait = [&](uint64_t* bar, uint32_t parity, volatile int* aw, int code) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, aw, code));
      };
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, KT, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, HD, 0, 1);
      const uint32_t q_smem = __shfl_sync(0xffffffffu, smem_u32(smem + L::Q_OFF), 0);
      const uint32_t k_smem = __shfl_sync(0xffffffffu, smem_u32(smem + L::K_OFF), 0);
      const uint32_t v_smem = __shfl_sync(0xffffffffu, smem_u32(smem + L::V_OFF), 0);
      auto issue_qk = [&](int t, int s) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * L::CHUNK_BYTES + (kk % 4) * 32;
          if (leader) umma_ss(TS[t], umma_desc_kmajor(q_smem + t * L::TILE_BYTES + off),
                  umma_desc_kmajor(k_smem + s * L::TILE_BYTES + off), idesc_qk, kk != 0);
        }
        if (elect_one()) umma_commit(&s_ready[t]);
      };
      auto issue_pv = [&](int t, int s, int j) {
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          if (leader) umma_ts(TO[t], TS[t] + kk * 8,
                  umma_desc_mnmajor(v_smem + s * L::TILE_BYTES + kk * 2048, L::CHUNK_BYTES), idesc_pv,
                  (j | kk) != 0);
        }
        if (elect_one()) umma_commit(&o_done[t]);
      };
      bool ok = wwait(q_full, 0, abort_word, ST_TIMEOUT_FULL);
      if (ok) ok = wwait(&k_full[0], 0, abort_word, ST_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        if (tile1_live) issue_qk(1, 0);
        if (elect_one()) umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const int sn = (j + 1) % KV_STAGES;
        const uint32_t phn = ((j + 1) / KV_STAGES) & 1;
        const bool more = (j + 1) < n_kv;
        if (!wwait(&v_full[s], ph, abort_word, ST_TIMEOUT_FULL)) break;
        // ---- tile 0
        if (!wwait(&p_ready[0], j & 1, abort_word, ST_TIMEOUT_OTHER)) break;
        tc_fence_after();
        issue_pv(0, s, j);
        if (more) {
          if (!wwait(&k_full[sn], phn, abort_word, ST_TIMEOUT_FULL)) break;
          tc_fence_after();
          issue_qk(0, sn);
        }
        // ---- tile 1
        if (tile1_live) {
          if (!wwait(&p_ready[1], j & 1, abort_word, ST_TIMEOUT_OTHER)) break;
          tc_fence_after();
          issue_pv(1, s, j);
        }
        if (elect_one()) umma_commit(&v_empty[s]);
        if (more) {
          if (tile1_live) issue_qk(1, sn);
          if (elect_one()) umma_commit(&k_empty[sn]);
        }
      }
    }
  } else if (warp < 4) {
    setmaxnreg_dec<72>();                       // idle warps of the producer warpgroup release registers too
  } else {
    // -------------------------------------------------------------- softmax (2 x 4 warps)
    setmaxnreg_inc<208>();
    const int t = (warp - 4) >> 2;              // Q tile of this warpgroup
    const int quarter = warp & 3;               // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;        // row inside the Q tile
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = TS[t] + lane_off, tO = TO[t] + lane_off;
    const bool live = (t == 0) || tile1_live;
    float m_used = -INFINITY, l = 0.f;
    const float c = p.scale_log2;
    bool ok = live;
    // this row's key ranges (structured mask); rows past the end see nothing and are never stored
    int rg[6] = {0, 0, 0, 0, 0, 0};
    if (MASKED) {
      const int qrow = q0 + t * QT + row;
      if (qrow < p.Sq) {
#pragma unroll
        for (int i = 0; i < 6; ++i) rg[i] = __ldg(p.mask.row_ranges + static_cast<long long>(qrow) * 6 + i);
      }
    }
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait(&s_ready[t], j & 1, abort_word, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = kv_tile(j) * KT;
      const int kv_valid = p.Sk - k0;           // >= 128 except on the last tile
      // the whole 128-score row of this thread in registers: four loads in flight, one wait
      uint32_t s[128];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) tmem_ld_32x32_at(tS + cc * 32, s + cc * 32);
      tmem_ld_wait();
      if (kv_valid < KT) {
#pragma unroll
        for (int e = 0; e < 128; ++e)
          if (e >= kv_valid) s[e] = __float_as_uint(-INFINITY);
      }
      if (MASKED && (kv_list[j] & kMaskPartialBit)) {
        // some row of the CTA sees this tile only in part: rows that one of their ranges covers whole skip the work
        const int k1 = min(k0 + KT, p.Sk);
        const bool whole = (rg[0] <= k0 && k1 <= rg[1]) || (rg[2] <= k0 && k1 <= rg[3]) || (rg[4] <= k0 && k1 <= rg[5]);
        if (!whole) {
#pragma unroll
          for (int e = 0; e < 128; ++e) {
            if (!mask_sees(rg, k0 + e)) s[e] = __float_as_uint(-INFINITY);
          }
        }
      }
      float mx = fmaxf(__uint_as_float(s[0]), __uint_as_float(s[1]));
#pragma unroll
      for (int e = 2; e < 128; e += 2) mx = max3f(mx, __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
      if (j == 0) {
        m_used = mx;
      } else {
        const float m_new = fmaxf(m_used, mx);
        const bool need = (m_new - m_used) * c > 8.0f;
        if (__any_sync(0xffffffffu, need)) {
          // O_t of the previous KV tile must have landed before it is rescaled in place
          if (!mbar_wait(&o_done[t], (j - 1) & 1, abort_word, ST_TIMEOUT_OTHER)) { ok = false; break; }
          tc_fence_after();
          const float f = need ? exp2_fast((m_used - m_new) * c) : 1.0f;
          if (need) m_used = m_new;
          l *= f;
#pragma unroll
          for (int cc = 0; cc < HD / 32; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(tO + cc * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * f);
            tmem_st_32x32(tO + cc * 32, r);
          }
          tmem_st_wait();
        }
      }
      // P = exp2(s * c - m * c) with packed fp32x2 arithmetic, bf16 pairs over the first 64 columns of S_t
      const float2 c2 = make_float2(c, c);
      // a row that has seen no key yet keeps m = -inf; its scores are all -inf and must give P = 0, not NaN
      const float m_exp = (MASKED && m_used == -INFINITY) ? 0.f : m_used;
      const float2 n2 = make_float2(-m_exp * c, -m_exp * c);
      float2 l2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int e = 0; e < 64; ++e) {
        const float2 tt = __ffma2_rn(make_float2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1])), c2, n2);
        // every other pair takes the FMA-pipe exponential so that MUFU and FMA pipes share the load
        const float2 pp = ((e & 3) == 3) ? exp2_poly2(tt) : make_float2(exp2_fast(tt.x), exp2_fast(tt.y));
        l2 = __fadd2_rn(l2, pp);
        s[e] = pack_bf16x2(pp.x, pp.y);
      }
      l += l2.x + l2.y;
      tmem_st_32x32_at(tS, s);
      tmem_st_32x32_at(tS + 32, s + 32);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[t]);
    }
    // ---- epilogue: O / l -> bf16 -> shared memory (the tile's Q buffer) -> TMA store
    if (ok) ok = mbar_wait(&o_done[t], (n_kv - 1) & 1, abort_word, ST_TIMEOUT_OTHER);
    if (ok) {
      tc_fence_after();
      const float inv_l = (MASKED && !(l > 0.f)) ? 0.f : 1.0f / l;
      uint8_t* obuf = smem + L::Q_OFF + t * L::TILE_BYTES;
#pragma unroll
      for (int cc = 0; cc < HD / 32; ++cc) {
        uint32_t r[32];
        tmem_ld_32x32(tO + cc * 32, r);
        tmem_ld_wait();
        uint8_t* dst = obuf + (cc / 2) * L::CHUNK_BYTES + row * 128;
        // Ulysses gather of the attention output: the row also goes straight to the rank that owns
        // this token, into the column block of this rank's heads (peer stores over NVLink).
        uint4* remote = nullptr;
        if (rs.active() && (q0 + t * QT + row) < p.Sq)
          remote = reinterpret_cast<uint4*>(rs.addr(q0 + t * QT + row, head * HD + cc * 32, 2));
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]) * inv_l, __uint_as_float(r[g * 8 + 1]) * inv_l);
          o.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]) * inv_l, __uint_as_float(r[g * 8 + 3]) * inv_l);
          o.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]) * inv_l, __uint_as_float(r[g * 8 + 5]) * inv_l);
          o.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]) * inv_l, __uint_as_float(r[g * 8 + 7]) * inv_l);
          const int piece = (cc & 1) * 4 + g;  // 16-byte piece inside the 128-byte row
          *reinterpret_cast<uint4*>(dst + ((piece ^ (row & 7)) << 4)) = o;
          if (remote != nullptr) remote[g] = o;
        }
      }
      const int qrow = q0 + t * QT + row;
      if (p.lse != nullptr && qrow < p.Sq)
        p.lse[(static_cast<long long>(batch) * p.H + head) * p.Sq + qrow] = m_used * p.scale + __logf(l);
      fence_proxy_async_smem();
      named_bar_sync(1 + t, 128);
      if (quarter == 0 && lane == 0) {
#pragma unroll
        for (int ch = 0; ch < L::CHUNKS; ++ch)
          tma_store_4d(&tmO, obuf + ch * L::CHUNK_BYTES, ch * 64, head, q0 + t * QT, batch);
        tma_store_commit();
        tma_store_wait_all<0>();
      }
    }
  }

  // ---------------------------------------------------------------- teardown
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

template <int HD, bool MASKED>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const CUtensorMap& to, const AttnParams& p, cudaStream_t st, const RowScatter& rs) {
  auto kern = attn_fwd_kernel<HD, MASKED>;
  static PerDeviceOnce configured;   // the attribute is per device
  if (configured.first()) {
    SOLAR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<HD>::TOTAL));
  }
  dim3 grid((p.Sq + 2 * QT - 1) / (2 * QT), p.H, p.B);
  kern<<<grid, ATT_THREADS, AttnSmem<HD>::TOTAL, st>>>(tq, tk, tv, to, p, rs);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

static int make_bshd_map(CUtensorMap* m, const void* ptr, int B, int S, int H, int D, long long stride_s,
                         long long stride_b) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)stride_s * 2, (uint64_t)stride_b * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_4d(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dims, strides, box);
}

}  // namespace solar

using namespace solar;

// q [B,Sq,H,D], k/v [B,Sk,H,D], o [B,Sq,H,D] bf16 with unit stride on D, stride D on H and the
// given element strides on the sequence and batch axes (so q/k/v may be slices of a fused QKV
// buffer).  lse [B,H,Sq] fp32 or null.
static int attn_fwd_entry(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                          int H, int D, long long q_ss, long long q_sb, long long k_ss, long long k_sb,
                          long long v_ss, long long v_sb, long long o_ss, long long o_sb, float scale, int* status,
                          void* stream, const RowScatter& rs, const AttnMask* mask = nullptr) {
  if (D != 64 && D != 128) return fail("attention: head_dim must be 64 or 128%s");
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0) return fail("attention: empty problem%s");
  CUtensorMap tq, tk, tv, to;
  int rc;
  if ((rc = make_bshd_map(&tq, q, B, Sq, H, D, q_ss, q_sb))) return rc;
  if ((rc = make_bshd_map(&tk, k, B, Sk, H, D, k_ss, k_sb))) return rc;
  if ((rc = make_bshd_map(&tv, v, B, Sk, H, D, v_ss, v_sb))) return rc;
  if ((rc = make_bshd_map(&to, o, B, Sq, H, D, o_ss, o_sb))) return rc;
  AttnParams p;
  p.Sq = Sq; p.Sk = Sk; p.H = H; p.B = B;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse;
  p.status = status;
  memset(&p.mask, 0, sizeof(p.mask));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (mask != nullptr) {
    p.mask = *mask;
    if (D == 128) return launch_attn_fwd<128, true>(tq, tk, tv, to, p, st, rs);
    return launch_attn_fwd<64, true>(tq, tk, tv, to, p, st, rs);
  }
  if (D == 128) return launch_attn_fwd<128, false>(tq, tk, tv, to, p, st, rs);
  return launch_attn_fwd<64, false>(tq, tk, tv, to, p, st, rs);
}

extern "C" int solar_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                              int Sq, int Sk, int H, int D, long long q_ss, long long q_sb,
                              long long k_ss, long long k_sb, long long v_ss, long long v_sb,
                              long long o_ss, long long o_sb, float scale, int* status, void* stream) {
  RowScatter none;
  memset(&none, 0, sizeof(none));
  return attn_fwd_entry(q, k, v, o, lse, B, Sq, Sk, H, D, q_ss, q_sb, k_ss, k_sb, v_ss, v_sb, o_ss, o_sb, scale,
                        status, stream, none);
}

// Attention under a structured mask: query row i attends the union of the key ranges row_ranges[i] (three [lo, hi)
// pairs).  tile_list / tile_count: for every block of 256 query rows, the 128-key tiles that some row of the block
// sees (bit 30 of an entry: some row sees the tile only in part), built by the caller (ops/attention_mask.py).
// All three tables are int32 in device memory; every block of rows must list at least one tile.
extern "C" int solar_attn_fwd_masked(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq,
                                     int Sk, int H, int D, long long q_ss, long long q_sb, long long k_ss,
                                     long long k_sb, long long v_ss, long long v_sb, long long o_ss, long long o_sb,
                                     float scale, int* status, void* stream, const int* row_ranges,
                                     const int* tile_list, const int* tile_count, int list_stride, const int* order) {
  if (row_ranges == nullptr || tile_list == nullptr || tile_count == nullptr || list_stride < 1)
    return fail("masked attention: the mask tables are required%s");
  RowScatter none;
  memset(&none, 0, sizeof(none));
  AttnMask m{row_ranges, tile_list, tile_count, list_stride, order};
  return attn_fwd_entry(q, k, v, o, lse, B, Sq, Sk, H, D, q_ss, q_sb, k_ss, k_sb, v_ss, v_sb, o_ss, o_sb, scale,
                        status, stream, none, &m);
}

// Attention over this rank's heads and the whole sequence whose output rows are, in addition to
// the local copy in `o`, stored into the token owner's buffer (Ulysses output exchange fused into
// the epilogue): row i goes to the rank r with row_start[r] <= i < row_start[r+1], at local row
// i - row_start[r], columns col_offset + head*D .. of a [*, dst_ld] matrix.  B must be 1.
extern "C" int solar_attn_fwd_scatter(const void* q, const void* k, const void* v, void* o, float* lse, int Sq,
                                      int Sk, int H, int D, long long q_ss, long long k_ss, long long v_ss,
                                      long long o_ss, float scale, int* status, void* stream,
                                      void* const* dst_bases, void* const* flag_ptrs, unsigned* counter,
                                      int n_ranks, long long dst_ld, long long dst_rows, const int* row_start,
                                      int col_offset) {
  if (n_ranks < 1 || n_ranks > kMaxPeers) return fail("attention scatter: rank count out of range%s");
  // every destination buffer holds dst_rows rows: a rank's row range may not be larger (the stores would run past
  // the buffer in the peer's memory)
  for (int i = 0; i < n_ranks; ++i)
    if (row_start[i + 1] < row_start[i] || row_start[i + 1] - row_start[i] > dst_rows)
      return fail("attention scatter: a rank's rows exceed the destination buffer%s");
  if (row_start[n_ranks] != Sq) return fail("attention scatter: row ranges must cover the sequence%s");
  RowScatter rs;
  memset(&rs, 0, sizeof(rs));
  rs.dst.n = n_ranks;
  rs.flags.n = n_ranks;
  for (int i = 0; i < n_ranks; ++i) {
    rs.dst.base[i] = dst_bases[i];
    rs.flags.flag[i] = static_cast<unsigned*>(flag_ptrs[i]);
    rs.row_start[i] = row_start[i];
  }
  rs.row_start[n_ranks] = row_start[n_ranks];
  rs.flags.local_counter = counter;
  rs.ld = dst_ld;
  rs.col_offset = col_offset;
  return attn_fwd_entry(q, k, v, o, lse, 1, Sq, Sk, H, D, q_ss, q_ss * Sq, k_ss, k_ss * Sk, v_ss, v_ss * Sk, o_ss,
                        o_ss * Sq, scale, status, stream, rs);
}
