// Row-wise normalisation kernels (memory-bound; one CTA of 128 threads per token row,
// the row lives in registers between the statistics pass and the output pass so every
// element is read from HBM exactly once):
//
//   norm_modulate   y = norm(x) [*w + b] * (1 + scale[g]) + shift[g]      (+ backward)
//   gated_residual  out = res + gate[g] * y                               (+ backward)
//   rmsnorm_rope    y = rope(rmsnorm_fulldim(x) * w)   (Wan q/k path)     (+ backward)
//   colreduce_*     deterministic per-group column reductions for the parameter gradients
//
// `g` is the modulation group of a row: either row / rows_per_group + group_offset
// (Wan: one adaLN vector set per latent frame) or an explicit int32 table (H3: adaLN
// table index t_idx*3 + tag per packed-document row).
//
// Replaces the eager chains LayerNorm -> (1+scale)*x+shift -> gate*y+x of the reference
// (solar/backends/wan22/runtime/modeling/causal_model.py:1636-1707), its Triton
// rmsnorm_modulate / gated_residual kernels (solar/backends/minimax_h3/fused_ops.py:39-206)
// and the fp64 complex rope_apply loop (solar/backends/wan22/runtime/modeling/model.py:38-66).
#include "comm.cuh"
#include "host_util.h"
#include "sm100.cuh"

namespace solar {

constexpr int ROW_THREADS = 128;
constexpr int MAXV = 8;  // uint4 (8 bf16) vectors per thread -> D <= 8192

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sum over the 128 threads of the CTA; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                       pack_bf16x2(f[6], f[7]));
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void load8f(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

struct GroupMap {
  const int* table;       // optional explicit group per row
  int rows_per_group;     // used when table == null (>= 1)
  int group_offset;
  __device__ __forceinline__ int operator()(long long row) const {
    return table ? table[row] : static_cast<int>(row / rows_per_group) + group_offset;
  }
};

// mode: 0 = LayerNorm (no affine), 1 = RMSNorm * w, 2 = LayerNorm * w + b
struct NormModParams {
  const __nv_bfloat16* x; long long ldx;
  __nv_bfloat16* y; long long ldy;
  float* stats;                 // [R,2] mean, rstd (written by fwd, read by bwd)
  const float* w; const float* b;
  const float* shift; const float* scale; long long mod_stride;  // null = no modulation
  GroupMap gm;
  int D; float eps; int mode;
};

__global__ void __launch_bounds__(ROW_THREADS) norm_modulate_fwd_kernel(NormModParams p) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const int nvec = p.D >> 3;
  const __nv_bfloat16* xr = p.x + row * p.ldx;
  float v[MAXV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
      load8(xr + vi * 8, v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[i][e];
    }
  }
  float mean = 0.f;
  if (p.mode != 1) mean = block_sum(s, red) / p.D;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float d = v[i][e] - mean;
        ss += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / p.D + p.eps);
  if (threadIdx.x == 0 && p.stats) {
    p.stats[row * 2] = mean;
    p.stats[row * 2 + 1] = rstd;
  }
  const float* sh = nullptr; const float* sc = nullptr;
  if (p.scale) {
    const long long g = p.gm(row);
    sc = p.scale + g * p.mod_stride;
    sh = p.shift + g * p.mod_stride;
  }
  __nv_bfloat16* yr = p.y + row * p.ldy;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
      float o[8], a[8], c[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[i][e] - mean) * rstd;
      if (p.mode >= 1) {
        load8f(p.w + vi * 8, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= a[e];
      }
      if (p.mode == 2) {
        load8f(p.b + vi * 8, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += a[e];
      }
      if (sc) {
        load8f(sc + vi * 8, a);
        load8f(sh + vi * 8, c);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = o[e] * (1.f + a[e]) + c[e];
      }
      store8(yr + vi * 8, o);
    }
  }
}


// Warp-per-row variant of the forward: lane l owns the 16-byte vectors l, l+32, ... of the row (NV of
// them), all loads of a row are in flight at once and both reductions are warp shuffles -- no shared
// memory and no block barrier.  Used whenever the row fits (D <= NV * 256).
template <int NV>
__global__ void __launch_bounds__(256) norm_modulate_fwd_warp_kernel(NormModParams p, long long rows) {
  const long long row = blockIdx.x * 8ll + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int nvec = p.D >> 3;
  const __nv_bfloat16* xr = p.x + row * p.ldx;
  uint4 raw[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + i * 32;
    raw[i] = vi < nvec ? *reinterpret_cast<const uint4*>(xr + vi * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const float2 a = unpack_bf16x2(raw[i].x), b = unpack_bf16x2(raw[i].y), c = unpack_bf16x2(raw[i].z),
                 d = unpack_bf16x2(raw[i].w);
    s += (a.x + a.y) + (b.x + b.y) + (c.x + c.y) + (d.x + d.y);
  }
  float mean = 0.f;
  if (p.mode != 1) mean = warp_sum(s) / p.D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + i * 32 < nvec) {
      const float2 a = unpack_bf16x2(raw[i].x), b = unpack_bf16x2(raw[i].y), c = unpack_bf16x2(raw[i].z),
                   d = unpack_bf16x2(raw[i].w);
      const float e[8] = {a.x - mean, a.y - mean, b.x - mean, b.y - mean, c.x - mean, c.y - mean, d.x - mean, d.y - mean};
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += e[k] * e[k];
    }
  }
  const float rstd = rsqrtf(warp_sum(ss) / p.D + p.eps);
  if (lane == 0 && p.stats) {
    p.stats[row * 2] = mean;
    p.stats[row * 2 + 1] = rstd;
  }
  const float* sh = nullptr; const float* sc = nullptr;
  if (p.scale) {
    const long long g = p.gm(row);
    sc = p.scale + g * p.mod_stride;
    sh = p.shift + g * p.mod_stride;
  }
  __nv_bfloat16* yr = p.y + row * p.ldy;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      const float2 a0 = unpack_bf16x2(raw[i].x), b0 = unpack_bf16x2(raw[i].y), c0 = unpack_bf16x2(raw[i].z),
                   d0 = unpack_bf16x2(raw[i].w);
      float o[8] = {a0.x, a0.y, b0.x, b0.y, c0.x, c0.y, d0.x, d0.y}, a[8], c[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (o[e] - mean) * rstd;
      if (p.mode >= 1) {
        load8f(p.w + vi * 8, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= a[e];
      }
      if (p.mode == 2) {
        load8f(p.b + vi * 8, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += a[e];
      }
      if (sc) {
        load8f(sc + vi * 8, a);
        load8f(sh + vi * 8, c);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = o[e] * (1.f + a[e]) + c[e];
      }
      store8(yr + vi * 8, o);
    }
  }
}

// dx for the row.  dy is the gradient of the modulated output.
struct NormModBwdParams {
  const __nv_bfloat16* dy; long long lddy;
  const __nv_bfloat16* x; long long ldx;
  __nv_bfloat16* dx; long long lddx;
  const float* stats;
  const float* w;
  const float* scale; long long mod_stride;
  GroupMap gm;
  int D; int mode;
  int accumulate;  // dx += (residual-path gradient already in dx)
};

__global__ void __launch_bounds__(ROW_THREADS) norm_modulate_bwd_kernel(NormModBwdParams p) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const int nvec = p.D >> 3;
  const float mean = p.stats[row * 2], rstd = p.stats[row * 2 + 1];
  const float* sc = p.scale ? p.scale + static_cast<long long>(p.gm(row)) * p.mod_stride : nullptr;
  float g[MAXV][8], n[MAXV][8];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
      float a[8];
      load8(p.dy + row * p.lddy + vi * 8, g[i]);
      load8(p.x + row * p.ldx + vi * 8, n[i]);
      if (sc) {
        load8f(sc + vi * 8, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[i][e] *= (1.f + a[e]);
      }
      if (p.mode >= 1) {
        load8f(p.w + vi * 8, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[i][e] *= a[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        n[i][e] = (n[i][e] - mean) * rstd;
        s1 += g[i][e];
        s2 += g[i][e] * n[i][e];
      }
    }
  }
  float m1 = 0.f;
  if (p.mode != 1) m1 = block_sum(s1, red) / p.D;
  const float m2 = block_sum(s2, red) / p.D;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rstd * (g[i][e] - m1 - n[i][e] * m2);
      __nv_bfloat16* d = p.dx + row * p.lddx + vi * 8;
      if (p.accumulate) {
        float a[8];
        load8(d, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += a[e];
      }
      store8(d, o);
    }
  }
}

// ----------------------------------------------------------------------------------------
// Column reductions.  grid = (ceil(D/64), groups, splits); block = 256 threads = 8 warps;
// a warp covers 64 columns (2 per lane) and strides over the rows of its split.
//   kind 0 (norm_modulate):  out0[g] = sum dy * nx  (d scale),  out1[g] = sum dy  (d shift)
//          where nx = norm(x) [*w+b] -- the un-modulated normalised activations
//   kind 1 (norm affine)  :  out0 = sum dyn * n (d w), out1 = sum dyn (d b), dyn = dy*(1+scale)
//   kind 2 (gated residual): out0[g] = sum dout * y (d gate)
//   kind 3 (bias gradient) : out0[g] = sum a
// Rows of a group must be contiguous: group g covers rows [g*rpg, (g+1)*rpg) (+row_base).
// ----------------------------------------------------------------------------------------
struct ColReduceParams {
  const __nv_bfloat16* a; long long lda;  // dy / dout
  const __nv_bfloat16* x; long long ldx;  // x (kind 0/1) or y (kind 2)
  const float* stats;
  const float* w; const float* b;         // affine terms of the norm (kind 0 with mode>=1)
  const float* scale; long long mod_stride; int group_offset;  // kind 1
  float* out0; float* out1;               // [splits, groups, D]
  long long rows; int rows_per_group; int groups; int D; int kind; int mode;
  int scale_rpg;                          // rows per modulation group for the kind-1 scale lookup
};

__global__ void __launch_bounds__(256) colreduce_kernel(ColReduceParams p) {
  __shared__ float sm0[8][64], sm1[8][64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + lane * 2;
  const int g = blockIdx.y;
  const int splits = gridDim.z, sp = blockIdx.z;
  const long long gstart = static_cast<long long>(g) * p.rows_per_group;
  long long gend = gstart + p.rows_per_group;
  if (gend > p.rows) gend = p.rows;
  const long long glen = gend - gstart;
  const long long per = (glen + splits - 1) / splits;
  const long long r0 = gstart + sp * per;
  long long r1 = r0 + per;
  if (r1 > gend) r1 = gend;
  float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
  if (col < p.D) {
    float w0 = 1.f, w1 = 1.f, bb0 = 0.f, bb1 = 0.f;
    if (p.kind == 0 && p.mode >= 1) { w0 = p.w[col]; w1 = p.w[col + 1]; }
    if (p.kind == 0 && p.mode == 2) { bb0 = p.b[col]; bb1 = p.b[col + 1]; }
    for (long long r = r0 + warp; r < r1; r += 8) {
      const float2 d = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.a + r * p.lda + col));
      if (p.kind == 3) {
        a0 += d.x; a1 += d.y;
        continue;
      }
      float2 xv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.x + r * p.ldx + col));
      if (p.kind == 2) {
        a0 += d.x * xv.x; a1 += d.y * xv.y;
      } else {
        const float mean = p.stats[r * 2], rstd = p.stats[r * 2 + 1];
        float n0 = (xv.x - mean) * rstd, n1 = (xv.y - mean) * rstd;
        if (p.kind == 0) {
          n0 = n0 * w0 + bb0; n1 = n1 * w1 + bb1;
          a0 += d.x * n0; a1 += d.y * n1; b0 += d.x; b1 += d.y;
        } else {
          float s0 = 1.f, s1 = 1.f;
          if (p.scale) {
            const float* sc = p.scale + (static_cast<long long>(r / p.scale_rpg) + p.group_offset) * p.mod_stride;
            s0 += sc[col]; s1 += sc[col + 1];
          }
          a0 += d.x * s0 * n0; a1 += d.y * s1 * n1; b0 += d.x * s0; b1 += d.y * s1;
        }
      }
    }
  }
  sm0[warp][lane * 2] = a0; sm0[warp][lane * 2 + 1] = a1;
  sm1[warp][lane * 2] = b0; sm1[warp][lane * 2 + 1] = b1;
  __syncthreads();
  if (threadIdx.x < 64) {
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < p.D) {
      float t0 = 0.f, t1 = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) { t0 += sm0[w][threadIdx.x]; t1 += sm1[w][threadIdx.x]; }
      const long long o = (static_cast<long long>(sp) * p.groups + g) * p.D + c;
      p.out0[o] = t0;
      if (p.out1) p.out1[o] = t1;
    }
  }
}

// ----------------------------------------------------------------------------------------
// gated residual: out = res + gate[g] * y ; backward dy = dout * gate[g]
// ----------------------------------------------------------------------------------------
struct GatedParams {
  const __nv_bfloat16* res; long long ldres;  // fwd: residual ; bwd: unused
  const __nv_bfloat16* y; long long ldy;      // fwd: branch ; bwd: dout
  __nv_bfloat16* out; long long ldo;
  const float* gate; long long mod_stride;    // null gate == 1
  GroupMap gm;
  int D; int backward;
};

__global__ void __launch_bounds__(ROW_THREADS) gated_residual_kernel(GatedParams p) {
  const long long row = blockIdx.x;
  const int nvec = p.D >> 3;
  const float* gt = p.gate ? p.gate + static_cast<long long>(p.gm(row)) * p.mod_stride : nullptr;
  for (int vi = threadIdx.x; vi < nvec; vi += ROW_THREADS) {
    float y[8], o[8], g[8];
    load8(p.y + row * p.ldy + vi * 8, y);
    if (gt) {
      load8f(gt + vi * 8, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] *= g[e];
    }
    if (!p.backward) {
      load8(p.res + row * p.ldres + vi * 8, o);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] += o[e];
    }
    store8(p.out + row * p.ldo + vi * 8, y);
  }
}

// ----------------------------------------------------------------------------------------
// Full-width RMSNorm * w followed by interleaved-pair RoPE per head (Wan q/k path).
// rope: [R, hd/2] float2 (cos, sin) per token; null = no rotation.
// ----------------------------------------------------------------------------------------
struct RmsRopeParams {
  const __nv_bfloat16* x; long long ldx;
  __nv_bfloat16* y; long long ldy;
  const float* w;
  const float2* rope; int half_hd;   // hd/2 complex pairs per head
  float* rstd;                       // [R]
  int D; float eps;
  int no_norm;                       // 1: rotation only
};

__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_rope_fwd_kernel(RmsRopeParams p, const __grid_constant__ ColScatter sc) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const int nvec = p.D >> 3;
  float v[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
      load8(p.x + row * p.ldx + vi * 8, v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  float rstd = 1.f;
  if (!p.no_norm) {
    rstd = rsqrtf(block_sum(ss, red) / p.D + p.eps);
    if (threadIdx.x == 0 && p.rstd) p.rstd[row] = rstd;
  }
  const float2* rp = p.rope ? p.rope + row * p.half_hd : nullptr;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
      float o[8];
      if (!p.no_norm) {
        float a[8];
        load8f(p.w + vi * 8, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd * a[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[i][e];
      }
      if (rp) {
        const int pair0 = ((vi * 8) % (2 * p.half_hd)) >> 1;  // first complex pair of this vector
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 cs = rp[pair0 + e];
          const float a = o[2 * e], b = o[2 * e + 1];
          o[2 * e] = a * cs.x - b * cs.y;
          o[2 * e + 1] = a * cs.y + b * cs.x;
        }
      }
      if (sc.active())   // heads -> ranks: straight into the owning rank's receive buffer
        store8(static_cast<__nv_bfloat16*>(sc.addr(row, vi * 8, 2)), o);
      else
        store8(p.y + row * p.ldy + vi * 8, o);
    }
  }
  if (sc.active()) cta_done_signal_peers(sc.flags);
}

// Backward: dy is the gradient of the rotated output; writes dx (may alias dy).
struct RmsRopeBwdParams {
  const __nv_bfloat16* dy; long long lddy;
  const __nv_bfloat16* x; long long ldx;
  __nv_bfloat16* dx; long long lddx;
  const float* w; const float2* rope; int half_hd;
  const float* rstd;
  int D; int no_norm;
};

__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_rope_bwd_kernel(RmsRopeBwdParams p) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const int nvec = p.D >> 3;
  const float rstd = p.no_norm ? 1.f : p.rstd[row];
  const float2* rp = p.rope ? p.rope + row * p.half_hd : nullptr;
  float g[MAXV][8], n[MAXV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
      load8(p.dy + row * p.lddy + vi * 8, g[i]);
      if (rp) {
        const int pair0 = ((vi * 8) % (2 * p.half_hd)) >> 1;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 cs = rp[pair0 + e];
          const float a = g[i][2 * e], b = g[i][2 * e + 1];
          g[i][2 * e] = a * cs.x + b * cs.y;
          g[i][2 * e + 1] = -a * cs.y + b * cs.x;
        }
      }
      if (!p.no_norm) {
        float a[8];
        load8(p.x + row * p.ldx + vi * 8, n[i]);
        load8f(p.w + vi * 8, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          n[i][e] *= rstd;
          g[i][e] *= a[e];
          s += g[i][e] * n[i][e];
        }
      }
    }
  }
  float m = 0.f;
  if (!p.no_norm) m = block_sum(s, red) / p.D;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * ROW_THREADS;
    if (vi < nvec) {
      float o[8];
      if (!p.no_norm) {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd * (g[i][e] - n[i][e] * m);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = g[i][e];
      }
      store8(p.dx + row * p.lddx + vi * 8, o);
    }
  }
}

// d w[c] = sum_r unrotate(dy)[r,c] * x[r,c] * rstd[r]; grid = (ceil(D/64), 1, splits)
struct RmsRopeDwParams {
  const __nv_bfloat16* dy; long long lddy;
  const __nv_bfloat16* x; long long ldx;
  const float2* rope; int half_hd; const float* rstd;
  float* out;  // [splits, D]
  long long rows; int D;
};
__global__ void __launch_bounds__(256) rmsnorm_rope_dw_kernel(RmsRopeDwParams p) {
  __shared__ float sm0[8][64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + lane * 2;  // even: one complex pair per lane
  const int splits = gridDim.z, sp = blockIdx.z;
  const long long per = (p.rows + splits - 1) / splits;
  const long long r0 = sp * per;
  long long r1 = r0 + per;
  if (r1 > p.rows) r1 = p.rows;
  float a0 = 0.f, a1 = 0.f;
  if (col < p.D) {
    const int pair = (col % (2 * p.half_hd)) >> 1;
    for (long long r = r0 + warp; r < r1; r += 8) {
      float2 d = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.dy + r * p.lddy + col));
      const float2 xv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.x + r * p.ldx + col));
      if (p.rope) {
        const float2 cs = p.rope[r * p.half_hd + pair];
        const float a = d.x, b = d.y;
        d.x = a * cs.x + b * cs.y;
        d.y = -a * cs.y + b * cs.x;
      }
      const float rs = p.rstd[r];
      a0 += d.x * xv.x * rs;
      a1 += d.y * xv.y * rs;
    }
  }
  sm0[warp][lane * 2] = a0; sm0[warp][lane * 2 + 1] = a1;
  __syncthreads();
  if (threadIdx.x < 64) {
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < p.D) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += sm0[w][threadIdx.x];
      p.out[static_cast<long long>(sp) * p.D + c] = t;
    }
  }
}

static int check_D(int D) {
  if (D <= 0 || D % 8 != 0 || D > MAXV * 8 * ROW_THREADS) return fail("row kernels need D %% 8 == 0 and D <= 8192%s");
  return 0;
}

}  // namespace solar

using namespace solar;

extern "C" int solar_norm_modulate_fwd(const void* x, long long ldx, void* y, long long ldy,
                                       float* stats, const float* w, const float* b,
                                       const float* shift, const float* scale, long long mod_stride,
                                       const int* group_table, int rows_per_group, int group_offset,
                                       long long rows, int D, float eps, int mode, void* stream) {
  if (check_D(D)) return -1;
  if (rows <= 0) return 0;
  NormModParams p{(const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)y, ldy, stats, w, b, shift, scale,
                  mod_stride, GroupMap{group_table, rows_per_group > 0 ? rows_per_group : 1, group_offset},
                  D, eps, mode};
  const unsigned grid8 = static_cast<unsigned>((rows + 7) / 8);
  if (D <= 12 * 256)
    norm_modulate_fwd_warp_kernel<12><<<grid8, 256, 0, (cudaStream_t)stream>>>(p, rows);
  else if (D <= 24 * 256)
    norm_modulate_fwd_warp_kernel<24><<<grid8, 256, 0, (cudaStream_t)stream>>>(p, rows);
  else
    norm_modulate_fwd_kernel<<<(unsigned)rows, ROW_THREADS, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_norm_modulate_bwd(const void* dy, long long lddy, const void* x, long long ldx,
                                       void* dx, long long lddx, const float* stats, const float* w,
                                       const float* scale, long long mod_stride,
                                       const int* group_table, int rows_per_group, int group_offset,
                                       long long rows, int D, int mode, int accumulate, void* stream) {
  if (check_D(D)) return -1;
  if (rows <= 0) return 0;
  NormModBwdParams p{(const __nv_bfloat16*)dy, lddy, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)dx,
                     lddx, stats, w, scale, mod_stride,
                     GroupMap{group_table, rows_per_group > 0 ? rows_per_group : 1, group_offset}, D,
                     mode, accumulate};
  norm_modulate_bwd_kernel<<<(unsigned)rows, ROW_THREADS, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_colreduce(const void* a, long long lda, const void* x, long long ldx,
                               const float* stats, const float* w, const float* b,
                               const float* scale, long long mod_stride, int group_offset,
                               float* out0, float* out1, long long rows, int rows_per_group,
                               int groups, int splits, int D, int kind, int mode, int scale_rpg,
                               void* stream) {
  if (D % 2 != 0) return fail("colreduce needs even D%s");
  if (rows <= 0) return 0;
  ColReduceParams p{(const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)x, ldx, stats, w, b, scale,
                    mod_stride, group_offset, out0, out1, rows, rows_per_group, groups, D, kind, mode,
                    scale_rpg > 0 ? scale_rpg : 1};
  dim3 grid((D + 63) / 64, groups, splits);
  colreduce_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_gated_residual(const void* res, long long ldres, const void* y, long long ldy,
                                    void* out, long long ldo, const float* gate, long long mod_stride,
                                    const int* group_table, int rows_per_group, int group_offset,
                                    long long rows, int D, int backward, void* stream) {
  if (D % 8 != 0) return fail("gated_residual needs D %% 8 == 0%s");
  if (rows <= 0) return 0;
  GatedParams p{(const __nv_bfloat16*)res, ldres, (const __nv_bfloat16*)y, ldy, (__nv_bfloat16*)out, ldo,
                gate, mod_stride, GroupMap{group_table, rows_per_group > 0 ? rows_per_group : 1, group_offset},
                D, backward};
  gated_residual_kernel<<<(unsigned)rows, ROW_THREADS, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_rmsnorm_rope_fwd(const void* x, long long ldx, void* y, long long ldy,
                                      const float* w, const void* rope, int half_hd, float* rstd,
                                      long long rows, int D, float eps, int no_norm, void* stream) {
  if (check_D(D)) return -1;
  if (rope && ((2 * half_hd) % 8 != 0)) return fail("rope needs head_dim %% 8 == 0%s");
  if (rows <= 0) return 0;
  RmsRopeParams p{(const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)y, ldy, w, (const float2*)rope, half_hd,
                  rstd, D, eps, no_norm};
  ColScatter none;
  memset(&none, 0, sizeof(none));
  rmsnorm_rope_fwd_kernel<<<(unsigned)rows, ROW_THREADS, 0, (cudaStream_t)stream>>>(p, none);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// Same operator with the Ulysses column scatter as its output stage: every 16-byte piece of the
// normalised, rotated row is stored into the receive buffer of the rank that owns its head, and the
// last CTA bumps the flag word on every rank.  `rstd` is still written locally for the backward.
extern "C" int solar_rmsnorm_rope_scatter(const void* x, long long ldx, const float* w, const void* rope,
                                          int half_hd, float* rstd, long long rows, int D, float eps,
                                          int no_norm, void* stream, void* const* dst_bases,
                                          void* const* flag_ptrs, unsigned* counter, int n_ranks,
                                          long long dst_ld, int cols_per_dest, int row_offset, int col_base) {
  if (check_D(D)) return -1;
  if (n_ranks < 1 || n_ranks > kMaxPeers) return fail("rmsnorm_rope scatter: rank count out of range%s");
  if (cols_per_dest % 8 != 0 || D % cols_per_dest != 0) return fail("rmsnorm_rope scatter: bad column blocks%s");
  if (rows <= 0) return fail("rmsnorm_rope scatter: every rank must launch at least one row%s");
  RmsRopeParams p{(const __nv_bfloat16*)x, ldx, nullptr, 0, w, (const float2*)rope, half_hd, rstd, D, eps, no_norm};
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
  sc.group_cols = D;
  sc.cols_per_dest = cols_per_dest;
  sc.row_offset = row_offset;
  sc.col_base = col_base;
  rmsnorm_rope_fwd_kernel<<<(unsigned)rows, ROW_THREADS, 0, (cudaStream_t)stream>>>(p, sc);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_rmsnorm_rope_bwd(const void* dy, long long lddy, const void* x, long long ldx,
                                      void* dx, long long lddx, const float* w, const void* rope,
                                      int half_hd, const float* rstd, float* dw_partial, int splits,
                                      long long rows, int D, int no_norm, void* stream) {
  if (check_D(D)) return -1;
  if (rows <= 0) return 0;
  if (dw_partial && !no_norm) {
    RmsRopeDwParams q{(const __nv_bfloat16*)dy, lddy, (const __nv_bfloat16*)x, ldx, (const float2*)rope,
                      half_hd, rstd, dw_partial, rows, D};
    dim3 grid((D + 63) / 64, 1, splits);
    rmsnorm_rope_dw_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(q);
    SOLAR_CUDA_OK(cudaGetLastError());
  }
  RmsRopeBwdParams p{(const __nv_bfloat16*)dy, lddy, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)dx,
                     lddx, w, (const float2*)rope, half_hd, rstd, D, no_norm};
  rmsnorm_rope_bwd_kernel<<<(unsigned)rows, ROW_THREADS, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}
