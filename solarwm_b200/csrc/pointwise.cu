// Streaming element-wise kernels (all HBM-bound; 16-byte vector accesses, grid-stride):
//   gelu_tanh fwd / bwd, SwiGLU fwd / bwd
//   fused AdamW on flat shards (fp32 master + moments, bf16 live copy, optional EMA shadow,
//     gradient scale read from device so the clip coefficient never syncs the host)
//   sum of squares (gradient norm), with deterministic two-stage reduction
//   flow-matching scheduler math: add_noise / velocity target / x0 / Euler step
//   weighted masked MSE forward + backward
//   bf16 CHW -> RGB8 HWC pixel conversion (device twin of the host routine in pixels.cpp)
//
// Reference behaviour: solar/training/optim.py:111-151 (FP32MasterAdamW), solar/training/ema.py:71-81,
// solar/backends/wan22/runtime/scheduler.py:100-112, solar/backends/wan22/objectives.py:147-195,
// solar/backends/minimax_h3/fused_ops.py:496-565 (SwiGLU), deploy/solar_wm/shared/media/pixels.c:20-34.
#include "host_util.h"
#include "sm100.cuh"

namespace solar {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                            pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// mode 0: y = gelu(x) ; mode 1: dx = dy * gelu'(x), and (optionally) act = gelu(x)
__global__ void gelu_kernel(const __nv_bfloat16* x, const __nv_bfloat16* dy, __nv_bfloat16* out,
                            __nv_bfloat16* act, long long nvec, int mode) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8], o[8];
    ld8(x + i * 8, a);
    if (mode == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = gelu_tanh(a[e]);
    } else {
      float g[8];
      ld8(dy + i * 8, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = g[e] * gelu_tanh_grad(a[e]);
      if (act) {
        float t[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) t[e] = gelu_tanh(a[e]);
        st8(act + i * 8, t);
      }
    }
    st8(out + i * 8, o);
  }
}

// SwiGLU over a [M, 2N] projection (gate | up halves): y = up * silu(gate)
__global__ void swiglu_kernel(const __nv_bfloat16* gu, const __nv_bfloat16* dy, __nv_bfloat16* out,
                              long long M, int N, int backward) {
  const int nv = N >> 3;
  const long long total = M * nv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nv;
    const int c = static_cast<int>(i - r * nv) * 8;
    float g[8], u[8];
    ld8(gu + r * 2 * N + c, g);
    ld8(gu + r * 2 * N + N + c, u);
    if (!backward) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = u[e] * (g[e] / (1.f + __expf(-g[e])));
      st8(out + r * N + c, o);
    } else {
      float d[8], dg[8], du[8];
      ld8(dy + r * N + c, d);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float s = 1.f / (1.f + __expf(-g[e]));
        du[e] = d[e] * g[e] * s;
        dg[e] = d[e] * u[e] * s * (1.f + g[e] * (1.f - s));
      }
      st8(out + r * 2 * N + c, dg);
      st8(out + r * 2 * N + N + c, du);
    }
  }
}

// ----------------------------------------------------------------------------------------
// Fused AdamW over a flat shard.  grad may be bf16 or fp32.  grad_scale (device) multiplies
// the gradient (clip coefficient / loss-scale); if *skip != 0 the kernel does nothing
// (non-finite step: the reference aborts before mutating state, training/engine.py:188-193).
// ----------------------------------------------------------------------------------------
struct AdamParams {
  float* master; float* m; float* v; __nv_bfloat16* live; float* ema;
  const void* grad; int grad_is_f32;
  const float* grad_scale; const int* skip;
  long long n;
  float lr, beta1, beta2, eps, wd, bc1, bc2, ema_decay;
};
__global__ void adamw_kernel(AdamParams p) {
  if (p.skip && *p.skip) return;
  const float gs = p.grad_scale ? *p.grad_scale : 1.f;
  const long long nv = p.n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float g[4];
    if (p.grad_is_f32) {
      const float4 t = reinterpret_cast<const float4*>(p.grad)[i];
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2*>(p.grad)[i];
      const float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    }
    float4 w = reinterpret_cast<float4*>(p.master)[i];
    float4 m = reinterpret_cast<float4*>(p.m)[i];
    float4 v = reinterpret_cast<float4*>(p.v)[i];
    float* wp = &w.x; float* mp = &m.x; float* vp = &v.x;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ge = g[e] * gs;
      wp[e] *= (1.f - p.lr * p.wd);
      mp[e] = p.beta1 * mp[e] + (1.f - p.beta1) * ge;
      vp[e] = p.beta2 * vp[e] + (1.f - p.beta2) * ge * ge;
      const float denom = sqrtf(vp[e] / p.bc2) + p.eps;
      wp[e] -= (p.lr / p.bc1) * (mp[e] / denom);
    }
    reinterpret_cast<float4*>(p.master)[i] = w;
    reinterpret_cast<float4*>(p.m)[i] = m;
    reinterpret_cast<float4*>(p.v)[i] = v;
    if (p.live)
      reinterpret_cast<uint2*>(p.live)[i] = make_uint2(pack_bf16x2(w.x, w.y), pack_bf16x2(w.z, w.w));
    if (p.ema) {
      float4 s = reinterpret_cast<float4*>(p.ema)[i];
      s.x = p.ema_decay * s.x + (1.f - p.ema_decay) * w.x;
      s.y = p.ema_decay * s.y + (1.f - p.ema_decay) * w.y;
      s.z = p.ema_decay * s.z + (1.f - p.ema_decay) * w.z;
      s.w = p.ema_decay * s.w + (1.f - p.ema_decay) * w.w;
      reinterpret_cast<float4*>(p.ema)[i] = s;
    }
  }
}

// partial[b] = sum of squares of the block's grid-stride slice; a second launch (1 block)
// adds the partials in a fixed order into out[0] (+= when accumulate).
__global__ void sumsq_kernel(const void* x, int is_f32, long long n, float* partial) {
  __shared__ float red[8];
  float s = 0.f;
  if (is_f32) {
    const long long nv = n >> 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      const float4 t = reinterpret_cast<const float4*>(x)[i];
      s += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
    }
  } else {
    const long long nv = n >> 3;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      float f[8];
      ld8(reinterpret_cast<const __nv_bfloat16*>(x) + i * 8, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += f[e] * f[e];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}
__global__ void sum_partials_kernel(const float* partial, int n, float* out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    out[0] = accumulate ? out[0] + t : t;
  }
}

// Flow-matching math on bf16 latents with a per-group sigma (group = i / group_size):
//   op 0: x_t = (1-s) x0 + s n ; target = n - x0        (out0 = x_t, out1 = target)
//   op 1: x0  = x_t - s v                               (out0)
//   op 2: Euler: x_next = x_t + (s_next - s) v          (out0), s_next in sigma2
//   op 3: renoise: x_next = (1-s2) x0 + s2 n            (out0)  (a = x0, b = n)
__global__ void flow_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, const float* sigma,
                            const float* sigma2, __nv_bfloat16* out0, __nv_bfloat16* out1,
                            long long n, long long group_size, int op) {
  const long long nv = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const long long g = (i * 8) / group_size;
    const float s = sigma[g];
    float x[8], y[8], o[8], t[8];
    ld8(a + i * 8, x);
    ld8(b + i * 8, y);
    if (op == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) { o[e] = (1.f - s) * x[e] + s * y[e]; t[e] = y[e] - x[e]; }
      st8(out0 + i * 8, o);
      if (out1) st8(out1 + i * 8, t);
    } else if (op == 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = x[e] - s * y[e];
      st8(out0 + i * 8, o);
    } else if (op == 2) {
      const float ds = sigma2[g] - s;
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = x[e] + ds * y[e];
      st8(out0 + i * 8, o);
    } else {
      const float s2 = sigma2[g];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (1.f - s2) * x[e] + s2 * y[e];
      st8(out0 + i * 8, o);
    }
  }
}

// Weighted masked MSE.  loss = sum_i w[g(i)] * m[g(i)] * (pred_i - tgt_i)^2 / denom, where the
// mask is applied to both operands before the subtraction (reference objectives.py:147-176).
// Forward writes per-block partials; backward writes dpred = 2 w m (pred - tgt) * gscale / denom.
__global__ void mse_kernel(const __nv_bfloat16* pred, const __nv_bfloat16* tgt, const float* w,
                           const float* mask, long long n, long long group_size, float inv_denom,
                           float* partial, __nv_bfloat16* dpred, const float* gscale) {
  __shared__ float red[8];
  const long long nv = n >> 3;
  const float gs = gscale ? *gscale : 1.f;
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const long long g = (i * 8) / group_size;
    const float wt = (w ? w[g] : 1.f);
    const float mk = (mask ? mask[g] : 1.f);
    float x[8], y[8], d[8];
    ld8(pred + i * 8, x);
    ld8(tgt + i * 8, y);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float df = x[e] * mk - y[e] * mk;
      s += wt * df * df;
      d[e] = 2.f * wt * mk * df * inv_denom * gs;
    }
    if (dpred) st8(dpred + i * 8, d);
  }
  if (partial) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < (blockDim.x >> 5); ++k) t += red[k];
      partial[blockIdx.x] = t * inv_denom;
    }
  }
}

// bf16 [3,H,W] (arbitrary element strides) -> uint8 [H,W,3]:  v*std[c]+mean[c], clamp [0,1],
// *255, round-to-nearest-even.  Three separately rounded fp32 operations (no fused multiply-
// add), as the reference's C routine is built with -ffp-contract=off.  A NaN pixel raises
// *nonfinite (the host routine returns 0 in that case).
struct Rgb8Params {
  const __nv_bfloat16* chw; uint8_t* hwc; int H, W;
  long long sc, sy, sx;
  float mean[3], std_[3];
  int* nonfinite;
};
__global__ void rgb8_kernel(Rgb8Params p) {
  const long long hw = (long long)p.H * p.W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < hw;
       i += (long long)gridDim.x * blockDim.x) {
    const long long y = i / p.W, x = i - y * p.W;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      float v = __bfloat162float(p.chw[c * p.sc + y * p.sy + x * p.sx]);
      v = __fadd_rn(__fmul_rn(v, p.std_[c]), p.mean[c]);
      if (isnan(v) && p.nonfinite) *p.nonfinite = 1;
      v = v < 0.f ? 0.f : (v > 1.f ? 1.f : v);
      v = __fmul_rn(v, 255.f);
      p.hwc[i * 3 + c] = static_cast<uint8_t>(nearbyintf(v));
    }
  }
}

// Tile blend + compensation of the streaming decoder's output: every output pixel is the ramp-weighted
// mean of the tiles that cover it (linear ramps across the overlaps, weights normalised to one), followed
// by x - (a + b x + c x^2) with per (channel, frame) constants.  One thread per output pixel, all channels
// and frames of it in registers; every tile pixel is read once.
struct TileBlendParams {
  const __nv_bfloat16* tiles; long long st, sc, sf;   // [T, 3, F, tH, tW], inner two dims contiguous
  float* out;                                         // [3, F, H, W]
  int T, F, tH, tW, H, W, ov;
  int py[32], px[32];                                 // pixel offsets of the tiles
  float a[3][4], b[3][4], c[3][4];                    // compensation constants (zero = none)
};

__device__ __forceinline__ float ramp_weight(int l, int n, bool lo, bool hi, int ov) {
  float w = 1.f;
  if (ov > 0) {
    const float step = 1.f / static_cast<float>(ov + 1);
    if (lo && l < ov) w = static_cast<float>(l + 1) * step;
    if (hi && l >= n - ov) w = 1.f - static_cast<float>(l - (n - ov) + 1) * step;
  }
  return w;
}

__global__ void tile_blend_kernel(TileBlendParams p) {
  const long long hw = (long long)p.H * p.W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < hw;
       i += (long long)gridDim.x * blockDim.x) {
    const int Y = static_cast<int>(i / p.W), X = static_cast<int>(i - (long long)Y * p.W);
    float acc[3][4];
#pragma unroll
    for (int c = 0; c < 3; ++c)
#pragma unroll
      for (int f = 0; f < 4; ++f) acc[c][f] = 0.f;
    float wsum = 0.f;
    for (int t = 0; t < p.T; ++t) {
      const int ly = Y - p.py[t], lx = X - p.px[t];
      if (ly < 0 || ly >= p.tH || lx < 0 || lx >= p.tW) continue;
      const float w = ramp_weight(ly, p.tH, p.py[t] > 0, p.py[t] + p.tH < p.H, p.ov) *
                      ramp_weight(lx, p.tW, p.px[t] > 0, p.px[t] + p.tW < p.W, p.ov);
      wsum += w;
      const __nv_bfloat16* src = p.tiles + t * p.st + (long long)ly * p.tW + lx;
#pragma unroll
      for (int c = 0; c < 3; ++c)
#pragma unroll
        for (int f = 0; f < 4; ++f)
          if (f < p.F) acc[c][f] += w * __bfloat162float(src[c * p.sc + f * p.sf]);
    }
    const float inv = 1.f / fmaxf(wsum, 1e-8f);
#pragma unroll
    for (int c = 0; c < 3; ++c)
#pragma unroll
      for (int f = 0; f < 4; ++f)
        if (f < p.F) {
          const float x = acc[c][f] * inv;
          p.out[((long long)c * p.F + f) * hw + i] = x - (p.a[c][f] + p.b[c][f] * x) - p.c[c][f] * x * x;
        }
  }
}

// Channel RMS norm (+ SiLU) of channels-last activations: y = x / max(||x||_2, 1e-12) * sqrt(C) * gamma, then
// optionally y * sigmoid(y).  One warp per pixel row; a lane keeps its 8-channel vectors in registers between
// the sum of squares and the write (C <= 1024).  The normalised value is rounded to bf16 before the gain and
// before the activation, as the unfused composition of the VAE blocks does.
__global__ void __launch_bounds__(256) rms_silu_cl_kernel(const __nv_bfloat16* __restrict__ x,
                                                          __nv_bfloat16* __restrict__ y,
                                                          const float* __restrict__ gamma, long long rows, int C,
                                                          int silu) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nvec = C >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(x + row * C);
  uint4 v[4];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = lane + 32 * k;
    if (i < nvec) {
      v[k] = src[i];
      const float2 a = unpack_bf16x2(v[k].x), b = unpack_bf16x2(v[k].y), c = unpack_bf16x2(v[k].z),
                   d = unpack_bf16x2(v[k].w);
      ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
  const float root_c = sqrtf(static_cast<float>(C));
  uint4* dst = reinterpret_cast<uint4*>(y + row * C);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = lane + 32 * k;
    if (i < nvec) {
      const uint32_t in[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
      uint32_t out[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(in[e]);
        const int ch = i * 8 + e * 2;
        float r[2] = {f.x * inv, f.y * inv};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          float t = __bfloat162float(__float2bfloat16(r[u]));                              // normalize -> bf16
          t = __bfloat162float(__float2bfloat16(t * root_c));                               // * sqrt(C)
          t = __bfloat162float(__float2bfloat16(t * __bfloat162float(__float2bfloat16(gamma[ch + u]))));
          if (silu) t = t / (1.f + __expf(-t));
          r[u] = t;
        }
        out[e] = pack_bf16x2(r[0], r[1]);
      }
      dst[i] = make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
}

static inline int grid_for(long long work, int block) {
  long long g = (work + block - 1) / block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace solar

using namespace solar;

extern "C" int solar_gelu(const void* x, const void* dy, void* out, void* act, long long n, int mode,
                          void* stream) {
  if (n % 8 != 0) return fail("gelu: n must be a multiple of 8%s");
  if (n == 0) return 0;
  gelu_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)out, (__nv_bfloat16*)act, n / 8, mode);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_swiglu(const void* gu, const void* dy, void* out, long long M, int N, int backward,
                            void* stream) {
  if (N % 8 != 0) return fail("swiglu: N must be a multiple of 8%s");
  if (M == 0) return 0;
  swiglu_kernel<<<grid_for(M * (N / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dy, (__nv_bfloat16*)out, M, N, backward);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_adamw(float* master, float* m, float* v, void* live, float* ema, const void* grad,
                           int grad_is_f32, const float* grad_scale, const int* skip, long long n,
                           float lr, float beta1, float beta2, float eps, float wd, float bc1,
                           float bc2, float ema_decay, void* stream) {
  if (n % 4 != 0) return fail("adamw: shard length must be a multiple of 4%s");
  if (n == 0) return 0;
  AdamParams p{master, m, v, (__nv_bfloat16*)live, ema, grad, grad_is_f32, grad_scale, skip, n,
               lr, beta1, beta2, eps, wd, bc1, bc2, ema_decay};
  adamw_kernel<<<grid_for(n / 4, 256), 256, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// scratch: >= 1024 floats of caller-provided device memory.
extern "C" int solar_sumsq(const void* x, int is_f32, long long n, float* scratch, float* out,
                           int accumulate, void* stream) {
  if (n % 8 != 0) return fail("sumsq: n must be a multiple of 8%s");
  int g = grid_for(n / 8, 256);
  if (g > 1024) g = 1024;
  sumsq_kernel<<<g, 256, 0, (cudaStream_t)stream>>>(x, is_f32, n, scratch);
  sum_partials_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(scratch, g, out, accumulate);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_flow(const void* a, const void* b, const float* sigma, const float* sigma2,
                          void* out0, void* out1, long long n, long long group_size, int op, void* stream) {
  if (n % 8 != 0 || group_size % 8 != 0) return fail("flow: sizes must be multiples of 8%s");
  if (n == 0) return 0;
  flow_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, sigma, sigma2, (__nv_bfloat16*)out0,
      (__nv_bfloat16*)out1, n, group_size, op);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// scratch: >= 1024 floats.  loss_out may be null (backward only); dpred may be null (forward only).
extern "C" int solar_mse(const void* pred, const void* tgt, const float* w, const float* mask,
                         long long n, long long group_size, float inv_denom, float* scratch,
                         float* loss_out, void* dpred, const float* gscale, void* stream) {
  if (n % 8 != 0 || group_size % 8 != 0) return fail("mse: sizes must be multiples of 8%s");
  int g = grid_for(n / 8, 256);
  if (g > 1024) g = 1024;
  mse_kernel<<<g, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)pred, (const __nv_bfloat16*)tgt, w,
                                                  mask, n, group_size, inv_denom,
                                                  loss_out ? scratch : nullptr, (__nv_bfloat16*)dpred, gscale);
  if (loss_out) sum_partials_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(scratch, g, loss_out, 0);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_rgb8(const void* chw, void* hwc, int H, int W, long long sc, long long sy,
                          long long sx, const float* mean3, const float* std3, int* nonfinite,
                          void* stream) {
  Rgb8Params p;
  p.chw = (const __nv_bfloat16*)chw; p.hwc = (uint8_t*)hwc; p.H = H; p.W = W;
  p.sc = sc; p.sy = sy; p.sx = sx;
  for (int c = 0; c < 3; ++c) { p.mean[c] = mean3[c]; p.std_[c] = std3[c]; }
  p.nonfinite = nonfinite;
  rgb8_kernel<<<grid_for((long long)H * W, 256), 256, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// coef: [3 (a, b, c), 3 channels, F] fp32 on the HOST, or null for no compensation.
extern "C" int solar_tile_blend(const void* tiles, long long st, long long sc, long long sf, void* out, int T,
                                int F, int tH, int tW, int H, int W, int ov, const int* py, const int* px,
                                const float* coef, void* stream) {
  if (T < 1 || T > 32) return fail("tile_blend: 1..32 tiles%s");
  if (F < 1 || F > 4) return fail("tile_blend: 1..4 frames per call%s");
  TileBlendParams p;
  p.tiles = (const __nv_bfloat16*)tiles; p.st = st; p.sc = sc; p.sf = sf; p.out = (float*)out;
  p.T = T; p.F = F; p.tH = tH; p.tW = tW; p.H = H; p.W = W; p.ov = ov;
  for (int t = 0; t < 32; ++t) { p.py[t] = t < T ? py[t] : 0; p.px[t] = t < T ? px[t] : 0; }
  for (int c = 0; c < 3; ++c)
    for (int f = 0; f < 4; ++f) {
      const bool on = coef != nullptr && f < F;
      p.a[c][f] = on ? coef[(0 * 3 + c) * F + f] : 0.f;
      p.b[c][f] = on ? coef[(1 * 3 + c) * F + f] : 0.f;
      p.c[c][f] = on ? coef[(2 * 3 + c) * F + f] : 0.f;
    }
  tile_blend_kernel<<<grid_for((long long)H * W, 256), 256, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_rms_silu_cl(const void* x, void* y, const float* gamma, long long rows, int C, int silu,
                                 void* stream) {
  if (C % 8 != 0 || C > 1024 || C < 8) return fail("rms_silu_cl: C must be a multiple of 8 in [8, 1024]%s");
  if (rows <= 0) return 0;
  const long long blocks = (rows * 32 + 255) / 256;
  rms_silu_cl_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, gamma, rows, C, silu);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}
