// Per-head fused operator of the MiniMax-H3-style attention path (head_dim 128):
//
//   y = PRoPE( MMRoPE( RMSNorm_head(x) * w ) )
//
//   * RMSNorm over the 128 channels of one (token, head) with a bf16/fp32 weight [128]
//   * MM-RoPE: rotate-half inside each of `sections` equal blocks of the first `rot_dims` channels
//     (H3: two blocks of 48 -> pairs (i, i+24)); cos/sin come from a per-token table [S, rot_dims]
//   * PRoPE: every 4-vector of channels [rot_dims, 128) is multiplied by the token's 4x4 camera
//     matrix (identity rows for tokens without a camera); backward applies the transposed matrix
//
// One warp per (token, head); lane l owns channels [4l, 4l+4), so a 4-vector of the PRoPE block is
// lane-local and the rotate-half partner is a fixed lane distance away (one shuffle).  The row is
// read once and written once.  With w == null the normalisation is skipped; with rope == null the
// rotation; with mats == null the camera transform.
//
// Replaces the reference's Triton kernels _qk_norm_rope_fwd/_bwd, _prope_kernel(_v2) and
// _rope_prope_kernel(_v2) (solar/backends/minimax_h3/fused_ops.py:216-469, fused_prope.py:31-472).
#include "host_util.h"
#include "sm100.cuh"

namespace solar {

struct HeadOpParams {
  const __nv_bfloat16* x; long long ld_row;   // [S, H*128], element stride between tokens
  __nv_bfloat16* y; long long ldy_row;
  const float* w;                             // [128] or null
  const float* cos_t; const float* sin_t;     // [S, rot_dims] or null
  const float* mats;                          // [S, 16] row-major 4x4 or null
  float* rstd;                                // [S, H] (written fwd, read bwd) or null
  long long S; int H; int rot_dims; int sections; float eps;
  int backward;
};

__global__ void __launch_bounds__(256) headop_kernel(HeadOpParams p) {
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= p.S * p.H) return;
  const long long tok = gw / p.H;
  const int head = static_cast<int>(gw - tok * p.H);
  const int c0 = lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(p.x + tok * p.ld_row + head * 128 + c0);
  float v[4];
  {
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  const int sec_len = p.sections > 0 ? p.rot_dims / p.sections : 0;   // e.g. 48
  const int half_lanes = sec_len / 8;                                 // partner distance in lanes (6)
  const bool in_rot = p.cos_t != nullptr && c0 < p.rot_dims;
  const bool in_cam = p.mats != nullptr && c0 >= p.rot_dims;

  auto rotate = [&](float (&u)[4], float sign) {
    // rotate-half: out = u * cos + rot(u) * sin, rot(u)[i] = -u[i + half] (first half), u[i - half] (second half)
    const int within = c0 % sec_len;
    const bool first_half = within < sec_len / 2;
    const int partner = first_half ? lane + half_lanes : lane - half_lanes;
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float other = __shfl_sync(0xffffffffu, u[e], partner & 31);
      const float c = p.cos_t[tok * p.rot_dims + c0 + e], s = p.sin_t[tok * p.rot_dims + c0 + e] * sign;
      o[e] = in_rot ? u[e] * c + (first_half ? -other : other) * s : u[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) u[e] = o[e];
  };
  auto camera = [&](float (&u)[4], bool transposed) {
    if (!in_cam) return;
    const float* m = p.mats + tok * 16;
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) acc += (transposed ? m[j * 4 + i] : m[i * 4 + j]) * u[j];
      o[i] = acc;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) u[e] = o[e];
  };

  if (!p.backward) {
    if (p.w != nullptr) {
      float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss / 128.f + p.eps);
      if (lane == 0 && p.rstd) p.rstd[gw] = rstd;
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = v[e] * rstd * p.w[c0 + e];
    }
    if (p.cos_t != nullptr) rotate(v, 1.f);
    camera(v, false);
  } else {
    // v holds dy; undo camera (transpose), undo rotation (negated sine), then the norm backward
    camera(v, true);
    if (p.cos_t != nullptr) rotate(v, -1.f);
  }
  uint2 out;
  out.x = pack_bf16x2(v[0], v[1]);
  out.y = pack_bf16x2(v[2], v[3]);
  *reinterpret_cast<uint2*>(p.y + tok * p.ldy_row + head * 128 + c0) = out;
}

// Backward of the normalisation part: dx = rstd * (g*w - n * mean(g*w*n)), n = x * rstd.
struct HeadNormBwdParams {
  const __nv_bfloat16* g; long long ldg;      // gradient after camera/rotation were undone
  const __nv_bfloat16* xin; long long ldx;    // forward input
  __nv_bfloat16* dx; long long lddx;
  const float* w; const float* rstd;
  long long S; int H;
};
__global__ void __launch_bounds__(256) headnorm_bwd_kernel(HeadNormBwdParams p) {
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= p.S * p.H) return;
  const long long tok = gw / p.H;
  const int head = static_cast<int>(gw - tok * p.H);
  const int c0 = lane * 4;
  const uint2 rg = *reinterpret_cast<const uint2*>(p.g + tok * p.ldg + head * 128 + c0);
  const uint2 rx = *reinterpret_cast<const uint2*>(p.xin + tok * p.ldx + head * 128 + c0);
  const float2 g0 = unpack_bf16x2(rg.x), g1 = unpack_bf16x2(rg.y), x0 = unpack_bf16x2(rx.x), x1 = unpack_bf16x2(rx.y);
  const float rstd = p.rstd[gw];
  float g[4] = {g0.x * p.w[c0], g0.y * p.w[c0 + 1], g1.x * p.w[c0 + 2], g1.y * p.w[c0 + 3]};
  float n[4] = {x0.x * rstd, x0.y * rstd, x1.x * rstd, x1.y * rstd};
  float dot = g[0] * n[0] + g[1] * n[1] + g[2] * n[2] + g[3] * n[3];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  const float m = dot / 128.f;
  uint2 out;
  out.x = pack_bf16x2(rstd * (g[0] - n[0] * m), rstd * (g[1] - n[1] * m));
  out.y = pack_bf16x2(rstd * (g[2] - n[2] * m), rstd * (g[3] - n[3] * m));
  *reinterpret_cast<uint2*>(p.dx + tok * p.lddx + head * 128 + c0) = out;
}

// Streaming ViT decoder step: per-head RMSNorm of q and k, rotate-half rotary over the whole head, and the
// write of k / v straight into their slot of the window cache.  One warp per (row, head); lane l owns the
// channel pairs (j, j + dh/2) for j = l, l + 32, ...  The qkv row is read once; q goes to a packed buffer,
// k and v to cache rows [lo, lo + N) of each batch entry.  Replaces the reference's Triton kernel for the
// decoder step (deploy/.../streaming.py:311-412).
struct VitQkvParams {
  const __nv_bfloat16* qkv; long long ld;     // [B*N, 3*H*dh]
  const float* qw; const float* kw;           // [dh]
  const float* cos_t; const float* sin_t;     // [N, dh] or null
  __nv_bfloat16* q_out;                       // [B*N, H*dh]
  __nv_bfloat16* k_cache; __nv_bfloat16* v_cache; long long cache_batch; long long lo;   // [B, rows, H*dh]
  long long B, N; int H, dh; float eps;
};

__global__ void __launch_bounds__(256) vit_qkv_kernel(VitQkvParams p) {
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= p.B * p.N * p.H) return;
  const long long row = gw / p.H;
  const int head = static_cast<int>(gw - row * p.H);
  const long long b = row / p.N, n = row - b * p.N;
  const int half = p.dh >> 1, a = p.H * p.dh;
  const __nv_bfloat16* src = p.qkv + row * p.ld + head * p.dh;
  const long long crow = b * p.cache_batch + (p.lo + n) * a + head * p.dh;
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* x = src + which * a;
    const float* w = which == 0 ? p.qw : p.kw;
    __nv_bfloat16* dst = which == 0 ? p.q_out + row * a + head * p.dh : p.k_cache + crow;
    float ss = 0.f;
    for (int j = lane; j < half; j += 32) {
      const float x0 = __bfloat162float(x[j]), x1 = __bfloat162float(x[j + half]);
      ss += x0 * x0 + x1 * x1;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / static_cast<float>(p.dh) + p.eps);
    for (int j = lane; j < half; j += 32) {
      // the normalised value is rounded to bf16 before the rotation, as the unfused composition does
      float y0 = __bfloat162float(__float2bfloat16(__bfloat162float(x[j]) * rstd * w[j]));
      float y1 = __bfloat162float(__float2bfloat16(__bfloat162float(x[j + half]) * rstd * w[j + half]));
      if (p.cos_t != nullptr) {
        const float* c = p.cos_t + n * p.dh;
        const float* s = p.sin_t + n * p.dh;
        const float r0 = y0 * c[j] - y1 * s[j];
        const float r1 = y1 * c[j + half] + y0 * s[j + half];
        y0 = r0; y1 = r1;
      }
      dst[j] = __float2bfloat16(y0);
      dst[j + half] = __float2bfloat16(y1);
    }
  }
  const __nv_bfloat16* v = src + 2 * a;
  __nv_bfloat16* vd = p.v_cache + crow;
  for (int j = lane; j < p.dh; j += 32) vd[j] = v[j];
}

}  // namespace solar

using namespace solar;

// Forward (backward = 0) or the camera/rotation part of the backward (backward = 1, w must be null;
// follow with solar_headnorm_bwd when the forward normalised).
extern "C" int solar_headop(const void* x, long long ld_row, void* y, long long ldy_row, const float* w,
                            const float* cos_t, const float* sin_t, const float* mats, float* rstd, long long S,
                            int H, int head_dim, int rot_dims, int sections, float eps, int backward, void* stream) {
  if (head_dim != 128) return fail("headop: head_dim must be 128%s");
  if (cos_t != nullptr && (sections < 1 || rot_dims % (8 * sections) != 0 || rot_dims > 128))
    return fail("headop: rot_dims must split into sections of a multiple of 8 channels%s");
  if (backward && w != nullptr) return fail("headop: backward takes w == null (use solar_headnorm_bwd)%s");
  if (S <= 0 || H <= 0) return 0;
  HeadOpParams p{(const __nv_bfloat16*)x, ld_row, (__nv_bfloat16*)y, ldy_row, w, cos_t, sin_t, mats, rstd, S, H,
                 rot_dims, sections, eps, backward};
  const long long warps = S * H;
  const long long blocks = (warps * 32 + 255) / 256;
  headop_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_headnorm_bwd(const void* g, long long ldg, const void* xin, long long ldx, void* dx,
                                  long long lddx, const float* w, const float* rstd, long long S, int H,
                                  void* stream) {
  if (S <= 0 || H <= 0) return 0;
  HeadNormBwdParams p{(const __nv_bfloat16*)g, ldg, (const __nv_bfloat16*)xin, ldx, (__nv_bfloat16*)dx, lddx, w, rstd, S, H};
  const long long blocks = (S * H * 32 + 255) / 256;
  headnorm_bwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int solar_vit_qkv(const void* qkv, long long ld, const float* qw, const float* kw, const float* cos_t,
                             const float* sin_t, void* q_out, void* k_cache, void* v_cache, long long cache_batch,
                             long long lo, long long B, long long N, int H, int dh, float eps, void* stream) {
  if (dh < 2 || dh % 2 != 0) return fail("vit_qkv: head_dim must be even%s");
  if (B <= 0 || N <= 0 || H <= 0) return 0;
  VitQkvParams p{(const __nv_bfloat16*)qkv, ld, qw, kw, cos_t, sin_t, (__nv_bfloat16*)q_out,
                 (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, cache_batch, lo, B, N, H, dh, eps};
  const long long blocks = (B * N * H * 32 + 255) / 256;
  vit_qkv_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}
