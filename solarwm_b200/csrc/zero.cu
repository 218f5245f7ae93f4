// Sharded optimizer step fused with its collectives over NVLink peer memory.
//
// Every rank keeps the whole bf16 parameter buffer and the whole fp32 gradient buffer of a flat
// unit in a symmetric (IPC-mapped) heap, but owns the fp32 master / moment state of one contiguous
// shard only.  After backward:
//
//   zero_reduce_kernel      out[i] = sum_r grad_r[shard_off + i]   (peer loads, 16 B per thread and
//                           peer), also accumulates sum(out^2) for the global-norm clip.  This is the
//                           reduce-scatter: each rank pulls only its shard from every peer.
//   zero_adamw_push_kernel  decoupled-weight-decay Adam on the shard in fp32, then the refreshed bf16
//                           parameters are stored into EVERY rank's parameter buffer (peer stores).
//                           This is the all-gather, folded into the optimizer's only pass over memory.
//
// Replaces FSDP1's reduce-scatter + clip_grad_norm_ + AdamW.step + all-gather of the next forward
// (solar/backends/wan22/runtime/distributed.py:73-123, solar/training/optim.py:111-151).
#include "comm.cuh"
#include "host_util.h"
#include "sm100.cuh"

namespace solar {

constexpr int ZERO_MAX_RANKS = 8;
struct ZeroPeers {
  const float* grad[ZERO_MAX_RANKS];     // base of every rank's fp32 gradient buffer
  __nv_bfloat16* param[ZERO_MAX_RANKS];  // base of every rank's bf16 parameter buffer (null: fp32 params)
  float* param32[ZERO_MAX_RANKS];        // base of every rank's fp32 parameter buffer (vector units)
  int n_ranks;
};

__global__ void __launch_bounds__(256) zero_reduce_kernel(ZeroPeers peers, long long shard_off, long long n,
                                                          float* __restrict__ out, float* __restrict__ sumsq) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  float acc = 0.f;
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n; i += stride) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < ZERO_MAX_RANKS; ++r) {
      if (r < peers.n_ranks) {
        const float4 v = *reinterpret_cast<const float4*>(peers.grad[r] + shard_off + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    *reinterpret_cast<float4*>(out + i) = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  __shared__ float part[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 8) {
    acc = part[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffu, acc, o);
    if (threadIdx.x == 0) atomicAdd(sumsq, acc);
  }
}

struct ZeroAdam {
  float lr, beta1, beta2, eps, wd, bc1, bc2, ema_decay;
  const float* grad_scale;   // device scalar (clip coefficient)
  const int* skip;           // device flag: non-zero leaves everything untouched
};

// One contiguous shard of one flat buffer, as the multi-buffer kernel sees it (a table of these lives in device
// memory and is built once).
struct ZeroSegment {
  long long param_off;    // byte offset of the buffer inside every rank's symmetric heap
  long long shard_off;    // first element of this rank's shard
  long long n;            // shard length (multiple of 4)
  long long chunk_begin;  // index of this segment's first work chunk (prefix sum over the table)
  float* master; float* m; float* v; const float* g; float* ema;
  int is_bf16; int pad;
};
constexpr long long ZERO_CHUNK = 8192;   // elements per work chunk

__device__ __forceinline__ void adam4(float (&w)[4], float (&mm)[4], float (&vv)[4], const float (&gg)[4], float lr,
                                      float beta1, float beta2, float eps, float wd, float bc1, float bc2) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    w[e] *= 1.f - lr * wd;
    mm[e] = beta1 * mm[e] + (1.f - beta1) * gg[e];
    vv[e] = beta2 * vv[e] + (1.f - beta2) * gg[e] * gg[e];
    const float denom = sqrtf(vv[e] / bc2) + eps;
    w[e] -= (lr / bc1) * (mm[e] / denom);
  }
}

// AdamW + parameter push over EVERY shard of the table in one launch.  lr and the two bias corrections are read
// from device memory (dyn[0..2]): they change every step, and a captured graph must not freeze them.
__global__ void __launch_bounds__(256)
zero_adamw_push_multi_kernel(const ZeroSegment* __restrict__ table, int n_seg, long long total_chunks, PeerTable heaps,
                             ZeroAdam h, const float* __restrict__ dyn) {
  if (*h.skip != 0) return;
  __shared__ long long s_begin[129];
  for (int i = threadIdx.x; i < n_seg; i += blockDim.x) s_begin[i] = table[i].chunk_begin;
  if (threadIdx.x == 0) s_begin[n_seg] = total_chunks;
  __syncthreads();
  const float gs = *h.grad_scale;
  const float lr = dyn[0], bc1 = dyn[1], bc2 = dyn[2];
  int seg = 0;
  for (long long c = blockIdx.x; c < total_chunks; c += gridDim.x) {
    while (c >= s_begin[seg + 1]) ++seg;
    const ZeroSegment sg = table[seg];
    const long long i0 = (c - sg.chunk_begin) * ZERO_CHUNK;
    const long long i1 = i0 + ZERO_CHUNK < sg.n ? i0 + ZERO_CHUNK : sg.n;
    for (long long i = i0 + threadIdx.x * 4; i < i1; i += blockDim.x * 4) {
      const float4 w4 = *reinterpret_cast<const float4*>(sg.master + i);
      const float4 m4 = *reinterpret_cast<const float4*>(sg.m + i);
      const float4 v4 = *reinterpret_cast<const float4*>(sg.v + i);
      const float4 g4 = *reinterpret_cast<const float4*>(sg.g + i);
      float w[4] = {w4.x, w4.y, w4.z, w4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
      const float gg[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
      adam4(w, mm, vv, gg, lr, h.beta1, h.beta2, h.eps, h.wd, bc1, bc2);
      *reinterpret_cast<float4*>(sg.master + i) = make_float4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<float4*>(sg.m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(sg.v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (sg.ema != nullptr) {
        float4 e4 = *reinterpret_cast<const float4*>(sg.ema + i);
        e4.x = h.ema_decay * e4.x + (1.f - h.ema_decay) * w[0];
        e4.y = h.ema_decay * e4.y + (1.f - h.ema_decay) * w[1];
        e4.z = h.ema_decay * e4.z + (1.f - h.ema_decay) * w[2];
        e4.w = h.ema_decay * e4.w + (1.f - h.ema_decay) * w[3];
        *reinterpret_cast<float4*>(sg.ema + i) = e4;
      }
      if (sg.is_bf16) {
        uint2 packed;
        packed.x = pack_bf16x2(w[0], w[1]);
        packed.y = pack_bf16x2(w[2], w[3]);
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
          if (r < heaps.n)
            *reinterpret_cast<uint2*>(static_cast<uint8_t*>(heaps.base[r]) + sg.param_off + (sg.shard_off + i) * 2) = packed;
      } else {
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
          if (r < heaps.n)
            *reinterpret_cast<float4*>(static_cast<uint8_t*>(heaps.base[r]) + sg.param_off + (sg.shard_off + i) * 4) =
                make_float4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
zero_adamw_push_kernel(ZeroPeers peers, long long shard_off, long long n, float* __restrict__ master,
                       float* __restrict__ m, float* __restrict__ v, const float* __restrict__ g,
                       float* __restrict__ ema, ZeroAdam h) {
  if (*h.skip != 0) return;
  const float gs = *h.grad_scale;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n; i += stride) {
    float4 w4 = *reinterpret_cast<const float4*>(master + i);
    float4 m4 = *reinterpret_cast<const float4*>(m + i);
    float4 v4 = *reinterpret_cast<const float4*>(v + i);
    const float4 g4 = *reinterpret_cast<const float4*>(g + i);
    float w[4] = {w4.x, w4.y, w4.z, w4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
    const float gg[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      w[e] *= 1.f - h.lr * h.wd;
      mm[e] = h.beta1 * mm[e] + (1.f - h.beta1) * gg[e];
      vv[e] = h.beta2 * vv[e] + (1.f - h.beta2) * gg[e] * gg[e];
      const float denom = sqrtf(vv[e] / h.bc2) + h.eps;
      w[e] -= (h.lr / h.bc1) * (mm[e] / denom);
    }
    *reinterpret_cast<float4*>(master + i) = make_float4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (ema != nullptr) {
      float4 e4 = *reinterpret_cast<const float4*>(ema + i);
      e4.x = h.ema_decay * e4.x + (1.f - h.ema_decay) * w[0];
      e4.y = h.ema_decay * e4.y + (1.f - h.ema_decay) * w[1];
      e4.z = h.ema_decay * e4.z + (1.f - h.ema_decay) * w[2];
      e4.w = h.ema_decay * e4.w + (1.f - h.ema_decay) * w[3];
      *reinterpret_cast<float4*>(ema + i) = e4;
    }
    uint2 packed;
    packed.x = pack_bf16x2(w[0], w[1]);
    packed.y = pack_bf16x2(w[2], w[3]);
#pragma unroll
    for (int r = 0; r < ZERO_MAX_RANKS; ++r) {
      if (r < peers.n_ranks) {
        if (peers.param[r] != nullptr)
          *reinterpret_cast<uint2*>(peers.param[r] + shard_off + i) = packed;
        else
          *reinterpret_cast<float4*>(peers.param32[r] + shard_off + i) = make_float4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

}  // namespace solar

using namespace solar;

static int fill_peers(ZeroPeers* zp, void* const* grads, void* const* params, int params_are_bf16, int n_ranks) {
  if (n_ranks < 1 || n_ranks > ZERO_MAX_RANKS) return fail("zero: 1..8 ranks supported%s");
  zp->n_ranks = n_ranks;
  for (int r = 0; r < ZERO_MAX_RANKS; ++r) {
    zp->grad[r] = r < n_ranks && grads ? static_cast<const float*>(grads[r]) : nullptr;
    zp->param[r] = (r < n_ranks && params && params_are_bf16) ? static_cast<__nv_bfloat16*>(params[r]) : nullptr;
    zp->param32[r] = (r < n_ranks && params && !params_are_bf16) ? static_cast<float*>(params[r]) : nullptr;
  }
  return 0;
}

// out[0..n) = sum over ranks of grads[r][shard_off .. shard_off+n); *sumsq += sum(out^2).
// n and shard_off must be multiples of 4; all pointers 16-byte aligned.
extern "C" int solar_zero_reduce(void* const* grads, int n_ranks, long long shard_off, long long n, float* out,
                                 float* sumsq, int max_ctas, void* stream) {
  if (n <= 0) return 0;
  if ((n | shard_off) & 3) return fail("zero reduce: shard offset and length must be multiples of 4%s");
  ZeroPeers zp;
  if (int rc = fill_peers(&zp, grads, nullptr, 1, n_ranks)) return rc;
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = static_cast<long long>(max_ctas > 0 ? max_ctas : sm_count() * 8);
  if (blocks > cap) blocks = cap;
  zero_reduce_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(zp, shard_off, n, out, sumsq);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// AdamW on the shard (fp32 master/m/v/g of length n), then store the new parameters at
// [shard_off, shard_off+n) of every rank's parameter buffer (bf16 or fp32).
extern "C" int solar_zero_adamw_push(void* const* params, int params_are_bf16, int n_ranks, long long shard_off,
                                     long long n, float* master, float* m, float* v, const float* g, float* ema,
                                     float lr, float beta1, float beta2, float eps, float wd, int step,
                                     float ema_decay, const float* grad_scale, const int* skip, int max_ctas,
                                     void* stream) {
  if (n <= 0) return 0;
  if ((n | shard_off) & 3) return fail("zero adamw: shard offset and length must be multiples of 4%s");
  if (step < 1) return fail("zero adamw: step counts from 1%s");
  ZeroPeers zp;
  if (int rc = fill_peers(&zp, nullptr, params, params_are_bf16, n_ranks)) return rc;
  ZeroAdam h{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), ema_decay,
             grad_scale, skip};
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = static_cast<long long>(max_ctas > 0 ? max_ctas : sm_count() * 8);
  if (blocks > cap) blocks = cap;
  zero_adamw_push_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(zp, shard_off, n, master, m, v, g, ema, h);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}

// Size of one table entry, so that the Python side can lay the table out without a second definition.
extern "C" int solar_zero_segment_bytes() { return static_cast<int>(sizeof(ZeroSegment)); }
extern "C" long long solar_zero_chunk_elems() { return ZERO_CHUNK; }

// Fill entry `index` of a HOST copy of the table (the caller uploads the bytes once).
extern "C" int solar_zero_segment_fill(void* host_table, int index, long long param_off, long long shard_off,
                                       long long n, long long chunk_begin, float* master, float* m, float* v,
                                       const float* g, float* ema, int is_bf16) {
  if ((n | shard_off) & 3) return fail("zero segment: shard offset and length must be multiples of 4%s");
  ZeroSegment* t = static_cast<ZeroSegment*>(host_table) + index;
  t->param_off = param_off; t->shard_off = shard_off; t->n = n; t->chunk_begin = chunk_begin;
  t->master = master; t->m = m; t->v = v; t->g = g; t->ema = ema; t->is_bf16 = is_bf16; t->pad = 0;
  return 0;
}

// AdamW + parameter push over all `n_seg` shards of the device table in ONE launch.  heap_bases[r]: rank r's
// symmetric heap; dyn: device fp32 [3] = {lr, 1 - beta1^t, 1 - beta2^t}, refreshed by the caller every step.
extern "C" int solar_zero_adamw_push_multi(const void* table_dev, int n_seg, long long total_chunks,
                                           void* const* heap_bases, int n_ranks, float beta1, float beta2, float eps,
                                           float wd, float ema_decay, const float* dyn, const float* grad_scale,
                                           const int* skip, int max_ctas, void* stream) {
  if (n_seg < 1 || n_seg > 128) return fail("zero adamw multi: 1..128 segments%s");
  if (n_ranks < 1 || n_ranks > kMaxPeers) return fail("zero: 1..8 ranks supported%s");
  if (total_chunks <= 0) return 0;
  PeerTable heaps;
  heaps.n = n_ranks;
  for (int i = 0; i < kMaxPeers; ++i) heaps.base[i] = i < n_ranks ? heap_bases[i] : nullptr;
  ZeroAdam h{0.f, beta1, beta2, eps, wd, 1.f, 1.f, ema_decay, grad_scale, skip};
  long long blocks = total_chunks;
  const long long cap = static_cast<long long>(max_ctas > 0 ? max_ctas : sm_count() * 8);
  if (blocks > cap) blocks = cap;
  zero_adamw_push_multi_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      static_cast<const ZeroSegment*>(table_dev), n_seg, total_chunks, heaps, h, dyn);
  SOLAR_CUDA_OK(cudaGetLastError());
  return 0;
}
