// Host-side helpers shared by the launchers: error reporting through a thread-local
// message (the C entry points return 0 on success and a negative code otherwise),
// TMA tensor-map encoding through the driver entry point, SM count cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

namespace solar {

inline char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}
inline int fail(const char* fmt, const char* a = "", long long b = 0, long long c = 0) {
  snprintf(last_error_buf(), 512, fmt, a, b, c);
  return -1;
}

#define SOLAR_CUDA_OK(expr)                                                         \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    if (_e != cudaSuccess) {                                                        \
      snprintf(::solar::last_error_buf(), 512, "%s failed: %s (%s:%d)", #expr,      \
               cudaGetErrorString(_e), __FILE__, __LINE__);                         \
      return -2;                                                                    \
    }                                                                               \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// The driver entry point needs a context bound to the calling thread.  A fresh thread whose device is already the
// default one (an autograd worker for device 0: setting device 0 there is a no-op) has none until its first runtime
// call, so an encode that is the thread's very first CUDA call fails with "invalid context": bind the current
// device's primary context (cudaFree(nullptr) does exactly that) and try once more.
template <class... Args>
inline CUresult encode_with_context(EncodeTiledFn fn, Args... args) {
  CUresult r = fn(args...);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    cudaFree(nullptr);
    r = fn(args...);
  }
  return r;
}

// Row-major 2-D tensor [rows, cols] with leading dimension `ld` (elements); the box is
// [box_rows, box_cols] and is stored in shared memory with the 128-byte swizzle, so
// box_cols * elt_bytes must equal 128.
inline int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elt_bytes,
                        uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                        uint32_t box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled entry point not available%s");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail("TMA base not 16-byte aligned%s");
  if ((ld * elt_bytes) % 16 != 0) return fail("TMA row stride not a multiple of 16 bytes%s");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elt_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_with_context(fn, out, dt, 2u, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed (code %s%lld)", "", (long long)r);
  return 0;
}

// 3-D tensor [d2, d1, d0] (d0 innermost) with byte strides s1 (for d1) and s2 (for d2).
inline int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elt_bytes,
                        uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes, uint64_t s2_bytes,
                        uint32_t b0, uint32_t b1, uint32_t b2) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled entry point not available%s");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail("TMA base not 16-byte aligned%s");
  if (s1_bytes % 16 != 0 || s2_bytes % 16 != 0) return fail("TMA stride not a multiple of 16 bytes%s");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  (void)elt_bytes;
  CUresult r = encode_with_context(fn, out, dt, 3u, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled(3d) failed (code %s%lld)", "", (long long)r);
  return 0;
}

// 4-D tensor (d0 innermost) with byte strides for d1..d3; 128-byte swizzle.
inline int make_tmap_4d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, const uint64_t dims[4],
                        const uint64_t strides_bytes[3], const uint32_t box[4]) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled entry point not available%s");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail("TMA base not 16-byte aligned%s");
  for (int i = 0; i < 3; ++i)
    if (strides_bytes[i] % 16 != 0) return fail("TMA stride not a multiple of 16 bytes%s");
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t s[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t b[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t e[4] = {1, 1, 1, 1};
  CUresult r = encode_with_context(fn, out, dt, 4u, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled(4d) failed (code %s%lld)", "", (long long)r);
  return 0;
}

constexpr int kMaxDevices = 64;

inline int current_device_index() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev < 0 || dev >= kMaxDevices) ? 0 : dev;
}

// SM count of the CURRENT device (cached per device: a process may drive several GPUs).
inline int sm_count() {
  static int n[kMaxDevices] = {0};
  const int dev = current_device_index();
  if (n[dev] == 0) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    n[dev] = v > 0 ? v : 148;
  }
  return n[dev];
}

// Function attributes (the dynamic shared-memory limit) are per device: a launcher keeps one
// `PerDeviceOnce` per kernel instantiation and sets the attribute the first time each device launches it.
struct PerDeviceOnce {
  bool done[kMaxDevices] = {false};
  bool first() {
    const int dev = current_device_index();
    if (done[dev]) return false;
    done[dev] = true;
    return true;
  }
};

}  // namespace solar
