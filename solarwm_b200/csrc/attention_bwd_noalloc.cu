// Allocation-free variant of the attention backward entry point; see solar_noalloc.h for who
// needs it, its size limit and its sharing rules.
#include "solar_noalloc.h"

#include "host_util.h"

// Work vectors of the backward pass (L2 and delta), shared by every call on this device.
static __device__ __align__(256) float g_attn_bwd_scratch[SOLAR_ATTN_BWD_NOALLOC_MAX_FLOATS];

extern "C" int solar_attn_bwd_serial(const void* q, const void* k, const void* v, const void* o, const void* dout,
                              const float* lse, void* dq, void* dk, void* dv, float* scratch, int B, int Sq,
                              int Sk, int H, int D, long long q_ss, long long q_sb, long long k_ss,
                              long long k_sb, long long v_ss, long long v_sb, long long o_ss, long long o_sb,
                                     long long do_ss, long long do_sb, float scale, int* status, void* stream);

namespace {

// Filled without a lock: two host threads that race here both store the same address.
float* g_scratch_addr[solar::kMaxDevices] = {nullptr};

// In host code the array's name is only a handle; the address a kernel can use has to be asked
// for, once per device, with that device current.
int scratch_for_current_device(float** out) {
  int dev = 0;
  SOLAR_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= solar::kMaxDevices) return solar::fail("attention backward (no-alloc): device index out of range%s");
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    SOLAR_CUDA_OK(cudaGetSymbolAddress(&p, g_attn_bwd_scratch));
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int solar_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o,
                                      const void* dout, const float* lse, void* dq, void* dk, void* dv, int B,
                                      int Sq, int Sk, int H, int D, long long q_ss, long long q_sb,
                                      long long k_ss, long long k_sb, long long v_ss, long long v_sb,
                                      long long o_ss, long long o_sb, long long do_ss, long long do_sb,
                                      float scale, int* status, void* stream) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0) return solar::fail("attention backward (no-alloc): empty problem%s");
  const long long sq_pad = (static_cast<long long>(Sq) + 127) / 128 * 128;
  const long long need = 2LL * B * H * sq_pad;
  if (need > SOLAR_ATTN_BWD_NOALLOC_MAX_FLOATS)
    return solar::fail("attention backward (no-alloc): needs %s%lld scratch floats, the built-in array holds %lld; "
                       "use solar_attn_bwd with caller-owned scratch",
                       "", need, static_cast<long long>(SOLAR_ATTN_BWD_NOALLOC_MAX_FLOATS));
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // the serial form: all kernels on the caller's stream, so no side stream or event is ever created from here
  return solar_attn_bwd_serial(q, k, v, o, dout, lse, dq, dk, dv, scratch, B, Sq, Sk, H, D, q_ss, q_sb, k_ss, k_sb, v_ss,
                        v_sb, o_ss, o_sb, do_ss, do_sb, scale, status, stream);
}
