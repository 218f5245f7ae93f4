// Allocation-free entry point.  This has no counterpart in the reference: it exists for
// embedders of this library that must not (or cannot) allocate device memory when they call
// into it -- a serving process that handed its whole memory budget to a fixed arena at start-up,
// a plug-in running inside another framework's allocator, a host that forbids cudaMalloc after
// initialisation because an allocation may synchronise the device or fail late under pressure.
//
// solar_attn_bwd_noalloc computes exactly what solar_attn_bwd computes (dq, dk, dv of softmax
// attention) but takes no scratch pointer: the two fp32 work vectors of the backward pass (the
// log2-scaled log-sum-exp and the row dot products O.dO, padded to 128 rows) live in a
// file-scope device array inside the library.
//
// Limits and rules
//   * 2 * B * H * round_up(Sq, 128) must not exceed SOLAR_ATTN_BWD_NOALLOC_MAX_FLOATS
//     (1 Mi floats = 4 MiB).  Larger problems are refused with return code -1 and a message
//     from solar_last_error(); use solar_attn_bwd with caller-owned scratch instead.
//   * Every GPU whose context loads the library holds those 4 MiB until the process exits.
//   * The first call on each device looks up the array's device address (no allocation, but a
//     runtime query): make that first call outside of any stream capture.
//   * All calls on a device share the one array and it keeps the previous call's values.  The
//     backward pass overwrites every element it later reads, so nothing has to be cleared, but
//     two calls whose kernels may overlap on the GPU (different streams, no ordering between
//     them) race on it.  Order such calls on one stream or with events.
//   * The entry point calls no cudaMalloc / cudaFree and no allocating library routine: it runs
//     its three kernels on the caller's stream (the tail-overlap switch of solar_attn_bwd, which
//     creates a side stream and two events, does not apply here).  What its first call on a
//     device does do, besides the address query, is set the kernels' shared-memory attribute
//     (cudaFuncSetAttribute) -- and, in a host thread that has no CUDA context bound yet, bind
//     the device's primary context -- so make that first call part of start-up.
//   * The per-device address cache is filled without a lock; host threads that race on a
//     device's first call store the same value.
#pragma once

#define SOLAR_ATTN_BWD_NOALLOC_MAX_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same tensor conventions as solar_attn_bwd: [B, S, H, D] bf16 with unit stride on D and stride
// D on H; *_ss / *_sb are element strides of the sequence and batch axes; lse is [B, H, Sq] fp32.
int solar_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* dout,
                           const float* lse, void* dq, void* dk, void* dv, int B, int Sq, int Sk, int H, int D,
                           long long q_ss, long long q_sb, long long k_ss, long long k_sb, long long v_ss,
                           long long v_sb, long long o_ss, long long o_sb, long long do_ss, long long do_sb,
                           float scale, int* status, void* stream);

#ifdef __cplusplus
}
#endif
