// RMSNorm backward without any allocation.  This entry point has no counterpart in the reference project.
//
// Who needs it: code that runs where cudaMalloc (and every allocating library call, torch's caching allocator
// included) is off limits — a host callback or a plugin invoked inside someone else's stream-ordered region, a
// process whose memory was fully pre-partitioned at start-up, or a thread that must never take the allocator's lock
// or trigger its implicit device synchronisation.  The regular entry point, mcb_rmsnorm_bwd, expects the caller to
// hand it an fp32 accumulator for the weight gradient, which in practice means allocating one per call.
//
// What it does: the same computation as mcb_rmsnorm_bwd (dx and the weight gradient of
// y = x * rsqrt(mean(x^2) + eps) * w, with w replaced by 1 + w when zero_centered is set), with the fp32
// weight-gradient accumulator kept in a fixed device array inside the library, and the weight gradient returned in
// bf16 in `dw_bf16` (pass NULL to skip it).  The caller provides every input and output buffer.
//
// Limits and rules:
//   * H <= 16384 (the array holds 16384 floats = 64 KiB, resident on every GPU that loads the library until the
//     process exits).  Larger H returns -20 and nothing is launched.  H and ldx must be multiples of 8.
//   * The first call on a device looks up the array's device address; make that first call outside any stream
//     capture.  Later calls on that device do no set-up.
//   * All calls share the one array.  Each call clears the part it uses, but two calls whose kernels can overlap on
//     the GPU (different streams, no ordering between them) race on it: serialise them.
//   * Returns 0 on success, a negative code for bad arguments, or a positive cudaError_t.
//   * No cudaMalloc / cudaFree / allocating library routine is called on any path.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int mcb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, void* dx, void* dw_bf16, long long rows,
                            int H, long long ldx, float eps, int zero_centered, void* stream);

#ifdef __cplusplus
}
#endif
