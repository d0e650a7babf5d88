/* Allocation-free entry point.  (This has no counterpart in the reference project.)
 *
 * Some callers of this library are not allowed to allocate device memory at the moment they need a
 * result: code running inside a memory-pool callback, a real-time inference or control loop whose
 * allocator is frozen after start-up, a plugin hosted by a framework that owns all device memory, or a
 * region where cudaMalloc would synchronise the device.  For them the library offers ONE operation that
 * never allocates: the abs-max reduction (max |x| over a float vector, the norm every QSGD-MaxNorm
 * reducer starts from).
 *
 * The regular abs-max op gets its scratch memory (per-block partial maxima and a ticket counter) from
 * the caller or from torch.  This variant keeps that scratch in a fixed array inside the library image:
 * GCB200_NOALLOC_SCRATCH_BYTES bytes of device memory are held on every GPU that loads the library, from
 * load until process exit.  The caller passes only the input and the output.
 *
 * Rules:
 *  - n must be in [0, GCB200_NOALLOC_MAX_ELEMS]; larger sizes are rejected with GCB200_NOALLOC_E_TOO_LARGE.
 *  - x: device pointer to n floats; out: device pointer to one float; stream: a cudaStream_t (0 = default).
 *  - The first call on a device looks up the device address of the scratch array for that device
 *    (cudaGetSymbolAddress with that device current).  Make that first call outside of any stream capture.
 *  - All calls on a device share the one scratch array.  Two calls that overlap on the GPU (different
 *    streams, no ordering between them) race on it; order them.  The array keeps the contents of the
 *    previous call, so every call re-zeroes the ticket word it depends on before launching.
 *  - No cudaMalloc / cudaFree / allocating library routine is called, on any path.
 *
 * Returns 0 on success, a negative GCB200_NOALLOC_E_* code for a rejected call, or a positive cudaError_t.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GCB200_NOALLOC_MAX_ELEMS (1ll << 30)   /* 4 GiB of fp32 */
#define GCB200_NOALLOC_SCRATCH_BYTES 4352      /* 1024 partial maxima + ticket word, rounded up to 256 */
#define GCB200_NOALLOC_E_BAD_ARG (-1)
#define GCB200_NOALLOC_E_TOO_LARGE (-2)
#define GCB200_NOALLOC_E_NO_DEVICE (-3)

int gcb200_absmax_noalloc(const float* x, int64_t n, float* out, void* stream);

/* Human-readable text for a return code of gcb200_absmax_noalloc. */
const char* gcb200_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
