// Device-side building blocks shared by the sm_100a kernels: vector loads, warp/block reductions,
// the row codec (one warp <-> one 128-element row of the packed wire layout) and bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>
#include "gc_common.h"

namespace gc {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}

// Block-wide max; result valid in every thread.  smem must hold 32 floats.
__device__ __forceinline__ float block_max(float v, float* smem) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  float r = (lane < nw) ? smem[lane] : 0.0f;
  r = warp_max(r);
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* smem) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  float r = (lane < nw) ? smem[lane] : 0.0f;
  r = warp_sum(r);
  return r;
}

// |x| with NaN propagated as +inf so that a poisoned gradient shows up in the norm.
__device__ __forceinline__ float abs_for_max(float x) {
  float a = fabsf(x);
  return (a == a) ? a : __int_as_float(0x7f800000);
}

// Load the quad (4 consecutive floats) starting at element e0 (a multiple of 4); zero beyond n.
// The base pointer must be 16-byte aligned for the vector path; `aligned` says whether it is.
__device__ __forceinline__ float4 load_quad(const float* __restrict__ x, int64_t e0, int64_t n, bool aligned) {
  if (aligned && e0 + 3 < n) return *reinterpret_cast<const float4*>(x + e0);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (e0 < n) v.x = x[e0];
  if (e0 + 1 < n) v.y = x[e0 + 1];
  if (e0 + 2 < n) v.z = x[e0 + 2];
  if (e0 + 3 < n) v.w = x[e0 + 3];
  return v;
}
__device__ __forceinline__ void store_quad(float* __restrict__ x, int64_t e0, int64_t n, bool aligned, float4 v) {
  if (aligned && e0 + 3 < n) { *reinterpret_cast<float4*>(x + e0) = v; return; }
  if (e0 < n) x[e0] = v.x;
  if (e0 + 1 < n) x[e0 + 1] = v.y;
  if (e0 + 2 < n) x[e0 + 2] = v.z;
  if (e0 + 3 < n) x[e0 + 3] = v.w;
}

// ---- row codec ------------------------------------------------------------------------------
// A warp owns row `row` (elements row*128 .. row*128+127); lane owns the quad at 4*lane.
// Magnitudes are stored in natural element order at MW bits each; bit planes as ballot words.
template <int MW>
__device__ __forceinline__ void store_row_mags(uint8_t* __restrict__ mags, int64_t row, int lane, const int (&m)[4]) {
  if (MW == 16) {
    uint2 v;
    v.x = (uint32_t)m[0] | ((uint32_t)m[1] << 16);
    v.y = (uint32_t)m[2] | ((uint32_t)m[3] << 16);
    reinterpret_cast<uint2*>(mags)[row * 32 + lane] = v;
  } else if (MW == 8) {
    uint32_t v = (uint32_t)m[0] | ((uint32_t)m[1] << 8) | ((uint32_t)m[2] << 16) | ((uint32_t)m[3] << 24);
    reinterpret_cast<uint32_t*>(mags)[row * 32 + lane] = v;
  } else if (MW == 4) {
    uint16_t v = (uint16_t)(m[0] | (m[1] << 4) | (m[2] << 8) | (m[3] << 12));
    reinterpret_cast<uint16_t*>(mags)[row * 32 + lane] = v;
  } else if (MW == 2) {
    uint8_t v = (uint8_t)(m[0] | (m[1] << 2) | (m[2] << 4) | (m[3] << 6));
    mags[row * 32 + lane] = v;
  } else {  // MW == 1: two lanes share a byte
    uint32_t v = (uint32_t)(m[0] | (m[1] << 1) | (m[2] << 2) | (m[3] << 3));
    uint32_t hi = __shfl_down_sync(FULL, v, 1);
    if ((lane & 1) == 0) mags[row * 16 + (lane >> 1)] = (uint8_t)(v | (hi << 4));
  }
}

template <int MW>
__device__ __forceinline__ void load_row_mags(const uint8_t* __restrict__ mags, int64_t row, int lane, int (&m)[4]) {
  if (MW == 16) {
    uint2 v = reinterpret_cast<const uint2*>(mags)[row * 32 + lane];
    m[0] = v.x & 0xffff; m[1] = v.x >> 16; m[2] = v.y & 0xffff; m[3] = v.y >> 16;
  } else if (MW == 8) {
    uint32_t v = reinterpret_cast<const uint32_t*>(mags)[row * 32 + lane];
    m[0] = v & 0xff; m[1] = (v >> 8) & 0xff; m[2] = (v >> 16) & 0xff; m[3] = v >> 24;
  } else if (MW == 4) {
    uint32_t v = reinterpret_cast<const uint16_t*>(mags)[row * 32 + lane];
    m[0] = v & 0xf; m[1] = (v >> 4) & 0xf; m[2] = (v >> 8) & 0xf; m[3] = (v >> 12) & 0xf;
  } else if (MW == 2) {
    uint32_t v = mags[row * 32 + lane];
    m[0] = v & 3; m[1] = (v >> 2) & 3; m[2] = (v >> 4) & 3; m[3] = (v >> 6) & 3;
  } else {
    uint32_t v = mags[row * 16 + (lane >> 1)];
    v = (lane & 1) ? (v >> 4) : v;
    m[0] = v & 1; m[1] = (v >> 1) & 1; m[2] = (v >> 2) & 1; m[3] = (v >> 3) & 1;
  }
}

// Bit plane of a row: 4 ballot words (word j, bit lane <-> element 4*lane + j).
__device__ __forceinline__ void store_row_plane(uint32_t* __restrict__ plane, int64_t row, int lane, const bool (&b)[4]) {
  uint32_t w0 = __ballot_sync(FULL, b[0]);
  uint32_t w1 = __ballot_sync(FULL, b[1]);
  uint32_t w2 = __ballot_sync(FULL, b[2]);
  uint32_t w3 = __ballot_sync(FULL, b[3]);
  if (lane == 0) reinterpret_cast<uint4*>(plane)[row] = make_uint4(w0, w1, w2, w3);
}
__device__ __forceinline__ void load_row_plane(const uint32_t* __restrict__ plane, int64_t row, int lane, bool (&b)[4]) {
  uint4 w = reinterpret_cast<const uint4*>(plane)[row];   // same address in every lane: one transaction
  b[0] = (w.x >> lane) & 1u; b[1] = (w.y >> lane) & 1u; b[2] = (w.z >> lane) & 1u; b[3] = (w.w >> lane) & 1u;
}

// ---- system-scope flags with bounded waits -------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}


// ---- programmatic dependent launch ---------------------------------------------------------------
// A kernel launched with launch_pdl() may be scheduled while the previous kernel of its stream is still
// draining, which hides its launch latency and prologue.  Such a kernel calls pdl_wait() before it touches
// memory (the wait returns once the previous kernel has completed and its writes are visible; it returns at once
// in a kernel launched the ordinary way), and pdl_launch_dependents() to let its own successor be scheduled.
// Off unless GCB200_PDL=1: inside a replayed CUDA graph, where the training step runs, kernel-to-kernel gaps are
// already about a microsecond.  Measured on the ResNet-50 step: with an explicit trigger at the top of every kernel 1.8 % slower
// (successors become resident while their predecessor is in full flight), with the implicit trigger at block exit 0.15 %
// faster (17 219 / 17 214 against 17 187 / 17 191 img/s); eager (uncaptured) loops are where it can pay.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
#if defined(GC_PDL_EARLY_TRIGGER)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");       // at the top of a kernel: successors become resident at once
#endif
  // default: no explicit trigger -- the successor is released as this kernel's blocks exit, so only its launch latency and
  // prologue overlap this kernel's tail, and it never takes SM resources from a kernel that is still in full flight
}

inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("GCB200_PDL");
    on = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace gc
