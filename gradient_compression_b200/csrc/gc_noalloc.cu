// Allocation-free abs-max: same reduction as gc_cuda_absmax, with its scratch memory in a file-scope
// device array instead of a caller-provided buffer.  See gc_noalloc.h for who needs this and the rules.
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_device.cuh"
#include "gc_noalloc.h"

using namespace gc;

namespace {

constexpr int kMaxBlocks = 1024;
constexpr int kThreads = 512;
constexpr int kMaxDevices = 64;

struct Scratch {
  float partial[kMaxBlocks];
  unsigned int ticket;
};
static_assert(sizeof(Scratch) <= GCB200_NOALLOC_SCRATCH_BYTES, "scratch array too small");

// Device memory owned by the library image; one instance per GPU that loads it.  In host code this name
// is only a handle for cudaGetSymbolAddress -- it is not a device address and must never be passed to a
// kernel as one.
static __device__ __align__(256) unsigned char g_noalloc_scratch[GCB200_NOALLOC_SCRATCH_BYTES];

// Per-device device address of g_noalloc_scratch, resolved on the first call made on that device.
Scratch* g_scratch_addr[kMaxDevices] = {nullptr};

__global__ void __launch_bounds__(kThreads) absmax_noalloc_kernel(const float* __restrict__ x, int64_t n, bool aligned,
                                                                  Scratch* __restrict__ scratch, float* __restrict__ out) {
  __shared__ float smem[32];
  __shared__ bool is_last;
  float m = 0.0f;
  int64_t nq = (n + 3) / 4;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < nq; q += stride) {
    float4 a = load_quad(x, q * 4, n, aligned);
    m = fmaxf(m, fmaxf(fmaxf(abs_for_max(a.x), abs_for_max(a.y)), fmaxf(abs_for_max(a.z), abs_for_max(a.w))));
  }
  m = block_max(m, smem);
  if (threadIdx.x == 0) {
    scratch->partial[blockIdx.x] = m;
    __threadfence();
    is_last = (atomicAdd(&scratch->ticket, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    float r = 0.0f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) r = fmaxf(r, ((volatile float*)scratch->partial)[i]);
    r = block_max(r, smem);
    if (threadIdx.x == 0) *out = r;
  }
}

}  // namespace

extern "C" int gcb200_absmax_noalloc(const float* x, int64_t n, float* out, void* stream) {
  if (out == nullptr || n < 0 || (n > 0 && x == nullptr)) return GCB200_NOALLOC_E_BAD_ARG;
  if (n > GCB200_NOALLOC_MAX_ELEMS) return GCB200_NOALLOC_E_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return GCB200_NOALLOC_E_NO_DEVICE;
  cudaStream_t st = (cudaStream_t)stream;
  if (g_scratch_addr[dev] == nullptr) {
    // set-up, once per device, with that device current: turn the symbol into its device address
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_addr[dev] = reinterpret_cast<Scratch*>(p);
  }
  Scratch* scratch = g_scratch_addr[dev];
  if (n == 0) return (int)cudaMemsetAsync(out, 0, sizeof(float), st);
  // the array still holds whatever the previous call left: the ticket must start at zero
  e = cudaMemsetAsync(&scratch->ticket, 0, sizeof(unsigned int), st);
  if (e != cudaSuccess) return (int)e;
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  int64_t need = ((n + 3) / 4 + kThreads - 1) / kThreads;
  int64_t cap = (int64_t)sms * 4;
  int grid = (int)(need < cap ? need : cap);
  if (grid > kMaxBlocks) grid = kMaxBlocks;
  if (grid < 1) grid = 1;
  bool aligned = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  absmax_noalloc_kernel<<<grid, kThreads, 0, st>>>(x, n, aligned, scratch, out);
  return (int)cudaGetLastError();
}

extern "C" const char* gcb200_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case GCB200_NOALLOC_E_BAD_ARG: return "gcb200_absmax_noalloc: null pointer or negative size";
    case GCB200_NOALLOC_E_TOO_LARGE:
      return "gcb200_absmax_noalloc: n exceeds GCB200_NOALLOC_MAX_ELEMS (2^30 elements); split the input or use "
             "the allocating entry point";
    case GCB200_NOALLOC_E_NO_DEVICE: return "gcb200_absmax_noalloc: no usable current CUDA device";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "gcb200_absmax_noalloc: unknown error";
  }
}
