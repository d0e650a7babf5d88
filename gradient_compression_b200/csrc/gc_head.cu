// The classifier head of the CIFAR models as one forward kernel and two backward kernels: global average pool over the
// last feature map, linear layer, softmax cross-entropy (mean over the batch) and the batch's top-1 / top-5 hit rates.
// The reference runs avg_pool2d + nn.Linear + CrossEntropyLoss + a second CrossEntropyLoss + topk / eq / sum with three
// .item() reads (models/resnet.py:106-108, model_dispatcher.py:127-128,140-164 of the reference): about twenty small
// kernels and three device synchronisations per step.  Here the metrics stay on the device.
//
//   head_fwd_kernel      one block per sample: pooled[n, :] = mean over positions of x[n, :, :] (NHWC), logits = pooled W^T + b,
//                        log-softmax, loss_n, rank of the true class; dlogits[n, :] = (softmax - onehot) / N is written for the
//                        backward pass.  The block that draws the last ticket adds the per-sample values in sample order
//                        (deterministic) into out[0:3] = {mean loss, top-1 rate, top-5 rate}.
//   head_bwd_dx_kernel   dx[n, p, c] = g * sum_k dlogits[n, k] W[k, c] / positions, the same value at every position
//   head_bwd_dw_kernel   dW[k, c] = g * sum_n dlogits[n, k] pooled[n, c], db[k] = g * sum_n dlogits[n, k]
// g is the gradient that reaches the loss (a device scalar, 1 for a plain loss.backward()).
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_device.cuh"

using namespace gc;

namespace {

constexpr int HEAD_THREADS = 256;
constexpr int HEAD_MAX_CLASSES = 32;
constexpr int HEAD_MAX_CHANNELS = 4096;

__global__ void __launch_bounds__(HEAD_THREADS) head_fwd_kernel(const float* __restrict__ x, int positions, int C,
                                                                const float* __restrict__ W, const float* __restrict__ bias, int K,
                                                                const int64_t* __restrict__ labels, int N,
                                                                float* __restrict__ pooled, float* __restrict__ logits,
                                                                float* __restrict__ dlogits, float* __restrict__ per_sample,
                                                                unsigned int* __restrict__ ticket, float* __restrict__ out3) {
  __shared__ __align__(16) float sp[HEAD_MAX_CHANNELS];
  __shared__ float slog[HEAD_MAX_CLASSES];
  __shared__ float spart[HEAD_THREADS / 32][HEAD_MAX_CLASSES];
  __shared__ int last;
  const int n = blockIdx.x;
  const float* xn = x + (int64_t)n * positions * C;
  const float inv_pos = 1.0f / (float)positions;
  for (int q = threadIdx.x; q < (C >> 2); q += HEAD_THREADS) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int p = 0; p < positions; ++p) {
      const float4 v = *reinterpret_cast<const float4*>(xn + (int64_t)p * C + 4 * q);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= inv_pos; acc.y *= inv_pos; acc.z *= inv_pos; acc.w *= inv_pos;
    *reinterpret_cast<float4*>(sp + 4 * q) = acc;
    *reinterpret_cast<float4*>(pooled + (int64_t)n * C + 4 * q) = acc;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    // every warp takes 128-channel slices of the pooled vector and all K classes at once (K independent 16-byte loads of
    // W in flight per lane); the eight warps' partial dot products meet in shared memory in a fixed order
    float acc[HEAD_MAX_CLASSES];
#pragma unroll
    for (int k = 0; k < HEAD_MAX_CLASSES; ++k) acc[k] = 0.f;
    for (int c = warp * 128 + lane * 4; c < C; c += (HEAD_THREADS / 32) * 128) {
      const float4 pv = *reinterpret_cast<const float4*>(sp + c);
#pragma unroll
      for (int k = 0; k < HEAD_MAX_CLASSES; ++k)
        if (k < K) {
          const float4 wv = *reinterpret_cast<const float4*>(W + (int64_t)k * C + c);
          acc[k] = fmaf(pv.x, wv.x, fmaf(pv.y, wv.y, fmaf(pv.z, wv.z, fmaf(pv.w, wv.w, acc[k]))));
        }
    }
#pragma unroll
    for (int k = 0; k < HEAD_MAX_CLASSES; ++k)
      if (k < K) {
        const float v = warp_sum(acc[k]);
        if (lane == 0) spart[warp][k] = v;
      }
    __syncthreads();
    if (threadIdx.x < K) {
      float v = bias != nullptr ? bias[threadIdx.x] : 0.f;
#pragma unroll
      for (int w = 0; w < HEAD_THREADS / 32; ++w) v += spart[w][threadIdx.x];
      slog[threadIdx.x] = v;
      logits[(int64_t)n * K + threadIdx.x] = v;
    }
  }
  __syncthreads();
  if (warp == 0) {
    const int label = (int)labels[n];
    const float z = lane < K ? slog[lane] : -INFINITY;
    const float zmax = warp_max(z);
    const float e = lane < K ? __expf(z - zmax) : 0.f;
    const float denom = warp_sum(e);
    const float zl = (label >= 0 && label < K) ? slog[label] : 0.f;
    // position of the true class in the descending order (ties go to the lower class index, as a stable sort would)
    const int ahead = (lane < K && (z > zl || (z == zl && lane < label))) ? 1 : 0;
    const int rank = __reduce_add_sync(FULL, ahead);
    if (lane < K) dlogits[(int64_t)n * K + lane] = (e / denom - (lane == label ? 1.f : 0.f)) / (float)N;
    if (lane == 0) {
      per_sample[3 * n] = __logf(denom) + zmax - zl;
      per_sample[3 * n + 1] = rank == 0 ? 1.f : 0.f;
      per_sample[3 * n + 2] = rank < 5 ? 1.f : 0.f;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(ticket, 1u) == gridDim.x - 1u ? 1 : 0;
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (threadIdx.x < 3) {
    float acc = 0.f;
    for (int i = 0; i < N; ++i) acc += __ldcg(per_sample + 3 * i + threadIdx.x);
    out3[threadIdx.x] = acc / (float)N;
  }
  if (threadIdx.x == 0) *ticket = 0u;
}

__global__ void __launch_bounds__(HEAD_THREADS) head_bwd_dx_kernel(const float* __restrict__ dlogits, const float* __restrict__ W,
                                                                   const float* __restrict__ g, int positions, int C, int K,
                                                                   float* __restrict__ dx) {
  __shared__ float sd[HEAD_MAX_CLASSES];
  const int n = blockIdx.y;
  if (threadIdx.x < K) sd[threadIdx.x] = dlogits[(int64_t)n * K + threadIdx.x] * (g != nullptr ? *g : 1.f) / (float)positions;
  __syncthreads();
  const int q = blockIdx.x * HEAD_THREADS + threadIdx.x;
  if (q >= (C >> 2)) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < K; ++k) {
    const float4 w = *reinterpret_cast<const float4*>(W + (int64_t)k * C + 4 * q);
    const float d = sd[k];
    acc.x = fmaf(d, w.x, acc.x); acc.y = fmaf(d, w.y, acc.y); acc.z = fmaf(d, w.z, acc.z); acc.w = fmaf(d, w.w, acc.w);
  }
  float* dn = dx + (int64_t)n * positions * C + 4 * q;
  for (int p = 0; p < positions; ++p) *reinterpret_cast<float4*>(dn + (int64_t)p * C) = acc;
}

// One block per 32 channels: warp w sums the samples w, w + 8, ... for its lane's channel and all classes, the eight partial
// sums meet in shared memory.
constexpr int HEAD_DW_CHANNELS = 32;

__global__ void __launch_bounds__(HEAD_THREADS) head_bwd_dw_kernel(const float* __restrict__ dlogits, const float* __restrict__ pooled,
                                                                   const float* __restrict__ g, int N, int C, int K,
                                                                   float* __restrict__ dW, float* __restrict__ db) {
  extern __shared__ float sdl[];                 // dlogits [N, K], then partial sums [8 warps][K][32 channels]
  float* part = sdl + N * K;
  for (int i = threadIdx.x; i < N * K; i += HEAD_THREADS) sdl[i] = dlogits[i];
  __syncthreads();
  const float gs = g != nullptr ? *g : 1.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * HEAD_DW_CHANNELS + lane;
  float acc[HEAD_MAX_CLASSES];
#pragma unroll
  for (int k = 0; k < HEAD_MAX_CLASSES; ++k) acc[k] = 0.f;
  if (c < C) {
    for (int n = warp; n < N; n += HEAD_THREADS / 32) {
      const float pv = pooled[(int64_t)n * C + c];
#pragma unroll
      for (int k = 0; k < HEAD_MAX_CLASSES; ++k)
        if (k < K) acc[k] = fmaf(sdl[n * K + k], pv, acc[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < HEAD_MAX_CLASSES; ++k)
    if (k < K) part[(warp * K + k) * HEAD_DW_CHANNELS + lane] = acc[k];
  __syncthreads();
  for (int i = threadIdx.x; i < K * HEAD_DW_CHANNELS; i += HEAD_THREADS) {
    const int k = i / HEAD_DW_CHANNELS, cc = blockIdx.x * HEAD_DW_CHANNELS + (i % HEAD_DW_CHANNELS);
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < HEAD_THREADS / 32; ++w) sum += part[(w * K + k) * HEAD_DW_CHANNELS + (i % HEAD_DW_CHANNELS)];   // fixed order
    if (cc < C) dW[(int64_t)k * C + cc] = sum * gs;
  }
  if (blockIdx.x == 0 && threadIdx.x < K && db != nullptr) {
    float sum = 0.f;
    for (int n = 0; n < N; ++n) sum += sdl[n * K + threadIdx.x];
    db[threadIdx.x] = sum * gs;
  }
}

}  // namespace

extern "C" {

// 1 when the head kernels cover the shape: C a multiple of 4 up to 4096, at most 32 classes, a batch whose dlogits fit the
// backward kernel's shared memory.
int gc_cuda_head_supported(int N, int positions, int C, int K) {
  return N >= 1 && positions >= 1 && C >= 4 && (C & 3) == 0 && C <= HEAD_MAX_CHANNELS && K >= 1 && K <= HEAD_MAX_CLASSES &&
         (int64_t)N * K * 4 + (HEAD_THREADS / 32) * K * HEAD_DW_CHANNELS * 4 <= 96 * 1024 ? 1 : 0;
}

// Bytes of the zero-initialised scratch (ticket + per-sample values) for batches of up to max_batch samples.
int64_t gc_cuda_head_scratch_bytes(int max_batch) { return 256 + (int64_t)max_batch * 3 * 4; }

// x [N, positions, C] (NHWC feature map), W [K, C], bias [K] or NULL, labels [N] int64.  Writes pooled [N, C], logits [N, K],
// dlogits [N, K] and out3 = {mean cross-entropy, top-1 rate, top-5 rate}.  scratch: gc_cuda_head_scratch_bytes(N), zeroed once.
int gc_cuda_head_forward(const float* x, int N, int positions, int C, const float* W, const float* bias, int K,
                         const int64_t* labels, float* pooled, float* logits, float* dlogits, void* scratch, float* out3, void* cs) {
  if (!gc_cuda_head_supported(N, positions, C, K)) return (int)cudaErrorInvalidValue;
  unsigned int* ticket = static_cast<unsigned int*>(scratch);
  float* per_sample = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + 256);
  head_fwd_kernel<<<N, HEAD_THREADS, 0, (cudaStream_t)cs>>>(x, positions, C, W, bias, K, labels, N, pooled, logits, dlogits, per_sample,
                                                            ticket, out3);
  return (int)cudaGetLastError();
}

// dx [N, positions, C], dW [K, C], db [K] (NULL: no bias) from what the forward kernel saved; g: device scalar (NULL = 1).
int gc_cuda_head_backward(const float* dlogits, const float* pooled, const float* W, const float* g, int N, int positions, int C,
                          int K, float* dx, float* dW, float* db, void* cs) {
  if (!gc_cuda_head_supported(N, positions, C, K)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)cs;
  if (dx != nullptr) {
    dim3 grid((unsigned)(((C >> 2) + HEAD_THREADS - 1) / HEAD_THREADS), (unsigned)N);
    head_bwd_dx_kernel<<<grid, HEAD_THREADS, 0, st>>>(dlogits, W, g, positions, C, K, dx);
  }
  if (dW != nullptr) {
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(head_bwd_dw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      configured = true;
    }
    const size_t smem = (size_t)N * K * 4 + (size_t)(HEAD_THREADS / 32) * K * HEAD_DW_CHANNELS * 4;
    head_bwd_dw_kernel<<<(unsigned)((C + HEAD_DW_CHANNELS - 1) / HEAD_DW_CHANNELS), HEAD_THREADS, smem, st>>>(dlogits, pooled, g, N, C, K,
                                                                                                        dW, db);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
