// Single-GPU sm_100a kernels: Philox fills, abs-max, stochastic quantise (+pack) / dequantise,
// RandK gather/scatter with on-device index generation, SGD-momentum update.  All are
// bandwidth-bound streaming kernels: 16-byte vector accesses, grid sized to the SM count.
// Plain C ABI launchers (raw device pointers + a cudaStream_t) so no libtorch is involved.
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_common.h"
#include "gc_device.cuh"
#include "gc_perm.h"

using namespace gc;

namespace {

int g_sm_count = 0;
int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

inline int grid_for(int64_t work_items, int threads, int per_sm) {
  int64_t need = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)sm_count() * per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

inline RngKey make_key(uint64_t seed, uint32_t stream, uint32_t step) {
  RngKey k;
  k.k0 = (uint32_t)seed;
  k.k1 = (uint32_t)(seed >> 32);
  k.step = step;
  k.stream = stream;
  return k;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// --------------------------------------------------------------------------- Philox fills
template <int KIND>  // 0 uniform float, 1 normal float, 2 raw u32
__global__ void philox_fill_kernel(RngKey key, const uint32_t* __restrict__ step_offset, int64_t n, void* __restrict__ out_) {
  if (step_offset != nullptr) key.step += *step_offset;      // a device-resident step counter: advances under graph replay
  int64_t nblk = (n + 3) / 4;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblk; b += stride) {
    U4 r = philox_block(key, (uint64_t)b);
    int64_t e0 = b * 4;
    if (KIND == 2) {
      uint32_t* out = (uint32_t*)out_;
      uint32_t w[4] = {r.x, r.y, r.z, r.w};
      if (e0 + 3 < n) *reinterpret_cast<uint4*>(out + e0) = make_uint4(w[0], w[1], w[2], w[3]);
      else for (int j = 0; j < 4 && e0 + j < n; ++j) out[e0 + j] = w[j];
    } else {
      float* out = (float*)out_;
      float4 v;
      if (KIND == 0) {
        v = make_float4(u01(r.x), u01(r.y), u01(r.z), u01(r.w));
      } else {
        float u1 = ((float)(r.x >> 8) + 1.0f) * (1.0f / 16777216.0f);
        float rad = sqrtf(-2.0f * logf(u1));
        float sn, cs;
        sincosf(6.283185307179586f * u01(r.y), &sn, &cs);
        v.x = rad * cs; v.y = rad * sn;
        u1 = ((float)(r.z >> 8) + 1.0f) * (1.0f / 16777216.0f);
        rad = sqrtf(-2.0f * logf(u1));
        sincosf(6.283185307179586f * u01(r.w), &sn, &cs);
        v.z = rad * cs; v.w = rad * sn;
      }
      if (e0 + 3 < n) *reinterpret_cast<float4*>(out + e0) = v;   // cudaMalloc'd / torch buffers are 16B aligned at e0 % 4 == 0
      else {
        float w[4] = {v.x, v.y, v.z, v.w};
        for (int j = 0; j < 4 && e0 + j < n; ++j) out[e0 + j] = w[j];
      }
    }
  }
}

// --------------------------------------------------------------------------- abs-max
// Two-level reduction without a second launch: every block writes its partial maximum to the
// scratch array, takes a ticket, and the block that draws the last ticket reduces the partials,
// writes the result and re-arms the ticket counter (so the scratch never needs clearing).
constexpr int ABSMAX_MAX_BLOCKS = 1024;
struct AbsmaxScratch {
  float partial[ABSMAX_MAX_BLOCKS];
  unsigned int ticket;
  unsigned int pad[3];
};

__global__ void __launch_bounds__(512) absmax_kernel(const float* __restrict__ x, int64_t n, bool aligned,
                                                     AbsmaxScratch* __restrict__ scratch, float* __restrict__ out) {
  __shared__ float smem[32];
  __shared__ bool is_last;
  float m = 0.0f;
  int64_t nq = (n + 3) / 4;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // two independent quads per iteration keep more loads in flight
  for (; q + stride < nq; q += 2 * stride) {
    float4 a = load_quad(x, q * 4, n, aligned);
    float4 b = load_quad(x, (q + stride) * 4, n, aligned);
    m = fmaxf(m, fmaxf(fmaxf(abs_for_max(a.x), abs_for_max(a.y)), fmaxf(abs_for_max(a.z), abs_for_max(a.w))));
    m = fmaxf(m, fmaxf(fmaxf(abs_for_max(b.x), abs_for_max(b.y)), fmaxf(abs_for_max(b.z), abs_for_max(b.w))));
  }
  if (q < nq) {
    float4 a = load_quad(x, q * 4, n, aligned);
    m = fmaxf(m, fmaxf(fmaxf(abs_for_max(a.x), abs_for_max(a.y)), fmaxf(abs_for_max(a.z), abs_for_max(a.w))));
  }
  m = block_max(m, smem);
  if (threadIdx.x == 0) {
    scratch->partial[blockIdx.x] = m;
    __threadfence();
    unsigned int t = atomicAdd(&scratch->ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    float r = 0.0f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) r = fmaxf(r, ((volatile float*)scratch->partial)[i]);
    r = block_max(r, smem);
    if (threadIdx.x == 0) {
      *out = r;
      scratch->ticket = 0;
    }
  }
}

// --------------------------------------------------------------------------- quantise to level containers
template <typename OUT>
__global__ void quantize_levels_kernel(const float* __restrict__ x, int64_t n, bool aligned,
                                       const float* __restrict__ norm_ptr, int s, int mode, RngKey key,
                                       OUT* __restrict__ out) {
  float norm = *norm_ptr;
  float scale = (norm > 0.0f) ? (float)s / norm : 0.0f;
  int64_t nq = (n + 3) / 4;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t qd = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; qd < nq; qd += stride) {
    int64_t e0 = qd * 4;
    float4 v = load_quad(x, e0, n, aligned);
    U4 r = (mode == 0 || mode == 2) ? philox_block(key, (uint64_t)qd) : U4{0, 0, 0, 0};
    float g[4] = {v.x, v.y, v.z, v.w};
    uint32_t rr[4] = {r.x, r.y, r.z, r.w};
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      switch (mode) {
        case 0: q[j] = quantize_level(g[j], scale, s, rr[j]); break;
        case 1: q[j] = quantize_level_biased(g[j], scale, s); break;
        case 2: q[j] = quantize_level_nu(g[j], scale, s, rr[j], false); break;
        default: q[j] = quantize_level_nu(g[j], scale, s, rr[j], true); break;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (e0 + j < n) out[e0 + j] = (OUT)q[j];
  }
}

template <typename IN>
__global__ void dequantize_levels_kernel(const IN* __restrict__ q, int64_t n, const float* __restrict__ norm_ptr,
                                         int s, int world, float* __restrict__ out) {
  float sc = dequant_scale(*norm_ptr, s, world);
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = mul_rn(sc, (float)q[i]);
}

// --------------------------------------------------------------------------- quantise + pack (wire layout)
template <int MW>
__global__ void __launch_bounds__(512) qsgd_pack_kernel(const float* __restrict__ x, int64_t n, bool aligned,
                                                        const float* __restrict__ norm_ptr, int s, RngKey key,
                                                        uint8_t* __restrict__ mags, uint32_t* __restrict__ signs) {
  float norm = *norm_ptr;
  float scale = (norm > 0.0f) ? (float)s / norm : 0.0f;
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  int64_t rows = (n + 127) / 128;
  for (int64_t row = warp; row < rows; row += nwarps) {
    int64_t e0 = row * 128 + lane * 4;
    float4 v = load_quad(x, e0, n, aligned);
    U4 r = philox_block(key, (uint64_t)(e0 >> 2));
    int q0 = quantize_level(v.x, scale, s, r.x);
    int q1 = quantize_level(v.y, scale, s, r.y);
    int q2 = quantize_level(v.z, scale, s, r.z);
    int q3 = quantize_level(v.w, scale, s, r.w);
    int m[4] = {abs(q0), abs(q1), abs(q2), abs(q3)};
    bool sg[4] = {q0 < 0, q1 < 0, q2 < 0, q3 < 0};
    store_row_mags<MW>(mags, row, lane, m);
    store_row_plane(signs, row, lane, sg);
  }
}

template <int MW>
__global__ void __launch_bounds__(512) qsgd_unpack_dequant_kernel(const uint8_t* __restrict__ mags,
                                                                  const uint32_t* __restrict__ signs, int64_t n,
                                                                  bool aligned, const float* __restrict__ norm_ptr,
                                                                  int s, int world, float* __restrict__ out) {
  float sc = dequant_scale(*norm_ptr, s, world);
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  int64_t rows = (n + 127) / 128;
  for (int64_t row = warp; row < rows; row += nwarps) {
    int m[4];
    bool sg[4];
    load_row_mags<MW>(mags, row, lane, m);
    load_row_plane(signs, row, lane, sg);
    float4 v;
    v.x = mul_rn(sc, (float)(sg[0] ? -m[0] : m[0]));
    v.y = mul_rn(sc, (float)(sg[1] ? -m[1] : m[1]));
    v.z = mul_rn(sc, (float)(sg[2] ? -m[2] : m[2]));
    v.w = mul_rn(sc, (float)(sg[3] ? -m[3] : m[3]));
    store_quad(out, row * 128 + lane * 4, n, aligned, v);
  }
}

// Pack / unpack of already-quantised int32 levels (API parity with the host packer).
template <int MW>
__global__ void pack_levels_kernel(const int32_t* __restrict__ q, int64_t n, uint8_t* __restrict__ mags,
                                   uint32_t* __restrict__ signs) {
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  int64_t rows = (n + 127) / 128;
  for (int64_t row = warp; row < rows; row += nwarps) {
    int64_t e0 = row * 128 + lane * 4;
    int m[4];
    bool sg[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int v = (e0 + j < n) ? q[e0 + j] : 0;
      m[j] = abs(v);
      sg[j] = v < 0;
    }
    store_row_mags<MW>(mags, row, lane, m);
    store_row_plane(signs, row, lane, sg);
  }
}
template <int MW>
__global__ void unpack_levels_kernel(const uint8_t* __restrict__ mags, const uint32_t* __restrict__ signs, int64_t n,
                                     int32_t* __restrict__ q) {
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  int64_t rows = (n + 127) / 128;
  for (int64_t row = warp; row < rows; row += nwarps) {
    int64_t e0 = row * 128 + lane * 4;
    int m[4];
    bool sg[4];
    load_row_mags<MW>(mags, row, lane, m);
    load_row_plane(signs, row, lane, sg);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (e0 + j < n) q[e0 + j] = sg[j] ? -m[j] : m[j];
  }
}

// --------------------------------------------------------------------------- RandK
__global__ void randk_gather_kernel(const float* __restrict__ x, PermKey pk, int64_t start, int64_t k,
                                    float* __restrict__ vals, int64_t* __restrict__ idx_out) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < k; i += stride) {
    uint64_t e = perm_eval(pk, (uint64_t)(start + i));
    vals[i] = x[e];
    if (idx_out) idx_out[i] = (int64_t)e;
  }
}
// out[perm(start+i)] = vals[i] * alpha ; with scale_rest != 1 the caller first scales the dense vector.
__global__ void randk_scatter_kernel(float* __restrict__ x, PermKey pk, int64_t start, int64_t k,
                                     const float* __restrict__ vals, float alpha) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < k; i += stride) {
    uint64_t e = perm_eval(pk, (uint64_t)(start + i));
    x[e] = vals[i] * alpha;
  }
}

// --------------------------------------------------------------------------- scale / axpy helpers
__global__ void scale_kernel(float* __restrict__ x, int64_t n, bool aligned, float alpha) {
  int64_t nq = (n + 3) / 4;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < nq; q += stride) {
    float4 v = load_quad(x, q * 4, n, aligned);
    v.x *= alpha; v.y *= alpha; v.z *= alpha; v.w *= alpha;
    store_quad(x, q * 4, n, aligned, v);
  }
}

// --------------------------------------------------------------------------- SGD (momentum, Nesterov, weight decay)
// hyper = {lr, momentum, weight_decay} lives in device memory so that a captured CUDA graph picks
// up a new learning rate without re-capture.
__global__ void __launch_bounds__(512) sgd_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                  float* __restrict__ m, int64_t n, bool aligned,
                                                  const float* __restrict__ hyper, int nesterov) {
  float lr = hyper[0], mu = hyper[1], wd = hyper[2];
  int64_t nq = (n + 3) / 4;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < nq; q += stride) {
    int64_t e0 = q * 4;
    float4 pv = load_quad(p, e0, n, aligned);
    float4 gv = load_quad(g, e0, n, aligned);
    float4 mv = load_quad(m, e0, n, aligned);
    float pp[4] = {pv.x, pv.y, pv.z, pv.w}, gg[4] = {gv.x, gv.y, gv.z, gv.w}, mm[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float d = fmaf(wd, pp[j], gg[j]);
      float mi = fmaf(mu, mm[j], d);
      mm[j] = mi;
      float upd = nesterov ? fmaf(mu, mi, d) : mi;
      pp[j] = fmaf(-lr, upd, pp[j]);
    }
    store_quad(p, e0, n, aligned, make_float4(pp[0], pp[1], pp[2], pp[3]));
    store_quad(m, e0, n, aligned, make_float4(mm[0], mm[1], mm[2], mm[3]));
  }
}

}  // namespace

#define GC_LAUNCH_CHECK() ((int)cudaGetLastError())

// Transposes of many small row-major matrices in one launch (the [Cout, Cin] weights of 1x1 convolutions
// -> [Cin, Cout], the K-major operand of the input-gradient GEMM).  Table rows: {src pointer, dst pointer,
// rows, cols, first tile, source row pitch, destination row pitch} (pitches in floats); a block moves one 32 x 32
// tile through shared memory.  With pitches larger than the matrix, one filter tap of a channels-last R x S filter
// [Cout][tap][Cin] is transposed into tap (R*S - 1 - tap) of [Cin][tap][Cout]: the rotated, channel-swapped filter that
// turns the input gradient of a stride-1 convolution into a forward convolution of the output gradient.
namespace {
constexpr int TR_FIELDS = 7;
__global__ void __launch_bounds__(256) batched_transpose_kernel(const int64_t* __restrict__ tab, int n_seg) {
  __shared__ float tile[32][33];
  int lo = 0, hi = n_seg - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (tab[(int64_t)mid * TR_FIELDS + 4] <= (int64_t)blockIdx.x) lo = mid; else hi = mid - 1;
  }
  const int64_t* t = tab + (int64_t)lo * TR_FIELDS;
  const float* __restrict__ src = reinterpret_cast<const float*>(t[0]);
  float* __restrict__ dst = reinterpret_cast<float*>(t[1]);
  const int rows = (int)t[2], cols = (int)t[3];
  const int64_t src_ld = t[5], dst_ld = t[6];
  const int tiles_c = (cols + 31) / 32;
  const int local = (int)((int64_t)blockIdx.x - t[4]);
  const int r0 = (local / tiles_c) * 32, c0 = (local % tiles_c) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = ty; j < 32; j += 8)
    if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = src[(int64_t)(r0 + j) * src_ld + c0 + tx];
  __syncthreads();
#pragma unroll
  for (int j = ty; j < 32; j += 8)
    if (c0 + j < cols && r0 + tx < rows) dst[(int64_t)(c0 + j) * dst_ld + r0 + tx] = tile[tx][j];
}
}  // namespace

extern "C" {

int gc_cuda_abi_version() { return 3; }

int gc_cuda_sm_count() { return sm_count(); }

// step_offset (device uint32, may be NULL) is added to `step` by the kernel: callers that replay the launch from a CUDA
// graph keep their step counter in device memory.
int gc_cuda_philox_fill(int kind, uint64_t seed, uint32_t stream_id, uint32_t step, const uint32_t* step_offset, int64_t n,
                        void* out, void* cs) {
  if (n <= 0) return 0;
  RngKey key = make_key(seed, stream_id, step);
  int threads = 256, grid = grid_for((n + 3) / 4, threads, 8);
  cudaStream_t st = (cudaStream_t)cs;
  if (kind == 0) philox_fill_kernel<0><<<grid, threads, 0, st>>>(key, step_offset, n, out);
  else if (kind == 1) philox_fill_kernel<1><<<grid, threads, 0, st>>>(key, step_offset, n, out);
  else philox_fill_kernel<2><<<grid, threads, 0, st>>>(key, step_offset, n, out);
  return GC_LAUNCH_CHECK();
}

int64_t gc_cuda_absmax_scratch_bytes() { return (int64_t)sizeof(AbsmaxScratch); }

// scratch: gc_cuda_absmax_scratch_bytes() bytes, zeroed once at allocation; out: one float.
int gc_cuda_absmax(const float* x, int64_t n, void* scratch, float* out, void* cs) {
  int threads = 512;
  int grid = grid_for((n + 3) / 4, threads * 2, 4);
  if (grid > ABSMAX_MAX_BLOCKS) grid = ABSMAX_MAX_BLOCKS;
  absmax_kernel<<<grid, threads, 0, (cudaStream_t)cs>>>(x, n, aligned16(x), (AbsmaxScratch*)scratch, out);
  return GC_LAUNCH_CHECK();
}

int gc_cuda_quantize_levels(const float* x, int64_t n, const float* norm_ptr, int s, int mode, uint64_t seed,
                            uint32_t stream_id, uint32_t step, void* out, int out_elem_size, void* cs) {
  if (n <= 0) return 0;
  RngKey key = make_key(seed, stream_id, step);
  int threads = 256, grid = grid_for((n + 3) / 4, threads, 8);
  cudaStream_t st = (cudaStream_t)cs;
  bool al = aligned16(x);
  if (out_elem_size == 1) quantize_levels_kernel<int8_t><<<grid, threads, 0, st>>>(x, n, al, norm_ptr, s, mode, key, (int8_t*)out);
  else if (out_elem_size == 2) quantize_levels_kernel<int16_t><<<grid, threads, 0, st>>>(x, n, al, norm_ptr, s, mode, key, (int16_t*)out);
  else if (out_elem_size == 4) quantize_levels_kernel<int32_t><<<grid, threads, 0, st>>>(x, n, al, norm_ptr, s, mode, key, (int32_t*)out);
  else return (int)cudaErrorInvalidValue;
  return GC_LAUNCH_CHECK();
}

int gc_cuda_dequantize_levels(const void* q, int elem_size, int64_t n, const float* norm_ptr, int s, int world,
                              float* out, void* cs) {
  if (n <= 0) return 0;
  int threads = 256, grid = grid_for(n, threads, 8);
  cudaStream_t st = (cudaStream_t)cs;
  if (elem_size == 1) dequantize_levels_kernel<int8_t><<<grid, threads, 0, st>>>((const int8_t*)q, n, norm_ptr, s, world, out);
  else if (elem_size == 2) dequantize_levels_kernel<int16_t><<<grid, threads, 0, st>>>((const int16_t*)q, n, norm_ptr, s, world, out);
  else if (elem_size == 4) dequantize_levels_kernel<int32_t><<<grid, threads, 0, st>>>((const int32_t*)q, n, norm_ptr, s, world, out);
  else return (int)cudaErrorInvalidValue;
  return GC_LAUNCH_CHECK();
}

#define GC_DISPATCH_MW(mw, CALL)                     \
  switch (mw) {                                      \
    case 1: { constexpr int MW = 1; CALL; } break;   \
    case 2: { constexpr int MW = 2; CALL; } break;   \
    case 4: { constexpr int MW = 4; CALL; } break;   \
    case 8: { constexpr int MW = 8; CALL; } break;   \
    case 16: { constexpr int MW = 16; CALL; } break; \
    default: return (int)cudaErrorInvalidValue;      \
  }

// mags: mag_bytes(pad128(n), mag_width(bits)) bytes; signs: plane_bytes(pad128(n)) bytes (16B aligned).
int gc_cuda_qsgd_pack(const float* x, int64_t n, const float* norm_ptr, int bits, uint64_t seed, uint32_t stream_id,
                      uint32_t step, void* mags, void* signs, void* cs) {
  if (n <= 0) return 0;
  int s = (1 << bits) - 1, mw = mag_width(bits);
  RngKey key = make_key(seed, stream_id, step);
  int threads = 512, grid = grid_for((n + 3) / 4, threads, 4);
  cudaStream_t st = (cudaStream_t)cs;
  bool al = aligned16(x);
  GC_DISPATCH_MW(mw, (qsgd_pack_kernel<MW><<<grid, threads, 0, st>>>(x, n, al, norm_ptr, s, key, (uint8_t*)mags, (uint32_t*)signs)));
  return GC_LAUNCH_CHECK();
}

int gc_cuda_qsgd_unpack_dequant(const void* mags, const void* signs, int64_t n, const float* norm_ptr, int bits,
                                int world, float* out, void* cs) {
  if (n <= 0) return 0;
  int s = (1 << bits) - 1, mw = mag_width(bits);
  int threads = 512, grid = grid_for((n + 3) / 4, threads, 4);
  cudaStream_t st = (cudaStream_t)cs;
  bool al = aligned16(out);
  GC_DISPATCH_MW(mw, (qsgd_unpack_dequant_kernel<MW><<<grid, threads, 0, st>>>((const uint8_t*)mags, (const uint32_t*)signs, n, al, norm_ptr, s, world, out)));
  return GC_LAUNCH_CHECK();
}

int gc_cuda_pack_levels(const int32_t* q, int64_t n, int mw, void* mags, void* signs, void* cs) {
  if (n <= 0) return 0;
  int threads = 256, grid = grid_for((n + 3) / 4, threads, 8);
  cudaStream_t st = (cudaStream_t)cs;
  GC_DISPATCH_MW(mw, (pack_levels_kernel<MW><<<grid, threads, 0, st>>>(q, n, (uint8_t*)mags, (uint32_t*)signs)));
  return GC_LAUNCH_CHECK();
}

int gc_cuda_unpack_levels(const void* mags, const void* signs, int64_t n, int mw, int32_t* q, void* cs) {
  if (n <= 0) return 0;
  int threads = 256, grid = grid_for((n + 3) / 4, threads, 8);
  cudaStream_t st = (cudaStream_t)cs;
  GC_DISPATCH_MW(mw, (unpack_levels_kernel<MW><<<grid, threads, 0, st>>>((const uint8_t*)mags, (const uint32_t*)signs, n, q)));
  return GC_LAUNCH_CHECK();
}

int gc_cuda_randk_gather(const float* x, int64_t n_total, uint64_t seed, uint32_t pass, int64_t start, int64_t k,
                         float* vals, int64_t* idx_out, void* cs) {
  if (k <= 0) return 0;
  PermKey pk = make_perm_key((uint64_t)n_total, seed, pass);
  int threads = 256, grid = grid_for(k, threads, 4);
  randk_gather_kernel<<<grid, threads, 0, (cudaStream_t)cs>>>(x, pk, start, k, vals, idx_out);
  return GC_LAUNCH_CHECK();
}

int gc_cuda_randk_scatter(float* x, int64_t n_total, uint64_t seed, uint32_t pass, int64_t start, int64_t k,
                          const float* vals, float alpha, void* cs) {
  if (k <= 0) return 0;
  PermKey pk = make_perm_key((uint64_t)n_total, seed, pass);
  int threads = 256, grid = grid_for(k, threads, 4);
  randk_scatter_kernel<<<grid, threads, 0, (cudaStream_t)cs>>>(x, pk, start, k, vals, alpha);
  return GC_LAUNCH_CHECK();
}

int gc_cuda_scale(float* x, int64_t n, float alpha, void* cs) {
  if (n <= 0) return 0;
  int threads = 256, grid = grid_for((n + 3) / 4, threads, 8);
  scale_kernel<<<grid, threads, 0, (cudaStream_t)cs>>>(x, n, aligned16(x), alpha);
  return GC_LAUNCH_CHECK();
}

int gc_cuda_sgd_step(float* p, const float* g, float* m, int64_t n, const float* hyper, int nesterov, void* cs) {
  if (n <= 0) return 0;
  int threads = 512, grid = grid_for((n + 3) / 4, threads, 4);
  bool al = aligned16(p) && aligned16(g) && aligned16(m);
  sgd_kernel<<<grid, threads, 0, (cudaStream_t)cs>>>(p, g, m, n, al, hyper, nesterov);
  return GC_LAUNCH_CHECK();
}

// tab: device table of n_seg rows {src, dst, rows, cols, first tile}; total_tiles = sum of ceil(rows/32) * ceil(cols/32).
int gc_cuda_batched_transpose(const int64_t* tab, int n_seg, int64_t total_tiles, void* cs) {
  if (n_seg <= 0 || total_tiles <= 0) return 0;
  batched_transpose_kernel<<<(unsigned)total_tiles, 256, 0, (cudaStream_t)cs>>>(tab, n_seg);
  return GC_LAUNCH_CHECK();
}

}  // extern "C"
