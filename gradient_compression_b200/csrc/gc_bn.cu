// Fused batch-norm (+ residual add) (+ ReLU), forward and backward, for NHWC fp32 activations
// x[M, C] with M = N*H*W.  Replaces the reference's chain  bn -> (+= shortcut) -> relu  (resnet.py:71-75,
// vgg.py:105-106), which costs 3 kernels and ~6 passes over the activation forward and ~8 backward, by
//   forward : stats (1 read)  +  apply (1 read [+1 residual], 1 write)
//   backward: reduce (2-3 reads) + apply (2-3 reads, 1-2 writes)
// The ReLU mask is never stored: it is recomputed from x (or read from the saved output when a
// residual was added).  Both "apply" kernels walk the tensor in REVERSE tile order so that they start
// with the lines the preceding reduction touched last and find them in the 126 MB L2.
// Reductions are deterministic: per-block partial sums go to scratch memory and a small second kernel
// (32 channels per block, coalesced over the partials) combines them in double precision.
// Where a 2x2 max-pool follows (vgg.py:101-103 of the reference: conv, bn, relu, ..., MaxPool2d), the *_pool variants fold it
// in: the forward writes only the pooled map, the backward routes the pooled gradient to each window's winner.
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_device.cuh"

using namespace gc;

namespace {

constexpr int BN_THREADS = 512;
constexpr int BN_MAX_BLOCKS = 296;   // 148 SMs x 2 resident blocks of 512 threads (about 50 registers per thread)

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

// Per-block accumulation of two per-channel sums.  Thread t owns the float4 column (t % vec) and visits
// rows (t / vec) + k * (BN_THREADS / vec).  Requires C % 4 == 0, vec = C / 4 <= BN_THREADS and
// BN_THREADS % vec == 0.  F(row-quad data) -> two float4 contributions.
// acc != NULL: the block's sums are added to acc[0:C] / acc[C:2C] (doubles) with atomics instead of being written to
// partial_out.
template <typename F>
__device__ __forceinline__ void block_two_sums(int64_t M, int C, int64_t row_begin, int64_t row_end, F f,
                                               float* __restrict__ partial_out /* [2C] for this block */,
                                               double* __restrict__ acc = nullptr) {
  extern __shared__ float smem[];   // 2 * BN_THREADS * 4 floats
  const int vec = C >> 2;
  const int col = threadIdx.x % vec;
  const int rofs = threadIdx.x / vec;
  const int rstep = BN_THREADS / vec;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
  if (row_end >= 0) {
#pragma unroll 4
    for (int64_t r = row_begin + rofs; r < row_end; r += rstep) f(r, col, a, b);
  } else {
    // interleaved mode (row_end < 0): the grid walks the tensor from its END in chunks of 4 * rstep rows, block b taking the
    // chunks b, b + gridDim.x, ...: the kernel that runs before a backward reduction wrote the gradient it reads, and the
    // end of that tensor is what the L2 still holds
    const int64_t chunk = (int64_t)rstep * 4;
    for (int64_t hi = M - (int64_t)blockIdx.x * chunk; hi > 0; hi -= (int64_t)gridDim.x * chunk) {
      const int64_t lo = hi - chunk;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t r = lo + rofs + (int64_t)k * rstep;
        if (r >= 0) f(r, col, a, b);
      }
    }
  }
  float4* sa = reinterpret_cast<float4*>(smem);
  float4* sb = sa + BN_THREADS;
  sa[threadIdx.x] = a;
  sb[threadIdx.x] = b;
  __syncthreads();
  // tree over the rstep threads that share a column
  for (int s = rstep >> 1; s > 0; s >>= 1) {
    if (rofs < s) {
      float4 o = sa[threadIdx.x + s * vec], p = sb[threadIdx.x + s * vec];
      float4 m = sa[threadIdx.x], q = sb[threadIdx.x];
      sa[threadIdx.x] = make_float4(m.x + o.x, m.y + o.y, m.z + o.z, m.w + o.w);
      sb[threadIdx.x] = make_float4(q.x + p.x, q.y + p.y, q.z + p.z, q.w + p.w);
    }
    __syncthreads();
  }
  if (threadIdx.x < vec) {
    if (acc != nullptr) {
      const float4 a4 = sa[threadIdx.x], b4 = sb[threadIdx.x];
      double* pa = acc + 4 * threadIdx.x;
      double* pb = acc + C + 4 * threadIdx.x;
      atomicAdd(pa, (double)a4.x); atomicAdd(pa + 1, (double)a4.y); atomicAdd(pa + 2, (double)a4.z); atomicAdd(pa + 3, (double)a4.w);
      atomicAdd(pb, (double)b4.x); atomicAdd(pb + 1, (double)b4.y); atomicAdd(pb + 2, (double)b4.z); atomicAdd(pb + 3, (double)b4.w);
    } else {
      st4(partial_out + 4 * threadIdx.x, sa[threadIdx.x]);
      st4(partial_out + C + 4 * threadIdx.x, sb[threadIdx.x]);
    }
  }
}

// After block_two_sums(..., acc): the block that draws the last ticket finds every block's contribution in acc, writes
// the totals as floats and leaves acc and the ticket zeroed for the next launch.
__device__ __forceinline__ void finish_two_sums(int C, double* __restrict__ acc, unsigned int* __restrict__ ticket,
                                                float* __restrict__ sums) {
  __shared__ int last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(ticket, 1u) == gridDim.x - 1u ? 1 : 0;
  __syncthreads();
  if (!last) return;
  __threadfence();
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) {
    sums[i] = (float)__ldcg(&acc[i]);
    acc[i] = 0.0;
  }
  if (threadIdx.x == 0) *ticket = 0u;
}

// Combine the per-block partials of blockDim.x consecutive channels (both sums) in double precision.
// block = (channels, FY, 2) with channels * FY <= 512: x = channel in the group, y strides over partial blocks, z = which of
// the two sums.  (32, 16, 2) by default; (8, 64, 2) when there are many partials of few channels (the 1024 row tiles of a
// 64- or 256-channel first-stage layer), which cuts the serial loads per thread fourfold.
constexpr int FIN_Y = 16;
__device__ __forceinline__ void combine_partials(const float* __restrict__ partials, int nparts, int C, double (&out)[2]) {
  __shared__ double red[2][512];
  const int cx = blockDim.x, fy = blockDim.y;
  int c = blockIdx.x * cx + threadIdx.x;
  double acc = 0.0;
  if (c < C) {
    const float* base = partials + threadIdx.z * C + c;
    int b = threadIdx.y;
    for (; b + 3 * fy < nparts; b += 4 * fy) {   // four independent loads in flight per thread
      float v0 = base[(int64_t)b * 2 * C], v1 = base[(int64_t)(b + fy) * 2 * C];
      float v2 = base[(int64_t)(b + 2 * fy) * 2 * C], v3 = base[(int64_t)(b + 3 * fy) * 2 * C];
      acc += ((double)v0 + (double)v1) + ((double)v2 + (double)v3);
    }
    for (; b < nparts; b += fy) acc += (double)base[(int64_t)b * 2 * C];
  }
  red[threadIdx.z][threadIdx.y * cx + threadIdx.x] = acc;
  __syncthreads();
  out[0] = out[1] = 0.0;
  if (threadIdx.y == 0 && threadIdx.z == 0) {
    for (int k = 0; k < fy; ++k) { out[0] += red[0][k * cx + threadIdx.x]; out[1] += red[1][k * cx + threadIdx.x]; }
  }
}

// Launch shape of the two finalize kernels for `nparts` partial rows of C channels.
inline void finalize_shape(int nparts, int C, dim3* grid, dim3* block) {
  const int cx = (nparts >= 256 && C <= 256) ? 8 : 32;
  *block = cx == 8 ? dim3(8, 64, 2) : dim3(32, FIN_Y, 2);
  *grid = dim3((C + cx - 1) / cx);
}

// ---------------------------------------------------------------------------------- forward statistics
// out stats[0:C] = mean, stats[C:2C] = rstd; running stats updated in place when given.
__global__ void __launch_bounds__(BN_THREADS) bn_stats_kernel(const float* __restrict__ x, int64_t M, int C,
                                                              int64_t rows_per_block, float* __restrict__ partials) {
  pdl_wait();
  pdl_launch_dependents();
  int64_t r0 = (int64_t)blockIdx.x * rows_per_block;
  int64_t r1 = r0 + rows_per_block < M ? r0 + rows_per_block : M;
  // shifted sums: k = the channel's value in row 0, so that sum (x-k)^2 does not cancel against
  // (sum (x-k))^2 when |mean| is large compared with the standard deviation
  const float4 k = ld4(x + 4 * (threadIdx.x % (C >> 2)));
  block_two_sums(M, C, r0, r1,
                 [&](int64_t r, int col, float4& a, float4& b) {
                   float4 v = ld4(x + r * C + 4 * col);
                   v.x -= k.x; v.y -= k.y; v.z -= k.z; v.w -= k.w;
                   a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
                   b.x = fmaf(v.x, v.x, b.x); b.y = fmaf(v.y, v.y, b.y); b.z = fmaf(v.z, v.z, b.z); b.w = fmaf(v.w, v.w, b.w);
                 },
                 partials + (int64_t)blockIdx.x * 2 * C);
}

__global__ void bn_stats_finalize_kernel(const float* __restrict__ partials, const float* __restrict__ x, int nparts,
                                         int64_t M, int C, float* __restrict__ stats, float* __restrict__ running_mean,
                                         float* __restrict__ running_var, float momentum, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  double sums[2];
  combine_partials(partials, nparts, C, sums);
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (threadIdx.y != 0 || threadIdx.z != 0 || c >= C) return;
  double dmean = sums[0] / (double)M;              // mean of the shifted values
  double var = sums[1] / (double)M - dmean * dmean;
  if (var < 0.0) var = 0.0;
  double mean = (x != nullptr ? (double)x[c] : 0.0) + dmean;     // x == NULL: the partials are unshifted sums
  stats[c] = (float)mean;
  stats[C + c] = (float)(1.0 / sqrt(var + (double)eps));
  if (running_mean != nullptr) {
    double unbiased = M > 1 ? var * (double)M / (double)(M - 1) : var;
    running_mean[c] = (1.0f - momentum) * running_mean[c] + momentum * (float)mean;
    running_var[c] = (1.0f - momentum) * running_var[c] + momentum * (float)unbiased;
  }
}

// ---------------------------------------------------------------------------------- forward apply
// y = act(gamma * (x - mean) * rstd + beta [+ residual]); quads visited from the end of the tensor backwards.
__global__ void __launch_bounds__(BN_THREADS) bn_apply_kernel(const float* __restrict__ x, int64_t M, int C,
                                                              const float* __restrict__ stats,
                                                              const float* __restrict__ gamma, const float* __restrict__ beta,
                                                              const float* __restrict__ residual, int relu,
                                                              float* __restrict__ y) {
  pdl_wait();
  pdl_launch_dependents();
  const int vec = C >> 2;
  const int64_t nq = M * vec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nq; i += stride) {
    int64_t q = nq - 1 - i;
    int c4 = (int)(q % vec) * 4;
    float4 v = ld4(x + q * 4);
    float4 mu = ld4(stats + c4), rs = ld4(stats + C + c4), g = ld4(gamma + c4), b = ld4(beta + c4);
    float4 o;
    o.x = fmaf((v.x - mu.x) * rs.x, g.x, b.x);
    o.y = fmaf((v.y - mu.y) * rs.y, g.y, b.y);
    o.z = fmaf((v.z - mu.z) * rs.z, g.z, b.z);
    o.w = fmaf((v.w - mu.w) * rs.w, g.w, b.w);
    if (residual != nullptr) {
      float4 r = ld4(residual + q * 4);
      o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
    }
    if (relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
    st4(y + q * 4, o);
  }
}

// ---------------------------------------------------------------------------------- backward reduce
// g = dy * mask (mask = act output > 0; from the saved output y when given, else recomputed from x);
// sums[0:C] = sum g (= dbeta), sums[C:2C] = sum g * xhat (= dgamma).
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_reduce_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                   const float* __restrict__ y, int64_t M, int C,
                                                                   int64_t rows_per_block, const float* __restrict__ stats,
                                                                   const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                   int relu, float* __restrict__ partials, double* __restrict__ acc,
                                                                   unsigned int* __restrict__ ticket, float* __restrict__ sums,
                                                                   int g_interleave) {
  pdl_wait();
  pdl_launch_dependents();
  int64_t r0 = (int64_t)blockIdx.x * rows_per_block;
  int64_t r1 = r0 + rows_per_block < M ? r0 + rows_per_block : M;
  if (g_interleave) r1 = -1;                      // block_two_sums: chunks from the end of the tensor, round-robin over blocks
  const int col = threadIdx.x % (C >> 2);
  const float4 mu = ld4(stats + 4 * col), rs = ld4(stats + C + 4 * col);
  const float4 gm = ld4(gamma + 4 * col), bt = ld4(beta + 4 * col);
  block_two_sums(M, C, r0, r1,
                 [&](int64_t r, int cc, float4& a, float4& b) {
                   float4 d = ld4(dy + r * C + 4 * cc);
                   float4 v = ld4(x + r * C + 4 * cc);
                   float4 xh = make_float4((v.x - mu.x) * rs.x, (v.y - mu.y) * rs.y, (v.z - mu.z) * rs.z, (v.w - mu.w) * rs.w);
                   if (relu) {
                     if (y != nullptr) {
                       float4 o = ld4(y + r * C + 4 * cc);
                       d.x = o.x > 0.f ? d.x : 0.f; d.y = o.y > 0.f ? d.y : 0.f; d.z = o.z > 0.f ? d.z : 0.f; d.w = o.w > 0.f ? d.w : 0.f;
                     } else {
                       d.x = fmaf(xh.x, gm.x, bt.x) > 0.f ? d.x : 0.f; d.y = fmaf(xh.y, gm.y, bt.y) > 0.f ? d.y : 0.f;
                       d.z = fmaf(xh.z, gm.z, bt.z) > 0.f ? d.z : 0.f; d.w = fmaf(xh.w, gm.w, bt.w) > 0.f ? d.w : 0.f;
                     }
                   }
                   a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
                   b.x = fmaf(d.x, xh.x, b.x); b.y = fmaf(d.y, xh.y, b.y); b.z = fmaf(d.z, xh.z, b.z); b.w = fmaf(d.w, xh.w, b.w);
                 },
                 partials + (int64_t)blockIdx.x * 2 * C, acc);
  if (acc != nullptr) finish_two_sums(C, acc, ticket, sums);
}

__global__ void bn_sums_finalize_kernel(const float* __restrict__ partials, int nparts, int C, float* __restrict__ sums) {
  pdl_wait();
  pdl_launch_dependents();
  double out[2];
  combine_partials(partials, nparts, C, out);
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (threadIdx.y != 0 || threadIdx.z != 0 || c >= C) return;
  sums[c] = (float)out[0];
  sums[C + c] = (float)out[1];
}

// ---------------------------------------------------------------------------------- backward apply
// dx = gamma * rstd * (g - dbeta / M - xhat * dgamma / M); optionally dres = g (gradient of the residual).
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_apply_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                  const float* __restrict__ y, int64_t M, int C,
                                                                  const float* __restrict__ stats, const float* __restrict__ gamma,
                                                                  const float* __restrict__ beta, const float* __restrict__ sums,
                                                                  int relu, float* __restrict__ dx, float* __restrict__ dres) {
  pdl_wait();
  pdl_launch_dependents();
  const int vec = C >> 2;
  const int64_t nq = M * vec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float inv_m = 1.0f / (float)M;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nq; i += stride) {
    int64_t q = nq - 1 - i;
    int c4 = (int)(q % vec) * 4;
    float4 d = ld4(dy + q * 4), v = ld4(x + q * 4);
    float4 mu = ld4(stats + c4), rs = ld4(stats + C + c4), gm = ld4(gamma + c4);
    float4 db = ld4(sums + c4), dg = ld4(sums + C + c4);
    float4 xh = make_float4((v.x - mu.x) * rs.x, (v.y - mu.y) * rs.y, (v.z - mu.z) * rs.z, (v.w - mu.w) * rs.w);
    if (relu) {
      if (y != nullptr) {
        float4 o = ld4(y + q * 4);
        d.x = o.x > 0.f ? d.x : 0.f; d.y = o.y > 0.f ? d.y : 0.f; d.z = o.z > 0.f ? d.z : 0.f; d.w = o.w > 0.f ? d.w : 0.f;
      } else {
        float4 bt = ld4(beta + c4);
        d.x = fmaf(xh.x, gm.x, bt.x) > 0.f ? d.x : 0.f; d.y = fmaf(xh.y, gm.y, bt.y) > 0.f ? d.y : 0.f;
        d.z = fmaf(xh.z, gm.z, bt.z) > 0.f ? d.z : 0.f; d.w = fmaf(xh.w, gm.w, bt.w) > 0.f ? d.w : 0.f;
      }
    }
    if (dres != nullptr) st4(dres + q * 4, d);
    float4 o;
    o.x = gm.x * rs.x * (d.x - db.x * inv_m - xh.x * dg.x * inv_m);
    o.y = gm.y * rs.y * (d.y - db.y * inv_m - xh.y * dg.y * inv_m);
    o.z = gm.z * rs.z * (d.z - db.z * inv_m - xh.z * dg.z * inv_m);
    o.w = gm.w * rs.w * (d.w - db.w * inv_m - xh.w * dg.w * inv_m);
    st4(dx + q * 4, o);
  }
}

// ---------------------------------------------------------------------------------- BN + ReLU + 2x2 max-pool
// VGG closes a group of layers with act = relu(bn(conv)) followed by a 2x2 / stride-2 max-pool.  The three kernels below
// never materialise act: the forward writes only the pooled map, the backward finds each window's winner again from the
// convolution output (first maximum in row-major window order, as torch's pooling does) and routes the pooled gradient
// there.  x: [N, H, W, C] convolution output (NHWC), H and W even; pooled tensors: [N, H/2, W/2, C].
struct PoolGeom { int H, W, Hp, Wp; };

// Rows (in units of C floats) of the four pixels of pooled pixel r.
__device__ __forceinline__ void pool_rows(const PoolGeom& g, int64_t r, int64_t (&row)[4]) {
  const int64_t n = r / ((int64_t)g.Hp * g.Wp);
  const int rem = (int)(r - n * g.Hp * g.Wp);
  const int hp = rem / g.Wp, wp = rem - hp * g.Wp;
  row[0] = (n * g.H + 2 * hp) * g.W + 2 * wp;
  row[1] = row[0] + 1;
  row[2] = row[0] + g.W;
  row[3] = row[2] + 1;
}

__device__ __forceinline__ float bn_act1(float v, float mu, float rs, float gm, float bt, int relu) {
  const float o = fmaf((v - mu) * rs, gm, bt);
  return relu ? fmaxf(o, 0.f) : o;
}

// Winner of one channel of one window: its position 0..3 and activation (first maximum wins, as a scan with > does).
__device__ __forceinline__ void pool_winner(const float (&a)[4], int& which, float& best) {
  which = 0; best = a[0];
#pragma unroll
  for (int j = 1; j < 4; ++j)
    if (a[j] > best) { best = a[j]; which = j; }
}

__global__ void __launch_bounds__(BN_THREADS) bn_apply_pool_kernel(const float* __restrict__ x, PoolGeom g, int64_t Mp, int C,
                                                                   const float* __restrict__ stats, const float* __restrict__ gamma,
                                                                   const float* __restrict__ beta, int relu, float* __restrict__ y) {
  pdl_wait();
  pdl_launch_dependents();
  const int vec = C >> 2;
  const int64_t nq = Mp * vec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nq; i += stride) {
    const int64_t q = nq - 1 - i;
    const int64_t r = q / vec;
    const int c4 = (int)(q - r * vec) * 4;
    int64_t row[4];
    pool_rows(g, r, row);
    const float4 mu = ld4(stats + c4), rs = ld4(stats + C + c4), gm = ld4(gamma + c4), bt = ld4(beta + c4);
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = ld4(x + row[j] * C + c4);
    float4 o;
    o.x = fmaxf(fmaxf(bn_act1(v[0].x, mu.x, rs.x, gm.x, bt.x, relu), bn_act1(v[1].x, mu.x, rs.x, gm.x, bt.x, relu)),
                fmaxf(bn_act1(v[2].x, mu.x, rs.x, gm.x, bt.x, relu), bn_act1(v[3].x, mu.x, rs.x, gm.x, bt.x, relu)));
    o.y = fmaxf(fmaxf(bn_act1(v[0].y, mu.y, rs.y, gm.y, bt.y, relu), bn_act1(v[1].y, mu.y, rs.y, gm.y, bt.y, relu)),
                fmaxf(bn_act1(v[2].y, mu.y, rs.y, gm.y, bt.y, relu), bn_act1(v[3].y, mu.y, rs.y, gm.y, bt.y, relu)));
    o.z = fmaxf(fmaxf(bn_act1(v[0].z, mu.z, rs.z, gm.z, bt.z, relu), bn_act1(v[1].z, mu.z, rs.z, gm.z, bt.z, relu)),
                fmaxf(bn_act1(v[2].z, mu.z, rs.z, gm.z, bt.z, relu), bn_act1(v[3].z, mu.z, rs.z, gm.z, bt.z, relu)));
    o.w = fmaxf(fmaxf(bn_act1(v[0].w, mu.w, rs.w, gm.w, bt.w, relu), bn_act1(v[1].w, mu.w, rs.w, gm.w, bt.w, relu)),
                fmaxf(bn_act1(v[2].w, mu.w, rs.w, gm.w, bt.w, relu), bn_act1(v[3].w, mu.w, rs.w, gm.w, bt.w, relu)));
    st4(y + q * 4, o);
  }
}

// One channel of one window in the backward pass: g = pooled gradient if the winner's activation passes the ReLU, at the
// winner's position; returns the position (or -1) and the winner's xhat.
__device__ __forceinline__ int pool_route(float v0, float v1, float v2, float v3, float mu, float rs, float gm, float bt, int relu,
                                          float& xh_win) {
  const float xh[4] = {(v0 - mu) * rs, (v1 - mu) * rs, (v2 - mu) * rs, (v3 - mu) * rs};
  float a[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float o = fmaf(xh[j], gm, bt);
    a[j] = relu ? fmaxf(o, 0.f) : o;
  }
  int which;
  float best;
  pool_winner(a, which, best);
  xh_win = xh[which];
  return (relu && !(best > 0.f)) ? -1 : which;
}

// sums over all N*H*W positions of g and g * xhat, where g is the pooled gradient at each window's winner and 0 elsewhere.
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_reduce_pool_kernel(const float* __restrict__ dpool, const float* __restrict__ x,
                                                                        PoolGeom g, int64_t Mp, int C, int64_t rows_per_block,
                                                                        const float* __restrict__ stats, const float* __restrict__ gamma,
                                                                        const float* __restrict__ beta, int relu,
                                                                        float* __restrict__ partials) {
  pdl_wait();
  pdl_launch_dependents();
  int64_t r0 = (int64_t)blockIdx.x * rows_per_block;
  int64_t r1 = r0 + rows_per_block < Mp ? r0 + rows_per_block : Mp;
  const int col = threadIdx.x % (C >> 2);
  const float4 mu = ld4(stats + 4 * col), rs = ld4(stats + C + 4 * col);
  const float4 gm = ld4(gamma + 4 * col), bt = ld4(beta + 4 * col);
  block_two_sums(Mp, C, r0, r1,
                 [&](int64_t r, int cc, float4& a, float4& b) {
                   int64_t row[4];
                   pool_rows(g, r, row);
                   const float4 d = ld4(dpool + r * C + 4 * cc);
                   float4 v[4];
#pragma unroll
                   for (int j = 0; j < 4; ++j) v[j] = ld4(x + row[j] * C + 4 * cc);
                   float xh;
                   if (pool_route(v[0].x, v[1].x, v[2].x, v[3].x, mu.x, rs.x, gm.x, bt.x, relu, xh) >= 0) { a.x += d.x; b.x = fmaf(d.x, xh, b.x); }
                   if (pool_route(v[0].y, v[1].y, v[2].y, v[3].y, mu.y, rs.y, gm.y, bt.y, relu, xh) >= 0) { a.y += d.y; b.y = fmaf(d.y, xh, b.y); }
                   if (pool_route(v[0].z, v[1].z, v[2].z, v[3].z, mu.z, rs.z, gm.z, bt.z, relu, xh) >= 0) { a.z += d.z; b.z = fmaf(d.z, xh, b.z); }
                   if (pool_route(v[0].w, v[1].w, v[2].w, v[3].w, mu.w, rs.w, gm.w, bt.w, relu, xh) >= 0) { a.w += d.w; b.w = fmaf(d.w, xh, b.w); }
                 },
                 partials + (int64_t)blockIdx.x * 2 * C);
}

// dx at all four positions of every window: gamma * rstd * (g - dbeta / M - xhat * dgamma / M), M = N*H*W.
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_apply_pool_kernel(const float* __restrict__ dpool, const float* __restrict__ x,
                                                                       PoolGeom g, int64_t Mp, int C, const float* __restrict__ stats,
                                                                       const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                       const float* __restrict__ sums, int relu, float* __restrict__ dx) {
  pdl_wait();
  pdl_launch_dependents();
  const int vec = C >> 2;
  const int64_t nq = Mp * vec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float inv_m = 1.0f / (float)(Mp * 4);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nq; i += stride) {
    const int64_t q = nq - 1 - i;
    const int64_t r = q / vec;
    const int c4 = (int)(q - r * vec) * 4;
    int64_t row[4];
    pool_rows(g, r, row);
    const float4 d = ld4(dpool + q * 4);
    const float4 mu = ld4(stats + c4), rs = ld4(stats + C + c4), gm = ld4(gamma + c4), bt = ld4(beta + c4);
    const float4 db = ld4(sums + c4), dg = ld4(sums + C + c4);
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = ld4(x + row[j] * C + c4);
    float xw;
    const int wx = pool_route(v[0].x, v[1].x, v[2].x, v[3].x, mu.x, rs.x, gm.x, bt.x, relu, xw);
    const int wy = pool_route(v[0].y, v[1].y, v[2].y, v[3].y, mu.y, rs.y, gm.y, bt.y, relu, xw);
    const int wz = pool_route(v[0].z, v[1].z, v[2].z, v[3].z, mu.z, rs.z, gm.z, bt.z, relu, xw);
    const int ww = pool_route(v[0].w, v[1].w, v[2].w, v[3].w, mu.w, rs.w, gm.w, bt.w, relu, xw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float4 o;
      o.x = gm.x * rs.x * ((wx == j ? d.x : 0.f) - db.x * inv_m - (v[j].x - mu.x) * rs.x * dg.x * inv_m);
      o.y = gm.y * rs.y * ((wy == j ? d.y : 0.f) - db.y * inv_m - (v[j].y - mu.y) * rs.y * dg.y * inv_m);
      o.z = gm.z * rs.z * ((wz == j ? d.z : 0.f) - db.z * inv_m - (v[j].z - mu.z) * rs.z * dg.z * inv_m);
      o.w = gm.w * rs.w * ((ww == j ? d.w : 0.f) - db.w * inv_m - (v[j].w - mu.w) * rs.w * dg.w * inv_m);
      st4(dx + row[j] * C + c4, o);
    }
  }
}

// ---------------------------------------------------------------------------------- small activations: one kernel per direction
// For the last stages of the networks (4x4 and 2x2 maps at batch 128: M <= 2048 rows) every BN kernel above runs for about
// three microseconds of launch and drain around a few hundred kilobytes of work, and a layer needs five to seven of them.
// Here a block owns 8 channels for ALL rows, so the statistics (forward) or the two gradient sums (backward) are complete
// inside the block and the apply pass follows in the same kernel: statistics + finalize + apply forward, reduce + finalize +
// apply backward.  256 threads = 2 channel quads x 128 row lanes.
constexpr int SMALL_THREADS = 256;
constexpr int SMALL_CH = 8;
constexpr int SMALL_MAX_ROWS = 2048;

// Sum of two float4 per-thread values over the 128 row lanes of each quad (fixed order); every thread leaves with the totals
// of its own quad in (a, b).
__device__ __forceinline__ void small_block_sums(float4& a, float4& b, float4* __restrict__ sm /* [2 * SMALL_THREADS] */) {
  sm[threadIdx.x] = a;
  sm[SMALL_THREADS + threadIdx.x] = b;
  __syncthreads();
  for (int s = SMALL_THREADS >> 1; s >= 2; s >>= 1) {          // thread t and t + s share the quad (s is even)
    if ((int)threadIdx.x < s) {
      const float4 o = sm[threadIdx.x + s], p = sm[SMALL_THREADS + threadIdx.x + s];
      float4 m = sm[threadIdx.x], q = sm[SMALL_THREADS + threadIdx.x];
      m.x += o.x; m.y += o.y; m.z += o.z; m.w += o.w;
      q.x += p.x; q.y += p.y; q.z += p.z; q.w += p.w;
      sm[threadIdx.x] = m;
      sm[SMALL_THREADS + threadIdx.x] = q;
    }
    __syncthreads();
  }
  a = sm[threadIdx.x & 1];
  b = sm[SMALL_THREADS + (threadIdx.x & 1)];
  __syncthreads();
}

// Forward: y = act(gamma * (x - mean) * rstd + beta [+ residual]) with the batch statistics computed here -- from the
// convolution kernel's per-tile partial sums when given (partials[nparts][2][C], unshifted), else from x itself (shifted sums).
// Writes stats[0:C] = mean, stats[C:2C] = rstd and updates the running statistics.
__global__ void __launch_bounds__(SMALL_THREADS) bn_small_fwd_kernel(const float* __restrict__ x, int M, int C,
                                                                     const float* __restrict__ partials, int nparts,
                                                                     const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                     const float* __restrict__ residual, int relu,
                                                                     float* __restrict__ running_mean, float* __restrict__ running_var,
                                                                     float momentum, float eps, float* __restrict__ stats,
                                                                     float* __restrict__ y) {
  __shared__ float4 sm[2 * SMALL_THREADS];
  __shared__ float s_mean[SMALL_CH], s_rstd[SMALL_CH];
  pdl_wait();
  pdl_launch_dependents();
  const int qd = threadIdx.x & 1, rl = threadIdx.x >> 1;
  const int c4 = blockIdx.x * SMALL_CH + 4 * qd;
  const bool live = c4 < C;                                     // C % 4 == 0: a quad is whole or absent
  if (partials == nullptr) {
    const float4 k = live ? ld4(x + c4) : make_float4(0.f, 0.f, 0.f, 0.f);     // shift: the channel's value in row 0
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (live)
      for (int r = rl; r < M; r += SMALL_THREADS / 2) {
        float4 v = ld4(x + (int64_t)r * C + c4);
        v.x -= k.x; v.y -= k.y; v.z -= k.z; v.w -= k.w;
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        b.x = fmaf(v.x, v.x, b.x); b.y = fmaf(v.y, v.y, b.y); b.z = fmaf(v.z, v.z, b.z); b.w = fmaf(v.w, v.w, b.w);
      }
    small_block_sums(a, b, sm);
    // (a, b) hold this thread's quad totals: lanes rl == 0 publish per-channel values
    if (rl == 0 && live) {
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w}, kv[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const double dmean = (double)av[j] / (double)M;
        double var = (double)bv[j] / (double)M - dmean * dmean;
        if (var < 0.0) var = 0.0;
        const double mean = (double)kv[j] + dmean;
        const int c = c4 + j;
        s_mean[4 * qd + j] = (float)mean;
        s_rstd[4 * qd + j] = (float)(1.0 / sqrt(var + (double)eps));
        stats[c] = (float)mean;
        stats[C + c] = s_rstd[4 * qd + j];
        if (running_mean != nullptr) {
          const double unbiased = M > 1 ? var * (double)M / (double)(M - 1) : var;
          running_mean[c] = (1.0f - momentum) * running_mean[c] + momentum * (float)mean;
          running_var[c] = (1.0f - momentum) * running_var[c] + momentum * (float)unbiased;
        }
      }
    }
  } else if (threadIdx.x < SMALL_CH) {
    const int c = blockIdx.x * SMALL_CH + threadIdx.x;
    if (c < C) {
      double sum = 0.0, sq = 0.0;
      for (int t = 0; t < nparts; ++t) {
        sum += (double)partials[((int64_t)t * 2) * C + c];
        sq += (double)partials[((int64_t)t * 2 + 1) * C + c];
      }
      const double mean = sum / (double)M;
      double var = sq / (double)M - mean * mean;
      if (var < 0.0) var = 0.0;
      s_mean[threadIdx.x] = (float)mean;
      s_rstd[threadIdx.x] = (float)(1.0 / sqrt(var + (double)eps));
      stats[c] = (float)mean;
      stats[C + c] = s_rstd[threadIdx.x];
      if (running_mean != nullptr) {
        const double unbiased = M > 1 ? var * (double)M / (double)(M - 1) : var;
        running_mean[c] = (1.0f - momentum) * running_mean[c] + momentum * (float)mean;
        running_var[c] = (1.0f - momentum) * running_var[c] + momentum * (float)unbiased;
      }
    }
  }
  __syncthreads();
  if (!live) return;
  const float4 mu = make_float4(s_mean[4 * qd], s_mean[4 * qd + 1], s_mean[4 * qd + 2], s_mean[4 * qd + 3]);
  const float4 rs = make_float4(s_rstd[4 * qd], s_rstd[4 * qd + 1], s_rstd[4 * qd + 2], s_rstd[4 * qd + 3]);
  const float4 g = ld4(gamma + c4), bt = ld4(beta + c4);
  for (int r = rl; r < M; r += SMALL_THREADS / 2) {
    const int64_t at = (int64_t)r * C + c4;
    const float4 v = ld4(x + at);
    float4 o;
    o.x = fmaf((v.x - mu.x) * rs.x, g.x, bt.x);
    o.y = fmaf((v.y - mu.y) * rs.y, g.y, bt.y);
    o.z = fmaf((v.z - mu.z) * rs.z, g.z, bt.z);
    o.w = fmaf((v.w - mu.w) * rs.w, g.w, bt.w);
    if (residual != nullptr) {
      const float4 rr = ld4(residual + at);
      o.x += rr.x; o.y += rr.y; o.z += rr.z; o.w += rr.w;
    }
    if (relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
    st4(y + at, o);
  }
}

// Backward: sums[0:C] = dbeta, sums[C:2C] = dgamma, dx = gamma * rstd * (g - dbeta / M - xhat * dgamma / M), dres = g
// (g = dy masked by the ReLU: from the saved output y when given, else recomputed from x).
__global__ void __launch_bounds__(SMALL_THREADS) bn_small_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                     const float* __restrict__ y, int M, int C,
                                                                     const float* __restrict__ stats, const float* __restrict__ gamma,
                                                                     const float* __restrict__ beta, int relu,
                                                                     float* __restrict__ sums, float* __restrict__ dx,
                                                                     float* __restrict__ dres) {
  __shared__ float4 sm[2 * SMALL_THREADS];
  pdl_wait();
  pdl_launch_dependents();
  const int qd = threadIdx.x & 1, rl = threadIdx.x >> 1;
  const int c4 = blockIdx.x * SMALL_CH + 4 * qd;
  const bool live = c4 < C;
  float4 mu = make_float4(0.f, 0.f, 0.f, 0.f), rs = mu, gm = mu, bt = mu;
  if (live) { mu = ld4(stats + c4); rs = ld4(stats + C + c4); gm = ld4(gamma + c4); bt = ld4(beta + c4); }
  auto masked = [&](int64_t at, const float4& xh) {
    float4 d = ld4(dy + at);
    if (relu) {
      if (y != nullptr) {
        const float4 o = ld4(y + at);
        d.x = o.x > 0.f ? d.x : 0.f; d.y = o.y > 0.f ? d.y : 0.f; d.z = o.z > 0.f ? d.z : 0.f; d.w = o.w > 0.f ? d.w : 0.f;
      } else {
        d.x = fmaf(xh.x, gm.x, bt.x) > 0.f ? d.x : 0.f; d.y = fmaf(xh.y, gm.y, bt.y) > 0.f ? d.y : 0.f;
        d.z = fmaf(xh.z, gm.z, bt.z) > 0.f ? d.z : 0.f; d.w = fmaf(xh.w, gm.w, bt.w) > 0.f ? d.w : 0.f;
      }
    }
    return d;
  };
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
  if (live)
    for (int r = rl; r < M; r += SMALL_THREADS / 2) {
      const int64_t at = (int64_t)r * C + c4;
      const float4 v = ld4(x + at);
      const float4 xh = make_float4((v.x - mu.x) * rs.x, (v.y - mu.y) * rs.y, (v.z - mu.z) * rs.z, (v.w - mu.w) * rs.w);
      const float4 d = masked(at, xh);
      a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
      b.x = fmaf(d.x, xh.x, b.x); b.y = fmaf(d.y, xh.y, b.y); b.z = fmaf(d.z, xh.z, b.z); b.w = fmaf(d.w, xh.w, b.w);
    }
  small_block_sums(a, b, sm);                                   // a = dbeta quad, b = dgamma quad
  if (!live) return;
  if (rl == 0) { st4(sums + c4, a); st4(sums + C + c4, b); }
  const float inv_m = 1.0f / (float)M;
  for (int r = rl; r < M; r += SMALL_THREADS / 2) {
    const int64_t at = (int64_t)r * C + c4;
    const float4 v = ld4(x + at);
    const float4 xh = make_float4((v.x - mu.x) * rs.x, (v.y - mu.y) * rs.y, (v.z - mu.z) * rs.z, (v.w - mu.w) * rs.w);
    const float4 d = masked(at, xh);
    if (dres != nullptr) st4(dres + at, d);
    float4 o;
    o.x = gm.x * rs.x * (d.x - a.x * inv_m - xh.x * b.x * inv_m);
    o.y = gm.y * rs.y * (d.y - a.y * inv_m - xh.y * b.y * inv_m);
    o.z = gm.z * rs.z * (d.z - a.z * inv_m - xh.z * b.z * inv_m);
    o.w = gm.w * rs.w * (d.w - a.w * inv_m - xh.w * b.w * inv_m);
    st4(dx + at, o);
  }
}

int bn_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

inline bool bn_shape_ok(int64_t M, int C) {
  if (M < 1 || C < 4 || (C & 3)) return false;
  int vec = C >> 2;
  return vec <= BN_THREADS && (BN_THREADS % vec) == 0;
}

inline int reduce_grid(int64_t M, int C, int64_t* rows_per_block) {
  int vec = C >> 2;
  int rstep = BN_THREADS / vec;
  int64_t min_rows = (int64_t)rstep * 8;                  // at least 8 rows per thread
  int64_t blocks = (M + min_rows - 1) / min_rows;
  int64_t cap = (int64_t)bn_sm_count() * 2;
  if (cap > BN_MAX_BLOCKS) cap = BN_MAX_BLOCKS;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  *rows_per_block = (M + blocks - 1) / blocks;
  return (int)((M + *rows_per_block - 1) / *rows_per_block);
}

int64_t g_bwd_fused_atomics_limit = 200000;
int g_bwd_reduce_interleave = 0;   // measured inside the ResNet-50 step: 7.47 ms with, 7.46 ms without

inline int apply_grid(int64_t nq) {
  int64_t need = (nq + BN_THREADS - 1) / BN_THREADS;
  int64_t cap = (int64_t)bn_sm_count() * 4;
  return (int)(need < cap ? (need < 1 ? 1 : need) : cap);
}

}  // namespace

extern "C" {

// Scratch for the two reductions: BN_MAX_BLOCKS * 2 * C floats (no initialisation needed).
int64_t gc_cuda_bn_scratch_bytes(int max_channels) { return (int64_t)BN_MAX_BLOCKS * 2 * max_channels * 4; }

int gc_cuda_bn_supported(int64_t M, int C) { return bn_shape_ok(M, C) ? 1 : 0; }

// stats[0:C] = batch mean, stats[C:2C] = 1/sqrt(biased var + eps); running stats (may be NULL) get the
// momentum update with the unbiased variance, as torch.nn.BatchNorm2d does.
int gc_cuda_bn_stats(const float* x, int64_t M, int C, void* scratch, float* stats, float* running_mean,
                     float* running_var, float momentum, float eps, void* cs) {
  if (!bn_shape_ok(M, C)) return (int)cudaErrorInvalidValue;
  int64_t rpb;
  int grid = reduce_grid(M, C, &rpb);
  size_t smem = 2 * BN_THREADS * sizeof(float4);
  launch_pdl(bn_stats_kernel, dim3(grid), dim3(BN_THREADS), smem, (cudaStream_t)cs, x, M, C, rpb, (float*)scratch);
  dim3 fg, fb;
  finalize_shape(grid, C, &fg, &fb);
  launch_pdl(bn_stats_finalize_kernel, fg, fb, 0, (cudaStream_t)cs, (const float*)scratch, x, grid, M,
             C, stats, running_mean, running_var, momentum, eps);
  return (int)cudaGetLastError();
}

// Statistics from partial column sums produced elsewhere (the GEMM epilogue): partials[nparts][2][C], unshifted.
int gc_cuda_bn_finalize_partials(const float* partials, int nparts, int64_t M, int C, float* stats, float* running_mean,
                                 float* running_var, float momentum, float eps, void* cs) {
  dim3 fg, fb;
  finalize_shape(nparts, C, &fg, &fb);
  launch_pdl(bn_stats_finalize_kernel, fg, fb, 0, (cudaStream_t)cs, partials, (const float*)nullptr,
             nparts, M, C, stats, running_mean, running_var, momentum, eps);
  return (int)cudaGetLastError();
}

int gc_cuda_bn_apply(const float* x, int64_t M, int C, const float* stats, const float* gamma, const float* beta,
                     const float* residual, int relu, float* y, void* cs) {
  if (!bn_shape_ok(M, C)) return (int)cudaErrorInvalidValue;
  launch_pdl(bn_apply_kernel, dim3(apply_grid(M * (C >> 2))), dim3(BN_THREADS), 0, (cudaStream_t)cs, x, M, C, stats, gamma, beta,
             residual, relu, y);
  return (int)cudaGetLastError();
}

// sums[0:C] = dbeta, sums[C:2C] = dgamma.  y: saved forward output (needed only when a residual was added).
// fin_scratch (may be NULL): a zero-initialised buffer of 256 + 2 * C * 8 bytes that every launch leaves zeroed (the one the
// GEMMs' statistics use).  When given and the grid is small against the tensor (few atomics per block) the blocks add their
// sums there with atomics and the last one writes `sums`: one launch instead of two.
int gc_cuda_bn_bwd_reduce(const float* dy, const float* x, const float* y, int64_t M, int C, const float* stats,
                          const float* gamma, const float* beta, int relu, void* scratch, float* sums, void* fin_scratch, void* cs) {
  if (!bn_shape_ok(M, C)) return (int)cudaErrorInvalidValue;
  int64_t rpb;
  int grid = reduce_grid(M, C, &rpb);
  size_t smem = 2 * BN_THREADS * sizeof(float4);
  const bool fused = fin_scratch != nullptr && (int64_t)grid * 2 * C <= g_bwd_fused_atomics_limit;
  double* acc = fused ? reinterpret_cast<double*>(static_cast<uint8_t*>(fin_scratch) + 256) : nullptr;
  unsigned int* ticket = fused ? static_cast<unsigned int*>(fin_scratch) : nullptr;
  launch_pdl(bn_bwd_reduce_kernel, dim3(grid), dim3(BN_THREADS), smem, (cudaStream_t)cs, dy, x, y, M, C, rpb, stats, gamma, beta,
             relu, (float*)scratch, acc, ticket, sums, g_bwd_reduce_interleave);
  if (!fused)
    {
      dim3 fg, fb;
      finalize_shape(grid, C, &fg, &fb);
      launch_pdl(bn_sums_finalize_kernel, fg, fb, 0, (cudaStream_t)cs, (const float*)scratch, grid, C, sums);
    }
  return (int)cudaGetLastError();
}

// Above this many atomics per launch (blocks x 2C) the backward reduction keeps its separate finalize kernel: with many
// blocks on a wide, short activation the atomics would cost more than the second launch.
void gc_cuda_bn_bwd_fused_limit(int64_t atomics) { g_bwd_fused_atomics_limit = atomics; }

// For measurements: 1 = the backward reduction walks the tensor from its end in interleaved chunks, 0 (default) = one
// contiguous row range per block.
void gc_cuda_bn_bwd_reduce_interleave(int on) { g_bwd_reduce_interleave = on ? 1 : 0; }

int gc_cuda_bn_bwd_apply(const float* dy, const float* x, const float* y, int64_t M, int C, const float* stats,
                         const float* gamma, const float* beta, const float* sums, int relu, float* dx, float* dres,
                         void* cs) {
  if (!bn_shape_ok(M, C)) return (int)cudaErrorInvalidValue;
  launch_pdl(bn_bwd_apply_kernel, dim3(apply_grid(M * (C >> 2))), dim3(BN_THREADS), 0, (cudaStream_t)cs, dy, x, y, M, C, stats, gamma,
             beta, sums, relu, dx, dres);
  return (int)cudaGetLastError();
}

// 1 when the pooled variants cover the shape: the plain kernels' rules for C, H and W even.
int gc_cuda_bn_pool_supported(int N, int H, int W, int C) {
  return N >= 1 && H >= 2 && W >= 2 && !(H & 1) && !(W & 1) && bn_shape_ok((int64_t)N * (H / 2) * (W / 2), C) ? 1 : 0;
}

// y[N, H/2, W/2, C] = maxpool2x2(act(gamma * (x - mean) * rstd + beta)); x: [N, H, W, C].
int gc_cuda_bn_apply_pool(const float* x, int N, int H, int W, int C, const float* stats, const float* gamma, const float* beta,
                          int relu, float* y, void* cs) {
  if (!gc_cuda_bn_pool_supported(N, H, W, C)) return (int)cudaErrorInvalidValue;
  const PoolGeom g{H, W, H / 2, W / 2};
  const int64_t Mp = (int64_t)N * g.Hp * g.Wp;
  launch_pdl(bn_apply_pool_kernel, dim3(apply_grid(Mp * (C >> 2))), dim3(BN_THREADS), 0, (cudaStream_t)cs, x, g, Mp, C, stats, gamma,
             beta, relu, y);
  return (int)cudaGetLastError();
}

// sums[0:C] = dbeta, sums[C:2C] = dgamma of the layer whose pooled output received the gradient dpool[N, H/2, W/2, C].
int gc_cuda_bn_bwd_reduce_pool(const float* dpool, const float* x, int N, int H, int W, int C, const float* stats,
                               const float* gamma, const float* beta, int relu, void* scratch, float* sums, void* cs) {
  if (!gc_cuda_bn_pool_supported(N, H, W, C)) return (int)cudaErrorInvalidValue;
  const PoolGeom g{H, W, H / 2, W / 2};
  const int64_t Mp = (int64_t)N * g.Hp * g.Wp;
  int64_t rpb;
  int grid = reduce_grid(Mp, C, &rpb);
  size_t smem = 2 * BN_THREADS * sizeof(float4);
  launch_pdl(bn_bwd_reduce_pool_kernel, dim3(grid), dim3(BN_THREADS), smem, (cudaStream_t)cs, dpool, x, g, Mp, C, rpb, stats, gamma,
             beta, relu, (float*)scratch);
  dim3 fg, fb;
  finalize_shape(grid, C, &fg, &fb);
  launch_pdl(bn_sums_finalize_kernel, fg, fb, 0, (cudaStream_t)cs, (const float*)scratch, grid, C, sums);
  return (int)cudaGetLastError();
}

// dx[N, H, W, C]: gradient of the convolution output.
int gc_cuda_bn_bwd_apply_pool(const float* dpool, const float* x, int N, int H, int W, int C, const float* stats,
                              const float* gamma, const float* beta, const float* sums, int relu, float* dx, void* cs) {
  if (!gc_cuda_bn_pool_supported(N, H, W, C)) return (int)cudaErrorInvalidValue;
  const PoolGeom g{H, W, H / 2, W / 2};
  const int64_t Mp = (int64_t)N * g.Hp * g.Wp;
  launch_pdl(bn_bwd_apply_pool_kernel, dim3(apply_grid(Mp * (C >> 2))), dim3(BN_THREADS), 0, (cudaStream_t)cs, dpool, x, g, Mp, C,
             stats, gamma, beta, sums, relu, dx);
  return (int)cudaGetLastError();
}

// 1 when the single-kernel forms cover the activation: at most 2048 rows, C a multiple of 4.
int gc_cuda_bn_small_supported(int64_t M, int C) { return M >= 1 && M <= SMALL_MAX_ROWS && C >= 4 && (C & 3) == 0 ? 1 : 0; }

// Statistics (from partials[nparts][2][C] when given, else from x) + running-statistics update + apply, one launch.
int gc_cuda_bn_small_forward(const float* x, int64_t M, int C, const float* partials, int nparts, const float* gamma, const float* beta,
                             const float* residual, int relu, float* running_mean, float* running_var, float momentum, float eps,
                             float* stats, float* y, void* cs) {
  if (!gc_cuda_bn_small_supported(M, C)) return (int)cudaErrorInvalidValue;
  launch_pdl(bn_small_fwd_kernel, dim3((C + SMALL_CH - 1) / SMALL_CH), dim3(SMALL_THREADS), 0, (cudaStream_t)cs, x, (int)M, C, partials,
             nparts, gamma, beta, residual, relu, running_mean, running_var, momentum, eps, stats, y);
  return (int)cudaGetLastError();
}

// Gradient sums + input gradient (+ residual gradient), one launch.
int gc_cuda_bn_small_backward(const float* dy, const float* x, const float* y, int64_t M, int C, const float* stats, const float* gamma,
                              const float* beta, int relu, float* sums, float* dx, float* dres, void* cs) {
  if (!gc_cuda_bn_small_supported(M, C)) return (int)cudaErrorInvalidValue;
  launch_pdl(bn_small_bwd_kernel, dim3((C + SMALL_CH - 1) / SMALL_CH), dim3(SMALL_THREADS), 0, (cudaStream_t)cs, dy, x, y, (int)M, C, stats,
             gamma, beta, relu, sums, dx, dres);
  return (int)cudaGetLastError();
}

}  // extern "C"
