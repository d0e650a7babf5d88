// Fused compress + collective kernels over the symmetric arena (one persistent cooperative launch
// per reducer step and rank):
//   fused_allreduce   fp32 two-shot all-reduce (AllReduce-SGD)
//   fused_qsgd        QSGD-MaxNorm: abs-max -> max exchange -> stochastic quantise + pack ->
//                     owner-pull packed reduce-scatter with int32 accumulators -> push of narrow
//                     integer sums to every peer -> dequantise into the fp32 gradient
//   fused_twoscale    two-scale variant: adds the 1-bit "fits the low scale" agreement round
//   fused_randk       shared-index gather -> (two-scale) quantised one-shot reduce -> scatter
//   fused_small_sum   one-shot fp32 sum of short vectors (PowerSGD P / Q / rank-1 tensors)
// Peers are reached with plain loads / stores through their mapped arenas; no TMA is involved.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "gc_comm.cuh"
#include "gc_perm.h"

using namespace gc;

namespace {

constexpr int THREADS = 512;
// Register cap of the dense fused kernels.  A bucketed reducer runs them beside backward kernels; the persistent tcgen05
// GEMM wants one CTA on every SM (352 threads x 96 registers = 33.8 K of the SM's 64 K) and assigns its tiles
// statically, so a reducer block that does not fit next to it keeps that SM's GEMM CTA -- and with it the whole GEMM --
// waiting until the reducer block leaves.  512 threads x 56 registers = 28.7 K fits beside it.
#define GC_FUSED_MAXNREG 56
enum Phase : int { PH_READY = 0, PH_DONE = 1, PH_MASK = 2, PH_STAGE = 3, PH_AUX = 4 };

struct Common {
  int64_t n;
  int world;
  int step_from_device;   // 1: Philox step = step + launches so far on this rank (for CUDA-graph replay)
  unsigned long long timeout_ns;
  uint32_t seed_lo, seed_hi, step;
};

__device__ __forceinline__ RngKey rng_key(const Common& c, uint32_t step, int rank, uint32_t purpose) {
  RngKey k;
  k.k0 = c.seed_lo;
  k.k1 = c.seed_hi;
  k.step = step;
  k.stream = ((uint32_t)rank << 8) | purpose;
  return k;
}

struct Ctx {   // per-block view of "which virtual rank am I"
  const RankView* v;
  ArenaHeader* hdr;
  int bid, nblocks;
  int64_t warp, nwarps;
  int lane;
};

__device__ __forceinline__ Ctx make_ctx(const LaunchViews& lv) {
  Ctx c;
  int vr = blockIdx.x / lv.blocks_per_rank;
  c.v = &lv.r[vr];
  c.hdr = reinterpret_cast<ArenaHeader*>(c.v->arena[c.v->rank]);
  c.bid = blockIdx.x % lv.blocks_per_rank;
  c.nblocks = lv.blocks_per_rank;
  c.lane = threadIdx.x & 31;
  c.warp = (int64_t)c.bid * (THREADS / 32) + (threadIdx.x >> 5);
  c.nwarps = (int64_t)c.nblocks * (THREADS / 32);
  return c;
}

__device__ __forceinline__ float quad_absmax(float4 a) {
  return fmaxf(fmaxf(abs_for_max(a.x), abs_for_max(a.y)), fmaxf(abs_for_max(a.z), abs_for_max(a.w)));
}

__device__ __forceinline__ float local_absmax(const Ctx& c, const float* __restrict__ x, int64_t n, bool al) {
  float m = 0.0f;
  int64_t nq = (n + 3) / 4;
  int64_t stride = (int64_t)c.nblocks * THREADS;
  int64_t q = (int64_t)c.bid * THREADS + threadIdx.x;
  // four independent 16-byte loads per thread and iteration keep ~64 KB in flight per SM
  for (; q + 3 * stride < nq; q += 4 * stride) {
    float4 a = load_quad(x, q * 4, n, al);
    float4 b = load_quad(x, (q + stride) * 4, n, al);
    float4 d = load_quad(x, (q + 2 * stride) * 4, n, al);
    float4 e = load_quad(x, (q + 3 * stride) * 4, n, al);
    m = fmaxf(m, fmaxf(fmaxf(quad_absmax(a), quad_absmax(b)), fmaxf(quad_absmax(d), quad_absmax(e))));
  }
  for (; q < nq; q += stride) m = fmaxf(m, quad_absmax(load_quad(x, q * 4, n, al)));
  return m;
}

// Raw (still packed) magnitudes of this lane's quad, and their decoding.
template <int MW>
struct RawMags { uint32_t a, b; };
template <int MW>
__device__ __forceinline__ RawMags<MW> load_raw_mags(const uint8_t* __restrict__ mags, int64_t row, int lane) {
  RawMags<MW> r;
  r.b = 0;
  if (MW == 16) { uint2 v = reinterpret_cast<const uint2*>(mags)[row * 32 + lane]; r.a = v.x; r.b = v.y; }
  else if (MW == 8) r.a = reinterpret_cast<const uint32_t*>(mags)[row * 32 + lane];
  else if (MW == 4) r.a = reinterpret_cast<const uint16_t*>(mags)[row * 32 + lane];
  else if (MW == 2) r.a = mags[row * 32 + lane];
  else r.a = mags[row * 16 + (lane >> 1)];
  return r;
}
template <int MW>
__device__ __forceinline__ void decode_mags(const RawMags<MW>& r, int lane, int (&m)[4]) {
  if (MW == 16) { m[0] = r.a & 0xffff; m[1] = r.a >> 16; m[2] = r.b & 0xffff; m[3] = r.b >> 16; }
  else if (MW == 8) { m[0] = r.a & 0xff; m[1] = (r.a >> 8) & 0xff; m[2] = (r.a >> 16) & 0xff; m[3] = r.a >> 24; }
  else if (MW == 4) { m[0] = r.a & 0xf; m[1] = (r.a >> 4) & 0xf; m[2] = (r.a >> 8) & 0xf; m[3] = (r.a >> 12) & 0xf; }
  else if (MW == 2) { m[0] = r.a & 3; m[1] = (r.a >> 2) & 3; m[2] = (r.a >> 4) & 3; m[3] = (r.a >> 6) & 3; }
  else { uint32_t v = (lane & 1) ? (r.a >> 4) : r.a; m[0] = v & 1; m[1] = (v >> 1) & 1; m[2] = (v >> 2) & 1; m[3] = (v >> 3) & 1; }
}

// One 32-bit load per lane fetches the bit plane of a row from ALL ranks: lane l holds word (l & 3) of rank
// (l >> 2).  plane_bit(word_of_rank(src, j)) then comes from a shuffle.
__device__ __forceinline__ uint32_t load_plane_all_ranks(const RankView& v, int world, int64_t off_plane, int64_t row, int lane) {
  int src = lane >> 2;
  if (src >= world) return 0u;
  return reinterpret_cast<const uint32_t*>(v.arena[src] + off_plane)[row * 4 + (lane & 3)];
}

template <int SUMB>
__device__ __forceinline__ void store_row_sums(uint8_t* __restrict__ sums, int64_t row, int lane, const int (&a)[4]) {
  if (SUMB == 1) {
    uint32_t v = (uint32_t)(a[0] & 0xff) | ((uint32_t)(a[1] & 0xff) << 8) | ((uint32_t)(a[2] & 0xff) << 16) |
                 ((uint32_t)(a[3] & 0xff) << 24);
    reinterpret_cast<uint32_t*>(sums)[row * 32 + lane] = v;
  } else if (SUMB == 2) {
    uint2 v;
    v.x = (uint32_t)(a[0] & 0xffff) | ((uint32_t)(a[1] & 0xffff) << 16);
    v.y = (uint32_t)(a[2] & 0xffff) | ((uint32_t)(a[3] & 0xffff) << 16);
    reinterpret_cast<uint2*>(sums)[row * 32 + lane] = v;
  } else {
    reinterpret_cast<int4*>(sums)[row * 32 + lane] = make_int4(a[0], a[1], a[2], a[3]);
  }
}
template <int SUMB>
__device__ __forceinline__ void load_row_sums(const uint8_t* __restrict__ sums, int64_t row, int lane, int (&a)[4]) {
  if (SUMB == 1) {
    uint32_t v = reinterpret_cast<const uint32_t*>(sums)[row * 32 + lane];
    a[0] = (int8_t)(v & 0xff); a[1] = (int8_t)((v >> 8) & 0xff); a[2] = (int8_t)((v >> 16) & 0xff); a[3] = (int8_t)(v >> 24);
  } else if (SUMB == 2) {
    uint2 v = reinterpret_cast<const uint2*>(sums)[row * 32 + lane];
    a[0] = (int16_t)(v.x & 0xffff); a[1] = (int16_t)(v.x >> 16); a[2] = (int16_t)(v.y & 0xffff); a[3] = (int16_t)(v.y >> 16);
  } else {
    int4 v = reinterpret_cast<const int4*>(sums)[row * 32 + lane];
    a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
  }
}

// ------------------------------------------------------------------------------------------ QSGD-MaxNorm
struct QsgdParams {
  Common c;
  int s;                  // 2^b - 1
  int64_t off_mags, off_signs, off_sums;   // byte offsets inside every arena
  int64_t chunk_rows;     // rows owned by each rank in the reduce-scatter
};

// Owner-pull reduce of the rows this rank owns, then push of the integer sums to every rank.  Two rows per
// warp and iteration: all peer loads of both rows are issued before the first one is consumed.
template <int MW, int SUMB>
__device__ __forceinline__ void reduce_scatter_rows(const Ctx& c, int world, int64_t rows, int64_t chunk_rows,
                                                    int64_t off_mags, int64_t off_signs, int64_t off_sums) {
  const RankView& v = *c.v;
  int64_t r0 = (int64_t)v.rank * chunk_rows;
  int64_t r1 = r0 + chunk_rows < rows ? r0 + chunk_rows : rows;
  for (int64_t rowa = r0 + c.warp; rowa < r1; rowa += 2 * c.nwarps) {
    int64_t rowb = rowa + c.nwarps;
    bool hasb = rowb < r1;
    RawMags<MW> ma[MAXW], mb[MAXW];
#pragma unroll
    for (int src = 0; src < MAXW; ++src)
      if (src < world) {
        ma[src] = load_raw_mags<MW>(v.arena[src] + off_mags, rowa, c.lane);
        if (hasb) mb[src] = load_raw_mags<MW>(v.arena[src] + off_mags, rowb, c.lane);
      }
    uint32_t sa = load_plane_all_ranks(v, world, off_signs, rowa, c.lane);
    uint32_t sb = hasb ? load_plane_all_ranks(v, world, off_signs, rowb, c.lane) : 0u;
    int acca[4] = {0, 0, 0, 0}, accb[4] = {0, 0, 0, 0};
#pragma unroll
    for (int src = 0; src < MAXW; ++src)
      if (src < world) {
        int m[4];
        decode_mags<MW>(ma[src], c.lane, m);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t w = __shfl_sync(FULL, sa, src * 4 + j);
          acca[j] += ((w >> c.lane) & 1u) ? -m[j] : m[j];
        }
        if (hasb) decode_mags<MW>(mb[src], c.lane, m);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t w = __shfl_sync(FULL, sb, src * 4 + j);
          if (hasb) accb[j] += ((w >> c.lane) & 1u) ? -m[j] : m[j];
        }
      }
#pragma unroll
    for (int dst = 0; dst < MAXW; ++dst)
      if (dst < world) {
        store_row_sums<SUMB>(v.arena[dst] + off_sums, rowa, c.lane, acca);
        if (hasb) store_row_sums<SUMB>(v.arena[dst] + off_sums, rowb, c.lane, accb);
      }
  }
}

template <int MW, int SUMB>
__global__ void __maxnreg__(GC_FUSED_MAXNREG) qsgd_fused_kernel(LaunchViews lv, QsgdParams p) {
  __shared__ float smem[32];
  Ctx c = make_ctx(lv);
  const RankView& v = *c.v;
  Waiter w{c.hdr, global_ns() + p.c.timeout_ns};
  const uint32_t epoch = next_epoch(c.hdr);
  const uint32_t rng_step = p.c.step + (p.c.step_from_device ? launch_calls(c.hdr) : 0u);
  const int64_t n = p.c.n;
  const int world = p.c.world;
  const bool al_in = (reinterpret_cast<uintptr_t>(v.in) & 15u) == 0;
  const bool al_out = (reinterpret_cast<uintptr_t>(v.out) & 15u) == 0;
  const int64_t rows = (n + 127) / 128;

  // P0: global max-norm
  float m = rank_max(w, local_absmax(c, v.in, n, al_in), c.bid, c.nblocks, smem, 0x20);
  commit_epoch(c.hdr, epoch, c.bid);
  float norm = (world > 1) ? exchange_max(w, v, world, epoch, m, c.bid == 0, smem) : m;
  float scale = (norm > 0.0f) ? (float)p.s / norm : 0.0f;
  float dq = dequant_scale(norm, p.s, world);
  RngKey key = rng_key(p.c, rng_step, v.rank, PURPOSE_ROUND);

  if (world == 1) {
    // single worker: quantise and dequantise in registers, one pass, four rows per warp in flight
    for (int64_t row0 = c.warp; row0 < rows; row0 += 4 * c.nwarps) {
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int64_t row = row0 + u * c.nwarps;
        x[u] = (row < rows) ? load_quad(v.in, row * 128 + c.lane * 4, n, al_in) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int64_t row = row0 + u * c.nwarps;
        if (row >= rows) break;
        int64_t e0 = row * 128 + c.lane * 4;
        U4 r = philox_block(key, (uint64_t)(e0 >> 2));
        float4 y;
        y.x = mul_rn(dq, (float)quantize_level(x[u].x, scale, p.s, r.x));
        y.y = mul_rn(dq, (float)quantize_level(x[u].y, scale, p.s, r.y));
        y.z = mul_rn(dq, (float)quantize_level(x[u].z, scale, p.s, r.z));
        y.w = mul_rn(dq, (float)quantize_level(x[u].w, scale, p.s, r.w));
        store_quad(v.out, e0, n, al_out, y);
      }
    }
    return;
  }

  // P1: quantise + pack into this rank's arena (four rows per warp in flight)
  uint8_t* my = v.arena[v.rank];
  for (int64_t row0 = c.warp; row0 < rows; row0 += 4 * c.nwarps) {
    float4 x[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int64_t row = row0 + u * c.nwarps;
      x[u] = (row < rows) ? load_quad(v.in, row * 128 + c.lane * 4, n, al_in) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int64_t row = row0 + u * c.nwarps;
      if (row >= rows) break;
      int64_t e0 = row * 128 + c.lane * 4;
      U4 r = philox_block(key, (uint64_t)(e0 >> 2));
      int q0 = quantize_level(x[u].x, scale, p.s, r.x), q1 = quantize_level(x[u].y, scale, p.s, r.y);
      int q2 = quantize_level(x[u].z, scale, p.s, r.z), q3 = quantize_level(x[u].w, scale, p.s, r.w);
      int mg[4] = {abs(q0), abs(q1), abs(q2), abs(q3)};
      bool sg[4] = {q0 < 0, q1 < 0, q2 < 0, q3 < 0};
      store_row_mags<MW>(my + p.off_mags, row, c.lane, mg);
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_signs), row, c.lane, sg);
    }
  }
  grid_barrier(w, c.nblocks, 0x21);
  if (c.bid == 0) signal_all(v, world, PH_READY, epoch);
  wait_all(w, world, PH_READY, epoch);

  // P2: packed reduce-scatter (pull) + push of the sums
  reduce_scatter_rows<MW, SUMB>(c, world, rows, p.chunk_rows, p.off_mags, p.off_signs, p.off_sums);
  grid_barrier(w, c.nblocks, 0x22);
  if (c.bid == 0) signal_all(v, world, PH_DONE, epoch);
  wait_all(w, world, PH_DONE, epoch);

  // P3: dequantise the summed levels into the fp32 gradient (1/W folded into dq)
  for (int64_t row0 = c.warp; row0 < rows; row0 += 4 * c.nwarps) {
    int a[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int64_t row = row0 + u * c.nwarps;
      if (row < rows) load_row_sums<SUMB>(my + p.off_sums, row, c.lane, a[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int64_t row = row0 + u * c.nwarps;
      if (row >= rows) break;
      float4 y = make_float4(mul_rn(dq, (float)a[u][0]), mul_rn(dq, (float)a[u][1]), mul_rn(dq, (float)a[u][2]),
                             mul_rn(dq, (float)a[u][3]));
      store_quad(v.out, row * 128 + c.lane * 4, n, al_out, y);
    }
  }
}

// ------------------------------------------------------------------------------------------ two-scale
struct TwoScaleParams {
  Common c;
  int s_lo, s_hi;
  int64_t off_mags, off_signs, off_sums, off_mask_local, off_mask_final;
  int64_t chunk_rows;
};

template <int MW, int SUMB>
__global__ void __maxnreg__(GC_FUSED_MAXNREG) twoscale_fused_kernel(LaunchViews lv, TwoScaleParams p) {
  __shared__ float smem[32];
  Ctx c = make_ctx(lv);
  const RankView& v = *c.v;
  Waiter w{c.hdr, global_ns() + p.c.timeout_ns};
  const uint32_t epoch = next_epoch(c.hdr);
  const uint32_t rng_step = p.c.step + (p.c.step_from_device ? launch_calls(c.hdr) : 0u);
  const int64_t n = p.c.n;
  const int world = p.c.world;
  const bool al_in = (reinterpret_cast<uintptr_t>(v.in) & 15u) == 0;
  const bool al_out = (reinterpret_cast<uintptr_t>(v.out) & 15u) == 0;
  const int64_t rows = (n + 127) / 128;
  uint8_t* my = v.arena[v.rank];

  float m = rank_max(w, local_absmax(c, v.in, n, al_in), c.bid, c.nblocks, smem, 0x30);
  commit_epoch(c.hdr, epoch, c.bid);
  float norm = (world > 1) ? exchange_max(w, v, world, epoch, m, c.bid == 0, smem) : m;
  float sc_lo = (norm > 0.0f) ? (float)p.s_lo / norm : 0.0f;
  float sc_hi = (norm > 0.0f) ? (float)p.s_hi / norm : 0.0f;
  float dq_lo = dequant_scale(norm, p.s_lo, world), dq_hi = dequant_scale(norm, p.s_hi, world);
  RngKey k_lo = rng_key(p.c, rng_step, v.rank, PURPOSE_ROUND), k_hi = rng_key(p.c, rng_step, v.rank, PURPOSE_ROUND_HI);

  // P1a: which elements' rounded high-scale level still fits the low range (this rank's vote)
  if (world > 1) {
    for (int64_t row = c.warp; row < rows; row += c.nwarps) {
      int64_t e0 = row * 128 + c.lane * 4;
      float4 x = load_quad(v.in, e0, n, al_in);
      U4 r = philox_block(k_hi, (uint64_t)(e0 >> 2));
      bool fit[4] = {abs(quantize_level(x.x, sc_hi, p.s_hi, r.x)) <= p.s_lo,
                     abs(quantize_level(x.y, sc_hi, p.s_hi, r.y)) <= p.s_lo,
                     abs(quantize_level(x.z, sc_hi, p.s_hi, r.z)) <= p.s_lo,
                     abs(quantize_level(x.w, sc_hi, p.s_hi, r.w)) <= p.s_lo};
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_mask_local), row, c.lane, fit);
    }
    grid_barrier(w, c.nblocks, 0x31);
    if (c.bid == 0) signal_all(v, world, PH_MASK, epoch);
    wait_all(w, world, PH_MASK, epoch);
  }

  // P1b: AND of all votes (one-shot read of every peer's bit plane), pick the scale, quantise
  for (int64_t row = c.warp; row < rows; row += c.nwarps) {
    int64_t e0 = row * 128 + c.lane * 4;
    float4 x = load_quad(v.in, e0, n, al_in);
    U4 rh = philox_block(k_hi, (uint64_t)(e0 >> 2));
    U4 rl = philox_block(k_lo, (uint64_t)(e0 >> 2));
    int qh[4] = {quantize_level(x.x, sc_hi, p.s_hi, rh.x), quantize_level(x.y, sc_hi, p.s_hi, rh.y),
                 quantize_level(x.z, sc_hi, p.s_hi, rh.z), quantize_level(x.w, sc_hi, p.s_hi, rh.w)};
    int ql[4] = {quantize_level(x.x, sc_lo, p.s_lo, rl.x), quantize_level(x.y, sc_lo, p.s_lo, rl.y),
                 quantize_level(x.z, sc_lo, p.s_lo, rl.z), quantize_level(x.w, sc_lo, p.s_lo, rl.w)};
    bool use_hi[4];
    if (world > 1) {
      uint32_t mine = load_plane_all_ranks(v, world, p.off_mask_local, row, c.lane);
      uint32_t andw[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
#pragma unroll
      for (int src = 0; src < MAXW; ++src)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t t = __shfl_sync(FULL, mine, src * 4 + j);
          if (src < world) andw[j] &= t;
        }
#pragma unroll
      for (int j = 0; j < 4; ++j) use_hi[j] = (andw[j] >> c.lane) & 1u;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) use_hi[j] = abs(qh[j]) <= p.s_lo;
    }
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = use_hi[j] ? qh[j] : ql[j];
    if (world == 1) {
      float4 y;
      y.x = mul_rn(use_hi[0] ? dq_hi : dq_lo, (float)q[0]);
      y.y = mul_rn(use_hi[1] ? dq_hi : dq_lo, (float)q[1]);
      y.z = mul_rn(use_hi[2] ? dq_hi : dq_lo, (float)q[2]);
      y.w = mul_rn(use_hi[3] ? dq_hi : dq_lo, (float)q[3]);
      store_quad(v.out, e0, n, al_out, y);
    } else {
      int mg[4] = {abs(q[0]), abs(q[1]), abs(q[2]), abs(q[3])};
      bool sg[4] = {q[0] < 0, q[1] < 0, q[2] < 0, q[3] < 0};
      store_row_mags<MW>(my + p.off_mags, row, c.lane, mg);
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_signs), row, c.lane, sg);
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_mask_final), row, c.lane, use_hi);
    }
  }
  if (world == 1) return;
  grid_barrier(w, c.nblocks, 0x32);
  if (c.bid == 0) signal_all(v, world, PH_READY, epoch);
  wait_all(w, world, PH_READY, epoch);

  reduce_scatter_rows<MW, SUMB>(c, world, rows, p.chunk_rows, p.off_mags, p.off_signs, p.off_sums);
  grid_barrier(w, c.nblocks, 0x33);
  if (c.bid == 0) signal_all(v, world, PH_DONE, epoch);
  wait_all(w, world, PH_DONE, epoch);

  for (int64_t row = c.warp; row < rows; row += c.nwarps) {
    int a[4];
    bool hi[4];
    load_row_sums<SUMB>(my + p.off_sums, row, c.lane, a);
    load_row_plane(reinterpret_cast<const uint32_t*>(my + p.off_mask_final), row, c.lane, hi);
    float4 y = make_float4(mul_rn(hi[0] ? dq_hi : dq_lo, (float)a[0]), mul_rn(hi[1] ? dq_hi : dq_lo, (float)a[1]),
                           mul_rn(hi[2] ? dq_hi : dq_lo, (float)a[2]), mul_rn(hi[3] ? dq_hi : dq_lo, (float)a[3]));
    store_quad(v.out, row * 128 + c.lane * 4, n, al_out, y);
  }
}

// ------------------------------------------------------------------------------------------ multi-scale (L <= 4)
// Per element every rank finds the finest scale l whose stochastically rounded level still fits the coarsest
// scale's range (|q_l| <= s_0); the ranks agree on the MINIMUM index (reference: all-reduce MIN of an int8 array,
// reducer.py:1680) through two bit planes in peer memory; everyone then sends the level of the agreed scale.
struct MultiScaleParams {
  Common c;
  int n_levels;
  int s[4];
  int64_t off_mags, off_signs, off_sums, off_idx_local[2], off_idx_final[2];
  int64_t chunk_rows;
};

template <int MW, int SUMB>
__global__ void __maxnreg__(GC_FUSED_MAXNREG) multiscale_fused_kernel(LaunchViews lv, MultiScaleParams p) {
  __shared__ float smem[32];
  Ctx c = make_ctx(lv);
  const RankView& v = *c.v;
  Waiter w{c.hdr, global_ns() + p.c.timeout_ns};
  const uint32_t epoch = next_epoch(c.hdr);
  const uint32_t rng_step = p.c.step + (p.c.step_from_device ? launch_calls(c.hdr) : 0u);
  const int64_t n = p.c.n;
  const int world = p.c.world;
  const int L = p.n_levels;
  const bool al_in = (reinterpret_cast<uintptr_t>(v.in) & 15u) == 0;
  const bool al_out = (reinterpret_cast<uintptr_t>(v.out) & 15u) == 0;
  const int64_t rows = (n + 127) / 128;
  uint8_t* my = v.arena[v.rank];

  float m = rank_max(w, local_absmax(c, v.in, n, al_in), c.bid, c.nblocks, smem, 0x80);
  commit_epoch(c.hdr, epoch, c.bid);
  float norm = (world > 1) ? exchange_max(w, v, world, epoch, m, c.bid == 0, smem) : m;
  float sc[4], dq[4];
#pragma unroll
  for (int l = 0; l < 4; ++l) {
    sc[l] = (l < L && norm > 0.0f) ? (float)p.s[l] / norm : 0.0f;
    dq[l] = l < L ? dequant_scale(norm, p.s[l], world) : 0.0f;
  }
  auto level_of = [&](float x, int l, uint64_t blk, int j) {
    U4 r = philox_block(rng_key(p.c, rng_step, v.rank, PURPOSE_LEVEL0 + (uint32_t)l), blk);
    uint32_t rnd = j == 0 ? r.x : (j == 1 ? r.y : (j == 2 ? r.z : r.w));
    return quantize_level(x, sc[l], p.s[l], rnd);
  };
  // finest scale whose rounded level fits the coarsest range (scale 0 always fits)
  auto local_index = [&](float x, uint64_t blk, int j) {
    int idx = 0;
    for (int l = 1; l < L; ++l)
      if (abs(level_of(x, l, blk, j)) <= p.s[0]) idx = l;
    return idx;
  };

  if (world > 1) {
    for (int64_t row = c.warp; row < rows; row += c.nwarps) {
      int64_t e0 = row * 128 + c.lane * 4;
      float4 x = load_quad(v.in, e0, n, al_in);
      float xs[4] = {x.x, x.y, x.z, x.w};
      bool b0[4], b1[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int idx = local_index(xs[j], (uint64_t)(e0 >> 2), j);
        b0[j] = idx & 1;
        b1[j] = (idx >> 1) & 1;
      }
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_idx_local[0]), row, c.lane, b0);
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_idx_local[1]), row, c.lane, b1);
    }
    grid_barrier(w, c.nblocks, 0x81);
    if (c.bid == 0) signal_all(v, world, PH_MASK, epoch);
    wait_all(w, world, PH_MASK, epoch);
  }

  for (int64_t row = c.warp; row < rows; row += c.nwarps) {
    int64_t e0 = row * 128 + c.lane * 4;
    float4 x = load_quad(v.in, e0, n, al_in);
    float xs[4] = {x.x, x.y, x.z, x.w};
    int idx[4];
    if (world > 1) {
      uint32_t p0 = load_plane_all_ranks(v, world, p.off_idx_local[0], row, c.lane);
      uint32_t p1 = load_plane_all_ranks(v, world, p.off_idx_local[1], row, c.lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) idx[j] = 3;
#pragma unroll
      for (int src = 0; src < MAXW; ++src)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t w0 = __shfl_sync(FULL, p0, src * 4 + j), w1 = __shfl_sync(FULL, p1, src * 4 + j);
          int r = (int)((w0 >> c.lane) & 1u) | ((int)((w1 >> c.lane) & 1u) << 1);
          if (src < world) idx[j] = r < idx[j] ? r : idx[j];
        }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) idx[j] = local_index(xs[j], (uint64_t)(e0 >> 2), j);
    }
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = level_of(xs[j], idx[j], (uint64_t)(e0 >> 2), j);
    if (world == 1) {
      float4 y = make_float4(mul_rn(dq[idx[0]], (float)q[0]), mul_rn(dq[idx[1]], (float)q[1]),
                             mul_rn(dq[idx[2]], (float)q[2]), mul_rn(dq[idx[3]], (float)q[3]));
      store_quad(v.out, e0, n, al_out, y);
    } else {
      int mg[4] = {abs(q[0]), abs(q[1]), abs(q[2]), abs(q[3])};
      bool sg[4] = {q[0] < 0, q[1] < 0, q[2] < 0, q[3] < 0};
      bool b0[4] = {(idx[0] & 1) != 0, (idx[1] & 1) != 0, (idx[2] & 1) != 0, (idx[3] & 1) != 0};
      bool b1[4] = {(idx[0] & 2) != 0, (idx[1] & 2) != 0, (idx[2] & 2) != 0, (idx[3] & 2) != 0};
      store_row_mags<MW>(my + p.off_mags, row, c.lane, mg);
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_signs), row, c.lane, sg);
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_idx_final[0]), row, c.lane, b0);
      store_row_plane(reinterpret_cast<uint32_t*>(my + p.off_idx_final[1]), row, c.lane, b1);
    }
  }
  if (world == 1) return;
  grid_barrier(w, c.nblocks, 0x82);
  if (c.bid == 0) signal_all(v, world, PH_READY, epoch);
  wait_all(w, world, PH_READY, epoch);

  reduce_scatter_rows<MW, SUMB>(c, world, rows, p.chunk_rows, p.off_mags, p.off_signs, p.off_sums);
  grid_barrier(w, c.nblocks, 0x83);
  if (c.bid == 0) signal_all(v, world, PH_DONE, epoch);
  wait_all(w, world, PH_DONE, epoch);

  for (int64_t row = c.warp; row < rows; row += c.nwarps) {
    int a[4];
    bool b0[4], b1[4];
    load_row_sums<SUMB>(my + p.off_sums, row, c.lane, a);
    load_row_plane(reinterpret_cast<const uint32_t*>(my + p.off_idx_final[0]), row, c.lane, b0);
    load_row_plane(reinterpret_cast<const uint32_t*>(my + p.off_idx_final[1]), row, c.lane, b1);
    float y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) y[j] = mul_rn(dq[(b0[j] ? 1 : 0) | (b1[j] ? 2 : 0)], (float)a[j]);
    store_quad(v.out, row * 128 + c.lane * 4, n, al_out, make_float4(y[0], y[1], y[2], y[3]));
  }
}

// ------------------------------------------------------------------------------------------ fp32 all-reduce
struct AllreduceParams {
  Common c;
  int64_t off_stage, off_result;
  int64_t chunk_quads;
  float alpha;   // 1 / W
};

__global__ void __maxnreg__(GC_FUSED_MAXNREG) allreduce_fused_kernel(LaunchViews lv, AllreduceParams p) {
  Ctx c = make_ctx(lv);
  const RankView& v = *c.v;
  Waiter w{c.hdr, global_ns() + p.c.timeout_ns};
  const uint32_t epoch = next_epoch(c.hdr);
  const uint32_t rng_step = p.c.step + (p.c.step_from_device ? launch_calls(c.hdr) : 0u);
  const int64_t n = p.c.n;
  const int world = p.c.world;
  const bool al_in = (reinterpret_cast<uintptr_t>(v.in) & 15u) == 0;
  const bool al_out = (reinterpret_cast<uintptr_t>(v.out) & 15u) == 0;
  const int64_t nq = (n + 3) / 4;
  const int64_t stride = (int64_t)c.nblocks * THREADS;
  const int64_t tid = (int64_t)c.bid * THREADS + threadIdx.x;
  if (world == 1) {
    if (v.in != v.out)
      for (int64_t q = tid; q < nq; q += stride) store_quad(v.out, q * 4, n, al_out, load_quad(v.in, q * 4, n, al_in));
    return;
  }
  float4* stage = reinterpret_cast<float4*>(v.arena[v.rank] + p.off_stage);
  {
    int64_t q = tid;
    for (; q + 3 * stride < nq; q += 4 * stride) {
      float4 a = load_quad(v.in, q * 4, n, al_in), b = load_quad(v.in, (q + stride) * 4, n, al_in);
      float4 d = load_quad(v.in, (q + 2 * stride) * 4, n, al_in), e = load_quad(v.in, (q + 3 * stride) * 4, n, al_in);
      stage[q] = a; stage[q + stride] = b; stage[q + 2 * stride] = d; stage[q + 3 * stride] = e;
    }
    for (; q < nq; q += stride) stage[q] = load_quad(v.in, q * 4, n, al_in);
  }
  grid_barrier(w, c.nblocks, 0x40);
  commit_epoch(c.hdr, epoch, c.bid);
  if (c.bid == 0) signal_all(v, world, PH_STAGE, epoch);
  wait_all(w, world, PH_STAGE, epoch);

  int64_t q0 = (int64_t)v.rank * p.chunk_quads;
  int64_t q1 = q0 + p.chunk_quads < nq ? q0 + p.chunk_quads : nq;
  for (int64_t q = q0 + tid; q < q1; q += stride) {
    float4 part[MAXW];
#pragma unroll
    for (int src = 0; src < MAXW; ++src)
      if (src < world) part[src] = reinterpret_cast<const float4*>(v.arena[src] + p.off_stage)[q];
    float4 acc = part[0];
#pragma unroll
    for (int src = 1; src < MAXW; ++src)
      if (src < world) { acc.x += part[src].x; acc.y += part[src].y; acc.z += part[src].z; acc.w += part[src].w; }
    acc.x *= p.alpha; acc.y *= p.alpha; acc.z *= p.alpha; acc.w *= p.alpha;
#pragma unroll
    for (int dst = 0; dst < MAXW; ++dst)
      if (dst < world) reinterpret_cast<float4*>(v.arena[dst] + p.off_result)[q] = acc;
  }
  grid_barrier(w, c.nblocks, 0x41);
  if (c.bid == 0) signal_all(v, world, PH_DONE, epoch);
  wait_all(w, world, PH_DONE, epoch);

  const float4* res = reinterpret_cast<const float4*>(v.arena[v.rank] + p.off_result);
  {
    int64_t q = tid;
    for (; q + 3 * stride < nq; q += 4 * stride) {
      float4 a = res[q], b = res[q + stride], d = res[q + 2 * stride], e = res[q + 3 * stride];
      store_quad(v.out, q * 4, n, al_out, a); store_quad(v.out, (q + stride) * 4, n, al_out, b);
      store_quad(v.out, (q + 2 * stride) * 4, n, al_out, d); store_quad(v.out, (q + 3 * stride) * 4, n, al_out, e);
    }
    for (; q < nq; q += stride) store_quad(v.out, q * 4, n, al_out, res[q]);
  }
}

// ------------------------------------------------------------------------------------------ small one-shot fp32 sum
struct SmallSumParams {
  Common c;
  int64_t off_buf;   // double-buffered by epoch parity: off_buf + parity * half_bytes
  int64_t half_bytes;   // distance between the two parity regions: fixed per arena, independent of the call's size
  float alpha;
};

__global__ void __launch_bounds__(THREADS) small_sum_kernel(LaunchViews lv, SmallSumParams p) {
  Ctx c = make_ctx(lv);
  const RankView& v = *c.v;
  Waiter w{c.hdr, global_ns() + p.c.timeout_ns};
  const uint32_t epoch = next_epoch(c.hdr);
  const uint32_t rng_step = p.c.step + (p.c.step_from_device ? launch_calls(c.hdr) : 0u);
  const int64_t n = p.c.n;
  const int world = p.c.world;
  const int64_t stride = (int64_t)c.nblocks * THREADS;
  const int64_t tid = (int64_t)c.bid * THREADS + threadIdx.x;
  if (world == 1) {
    for (int64_t i = tid; i < n; i += stride) v.out[i] = v.in[i] * p.alpha;
    return;
  }
  int64_t off = p.off_buf + (int64_t)(epoch & 1) * p.half_bytes;
  float* mine = reinterpret_cast<float*>(v.arena[v.rank] + off);
  for (int64_t i = tid; i < n; i += stride) mine[i] = v.in[i];
  grid_barrier(w, c.nblocks, 0x50);
  commit_epoch(c.hdr, epoch, c.bid);
  if (c.bid == 0) signal_all(v, world, PH_AUX, epoch);
  wait_all(w, world, PH_AUX, epoch);
  for (int64_t i = tid; i < n; i += stride) {
    float acc = 0.0f;
#pragma unroll
    for (int src = 0; src < MAXW; ++src)
      if (src < world) acc += reinterpret_cast<const float*>(v.arena[src] + off)[i];
    v.out[i] = acc * p.alpha;
  }
}

// ------------------------------------------------------------------------------------------ Rand-K
struct RandkParams {
  Common c;
  PermKey perm;
  int64_t start, k;
  int s_lo, s_hi;          // s_hi == 0: single scale
  int zero_unselected;     // 0: unselected coordinates become in / W ; 1: zero
  int64_t off_vals, off_levels, off_mask;   // scratch regions inside a parity region (selected by epoch & 1)
  int64_t half_bytes;                       // distance between the two parity regions: fixed per arena
  int64_t* window;         // device-resident start of this step's window (may be NULL: p.start is used).  The kernel
                           // advances it by K, wrapping at n, so a launch replayed from a CUDA graph walks the
                           // permutation like a sequence of fresh launches does.
};

__global__ void __launch_bounds__(THREADS) randk_fused_kernel(LaunchViews lv, RandkParams p) {
  __shared__ float smem[32];
  Ctx c = make_ctx(lv);
  const RankView& v = *c.v;
  Waiter w{c.hdr, global_ns() + p.c.timeout_ns};
  const uint32_t epoch = next_epoch(c.hdr);
  const uint32_t rng_step = p.c.step + (p.c.step_from_device ? launch_calls(c.hdr) : 0u);
  const int64_t n = p.c.n;
  const int64_t start = p.window != nullptr ? *((volatile const int64_t*)p.window) : p.start;
  const int64_t k = p.k < n - start ? p.k : n - start;
  const int world = p.c.world;
  const bool al_in = (reinterpret_cast<uintptr_t>(v.in) & 15u) == 0;
  const bool al_out = (reinterpret_cast<uintptr_t>(v.out) & 15u) == 0;
  const int64_t stride = (int64_t)c.nblocks * THREADS;
  const int64_t tid = (int64_t)c.bid * THREADS + threadIdx.x;
  uint8_t* my = v.arena[v.rank];
  const int64_t par_off = (int64_t)(epoch & 1) * p.half_bytes;
  float* vals = reinterpret_cast<float*>(my + p.off_vals + par_off);
  int32_t* levels = reinterpret_cast<int32_t*>(my + p.off_levels + par_off);
  uint8_t* mask = my + p.off_mask + par_off;

  // gather the K selected coordinates first (the dense pass below may overwrite them in place)
  float m = 0.0f;
  for (int64_t i = tid; i < k; i += stride) {
    const uint64_t at = perm_eval(p.perm, (uint64_t)(start + i));
    float x = GC_INDEX_OK(w, at, n) ? v.in[at] : 0.0f;
    vals[i] = x;
    m = fmaxf(m, abs_for_max(x));
  }
  m = rank_max(w, m, c.bid, c.nblocks, smem, 0x60);   // grid barrier inside: every gather is done
  commit_epoch(c.hdr, epoch, c.bid);
  // dense pass: what the unselected coordinates become
  {
    float alpha = p.zero_unselected ? 0.0f : 1.0f / (float)world;
    if (!(alpha == 1.0f && v.in == v.out)) {
      int64_t nq = (n + 3) / 4;
      int64_t q = tid;
      for (; q + 3 * stride < nq; q += 4 * stride) {
        float4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) x[u] = load_quad(v.in, (q + u * stride) * 4, n, al_in);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          x[u].x *= alpha; x[u].y *= alpha; x[u].z *= alpha; x[u].w *= alpha;
          store_quad(v.out, (q + u * stride) * 4, n, al_out, x[u]);
        }
      }
      for (; q < nq; q += stride) {
        float4 x = load_quad(v.in, q * 4, n, al_in);
        x.x *= alpha; x.y *= alpha; x.z *= alpha; x.w *= alpha;
        store_quad(v.out, q * 4, n, al_out, x);
      }
    }
  }
  float norm = (world > 1) ? exchange_max(w, v, world, epoch, m, c.bid == 0, smem) : m;
  // every block of every rank of this launch has read the window by now (own rank: the grid barrier inside rank_max;
  // other virtual ranks of an emulated group: they published their maxima after theirs): one thread advances it
  if (p.window != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *p.window = start + k >= n ? 0 : start + k;
  const bool two = p.s_hi > 0;
  float sc_lo = (norm > 0.0f) ? (float)p.s_lo / norm : 0.0f;
  float sc_hi = (norm > 0.0f && two) ? (float)p.s_hi / norm : 0.0f;
  float dq_lo = dequant_scale(norm, p.s_lo, world), dq_hi = two ? dequant_scale(norm, p.s_hi, world) : 0.0f;
  RngKey k_lo = rng_key(p.c, rng_step, v.rank, PURPOSE_ROUND), k_hi = rng_key(p.c, rng_step, v.rank, PURPOSE_ROUND_HI);

  auto word_of = [](const U4& r, int j) { return j == 0 ? r.x : j == 1 ? r.y : j == 2 ? r.z : r.w; };

  if (two && world > 1) {
    for (int64_t i = tid; i < k; i += stride) {
      U4 rh = philox_block(k_hi, (uint64_t)(i >> 2));
      int qh = quantize_level(vals[i], sc_hi, p.s_hi, word_of(rh, (int)(i & 3)));
      mask[i] = abs(qh) <= p.s_lo ? 1 : 0;
    }
    grid_barrier(w, c.nblocks, 0x61);
    if (c.bid == 0) signal_all(v, world, PH_MASK, epoch);
    wait_all(w, world, PH_MASK, epoch);
  }
  for (int64_t i = tid; i < k; i += stride) {
    float x = vals[i];
    U4 rl = philox_block(k_lo, (uint64_t)(i >> 2));
    int q = quantize_level(x, sc_lo, p.s_lo, word_of(rl, (int)(i & 3)));
    bool hi = false;
    if (two) {
      U4 rh = philox_block(k_hi, (uint64_t)(i >> 2));
      int qh = quantize_level(x, sc_hi, p.s_hi, word_of(rh, (int)(i & 3)));
      hi = abs(qh) <= p.s_lo;
      if (world > 1) {
#pragma unroll
        for (int src = 0; src < MAXW; ++src)
          if (src < world) hi = hi && (v.arena[src] + p.off_mask + par_off)[i] != 0;
      }
      if (hi) q = qh;
    }
    levels[i] = q;
    vals[i] = hi ? 1.0f : 0.0f;   // the gathered value is consumed; keep the agreed scale flag in its place
  }
  if (world > 1) {
    grid_barrier(w, c.nblocks, 0x62);
    if (c.bid == 0) signal_all(v, world, PH_READY, epoch);
    wait_all(w, world, PH_READY, epoch);
  } else {
    grid_barrier(w, c.nblocks, 0x62);
  }
  for (int64_t i = tid; i < k; i += stride) {
    int acc = 0;
#pragma unroll
    for (int src = 0; src < MAXW; ++src)
      if (src < world) acc += reinterpret_cast<const int32_t*>(v.arena[src] + p.off_levels + par_off)[i];
    bool hi = two && vals[i] != 0.0f;
    const uint64_t at = perm_eval(p.perm, (uint64_t)(start + i));
    if (GC_INDEX_OK(w, at, n)) v.out[at] = mul_rn(hi ? dq_hi : dq_lo, (float)acc);
  }
}

// ------------------------------------------------------------------------------------------ sparse exchange
// Every rank contributes `count` (index, value) pairs; the result is out = alpha * sum over ranks of the
// scattered pairs (zero elsewhere).  Lists are published in the arena, read by every rank (one-shot), and
// applied rank by rank with a grid barrier in between, so the floating-point sum has a fixed order and no
// atomics are needed (indices are unique within one rank's list).
struct SparseParams {
  Common c;
  int64_t count;
  int64_t off_idx, off_val, half_bytes;     // list regions inside a parity region; fixed distance between the two regions
  float alpha;
};

__global__ void __launch_bounds__(THREADS, 2) sparse_fused_kernel(LaunchViews lv, SparseParams p) {
  Ctx c = make_ctx(lv);
  const RankView& v = *c.v;
  Waiter w{c.hdr, global_ns() + p.c.timeout_ns};
  const uint32_t epoch = next_epoch(c.hdr);
  const int64_t n = p.c.n;
  const int world = p.c.world;
  const bool al_out = (reinterpret_cast<uintptr_t>(v.out) & 15u) == 0;
  const int64_t stride = (int64_t)c.nblocks * THREADS;
  const int64_t tid = (int64_t)c.bid * THREADS + threadIdx.x;
  const int64_t par_off = (int64_t)(epoch & 1) * p.half_bytes;
  const int32_t* my_idx = reinterpret_cast<const int32_t*>(v.aux);
  {
    int64_t nq = (n + 3) / 4;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t q = tid; q < nq; q += stride) store_quad(v.out, q * 4, n, al_out, z);
  }
  if (world > 1) {
    int32_t* pub_idx = reinterpret_cast<int32_t*>(v.arena[v.rank] + p.off_idx + par_off);
    float* pub_val = reinterpret_cast<float*>(v.arena[v.rank] + p.off_val + par_off);
    for (int64_t i = tid; i < p.count; i += stride) { pub_idx[i] = my_idx[i]; pub_val[i] = v.in[i]; }
  }
  grid_barrier(w, c.nblocks, 0x70);
  commit_epoch(c.hdr, epoch, c.bid);
  if (world > 1) {
    if (c.bid == 0) signal_all(v, world, PH_AUX, epoch);
    wait_all(w, world, PH_AUX, epoch);
  }
  for (int src = 0; src < world; ++src) {
    const int32_t* idx = world > 1 ? reinterpret_cast<const int32_t*>(v.arena[src] + p.off_idx + par_off) : my_idx;
    const float* val = world > 1 ? reinterpret_cast<const float*>(v.arena[src] + p.off_val + par_off) : v.in;
    for (int64_t i = tid; i < p.count; i += stride) {
      int32_t at = idx[i];
      if (at >= 0 && at < n) v.out[at] += p.alpha * val[i];
      else w.out_of_bounds(at);                 // an index list from outside this library: reported, never followed
    }
    if (src + 1 < world) grid_barrier(w, c.nblocks, 0x71);
  }
}

// ------------------------------------------------------------------------------------------ host side
struct CommCtx {
  int world, rank, device;
  int64_t bytes;
  uint8_t* local;
  uint8_t* peers[MAXW];
  bool ipc_opened[MAXW];
  int step_from_device;
  int sm_count;
};

int max_coresident(const void* kernel, int sm_count) {
  int per_sm = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, 0);
  if (per_sm < 1) per_sm = 1;
  return per_sm * sm_count;
}

// Blocks that a problem of `n` elements can keep busy: small messages get a small grid, which keeps the
// grid barriers (and hence the latency floor of the fused kernels) short.
int blocks_for_elems(int64_t n) {
  int64_t per_block = (int64_t)THREADS * 16;      // four 16-byte accesses per thread
  int64_t b = (n + per_block - 1) / per_block;
  return (int)(b < 1 ? 1 : (b > 4096 ? 4096 : b));
}

int fill_views(CommCtx** ctxs, int n_virtual, const float* const* ins, float* const* outs, int coresident,
               int max_blocks, LaunchViews* lv, const void* const* auxs = nullptr, int64_t work_elems = -1) {
  if (n_virtual < 1 || n_virtual > MAXW) return -1;
  int world = ctxs[0]->world;
  int total = coresident;
  if (work_elems >= 0) {
    int want = blocks_for_elems(work_elems);
    if (max_blocks <= 0 || want < max_blocks) max_blocks = want;
  }
  if (max_blocks > 0 && max_blocks * n_virtual < total) total = max_blocks * n_virtual;
  int per = total / n_virtual;
  if (per > MAX_PARTIALS / 2) per = MAX_PARTIALS / 2;
  if (per < 1) return -2;
  lv->n_virtual = n_virtual;
  lv->blocks_per_rank = per;
  for (int i = 0; i < n_virtual; ++i) {
    RankView& r = lv->r[i];
    for (int p = 0; p < MAXW; ++p) r.arena[p] = p < world ? ctxs[i]->peers[p] : nullptr;
    r.in = ins[i];
    r.out = outs[i];
    r.aux = auxs ? auxs[i] : nullptr;
    r.rank = ctxs[i]->rank;
    r.pad = 0;
    for (int p = 0; p < world; ++p)
      if (r.arena[p] == nullptr) return -3;
  }
  return 0;
}

// 0: always a cooperative launch (co-residency of the grid is guaranteed by the driver).  1: grids of at most one block
// per SM are launched as ordinary kernels.  Their blocks still all become resident -- nothing else on the device ever
// waits for them, so the scheduler places them as soon as the kernels they run beside retire blocks, and every wait is
// bounded anyway -- but an ordinary launch may overlap with the kernels of other streams, which is what the bucketed
// reducer wants for the reduces it runs beside backward (a cooperative launch measured as a barrier between them).
int g_small_grid_plain_launch = 0;

template <typename P>
int coop_launch(const void* kernel, const LaunchViews& lv, const P& params, cudaStream_t st) {
  void* args[2] = {(void*)&lv, (void*)&params};
  dim3 grid((unsigned)(lv.n_virtual * lv.blocks_per_rank)), block(THREADS);
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaError_t e;
  if (g_small_grid_plain_launch && (int)grid.x <= sms) e = cudaLaunchKernel(kernel, grid, block, args, 0, st);
  else e = cudaLaunchCooperativeKernel(kernel, grid, block, args, 0, st);
  return (int)e;
}

Common make_common(CommCtx** ctxs, int n_virtual, int64_t n, uint64_t seed, uint32_t step, int timeout_ms) {
  Common c;
  c.n = n;
  c.world = ctxs[0]->world;
  c.step_from_device = ctxs[0]->step_from_device;
  (void)n_virtual;
  c.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 30000) * 1000000ull;
  c.seed_lo = (uint32_t)seed;
  c.seed_hi = (uint32_t)(seed >> 32);
  c.step = step;
  return c;
}

inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// The one-shot kernels (small sum, sparse exchange, Rand-K) have no closing round: a fast rank may start step e + 1
// while a slower peer still reads what it published in step e.  They therefore alternate between two regions of the
// arena by epoch parity, and the distance between the regions depends on the ARENA only -- never on the size of a
// call -- so that launches of different sizes (buckets, different reducers on one arena) cannot make step e + 1's
// region overlap step e's.
inline int64_t parity_half_bytes(int64_t arena_bytes) { return (arena_bytes - ARENA_HEADER_BYTES) / 2 / 256 * 256; }

}  // namespace

extern "C" {

int64_t gc_comm_header_bytes() { return ARENA_HEADER_BYTES; }
void gc_fused_small_grid_plain_launch(int on) { g_small_grid_plain_launch = on ? 1 : 0; }
int gc_comm_max_world() { return MAXW; }

// Bytes of arena a one-shot kernel needs when each of its parity regions holds `region_bytes`.
int64_t gc_comm_oneshot_bytes(int64_t region_bytes) { return ARENA_HEADER_BYTES + 2 * align_up(region_bytes, 256) + 512; }

// Bytes of arena needed by the largest fused op on an n-element gradient.
int64_t gc_comm_required_bytes(int64_t n) {
  int64_t npad = pad128(n);
  int64_t qsgd = mag_bytes(npad, 16) + 5 * plane_bytes(npad) + npad * 4 + 8 * 256;   // mags(16b) + signs + 4 index planes + int32 sums
  int64_t ar = 2 * npad * 4;                                               // fp32 stage + result
  int64_t need = qsgd > ar ? qsgd : ar;
  return ARENA_HEADER_BYTES + need + 4096;
}

int gc_comm_create(int world, int rank, int64_t bytes, void** out_ctx) {
  if (world < 1 || world > MAXW || rank < 0 || rank >= world || bytes < ARENA_HEADER_BYTES) return (int)cudaErrorInvalidValue;
  CommCtx* c = new CommCtx();
  memset(c, 0, sizeof(*c));
  c->world = world;
  c->rank = rank;
  c->bytes = bytes;
  cudaGetDevice(&c->device);
  cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, c->device);
  cudaError_t e = cudaMalloc((void**)&c->local, (size_t)bytes);
  if (e != cudaSuccess) { delete c; return (int)e; }
  e = cudaMemset(c->local, 0, (size_t)bytes);
  if (e != cudaSuccess) { cudaFree(c->local); delete c; return (int)e; }
  cudaDeviceSynchronize();
  c->peers[rank] = c->local;
  *out_ctx = c;
  return 0;
}

int gc_comm_ipc_handle(void* ctx, void* out64) {
  CommCtx* c = (CommCtx*)ctx;
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, c->local);
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out64, &h, 64);
  return 0;
}

// handles: world * 64 bytes, entry r = rank r's handle (own entry ignored).
int gc_comm_open_peers(void* ctx, const void* handles) {
  CommCtx* c = (CommCtx*)ctx;
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const uint8_t*)handles + 64 * r, 64);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    c->peers[r] = (uint8_t*)p;
    c->ipc_opened[r] = true;
  }
  return 0;
}

// Same-process wiring (single-GPU emulation of a group, or tests): rank r's arena is at `ptr`.
int gc_comm_set_peer(void* ctx, int r, void* ptr) {
  CommCtx* c = (CommCtx*)ctx;
  if (r < 0 || r >= c->world) return (int)cudaErrorInvalidValue;
  c->peers[r] = (uint8_t*)ptr;
  return 0;
}

void* gc_comm_arena_ptr(void* ctx) { return ((CommCtx*)ctx)->local; }
int64_t gc_comm_arena_bytes(void* ctx) { return ((CommCtx*)ctx)->bytes; }
// 1: kernels add the rank's launch counter to the Philox step (set before capturing a CUDA graph).
void gc_comm_set_step_from_device(void* ctx, int on) { ((CommCtx*)ctx)->step_from_device = on ? 1 : 0; }

// Reads (status, detail) of this rank's arena; synchronises the given stream.
int gc_comm_status(void* ctx, uint32_t* out2, void* cs) {
  CommCtx* c = (CommCtx*)ctx;
  ArenaHeader* h = (ArenaHeader*)c->local;
  cudaError_t e = cudaMemcpyAsync(out2, &h->status, 8, cudaMemcpyDeviceToHost, (cudaStream_t)cs);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize((cudaStream_t)cs);
}

// Enqueue a copy of (status, detail) into pinned host memory on the given stream; does not wait.  The caller reads the
// words after an event recorded behind the copy has completed.
int gc_comm_status_async(void* ctx, uint32_t* pinned_out2, void* cs) {
  CommCtx* c = (CommCtx*)ctx;
  ArenaHeader* h = (ArenaHeader*)c->local;
  return (int)cudaMemcpyAsync(pinned_out2, &h->status, 8, cudaMemcpyDeviceToHost, (cudaStream_t)cs);
}

// 1 when this library was built with the debug bounds checks.
int gc_comm_debug_bounds() {
#if defined(GC_DEBUG_BOUNDS)
  return 1;
#else
  return 0;
#endif
}

int gc_comm_clear_status(void* ctx, void* cs) {
  CommCtx* c = (CommCtx*)ctx;
  ArenaHeader* h = (ArenaHeader*)c->local;
  // status, status_detail, abort are adjacent; the barrier words are reset too (a timed-out barrier
  // may have left arrivals behind)
  return (int)cudaMemsetAsync(&h->bar_count, 0, 5 * sizeof(uint32_t), (cudaStream_t)cs);   // bar_count .. abort
}

int gc_comm_destroy(void* ctx) {
  CommCtx* c = (CommCtx*)ctx;
  if (!c) return 0;
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (c->ipc_opened[r]) cudaIpcCloseMemHandle(c->peers[r]);
  cudaFree(c->local);
  delete c;
  return 0;
}

#define GC_KERNEL_TABLE(NAME, KERNEL)                                         \
  static const void* NAME(int mw, int sumb) {                                 \
    switch (mw * 8 + sumb) {                                                  \
      case 1 * 8 + 1: return (const void*)KERNEL<1, 1>;                       \
      case 1 * 8 + 2: return (const void*)KERNEL<1, 2>;                       \
      case 1 * 8 + 4: return (const void*)KERNEL<1, 4>;                       \
      case 2 * 8 + 1: return (const void*)KERNEL<2, 1>;                       \
      case 2 * 8 + 2: return (const void*)KERNEL<2, 2>;                       \
      case 2 * 8 + 4: return (const void*)KERNEL<2, 4>;                       \
      case 4 * 8 + 1: return (const void*)KERNEL<4, 1>;                       \
      case 4 * 8 + 2: return (const void*)KERNEL<4, 2>;                       \
      case 4 * 8 + 4: return (const void*)KERNEL<4, 4>;                       \
      case 8 * 8 + 1: return (const void*)KERNEL<8, 1>;                       \
      case 8 * 8 + 2: return (const void*)KERNEL<8, 2>;                       \
      case 8 * 8 + 4: return (const void*)KERNEL<8, 4>;                       \
      case 16 * 8 + 1: return (const void*)KERNEL<16, 1>;                     \
      case 16 * 8 + 2: return (const void*)KERNEL<16, 2>;                     \
      case 16 * 8 + 4: return (const void*)KERNEL<16, 4>;                     \
    }                                                                         \
    return nullptr;                                                           \
  }
GC_KERNEL_TABLE(qsgd_kernel_for, qsgd_fused_kernel)
GC_KERNEL_TABLE(twoscale_kernel_for, twoscale_fused_kernel)
GC_KERNEL_TABLE(multiscale_kernel_for, multiscale_fused_kernel)

// One QSGD-MaxNorm reduce step.  ctxs: n_virtual contexts (1 in multi-GPU runs; all ranks of an
// emulated group otherwise); ins / outs: one gradient pointer per context.
int gc_fused_qsgd(void** ctxs_, int n_virtual, const float* const* ins, float* const* outs, int64_t n, int bits,
                  uint64_t seed, uint32_t step, int timeout_ms, int max_blocks, void* cs) {
  CommCtx** ctxs = (CommCtx**)ctxs_;
  int world = ctxs[0]->world;
  int s = (1 << bits) - 1, mw = mag_width(bits), sumb = sum_container_bytes(s, world);
  int64_t npad = pad128(n);
  QsgdParams p;
  p.s = s;
  p.off_mags = ARENA_HEADER_BYTES;
  p.off_signs = align_up(p.off_mags + mag_bytes(npad, mw), 256);
  p.off_sums = align_up(p.off_signs + plane_bytes(npad), 256);
  if (p.off_sums + npad * sumb > ctxs[0]->bytes) return (int)cudaErrorMemoryAllocation;
  int64_t rows = npad / 128;
  p.chunk_rows = (rows + world - 1) / world;
  const void* kern = qsgd_kernel_for(mw, sumb);
  if (kern == nullptr) return (int)cudaErrorInvalidValue;
  LaunchViews lv;
  if (fill_views(ctxs, n_virtual, ins, outs, max_coresident(kern, ctxs[0]->sm_count), max_blocks, &lv, nullptr, n) != 0)
    return (int)cudaErrorInvalidValue;
  p.c = make_common(ctxs, n_virtual, n, seed, step, timeout_ms);
  return coop_launch(kern, lv, p, (cudaStream_t)cs);
}

int gc_fused_twoscale(void** ctxs_, int n_virtual, const float* const* ins, float* const* outs, int64_t n, int bits_lo,
                      int bits_hi, uint64_t seed, uint32_t step, int timeout_ms, int max_blocks, void* cs) {
  CommCtx** ctxs = (CommCtx**)ctxs_;
  int world = ctxs[0]->world;
  int s_lo = (1 << bits_lo) - 1, s_hi = (1 << bits_hi) - 1, mw = mag_width(bits_lo);
  int sumb = sum_container_bytes(s_lo, world);
  int64_t npad = pad128(n);
  TwoScaleParams p;
  p.s_lo = s_lo;
  p.s_hi = s_hi;
  p.off_mags = ARENA_HEADER_BYTES;
  p.off_signs = align_up(p.off_mags + mag_bytes(npad, mw), 256);
  p.off_mask_local = align_up(p.off_signs + plane_bytes(npad), 256);
  p.off_mask_final = align_up(p.off_mask_local + plane_bytes(npad), 256);
  p.off_sums = align_up(p.off_mask_final + plane_bytes(npad), 256);
  if (p.off_sums + npad * sumb > ctxs[0]->bytes) return (int)cudaErrorMemoryAllocation;
  int64_t rows = npad / 128;
  p.chunk_rows = (rows + world - 1) / world;
  const void* kern = twoscale_kernel_for(mw, sumb);
  if (kern == nullptr) return (int)cudaErrorInvalidValue;
  LaunchViews lv;
  if (fill_views(ctxs, n_virtual, ins, outs, max_coresident(kern, ctxs[0]->sm_count), max_blocks, &lv, nullptr, n) != 0)
    return (int)cudaErrorInvalidValue;
  p.c = make_common(ctxs, n_virtual, n, seed, step, timeout_ms);
  return coop_launch(kern, lv, p, (cudaStream_t)cs);
}

// levels: n_levels ascending bit widths (2 <= n_levels <= 4); values on the wire never exceed 2^levels[0] - 1.
int gc_fused_multiscale(void** ctxs_, int n_virtual, const float* const* ins, float* const* outs, int64_t n,
                        const int* levels, int n_levels, uint64_t seed, uint32_t step, int timeout_ms, int max_blocks,
                        void* cs) {
  CommCtx** ctxs = (CommCtx**)ctxs_;
  if (n_levels < 1 || n_levels > 4) return (int)cudaErrorInvalidValue;
  int world = ctxs[0]->world;
  MultiScaleParams p;
  p.n_levels = n_levels;
  for (int l = 0; l < 4; ++l) p.s[l] = l < n_levels ? (1 << levels[l]) - 1 : 0;
  int mw = mag_width(levels[0]), sumb = sum_container_bytes(p.s[0], world);
  int64_t npad = pad128(n), off = ARENA_HEADER_BYTES;
  auto take = [&](int64_t bytes) { int64_t r = off; off = align_up(off + bytes, 256); return r; };
  p.off_mags = take(mag_bytes(npad, mw));
  p.off_signs = take(plane_bytes(npad));
  p.off_idx_local[0] = take(plane_bytes(npad));
  p.off_idx_local[1] = take(plane_bytes(npad));
  p.off_idx_final[0] = take(plane_bytes(npad));
  p.off_idx_final[1] = take(plane_bytes(npad));
  p.off_sums = take(npad * sumb);
  if (off > ctxs[0]->bytes) return (int)cudaErrorMemoryAllocation;
  int64_t rows = npad / 128;
  p.chunk_rows = (rows + world - 1) / world;
  const void* kern = multiscale_kernel_for(mw, sumb);
  if (kern == nullptr) return (int)cudaErrorInvalidValue;
  LaunchViews lv;
  if (fill_views(ctxs, n_virtual, ins, outs, max_coresident(kern, ctxs[0]->sm_count), max_blocks, &lv, nullptr, n) != 0)
    return (int)cudaErrorInvalidValue;
  p.c = make_common(ctxs, n_virtual, n, seed, step, timeout_ms);
  return coop_launch(kern, lv, p, (cudaStream_t)cs);
}

int gc_fused_allreduce(void** ctxs_, int n_virtual, const float* const* ins, float* const* outs, int64_t n,
                       int timeout_ms, int max_blocks, void* cs) {
  CommCtx** ctxs = (CommCtx**)ctxs_;
  int world = ctxs[0]->world;
  int64_t npad = pad128(n);
  AllreduceParams p;
  p.off_stage = ARENA_HEADER_BYTES;
  p.off_result = align_up(p.off_stage + npad * 4, 256);
  if (world > 1 && p.off_result + npad * 4 > ctxs[0]->bytes) return (int)cudaErrorMemoryAllocation;
  int64_t nq = npad / 4;
  p.chunk_quads = (nq + world - 1) / world;
  p.alpha = 1.0f / (float)world;
  const void* kern = (const void*)allreduce_fused_kernel;
  LaunchViews lv;
  if (fill_views(ctxs, n_virtual, ins, outs, max_coresident(kern, ctxs[0]->sm_count), max_blocks, &lv, nullptr, n) != 0)
    return (int)cudaErrorInvalidValue;
  p.c = make_common(ctxs, n_virtual, n, 0, 0, timeout_ms);
  return coop_launch(kern, lv, p, (cudaStream_t)cs);
}

// out = alpha * sum over ranks of in, for short vectors (n * 4 * 2 bytes of arena after the header).
int gc_fused_small_sum(void** ctxs_, int n_virtual, const float* const* ins, float* const* outs, int64_t n, float alpha,
                       int timeout_ms, int max_blocks, void* cs) {
  CommCtx** ctxs = (CommCtx**)ctxs_;
  SmallSumParams p;
  p.off_buf = ARENA_HEADER_BYTES;
  p.half_bytes = parity_half_bytes(ctxs[0]->bytes);
  if (ctxs[0]->world > 1 && align_up(n * 4, 256) > p.half_bytes) return (int)cudaErrorMemoryAllocation;
  p.alpha = alpha;
  const void* kern = (const void*)small_sum_kernel;
  LaunchViews lv;
  int blocks = (int)((n + THREADS - 1) / THREADS);
  if (blocks < 1) blocks = 1;
  if (max_blocks <= 0 || blocks < max_blocks) max_blocks = blocks;
  if (fill_views(ctxs, n_virtual, ins, outs, max_coresident(kern, ctxs[0]->sm_count), max_blocks, &lv) != 0)
    return (int)cudaErrorInvalidValue;
  p.c = make_common(ctxs, n_virtual, n, 0, 0, timeout_ms);
  return coop_launch(kern, lv, p, (cudaStream_t)cs);
}

// Sparse all-gather + scatter-add: out (n floats) = alpha * sum over ranks of scatter(idx, val); `count` pairs
// per rank (the same on every rank).  Needs 4 * align256(count * 4) bytes of arena after the header.
int gc_fused_sparse(void** ctxs_, int n_virtual, const float* const* vals, float* const* outs, const void* const* idxs,
                    int64_t n, int64_t count, float alpha, int timeout_ms, int max_blocks, void* cs) {
  CommCtx** ctxs = (CommCtx**)ctxs_;
  SparseParams p;
  p.count = count;
  p.alpha = alpha;
  const int64_t region = align_up(count * 4, 256);
  p.half_bytes = parity_half_bytes(ctxs[0]->bytes);
  p.off_idx = ARENA_HEADER_BYTES;
  p.off_val = p.off_idx + region;
  if (ctxs[0]->world > 1 && 2 * region > p.half_bytes) return (int)cudaErrorMemoryAllocation;
  const void* kern = (const void*)sparse_fused_kernel;
  LaunchViews lv;
  if (fill_views(ctxs, n_virtual, vals, outs, max_coresident(kern, ctxs[0]->sm_count), max_blocks, &lv, idxs, n) != 0)
    return (int)cudaErrorInvalidValue;
  p.c = make_common(ctxs, n_virtual, n, 0, 0, timeout_ms);
  return coop_launch(kern, lv, p, (cudaStream_t)cs);
}

// One Rand-K (optionally two-scale: bits_hi > 0) reduce step on the window [start, start + k) of the
// keyed permutation of [0, n).  window (device int64, may be NULL): when given, the window starts at *window instead of
// `start`, holds min(k, n - *window) coordinates, and the kernel stores the next step's start there (0 after the last
// window of a pass); every rank of a group must pass its own counter with the same value.
int gc_fused_randk(void** ctxs_, int n_virtual, const float* const* ins, float* const* outs, int64_t n, uint64_t seed,
                   uint32_t npass, int64_t start, int64_t k, int bits_lo, int bits_hi, int zero_unselected,
                   uint32_t step, int64_t* window, int timeout_ms, int max_blocks, void* cs) {
  CommCtx** ctxs = (CommCtx**)ctxs_;
  RandkParams p;
  p.perm = make_perm_key((uint64_t)n, seed, npass);
  p.start = start;
  p.k = k;
  p.window = window;
  p.s_lo = (1 << bits_lo) - 1;
  p.s_hi = bits_hi > 0 ? (1 << bits_hi) - 1 : 0;
  p.zero_unselected = zero_unselected;
  const int64_t region = align_up(k * 4, 256);
  p.half_bytes = parity_half_bytes(ctxs[0]->bytes);
  p.off_vals = ARENA_HEADER_BYTES;
  p.off_levels = p.off_vals + region;
  p.off_mask = p.off_levels + region;
  if (3 * region > p.half_bytes) return (int)cudaErrorMemoryAllocation;
  const void* kern = (const void*)randk_fused_kernel;
  LaunchViews lv;
  if (fill_views(ctxs, n_virtual, ins, outs, max_coresident(kern, ctxs[0]->sm_count), max_blocks, &lv, nullptr, n) != 0)
    return (int)cudaErrorInvalidValue;
  p.c = make_common(ctxs, n_virtual, n, seed, step, timeout_ms);
  return coop_launch(kern, lv, p, (cudaStream_t)cs);
}

}  // extern "C"
