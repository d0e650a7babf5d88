// Shared host/device definitions: Philox4x32-10, the stochastic quantiser and the packed wire
// layout.  Every function here compiles both for the CPU oracle (g++) and for sm_100a (nvcc), so a
// kernel and its oracle consume the same random bits and produce the same integers.
#pragma once
#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define GC_HD __host__ __device__ __forceinline__
#else
#define GC_HD inline
#endif

namespace gc {

// ---------------------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
// key = (seed_lo, seed_hi); counter = (block_lo, block_hi, step, stream).  One call gives four
// 32-bit words; element i of a tensor uses word i%4 of block i/4.
// ---------------------------------------------------------------------------------------------
struct U4 { uint32_t x, y, z, w; };

GC_HD void mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
#if defined(__CUDA_ARCH__)
  lo = a * b;
  hi = __umulhi(a, b);
#else
  uint64_t p = (uint64_t)a * (uint64_t)b;
  lo = (uint32_t)p;
  hi = (uint32_t)(p >> 32);
#endif
}

GC_HD U4 philox4x32_10(U4 c, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    mulhilo(0xD2511F53u, c.x, hi0, lo0);
    mulhilo(0xCD9E8D57u, c.z, hi1, lo1);
    U4 n;
    n.x = hi1 ^ c.y ^ k0;
    n.y = lo1;
    n.z = hi0 ^ c.w ^ k1;
    n.w = lo0;
    c = n;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c;
}

struct RngKey {
  uint32_t k0, k1;   // seed
  uint32_t step;     // advanced once per reduce() call
  uint32_t stream;   // (rank << 8) | purpose  -- rounding noise differs per rank, index sets do not
};

GC_HD U4 philox_block(const RngKey& k, uint64_t block) {
  U4 c;
  c.x = (uint32_t)block;
  c.y = (uint32_t)(block >> 32);
  c.z = k.step;
  c.w = k.stream;
  return philox4x32_10(c, k.k0, k.k1);
}

GC_HD float u01(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }   // [0, 1)

GC_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);   // never contracted into an FMA, so host and device agree bit for bit
#else
  return a * b;
#endif
}

// ---------------------------------------------------------------------------------------------
// Stochastic quantiser (QSGD with a supplied norm; reference maths: compressors.py:299-316).
// scale = s / norm (0 when norm == 0).  Returns the signed level in [-s, s].
// ---------------------------------------------------------------------------------------------
GC_HD int quantize_level(float g, float scale, int s, uint32_t rnd) {
  float a = fabsf(g);
  float l = mul_rn(a, scale);
  int xi;
  if (!(l < (float)s)) {
    xi = s;                    // also catches inf / nan inputs
  } else {
    float fl = floorf(l);
    float p = l - fl;
    xi = (int)fl + ((u01(rnd) < p) ? 1 : 0);
  }
  return (g < 0.0f) ? -xi : xi;
}

// Deterministic (biased) variant: truncation toward zero (compressors.py:562-568).
GC_HD int quantize_level_biased(float g, float scale, int s) {
  float l = mul_rn(fabsf(g), scale);
  int xi = (!(l < (float)s)) ? s : (int)floorf(l);
  return (g < 0.0f) ? -xi : xi;
}

// Non-uniform (power-of-two levels) quantiser (compressors.py:520-541).  scale = 2^b / norm.
// r < 1 rounds between 0 and 1; otherwise between 2^k and 2^(k+1), k = floor(log2 r).
GC_HD int quantize_level_nu(float g, float scale, int smax, uint32_t rnd, bool biased) {
  float r = mul_rn(fabsf(g), scale);
  int h;
  if (!(r < (float)smax)) {
    h = smax;
  } else if (r < 1.0f) {
    h = biased ? 0 : ((u01(rnd) < r) ? 1 : 0);
  } else {
    int e;
    (void)frexpf(r, &e);           // r = m * 2^e, m in [0.5, 1)  ->  floor(log2 r) = e - 1
    float lo = ldexpf(1.0f, e - 1);
    float p = (r - lo) / lo;        // (r - 2^k) / (2^(k+1) - 2^k)
    h = (int)lo;
    if (!biased && u01(rnd) < p) h *= 2;
  }
  return (g < 0.0f) ? -h : h;
}

GC_HD float dequant_scale(float norm, int s, int world) {
  return norm / ((float)s * (float)world);
}

// ---------------------------------------------------------------------------------------------
// Packed wire layout.  n is padded to a multiple of 128 (a "row": 32 lanes x 4 elements).
//   magnitudes: element e occupies bits [e*mw, (e+1)*mw) of a little-endian bit stream,
//               mw = container width in {1,2,4,8,16} = next power of two >= b
//   bit planes (signs, scale masks): element e = row*128 + 4*lane + j  ->  word row*4 + j, bit lane
// ---------------------------------------------------------------------------------------------
GC_HD int mag_width(int bits) {
  int w = 1;
  while (w < bits) w <<= 1;
  return w;
}
GC_HD int64_t pad128(int64_t n) { return (n + 127) / 128 * 128; }
GC_HD int64_t mag_bytes(int64_t n_pad, int mw) { return n_pad * mw / 8; }
GC_HD int64_t plane_bytes(int64_t n_pad) { return n_pad / 8; }
GC_HD int64_t plane_word(int64_t e) { return (e / 128) * 4 + (e & 3); }
GC_HD int plane_bit(int64_t e) { return (int)((e & 127) >> 2); }

// Smallest signed container (bytes) that holds a sum of `world` levels bounded by s.
GC_HD int sum_container_bytes(int s, int world) {
  int64_t m = (int64_t)s * world;
  return m <= 127 ? 1 : (m <= 32767 ? 2 : 4);
}

// Purposes (low byte of RngKey::stream)
enum : uint32_t {
  PURPOSE_ROUND = 1,       // rounding noise, single scale / lower scale
  PURPOSE_ROUND_HI = 2,    // rounding noise, higher scale of the two-scale codec
  PURPOSE_INDEX = 3,       // RandK index permutation (rank field = 0 on every rank)
  PURPOSE_QINIT = 4,       // PowerSGD query matrices (rank field = 0 on every rank)
  PURPOSE_LEVEL0 = 16,     // multi-scale: PURPOSE_LEVEL0 + level index
  PURPOSE_USER = 64,
};

// Status words written by kernels instead of trapping.
enum : int {
  STATUS_OK = 0,
  STATUS_TIMEOUT = 1,      // a bounded wait on a peer flag ran out
  STATUS_BOUNDS = 3,       // an index outside its tensor was met (and not followed); the first one is recorded next to the status
};

}  // namespace gc
