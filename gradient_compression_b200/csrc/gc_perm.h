// Keyed pseudo-random permutation of [0, n) evaluated point-wise (no table, no memory):
// a 4-round balanced Feistel network over 2*h bits, h = ceil(log2(n) / 2), with cycle walking
// for values that land outside [0, n).  Every rank evaluates perm(position) for the K positions
// of the current step, so the RandK index set is identical on all ranks without any transfer
// (the reference builds a CPU randperm(N) and uploads K indices every step: reducer.py:717-723).
#pragma once
#include "gc_common.h"

namespace gc {

struct PermKey {
  uint64_t n;
  uint32_t half_bits;
  uint32_t half_mask;
  uint32_t rk[4];
};

GC_HD uint32_t perm_mix(uint32_t x, uint32_t k) {
  x ^= k;
  x *= 0x85EBCA6Bu;
  x ^= x >> 13;
  x *= 0xC2B2AE35u;
  x ^= x >> 16;
  x += k * 0x9E3779B9u;
  x ^= x >> 15;
  x *= 0x2C1B3C6Du;
  x ^= x >> 12;
  return x;
}

inline PermKey make_perm_key(uint64_t n, uint64_t seed, uint32_t pass) {
  PermKey k;
  k.n = n;
  uint32_t bits = 1;
  while (bits < 64 && (1ull << bits) < n) ++bits;
  k.half_bits = (bits + 1) / 2;
  if (k.half_bits < 1) k.half_bits = 1;
  k.half_mask = (k.half_bits >= 32) ? 0xFFFFFFFFu : ((1u << k.half_bits) - 1u);
  RngKey rk;
  rk.k0 = (uint32_t)seed;
  rk.k1 = (uint32_t)(seed >> 32);
  rk.step = pass;
  rk.stream = PURPOSE_INDEX;
  U4 r = philox_block(rk, 0);
  k.rk[0] = r.x; k.rk[1] = r.y; k.rk[2] = r.z; k.rk[3] = r.w;
  return k;
}

GC_HD uint64_t perm_eval(const PermKey& k, uint64_t pos) {
  uint64_t v = pos;
  // cycle walking terminates: the Feistel network is a bijection on [0, 2^(2h)) and pos < n
  for (int guard = 0; guard < 1024; ++guard) {
    uint32_t l = (uint32_t)(v >> k.half_bits) & k.half_mask;
    uint32_t r = (uint32_t)v & k.half_mask;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t f = perm_mix(r, k.rk[i]) & k.half_mask;
      uint32_t nl = r;
      r = l ^ f;
      l = nl;
    }
    v = ((uint64_t)l << k.half_bits) | (uint64_t)r;
    if (v < k.n) return v;
  }
  return pos;   // unreachable for a bijection; keeps the loop bounded on the device
}

}  // namespace gc
