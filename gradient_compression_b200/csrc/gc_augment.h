// CIFAR training augmentation shared by the host oracle and the device kernel (reference transforms:
// RandomCrop(32, padding=4) + RandomHorizontalFlip + ToTensor + Normalize, model_dispatcher.py:37-44).
// One Philox block per sample decides the crop offset (dx, dy in [0, 8]) and the flip; the sample index comes
// from the same keyed permutation the Rand-K reducers use, so an epoch visits every image once per rank set.
#pragma once
#include "gc_common.h"

namespace gc {

struct AugmentDraw { int dx, dy, flip; };

GC_HD AugmentDraw augment_draw(uint64_t seed, uint32_t epoch, uint64_t sample_slot) {
  RngKey k;
  k.k0 = (uint32_t)seed;
  k.k1 = (uint32_t)(seed >> 32);
  k.step = epoch;
  k.stream = PURPOSE_USER + 1;
  U4 r = philox_block(k, sample_slot);
  AugmentDraw d;
  d.dx = (int)(r.x % 9u);
  d.dy = (int)(r.y % 9u);
  d.flip = (int)(r.z & 1u);
  return d;
}

// Output pixel (y, x, c) of a sample: source pixel of the zero-padded (4 on every side) image after crop and flip.
GC_HD float augment_pixel(const uint8_t* img /* 32x32x3, HWC */, const AugmentDraw& d, int y, int x, int c, float mean, float inv_std,
                          bool train) {
  int sx = train ? (d.flip ? 31 - x : x) + d.dx - 4 : x;
  int sy = train ? y + d.dy - 4 : y;
  float v = 0.0f;
  if (sx >= 0 && sx < 32 && sy >= 0 && sy < 32) v = (float)img[(sy * 32 + sx) * 3 + c] * (1.0f / 255.0f);
  return (v - mean) * inv_std;
}

}  // namespace gc
