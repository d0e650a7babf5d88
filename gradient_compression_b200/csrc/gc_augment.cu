// Device-resident CIFAR input pipeline: the uint8 dataset (150 MB) lives in HBM; one kernel per step draws the
// batch (keyed permutation), applies random crop (padding 4) + horizontal flip + normalisation and writes the
// fp32 channels-last batch -- no DataLoader workers, no pinned staging, no H2D copy on the step's critical path.
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_augment.h"
#include "gc_perm.h"

using namespace gc;

namespace {

__global__ void __launch_bounds__(256) augment_kernel(const uint8_t* __restrict__ images, const int64_t* __restrict__ labels,
                                                      PermKey pk, uint64_t seed, uint32_t epoch, int64_t first_slot,
                                                      int64_t slot_stride, int batch, int train, int shuffle, float m0, float m1,
                                                      float m2, float s0, float s1, float s2, float* __restrict__ out,
                                                      int64_t* __restrict__ out_labels) {
  int b = blockIdx.x;
  if (b >= batch) return;
  uint64_t slot = (uint64_t)(first_slot + (int64_t)b * slot_stride);
  uint64_t src = shuffle ? perm_eval(pk, slot % pk.n) : slot % pk.n;
  AugmentDraw d = augment_draw(seed, epoch, slot);
  const uint8_t* img = images + src * 3072;
  const float mean[3] = {m0, m1, m2}, inv_std[3] = {s0, s1, s2};
  for (int i = threadIdx.x; i < 3072; i += blockDim.x) {
    int c = i % 3, x = (i / 3) % 32, y = i / 96;
    out[(int64_t)b * 3072 + i] = augment_pixel(img, d, y, x, c, mean[c], inv_std[c], train != 0);
  }
  if (threadIdx.x == 0) out_labels[b] = labels[src];
}

}  // namespace

extern "C" int gc_cuda_augment(const uint8_t* images, const int64_t* labels, int64_t n_images, uint64_t seed, uint32_t epoch,
                               int64_t first_slot, int64_t slot_stride, int batch, int train, int shuffle, const float* mean,
                               const float* inv_std, float* out, int64_t* out_labels, void* cs) {
  if (batch <= 0) return 0;
  PermKey pk = make_perm_key((uint64_t)n_images, seed, epoch);
  augment_kernel<<<batch, 256, 0, (cudaStream_t)cs>>>(images, labels, pk, seed, epoch, first_slot, slot_stride, batch, train,
                                                       shuffle, mean[0], mean[1], mean[2], inv_std[0], inv_std[1], inv_std[2],
                                                       out, out_labels);
  return (int)cudaGetLastError();
}
