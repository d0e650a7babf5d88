// Tiling of a 3x3, stride-1, padding-1 convolution on an NHWC fp32 activation as an implicit GEMM
//   Y[N*H*W, Cout] = sum over the 9 filter taps (r, s) and the input channels c of
//                    X[n, h + r - 1, w + s - 1, c] * Wt[Cout][r][s][c]
// for TMA: one output tile = 128 consecutive positions in (n, h, w) order = one 4-D box of the input per filter
// tap and 32-channel block, shifted by (s - 1, r - 1) in (w, h); positions outside the image are the box's
// out-of-range part, which TMA fills with zeros -- that is the padding.  The weight matrix is the channels-last
// filter tensor read as [Cout, 9 * Cin] (K index = tap * Cin + c), the reference's `nn.Conv2d(..., kernel_size=3,
// padding=1)` (models/resnet.py:52, models/vgg.py:104 of the reference) in the layout cuDNN also prefers.
// Shared by the kernel (producer warp) and by the host library (tests emulate the boxes with numpy).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define GC_GEOM_HD __host__ __device__ __forceinline__
#else
#define GC_GEOM_HD inline
#endif

namespace gc {

struct Conv3x3Geom {
  int N, H, W, C;            // input [N, H, W, C], C a multiple of 32
  int box_w, box_h, box_n;   // positions of one tile: box_n images x box_h rows x box_w columns = 128
  int cblocks;               // C / 32
  int tiles;                 // ceil(N * H * W / 128)
  int kblocks;               // 9 * cblocks
};

// 0 when the shape cannot be tiled this way: W must divide 128 (so W is a power of two <= 128) and an image must be
// a whole number of tiles or a tile a whole number of images.
GC_GEOM_HD int conv3x3_geom(int N, int H, int W, int C, Conv3x3Geom* g) {
  if (N < 1 || H < 1 || W < 1 || C < 32 || (C & 31)) return 0;
  if (W > 128 || (128 % W) != 0) return 0;
  const int hw = H * W;
  if (hw >= 128) {
    if (hw % 128) return 0;
    g->box_w = W; g->box_h = 128 / W; g->box_n = 1;
  } else {
    if (128 % hw) return 0;
    g->box_w = W; g->box_h = H; g->box_n = 128 / hw;
  }
  g->N = N; g->H = H; g->W = W; g->C = C;
  g->cblocks = C / 32;
  g->kblocks = 9 * g->cblocks;
  const int64_t positions = (int64_t)N * hw;
  g->tiles = (int)((positions + 127) / 128);
  return 1;
}

// TMA coordinates {c, w, h, n} of the input box of output tile `tile` and k-block `kb`.
GC_GEOM_HD void conv3x3_box(const Conv3x3Geom& g, int tile, int kb, int (&coord)[4]) {
  const int hw = g.H * g.W;
  const int64_t p0 = (int64_t)tile * 128;
  const int n0 = (int)(p0 / hw);
  const int h0 = (int)((p0 % hw) / g.W);       // 0 when a tile holds whole images
  const int tap = kb / g.cblocks;
  coord[0] = (kb % g.cblocks) * 32;
  coord[1] = tap % 3 - 1;
  coord[2] = h0 + tap / 3 - 1;
  coord[3] = n0;
}

}  // namespace gc
