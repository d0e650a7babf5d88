// Convolutions of NHWC fp32 activations as implicit GEMMs on the 5th-generation tensor cores (tcgen05, kind::tf32,
// accumulator in TMEM), the layers the reference builds with nn.Conv2d (models/resnet.py:52,84 and models/vgg.py:104
// of the reference: 3x3 with padding 1 at stride 1 or 2, 1x1 at stride 2 in projection shortcuts).
//
//   forward / input gradient   Y[N*Ho*Wo, Cout] (=, +=) sum over taps (r, s), channels c of
//                              X[n, ho*stride + r - pad, wo*stride + s - pad, c] * Wt[Cout][r][s][c]  (+ bias)
//                              = gemm_tf32_persistent_kernel whose A operand is one shifted 4-D TMA box per filter tap
//                              and 32-channel block (k-block = tap * Cin/32 + channel block); pixels outside the image
//                              are the box's out-of-range part, which TMA fills with zeros: that is the padding.  The
//                              convolution stride is the map's element stride.  The weight matrix is the channels-last
//                              filter read as [Cout, R*S*Cin].  The input gradient of a stride-1 convolution is the same
//                              kernel on dY with the filter rotated by 180 degrees and its channel axes swapped.
//                              Batch-norm statistics and bias come from the GEMM epilogue as for the 1x1 case.
//   weight gradient            dW[Cout, R*S*Cin] += dY[P, Cout]^T * X_shifted[P, Cin] per tap = gemm_tn_tf32_kernel
//                              whose B operand is a shifted 4-D box of 64 output positions x 32 channels.
//   im2col_small_kernel        the 3-channel stem: its rows are 12 bytes apart, which no tensor map can describe,
//                              so the 27 taps of every position are gathered into rows of 32 floats once and the
//                              convolution becomes a plain GEMM with K = 32.
#include "gc_tc.cuh"

namespace {

struct Shape {
  int N, H, W, Cin, Cout, R, stride, pad, Ho, Wo;
};

bool make_shape(int N, int H, int W, int Cin, int Cout, int R, int stride, int pad, Shape* s) {
  if (N < 1 || H < 1 || W < 1 || Cin < 1 || Cout < 1 || R < 1 || R > 7 || stride < 1 || stride > 2 || pad < 0 || pad >= R) return false;
  if (H + 2 * pad < R || W + 2 * pad < R) return false;
  *s = Shape{N, H, W, Cin, Cout, R, stride, pad, (H + 2 * pad - R) / stride + 1, (W + 2 * pad - R) / stride + 1};
  return true;
}

// `rows` consecutive output positions in (n, ho, wo) order as one box of bw x bh x bn positions: part of an output
// row, whole output rows of one image, or whole images.
bool box_for(int rows, int Ho, int Wo, int* bw, int* bh, int* bn) {
  if (Wo >= rows) {
    if (Wo % rows) return false;
    *bw = rows; *bh = 1; *bn = 1;
    return true;
  }
  if (rows % Wo) return false;
  const int r = rows / Wo;
  if (Ho >= r) {
    if (Ho % r) return false;
    *bw = Wo; *bh = r; *bn = 1;
    return true;
  }
  if (r % Ho) return false;
  *bw = Wo; *bh = Ho; *bn = r / Ho;
  return true;
}

// 4-D map {C, W, H, N} of an NHWC activation; one box = 32 channels of bw x bh x bn output positions, read at the
// convolution's stride.  128-byte rows in shared memory, swizzled as the operand kind needs.
int make_map_nhwc(CUtensorMap* map, const float* base, const Shape& s, int bw, int bh, int bn, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)s.Cin, (cuuint64_t)s.W, (cuuint64_t)s.H, (cuuint64_t)s.N};
  cuuint64_t strides[3] = {(cuuint64_t)s.Cin * 4, (cuuint64_t)s.W * s.Cin * 4, (cuuint64_t)s.H * s.W * s.Cin * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)(bw * s.stride), (cuuint32_t)(bh * s.stride), (cuuint32_t)bn};
  cuuint32_t estr[4] = {1, (cuuint32_t)s.stride, (cuuint32_t)s.stride, 1};
  if (box[1] > 256 || box[2] > 256 || box[3] > 256) return -3;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

ConvA conv_a(const Shape& s) { return ConvA{s.R * s.R, s.R, s.Cin / 32, s.Ho * s.Wo, s.Wo, s.stride, s.pad}; }

bool fwd_ok(const Shape& s) {
  int bw, bh, bn;
  if ((s.Cin & 31) || (s.Cout & 3) || s.Cout < 32) return false;
  if ((int64_t)s.N * s.Ho * s.Wo > 0x7fffffff) return false;
  return box_for(BM, s.Ho, s.Wo, &bw, &bh, &bn) && encode_fn() != nullptr;
}

bool wgrad_ok(const Shape& s) {
  int bw, bh, bn;
  if ((s.Cin & 63) || (s.Cout & 31)) return false;
  return box_for(TBK, s.Ho, s.Wo, &bw, &bh, &bn) && encode_fn() != nullptr;
}

// A[p][k] = x[n, h + r - pad, w + s - pad, c] with k = (r * R + s) * Cin + c (zero outside the image and for
// k >= R*R*Cin), stride 1; wpad[co][k] = w[co][k] padded to Kp columns.  One thread per (position, 4 columns).
constexpr int IM2COL_MAX_KP = 128;

__global__ void __launch_bounds__(256) im2col_small_kernel(const float* __restrict__ x, float* __restrict__ A, int N, int H, int W,
                                                           int Cin, int R, int pad, int Kp, const float* __restrict__ w,
                                                           float* __restrict__ wpad, int Cout, int64_t quads) {
  const int K = R * R * Cin;
  const int qpr = Kp >> 2;
  // column k -> (row offset, column offset, channel) of its filter tap, once per block (no divisions per element); -1: padding
  __shared__ int tap_dh[IM2COL_MAX_KP], tap_dw[IM2COL_MAX_KP], tap_c[IM2COL_MAX_KP];
  for (int k = threadIdx.x; k < Kp; k += blockDim.x) {
    const int tap = k / Cin;
    tap_c[k] = k < K ? k - tap * Cin : -1;
    tap_dh[k] = tap / R - pad;
    tap_dw[k] = tap % R - pad;
  }
  __syncthreads();
  const uint32_t uq = (uint32_t)quads, uqpr = (uint32_t)qpr, uW = (uint32_t)W, uH = (uint32_t)H;      // host: quads < 2^31
  for (uint32_t q = blockIdx.x * blockDim.x + threadIdx.x; q < uq; q += gridDim.x * blockDim.x) {
    const uint32_t p = q / uqpr;
    const int k0 = (int)(q - p * uqpr) * 4;
    const uint32_t row = p / uW;
    const int wo = (int)(p - row * uW);
    const uint32_t n = row / uH;
    const int ho = (int)(row - n * uH);
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + j;
      const int c = tap_c[k], hi = ho + tap_dh[k], wi = wo + tap_dw[k];
      v[j] = (c >= 0 && hi >= 0 && hi < H && wi >= 0 && wi < W) ? x[(((int64_t)n * H + hi) * W + wi) * Cin + c] : 0.f;
    }
    *reinterpret_cast<float4*>(A + (int64_t)p * Kp + k0) = make_float4(v[0], v[1], v[2], v[3]);
  }
  if (wpad != nullptr) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < Cout * Kp; i += gridDim.x * blockDim.x) {
      const int co = i / Kp, k = i - co * Kp;
      wpad[i] = k < K ? w[co * K + k] : 0.f;
    }
  }
}

}  // namespace

extern "C" {

// 1 when forward (and, on rotated weights, the input gradient) of this convolution can run on the tensor cores:
// Cin a multiple of 32, Cout a multiple of 4 and >= 32, and 128 consecutive output positions form one box.
int gc_cuda_conv_fwd_supported(int N, int H, int W, int Cin, int Cout, int R, int stride, int pad) {
  Shape s;
  return make_shape(N, H, W, Cin, Cout, R, stride, pad, &s) && fwd_ok(s) ? 1 : 0;
}

// y[N*Ho*Wo, Cout] (=, += when accumulate) conv(x[N, H, W, Cin], w[Cout, R*R*Cin]) (+ bias[Cout]); x, w, y 16-byte aligned.
// col_partials (may be NULL): [ceil(N*Ho*Wo / 128)][2][Cout] per-tile column sums and sums of squares of y.
// bn_fin (may be NULL): a BnFinHost; the kernel then finishes the batch-norm statistics of y itself.
int gc_cuda_conv_fwd(const float* x, const float* w, float* y, const float* bias, int N, int H, int W, int Cin, int Cout, int R,
                     int stride, int pad, int accumulate, float* col_partials, int* error_flag, void* cs, const void* bn_fin) {
  Shape s;
  if (!make_shape(N, H, W, Cin, Cout, R, stride, pad, &s) || !fwd_ok(s)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(w) & 15u) || (reinterpret_cast<uintptr_t>(y) & 15u))
    return (int)cudaErrorInvalidValue;
  const int M = N * s.Ho * s.Wo, K = R * R * Cin;
  int bw, bh, bn;
  box_for(BM, s.Ho, s.Wo, &bw, &bh, &bn);
  cudaStream_t st = (cudaStream_t)cs;
  const BnFin fin_dev = bn_fin_from_host(bn_fin);
  const BnFin* fin = fin_dev.acc != nullptr ? &fin_dev : nullptr;
  int tile = gctc::tile_choice ? gctc::tile_choice : pick_bn_persistent(M, Cout, K), splits = 1;
  if (col_partials == nullptr && fin == nullptr)       // few output tiles and a long contraction: split it over the idle SMs
    plan_persistent(M, Cout, K, accumulate ? 0.0 : zero_cycles((int64_t)M * Cout), &tile, &splits);
  CUtensorMap ma, mb, mc;
  if (make_map_nhwc(&ma, x, s, bw, bh, bn, CU_TENSOR_MAP_SWIZZLE_128B) != 0 || make_map(&mb, w, Cout, K, K, tile) != 0 ||
      make_map(&mc, y, M, Cout, Cout, BM) != 0)
    return (int)cudaErrorInvalidValue;
  const ConvA ca = conv_a(s);
  if (splits > 1 && !accumulate) {
    cudaError_t e = cudaMemsetAsync(y, 0, (size_t)M * Cout * 4, st);
    if (e != cudaSuccess) return (int)e;
  }
  const int acc = (accumulate || splits > 1) ? 1 : 0;
  switch (tile) {
    case 64: return launch_persistent_maps<64>(ma, mb, mc, ca, bias, M, Cout, K, acc, col_partials, error_flag, st, fin, nullptr, splits);
    case 128: return launch_persistent_maps<128>(ma, mb, mc, ca, bias, M, Cout, K, acc, col_partials, error_flag, st, fin, nullptr, splits);
    case 256: return launch_persistent_maps<256>(ma, mb, mc, ca, bias, M, Cout, K, acc, col_partials, error_flag, st, fin, nullptr, splits);
    default: return (int)cudaErrorInvalidValue;
  }
}

// Contraction splits gc_cuda_conv_fwd would use for this shape if the caller gave up the in-kernel column statistics and
// computed them in a pass of its own over y (whose modelled cost is charged to the split plan).  1: keep the statistics in
// the kernel.
int gc_cuda_conv_fwd_splits(int N, int H, int W, int Cin, int Cout, int R, int stride, int pad) {
  Shape s;
  if (!make_shape(N, H, W, Cin, Cout, R, stride, pad, &s) || !fwd_ok(s)) return 1;
  const int M = N * s.Ho * s.Wo;
  int tile, splits;
  plan_persistent(M, Cout, R * R * Cin, zero_cycles((int64_t)M * Cout) + stats_pass_cycles((int64_t)M * Cout), &tile, &splits);
  return splits;
}

// Map of the forward filter w[Cout][R*R*Cin] as the MN-major B operand of an input-gradient launch with tiles of `tile`
// columns: one 3-D box per stage when every tap starts on a 32-float chunk (Cin a multiple of 32), else tile / 32 boxes.
static int filter_map(CUtensorMap* mb, ConvA* ca, const float* w, int Cout, int R, int Cin, int tile) {
  const int64_t cols = (int64_t)R * R * Cin;
  if ((Cin & 31) == 0 && make_map_mn3(mb, w, Cout, cols, cols, BK, tile / 32) == 0) {
    ca->b_mn = 2;
    return 0;
  }
  ca->b_mn = 1;
  return make_map_mn(mb, w, Cout, cols, cols, BK);
}

// 1 when the stride-1 input gradient of conv2d(x[N, H, W, Cin], w[Cout, R, R, Cin], pad) can run on the tensor cores reading
// the forward filter in place: Cout a multiple of 32 (the contraction), Cin a multiple of 4 and >= 32, and -- unless R = 1 with
// no padding, where dY is read as a plain matrix -- 128 consecutive input positions form one box of dY.
int gc_cuda_conv_dgrad_supported(int N, int H, int W, int Cin, int Cout, int R, int pad) {
  if (N < 1 || H < 1 || W < 1 || R < 1 || pad < 0 || pad > R - 1 || (Cout & 31) || (Cin & 3) || Cin < 32) return 0;
  if ((int64_t)N * H * W > 0x7fffffff || encode_fn() == nullptr) return 0;
  if (R == 1 && pad == 0) return 1;
  const int Ho = H + 2 * pad - R + 1, Wo = W + 2 * pad - R + 1;
  Shape s;
  return Ho >= 1 && Wo >= 1 && make_shape(N, Ho, Wo, Cout, Cin, R, 1, R - 1 - pad, &s) && s.Ho == H && s.Wo == W && fwd_ok(s) ? 1 : 0;
}

// dx[N, H, W, Cin] (=, += when accumulate) input gradient of the stride-1 convolution with filter w[Cout][R][R][Cin] (channels-last
// memory order) given dy[N, Ho, Wo, Cout]: the forward kernel run on dy with the filter taps rotated by 180 degrees, the filter read
// in place as the MN-major B operand (K = Cout rows of R*R*Cin floats; no transposed copy is kept).
int gc_cuda_conv_dgrad(const float* dy, const float* w, float* dx, int N, int H, int W, int Cin, int Cout, int R, int pad,
                       int accumulate, int* error_flag, void* cs) {
  if (!gc_cuda_conv_dgrad_supported(N, H, W, Cin, Cout, R, pad)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(dy) & 15u) || (reinterpret_cast<uintptr_t>(w) & 15u) || (reinterpret_cast<uintptr_t>(dx) & 15u))
    return (int)cudaErrorInvalidValue;
  const int M = N * H * W, K = R * R * Cout;
  cudaStream_t st = (cudaStream_t)cs;
  int tile, splits;
  plan_persistent(M, Cin, K, accumulate ? 0.0 : zero_cycles((int64_t)M * Cin), &tile, &splits);
  CUtensorMap ma, mb, mc;
  ConvA ca{};
  if (R == 1 && pad == 0) {
    if (make_map(&ma, dy, M, Cout, Cout, BM) != 0) return (int)cudaErrorInvalidValue;
  } else {
    Shape s;
    make_shape(N, H + 2 * pad - R + 1, W + 2 * pad - R + 1, Cout, Cin, R, 1, R - 1 - pad, &s);
    int bw, bh, bn;
    box_for(BM, s.Ho, s.Wo, &bw, &bh, &bn);
    if (make_map_nhwc(&ma, dy, s, bw, bh, bn, CU_TENSOR_MAP_SWIZZLE_128B) != 0) return (int)cudaErrorInvalidValue;
    ca = conv_a(s);
  }
  ca.b_ldtap = Cin; ca.b_fs = R;
  ca.b_r0 = R - 1; ca.b_dr = -1; ca.b_s0 = R - 1; ca.b_ds = -1;
  if (filter_map(&mb, &ca, w, Cout, R, Cin, tile) != 0 || make_map(&mc, dx, M, Cin, Cin, BM) != 0)
    return (int)cudaErrorInvalidValue;
  if (splits > 1 && !accumulate) {
    cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)M * Cin * 4, st);
    if (e != cudaSuccess) return (int)e;
  }
  const int acc = (accumulate || splits > 1) ? 1 : 0;
  switch (tile) {
    case 64: return launch_persistent_maps<64>(ma, mb, mc, ca, nullptr, M, Cin, K, acc, nullptr, error_flag, st, nullptr, nullptr, splits);
    case 128: return launch_persistent_maps<128>(ma, mb, mc, ca, nullptr, M, Cin, K, acc, nullptr, error_flag, st, nullptr, nullptr, splits);
    case 256: return launch_persistent_maps<256>(ma, mb, mc, ca, nullptr, M, Cin, K, acc, nullptr, error_flag, st, nullptr, nullptr, splits);
    default: return (int)cudaErrorInvalidValue;
  }
}

// For measurements: 1 = weight gradients at Cin = 128 use 256-column tiles that hold two filter taps (measured slower than
// one tap per 128-column tile: 35.8 vs 33.8 us at 16x16, 25.6 vs 21.5 us at 8x8 -- two 96 KB stages do not hide the loads).
void gc_cuda_conv_wgrad_two_taps(int on) { gctc::wgrad_two_taps = on ? 1 : 0; }

// 1 when the weight gradient of this convolution can run on the tensor cores: Cin a multiple of 64, Cout of 32, and
// 64 consecutive output positions form one box.
int gc_cuda_conv_wgrad_supported(int N, int H, int W, int Cin, int Cout, int R, int stride, int pad) {
  Shape s;
  return make_shape(N, H, W, Cin, Cout, R, stride, pad, &s) && wgrad_ok(s) ? 1 : 0;
}

// dw[Cout, R*R*Cin] += dy[N*Ho*Wo, Cout]^T x_shifted: zero dw first for a plain gradient (the split contraction adds its
// partial tiles with TMA reduce stores, in no fixed order).
int gc_cuda_conv_wgrad(const float* dy, const float* x, float* dw, int N, int H, int W, int Cin, int Cout, int R, int stride,
                       int pad, int* error_flag, void* cs) {
  Shape s;
  if (!make_shape(N, H, W, Cin, Cout, R, stride, pad, &s) || !wgrad_ok(s)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(dy) & 15u) || (reinterpret_cast<uintptr_t>(dw) & 15u))
    return (int)cudaErrorInvalidValue;
  const int P = N * s.Ho * s.Wo, No = R * R * Cin;
  int bw, bh, bn;
  box_for(TBK, s.Ho, s.Wo, &bw, &bh, &bn);
  // a tile's columns stay inside one filter tap, except at Cin = 64: there a tile of 192 columns holds three taps side by
  // side (64-column MMAs leave the issuing thread, not the tensor pipe, as the limit)
  int tile = (Cin % 256 == 0) ? 256 : ((Cin % 128 == 0) ? 128 : ((Cin == 64 && No % 192 == 0) ? 192 : 64));
  if (gctc::wgrad_two_taps && Cin == 128 && R > 1) tile = 256;            // two taps side by side: MMAs of 256 columns
  if (gctc::tile_choice && (Cin % gctc::tile_choice == 0 || (Cin == 64 && No % gctc::tile_choice == 0))) tile = gctc::tile_choice;
  CUtensorMap ma, mb, mc;
  int box3d = 0;        // dy as one 3-D box per stage where the driver accepts that view, else four 2-D boxes
  if (make_map_mn3(&ma, dy, P, Cout, Cout, TBK, BM / 32) == 0) box3d = 1;
  else if (make_map_mn(&ma, dy, P, Cout, Cout) != 0) return (int)cudaErrorInvalidValue;
  if (make_map_nhwc(&mb, x, s, bw, bh, bn, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B) != 0 ||
      make_map(&mc, dw, Cout, No, No, BM) != 0)
    return (int)cudaErrorInvalidValue;
  const ConvA ca = conv_a(s);
  cudaStream_t st = (cudaStream_t)cs;
  switch (tile) {
    case 64: return launch_tn_maps<64>(ma, mb, mc, ca, P, Cout, No, error_flag, st, box3d);
    case 128: return launch_tn_maps<128>(ma, mb, mc, ca, P, Cout, No, error_flag, st, box3d);
    case 192: return launch_tn_maps<192>(ma, mb, mc, ca, P, Cout, No, error_flag, st, box3d);
    case 256: return launch_tn_maps<256>(ma, mb, mc, ca, P, Cout, No, error_flag, st, box3d);
    default: return (int)cudaErrorInvalidValue;
  }
}

// Taps of a stride-2 convolution that reach input pixels of parity `par` along one axis: r = par + pad - 2 d for d = 0, 1, ...
// while 0 <= r < R.  Returns their count; the d-th tap reads the output gradient at offset +d.
static int class_taps(int par, int pad, int R) {
  int count = 0;
  for (int d = 0;; ++d) {
    const int r = par + pad - 2 * d;
    if (r < 0) break;
    if (r < R) ++count;
    else if (count == 0) continue;     // (r >= R before the first valid tap: keep looking at smaller r)
  }
  return count;
}

// The first offset d of that list (taps with r >= R are skipped from the front).
static int class_first(int par, int pad, int R) {
  for (int d = 0;; ++d) {
    const int r = par + pad - 2 * d;
    if (r < 0) return 0;
    if (r < R) return d;
  }
}

// 1 when the input gradient of this stride-2 convolution can run on the tensor cores: H and W even, Cout (the contraction)
// a multiple of 32, Cin a multiple of 4 and >= 32, 128 consecutive pixels of the half-resolution grid form one box, and
// every parity class starts its taps at offset 0 (true for R = 1, pad 0 and R = 3, pad 1).
int gc_cuda_conv_dgrad_s2_supported(int N, int H, int W, int Cin, int Cout, int R, int pad) {
  Shape s;
  if ((H & 1) || (W & 1) || !make_shape(N, H, W, Cin, Cout, R, 2, pad, &s) || s.Ho != H / 2 || s.Wo != W / 2) return 0;
  if ((Cout & 31) || (Cin & 3) || Cin < 32) return 0;
  for (int par = 0; par < 2; ++par)
    if (class_first(par, pad, R) != 0) return 0;
  int bw, bh, bn;
  return box_for(BM, s.Ho, s.Wo, &bw, &bh, &bn) && encode_fn() != nullptr ? 1 : 0;
}

// dx[N, H, W, Cin] = input gradient of conv2d(x, w, stride 2, pad) given dy[N, H/2, W/2, Cout].  One launch per parity class
// (ph, pw) of input pixels: the pixels (2i + ph, 2j + pw) receive a stride-1 convolution of dy with the filter taps
// r = ph + pad - 2 fr, s = pw + pad - 2 fs (fr, fs = 0, 1, ...: the offsets at which dy is read), and are written through a 4-D
// store map over that strided sub-grid of dx.  w: the forward filter [Cout][R][R][Cin] (channels-last memory order), read in
// place as the MN-major B operand.  Classes without taps (a 1x1 filter reaches only the even pixels) are zero: dx is cleared
// first when there is one.
int gc_cuda_conv_dgrad_s2(const float* dy, const float* w, float* dx, int N, int H, int W, int Cin, int Cout, int R, int pad,
                          int* error_flag, void* cs) {
  if (!gc_cuda_conv_dgrad_s2_supported(N, H, W, Cin, Cout, R, pad)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(dy) & 15u) || (reinterpret_cast<uintptr_t>(w) & 15u) || (reinterpret_cast<uintptr_t>(dx) & 15u))
    return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)cs;
  const int Ho = H / 2, Wo = W / 2, M = N * Ho * Wo;
  bool any_empty = false;
  for (int c = 0; c < 4; ++c) any_empty |= class_taps(c >> 1, pad, R) * class_taps(c & 1, pad, R) == 0;
  if (any_empty) {
    cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)N * H * W * Cin * 4, st);
    if (e != cudaSuccess) return (int)e;
  }
  Shape sy{N, Ho, Wo, Cout, Cin, 1, 1, 0, Ho, Wo};          // the class problem reads dy at stride 1, no padding
  int bw, bh, bn;
  box_for(BM, Ho, Wo, &bw, &bh, &bn);
  EncodeTiledFn fn = encode_fn();
  for (int c = 0; c < 4; ++c) {
    const int ph = c >> 1, pw = c & 1;
    const int th = class_taps(ph, pad, R), tw = class_taps(pw, pad, R);
    if (th * tw == 0) continue;
    const int K = th * tw * Cout;
    const int tile = gctc::tile_choice ? gctc::tile_choice : pick_bn_persistent(M, Cin, K);
    CUtensorMap ma, mb, mc;
    ConvA ca{th * tw, tw, Cout / 32, Ho * Wo, Wo, 1, 0};
    ca.b_ldtap = Cin; ca.b_fs = R;
    ca.b_r0 = ph + pad; ca.b_dr = -2; ca.b_s0 = pw + pad; ca.b_ds = -2;
    if (make_map_nhwc(&ma, dy, sy, bw, bh, bn, CU_TENSOR_MAP_SWIZZLE_128B) != 0 || filter_map(&mb, &ca, w, Cout, R, Cin, tile) != 0)
      return (int)cudaErrorInvalidValue;
    {   // pixels (2i + ph, 2j + pw) of dx as the 4-D tensor {Cin, W/2, H/2, N}
      cuuint64_t dims[4] = {(cuuint64_t)Cin, (cuuint64_t)Wo, (cuuint64_t)Ho, (cuuint64_t)N};
      cuuint64_t strides[3] = {(cuuint64_t)2 * Cin * 4, (cuuint64_t)2 * W * Cin * 4, (cuuint64_t)H * W * Cin * 4};
      cuuint32_t box[4] = {32, (cuuint32_t)bw, (cuuint32_t)bh, (cuuint32_t)bn};
      cuuint32_t estr[4] = {1, 1, 1, 1};
      if (fn(&mc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)(dx + ((int64_t)ph * W + pw) * Cin), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return (int)cudaErrorInvalidValue;
    }
    const ConvC cc{Ho * Wo, Wo};
    int err;
    switch (tile) {
      case 64: err = launch_persistent_maps<64>(ma, mb, mc, ca, nullptr, M, Cin, K, 0, nullptr, error_flag, st, nullptr, &cc); break;
      case 128: err = launch_persistent_maps<128>(ma, mb, mc, ca, nullptr, M, Cin, K, 0, nullptr, error_flag, st, nullptr, &cc); break;
      case 256: err = launch_persistent_maps<256>(ma, mb, mc, ca, nullptr, M, Cin, K, 0, nullptr, error_flag, st, nullptr, &cc); break;
      default: err = (int)cudaErrorInvalidValue;
    }
    if (err != 0) return err;
  }
  return 0;
}

// Rows of Kp = 32-float-padded filter taps for a stride-1 convolution with few input channels (the 3-channel stem):
// A[N*H*W, Kp] from x[N, H, W, Cin], and (when wpad is given) the filter w[Cout, R*R*Cin] padded to wpad[Cout, Kp].
int gc_cuda_im2col_small(const float* x, float* A, int N, int H, int W, int Cin, int R, int pad, int Kp, const float* w,
                         float* wpad, int Cout, void* cs) {
  if (N < 1 || H < 1 || W < 1 || Cin < 1 || R < 1 || pad < 0 || Kp < R * R * Cin || (Kp & 3) || 2 * pad != R - 1) return (int)cudaErrorInvalidValue;
  const int64_t quads = (int64_t)N * H * W * (Kp >> 2);
  if (Kp > IM2COL_MAX_KP || quads > 0x7fffffff) return (int)cudaErrorInvalidValue;
  int64_t blocks = (quads + 255) / 256;
  if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
  im2col_small_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)cs>>>(x, A, N, H, W, Cin, R, pad, Kp, w, wpad, Cout, quads);
  return (int)cudaGetLastError();
}

}  // extern "C"
