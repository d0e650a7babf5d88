// CPU restatements ("oracles") of every device kernel plus the native host-side helpers
// (packers with the reference extensions' bit layouts, index generation, selection).  Plain C ABI
// so that Python binds it with ctypes and so that no libtorch / CUDA runtime is needed on the CPU.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#include "gc_common.h"
#include "gc_perm.h"

using namespace gc;

static RngKey make_key(uint64_t seed, uint32_t stream, uint32_t step) {
  RngKey k;
  k.k0 = (uint32_t)seed;
  k.k1 = (uint32_t)(seed >> 32);
  k.step = step;
  k.stream = stream;
  return k;
}

static inline uint32_t word_of(const U4& r, int lane) {
  return lane == 0 ? r.x : lane == 1 ? r.y : lane == 2 ? r.z : r.w;
}

extern "C" {

int gc_host_abi_version() { return 3; }

void gc_host_philox_u32(uint64_t seed, uint32_t stream, uint32_t step, int64_t n, uint32_t* out) {
  RngKey k = make_key(seed, stream, step);
  for (int64_t b = 0; b * 4 < n; ++b) {
    U4 r = philox_block(k, (uint64_t)b);
    for (int j = 0; j < 4 && b * 4 + j < n; ++j) out[b * 4 + j] = word_of(r, j);
  }
}

void gc_host_philox_uniform(uint64_t seed, uint32_t stream, uint32_t step, int64_t n, float* out) {
  RngKey k = make_key(seed, stream, step);
  for (int64_t b = 0; b * 4 < n; ++b) {
    U4 r = philox_block(k, (uint64_t)b);
    for (int j = 0; j < 4 && b * 4 + j < n; ++j) out[b * 4 + j] = u01(word_of(r, j));
  }
}

// Box-Muller on word pairs: (x,y) -> elements 0,1 ; (z,w) -> elements 2,3 of the block.
void gc_host_philox_normal(uint64_t seed, uint32_t stream, uint32_t step, int64_t n, float* out) {
  RngKey k = make_key(seed, stream, step);
  for (int64_t b = 0; b * 4 < n; ++b) {
    U4 r = philox_block(k, (uint64_t)b);
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
    for (int h = 0; h < 2; ++h) {
      float u1 = ((float)(w[2 * h] >> 8) + 1.0f) * (1.0f / 16777216.0f);
      float u2 = u01(w[2 * h + 1]);
      float rad = sqrtf(-2.0f * logf(u1));
      float ang = 6.283185307179586f * u2;
      float z[2] = {rad * cosf(ang), rad * sinf(ang)};
      for (int j = 0; j < 2; ++j) {
        int64_t e = b * 4 + 2 * h + j;
        if (e < n) out[e] = z[j];
      }
    }
  }
}

float gc_host_absmax(const float* x, int64_t n) {
  float m = 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    float a = fabsf(x[i]);
    if (std::isnan(a)) a = INFINITY;   // same rule as the device kernel: a poisoned gradient shows as +inf
    if (a > m) m = a;
  }
  return m;
}

// mode: 0 stochastic uniform, 1 biased uniform, 2 stochastic power-of-two, 3 biased power-of-two
void gc_host_quantize_levels(const float* x, int64_t n, float norm, int s, int mode, uint64_t seed,
                             uint32_t stream, uint32_t step, int32_t* out) {
  RngKey k = make_key(seed, stream, step);
  float scale = (norm > 0.0f) ? (float)s / norm : 0.0f;
  for (int64_t b = 0; b * 4 < n; ++b) {
    U4 r = (mode == 0 || mode == 2) ? philox_block(k, (uint64_t)b) : U4{0, 0, 0, 0};
    for (int j = 0; j < 4 && b * 4 + j < n; ++j) {
      int64_t e = b * 4 + j;
      uint32_t rnd = word_of(r, j);
      int q;
      switch (mode) {
        case 0: q = quantize_level(x[e], scale, s, rnd); break;
        case 1: q = quantize_level_biased(x[e], scale, s); break;
        case 2: q = quantize_level_nu(x[e], scale, s, rnd, false); break;
        default: q = quantize_level_nu(x[e], scale, s, rnd, true); break;
      }
      out[e] = q;
    }
  }
}

void gc_host_dequantize_levels(const int32_t* q, int64_t n, float norm, int s, int world, float* out) {
  float sc = dequant_scale(norm, s, world);
  for (int64_t i = 0; i < n; ++i) out[i] = mul_rn(sc, (float)q[i]);
}

// Packed wire layout (see gc_common.h).  levels: n signed ints with |q| < 2^mw.  mags must hold
// mag_bytes(pad128(n), mw) bytes, signs plane_bytes(pad128(n)) bytes; both are fully overwritten.
void gc_host_pack(const int32_t* q, int64_t n, int mw, uint8_t* mags, uint32_t* signs) {
  int64_t np = pad128(n);
  memset(mags, 0, (size_t)mag_bytes(np, mw));
  memset(signs, 0, (size_t)plane_bytes(np));
  for (int64_t e = 0; e < n; ++e) {
    uint32_t m = (uint32_t)(q[e] < 0 ? -q[e] : q[e]);
    if (mw == 16) {
      ((uint16_t*)mags)[e] = (uint16_t)m;
    } else if (mw == 8) {
      mags[e] = (uint8_t)m;
    } else {
      int per = 8 / mw;
      mags[e / per] |= (uint8_t)((m & ((1u << mw) - 1u)) << ((e % per) * mw));
    }
    if (q[e] < 0) signs[plane_word(e)] |= (1u << plane_bit(e));
  }
}

void gc_host_unpack(const uint8_t* mags, const uint32_t* signs, int64_t n, int mw, int32_t* q) {
  for (int64_t e = 0; e < n; ++e) {
    uint32_t m;
    if (mw == 16) m = ((const uint16_t*)mags)[e];
    else if (mw == 8) m = mags[e];
    else {
      int per = 8 / mw;
      m = (mags[e / per] >> ((e % per) * mw)) & ((1u << mw) - 1u);
    }
    bool neg = (signs[plane_word(e)] >> plane_bit(e)) & 1u;
    q[e] = neg ? -(int32_t)m : (int32_t)m;
  }
}

void gc_host_plane_pack(const uint8_t* bits, int64_t n, uint32_t* words) {
  memset(words, 0, (size_t)plane_bytes(pad128(n)));
  for (int64_t e = 0; e < n; ++e)
    if (bits[e]) words[plane_word(e)] |= (1u << plane_bit(e));
}

void gc_host_plane_unpack(const uint32_t* words, int64_t n, uint8_t* bits) {
  for (int64_t e = 0; e < n; ++e) bits[e] = (words[plane_word(e)] >> plane_bit(e)) & 1u;
}

// ---------------------------------------------------------------------------------------------
// Greedy variable-width packer with the bit layout of the reference's CPU/"GPU" extensions
// (extensions/Extension CPU/bitpacking.cpp:19-52): word = mode << 30 | payload;
//   mode 0: 15 x 2 bit at shifts 28..0   (next 15 values all < 4)
//   mode 1:  7 x 4 bit at shifts 26..2   (next 7 < 16)
//   mode 2:  4 x 7 bit at shifts 23..2   (next 4 < 128)
//   mode 3:  3 x 8 bit at shifts 22..6   (next 3 < 256)
// Values outside [0, 255] are rejected (return -1) instead of looping forever.
// Returns the number of 32-bit words written (out may be NULL to only count).
// ---------------------------------------------------------------------------------------------
static const int kCnt[4] = {15, 7, 4, 3};
static const int kBits[4] = {2, 4, 7, 8};
static const int kTop[4] = {28, 26, 23, 22};

int64_t gc_host_varpack(const int32_t* src, int64_t n, uint32_t* out) {
  for (int64_t i = 0; i < n; ++i)
    if (src[i] < 0 || src[i] > 255) return -1;
  int64_t ind = 0, words = 0;
  while (ind < n) {
    int mode = 3;
    for (int m = 0; m < 4; ++m) {
      int lim = 1 << kBits[m];
      bool ok = true;
      for (int j = 0; j < kCnt[m] && ind + j < n; ++j)
        if (src[ind + j] >= lim) { ok = false; break; }
      if (ok) { mode = m; break; }
    }
    uint32_t code = (uint32_t)mode << 30;
    for (int j = 0; j < kCnt[mode] && ind + j < n; ++j)
      code |= (uint32_t)src[ind + j] << (kTop[mode] - j * kBits[mode]);
    if (out) out[words] = code;
    ++words;
    ind += kCnt[mode];
  }
  return words;
}

// Emits the full count of every word (callers trim to the original length, as the reference's
// demo does).  Returns the number of values written (out may be NULL to only count).
int64_t gc_host_varunpack(const uint32_t* src, int64_t n_words, int32_t* out) {
  int64_t cnt = 0;
  for (int64_t w = 0; w < n_words; ++w) {
    uint32_t code = src[w];
    int mode = (int)(code >> 30);
    for (int j = 0; j < kCnt[mode]; ++j) {
      if (out) out[cnt] = (int32_t)((code >> (kTop[mode] - j * kBits[mode])) & ((1u << kBits[mode]) - 1u));
      ++cnt;
    }
  }
  return cnt;
}

// Fixed 8 x 8-bit -> one int64 (extensions/Extension CPU BP/bytepacking.cpp:21-24): element j of a
// group goes to byte 7-j after & 0xff.  out holds ceil(n/8) words.
void gc_host_bytepack(const int32_t* src, int64_t n, int64_t* out) {
  int64_t words = (n + 7) / 8;
  for (int64_t w = 0; w < words; ++w) {
    uint64_t code = 0;
    for (int j = 0; j < 8 && w * 8 + j < n; ++j)
      code |= ((uint64_t)(src[w * 8 + j] & 0xff)) << (8 * (7 - j));
    out[w] = (int64_t)code;
  }
}

// Each byte is returned sign-extended (int8 semantics), 8 values per word.
void gc_host_byteunpack(const int64_t* src, int64_t n_words, int32_t* out) {
  for (int64_t w = 0; w < n_words; ++w)
    for (int j = 0; j < 8; ++j)
      out[w * 8 + j] = (int32_t)(int8_t)(((uint64_t)src[w]) >> (8 * (7 - j)) & 0xff);
}

// RandK: indices perm(start), ..., perm(start + k - 1) of the keyed permutation of [0, n).
void gc_host_randk_indices(uint64_t seed, uint32_t pass, int64_t n, int64_t start, int64_t k, int64_t* out) {
  PermKey key = make_perm_key((uint64_t)n, seed, pass);
  for (int64_t i = 0; i < k; ++i) out[i] = (int64_t)perm_eval(key, (uint64_t)(start + i));
}

// Classical Gram-Schmidt, column by column, on a row-major n x r matrix (reducer.py:1847-1855):
// col /= ||col|| + eps; rest -= (col . rest) col.
void gc_host_gram_schmidt(float* p, int64_t n, int r, float eps) {
  for (int i = 0; i < r; ++i) {
    double ss = 0.0;
    for (int64_t row = 0; row < n; ++row) ss += (double)p[row * r + i] * p[row * r + i];
    float inv = 1.0f / ((float)std::sqrt(ss) + eps);
    for (int64_t row = 0; row < n; ++row) p[row * r + i] *= inv;
    for (int j = i + 1; j < r; ++j) {
      double dot = 0.0;
      for (int64_t row = 0; row < n; ++row) dot += (double)p[row * r + i] * p[row * r + j];
      float d = (float)dot;
      for (int64_t row = 0; row < n; ++row) p[row * r + j] -= d * p[row * r + i];
    }
  }
}

// Indices of the k largest |x| (ties broken toward the lower index); output sorted by index.
void gc_host_topk_abs(const float* x, int64_t n, int64_t k, int64_t* out) {
  std::vector<int64_t> idx((size_t)n);
  std::iota(idx.begin(), idx.end(), 0);
  auto cmp = [&](int64_t a, int64_t b) {
    float fa = fabsf(x[a]), fb = fabsf(x[b]);
    return fa > fb || (fa == fb && a < b);
  };
  if (k < n) std::nth_element(idx.begin(), idx.begin() + k, idx.end(), cmp);
  std::sort(idx.begin(), idx.begin() + k);
  for (int64_t i = 0; i < k; ++i) out[i] = idx[(size_t)i];
}

// SGD with momentum / Nesterov / weight decay on flat arrays (torch.optim.SGD semantics,
// dampening 0): d = g + wd p; m = mu m + d; d = nesterov ? d + mu m : m; p -= lr d.
void gc_host_sgd_step(float* p, const float* g, float* m, int64_t n, float lr, float mu, float wd, int nesterov) {
  for (int64_t i = 0; i < n; ++i) {
    float d = fmaf(wd, p[i], g[i]);
    float mi = fmaf(mu, m[i], d);
    m[i] = mi;
    float upd = nesterov ? fmaf(mu, mi, d) : mi;
    p[i] = fmaf(-lr, upd, p[i]);
  }
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Elias-omega coded QSGD stream (reference: compressors.py:52-149, there as Python strings).
// Bit string = 32 bits of the float `norm_over_s`, then per element one sign bit (1 = negative)
// followed by Elias-omega(|q| + 1); the string is cut into 62-bit payloads, each stored in an
// int64 under a leading 1 sentinel (the last word may be shorter).  Coding |q| + 1 makes zero
// representable (the reference codes 0 and 1 identically).
// ---------------------------------------------------------------------------------------------
namespace {
struct BitWriter {
  std::vector<int64_t>* out;
  uint64_t cur = 1;  // sentinel
  int nbits = 0;
  void put(int bit) {
    cur = (cur << 1) | (uint64_t)(bit & 1);
    if (++nbits == 62) flush();
  }
  void flush() {
    out->push_back((int64_t)cur);
    cur = 1;
    nbits = 0;
  }
  void finish() { out->push_back((int64_t)cur); }  // always emits a (possibly empty) tail word, as the reference does
};
void omega_put(BitWriter& w, uint32_t n) {  // n >= 1
  int groups[8];
  uint32_t vals[8];
  int ng = 0;
  while (n > 1) {
    int len = 32 - __builtin_clz(n);
    vals[ng] = n;
    groups[ng] = len;
    ++ng;
    n = (uint32_t)(len - 1);
  }
  for (int g = ng - 1; g >= 0; --g)
    for (int b = groups[g] - 1; b >= 0; --b) w.put((vals[g] >> b) & 1);
  w.put(0);
}
struct BitReader {
  const int64_t* src;
  int64_t n_words;
  int64_t word = 0;
  int pos = 0;   // bits consumed in the current word
  int avail = 0; // payload bits in the current word
  bool load() {
    while (word < n_words) {
      uint64_t v = (uint64_t)src[word];
      avail = 63 - __builtin_clzll(v);  // bits below the sentinel
      pos = 0;
      if (avail > 0) return true;
      ++word;
    }
    return false;
  }
  bool init() { return load(); }
  int get(bool& ok) {
    if (pos >= avail) {
      ++word;
      if (!load()) { ok = false; return 0; }
    }
    uint64_t v = (uint64_t)src[word];
    int bit = (int)((v >> (avail - 1 - pos)) & 1);
    ++pos;
    return bit;
  }
  bool done() {
    if (pos < avail) return false;
    int64_t w = word + 1;
    while (w < n_words) {
      uint64_t v = (uint64_t)src[w];
      if (63 - __builtin_clzll(v) > 0) return false;
      ++w;
    }
    return true;
  }
};
}  // namespace

extern "C" {

// Returns the number of int64 words; writes at most `cap` of them (call with cap = 0 to size).
int64_t gc_host_elias_encode(const int32_t* q, int64_t n, float norm_over_s, int64_t* out, int64_t cap) {
  std::vector<int64_t> words;
  words.reserve((size_t)(n / 8 + 4));
  BitWriter w;
  w.out = &words;
  uint32_t fb;
  memcpy(&fb, &norm_over_s, 4);
  for (int b = 31; b >= 0; --b) w.put((fb >> b) & 1);
  for (int64_t i = 0; i < n; ++i) {
    w.put(q[i] < 0 ? 1 : 0);
    omega_put(w, (uint32_t)(q[i] < 0 ? -q[i] : q[i]) + 1u);
  }
  w.finish();
  int64_t nw = (int64_t)words.size();
  for (int64_t i = 0; i < nw && i < cap; ++i) out[i] = words[(size_t)i];
  return nw;
}

// Decodes up to `cap` levels; returns how many the stream holds (-1 on a malformed stream).
int64_t gc_host_elias_decode(const int64_t* src, int64_t n_words, float* norm_over_s, int32_t* q, int64_t cap) {
  BitReader r;
  r.src = src;
  r.n_words = n_words;
  if (!r.init()) return -1;
  bool ok = true;
  uint32_t fb = 0;
  for (int b = 0; b < 32; ++b) fb = (fb << 1) | (uint32_t)r.get(ok);
  if (!ok) return -1;
  memcpy(norm_over_s, &fb, 4);
  int64_t cnt = 0;
  while (!r.done()) {
    int sign = r.get(ok);
    uint32_t n = 1;
    for (int guard = 0; guard < 8; ++guard) {
      int bit = r.get(ok);
      if (!ok) return -1;
      if (bit == 0) break;
      uint32_t m = 1;
      for (uint32_t j = 0; j < n; ++j) m = (m << 1) | (uint32_t)r.get(ok);
      if (!ok) return -1;
      n = m;
    }
    int32_t v = (int32_t)(n - 1);
    if (cnt < cap) q[cnt] = sign ? -v : v;
    ++cnt;
  }
  return cnt;
}

}  // extern "C"

#include "gc_augment.h"

extern "C" {

// out: [batch, 32, 32, 3] fp32 (NHWC); images: [n_images, 32, 32, 3] uint8; sample b of the batch is image
// perm(first_slot + b) of the keyed permutation of [0, n_images) (identity when shuffle == 0).
void gc_host_augment(const uint8_t* images, const int64_t* labels, int64_t n_images, uint64_t seed, uint32_t epoch,
                     int64_t first_slot, int64_t slot_stride, int batch, int train, int shuffle, const float* mean,
                     const float* inv_std, float* out, int64_t* out_labels) {
  PermKey pk = make_perm_key((uint64_t)n_images, seed, epoch);
  for (int b = 0; b < batch; ++b) {
    uint64_t slot = (uint64_t)(first_slot + (int64_t)b * slot_stride);
    uint64_t src = shuffle ? perm_eval(pk, slot % (uint64_t)n_images) : slot % (uint64_t)n_images;
    AugmentDraw d = augment_draw(seed, epoch, slot);
    const uint8_t* img = images + src * 3072;
    for (int y = 0; y < 32; ++y)
      for (int x = 0; x < 32; ++x)
        for (int c = 0; c < 3; ++c)
          out[(((int64_t)b * 32 + y) * 32 + x) * 3 + c] = augment_pixel(img, d, y, x, c, mean[c], inv_std[c], train != 0);
    out_labels[b] = labels[src];
  }
}

}  // extern "C"

#include "gc_conv_geom.h"

extern "C" {

// Geometry of the implicit-GEMM tiling of a 3x3 convolution (gc_conv_geom.h): out = {box_w, box_h, box_n, cblocks,
// tiles, kblocks}; returns 0 for shapes the tiling does not cover.
int gc_host_conv3x3_geom(int N, int H, int W, int C, int* out) {
  gc::Conv3x3Geom g;
  if (!gc::conv3x3_geom(N, H, W, C, &g)) return 0;
  out[0] = g.box_w; out[1] = g.box_h; out[2] = g.box_n; out[3] = g.cblocks; out[4] = g.tiles; out[5] = g.kblocks;
  return 1;
}

// Box coordinates {c, w, h, n} of (tile, k-block).
int gc_host_conv3x3_box(int N, int H, int W, int C, int tile, int kb, int* coord) {
  gc::Conv3x3Geom g;
  if (!gc::conv3x3_geom(N, H, W, C, &g) || tile < 0 || tile >= g.tiles || kb < 0 || kb >= g.kblocks) return 0;
  int c[4];
  gc::conv3x3_box(g, tile, kb, c);
  for (int i = 0; i < 4; ++i) coord[i] = c[i];
  return 1;
}

}  // extern "C"
