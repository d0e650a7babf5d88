// GPU version of the greedy variable-width packer whose bit layout the reference's extensions define
// (extensions/Extension CPU/bitpacking.cpp:19-52; its "GPU" extension runs the same loop on the host with one
// device sync per element).  word = mode << 30 | payload; mode 0: 15 x 2 bit, 1: 7 x 4 bit, 2: 4 x 7 bit,
// 3: 3 x 8 bit, chosen greedily from the maximum of the next 15 / 7 / 4 / 3 values.
//
// The greedy scan is sequential (where a word starts depends on every earlier choice), but a word covers at
// most 15 values, so a chunk of 256 values can only be entered at 15 different offsets.  Parallel form:
//   1. step[i]   = how many values a word starting at i would take            (one thread per value)
//   2. chunk map = for each of the 15 entry offsets: exit offset + word count   (one thread per chunk x entry)
//   3. the same composition over groups of 256 chunks, a short serial scan over the groups, and the
//      expansion back to per-chunk entry offsets and word bases
//   4. every chunk emits its words from its now-known entry offset              (one thread per chunk)
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int VCHUNK = 256;
constexpr int VENTRY = 15;
constexpr int VGROUP = 256;

// Mode the greedy packer picks for a word that starts at i: the widest payload whose window fits.
__device__ __forceinline__ int mode_at(const int32_t* __restrict__ src, int64_t n, int64_t i) {
  int m4 = 0, m7 = 0, m15 = 0;       // maxima over the next 4 / 7 / 15 values (windows end at n)
  for (int j = 0; j < 15 && i + j < n; ++j) {
    int v = src[i + j];
    if (j < 4) m4 = v > m4 ? v : m4;
    if (j < 7) m7 = v > m7 ? v : m7;
    m15 = v > m15 ? v : m15;
  }
  if (m15 < 4) return 0;
  if (m7 < 16) return 1;
  if (m4 < 128) return 2;
  return 3;
}

__global__ void varpack_step_kernel(const int32_t* __restrict__ src, int64_t n, uint8_t* __restrict__ mode_out, int* __restrict__ bad) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int v = src[i];
    if (v < 0 || v > 255) atomicExch(bad, 1);
    mode_out[i] = (uint8_t)mode_at(src, n, i);
  }
}

__device__ __forceinline__ int count_of(int mode) { return mode == 0 ? 15 : (mode == 1 ? 7 : (mode == 2 ? 4 : 3)); }

// exit / words of chunk c for every entry offset e (entry position = c * VCHUNK + e).
__global__ void varpack_chunkmap_kernel(const uint8_t* __restrict__ mode, int64_t n, int64_t n_chunks, uint8_t* __restrict__ exit_off,
                                        uint16_t* __restrict__ words) {
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_chunks * VENTRY) return;
  int64_t c = t / VENTRY;
  int e = (int)(t % VENTRY);
  int64_t end = (c + 1) * VCHUNK;
  int64_t pos = c * VCHUNK + e;
  int w = 0;
  while (pos < end && pos < n) { pos += count_of(mode[pos]); ++w; }
  exit_off[t] = (uint8_t)(pos >= end ? (pos - end) : 0);
  words[t] = (uint16_t)w;
}

// Composition over one group of VGROUP chunks, for every entry offset into the group's first chunk.
__global__ void varpack_groupmap_kernel(const uint8_t* __restrict__ exit_off, const uint16_t* __restrict__ words, int64_t n_chunks,
                                        int64_t n_groups, uint8_t* __restrict__ g_exit, uint32_t* __restrict__ g_words) {
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_groups * VENTRY) return;
  int64_t g = t / VENTRY;
  int e = (int)(t % VENTRY);
  uint32_t w = 0;
  int64_t c1 = (g + 1) * VGROUP < n_chunks ? (g + 1) * VGROUP : n_chunks;
  for (int64_t c = g * VGROUP; c < c1; ++c) {
    w += words[c * VENTRY + e];
    e = exit_off[c * VENTRY + e];
  }
  g_exit[t] = (uint8_t)e;
  g_words[t] = w;
}

// Serial over groups (n / 65536 of them): entry offset and word base of every group, and the total.
__global__ void varpack_scan_kernel(const uint8_t* __restrict__ g_exit, const uint32_t* __restrict__ g_words, int64_t n_groups,
                                    uint8_t* __restrict__ g_entry, int64_t* __restrict__ g_base, int64_t* __restrict__ total) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int e = 0;
  int64_t base = 0;
  for (int64_t g = 0; g < n_groups; ++g) {
    g_entry[g] = (uint8_t)e;
    g_base[g] = base;
    base += g_words[g * VENTRY + e];
    e = g_exit[g * VENTRY + e];
  }
  *total = base;
}

__global__ void varpack_fill_kernel(const uint8_t* __restrict__ exit_off, const uint16_t* __restrict__ words, int64_t n_chunks,
                                    int64_t n_groups, const uint8_t* __restrict__ g_entry, const int64_t* __restrict__ g_base,
                                    uint8_t* __restrict__ c_entry, int64_t* __restrict__ c_base) {
  int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups) return;
  int e = g_entry[g];
  int64_t base = g_base[g];
  int64_t c1 = (g + 1) * VGROUP < n_chunks ? (g + 1) * VGROUP : n_chunks;
  for (int64_t c = g * VGROUP; c < c1; ++c) {
    c_entry[c] = (uint8_t)e;
    c_base[c] = base;
    base += words[c * VENTRY + e];
    e = exit_off[c * VENTRY + e];
  }
}

__global__ void varpack_emit_kernel(const int32_t* __restrict__ src, const uint8_t* __restrict__ mode, int64_t n, int64_t n_chunks,
                                    const uint8_t* __restrict__ c_entry, const int64_t* __restrict__ c_base, uint32_t* __restrict__ out) {
  int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_chunks) return;
  const int bits[4] = {2, 4, 7, 8};
  const int top[4] = {28, 26, 23, 22};
  int64_t end = (c + 1) * VCHUNK;
  int64_t pos = c * VCHUNK + c_entry[c];
  int64_t w = c_base[c];
  while (pos < end && pos < n) {
    int m = mode[pos];
    int cnt = count_of(m);
    uint32_t code = (uint32_t)m << 30;
    for (int j = 0; j < cnt && pos + j < n; ++j) code |= (uint32_t)src[pos + j] << (top[m] - j * bits[m]);
    out[w++] = code;
    pos += cnt;
  }
}

// Unpack: value counts per word -> caller's exclusive prefix sum -> every word writes its values.
__global__ void varunpack_count_kernel(const uint32_t* __restrict__ words, int64_t n_words, int64_t* __restrict__ counts) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) counts[i] = count_of((int)(words[i] >> 30));
}
__global__ void varunpack_emit_kernel(const uint32_t* __restrict__ words, int64_t n_words, const int64_t* __restrict__ offsets,
                                      int32_t* __restrict__ out) {
  const int bits[4] = {2, 4, 7, 8};
  const int top[4] = {28, 26, 23, 22};
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) {
    uint32_t code = words[i];
    int m = (int)(code >> 30);
    int cnt = count_of(m);
    int64_t o = offsets[i];
    for (int j = 0; j < cnt; ++j) out[o + j] = (int32_t)((code >> (top[m] - j * bits[m])) & ((1u << bits[m]) - 1u));
  }
}

// Fixed 8 x 8-bit -> int64 packing (extensions/Extension CPU BP/bytepacking.cpp:21-24): element j of a group goes
// to byte 7 - j; unpacking sign-extends every byte.
__global__ void bytepack_kernel(const int32_t* __restrict__ src, int64_t n, int64_t* __restrict__ out) {
  int64_t words = (n + 7) / 8;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += stride) {
    unsigned long long code = 0;
    for (int j = 0; j < 8 && w * 8 + j < n; ++j) code |= (unsigned long long)(src[w * 8 + j] & 0xff) << (8 * (7 - j));
    out[w] = (int64_t)code;
  }
}
__global__ void byteunpack_kernel(const int64_t* __restrict__ src, int64_t n_words, int32_t* __restrict__ out) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words; w += stride) {
    unsigned long long code = (unsigned long long)src[w];
#pragma unroll
    for (int j = 0; j < 8; ++j) out[w * 8 + j] = (int32_t)(int8_t)((code >> (8 * (7 - j))) & 0xff);
  }
}

inline int blocks_for(int64_t items, int threads) {
  int64_t b = (items + threads - 1) / threads;
  return (int)(b < 1 ? 1 : (b > 65535 * 16 ? 65535 * 16 : b));
}

}  // namespace

extern "C" {

// Bytes of workspace for n values.
int64_t gc_cuda_varpack_workspace_bytes(int64_t n) {
  int64_t chunks = (n + VCHUNK - 1) / VCHUNK, groups = (chunks + VGROUP - 1) / VGROUP;
  return n + chunks * VENTRY * 3 + groups * VENTRY * 5 + groups * 9 + chunks * 9 + 64 + 8 * 16;
}

// Phase 1: everything up to the word count.  ws layout is private; *total_dev (int64, device) receives the
// number of words, *bad_dev (int, device) is set when a value is outside [0, 255].
int gc_cuda_varpack_plan(const int32_t* src, int64_t n, uint8_t* ws, int64_t* total_dev, int* bad_dev, void* cs) {
  cudaStream_t st = (cudaStream_t)cs;
  int64_t chunks = (n + VCHUNK - 1) / VCHUNK, groups = (chunks + VGROUP - 1) / VGROUP;
  uint8_t* p = ws;
  auto take = [&](int64_t bytes) { uint8_t* r = p; p += (bytes + 15) / 16 * 16; return r; };
  uint8_t* mode = take(n);
  uint8_t* exit_off = take(chunks * VENTRY);
  uint16_t* words = (uint16_t*)take(chunks * VENTRY * 2);
  uint8_t* g_exit = take(groups * VENTRY);
  uint32_t* g_words = (uint32_t*)take(groups * VENTRY * 4);
  uint8_t* g_entry = take(groups);
  int64_t* g_base = (int64_t*)take(groups * 8);
  uint8_t* c_entry = take(chunks);
  int64_t* c_base = (int64_t*)take(chunks * 8);
  cudaMemsetAsync(bad_dev, 0, sizeof(int), st);
  varpack_step_kernel<<<blocks_for(n, 256) > 4096 ? 4096 : blocks_for(n, 256), 256, 0, st>>>(src, n, mode, bad_dev);
  varpack_chunkmap_kernel<<<blocks_for(chunks * VENTRY, 256), 256, 0, st>>>(mode, n, chunks, exit_off, words);
  varpack_groupmap_kernel<<<blocks_for(groups * VENTRY, 128), 128, 0, st>>>(exit_off, words, chunks, groups, g_exit, g_words);
  varpack_scan_kernel<<<1, 32, 0, st>>>(g_exit, g_words, groups, g_entry, g_base, total_dev);
  varpack_fill_kernel<<<blocks_for(groups, 128), 128, 0, st>>>(exit_off, words, chunks, groups, g_entry, g_base, c_entry, c_base);
  return (int)cudaGetLastError();
}

// Phase 2: emit the words (out holds *total_dev words); same ws as phase 1.
int gc_cuda_varpack_emit(const int32_t* src, int64_t n, uint8_t* ws, uint32_t* out, void* cs) {
  int64_t chunks = (n + VCHUNK - 1) / VCHUNK, groups = (chunks + VGROUP - 1) / VGROUP;
  uint8_t* p = ws;
  auto take = [&](int64_t bytes) { uint8_t* r = p; p += (bytes + 15) / 16 * 16; return r; };
  uint8_t* mode = take(n);
  take(chunks * VENTRY);
  take(chunks * VENTRY * 2);
  take(groups * VENTRY);
  take(groups * VENTRY * 4);
  take(groups);
  take(groups * 8);
  uint8_t* c_entry = take(chunks);
  int64_t* c_base = (int64_t*)take(chunks * 8);
  varpack_emit_kernel<<<blocks_for(chunks, 128), 128, 0, (cudaStream_t)cs>>>(src, mode, n, chunks, c_entry, c_base, out);
  return (int)cudaGetLastError();
}

int gc_cuda_bytepack(const int32_t* src, int64_t n, int64_t* out, void* cs) {
  if (n <= 0) return 0;
  int b = blocks_for((n + 7) / 8, 256);
  bytepack_kernel<<<b > 4096 ? 4096 : b, 256, 0, (cudaStream_t)cs>>>(src, n, out);
  return (int)cudaGetLastError();
}

int gc_cuda_byteunpack(const int64_t* src, int64_t n_words, int32_t* out, void* cs) {
  if (n_words <= 0) return 0;
  int b = blocks_for(n_words, 256);
  byteunpack_kernel<<<b > 4096 ? 4096 : b, 256, 0, (cudaStream_t)cs>>>(src, n_words, out);
  return (int)cudaGetLastError();
}

int gc_cuda_varunpack_counts(const uint32_t* words, int64_t n_words, int64_t* counts, void* cs) {
  if (n_words <= 0) return 0;
  int b = blocks_for(n_words, 256);
  varunpack_count_kernel<<<b > 4096 ? 4096 : b, 256, 0, (cudaStream_t)cs>>>(words, n_words, counts);
  return (int)cudaGetLastError();
}

int gc_cuda_varunpack_emit(const uint32_t* words, int64_t n_words, const int64_t* offsets, int32_t* out, void* cs) {
  if (n_words <= 0) return 0;
  int b = blocks_for(n_words, 256);
  varunpack_emit_kernel<<<b > 4096 ? 4096 : b, 256, 0, (cudaStream_t)cs>>>(words, n_words, offsets, out);
  return (int)cudaGetLastError();
}

}  // extern "C"
