// Building blocks of the tcgen05 kernels (TF32 GEMMs and implicit-GEMM convolutions): mbarrier / TMA / UMMA
// wrappers, shared-memory descriptors, and the two kernel templates that both the GEMM entry points
// (gc_gemm_tc.cu) and the convolution entry points (gc_conv_tc.cu) instantiate:
//
//   gemm_tf32_persistent_kernel  C[M, N] (=, +=) A[M, K] * B[N, K]^T (+ bias), K-major operands, one CTA per SM.
//                                A comes either from a 2-D map (plain GEMM, 1x1 convolution) or from a 4-D map over
//                                an NHWC activation, one shifted box per filter tap and 32-channel block (implicit
//                                GEMM of an R x S convolution, stride 1 or 2; the zero padding is the TMA's
//                                out-of-range fill).
//   gemm_tn_tf32_kernel          C[Mo, No] += A[P, Mo]^T * B[P, No], MN-major operands, split-K.  B comes either from
//                                a 2-D map or from shifted 4-D boxes of the activation (weight gradient of an R x S
//                                convolution: one filter tap per output tile).
//
// No clusters, no multicast: every CTA loads its own operands.  Every mbarrier wait is bounded; when one runs out
// the CTA sets *error_flag, abandons its tile, frees its TMEM and returns.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_device.cuh"

// Measurement knobs shared by every translation unit of the library (set through gc_cuda_gemm_tf32_config /
// gc_cuda_gemm_tn_config): forced tile width (0 = choose), CTAs per SM the split contraction aims at, fewest
// k-blocks (of 64 rows) a split may get.
namespace gctc {
inline int tile_choice = 0;
inline int tn_ctas_per_sm = 1;
inline int tn_min_kblocks = 4;
inline int wgrad_two_taps = 0;
inline int split_choice = 0;   // contraction splits of the persistent kernel: 0 = modelled, 1 = never, n = n where a product allows it
inline int tma_mode = 1;   // bit 0: prefetch the tensor maps at kernel start; bit 2: epilogue warps sleep between polls while a tile is being accumulated
}  // namespace gctc

namespace {

constexpr int BM = 128;
constexpr int BK = 32;                       // 32 fp32 = 128 bytes = one swizzle row
constexpr int UMMA_K = 8;                    // tf32
constexpr int TBK = 64;                      // contraction rows per stage of the split-K (MN-major) kernel: 8 KB TMA boxes
constexpr int GEMM_THREADS = 192;           // one-tile-per-CTA kernel: producer warp, MMA warp, four epilogue warps
// The persistent and the split-K kernels have TWO producer warps that take alternate stages of the ring.  One thread
// needs about 500 cycles per stage (a try_wait that succeeds at once ~170, arrive.expect_tx ~55, the first TMA
// instruction ~280, each further one ~130: measured on a B200 with clock64), which is 32 bytes per cycle for a 16 KB
// stage -- half of what the TMA unit of an SM sustains (about 62 B/cycle with 16 KB boxes).  Two issuing threads in
// different warps bring the ring up to the unit's rate.
constexpr int PRODUCER_WARPS = 2;
constexpr int MMA_WARP = PRODUCER_WARPS;     // warp that allocates TMEM and issues tcgen05.mma
constexpr int FIRST_EPI_WARP = PRODUCER_WARPS + 1;
constexpr int TN_THREADS = 32 * FIRST_EPI_WARP + 128;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // a wait gives up after two seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint32_t addr = smem_u32(bar);
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 63u) == 63u) {
      if (*abort_flag) return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) break;
    }
  }
  *abort_flag = 1;
  return false;
}

// The same wait for warps that have nothing to do for a long time (the epilogue warps during a tile's main loop): between
// polls they sleep, so that their polling does not take issue slots from the single threads that feed the TMA unit and
// the tensor core on the same SM sub-partitions.
__device__ __forceinline__ bool mbar_wait_idle(uint64_t* bar, uint32_t parity, volatile int* abort_flag, unsigned sleep_ns) {
  uint32_t addr = smem_u32(bar);
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((it & 15u) == 15u) {
      if (*abort_flag) return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) break;
    }
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Where the rows of an operand come from when it is an NHWC activation [N, H, W, C] read through a 4-D map
// {C, W, H, N} instead of a matrix: output position p = (n, ho, wo) and filter tap (r, s) read the pixel
// (n, ho * stride + r - pad, wo * stride + s - pad); `rows_per_box` consecutive output positions are one box
// (whole output rows of one image, or whole images), taps == 0 means "a plain 2-D matrix".  The map's element
// strides carry the convolution stride, so a box always starts at the first position's pixel.
struct ConvA {
  int taps;        // R * S, 0 = plain matrix
  int fs;          // S (filter width)
  int cblocks;     // C / 32: k-blocks per tap
  int hw_out;      // output positions per image
  int w_out;       // output width
  int stride, pad;
  // B operand given as a matrix W[K rows, taps * ldtap columns] whose N index is the contiguous one (an input gradient
  // reading the forward filter [Cout][R][S][Cin] in place: K = Cout, N = Cin): b_mn = 1.  The A-side tap (fr, fs) then
  // multiplies the filter tap (b_r0 + b_dr * fr, b_s0 + b_ds * fs) -- rotation by 180 degrees for a stride-1 input gradient,
  // every second tap for a parity class of a stride-2 one -- found at column ((r * b_fs + s) * b_ldtap + n).  b_mn = 2: the
  // map is the 3-D view {32 floats, K rows, columns / 32} of the same matrix (b_ldtap a multiple of 32) and one box loads
  // a whole stage of B.
  int b_mn, b_ldtap, b_fs, b_r0, b_dr, b_s0, b_ds;
};

// Where the rows of the OUTPUT go when it is not a matrix but a strided sub-grid of an NHWC tensor read through a 4-D map
// {C, W', H', N} (the input gradient of a stride-2 convolution: one launch per parity class of input pixels): row
// p = (n, i, j) of the result is stored at coordinates (column, j, i, n).  hw == 0: a plain 2-D matrix.
struct ConvC {
  int hw;          // rows per image (H' * W'), 0 = plain matrix
  int w;           // W'
};

// Batch-norm statistics finished inside the GEMM that produces the activation: every CTA keeps per-column sums and sums
// of squares of its tiles, adds them to `acc` ([2][N] doubles, zero on entry) with atomics when it is done, and the
// epilogue group that draws the last ticket turns the totals into mean / 1 / sqrt(var + eps) (`stats`, [2N] floats),
// updates the running statistics and leaves `acc` and `ticket` zeroed for the next launch.  Needs every CTA to stay on
// one column tile (the launcher makes the grid a multiple of the number of column tiles).  acc == NULL: off.
struct BnFin {
  double* acc;
  unsigned int* ticket;
  float* stats;
  float* running_mean;     // may be NULL
  float* running_var;
  float momentum, eps;
};

// What the host passes to ask for it: `scratch` holds the ticket (first 256 bytes) and the totals (2 * N doubles), is
// zeroed once when allocated (gc_cuda_bn_fin_scratch_bytes) and is left zeroed by every launch that uses it.
struct BnFinHost {
  void* scratch;
  float* stats;
  float* running_mean;
  float* running_var;
  float momentum, eps;
};

inline BnFin bn_fin_from_host(const void* host_args) {
  BnFin f{};
  if (host_args != nullptr) {
    const BnFinHost* h = static_cast<const BnFinHost*>(host_args);
    if (h->scratch != nullptr) {
      f.ticket = static_cast<unsigned int*>(h->scratch);
      f.acc = reinterpret_cast<double*>(static_cast<uint8_t*>(h->scratch) + 256);
      f.stats = h->stats;
      f.running_mean = h->running_mean;
      f.running_var = h->running_var;
      f.momentum = h->momentum;
      f.eps = h->eps;
    }
  }
  return f;
}

// TMA coordinates {c, w, h, n} of the box that holds output positions p0 .. of filter tap `tap`, channel block `cb`.
__device__ __forceinline__ void conv_box(const ConvA& ca, int64_t p0, int tap, int cb, int (&co)[4]) {
  const int n = (int)(p0 / ca.hw_out);
  const int rem = (int)(p0 - (int64_t)n * ca.hw_out);
  const int h0 = rem / ca.w_out, w0 = rem - h0 * ca.w_out;
  const int r = tap / ca.fs, s = tap - r * ca.fs;
  co[0] = cb * 32;
  co[1] = w0 * ca.stride + s - ca.pad;
  co[2] = h0 * ca.stride + r - ca.pad;
  co[3] = n;
}

// K-major operand tile in the canonical 128-byte-swizzled layout (rows of 128 B, groups of 8 rows = 1024 B).
__device__ __forceinline__ uint64_t make_smem_desc(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);      // start address, bits [0, 14)
  d |= (uint64_t)1 << 16;                                // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset: 8 rows * 128 B
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                                // layout type: SWIZZLE_128B
  return d;
}

// MN-major operand tile: chunks of 32 floats of the M / N dimension x `rows` K rows (128 bytes each), one after the other.
__device__ __forceinline__ uint64_t make_smem_desc_mn_rows(const void* tile, int rows) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);      // start address
  d |= (uint64_t)((rows * 128) >> 4) << 16;              // leading byte offset: next 32-float chunk of the M / N dimension
  d |= (uint64_t)(512 >> 4) << 32;                       // stride byte offset: next group of 4 K rows
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  d |= (uint64_t)1 << 61;                                // layout type: SWIZZLE_128B_BASE32B
  return d;
}

__device__ __forceinline__ uint64_t make_smem_desc_mn(const void* tile) { return make_smem_desc_mn_rows(tile, TBK); }

// kind::tf32, fp32 accumulate, both operands K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
  return (1u << 4)                 // C format: F32
         | (2u << 7)               // A format: TF32
         | (2u << 10)              // B format: TF32
         | ((uint32_t)(n >> 3) << 17)
         | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }


// ------------------------------------------------------------------------------------------------
// Persistent variant: one CTA per SM walks a strided list of output tiles.  The accumulator is double
// buffered in TMEM (2 x BN columns), so the MMA warp works on tile i + 1 while the epilogue warps drain
// tile i; the TMA loads run ahead across tile boundaries through the same ring of stages; two groups of
// four epilogue warps take alternate 32-column slabs, each group staging them in its own ring of dedicated
// buffers and waiting for a TMA store only when it needs that store's buffer back.  Tiles are ordered
// with the column tile fastest: CTAs that run at the same time share the rows of A in L2.
template <int BN>
struct PSmem {
  static constexpr int STAGES = (BN <= 64) ? 5 : ((BN <= 128) ? 4 : 3);
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN * BK * 4;               // a multiple of 1024 for BN >= 8
  static constexpr int NSLAB = 4;
  static constexpr int SLAB_BYTES = BM * 128;
  static constexpr int RING_BYTES = STAGES * (A_BYTES + B_BYTES);
  static constexpr int STAGING_OFF = RING_BYTES;
  static constexpr int BAR_OFF = STAGING_OFF + NSLAB * SLAB_BYTES;
  static constexpr int COLSUM_OFF = BAR_OFF + 256;
  static constexpr int TOTAL = 1024 /* alignment slack */ + COLSUM_OFF + 4 * BN * 2 * 4;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(BN == 64 || BN == 128 || BN == 256, "tile widths of the persistent kernel");
  static_assert(TOTAL <= 232448, "shared memory of one CTA");
};

// Named barrier of one epilogue group (ids 1 and 2; 0 is __syncthreads).
__device__ __forceinline__ void group_bar(int grp) {
  if (grp == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
  else asm volatile("bar.sync 2, 128;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

constexpr int EPI_GROUPS = 2;
constexpr int PERSISTENT_THREADS = 32 * FIRST_EPI_WARP + 128 * EPI_GROUPS;

template <int BN>
__global__ void __launch_bounds__(PERSISTENT_THREADS, 1)
gemm_tf32_persistent_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                            const __grid_constant__ CUtensorMap tma_c, const ConvA ca, const float* __restrict__ bias, int M, int N, int K,
                            int tiles_m, int tiles_n, int splits, int accumulate, float* __restrict__ col_partials,
                            int* __restrict__ error_flag, int tma_mode, const BnFin fin, const ConvC cc) {
  using S = PSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_tiles = base;
  uint8_t* b_tiles = base + S::STAGES * S::A_BYTES;
  uint8_t* staging = base + S::STAGING_OFF;
  uint64_t* full = reinterpret_cast<uint64_t*>(base + S::BAR_OFF);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_full = empty + S::STAGES;      // [2] MMA -> epilogue: accumulator complete
  uint64_t* acc_empty = acc_full + 2;          // [2] epilogue -> MMA: accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* colsum = reinterpret_cast<float*>(base + S::COLSUM_OFF);      // [4 row quarters][BN columns][2]
  __shared__ int abort_flag;
  __shared__ int epi_go[EPI_GROUPS];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k = (K + BK - 1) / BK;
  // work item = (output tile, split of the contraction); the splits of one tile are neighbours in the list, so they run
  // at the same time on different SMs and add their partial tiles in L2 (the host passes accumulate = 1 and a zeroed C)
  const int total_items = tiles_m * tiles_n * splits;
  const int kps = (num_k + splits - 1) / splits;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int g = 0; g < EPI_GROUPS; ++g) epi_go[g] = 1;
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128 * EPI_GROUPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above (barriers, TMEM) overlapped the tail of the previous kernel of the stream; its results are
  // needed from here on
  gc::pdl_wait();
  gc::pdl_launch_dependents();

  if (warp < PRODUCER_WARPS) {
    // producer warp p fills the stages it == p (mod PRODUCER_WARPS) of the ring
    if (lane == 0) {
      if (tma_mode & 1) { tma_prefetch_map(&tma_a); tma_prefetch_map(&tma_b); }
      uint32_t it = 0;                                        // k-blocks issued so far by all producers, over all tiles
      bool ok = true;
      for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
        const int tile = t / splits, sp = t - tile * splits;
        const int kbeg = sp * kps, kend = min(num_k, kbeg + kps);
        const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
        int box[4] = {0, 0, 0, 0};
        if (ca.taps != 0) conv_box(ca, (int64_t)m0, 0, 0, box);  // pixel of the tile's first position at tap (0, 0)
        int kk = kbeg;
        int cb = 0, fr = 0, fs = 0;                             // k-block = (filter tap (fr, fs), 32-channel block cb)
        if (ca.taps != 0) {
          const int tap = kk / ca.cblocks;
          cb = kk - tap * ca.cblocks;
          fr = tap / ca.fs;
          fs = tap - fr * ca.fs;
        }
        for (int k = kbeg; k < kend; ++k, ++it) {
          if ((int)(it % PRODUCER_WARPS) == warp) {
            const int s = (int)(it % S::STAGES);
            const uint32_t phase = (it / S::STAGES) & 1u;
            if (!mbar_wait(&empty[s], phase ^ 1u, &abort_flag)) { ok = false; break; }
            mbar_expect_tx(&full[s], (uint32_t)(S::A_BYTES + S::B_BYTES));
            if (ca.taps == 0)
              tma_load_2d(a_tiles + s * S::A_BYTES, &tma_a, kk * BK, m0, &full[s]);
            else
              tma_load_4d(a_tiles + s * S::A_BYTES, &tma_a, cb * 32, box[1] + fs, box[2] + fr, box[3], &full[s]);
            if (!ca.b_mn) {
              tma_load_2d(b_tiles + s * S::B_BYTES, &tma_b, kk * BK, n0, &full[s]);
            } else {
              // BN / 32 boxes of 32 N-floats x 32 K-rows: the filter read in place (no transposed copy)
              const int tapcol = ca.taps == 0 ? 0 : ((ca.b_r0 + ca.b_dr * fr) * ca.b_fs + (ca.b_s0 + ca.b_ds * fs)) * ca.b_ldtap;
              const int krow = (ca.taps == 0 ? kk : cb) * BK;
              if (ca.b_mn == 2) {
                // the matrix seen as {32 floats, K rows, N / 32 chunks}: one box brings all BN / 32 chunks of the stage
                tma_load_3d(b_tiles + s * S::B_BYTES, &tma_b, 0, krow, (tapcol + n0) >> 5, &full[s]);
              } else {
#pragma unroll
                for (int c = 0; c < BN / 32; ++c)
                  tma_load_2d(b_tiles + s * S::B_BYTES + c * (BK * 128), &tma_b, tapcol + n0 + c * 32, krow, &full[s]);
              }
            }
          }
          ++kk;
          if (++cb == ca.cblocks) {                             // (never true for a plain matrix: cblocks == 0)
            cb = 0;
            if (++fs == ca.fs) { fs = 0; ++fr; }
          }
        }
      }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN);
      uint32_t it = 0, lt = 0;                                // k-blocks consumed, tiles started
      bool ok = true;
      for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x, ++lt) {
        const int sp = t % splits;
        const int nk = min(num_k, (sp + 1) * kps) - sp * kps;
        const uint32_t buf = lt & 1u, aphase = (lt >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], aphase ^ 1u, &abort_flag)) break;      // first use of a buffer passes at once
        tc_fence_after();
        const uint32_t tmem_c = tmem_base + buf * (uint32_t)BN;
        for (int k = 0; k < nk; ++k, ++it) {
          const int s = (int)(it % S::STAGES);
          const uint32_t phase = (it / S::STAGES) & 1u;
          if (!mbar_wait(&full[s], phase, &abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(a_tiles + s * S::A_BYTES);
          if (!ca.b_mn) {
            const uint64_t bdesc = make_smem_desc(b_tiles + s * S::B_BYTES);
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk)
              umma_tf32(tmem_c, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (k | kk) != 0 ? 1u : 0u);
          } else {
            // B is MN-major: 4 KB chunks of 32 N-floats x 32 K-rows; 8 K-rows = 1024 bytes = 64 address units per MMA
            const uint64_t bdesc = make_smem_desc_mn_rows(b_tiles + s * S::B_BYTES, BK);
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk)
              umma_tf32(tmem_c, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 64), idesc | (1u << 16), (k | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // Two epilogue groups of four warps (TMEM lane quarters warp & 3); group g drains the 32-column slabs
    // g, g + 2, ... of every tile through its own half of the staging ring, with its own named barrier and its
    // own store-issuing thread, so the groups never wait for each other.
    const int ew = warp - FIRST_EPI_WARP;
    const int grp = ew >> 2;
    const int lg = warp & 3;
    const int r = lg * 32 + lane;                              // row of the tile this thread owns
    const int te = (ew & 3) * 32 + lane;                       // 0..127 inside the group
    const bool issuer = te == 0;                               // owns the group's bulk store groups
    constexpr int SLABS = BN / 32;
    constexpr int RING = S::NSLAB / EPI_GROUPS;                // staging buffers per group
    uint8_t* my_staging = staging + grp * (RING * S::SLAB_BYTES);
    float* my_colsum = colsum;                                 // [4 row quarters][BN][2]; a group only touches its slabs' columns
    uint32_t lt = 0, sc = 0;                                   // tiles drained, slabs staged by this group
    const bool fin_on = fin.acc != nullptr;
    const bool want_sums = col_partials != nullptr || fin_on;
    float run_a = 0.f, run_b = 0.f;                            // fin_on: this thread's column, summed over the CTA's tiles
    bool drained_all = true;
    for (int t = blockIdx.x; t < total_items; t += gridDim.x, ++lt) {
      const int tile = t / splits;
      const bool add_bias = bias != nullptr && t == tile * splits;      // the first split of a tile carries the bias
      const int mi = tile / tiles_n;
      const int m0 = mi * BM, n0 = (tile % tiles_n) * BN;
      const uint32_t buf = lt & 1u, aphase = (lt >> 1) & 1u;
      const bool got = (tma_mode & 4) ? mbar_wait_idle(&acc_full[buf], aphase, &abort_flag, 128u) : mbar_wait(&acc_full[buf], aphase, &abort_flag);
      // one thread decides for the group: the TMEM loads are warp-collective and the named barriers below
      // involve all four warps, so either every one of them drains this tile or none does
      if (issuer) epi_go[grp] = (got && abort_flag == 0) ? 1 : 0;
      group_bar(grp);
      if (!epi_go[grp]) { drained_all = false; break; }
      tc_fence_after();
      const uint32_t lane_base = tmem_base + ((uint32_t)(lg * 32) << 16) + buf * (uint32_t)BN;
      const bool full_rows = m0 + BM <= M;
#pragma unroll 1
      for (int sl = grp; sl < SLABS; sl += EPI_GROUPS, ++sc) {
        uint8_t* slab = my_staging + (sc % RING) * S::SLAB_BYTES;
        // the store that last read this buffer was committed RING groups ago
        if (issuer) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(RING - 1) : "memory");
        group_bar(grp);
        uint32_t ra[16], rb[16];
        tmem_ld16_nowait(lane_base + (uint32_t)(sl * 32), ra);
        tmem_ld16_nowait(lane_base + (uint32_t)(sl * 32 + 16), rb);
        tmem_ld_wait();
        if (sl + EPI_GROUPS >= SLABS) {                        // this thread has read its share of the accumulator
          tc_fence_before();
          mbar_arrive(&acc_empty[buf]);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t* src = c < 4 ? &ra[c * 4] : &rb[(c - 4) * 4];
          float4 o = make_float4(__uint_as_float(src[0]), __uint_as_float(src[1]), __uint_as_float(src[2]), __uint_as_float(src[3]));
          if (add_bias) {
            int col = n0 + sl * 32 + c * 4;
            o.x += col < N ? bias[col] : 0.f; o.y += col + 1 < N ? bias[col + 1] : 0.f;
            o.z += col + 2 < N ? bias[col + 2] : 0.f; o.w += col + 3 < N ? bias[col + 3] : 0.f;
          }
          *reinterpret_cast<float4*>(slab + r * 128 + ((c ^ (r & 7)) << 4)) = o;     // 128-byte swizzle of the store map
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        group_bar(grp);
        if (issuer) {
          if (n0 + sl * 32 < N) {
            if (cc.hw != 0) {                    // rows = pixels (n, i, j) of a strided sub-grid: 4-D store map
              const int img = m0 / cc.hw, rem = m0 - img * cc.hw;
              const int i0 = rem / cc.w, j0 = rem - i0 * cc.w;
              asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                           ::"l"(&tma_c), "r"(smem_u32(slab)), "r"(n0 + sl * 32), "r"(j0), "r"(i0), "r"(img)
                           : "memory");
            } else if (accumulate)               // C += tile: the add happens in L2, C is never read by the SM
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&tma_c), "r"(smem_u32(slab)), "r"(n0 + sl * 32), "r"(m0)
                           : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&tma_c), "r"(smem_u32(slab)), "r"(n0 + sl * 32), "r"(m0)
                           : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");              // one group per slab, empty ones included
        }
        if (want_sums) {
          // sum and sum of squares of 32 rows of one column, read back from the staged slab (a row of a slab is
          // one 128-byte line: conflict free); four independent chains each
          const int col = te & 31, quarter = te >> 5;
          const uint8_t* colbase = slab + (quarter * 32) * 128 + ((col & 3) << 2);
          const int chunk = col >> 2;
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
          if (full_rows) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float v0 = *reinterpret_cast<const float*>(colbase + (j + 0) * 128 + ((chunk ^ ((j + 0) & 7)) << 4));
              float v1 = *reinterpret_cast<const float*>(colbase + (j + 1) * 128 + ((chunk ^ ((j + 1) & 7)) << 4));
              float v2 = *reinterpret_cast<const float*>(colbase + (j + 2) * 128 + ((chunk ^ ((j + 2) & 7)) << 4));
              float v3 = *reinterpret_cast<const float*>(colbase + (j + 3) * 128 + ((chunk ^ ((j + 3) & 7)) << 4));
              s0 += v0; s1 += v1; s2 += v2; s3 += v3;
              q0 = fmaf(v0, v0, q0); q1 = fmaf(v1, v1, q1); q2 = fmaf(v2, v2, q2); q3 = fmaf(v3, v3, q3);
            }
          } else {
#pragma unroll 4
            for (int j = 0; j < 32; ++j) {
              float v = *reinterpret_cast<const float*>(colbase + j * 128 + ((chunk ^ (j & 7)) << 4));
              v = (m0 + quarter * 32 + j < M) ? v : 0.f;
              s0 += v;
              q0 = fmaf(v, v, q0);
            }
          }
          my_colsum[(quarter * BN + sl * 32 + col) * 2] = (s0 + s1) + (s2 + s3);
          my_colsum[(quarter * BN + sl * 32 + col) * 2 + 1] = (q0 + q1) + (q2 + q3);
        }
      }
      if (want_sums) {
        group_bar(grp);
        static_assert((SLABS / EPI_GROUPS) * 32 <= 128, "one column per thread and tile");
        for (int idx = te; idx < (SLABS / EPI_GROUPS) * 32; idx += 128) {       // the columns of this group's slabs
          const int c = (grp + EPI_GROUPS * (idx >> 5)) * 32 + (idx & 31);
          const int gc = n0 + c;
          if (gc < N) {
            float a = (my_colsum[c * 2] + my_colsum[(BN + c) * 2]) + (my_colsum[(2 * BN + c) * 2] + my_colsum[(3 * BN + c) * 2]);
            float b = (my_colsum[c * 2 + 1] + my_colsum[(BN + c) * 2 + 1]) + (my_colsum[(2 * BN + c) * 2 + 1] + my_colsum[(3 * BN + c) * 2 + 1]);
            if (fin_on) {
              run_a += a;
              run_b += b;
            } else {
              col_partials[((int64_t)mi * 2) * N + gc] = a;
              col_partials[((int64_t)mi * 2 + 1) * N + gc] = b;
            }
          }
        }
      }
    }
    if (fin_on && drained_all) {
      // this CTA's column sums -> the global totals; the group that draws the last of gridDim.x * EPI_GROUPS tickets
      // finds every contribution in place and finishes the statistics
      if (te < (SLABS / EPI_GROUPS) * 32) {
        const int c = (grp + EPI_GROUPS * (te >> 5)) * 32 + (te & 31);
        const int gc = (int)(blockIdx.x % (unsigned)tiles_n) * BN + c;
        if (gc < N) {
          atomicAdd(&fin.acc[gc], (double)run_a);
          atomicAdd(&fin.acc[N + gc], (double)run_b);
        }
      }
      __threadfence();
      group_bar(grp);
      if (issuer) epi_go[grp] = atomicAdd(fin.ticket, 1u) == gridDim.x * (unsigned)EPI_GROUPS - 1u ? 2 : 1;
      group_bar(grp);
      if (epi_go[grp] == 2) {
        __threadfence();
        const double inv_m = 1.0 / (double)M;
        for (int c = te; c < N; c += 128) {
          const double sum = __ldcg(&fin.acc[c]), sq = __ldcg(&fin.acc[N + c]);
          const double mean = sum * inv_m;
          double var = sq * inv_m - mean * mean;
          if (var < 0.0) var = 0.0;
          fin.stats[c] = (float)mean;
          fin.stats[N + c] = (float)(1.0 / sqrt(var + (double)fin.eps));
          if (fin.running_mean != nullptr) {
            const double unbiased = M > 1 ? var * (double)M / (double)(M - 1) : var;
            fin.running_mean[c] = (1.0f - fin.momentum) * fin.running_mean[c] + fin.momentum * (float)mean;
            fin.running_var[c] = (1.0f - fin.momentum) * fin.running_var[c] + fin.momentum * (float)unbiased;
          }
          fin.acc[c] = 0.0;
          fin.acc[N + c] = 0.0;
        }
        if (issuer) *fin.ticket = 0u;
      }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory outlives the stores
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag && error_flag != nullptr) atomicExch(error_flag, 1);
}

// ------------------------------------------------------------------------------------------------
// "TN" GEMM for weight gradients:  C[Mo, No] += A[P, Mo]^T * B[P, No], contraction over the rows P (the
// N*H*W positions of a 1x1 convolution: A = dY, B = X, C = dW).  Both operands are MN-major for the tensor
// core (the contraction index is the slow one in memory).  For 32-bit elements that takes the shared-memory
// layout "128-byte swizzle with 32-byte atoms": 32 consecutive output-dimension floats (128 B) of one
// position form a row, 32 positions a 4 KB chunk (one TMA box), and the chunks of a k-block lie one after the
// other.  In descriptor terms: leading byte offset = 4096
// (next 32 floats of the output dimension), stride byte offset = 512 (next group of 4 positions), one MMA
// (K = 8 positions) advances the start address by 1024 bytes.
// Split-K: CTA (tile, split) contracts its slice of positions and adds its 128 x BN partial result onto C
// with TMA reduce stores, so C must hold the value to add to (zeros for a plain product).
template <int BN>
struct TnSmem {
  static constexpr int STAGES = (BN <= 64) ? 4 : ((BN <= 128) ? 3 : 2);
  static constexpr int CHUNK_BYTES = TBK * 128;             // one TMA box: 32 floats of the output dimension x TBK rows
  static constexpr int A_BYTES = BM * TBK * 4;
  static constexpr int B_BYTES = BN * TBK * 4;
  static constexpr int RING_BYTES = STAGES * (A_BYTES + B_BYTES);
  static constexpr int NSLAB = 2;
  static constexpr int SLAB_BYTES = BM * 128;
  static constexpr int STAGING_OFF = RING_BYTES;
  static constexpr int BAR_OFF = STAGING_OFF + NSLAB * SLAB_BYTES;
  static constexpr int TOTAL = 1024 + BAR_OFF + 256;
  static constexpr int TMEM_COLS = BN == 192 ? 256 : BN;    // TMEM is allocated in powers of two
  static_assert(TOTAL <= 232448, "shared memory of one CTA");
};

__host__ __device__ constexpr uint32_t make_idesc_mn(int n) {
  return make_idesc(n) | (1u << 15) | (1u << 16);        // A and B are MN-major
}

template <int BN>
__global__ void __launch_bounds__(TN_THREADS, 1)
gemm_tn_tf32_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_c, const ConvA ca, int P, int Mo, int No, int tiles_n, int splits,
                    int kblocks_per_split, int* __restrict__ error_flag, int tma_mode, int box3d) {
  using S = TnSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_tiles = base;
  uint8_t* b_tiles = base + S::STAGES * S::A_BYTES;
  uint8_t* staging = base + S::STAGING_OFF;
  uint64_t* full = reinterpret_cast<uint64_t*>(base + S::BAR_OFF);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_ready = empty + S::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  __shared__ int abort_flag;
  __shared__ int epi_go;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x % splits;
  const int tile = blockIdx.x / splits;
  const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
  const int total_k = (P + TBK - 1) / TBK;
  const int k_begin = split * kblocks_per_split;
  const int k_end = k_begin + kblocks_per_split < total_k ? k_begin + kblocks_per_split : total_k;
  const int num_k = k_end > k_begin ? k_end - k_begin : 0;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    epi_go = 1;
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_ready, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (num_k > 0) {
    if (warp < PRODUCER_WARPS) {
      // a stage is BM / 32 + BN / 32 boxes of 32 floats x TBK rows; producer warp p fills the stages k == p (mod PRODUCER_WARPS)
      if (lane == 0) {
        if (tma_mode & 1) { tma_prefetch_map(&tma_a); tma_prefetch_map(&tma_b); }
        // weight gradient of an R x S convolution: column n of dW[Cout, taps * Cin] belongs to filter tap n / Cin, channel
        // n % Cin; a tile narrower than Cin stays inside one tap, a wider one (Cin = 64) covers several taps side by side.
        // Box c of a stage reads the pixels of its tap, shifted by (fr, fs), for the TBK output positions of the k-block.
        int co[4] = {0, 0, 0, 0};
        int box_ch[BN / 32], box_fr[BN / 32], box_fs[BN / 32];
        if (ca.taps != 0) {
          const int cin = ca.cblocks * 32;
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            const int n = n0 + c * 32, tap = n / cin;
            box_ch[c] = n - tap * cin;
            box_fr[c] = tap / ca.fs;
            box_fs[c] = tap - box_fr[c] * ca.fs;
          }
        }
        // boxes that lie wholly beyond the matrix (Mo < 128: the 64-channel layers; No < n0 + BN) are not loaded at all: the
        // rows and columns of the accumulator they feed are never stored
        int a_boxes = (Mo - m0 + 31) / 32, b_boxes = (No - n0 + 31) / 32;
        a_boxes = a_boxes < BM / 32 ? a_boxes : BM / 32;
        b_boxes = b_boxes < BN / 32 ? b_boxes : BN / 32;
        // box3d bit 0 / 1: the A / B map is the 3-D view {32 floats, rows, chunks} of the matrix and ONE box brings the whole
        // operand of a stage (chunks beyond the matrix arrive as zeros and count as bytes)
        const bool a3 = (box3d & 1) != 0, b3 = (box3d & 2) != 0 && ca.taps == 0;
        const uint32_t stage_tx = (uint32_t)((a3 ? BM / 32 : a_boxes) * S::CHUNK_BYTES + (b3 ? BN / 32 : b_boxes) * S::CHUNK_BYTES);
        for (int k = warp; k < num_k; k += PRODUCER_WARPS) {
          const int s = k % S::STAGES;
          const uint32_t phase = (uint32_t)(k / S::STAGES) & 1u;
          if (!mbar_wait(&empty[s], phase ^ 1u, &abort_flag)) break;
          mbar_expect_tx(&full[s], stage_tx);
          const int row0 = (k_begin + k) * TBK;
          if (a3) {
            tma_load_3d(a_tiles + s * S::A_BYTES, &tma_a, 0, row0, m0 >> 5, &full[s]);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 32; ++c)
              if (c < a_boxes) tma_load_2d(a_tiles + s * S::A_BYTES + c * S::CHUNK_BYTES, &tma_a, m0 + c * 32, row0, &full[s]);
          }
          if (b3) {
            tma_load_3d(b_tiles + s * S::B_BYTES, &tma_b, 0, row0, n0 >> 5, &full[s]);
          } else if (ca.taps == 0) {
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
              if (c < b_boxes) tma_load_2d(b_tiles + s * S::B_BYTES + c * S::CHUNK_BYTES, &tma_b, n0 + c * 32, row0, &full[s]);
          } else {
            conv_box(ca, (int64_t)row0, 0, 0, co);           // the k-block's first position at tap (0, 0)
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
              if (c < b_boxes)
                tma_load_4d(b_tiles + s * S::B_BYTES + c * S::CHUNK_BYTES, &tma_b, box_ch[c], co[1] + box_fs[c], co[2] + box_fr[c], co[3],
                            &full[s]);
          }
        }
      }
    } else if (warp == MMA_WARP) {
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc_mn(BN);
        bool ok = true;
        for (int k = 0; k < num_k; ++k) {
          const int s = k % S::STAGES;
          const uint32_t phase = (uint32_t)(k / S::STAGES) & 1u;
          if (!mbar_wait(&full[s], phase, &abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc_mn(a_tiles + s * S::A_BYTES);
          const uint64_t bdesc = make_smem_desc_mn(b_tiles + s * S::B_BYTES);
#pragma unroll
          for (int kk = 0; kk < TBK / UMMA_K; ++kk)    // 8 positions = 8 rows of 128 bytes = 1024 bytes = 64 address units
            umma_tf32(tmem_base, adesc + (uint64_t)(kk * 64), bdesc + (uint64_t)(kk * 64), idesc, (k | kk) != 0 ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(acc_ready);
      }
    } else {
      const int lg = warp & 3;
      const int r = lg * 32 + lane;
      const int te = (warp - FIRST_EPI_WARP) * 32 + lane;
      const bool issuer = te == 0;
      const bool got = (tma_mode & 4) ? mbar_wait_idle(acc_ready, 0u, &abort_flag, 128u) : mbar_wait(acc_ready, 0u, &abort_flag);
      if (issuer) epi_go = (got && abort_flag == 0) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (epi_go) {
        tc_fence_after();
        const uint32_t lane_base = tmem_base + ((uint32_t)(lg * 32) << 16);
        constexpr int SLABS = BN / 32;
#pragma unroll 1
        for (int sl = 0; sl < SLABS; ++sl) {
          uint8_t* slab = staging + (sl % S::NSLAB) * S::SLAB_BYTES;
          if (issuer) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(S::NSLAB - 1) : "memory");
          asm volatile("bar.sync 1, 128;" ::: "memory");
          uint32_t ra[16], rb[16];
          tmem_ld16_nowait(lane_base + (uint32_t)(sl * 32), ra);
          tmem_ld16_nowait(lane_base + (uint32_t)(sl * 32 + 16), rb);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t* src = c < 4 ? &ra[c * 4] : &rb[(c - 4) * 4];
            *reinterpret_cast<float4*>(slab + r * 128 + ((c ^ (r & 7)) << 4)) =
                make_float4(__uint_as_float(src[0]), __uint_as_float(src[1]), __uint_as_float(src[2]), __uint_as_float(src[3]));
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (issuer) {
            if (n0 + sl * 32 < No)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&tma_c), "r"(smem_u32(slab)), "r"(n0 + sl * 32), "r"(m0)
                           : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      }
      if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag && error_flag != nullptr) atomicExch(error_flag, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

// 2-D fp32 tensor [rows, cols] with row stride ld (elements); box = box_rows x 32 columns, 128-byte swizzle.
int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);

bool tma_store_ok(const float* C, int64_t ldc) { return (reinterpret_cast<uintptr_t>(C) & 15u) == 0 && (ldc & 3) == 0; }

int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}



// Row-major [P, D] fp32 matrix as an MN-major operand: box = 32 floats x 32 rows (4 KB), shared-memory layout
// "128-byte swizzle, 32-byte atoms" (the MN-major layout of 32-bit types).
int make_map_mn(CUtensorMap* map, const float* base, int64_t P, int64_t D, int64_t ld, int box_rows = TBK) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)P};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}



// The row-major matrix [K, D] (row stride ld floats, D and ld multiples of 32 for whole chunks) as the 3-D tensor
// {32 floats, K rows, D / 32 chunks}: a box of 32 x box_rows x chunks lands in shared memory chunk after chunk, each chunk
// box_rows rows of 128 bytes -- the MN-major operand layout -- with ONE copy instruction.
int make_map_mn3(CUtensorMap* map, const float* base, int64_t K, int64_t D, int64_t ld, int box_rows, int chunks) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[3] = {32, (cuuint64_t)K, (cuuint64_t)((D + 31) / 32)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4, 128};
  cuuint32_t box[3] = {32, (cuuint32_t)box_rows, (cuuint32_t)chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// Launch the persistent kernel on ready-made tensor maps (ca.taps == 0: ma is a 2-D map of A[M, K]).
template <int BN>
int launch_persistent_maps(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const ConvA& ca, const float* bias,
                           int M, int N, int K, int accumulate, float* col_partials, int* error_flag, cudaStream_t st,
                           const BnFin* fin = nullptr, const ConvC* cc = nullptr, int splits = 1) {
  using S = PSmem<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_persistent_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  if (splits < 1 || splits > (K + BK - 1) / BK) return (int)cudaErrorInvalidValue;
  // a split contraction adds partial tiles into C: the caller zeroed C (or wants C += ...), and nothing that needs the
  // finished values (column statistics) or a store map without a reduce form can ride along
  if (splits > 1 && (!accumulate || col_partials != nullptr || (fin != nullptr && fin->acc != nullptr) || cc != nullptr))
    return (int)cudaErrorInvalidValue;
  int64_t total = (int64_t)tiles_m * tiles_n * splits;
  int64_t grid = total < sm_count() ? total : sm_count();
  BnFin f{};
  if (fin != nullptr && fin->acc != nullptr) {
    if (col_partials != nullptr || tiles_n > grid) return (int)cudaErrorInvalidValue;
    grid = grid / tiles_n * tiles_n;             // every CTA stays on one column tile
    f = *fin;
  }
  gc::launch_pdl(gemm_tf32_persistent_kernel<BN>, dim3((unsigned)grid), dim3(PERSISTENT_THREADS), (size_t)S::TOTAL, st, ma, mb, mc, ca,
                 bias, M, N, K, tiles_m, tiles_n, splits, accumulate, col_partials, error_flag, gctc::tma_mode, f,
                 cc != nullptr ? *cc : ConvC{0, 0});
  return (int)cudaGetLastError();
}

// Launch the split-K TN kernel on ready-made tensor maps.  At most tn_ctas_per_sm CTAs per SM over all tiles, at least
// tn_min_kblocks k-blocks each so that the pipeline fills.  One CTA per SM measured 10-25 % faster than two on the
// 131072- and 32768-position weight gradients of ResNet-50 (fewer partial tiles to add, longer pipelines), equal below.
template <int BN>
int launch_tn_maps(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const ConvA& ca, int P, int Mo, int No,
                   int* error_flag, cudaStream_t st, int box3d = 0) {
  using S = TnSmem<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tn_tf32_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int tiles_m = (Mo + BM - 1) / BM, tiles_n = (No + BN - 1) / BN;
  int tiles = tiles_m * tiles_n;
  int total_k = (P + TBK - 1) / TBK;
  // never more CTAs than fit at once (one per SM at this shared-memory size): a second, nearly empty wave would double the
  // kernel's time (measured: 153 CTAs on 148 SMs ran 37 us with the SMs 62 % busy)
  int splits = gctc::tn_ctas_per_sm * sm_count() / tiles;
  if (splits > (total_k + gctc::tn_min_kblocks - 1) / gctc::tn_min_kblocks) splits = (total_k + gctc::tn_min_kblocks - 1) / gctc::tn_min_kblocks;
  if (splits < 1) splits = 1;
  int per = (total_k + splits - 1) / splits;
  splits = (total_k + per - 1) / per;
  gemm_tn_tf32_kernel<BN><<<(unsigned)(tiles * splits), TN_THREADS, S::TOTAL, st>>>(ma, mb, mc, ca, P, Mo, No, tiles_n, splits, per,
                                                                                     error_flag, gctc::tma_mode, box3d);
  return (int)cudaGetLastError();
}

// Tile width of the persistent kernel: the candidate with the lowest modelled time.  A tile costs the larger of
// its DRAM share (C written once, A read once per row of tiles) and its shared-memory fill (A and B per
// k-block), plus a fixed start-up; CTAs work through ceil(tiles / SMs) tiles one after the other.
int pick_bn_persistent(int M, int N, int K) {
  int sms = sm_count();
  int64_t mt = (M + BM - 1) / BM;
  const int cand[3] = {256, 128, 64};
  int best = 64;
  double best_t = 1e30;
  for (int i = 0; i < 3; ++i) {
    int bn = cand[i];
    if (bn == 256 && N <= 128) continue;
    if (bn == 128 && N <= 64) continue;
    int64_t nt = (N + bn - 1) / bn;
    int64_t waves = (mt * nt + sms - 1) / sms;
    double dram = (double)BM * bn * 4.0 + (double)BM * K * 4.0 / (double)nt;      // bytes per tile
    double fill = (double)(BM + bn) * K * 4.0;
    double t_tile = dram / 40.0;                                                    // ~40 B/ns of DRAM per SM
    if (fill / 110.0 > t_tile) t_tile = fill / 110.0;                               // ~110 B/ns from L2 into one SM
    double t = (double)waves * (t_tile + 300.0);
    if (t < best_t) { best_t = t; best = bn; }
  }
  return best;
}

// Modelled cycles of zeroing `elements` floats with a memset node, and of one more pass over them for column statistics.
inline double zero_cycles(int64_t elements) { return 3000.0 + (double)elements * 4.0 / 3000.0; }
inline double stats_pass_cycles(int64_t elements) { return 8000.0 + (double)elements * 4.0 / 2000.0; }

// Tile width and number of contraction splits for a product whose output may be built from partial tiles (no column
// statistics wanted, plain 2-D output).  Modelled cycles of the slowest CTA: a k-block costs the issuing thread about
// 200 cycles of waiting and committing plus the larger of four MMA issues and their tensor time (420 / 500 / 720 cycles
// for 64 / 128 / 256 columns, measured with clock64 inside the kernel), a work item about 2500 cycles of fill and
// drain.  extra_split_cycles: what a caller pays elsewhere when the product is split (zeroing C, a separate pass for the
// statistics).  Returns splits = 1 with pick_bn_persistent's width when splitting does not pay.
inline void plan_persistent(int M, int N, int K, double extra_split_cycles, int* bn_out, int* splits_out) {
  *bn_out = gctc::tile_choice ? gctc::tile_choice : pick_bn_persistent(M, N, K);
  *splits_out = 1;
  if (gctc::split_choice == 1) return;
  const int sms = sm_count();
  const int num_k = (K + BK - 1) / BK;
  const int64_t mt = (M + BM - 1) / BM;
  auto cycles = [&](int bn, int splits) {
    const double stage = bn == 64 ? 420.0 : (bn == 128 ? 500.0 : 720.0);
    const int64_t items = mt * ((N + bn - 1) / bn) * splits;
    const int64_t waves = (items + sms - 1) / sms;
    return (double)waves * ((double)((num_k + splits - 1) / splits) * stage + 2500.0) + (splits > 1 ? extra_split_cycles : 0.0);
  };
  double best = cycles(*bn_out, 1);
  const int cand[3] = {256, 128, 64};
  for (int i = 0; i < 3; ++i) {
    const int bn = cand[i];
    if ((bn == 256 && N <= 128) || (bn == 128 && N <= 64)) continue;
    if (gctc::tile_choice && bn != gctc::tile_choice) continue;
    for (int splits = 2; splits <= 16; ++splits) {
      const int per = (num_k + splits - 1) / splits;
      if (per < 6 || (splits - 1) * per >= num_k) continue;      // every split non-empty and long enough to fill the ring
      if (gctc::split_choice > 1 && splits != gctc::split_choice) continue;
      const double c = cycles(bn, splits);
      if (c < best * 0.93 || (gctc::split_choice > 1 && *splits_out == 1)) { best = c; *bn_out = bn; *splits_out = splits; }
    }
  }
}

}  // namespace
