// TF32 GEMMs on the 5th-generation tensor cores, fp32 in memory, kind::tf32 in the MMA (the tensor core reads
// the upper 19 bits of every fp32 word -- the same precision cuDNN uses for the reference's convolutions).
//
//   gemm_tf32_persistent_kernel  C[M, N] (=, +=) A[M, K] * B[N, K]^T (+ bias): both operands K-major.  1x1 convolutions
//                                on channels-last activations (A = activations [N*H*W, Cin], B = weight [Cout, Cin]) and
//                                their input gradients; optional per-column sums of C (batch-norm statistics) from the
//                                epilogue.  One CTA per SM walks the tiles with a double-buffered TMEM accumulator.
//   gemm_tf32_kernel             the same product with one CTA per 128 x BN tile: narrow outputs (N <= 16) and outputs that
//                                do not meet the TMA store rules (plain-store epilogue).
//   gemm_tn_tf32_kernel          C[Mo, No] += A[P, Mo]^T * B[P, No]: both operands MN-major, split-K.  Weight gradients.
//
// Common structure, no clusters, no multicast:
//   warp 0   TMA producer: cp.async.bulk.tensor.2d (128-byte swizzle) into a ring of shared-memory stages
//   warp 1   allocates TMEM, issues tcgen05.mma (one elected thread), commits stages back to the producer
//   warps 2+ epilogue: tcgen05.ld of the fp32 accumulator from TMEM, bias add, 32-column slabs staged in shared
//            memory (128-byte swizzled, bank-conflict free) and written with TMA stores / TMA reduce stores
// Every mbarrier wait is bounded; when one runs out the CTA sets *error_flag, abandons its tile, frees
// its TMEM and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_device.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 32;                       // 32 fp32 = 128 bytes = one swizzle row
constexpr int UMMA_K = 8;                    // tf32
constexpr int GEMM_THREADS = 192;
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

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
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

template <int BN>
struct Smem {
  // ring depth chosen so that two CTAs fit on one SM (<= ~100 KB each): while one CTA drains its accumulator
  // through the epilogue, the other one's TMA loads and MMAs keep the SM busy
  static constexpr int STAGES = (BN <= 16) ? 5 : ((BN <= 64) ? 4 : ((BN <= 128) ? 3 : 2));
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int B_STRIDE = (B_BYTES + 1023) / 1024 * 1024;     // every stage starts 1024-byte aligned
  static constexpr int TILE_BYTES = STAGES * (A_BYTES + B_STRIDE);
  static constexpr int TOTAL = TILE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + 1024 /* column sums */;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
};

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 2)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, int use_tma_store,
                 float* __restrict__ C, const float* __restrict__ bias, int M, int N, int K, int64_t ldc,
                 float* __restrict__ col_partials, int* __restrict__ error_flag) {
  using S = Smem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_tiles = tiles;
  uint8_t* b_tiles = tiles + S::STAGES * S::A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + S::TILE_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_ready = empty + S::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  float* colsum = reinterpret_cast<float*>(tiles + S::TILE_BYTES + 256);      // [4 row quarters][32 columns][2]
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int num_k = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_ready, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int k = 0; k < num_k; ++k) {
        int s = k % S::STAGES;
        uint32_t phase = (uint32_t)(k / S::STAGES) & 1u;
        if (!mbar_wait(&empty[s], phase ^ 1u, &abort_flag)) break;
        mbar_expect_tx(&full[s], (uint32_t)(S::A_BYTES + S::B_BYTES));
        tma_load_2d(a_tiles + s * S::A_BYTES, &tma_a, k * BK, m0, &full[s]);
        tma_load_2d(b_tiles + s * S::B_STRIDE, &tma_b, k * BK, n0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN);
      bool ok = true;
      for (int k = 0; k < num_k && ok; ++k) {
        int s = k % S::STAGES;
        uint32_t phase = (uint32_t)(k / S::STAGES) & 1u;
        ok = mbar_wait(&full[s], phase, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        uint64_t adesc = make_smem_desc(a_tiles + s * S::A_BYTES);
        uint64_t bdesc = make_smem_desc(b_tiles + s * S::B_STRIDE);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          // advance both descriptors by 8 fp32 = 32 bytes inside the swizzled row (address field is in 16-byte units)
          umma_tf32(tmem_base, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (k | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&empty[s]);        // the stage may be refilled once these MMAs have read it
      }
      umma_commit(acc_ready);          // fires when every MMA issued above has completed
    }
  } else {
    // epilogue warps 2..5 -> TMEM lane groups 2, 3, 0, 1
    const int lg = warp & 3;
    mbar_wait(acc_ready, 0u, &abort_flag);
    // decide as a group: the TMEM loads are warp-collective and the staged store below synchronises all four
    // epilogue warps, so either every one of them runs the epilogue or none does
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool ok = abort_flag == 0;
    tc_fence_after();
    if (ok && num_k > 0) {
      const int row = m0 + lg * 32 + lane;
      const uint32_t lane_base = tmem_base + ((uint32_t)(lg * 32) << 16);
      if (use_tma_store) {
        // Stage the tile as 32-column slabs of 128 rows x 128 bytes in the (now idle) pipeline buffers, in the
        // 128-byte swizzle the store descriptor expects: 16-byte chunk c of row r lives at chunk c ^ (r & 7).
        const int r = lg * 32 + lane;
        constexpr int SLABS = (BN + 31) / 32;
        constexpr int CAP = S::TILE_BYTES / (BM * 128);                 // slabs the drained buffers can hold at once
        constexpr int PER_ROUND = SLABS < CAP ? SLABS : CAP;
#pragma unroll 1
        for (int s0 = 0; s0 < SLABS; s0 += PER_ROUND) {
#pragma unroll 1
          for (int sl = s0; sl < s0 + PER_ROUND && sl < SLABS; ++sl) {
            uint8_t* slab = tiles + (sl - s0) * (BM * 128);
            uint32_t ra[16], rb[16];
            tmem_ld16_nowait(lane_base + (uint32_t)(sl * 32), ra);
            if (BN >= 32) tmem_ld16_nowait(lane_base + (uint32_t)(sl * 32 + 16), rb);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              if (BN < 32 && c >= 4) break;
              const uint32_t* src = c < 4 ? &ra[c * 4] : &rb[(c - 4) * 4];
              float4 o = make_float4(__uint_as_float(src[0]), __uint_as_float(src[1]), __uint_as_float(src[2]), __uint_as_float(src[3]));
              if (bias != nullptr) {
                int col = n0 + sl * 32 + c * 4;
                o.x += col < N ? bias[col] : 0.f; o.y += col + 1 < N ? bias[col + 1] : 0.f;
                o.z += col + 2 < N ? bias[col + 2] : 0.f; o.w += col + 3 < N ? bias[col + 3] : 0.f;
              }
              *reinterpret_cast<float4*>(slab + r * 128 + ((c ^ (r & 7)) << 4)) = o;
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 1, 128;" ::: "memory");                     // the four epilogue warps only
          if (col_partials != nullptr) {
            // per-column sum and sum of squares over this CTA's 128 rows, read back from the staged slabs:
            // thread (quarter, col) adds 32 rows of one column; a row of a slab is one conflict-free 128-byte line
            const int te = (warp - 2) * 32 + lane, col = te & 31, quarter = te >> 5;
#pragma unroll 1
            for (int sl = s0; sl < s0 + PER_ROUND && sl < SLABS; ++sl) {
              const uint8_t* slab = tiles + (sl - s0) * (BM * 128);
              float sum = 0.f, sq = 0.f;
#pragma unroll 8
              for (int rr = quarter * 32; rr < quarter * 32 + 32; ++rr) {
                float v = *reinterpret_cast<const float*>(slab + rr * 128 + (((col >> 2) ^ (rr & 7)) << 4) + ((col & 3) << 2));
                v = (m0 + rr < M) ? v : 0.f;
                sum += v;
                sq = fmaf(v, v, sq);
              }
              colsum[(quarter * 32 + col) * 2] = sum;
              colsum[(quarter * 32 + col) * 2 + 1] = sq;
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (quarter == 0) {
                int gc = n0 + sl * 32 + col;
                if (gc < N) {
                  float a = colsum[col * 2] + colsum[(32 + col) * 2] + colsum[(64 + col) * 2] + colsum[(96 + col) * 2];
                  float b = colsum[col * 2 + 1] + colsum[(32 + col) * 2 + 1] + colsum[(64 + col) * 2 + 1] + colsum[(96 + col) * 2 + 1];
                  col_partials[((int64_t)blockIdx.x * 2) * N + gc] = a;
                  col_partials[((int64_t)blockIdx.x * 2 + 1) * N + gc] = b;
                }
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");
            }
          }
          if (warp == 2 && lane == 0) {
#pragma unroll 1
            for (int sl = s0; sl < s0 + PER_ROUND && sl < SLABS; ++sl) {
              if (n0 + sl * 32 >= N) break;
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&tma_c), "r"(smem_u32(tiles + (sl - s0) * (BM * 128))), "r"(n0 + sl * 32), "r"(m0)
                           : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the staging buffers are free again
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      } else {
      auto store16 = [&](const uint32_t (&r)[16], int c0) {
        if (row >= M) return;
        float* dst = C + (int64_t)row * ldc + n0 + c0;
        if (n0 + c0 + 15 < N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            float4 o = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            if (bias != nullptr) {
              o.x += bias[n0 + c0 + j]; o.y += bias[n0 + c0 + j + 1]; o.z += bias[n0 + c0 + j + 2]; o.w += bias[n0 + c0 + j + 3];
            }
            *reinterpret_cast<float4*>(dst + j) = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (n0 + c0 + j < N) dst[j] = __uint_as_float(r[j]) + (bias != nullptr ? bias[n0 + c0 + j] : 0.0f);
        }
      };
      if (BN >= 32) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {     // two TMEM loads in flight, then 128 bytes of stores per thread
          uint32_t ra[16], rb[16];
          tmem_ld16_nowait(lane_base + (uint32_t)c0, ra);
          tmem_ld16_nowait(lane_base + (uint32_t)(c0 + 16), rb);
          tmem_ld_wait();
          store16(ra, c0);
          store16(rb, c0 + 16);
        }
      } else {
        uint32_t ra[16];
        tmem_ld16_nowait(lane_base, ra);
        tmem_ld_wait();
        store16(ra, 0);
      }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag && error_flag != nullptr) atomicExch(error_flag, 1);
}

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
constexpr int PERSISTENT_THREADS = 64 + 128 * EPI_GROUPS;

template <int BN>
__global__ void __launch_bounds__(PERSISTENT_THREADS, 1)
gemm_tf32_persistent_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                            const __grid_constant__ CUtensorMap tma_c, const float* __restrict__ bias, int M, int N, int K,
                            int tiles_m, int tiles_n, int accumulate, float* __restrict__ col_partials,
                            int* __restrict__ error_flag) {
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
  const int total_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int g = 0; g < EPI_GROUPS; ++g) epi_go[g] = 1;
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128 * EPI_GROUPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
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

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;                                        // k-blocks issued so far, over all tiles
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m0 = (t / tiles_n) * BM, n0 = (t % tiles_n) * BN;
        for (int k = 0; k < num_k; ++k, ++it) {
          const int s = (int)(it % S::STAGES);
          const uint32_t phase = (it / S::STAGES) & 1u;
          if (!mbar_wait(&empty[s], phase ^ 1u, &abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full[s], (uint32_t)(S::A_BYTES + S::B_BYTES));
          tma_load_2d(a_tiles + s * S::A_BYTES, &tma_a, k * BK, m0, &full[s]);
          tma_load_2d(b_tiles + s * S::B_BYTES, &tma_b, k * BK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN);
      uint32_t it = 0, lt = 0;                                // k-blocks consumed, tiles started
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++lt) {
        const uint32_t buf = lt & 1u, aphase = (lt >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], aphase ^ 1u, &abort_flag)) break;      // first use of a buffer passes at once
        tc_fence_after();
        const uint32_t tmem_c = tmem_base + buf * (uint32_t)BN;
        for (int k = 0; k < num_k; ++k, ++it) {
          const int s = (int)(it % S::STAGES);
          const uint32_t phase = (it / S::STAGES) & 1u;
          if (!mbar_wait(&full[s], phase, &abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(a_tiles + s * S::A_BYTES);
          const uint64_t bdesc = make_smem_desc(b_tiles + s * S::B_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_tf32(tmem_c, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (k | kk) != 0 ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // Two epilogue groups of four warps (TMEM lane quarters warp & 3); group g drains the 32-column slabs
    // g, g + 2, ... of every tile through its own half of the staging ring, with its own named barrier and its
    // own store-issuing thread, so the groups never wait for each other.
    const int ew = warp - 2;
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
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++lt) {
      const int mi = t / tiles_n;
      const int m0 = mi * BM, n0 = (t % tiles_n) * BN;
      const uint32_t buf = lt & 1u, aphase = (lt >> 1) & 1u;
      const bool got = mbar_wait(&acc_full[buf], aphase, &abort_flag);
      // one thread decides for the group: the TMEM loads are warp-collective and the named barriers below
      // involve all four warps, so either every one of them drains this tile or none does
      if (issuer) epi_go[grp] = (got && abort_flag == 0) ? 1 : 0;
      group_bar(grp);
      if (!epi_go[grp]) break;
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
          if (bias != nullptr) {
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
            if (accumulate)                      // C += tile: the add happens in L2, C is never read by the SM
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
        if (col_partials != nullptr) {
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
      if (col_partials != nullptr) {
        group_bar(grp);
        for (int idx = te; idx < (SLABS / EPI_GROUPS) * 32; idx += 128) {       // the columns of this group's slabs
          const int c = (grp + EPI_GROUPS * (idx >> 5)) * 32 + (idx & 31);
          const int gc = n0 + c;
          if (gc < N) {
            float a = (my_colsum[c * 2] + my_colsum[(BN + c) * 2]) + (my_colsum[(2 * BN + c) * 2] + my_colsum[(3 * BN + c) * 2]);
            float b = (my_colsum[c * 2 + 1] + my_colsum[(BN + c) * 2 + 1]) + (my_colsum[(2 * BN + c) * 2 + 1] + my_colsum[(3 * BN + c) * 2 + 1]);
            col_partials[((int64_t)mi * 2) * N + gc] = a;
            col_partials[((int64_t)mi * 2 + 1) * N + gc] = b;
          }
        }
      }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory outlives the stores
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
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
  static constexpr int STAGES = (BN <= 64) ? 6 : ((BN <= 128) ? 5 : 3);
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int RING_BYTES = STAGES * (A_BYTES + B_BYTES);
  static constexpr int NSLAB = 2;
  static constexpr int SLAB_BYTES = BM * 128;
  static constexpr int STAGING_OFF = RING_BYTES;
  static constexpr int BAR_OFF = STAGING_OFF + NSLAB * SLAB_BYTES;
  static constexpr int TOTAL = 1024 + BAR_OFF + 256;
  static constexpr int TMEM_COLS = BN;
  static_assert(TOTAL <= 232448, "shared memory of one CTA");
};

__device__ __forceinline__ uint64_t make_smem_desc_mn(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);      // start address
  d |= (uint64_t)(4096 >> 4) << 16;                      // leading byte offset: next 32-float chunk of the M / N dimension
  d |= (uint64_t)(512 >> 4) << 32;                       // stride byte offset: next group of 4 K rows
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  d |= (uint64_t)1 << 61;                                // layout type: SWIZZLE_128B_BASE32B
  return d;
}

__host__ __device__ constexpr uint32_t make_idesc_mn(int n) {
  return make_idesc(n) | (1u << 15) | (1u << 16);        // A and B are MN-major
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tn_tf32_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_c, int P, int Mo, int No, int tiles_n, int splits,
                    int kblocks_per_split, int* __restrict__ error_flag) {
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
  const int total_k = (P + BK - 1) / BK;
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
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (num_k > 0) {
    if (warp == 0) {
      if (lane == 0) {
        for (int k = 0; k < num_k; ++k) {
          const int s = k % S::STAGES;
          const uint32_t phase = (uint32_t)(k / S::STAGES) & 1u;
          if (!mbar_wait(&empty[s], phase ^ 1u, &abort_flag)) break;
          mbar_expect_tx(&full[s], (uint32_t)(S::A_BYTES + S::B_BYTES));
          // one 4 KB box (32 floats x 32 positions) per 32-float chunk of the output dimensions
#pragma unroll
          for (int c = 0; c < BM / 32; ++c)
            tma_load_2d(a_tiles + s * S::A_BYTES + c * 4096, &tma_a, m0 + c * 32, (k_begin + k) * BK, &full[s]);
#pragma unroll
          for (int c = 0; c < BN / 32; ++c)
            tma_load_2d(b_tiles + s * S::B_BYTES + c * 4096, &tma_b, n0 + c * 32, (k_begin + k) * BK, &full[s]);
        }
      }
    } else if (warp == 1) {
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
          for (int kk = 0; kk < BK / UMMA_K; ++kk)     // 8 positions = 8 rows of 128 bytes = 1024 bytes = 64 address units
            umma_tf32(tmem_base, adesc + (uint64_t)(kk * 64), bdesc + (uint64_t)(kk * 64), idesc, (k | kk) != 0 ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(acc_ready);
      }
    } else {
      const int lg = warp & 3;
      const int r = lg * 32 + lane;
      const int te = (warp - 2) * 32 + lane;
      const bool issuer = te == 0;
      const bool got = mbar_wait(acc_ready, 0u, &abort_flag);
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
  if (warp == 1) {
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

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

template <int BN>
int launch(const float* A, const float* B, float* C, const float* bias, int M, int N, int K, int64_t lda, int64_t ldb,
           int64_t ldc, float* col_partials, int* error_flag, cudaStream_t st) {
  using S = Smem<BN>;
  CUtensorMap ma, mb, mc;
  if (make_map(&ma, A, M, K, lda, BM) != 0 || make_map(&mb, B, N, K, ldb, BN) != 0) return (int)cudaErrorInvalidValue;
  int use_tma_store = tma_store_ok(C, ldc) && make_map(&mc, C, M, N, ldc, BM) == 0 ? 1 : 0;
  if (!use_tma_store) {
    if (col_partials != nullptr) return (int)cudaErrorInvalidValue;     // the column sums ride the staged epilogue
    mc = ma;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)((N + BN - 1) / BN));
  gemm_tf32_kernel<BN><<<grid, GEMM_THREADS, S::TOTAL, st>>>(ma, mb, mc, use_tma_store, C, bias, M, N, K, ldc, col_partials, error_flag);
  return (int)cudaGetLastError();
}

template <int BN>
int launch_persistent(const float* A, const float* B, float* C, const float* bias, int M, int N, int K, int64_t lda,
                      int64_t ldb, int64_t ldc, int accumulate, float* col_partials, int* error_flag, cudaStream_t st) {
  using S = PSmem<BN>;
  CUtensorMap ma, mb, mc;
  if (make_map(&ma, A, M, K, lda, BM) != 0 || make_map(&mb, B, N, K, ldb, BN) != 0 || make_map(&mc, C, M, N, ldc, BM) != 0)
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_persistent_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  int64_t total = (int64_t)tiles_m * tiles_n;
  int64_t grid = total < sm_count() ? total : sm_count();
  gc::launch_pdl(gemm_tf32_persistent_kernel<BN>, dim3((unsigned)grid), dim3(PERSISTENT_THREADS), (size_t)S::TOTAL, st, ma, mb, mc, bias,
                 M, N, K, tiles_m, tiles_n, accumulate, col_partials, error_flag);
  return (int)cudaGetLastError();
}


// Row-major [P, D] fp32 matrix as an MN-major operand: box = 32 floats x 32 rows (4 KB), shared-memory layout
// "128-byte swizzle, 32-byte atoms" (the MN-major layout of 32-bit types).
int make_map_mn(CUtensorMap* map, const float* base, int64_t P, int64_t D, int64_t ld) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)P};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)BK};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// split-K policy of the TN kernel (see gc_cuda_gemm_tn_config).  One CTA per SM: measured 10-25 % faster than two on the
// 131072- and 32768-position weight gradients of ResNet-50 (fewer partial tiles to add, longer pipelines), equal below.
int g_tn_ctas_per_sm = 1, g_tn_min_kblocks = 8;

template <int BN>
int launch_tn(const float* A, const float* B, float* C, int P, int Mo, int No, int64_t lda, int64_t ldb, int64_t ldc,
              int* error_flag, cudaStream_t st) {
  using S = TnSmem<BN>;
  CUtensorMap ma, mb, mc;
  if (make_map_mn(&ma, A, P, Mo, lda) != 0 || make_map_mn(&mb, B, P, No, ldb) != 0 ||
      make_map(&mc, C, Mo, No, ldc, BM) != 0)
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tn_tf32_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int tiles_m = (Mo + BM - 1) / BM, tiles_n = (No + BN - 1) / BN;
  int tiles = tiles_m * tiles_n;
  int total_k = (P + BK - 1) / BK;
  // about g_tn_ctas_per_sm CTAs per SM over all tiles, at least g_tn_min_kblocks k-blocks each so that the pipeline fills
  int splits = (g_tn_ctas_per_sm * sm_count() + tiles - 1) / tiles;
  if (splits > (total_k + g_tn_min_kblocks - 1) / g_tn_min_kblocks) splits = (total_k + g_tn_min_kblocks - 1) / g_tn_min_kblocks;
  if (splits < 1) splits = 1;
  int per = (total_k + splits - 1) / splits;
  splits = (total_k + per - 1) / per;
  gemm_tn_tf32_kernel<BN><<<(unsigned)(tiles * splits), GEMM_THREADS, S::TOTAL, st>>>(ma, mb, mc, P, Mo, No, tiles_n, splits, per,
                                                                                     error_flag);
  return (int)cudaGetLastError();
}

// 0 = choose, 1 = one tile per CTA, 2 = persistent;  tile width 0 = choose
int g_kernel_choice = 0, g_tile_choice = 0;

}  // namespace

extern "C" {

// 1 when the shapes / pointers meet the TMA rules: 16-byte aligned bases, row strides multiples of 16 bytes.
int gc_cuda_gemm_tf32_supported(const void* A, const void* B, int M, int N, int K, int64_t lda, int64_t ldb) {
  if (M < 1 || N < 1 || K < 1) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u)) return 0;
  if ((lda & 3) || (ldb & 3) || lda < K || ldb < K) return 0;
  return encode_fn() != nullptr ? 1 : 0;
}

// Tile width of the one-tile-per-CTA kernel: the widest of 256 / 128 / 64 columns that still yields at least
// ~2 CTAs per SM, so that wide N reads A once while small problems keep all SMs busy.
static int pick_bn(int M, int N) {
  if (N <= 16) return 16;
  if (N <= 64) return 64;
  int sms = sm_count();
  int64_t mt = (M + BM - 1) / BM;
  const int cand[3] = {256, 128, 64};
  for (int i = 0; i < 3; ++i) {
    int bn = cand[i];
    if (bn == 256 && N <= 128) continue;
    if (bn == 128 && N <= 64) continue;
    if (mt * ((N + bn - 1) / bn) >= 2 * sms) return bn;
  }
  return 64;
}

// Tile width of the persistent kernel: the candidate with the lowest modelled time.  A tile costs the larger of
// its DRAM share (C written once, A read once per row of tiles) and its shared-memory fill (A and B per
// k-block), plus a fixed start-up; CTAs work through ceil(tiles / SMs) tiles one after the other.
static int pick_bn_persistent(int M, int N, int K) {
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

int gc_cuda_gemm_tf32_m_tiles(int M) { return (M + BM - 1) / BM; }

// For measurements: kernel 0 = choose, 1 = one tile per CTA, 2 = persistent; tile width 0 = choose, else 64 / 128 / 256.
void gc_cuda_gemm_tf32_config(int kernel, int tile_n) {
  g_kernel_choice = kernel;
  g_tile_choice = tile_n;
}

// C[M, N] = A[M, K] * B[N, K]^T (+ bias[N]), or C += ... when accumulate != 0 (persistent kernel only: needs N > 16 and
// a C that meets the TMA rules; the additions are done by TMA reduce stores, i.e. in L2);
// error_flag (device int, may be NULL) is set when a wait ran out.
// col_partials (may be NULL): [m_tiles][2][N] floats receiving, per 128-row tile, the column sums and sums of
// squares of C -- the batch-norm statistics of a 1x1 convolution's output without another pass over it.
int gc_cuda_gemm_tf32(const float* A, const float* B, float* C, const float* bias, int M, int N, int K, int64_t lda,
                      int64_t ldb, int64_t ldc, int accumulate, float* col_partials, int* error_flag, void* cs) {
  if (!gc_cuda_gemm_tf32_supported(A, B, M, N, K, lda, ldb)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)cs;
  bool persistent = (g_kernel_choice != 1 || accumulate) && N > 16 && tma_store_ok(C, ldc);
  if (accumulate && !persistent) return (int)cudaErrorInvalidValue;
  if (persistent) {
    int bn = g_tile_choice ? g_tile_choice : pick_bn_persistent(M, N, K);
    switch (bn) {
      case 64: return launch_persistent<64>(A, B, C, bias, M, N, K, lda, ldb, ldc, accumulate, col_partials, error_flag, st);
      case 128: return launch_persistent<128>(A, B, C, bias, M, N, K, lda, ldb, ldc, accumulate, col_partials, error_flag, st);
      case 256: return launch_persistent<256>(A, B, C, bias, M, N, K, lda, ldb, ldc, accumulate, col_partials, error_flag, st);
      default: return (int)cudaErrorInvalidValue;
    }
  }
  switch (g_tile_choice && N > 16 ? g_tile_choice : pick_bn(M, N)) {
    case 16: return launch<16>(A, B, C, bias, M, N, K, lda, ldb, ldc, col_partials, error_flag, st);
    case 64: return launch<64>(A, B, C, bias, M, N, K, lda, ldb, ldc, col_partials, error_flag, st);
    case 128: return launch<128>(A, B, C, bias, M, N, K, lda, ldb, ldc, col_partials, error_flag, st);
    default: return launch<256>(A, B, C, bias, M, N, K, lda, ldb, ldc, col_partials, error_flag, st);
  }
}

// For measurements: CTAs per SM the split contraction aims at, and the fewest k-blocks (of 32 rows) a split may get.
void gc_cuda_gemm_tn_config(int ctas_per_sm, int min_kblocks) {
  g_tn_ctas_per_sm = ctas_per_sm > 0 ? ctas_per_sm : 1;
  g_tn_min_kblocks = min_kblocks > 0 ? min_kblocks : 8;
}

// 1 when C[Mo, No] += A[P, Mo]^T B[P, No] can run on the tensor cores: Mo and No multiples of 32, 16-byte aligned
// bases, row strides multiples of 16 bytes.
int gc_cuda_gemm_tn_tf32_supported(const void* A, const void* B, const void* C, int P, int Mo, int No, int64_t lda, int64_t ldb,
                                   int64_t ldc) {
  if (P < 1 || Mo < 32 || No < 32 || (Mo & 31) || (No & 31)) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u) || (reinterpret_cast<uintptr_t>(C) & 15u)) return 0;
  if ((lda & 3) || (ldb & 3) || (ldc & 3) || lda < Mo || ldb < No || ldc < No) return 0;
  return encode_fn() != nullptr ? 1 : 0;
}

// C[Mo, No] += A[P, Mo]^T * B[P, No] (weight gradient of a 1x1 convolution: A = dY, B = X).  The partial products of
// the split contraction are added onto C by TMA reduce stores: zero C first for a plain product.
int gc_cuda_gemm_tn_tf32(const float* A, const float* B, float* C, int P, int Mo, int No, int64_t lda, int64_t ldb, int64_t ldc,
                         int* error_flag, void* cs) {
  if (!gc_cuda_gemm_tn_tf32_supported(A, B, C, P, Mo, No, lda, ldb, ldc)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)cs;
  int bn = g_tile_choice ? g_tile_choice : (No <= 64 ? 64 : (No <= 128 ? 128 : 256));
  switch (bn) {
    case 64: return launch_tn<64>(A, B, C, P, Mo, No, lda, ldb, ldc, error_flag, st);
    case 128: return launch_tn<128>(A, B, C, P, Mo, No, lda, ldb, ldc, error_flag, st);
    case 256: return launch_tn<256>(A, B, C, P, Mo, No, lda, ldb, ldc, error_flag, st);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // extern "C"
