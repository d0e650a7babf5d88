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
// Common structure, no clusters, no multicast (the persistent and the TN kernel are templates in gc_tc.cuh, shared with the
// convolution entry points of gc_conv_tc.cu; they run two producer warps, the tile kernel in this file one):
//   producer warps  TMA loads (cp.async.bulk.tensor, 128-byte swizzle) into a ring of shared-memory stages
//   MMA warp        allocates TMEM, issues tcgen05.mma (one elected thread), commits stages back to the producers
//   epilogue warps  tcgen05.ld of the fp32 accumulator from TMEM, bias add, 32-column slabs staged in shared
//                   memory (128-byte swizzled, bank-conflict free) and written with TMA stores / TMA reduce stores
// Every mbarrier wait is bounded; when one runs out the CTA sets *error_flag, abandons its tile, frees
// its TMEM and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_tc.cuh"

namespace {

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
                      int64_t ldb, int64_t ldc, int accumulate, float* col_partials, int* error_flag, cudaStream_t st,
                      const BnFin* fin, int splits) {
  CUtensorMap ma, mb, mc;
  if (make_map(&ma, A, M, K, lda, BM) != 0 || make_map(&mb, B, N, K, ldb, BN) != 0 || make_map(&mc, C, M, N, ldc, BM) != 0)
    return (int)cudaErrorInvalidValue;
  if (splits > 1 && !accumulate) {
    cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, st);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_persistent_maps<BN>(ma, mb, mc, ConvA{}, bias, M, N, K, (accumulate || splits > 1) ? 1 : 0, col_partials, error_flag,
                                    st, fin, nullptr, splits);
}

template <int BN>
int launch_tn(const float* A, const float* B, float* C, int P, int Mo, int No, int64_t lda, int64_t ldb, int64_t ldc,
              int* error_flag, cudaStream_t st) {
  CUtensorMap ma, mb, mc;
  int box3d = 0;        // whole-operand 3-D boxes where the matrix is made of whole 32-float chunks
  if ((Mo & 31) == 0 && make_map_mn3(&ma, A, P, Mo, lda, TBK, BM / 32) == 0) box3d |= 1;
  else if (make_map_mn(&ma, A, P, Mo, lda) != 0) return (int)cudaErrorInvalidValue;
  if ((No & 31) == 0 && make_map_mn3(&mb, B, P, No, ldb, TBK, BN / 32) == 0) box3d |= 2;
  else if (make_map_mn(&mb, B, P, No, ldb) != 0) return (int)cudaErrorInvalidValue;
  if (make_map(&mc, C, Mo, No, ldc, BM) != 0)
    return (int)cudaErrorInvalidValue;
  return launch_tn_maps<BN>(ma, mb, mc, ConvA{}, P, Mo, No, error_flag, st, box3d);
}

// 0 = choose, 1 = one tile per CTA, 2 = persistent;  tile width 0 = choose
int g_kernel_choice = 0;

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

int gc_cuda_gemm_tf32_m_tiles(int M) { return (M + BM - 1) / BM; }

// Bytes of the zero-initialised scratch a BnFinHost points to, for outputs of up to max_channels columns.
int64_t gc_cuda_bn_fin_scratch_bytes(int max_channels) { return 256 + (int64_t)2 * max_channels * 8; }

// For measurements: kernel 0 = choose, 1 = one tile per CTA, 2 = persistent; tile width 0 = choose, else 64 / 128 / 256.
void gc_cuda_gemm_tf32_config(int kernel, int tile_n) {
  g_kernel_choice = kernel;
  gctc::tile_choice = tile_n;
}

// C[M, N] = A[M, K] * B[N, K]^T (+ bias[N]), or C += ... when accumulate != 0 (persistent kernel only: needs N > 16 and
// a C that meets the TMA rules; the additions are done by TMA reduce stores, i.e. in L2);
// error_flag (device int, may be NULL) is set when a wait ran out.
// col_partials (may be NULL): [m_tiles][2][N] floats receiving, per 128-row tile, the column sums and sums of
// squares of C -- the batch-norm statistics of a 1x1 convolution's output without another pass over it.
// bn_fin (may be NULL): a BnFinHost; the kernel then finishes the batch-norm statistics of C itself (mean and
// 1 / sqrt(var + eps) into stats[2N], running statistics updated) instead of emitting col_partials.  Persistent kernel only.
int gc_cuda_gemm_tf32(const float* A, const float* B, float* C, const float* bias, int M, int N, int K, int64_t lda,
                      int64_t ldb, int64_t ldc, int accumulate, float* col_partials, int* error_flag, void* cs,
                      const void* bn_fin) {
  if (!gc_cuda_gemm_tf32_supported(A, B, M, N, K, lda, ldb)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)cs;
  const BnFin fin_dev = bn_fin_from_host(bn_fin);
  const BnFin* fin = fin_dev.acc != nullptr ? &fin_dev : nullptr;
  bool persistent = (g_kernel_choice != 1 || accumulate || fin != nullptr) && N > 16 && tma_store_ok(C, ldc);
  if ((accumulate || fin != nullptr) && !persistent) return (int)cudaErrorInvalidValue;
  if (persistent) {
    int bn = gctc::tile_choice ? gctc::tile_choice : pick_bn_persistent(M, N, K), splits = 1;
    if (col_partials == nullptr && fin == nullptr)
      plan_persistent(M, N, K, accumulate ? 0.0 : zero_cycles((int64_t)M * N), &bn, &splits);
    switch (bn) {
      case 64: return launch_persistent<64>(A, B, C, bias, M, N, K, lda, ldb, ldc, accumulate, col_partials, error_flag, st, fin, splits);
      case 128: return launch_persistent<128>(A, B, C, bias, M, N, K, lda, ldb, ldc, accumulate, col_partials, error_flag, st, fin, splits);
      case 256: return launch_persistent<256>(A, B, C, bias, M, N, K, lda, ldb, ldc, accumulate, col_partials, error_flag, st, fin, splits);
      default: return (int)cudaErrorInvalidValue;
    }
  }
  switch (gctc::tile_choice && N > 16 ? gctc::tile_choice : pick_bn(M, N)) {
    case 16: return launch<16>(A, B, C, bias, M, N, K, lda, ldb, ldc, col_partials, error_flag, st);
    case 64: return launch<64>(A, B, C, bias, M, N, K, lda, ldb, ldc, col_partials, error_flag, st);
    case 128: return launch<128>(A, B, C, bias, M, N, K, lda, ldb, ldc, col_partials, error_flag, st);
    default: return launch<256>(A, B, C, bias, M, N, K, lda, ldb, ldc, col_partials, error_flag, st);
  }
}

// Contraction splits gc_cuda_gemm_tf32 would use for C[M, N] over K if the caller computed the column statistics in a
// pass of its own over C instead of asking for col_partials (that pass is charged to the split plan).  1: do not split.
int gc_cuda_gemm_tf32_splits(int M, int N, int K) {
  if (N <= 16) return 1;
  int bn, splits;
  plan_persistent(M, N, K, zero_cycles((int64_t)M * N) + stats_pass_cycles((int64_t)M * N), &bn, &splits);
  return splits;
}

// For measurements: contraction splits of the persistent kernel (0 = modelled, 1 = never, n = n wherever a product allows it).
void gc_cuda_tc_split_config(int splits) { gctc::split_choice = splits; }

// For measurements: how the producer warps issue their TMA loads (bit 0: prefetch the tensor maps; bit 1: spread the
// loads of a stage over several lanes).
void gc_cuda_tc_tma_mode(int mode) { gctc::tma_mode = mode; }

// For measurements: CTAs per SM the split contraction aims at, and the fewest k-blocks (of 32 rows) a split may get.
void gc_cuda_gemm_tn_config(int ctas_per_sm, int min_kblocks) {
  gctc::tn_ctas_per_sm = ctas_per_sm > 0 ? ctas_per_sm : 1;
  gctc::tn_min_kblocks = min_kblocks > 0 ? min_kblocks : 4;
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
  int bn = gctc::tile_choice ? gctc::tile_choice : (No <= 64 ? 64 : (No <= 128 ? 128 : 256));
  switch (bn) {
    case 64: return launch_tn<64>(A, B, C, P, Mo, No, lda, ldb, ldc, error_flag, st);
    case 128: return launch_tn<128>(A, B, C, P, Mo, No, lda, ldb, ldc, error_flag, st);
    case 256: return launch_tn<256>(A, B, C, P, Mo, No, lda, ldb, ldc, error_flag, st);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // extern "C"
