// Symmetric-arena communication substrate: the arena header (flags, norm slots, barrier words,
// status), bounded waits, the per-rank grid barrier and the cross-rank signal/wait protocol used by
// every fused compress+collective kernel.
//
// One arena per rank, same layout on all ranks, mapped into every peer (CUDA IPC).  A kernel gets
// the table of arena base pointers as seen from its own rank.  Synchronisation uses monotonically
// increasing epochs (never reset), so a flag value left over from an earlier step can never satisfy
// a later wait, and no cleanup pass is needed between steps.
//
// Every wait is bounded (globaltimer deadline).  When a wait runs out the kernel records
// STATUS_TIMEOUT (phase, peer) in its own header, raises the header's abort word so that all later
// waits of the same launch return immediately, and runs to completion; the host reads the status.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_common.h"
#include "gc_device.cuh"

namespace gc {

constexpr int MAXW = 8;            // ranks per node (one NVSwitch domain)
constexpr int NFLAGS = 6;          // distinct signal phases per step
constexpr int MAX_PARTIALS = 1024;
constexpr int64_t ARENA_HEADER_BYTES = 16384;

struct ArenaHeader {
  unsigned long long norm_slot[2][MAXW];   // (epoch << 32) | float bits ; [epoch parity][source rank]
  uint32_t flag[NFLAGS][MAXW];             // flag[phase][source rank] = epoch of the last signal
  uint32_t bar_count;                      // per-rank grid barrier: arrivals of the current generation
  uint32_t bar_gen;                        // per-rank grid barrier: generation
  uint32_t status;                         // STATUS_* of the first failure (0 = ok)
  uint32_t status_detail;                  // (phase << 16) | peer for timeouts, index for bounds errors
  uint32_t abort;                          // non-zero: skip all remaining waits of this launch
  uint32_t epoch;                          // epoch of the last fused launch on this rank (device-resident so that
                                           // a replayed CUDA graph still advances it)
  uint32_t calls;                          // launches so far; optional source of the Philox step
  uint32_t pad0[1];
  float partial[MAX_PARTIALS];             // per-block partial maxima
  float reduced[8];                        // small per-step results (local norm, ...)
};
static_assert(sizeof(ArenaHeader) <= ARENA_HEADER_BYTES, "arena header too large");

struct RankView {
  uint8_t* arena[MAXW];   // arena base of every rank as mapped into THIS rank's address space
  const float* in;        // this rank's input gradient
  float* out;             // this rank's output gradient
  const void* aux;        // optional second input (index list of the sparse exchange)
  int rank;
  int pad;
};

// Up to MAXW virtual ranks per launch: real multi-GPU runs use exactly one (its own rank); the
// single-GPU emulation runs all ranks of a group side by side in one cooperative launch.
struct LaunchViews {
  RankView r[MAXW];
  int n_virtual;
  int blocks_per_rank;
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

struct Waiter {
  ArenaHeader* hdr;
  unsigned long long deadline;
  __device__ __forceinline__ bool aborted() const { return *((volatile uint32_t*)&hdr->abort) != 0; }
  __device__ __forceinline__ void fail(int phase, int peer) {
    if (atomicCAS(&hdr->status, 0u, (uint32_t)STATUS_TIMEOUT) == 0u)
      hdr->status_detail = ((uint32_t)phase << 16) | (uint32_t)(peer & 0xffff);
    atomicExch(&hdr->abort, 1u);
    __threadfence();
  }
  // An index that would have gone outside its tensor: the access is not made; the first such index is kept beside
  // STATUS_BOUNDS for the host (the launch carries on: other elements are unaffected).
  __device__ __forceinline__ void out_of_bounds(long long index) {
    if (atomicCAS(&hdr->status, 0u, (uint32_t)STATUS_BOUNDS) == 0u) hdr->status_detail = (uint32_t)index;
  }
};

// Debug build (-DGC_DEBUG_BOUNDS, `python -m gradient_compression_b200.build --debug-bounds`): every computed index of the
// gather / scatter paths is checked before use; a failing one is recorded (Waiter::out_of_bounds) and its access skipped.
// The regular build keeps only the checks on indices that come from user data (the sparse exchange's index lists).
#if defined(GC_DEBUG_BOUNDS)
#define GC_INDEX_OK(w, i, n) (((i) >= 0 && (long long)(i) < (long long)(n)) ? true : ((w).out_of_bounds((long long)(i)), false))
#else
#define GC_INDEX_OK(w, i, n) true
#endif

// Per-rank grid barrier (generation counting, works for any block count per launch).
__device__ __forceinline__ void grid_barrier(Waiter& w, int nblocks, int phase) {
  __syncthreads();
  if (threadIdx.x == 0) {
    ArenaHeader* h = w.hdr;
    __threadfence_system();   // cumulative: publishes the whole block's writes (ordered by bar.sync)
    uint32_t gen = ld_acquire_gpu(&h->bar_gen);
    uint32_t prev = atomicAdd(&h->bar_count, 1u);
    if (prev == (uint32_t)nblocks - 1u) {
      h->bar_count = 0;
      __threadfence();
      atomicAdd(&h->bar_gen, 1u);
    } else {
      int it = 0;
      while (ld_acquire_gpu(&h->bar_gen) == gen) {
        if ((++it & 63) == 0) {
          if (w.aborted()) break;
          if (global_ns() > w.deadline) { w.fail(phase, 0xfffe); break; }
        }
      }
    }
  }
  __syncthreads();
}

// Signal phase `phase` with `epoch` to every rank (called by ONE block after a grid barrier).
__device__ __forceinline__ void signal_all(const RankView& v, int world, int phase, uint32_t epoch) {
  if (threadIdx.x < world) {
    ArenaHeader* peer = reinterpret_cast<ArenaHeader*>(v.arena[threadIdx.x]);
    __threadfence_system();
    st_release_sys(&peer->flag[phase][v.rank], epoch);
  }
}

// Wait until every rank has signalled `phase` for `epoch` (every block calls this).
__device__ __forceinline__ void wait_all(Waiter& w, int world, int phase, uint32_t epoch) {
  if (threadIdx.x < world) {
    const uint32_t* f = &w.hdr->flag[phase][threadIdx.x];
    int it = 0;
    while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
      if ((++it & 63) == 0) {
        if (w.aborted()) break;
        if (global_ns() > w.deadline) { w.fail(phase, threadIdx.x); break; }
      }
    }
  }
  __syncthreads();
}

// Epoch of this launch: one more than the last completed launch.  Every block reads it before the
// first grid barrier; commit_epoch() (one thread, after that barrier) stores it back.
__device__ __forceinline__ uint32_t next_epoch(const ArenaHeader* h) { return *((volatile const uint32_t*)&h->epoch) + 1u; }
__device__ __forceinline__ uint32_t launch_calls(const ArenaHeader* h) { return *((volatile const uint32_t*)&h->calls); }
__device__ __forceinline__ void commit_epoch(ArenaHeader* h, uint32_t epoch, int bid) {
  if (bid == 0 && threadIdx.x == 0) {
    h->epoch = epoch;
    h->calls = h->calls + 1u;
  }
}

// Exchange one float per rank and return the maximum over ranks (valid in every thread).
// `local` must be valid in thread 0 of the calling block; only block `is_sender` publishes.
__device__ __forceinline__ float exchange_max(Waiter& w, const RankView& v, int world, uint32_t epoch, float local,
                                              bool is_sender, float* smem) {
  int par = epoch & 1;
  if (is_sender && threadIdx.x < world) {
    ArenaHeader* peer = reinterpret_cast<ArenaHeader*>(v.arena[threadIdx.x]);
    unsigned long long word = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(local);
    st_relaxed_sys_u64(&peer->norm_slot[par][v.rank], word);
  }
  float got = 0.0f;
  if (threadIdx.x < world) {
    const unsigned long long* slot = &w.hdr->norm_slot[par][threadIdx.x];
    int it = 0;
    for (;;) {
      unsigned long long word = ld_relaxed_sys_u64(slot);
      if ((uint32_t)(word >> 32) == epoch) { got = __uint_as_float((uint32_t)word); break; }
      if ((++it & 63) == 0) {
        if (w.aborted()) break;
        if (global_ns() > w.deadline) { w.fail(0x10, threadIdx.x); break; }
      }
    }
  }
  if (threadIdx.x < 32) {
    got = warp_max(got);
    if (threadIdx.x == 0) smem[0] = got;
  }
  __syncthreads();
  float r = smem[0];
  __syncthreads();
  return r;
}

// Grid-wide maximum of per-thread values within one rank; result valid in every thread of every block.
__device__ __forceinline__ float rank_max(Waiter& w, float v, int bid, int nblocks, float* smem, int phase) {
  float m = block_max(v, smem);
  if (threadIdx.x == 0) w.hdr->partial[bid] = m;
  grid_barrier(w, nblocks, phase);
  float r = 0.0f;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) r = fmaxf(r, ((volatile float*)w.hdr->partial)[i]);
  r = block_max(r, smem);
  __syncthreads();
  return r;
}

}  // namespace gc
