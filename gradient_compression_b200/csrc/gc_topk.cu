// Top-K selection by |value| for many segments (tensors) of one flat buffer at once: exact radix select on
// the IEEE bit pattern of |a| (3 passes of 11 + 11 + 10 bits), then compaction into (index, value) lists.
// Error feedback is fused: pass 0 forms a = g + e and stores it in e; compaction zeroes the selected
// entries of e, so afterwards e is exactly the memory the reference keeps (reducer.py:1161,1186-1189), and
// the reference's per-tensor torch.topk calls (reducer.py:1180; 161 launches + sorts for ResNet-50) become
// 7 launches that each stream the gradient once.
// Segment table: int64 rows of {start, len, k, out_off, chunk_start, 0}.
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_device.cuh"

using namespace gc;

namespace {

constexpr int SEG_FIELDS = 6;
constexpr int CHUNK = 4096;
constexpr int BINS = 2048;
constexpr int TK_THREADS = 256;

struct SegState {          // per segment, device resident
  uint32_t prefix;         // selected high bits so far
  int32_t k_rem;           // how many still to take among the elements that match the prefix
  uint32_t gt_count;       // compaction: slots handed to keys > threshold
  uint32_t eq_count;       // compaction: keys == threshold seen
};

__device__ __forceinline__ int find_seg(const int64_t* __restrict__ tab, int n_seg, int64_t chunk) {
  int lo = 0, hi = n_seg - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (tab[(int64_t)mid * SEG_FIELDS + 4] <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ uint32_t key_of(float a) { return __float_as_uint(a) & 0x7fffffffu; }

// pass: 0, 1, 2.  Pass 0 also folds the error memory: e <- g + e.
template <int PASS>
__global__ void __launch_bounds__(TK_THREADS) topk_hist_kernel(const float* __restrict__ g, float* __restrict__ e,
                                                               const int64_t* __restrict__ tab, int n_seg,
                                                               const SegState* __restrict__ state,
                                                               uint32_t* __restrict__ hist) {
  __shared__ uint32_t sh[BINS];
  int seg = find_seg(tab, n_seg, (int64_t)blockIdx.x);
  const int64_t* t = tab + (int64_t)seg * SEG_FIELDS;
  int64_t start = t[0], len = t[1], k = t[2];
  int64_t c0 = ((int64_t)blockIdx.x - t[4]) * CHUNK;
  int64_t c1 = c0 + CHUNK < len ? c0 + CHUNK : len;
  bool skip = k >= len;       // everything is taken: no threshold needed
  for (int i = threadIdx.x; i < BINS; i += TK_THREADS) sh[i] = 0;
  __syncthreads();
  uint32_t prefix = PASS == 0 ? 0u : state[seg].prefix;
  for (int64_t i = c0 + threadIdx.x; i < c1; i += TK_THREADS) {
    float a;
    if (PASS == 0) {
      a = g[start + i] + (e != nullptr ? e[start + i] : 0.0f);
      if (e != nullptr) e[start + i] = a;
    } else {
      a = e != nullptr ? e[start + i] : g[start + i];
    }
    if (skip) continue;
    uint32_t key = key_of(a);
    if (PASS == 0) atomicAdd(&sh[key >> 21], 1u);
    else if (PASS == 1) { if ((key >> 21) == prefix) atomicAdd(&sh[(key >> 10) & 0x7ffu], 1u); }
    else { if ((key >> 10) == prefix) atomicAdd(&sh[key & 0x3ffu], 1u); }
  }
  __syncthreads();
  if (skip) return;
  for (int i = threadIdx.x; i < BINS; i += TK_THREADS)
    if (sh[i]) atomicAdd(&hist[(int64_t)seg * BINS + i], sh[i]);
}

// One block per segment: pick the bin that holds the k_rem-th largest key, refine prefix / k_rem, clear hist.
template <int PASS>
__global__ void __launch_bounds__(TK_THREADS) topk_select_kernel(const int64_t* __restrict__ tab, SegState* __restrict__ state,
                                                                 uint32_t* __restrict__ hist) {
  __shared__ uint32_t part[TK_THREADS];
  __shared__ int chosen;
  __shared__ uint32_t above;
  int seg = blockIdx.x;
  const int64_t* t = tab + (int64_t)seg * SEG_FIELDS;
  int64_t len = t[1], k = t[2];
  uint32_t* h = hist + (int64_t)seg * BINS;
  constexpr int PER = BINS / TK_THREADS;     // 8 consecutive bins per thread, thread 0 owns the TOP bins
  int top = BINS - 1 - threadIdx.x * PER;
  uint32_t local[PER], sum = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) { local[j] = h[top - j]; sum += local[j]; h[top - j] = 0; }
  part[threadIdx.x] = sum;
  if (threadIdx.x == 0) { chosen = -1; above = 0; }
  __syncthreads();
  if (k >= len) {
    if (threadIdx.x == 0 && PASS == 0) { state[seg].prefix = 0; state[seg].k_rem = (int32_t)k; state[seg].gt_count = 0; state[seg].eq_count = 0; }
    return;
  }
  // exclusive prefix over threads (= number of keys in higher bins than this thread's first bin)
  uint32_t excl = 0;
  for (int i = 0; i < (int)threadIdx.x; ++i) excl += part[i];
  int32_t k_rem = PASS == 0 ? (int32_t)k : state[seg].k_rem;
  uint32_t run = excl;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    if (run < (uint32_t)k_rem && run + local[j] >= (uint32_t)k_rem) { chosen = top - j; above = run; }
    run += local[j];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int b = chosen < 0 ? 0 : chosen;
    uint32_t prev = PASS == 0 ? 0u : state[seg].prefix;
    state[seg].prefix = PASS == 0 ? (uint32_t)b : (PASS == 1 ? ((prev << 11) | (uint32_t)b) : ((prev << 10) | (uint32_t)b));
    state[seg].k_rem = k_rem - (int32_t)above;
    if (PASS == 0) { state[seg].gt_count = 0; state[seg].eq_count = 0; }
  }
}

// Compaction: (global index, value) of the selected entries -> out lists; selected entries of e are zeroed.
__global__ void __launch_bounds__(TK_THREADS) topk_compact_kernel(const float* __restrict__ g, float* __restrict__ e,
                                                                  const int64_t* __restrict__ tab, int n_seg,
                                                                  SegState* __restrict__ state, int32_t* __restrict__ out_idx,
                                                                  float* __restrict__ out_val) {
  int seg = find_seg(tab, n_seg, (int64_t)blockIdx.x);
  const int64_t* t = tab + (int64_t)seg * SEG_FIELDS;
  int64_t start = t[0], len = t[1], k = t[2], out_off = t[3];
  int64_t c0 = ((int64_t)blockIdx.x - t[4]) * CHUNK;
  int64_t c1 = c0 + CHUNK < len ? c0 + CHUNK : len;
  bool all = k >= len;
  uint32_t thr = state[seg].prefix;
  int32_t need_eq = state[seg].k_rem;
  int64_t n_gt = k - need_eq;
  const int lane = threadIdx.x & 31;
  for (int64_t ib = c0; ib < c1; ib += TK_THREADS) {       // uniform trip count: the ballots below need whole warps
    int64_t i = ib + threadIdx.x;
    bool valid = i < c1;
    float a = 0.f;
    if (valid) a = e != nullptr ? e[start + i] : g[start + i];
    int64_t slot = -1;
    if (all) {
      if (valid) slot = i;
    } else {
      uint32_t key = key_of(a);
      bool gt = valid && key > thr, eq = valid && key == thr;
      // warp-aggregated slot allocation: one atomic per warp and class instead of one per selected element
      unsigned mgt = __ballot_sync(0xffffffffu, gt), meq = __ballot_sync(0xffffffffu, eq);
      uint32_t base_gt = 0, base_eq = 0;
      if (lane == 0) {
        if (mgt) base_gt = atomicAdd(&state[seg].gt_count, (uint32_t)__popc(mgt));
        if (meq) base_eq = atomicAdd(&state[seg].eq_count, (uint32_t)__popc(meq));
      }
      base_gt = __shfl_sync(0xffffffffu, base_gt, 0);
      base_eq = __shfl_sync(0xffffffffu, base_eq, 0);
      unsigned below = (1u << lane) - 1u;
      if (gt) slot = (int64_t)base_gt + __popc(mgt & below);
      else if (eq) {
        uint32_t q = base_eq + (uint32_t)__popc(meq & below);
        if ((int32_t)q < need_eq) slot = n_gt + q;
      }
    }
    if (slot >= 0) {
      out_idx[out_off + slot] = (int32_t)(start + i);
      out_val[out_off + slot] = a;
      if (e != nullptr) e[start + i] = 0.0f;
    }
  }
}

}  // namespace

extern "C" {

int64_t gc_cuda_topk_state_bytes(int n_seg) { return (int64_t)n_seg * (sizeof(SegState) + BINS * 4); }
int gc_cuda_topk_chunk() { return CHUNK; }

// g: gradient (read only); e: error memory (updated in place; NULL = no error feedback, selection on g).
// state: gc_cuda_topk_state_bytes(n_seg) bytes, zeroed once after allocation.  out_idx / out_val: sum of k entries.
int gc_cuda_topk_select(const float* g, float* e, const int64_t* tab, int n_seg, int64_t total_chunks, void* state_,
                        int32_t* out_idx, float* out_val, void* cs) {
  if (n_seg <= 0 || total_chunks <= 0) return 0;
  cudaStream_t st = (cudaStream_t)cs;
  SegState* state = (SegState*)state_;
  uint32_t* hist = (uint32_t*)((uint8_t*)state_ + (int64_t)n_seg * sizeof(SegState));
  unsigned grid = (unsigned)total_chunks;
  topk_hist_kernel<0><<<grid, TK_THREADS, 0, st>>>(g, e, tab, n_seg, state, hist);
  topk_select_kernel<0><<<n_seg, TK_THREADS, 0, st>>>(tab, state, hist);
  topk_hist_kernel<1><<<grid, TK_THREADS, 0, st>>>(g, e, tab, n_seg, state, hist);
  topk_select_kernel<1><<<n_seg, TK_THREADS, 0, st>>>(tab, state, hist);
  topk_hist_kernel<2><<<grid, TK_THREADS, 0, st>>>(g, e, tab, n_seg, state, hist);
  topk_select_kernel<2><<<n_seg, TK_THREADS, 0, st>>>(tab, state, hist);
  topk_compact_kernel<<<grid, TK_THREADS, 0, st>>>(g, e, tab, n_seg, state, out_idx, out_val);
  return (int)cudaGetLastError();
}

}  // extern "C"
