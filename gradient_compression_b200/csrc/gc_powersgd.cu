// PowerSGD rank-r pipeline on the flat gradient (reference: reducer.py:1718-1858, there ~5 Python loops
// over 54 layers of cuBLAS GEMV calls and ~5 tiny kernels per Gram-Schmidt column):
//   psgd_p     P = (G + E) Q for every matrix in ONE launch (warp per matrix row); E <- G + E in place;
//              1-D tensors are packed behind P so that one exchange carries both
//   psgd_gs    classical Gram-Schmidt of every P in one launch (block per matrix)
//   psgd_q     Q' = M^T P for every matrix in one launch (block per 128-column tile, no atomics)
//   psgd_out   G <- P Q'^T, E <- M - P Q'^T; 1-D tensors get the plain mean
// All products are bandwidth-bound at r <= 4 (each streams the 94 MB gradient once), so they run on the
// CUDA cores with 16-byte loads; the two all-reduces in between use the one-shot peer-memory sum.
// Matrix table: int64 rows of {off, n, m, r, p_off, q_off, row_start, tile_start}.
// Vector table: int64 rows of {off, len, dst}.
#include <cuda_runtime.h>
#include <stdint.h>

#include "gc_device.cuh"

using namespace gc;

namespace {

constexpr int RMAX = 4;
constexpr int MAT_FIELDS = 8;

struct Mat { int64_t off; int n, m, r; int64_t p_off, q_off; };

__device__ __forceinline__ Mat load_mat(const int64_t* __restrict__ tab, int i) {
  const int64_t* t = tab + (int64_t)i * MAT_FIELDS;
  Mat m;
  m.off = t[0]; m.n = (int)t[1]; m.m = (int)t[2]; m.r = (int)t[3]; m.p_off = t[4]; m.q_off = t[5];
  return m;
}

// Largest i with tab[i][field] <= key.
__device__ __forceinline__ int find_mat(const int64_t* __restrict__ tab, int n_mats, int field, int64_t key) {
  int lo = 0, hi = n_mats - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (tab[(int64_t)mid * MAT_FIELDS + field] <= key) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// ------------------------------------------------------------------------------------------ P = (G + E) Q
// acc[j] += sum_t v[t] * q[(k + t) * R + j] with the 4 * R query values fetched by 16-byte loads.
template <int R>
__device__ __forceinline__ void dot4(const float (&v)[4], const float* __restrict__ qk, float (&acc)[RMAX]) {
  if (R == 1) {
    float4 q = *reinterpret_cast<const float4*>(qk);
    acc[0] = fmaf(v[0], q.x, fmaf(v[1], q.y, fmaf(v[2], q.z, fmaf(v[3], q.w, acc[0]))));
  } else if (R == 2) {
    float4 a = *reinterpret_cast<const float4*>(qk), b = *reinterpret_cast<const float4*>(qk + 4);
    acc[0] = fmaf(v[0], a.x, fmaf(v[1], a.z, fmaf(v[2], b.x, fmaf(v[3], b.z, acc[0]))));
    acc[1] = fmaf(v[0], a.y, fmaf(v[1], a.w, fmaf(v[2], b.y, fmaf(v[3], b.w, acc[1]))));
  } else if (R == 4) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float4 q = *reinterpret_cast<const float4*>(qk + 4 * t);
      acc[0] = fmaf(v[t], q.x, acc[0]); acc[1] = fmaf(v[t], q.y, acc[1]);
      acc[2] = fmaf(v[t], q.z, acc[2]); acc[3] = fmaf(v[t], q.w, acc[3]);
    }
  } else {
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int j = 0; j < R; ++j) acc[j] = fmaf(v[t], qk[t * R + j], acc[j]);
  }
}

template <int R>
__device__ __forceinline__ void p_row_vec(const float* __restrict__ g, float* __restrict__ e, int64_t base, int m,
                                          const float* __restrict__ qm, int lane, float (&acc)[RMAX]) {
  int k = lane * 4;
  for (; k + 128 < m; k += 256) {     // two independent 512-byte pieces of the row per iteration
    float4 a0 = *reinterpret_cast<const float4*>(g + base + k), b0 = *reinterpret_cast<const float4*>(e + base + k);
    float4 a1 = *reinterpret_cast<const float4*>(g + base + k + 128), b1 = *reinterpret_cast<const float4*>(e + base + k + 128);
    a0.x += b0.x; a0.y += b0.y; a0.z += b0.z; a0.w += b0.w;
    a1.x += b1.x; a1.y += b1.y; a1.z += b1.z; a1.w += b1.w;
    *reinterpret_cast<float4*>(e + base + k) = a0;
    *reinterpret_cast<float4*>(e + base + k + 128) = a1;
    float v0[4] = {a0.x, a0.y, a0.z, a0.w}, v1[4] = {a1.x, a1.y, a1.z, a1.w};
    dot4<R>(v0, qm + (int64_t)k * R, acc);
    dot4<R>(v1, qm + (int64_t)(k + 128) * R, acc);
  }
  for (; k < m; k += 128) {
    float4 a = *reinterpret_cast<const float4*>(g + base + k), b = *reinterpret_cast<const float4*>(e + base + k);
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    *reinterpret_cast<float4*>(e + base + k) = a;
    float v[4] = {a.x, a.y, a.z, a.w};
    dot4<R>(v, qm + (int64_t)k * R, acc);
  }
}

__global__ void __launch_bounds__(256) psgd_p_kernel(const float* __restrict__ g, float* __restrict__ e,
                                                     const int64_t* __restrict__ tab, int n_mats, int64_t total_rows,
                                                     const float* __restrict__ q, float* __restrict__ p) {
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row_g = warp; row_g < total_rows; row_g += nwarps) {
    int mi = find_mat(tab, n_mats, 6, row_g);
    Mat mt = load_mat(tab, mi);
    int row = (int)(row_g - tab[(int64_t)mi * MAT_FIELDS + 6]);
    int64_t base = mt.off + (int64_t)row * mt.m;
    const float* qm = q + mt.q_off;
    float acc[RMAX] = {0.f, 0.f, 0.f, 0.f};
    // 16-byte path: row start, row length and the query block must all be 16-byte aligned
    bool vec = ((base & 3) == 0) && ((mt.m & 3) == 0) && ((mt.q_off & 3) == 0);
    if (vec && mt.r == 1) p_row_vec<1>(g, e, base, mt.m, qm, lane, acc);
    else if (vec && mt.r == 2) p_row_vec<2>(g, e, base, mt.m, qm, lane, acc);
    else if (vec && mt.r == 4) p_row_vec<4>(g, e, base, mt.m, qm, lane, acc);
    else {
      for (int k = lane; k < mt.m; k += 32) {
        float a = g[base + k] + e[base + k];
        e[base + k] = a;
        for (int j = 0; j < mt.r; ++j) acc[j] = fmaf(a, qm[(int64_t)k * mt.r + j], acc[j]);
      }
    }
    for (int j = 0; j < mt.r; ++j) {
      float s = warp_sum(acc[j]);
      if (lane == 0) p[mt.p_off + (int64_t)row * mt.r + j] = s;
    }
  }
}

// 1-D tensors: stage[dst + i] = g[off + i] (their error memory is identically zero).
__global__ void psgd_pack_vec_kernel(const float* __restrict__ g, const int64_t* __restrict__ vtab, int n_vecs,
                                     float* __restrict__ stage) {
  for (int v = blockIdx.x; v < n_vecs; v += gridDim.x) {
    int64_t off = vtab[v * 3], len = vtab[v * 3 + 1], dst = vtab[v * 3 + 2];
    for (int64_t i = threadIdx.x; i < len; i += blockDim.x) stage[dst + i] = g[off + i];
  }
}

// ------------------------------------------------------------------------------------------ Gram-Schmidt
__global__ void __launch_bounds__(256) psgd_gs_kernel(float* __restrict__ p, const int64_t* __restrict__ tab, float eps) {
  __shared__ float smem[32];
  Mat mt = load_mat(tab, blockIdx.x);
  float* pm = p + mt.p_off;
  for (int i = 0; i < mt.r; ++i) {
    float ss = 0.f;
    for (int row = threadIdx.x; row < mt.n; row += blockDim.x) { float v = pm[(int64_t)row * mt.r + i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, smem);
    float inv = 1.0f / (sqrtf(ss) + eps);
    __syncthreads();
    for (int row = threadIdx.x; row < mt.n; row += blockDim.x) pm[(int64_t)row * mt.r + i] *= inv;
    __syncthreads();
    for (int j = i + 1; j < mt.r; ++j) {
      float dot = 0.f;
      for (int row = threadIdx.x; row < mt.n; row += blockDim.x)
        dot = fmaf(pm[(int64_t)row * mt.r + i], pm[(int64_t)row * mt.r + j], dot);
      dot = block_sum(dot, smem);
      __syncthreads();
      for (int row = threadIdx.x; row < mt.n; row += blockDim.x)
        pm[(int64_t)row * mt.r + j] = fmaf(-dot, pm[(int64_t)row * mt.r + i], pm[(int64_t)row * mt.r + j]);
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------------------------------ Q' = M^T P
// Block = one 128-column tile of one matrix; thread (c = tid % 32, rl = tid / 32) owns columns 4c..4c+3 of the
// tile and rows rl, rl + 8, ...; the eight row lanes are combined through shared memory in a fixed order.
constexpr int Q_ROWCHUNK = 256;    // rows per block along grid.y (1024 left ResNet-50 with ~700 blocks at 1.3 TB/s)

__global__ void __launch_bounds__(256) psgd_q_kernel(const float* __restrict__ e /* holds M = G + E */,
                                                     const int64_t* __restrict__ tab, int n_mats,
                                                     const float* __restrict__ p, float* __restrict__ qout,
                                                     int64_t q_total) {
  __shared__ float red[8][32][4 * RMAX];
  int mi = find_mat(tab, n_mats, 7, (int64_t)blockIdx.x);
  Mat mt = load_mat(tab, mi);
  // the table counts, per matrix, column tiles x row chunks (a grid over tiles x the largest chunk count left two thirds of
  // ResNet-50's blocks without rows: 57 us for a 94 MB read)
  const int local = (int)((int64_t)blockIdx.x - tab[(int64_t)mi * MAT_FIELDS + 7]);
  const int tiles_m = (mt.m + 127) / 128;
  const int tile = local % tiles_m, chunk = local / tiles_m;
  int c = threadIdx.x & 31, rl = threadIdx.x >> 5;
  int k0 = tile * 128 + c * 4;
  float acc[4][RMAX];
#pragma unroll
  for (int t = 0; t < 4; ++t)
#pragma unroll
    for (int j = 0; j < RMAX; ++j) acc[t][j] = 0.f;
  const float* pm = p + mt.p_off;
  bool vec = ((mt.off & 3) == 0) && ((mt.m & 3) == 0);
  const int row_lo = chunk * Q_ROWCHUNK;
  const int row_hi = row_lo + Q_ROWCHUNK < mt.n ? row_lo + Q_ROWCHUNK : mt.n;
  float* qdst = qout + (int64_t)chunk * q_total;          // chunk y writes its own partial copy (copies of chunks a matrix
                                                          // does not have stay zero: the buffer is zeroed once)
  if (k0 < mt.m) {
    if (vec) {
      // four rows (8 apart) per iteration: four independent 16-byte loads in flight per thread
      for (int row = row_lo + rl; row < row_hi; row += 32) {
        float4 a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          int rr = row + 8 * u;
          a[u] = rr < row_hi ? *reinterpret_cast<const float4*>(e + mt.off + (int64_t)rr * mt.m + k0) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          int rr = row + 8 * u;
          if (rr >= row_hi) break;
          float v[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
          for (int j = 0; j < mt.r; ++j) {
            float pv = pm[(int64_t)rr * mt.r + j];
#pragma unroll
            for (int t = 0; t < 4; ++t) acc[t][j] = fmaf(v[t], pv, acc[t][j]);
          }
        }
      }
    } else {
      for (int row = row_lo + rl; row < row_hi; row += 8) {
        float v[4];
        int64_t base = mt.off + (int64_t)row * mt.m + k0;
#pragma unroll
        for (int t = 0; t < 4; ++t) v[t] = (k0 + t < mt.m) ? e[base + t] : 0.f;
        for (int j = 0; j < mt.r; ++j) {
          float pv = pm[(int64_t)row * mt.r + j];
#pragma unroll
          for (int t = 0; t < 4; ++t) acc[t][j] = fmaf(v[t], pv, acc[t][j]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 4; ++t)
#pragma unroll
    for (int j = 0; j < RMAX; ++j) red[rl][c][t * RMAX + j] = acc[t][j];
  __syncthreads();
  if (rl == 0 && k0 < mt.m) {
    for (int t = 0; t < 4 && k0 + t < mt.m; ++t)
      for (int j = 0; j < mt.r; ++j) {
        float s = 0.f;
#pragma unroll
        for (int l = 0; l < 8; ++l) s += red[l][c][t * RMAX + j];
        qdst[mt.q_off + (int64_t)(k0 + t) * mt.r + j] = s;
      }
  }
}

// Sum of the row-chunk partials (only launched when some matrix has more than Q_ROWCHUNK rows).
__global__ void psgd_q_sum_kernel(float* __restrict__ q, int64_t q_total, int chunks) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < q_total; i += stride) {
    float s = q[i];
    for (int c = 1; c < chunks; ++c) s += q[(int64_t)c * q_total + i];
    q[i] = s;
  }
}

// ------------------------------------------------------------------------------------------ G = P Q'^T ; E = M - G
__global__ void __launch_bounds__(256) psgd_out_kernel(float* __restrict__ g, float* __restrict__ e,
                                                       const int64_t* __restrict__ tab, int n_mats, int64_t total_rows,
                                                       const float* __restrict__ p, const float* __restrict__ q) {
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row_g = warp; row_g < total_rows; row_g += nwarps) {
    int mi = find_mat(tab, n_mats, 6, row_g);
    Mat mt = load_mat(tab, mi);
    int row = (int)(row_g - tab[(int64_t)mi * MAT_FIELDS + 6]);
    int64_t base = mt.off + (int64_t)row * mt.m;
    const float* qm = q + mt.q_off;
    float pr[RMAX] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < mt.r; ++j) pr[j] = p[mt.p_off + (int64_t)row * mt.r + j];
    bool vec = ((base & 3) == 0) && ((mt.m & 3) == 0) && ((mt.q_off & 3) == 0) && (mt.r == 1 || mt.r == 2 || mt.r == 4);
    if (vec) {
      for (int k = lane * 4; k < mt.m; k += 128) {
        float o[4];
        const float* qk = qm + (int64_t)k * mt.r;
        if (mt.r == 1) {
          float4 q0 = *reinterpret_cast<const float4*>(qk);
          o[0] = pr[0] * q0.x; o[1] = pr[0] * q0.y; o[2] = pr[0] * q0.z; o[3] = pr[0] * q0.w;
        } else if (mt.r == 2) {
          float4 q0 = *reinterpret_cast<const float4*>(qk), q1 = *reinterpret_cast<const float4*>(qk + 4);
          o[0] = fmaf(pr[1], q0.y, pr[0] * q0.x); o[1] = fmaf(pr[1], q0.w, pr[0] * q0.z);
          o[2] = fmaf(pr[1], q1.y, pr[0] * q1.x); o[3] = fmaf(pr[1], q1.w, pr[0] * q1.z);
        } else {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            float4 qq = *reinterpret_cast<const float4*>(qk + 4 * t);
            o[t] = fmaf(pr[3], qq.w, fmaf(pr[2], qq.z, fmaf(pr[1], qq.y, pr[0] * qq.x)));
          }
        }
        float4 mv = *reinterpret_cast<const float4*>(e + base + k);
        *reinterpret_cast<float4*>(g + base + k) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4*>(e + base + k) = make_float4(mv.x - o[0], mv.y - o[1], mv.z - o[2], mv.w - o[3]);
      }
    } else {
      for (int k = lane; k < mt.m; k += 32) {
        float s = 0.f;
        for (int j = 0; j < mt.r; ++j) s = fmaf(pr[j], qm[(int64_t)k * mt.r + j], s);
        g[base + k] = s;
        e[base + k] -= s;
      }
    }
  }
}

// 1-D tensors: g[off + i] = alpha * summed[dst + i]; their error memory stays zero.
__global__ void psgd_unpack_vec_kernel(float* __restrict__ g, float* __restrict__ e, const int64_t* __restrict__ vtab,
                                       int n_vecs, const float* __restrict__ summed, float alpha) {
  for (int v = blockIdx.x; v < n_vecs; v += gridDim.x) {
    int64_t off = vtab[v * 3], len = vtab[v * 3 + 1], dst = vtab[v * 3 + 2];
    for (int64_t i = threadIdx.x; i < len; i += blockDim.x) {
      g[off + i] = alpha * summed[dst + i];
      e[off + i] = 0.f;
    }
  }
}

int psgd_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

}  // namespace

extern "C" {

int gc_cuda_psgd_max_rank() { return RMAX; }

// stage = [P (p_total floats) | packed 1-D tensors]; e <- g + e for the matrices.
int gc_cuda_psgd_p(const float* g, float* e, const int64_t* tab, int n_mats, int64_t total_rows, const float* q,
                   float* stage, const int64_t* vtab, int n_vecs, int64_t vec_base, void* cs) {
  cudaStream_t st = (cudaStream_t)cs;
  if (n_mats > 0 && total_rows > 0) {
    int64_t blocks = (total_rows + 7) / 8;
    int64_t cap = (int64_t)psgd_sms() * 8;
    psgd_p_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, st>>>(g, e, tab, n_mats, total_rows, q, stage);
  }
  if (n_vecs > 0) psgd_pack_vec_kernel<<<n_vecs < 256 ? n_vecs : 256, 512, 0, st>>>(g, vtab, n_vecs, stage + vec_base);
  return (int)cudaGetLastError();
}

int gc_cuda_psgd_gs(float* p, const int64_t* tab, int n_mats, float eps, void* cs) {
  if (n_mats > 0) psgd_gs_kernel<<<n_mats, 256, 0, (cudaStream_t)cs>>>(p, tab, eps);
  return (int)cudaGetLastError();
}

int gc_cuda_psgd_q_chunks(int max_rows) { return (max_rows + Q_ROWCHUNK - 1) / Q_ROWCHUNK; }

// Blocks the Q' kernel runs for an n x m matrix: 128-column tiles x row chunks (the table's tile_start column counts these).
int64_t gc_cuda_psgd_q_blocks(int n, int m) { return (int64_t)((m + 127) / 128) * ((n + Q_ROWCHUNK - 1) / Q_ROWCHUNK); }

// qout must hold gc_cuda_psgd_q_chunks(max_rows) * q_total floats, zeroed once; the result ends up in its first q_total.
// total_tiles: sum over matrices of gc_cuda_psgd_q_blocks(n, m), the same count the table's tile_start column accumulates.
int gc_cuda_psgd_q(const float* e, const int64_t* tab, int n_mats, int64_t total_tiles, const float* p, float* qout,
                   int64_t q_total, int max_rows, void* cs) {
  if (n_mats > 0 && total_tiles > 0) {
    int chunks = gc_cuda_psgd_q_chunks(max_rows);
    psgd_q_kernel<<<dim3((unsigned)total_tiles), 256, 0, (cudaStream_t)cs>>>(e, tab, n_mats, p, qout, q_total);
    if (chunks > 1) {
      int64_t blocks = (q_total + 255) / 256;
      psgd_q_sum_kernel<<<(int)(blocks < 1024 ? blocks : 1024), 256, 0, (cudaStream_t)cs>>>(qout, q_total, chunks);
    }
  }
  return (int)cudaGetLastError();
}

int gc_cuda_psgd_out(float* g, float* e, const int64_t* tab, int n_mats, int64_t total_rows, const float* p,
                     const float* q, const int64_t* vtab, int n_vecs, const float* summed_vecs, float alpha, void* cs) {
  cudaStream_t st = (cudaStream_t)cs;
  if (n_mats > 0 && total_rows > 0) {
    int64_t blocks = (total_rows + 7) / 8;
    int64_t cap = (int64_t)psgd_sms() * 8;
    psgd_out_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, st>>>(g, e, tab, n_mats, total_rows, p, q);
  }
  if (n_vecs > 0)
    psgd_unpack_vec_kernel<<<n_vecs < 256 ? n_vecs : 256, 512, 0, st>>>(g, e, vtab, n_vecs, summed_vecs, alpha);
  return (int)cudaGetLastError();
}

}  // extern "C"
