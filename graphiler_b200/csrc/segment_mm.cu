// Typed linear (segment matrix multiply) for sm_100a: y[p_t:p_{t+1}] = x[p_t:p_{t+1}] @ w[t].
//
// One launch covers every type: the grid is sized for the worst case (ceil(m/TM) + n_types
// row tiles) and each block finds its (type, row tile) by walking the device-resident type
// pointer, so the pointer is never copied to the host.  Row tiles never straddle a type
// boundary.  Optional row gather (x[gather_idx[i]]) fuses the node->edge broadcast that
// precedes the edge-typed linear.  This file holds the exact-fp32 SIMT path (shared-memory
// tiled, 4x4 register blocking, products and sums in double), the fallback for
// shapes the tensor-core kernel does not take, and the kernel for narrow weights (K <= 64,
// N <= 32: a relation matrix of a few KB), where a 128-row tensor-core tile is mostly padding and
// per-tile latency: one thread per (row, four output columns), the type's weights widened to
// double in shared memory, products and sums in double (exact products, 2^-53 per addition),
// one rounding to float at the end.  That path is bound by the rows it reads and writes.
#include "common.cuh"

namespace gphl {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256) segment_mm_simt_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                              const int32_t *__restrict__ ptr, int32_t n_types,
                                                              int64_t m, int32_t K, int32_t N,
                                                              const int64_t *__restrict__ gather,
                                                              float *__restrict__ y) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  __shared__ int s_seg, s_row0, s_rows;
  const int tid = threadIdx.x;
  if (tid < 32) {
    // which (type, row tile) is this block?  32 types per step: tile counts, warp prefix sum, one hit
    const int lane = tid;
    const int64_t b = blockIdx.x;
    if (lane == 0) s_rows = 0;
    __syncwarp();
    int64_t base = 0;
    for (int t0 = 0; t0 < n_types; t0 += 32) {
      const int t = t0 + lane;
      const int lo = t < n_types ? __ldg(ptr + t) : 0, hi = t < n_types ? __ldg(ptr + t + 1) : lo;
      const int nt = (hi - lo + TM - 1) / TM;
      int incl = nt;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(FULL, incl, d);
        if (lane >= d) incl += v;
      }
      const bool hit = t < n_types && b >= base + incl - nt && b < base + incl;
      if (hit) {
        s_seg = t;
        s_row0 = lo + (int)(b - (base + incl - nt)) * TM;
        s_rows = min(TM, hi - s_row0);
      }
      if (__any_sync(FULL, hit)) break;
      base += __shfl_sync(FULL, incl, 31);
    }
  }
  __syncthreads();
  const int rows = s_rows;
  if (rows == 0) return;
  const int seg = s_seg, row0 = s_row0;
  const int n0 = blockIdx.y * TN;
  const int tx = tid & 15, ty = tid >> 4;
  const float *wt = w + (int64_t)seg * K * N;

  double acc[4][4];   // a plain fp32 chain of a few hundred products misses atol 1e-6 now and then; products of fp32
                      // values are exact in double and each addition errs by 2^-53
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;

  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / TK, kk = e % TK;
      float v = 0.f;
      if (r < rows && k0 + kk < K) {
        const int64_t srow = gather ? __ldg(gather + row0 + r) : (int64_t)(row0 + r);
        v = __ldg(x + srow * K + k0 + kk);
      }
      As[kk][r] = v;
      const int kb = e / TN, c = e % TN;
      float u = 0.f;
      if (k0 + kb < K && n0 + c < N) u = __ldg(wt + (int64_t)(k0 + kb) * N + n0 + c);
      Bs[kb][c] = u;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      double a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = (double)As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = (double)Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c < N) y[(int64_t)(row0 + r) * N + c] = (float)acc[i][j];
    }
  }
}

constexpr int NK_MAX = 64, NN_MAX = 32;

// Shared block-to-tile lookup of this file's kernels: 32 types per step, tile counts, warp prefix sum, one hit.
// Called by warp 0; leaves rows == 0 for a block beyond the last tile.
__device__ __forceinline__ void find_tile(const int32_t *ptr, int32_t n_types, int tile_rows, int64_t b, int lane,
                                          int &seg, int &row0, int &rows) {
  int64_t base = 0;
  for (int t0 = 0; t0 < n_types; t0 += 32) {
    const int t = t0 + lane;
    const int lo = t < n_types ? __ldg(ptr + t) : 0, hi = t < n_types ? __ldg(ptr + t + 1) : lo;
    const int nt = (hi - lo + tile_rows - 1) / tile_rows;
    int incl = nt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(FULL, incl, d);
      if (lane >= d) incl += v;
    }
    const bool hit = t < n_types && b >= base + incl - nt && b < base + incl;
    if (hit) {
      seg = t;
      row0 = lo + (int)(b - (base + incl - nt)) * tile_rows;
      rows = min(tile_rows, hi - row0);
    }
    if (__any_sync(FULL, hit)) break;
    base += __shfl_sync(FULL, incl, 31);
  }
}

// groups = ceil(N / 4) threads per row; every thread carries NR rows (a weight read from shared memory then serves
// NR rows: with one row per thread the kernel is bound by shared-memory bandwidth); NR * 256 / groups rows per tile.
template <int NR>
__global__ void __launch_bounds__(256) segment_mm_narrow_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                                const int32_t *__restrict__ ptr, int32_t n_types,
                                                                int32_t K, int32_t N, int32_t groups, int32_t tile_rows,
                                                                const int64_t *__restrict__ gather,
                                                                float *__restrict__ y) {
  __shared__ __align__(16) double Ws[NK_MAX][NN_MAX];
  __shared__ int s_seg, s_row0, s_rows;
  const int tid = threadIdx.x;
  if (tid == 0) s_rows = 0;
  __syncthreads();
  if (tid < 32) {
    int seg = 0, row0 = 0, rows = 0;
    find_tile(ptr, n_types, tile_rows, blockIdx.x, tid, seg, row0, rows);
    if (rows > 0) s_seg = seg, s_row0 = row0, s_rows = rows;    // written by the one lane that hit
  }
  __syncthreads();
  const int rows = s_rows;
  if (rows == 0) return;
  const int seg = s_seg, row0 = s_row0;
  const float *wt = w + (int64_t)seg * K * N;
  const int npad = groups * 4;
  for (int e = tid; e < K * npad; e += 256) {
    const int k = e / npad, c = e % npad;
    Ws[k][c] = c < N ? (double)__ldg(wt + (int64_t)k * N + c) : 0.0;
  }
  __syncthreads();
  const int rstep = 256 / groups;                 // rows covered by one pass of the block
  const int r0 = tid / groups, c0 = (tid % groups) * 4;
  if (r0 >= rstep) return;                         // 256 % groups leftover threads
  const bool xvec = (K & 3) == 0 && aligned16_dev(x);
  const bool yvec = (N & 3) == 0 && aligned16_dev(y);
  // the tile is many passes long, so that finding it and staging the weights is paid once per few thousand rows
  for (int rbase = 0; rbase < rows; rbase += rstep * NR) {
    const float *xr[NR];
    bool rok[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
      const int r = rbase + r0 + j * rstep;
      rok[j] = r < rows;
      const int64_t srow = rok[j] ? (gather ? __ldg(gather + row0 + r) : (int64_t)(row0 + r)) : 0;
      xr[j] = x + srow * K;
    }
    double acc[NR][4];
#pragma unroll
    for (int j = 0; j < NR; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[j][q] = 0.0;
    for (int k0 = 0; k0 < K; k0 += 4) {
      float xv[NR][4];
#pragma unroll
      for (int j = 0; j < NR; ++j) {
        if (xvec) {
          const float4 t = rok[j] ? __ldg(reinterpret_cast<const float4 *>(xr[j] + k0)) : make_float4(0.f, 0.f, 0.f, 0.f);
          xv[j][0] = t.x, xv[j][1] = t.y, xv[j][2] = t.z, xv[j][3] = t.w;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) xv[j][i] = (rok[j] && k0 + i < K) ? __ldg(xr[j] + k0 + i) : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (k0 + i >= K) break;
        const double2 w01 = *reinterpret_cast<const double2 *>(&Ws[k0 + i][c0]);
        const double2 w23 = *reinterpret_cast<const double2 *>(&Ws[k0 + i][c0 + 2]);
#pragma unroll
        for (int j = 0; j < NR; ++j) {
          const double xd = (double)xv[j][i];
          acc[j][0] = fma(xd, w01.x, acc[j][0]), acc[j][1] = fma(xd, w01.y, acc[j][1]);
          acc[j][2] = fma(xd, w23.x, acc[j][2]), acc[j][3] = fma(xd, w23.y, acc[j][3]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
      if (!rok[j]) continue;
      float *yr = y + (int64_t)(row0 + rbase + r0 + j * rstep) * N + c0;
      if (yvec) {
        *reinterpret_cast<float4 *>(yr) = make_float4((float)acc[j][0], (float)acc[j][1], (float)acc[j][2], (float)acc[j][3]);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (c0 + q < N) yr[q] = (float)acc[j][q];
      }
    }
  }
}

}  // namespace gphl

using namespace gphl;

extern "C" int gphl_segment_mm_f32(const float *x, const float *w, const int32_t *type_pointer, int64_t n_types,
                                   int64_t m, int64_t k, int64_t n, const int64_t *gather_idx, float *y,
                                   void *stream_) {
  GPHL_REQUIRE(n_types >= 0 && m >= 0 && k >= 0 && n >= 0, "negative size");
  GPHL_REQUIRE(m < INT32_MAX && k < (1 << 20) && n < (1 << 20) && n_types < (1 << 24), "size out of range");
  if (m == 0 || n == 0 || n_types == 0) return GPHL_OK;
  GPHL_REQUIRE(x && w && type_pointer && y, "null pointer argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (k >= 1 && k <= NK_MAX && n <= NN_MAX) {
    // two rows per thread and tiles of a few passes measured best on a 10^6 x 16 x 16 relation-typed linear
    // (one row: shared-memory reads dominate; four: too few resident warps for the row gathers)
    constexpr int nr = 2;
    const int32_t groups = (int32_t)((n + 3) / 4), pass_rows = nr * (256 / groups);
    const int64_t passes = std::min<int64_t>(8, std::max<int64_t>(1, m / (148LL * 8 * pass_rows)));
    const int32_t tile_rows = (int32_t)(passes * pass_rows);
    const int64_t tiles = (m + tile_rows - 1) / tile_rows + n_types;
    GPHL_REQUIRE(tiles <= 2147483647LL, "too many tiles");
    segment_mm_narrow_kernel<nr><<<(unsigned)tiles, 256, 0, stream>>>(x, w, type_pointer, (int32_t)n_types, (int32_t)k,
                                                                     (int32_t)n, groups, tile_rows, gather_idx, y);
    return launched("segment_mm_narrow_kernel");
  }
  const int64_t tiles = (m + TM - 1) / TM + n_types;
  dim3 grid((unsigned)tiles, (unsigned)((n + TN - 1) / TN));
  segment_mm_simt_kernel<<<grid, 256, 0, stream>>>(x, w, type_pointer, (int32_t)n_types, m, (int32_t)k, (int32_t)n,
                                                   gather_idx, y);
  return launched("segment_mm_simt_kernel");
}
