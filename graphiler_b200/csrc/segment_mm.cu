// Typed linear (segment matrix multiply) for sm_100a: y[p_t:p_{t+1}] = x[p_t:p_{t+1}] @ w[t].
//
// One launch covers every type: the grid is sized for the worst case (ceil(m/TM) + n_types
// row tiles) and each block finds its (type, row tile) by walking the device-resident type
// pointer, so the pointer is never copied to the host.  Row tiles never straddle a type
// boundary.  Optional row gather (x[gather_idx[i]]) fuses the node->edge broadcast that
// precedes the edge-typed linear.  This file holds the exact-fp32 SIMT path (shared-memory
// tiled, 4x4 register blocking, exact-product compensated accumulation); it is the fallback for
// shapes the tensor-core kernel does not take.
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

  Acc acc[4][4];   // compensated: a plain fp32 chain of a few hundred products misses atol 1e-6 now and then
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j].hi = 0.f, acc[i][j].lo = 0.f;

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
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j].fma_exact(a[i], b[j]);
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
      if (c < N) y[(int64_t)(row0 + r) * N + c] = acc[i][j].value();
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
  const int64_t tiles = (m + TM - 1) / TM + n_types;
  dim3 grid((unsigned)tiles, (unsigned)((n + TN - 1) / TN));
  segment_mm_simt_kernel<<<grid, 256, 0, stream>>>(x, w, type_pointer, (int32_t)n_types, m, (int32_t)k, (int32_t)n,
                                                   gather_idx, y);
  return launched("segment_mm_simt_kernel");
}
