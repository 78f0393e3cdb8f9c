// Edge-parallel SDDMM kernels for sm_100a: u_add_v and u_dot_v over the COO arrays.
//
// One thread produces one 16-byte output vector (u_add_v) or one (edge, head) dot product
// (u_dot_v); consecutive threads own consecutive outputs of the same edge, so the gathered
// reads of one endpoint row and the output writes are contiguous.  Dot products are
// accumulated in double (exact products, 2^-53 per addition) and rounded once.
#include <algorithm>

#include "common.cuh"

namespace gphl {

// `lanes` = min(FV, 256) threads share one edge; a thread's column and edge slot are fixed (two 32-bit divisions per
// thread instead of a 64-bit division per output vector).
template <typename I>
__global__ void __launch_bounds__(256) u_add_v_vec_kernel(const I *__restrict__ src, const I *__restrict__ dst, int64_t n_edges,
                                                          int32_t FV, int32_t lanes, const float4 *__restrict__ l,
                                                          const float4 *__restrict__ r, float4 *__restrict__ z) {
  const int per_block = 256 / lanes;
  const int slot = (int)threadIdx.x / lanes, c0 = (int)threadIdx.x - slot * lanes;
  if (slot >= per_block) return;
  for (int64_t e = (int64_t)blockIdx.x * per_block + slot; e < n_edges; e += (int64_t)gridDim.x * per_block) {
    const float4 *a = l + (int64_t)__ldg(src + e) * FV, *b = r + (int64_t)__ldg(dst + e) * FV;
    float4 *o = z + e * FV;
    for (int c = c0; c < FV; c += lanes) {
      const float4 p = __ldg(a + c), q = __ldg(b + c);
      o[c] = make_float4(p.x + q.x, p.y + q.y, p.z + q.z, p.w + q.w);
    }
  }
}

template <typename I>
__global__ void u_add_v_scalar_kernel(const I *__restrict__ src, const I *__restrict__ dst, int64_t n_edges, int32_t F,
                                      const float *__restrict__ l, const float *__restrict__ r, float *__restrict__ z) {
  const int64_t total = n_edges * F;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = t / F;
    const int c = (int)(t - e * F);
    z[t] = __ldg(l + (int64_t)__ldg(src + e) * F + c) + __ldg(r + (int64_t)__ldg(dst + e) * F + c);
  }
}

template <typename I, bool VEC4>
__global__ void u_dot_v_kernel(const I *__restrict__ src, const I *__restrict__ dst, int64_t n_edges, int32_t H,
                               int32_t D, const float *__restrict__ l, const float *__restrict__ r,
                               float *__restrict__ z) {
  // min(H, 256) threads share an edge; a thread's head and edge slot are fixed (no 64-bit division per output)
  const int lanes = H < 256 ? H : 256, per_block = 256 / lanes;
  const int slot = (int)threadIdx.x / lanes, h0 = (int)threadIdx.x - slot * lanes;
  if (slot >= per_block) return;
  for (int64_t e = (int64_t)blockIdx.x * per_block + slot; e < n_edges; e += (int64_t)gridDim.x * per_block)
  for (int h = h0; h < H; h += lanes) {
    const int64_t t = e * H + h;
    const float *a = l + ((int64_t)__ldg(src + e) * H + h) * D;
    const float *b = r + ((int64_t)__ldg(dst + e) * H + h) * D;
    // products of fp32 values are exact in double and each addition errs by 2^-53: the dot product is exact to the
    // final rounding, with one fused multiply-add per term (the compensated fp32 form takes ten operations)
    double acc = 0.0;
    Acc2 acc2{0, 0};
    if (VEC4) {
      for (int d = 0; d < D; d += 4) {
        const float4 p = __ldg(reinterpret_cast<const float4 *>(a + d));
        const float4 q = __ldg(reinterpret_cast<const float4 *>(b + d));
        acc = fma((double)p.x, (double)q.x, acc), acc = fma((double)p.y, (double)q.y, acc);
        acc2.fma_exact(pack2(p.z, p.w), pack2(q.z, q.w));           // the other half on the fp32 pipe
      }
      float h0, h1, l0, l1;
      unpack2(acc2.hi, h0, h1);
      unpack2(acc2.lo, l0, l1);
      acc += ((double)h0 + (double)h1) + ((double)l0 + (double)l1);
    } else {
      for (int d = 0; d < D; ++d) acc = fma((double)__ldg(a + d), (double)__ldg(b + d), acc);
    }
    z[t] = (float)acc;
  }
}

// u_dot_v with coalesced row reads: a sub-warp group of LPR lanes reads one edge's two endpoint rows, NV consecutive
// 16-byte vectors per lane (all of one head: NV divides the DV = D / 4 vectors of a head), multiplies exactly (half
// of the terms in double, half as compensated fp32 pairs), and the DV / NV lanes that share a head reduce with shuffles.  32 / LPR edges are in flight per
// warp instruction, U per group.
template <typename I, int LPR, int NV>
__global__ void __launch_bounds__(256) u_dot_v_rows_kernel(const I *__restrict__ src, const I *__restrict__ dst,
                                                           int64_t n_edges, int32_t H, int32_t FV, int32_t DV,
                                                           const float4 *__restrict__ l, const float4 *__restrict__ r,
                                                           float *__restrict__ z) {
  constexpr int G = 32 / LPR, U = (NV >= 2) ? 2 : 4;
  const int lane = threadIdx.x & 31, g = lane / LPR, ll = lane % LPR;
  const int cv0 = ll * NV;                                   // first vector of this lane
  const bool cok = cv0 < FV;                                 // FV is a multiple of NV: all or none of the lane's vectors
  const int lanes_per_head = DV / NV;
  const bool writer = cok && (ll % lanes_per_head) == 0;     // hoisted: integer division by a run-time value is dear
  const int my_head = cv0 / DV;
  const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp_id * 32; base < n_edges; base += n_warps * 32) {
    const int n = (n_edges - base) < 32 ? (int)(n_edges - base) : 32;
    int64_t my_s = 0, my_d = 0;
    if (lane < n) my_s = (int64_t)__ldg(src + base + lane), my_d = (int64_t)__ldg(dst + base + lane);
#pragma unroll 1
    for (int jj = 0; jj < n; jj += G * U) {
      float4 a[U][NV], b[U][NV];
      int e[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        e[u] = jj + u * G + g;
        const int64_t s_row = __shfl_sync(FULL, my_s, e[u] & 31), d_row = __shfl_sync(FULL, my_d, e[u] & 31);
        const bool ok = e[u] < n && cok;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          a[u][v] = ok ? __ldg(l + s_row * FV + cv0 + v) : make_float4(0.f, 0.f, 0.f, 0.f);
          b[u][v] = ok ? __ldg(r + d_row * FV + cv0 + v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        // Exact products on both pipes (the fp64 pipe alone bounds this kernel, as the fp32 pipe alone did): the first
        // half of every vector in double (a product of fp32 values is exact there), the second as packed fp32
        // products with their rounding errors in a compensated pair; joined in double.
        double accd = 0.0;
        Acc2 acc2{0, 0};
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          accd = fma((double)a[u][v].x, (double)b[u][v].x, accd), accd = fma((double)a[u][v].y, (double)b[u][v].y, accd);
          acc2.fma_exact(pack2(a[u][v].z, a[u][v].w), pack2(b[u][v].z, b[u][v].w));
        }
        float h0, h1, l0, l1;
        unpack2(acc2.hi, h0, h1);
        unpack2(acc2.lo, l0, l1);
        double acc = accd + (((double)h0 + (double)h1) + ((double)l0 + (double)l1));
#pragma unroll
        for (int off = 1; off < 32; off <<= 1)
          if (off < lanes_per_head) acc += __shfl_xor_sync(FULL, acc, off);      // a power of two <= LPR; uniform condition
        if (e[u] < n && writer) z[(base + e[u]) * H + my_head] = (float)acc;
      }
    }
  }
}

template <typename I, int LPR, int NV>
static int launch_u_dot_v_rows(const I *src, const I *dst, int64_t n_edges, int64_t heads, int64_t fv, int64_t dv,
                               const float *l, const float *r, float *z, cudaStream_t stream) {
  const int64_t warps = (n_edges + 31) / 32;
  const int64_t blocks = std::min<int64_t>((warps + 7) / 8, 148LL * 32);
  u_dot_v_rows_kernel<I, LPR, NV><<<(unsigned)blocks, 256, 0, stream>>>(
      src, dst, n_edges, (int32_t)heads, (int32_t)fv, (int32_t)dv, reinterpret_cast<const float4 *>(l),
      reinterpret_cast<const float4 *>(r), z);
  return launched("u_dot_v_rows_kernel");
}

// u_dot_v in destination-row (CSC) order.  The COO kernels above fetch both endpoint rows for every edge; walking the
// destination segments instead, a warp takes one work item of the row-split plan, keeps its destination row r[v] in
// registers (half of each vector widened to double once, the other half as packed fp32 pairs), and gathers only the
// source rows l[src]: half the gathered bytes, and half the conversions of the exact products.  Results go to
// z[edge id] (scattered by the row's edge ids; contiguous when edge ids are destination-sorted).  Pieces of a cut
// row need no combination: every edge's output is independent.  Lane layout as in u_dot_v_rows_kernel.
template <int LPR, int NV, bool MIX>
__global__ void __launch_bounds__(256) u_dot_v_csc_kernel(const Item *__restrict__ items, int64_t n_items,
                                                          const int32_t *__restrict__ pointer,
                                                          const int32_t *__restrict__ idx, const int32_t *__restrict__ eidx,
                                                          int32_t H, int32_t FV, int32_t DV, const float4 *__restrict__ l,
                                                          const float4 *__restrict__ r, float *__restrict__ z) {
  constexpr int G = 32 / LPR, U = (NV >= 2) ? 2 : 4;
  const int lane = threadIdx.x & 31, g = lane / LPR, ll = lane % LPR;
  const int64_t item_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (item_id >= n_items) return;
  const Item it = fetch_item(items, pointer, item_id);
  const int cv0 = ll * NV;
  const bool cok = cv0 < FV;
  const int lanes_per_head = DV / NV;
  const bool writer = cok && (ll % lanes_per_head) == 0;     // hoisted: integer division by a run-time value is dear
  const int my_head = cv0 / DV;
  // MIX: the second half of every vector as packed fp32 products with compensated errors (the fp32 pipe shares the
  // work); otherwise all four columns in double (one conversion and one fused multiply-add per term)
  double rd[NV][4];
  uint64_t rp[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const float4 q = cok ? __ldg(r + (int64_t)it.row * FV + cv0 + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    rd[v][0] = (double)q.x, rd[v][1] = (double)q.y, rd[v][2] = (double)q.z, rd[v][3] = (double)q.w;
    rp[v] = pack2(q.z, q.w);
  }
  int next_idx = 0, next_eid = 0;
  if (it.begin + lane < it.end) {
    next_idx = __ldg(idx + it.begin + lane);
    next_eid = eidx ? __ldg(eidx + it.begin + lane) : it.begin + lane;
  }
  for (int base = it.begin; base < it.end; base += 32) {
    const int n = min(32, it.end - base);
    const int my_idx = next_idx, my_eid = next_eid;
    if (base + 32 + lane < it.end) {
      next_idx = __ldg(idx + base + 32 + lane);
      next_eid = eidx ? __ldg(eidx + base + 32 + lane) : base + 32 + lane;
    }
#pragma unroll 1
    for (int jj = 0; jj < n; jj += G * U) {
      float4 a[U][NV];
      int e[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        e[u] = jj + u * G + g;
        const int64_t s_row = __shfl_sync(FULL, my_idx, e[u] & 31);
        const bool ok = e[u] < n && cok;
#pragma unroll
        for (int v = 0; v < NV; ++v) a[u][v] = ok ? __ldg(l + s_row * FV + cv0 + v) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        double acc = 0.0, acc1 = 0.0;
        if constexpr (MIX) {
          Acc2 acc2{0, 0};
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            acc = fma((double)a[u][v].x, rd[v][0], acc), acc1 = fma((double)a[u][v].y, rd[v][1], acc1);
            acc2.fma_exact(pack2(a[u][v].z, a[u][v].w), rp[v]);
          }
          float h0, h1, l0, l1;
          unpack2(acc2.hi, h0, h1);
          unpack2(acc2.lo, l0, l1);
          acc = (acc + acc1) + (((double)h0 + (double)h1) + ((double)l0 + (double)l1));
        } else {
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            acc = fma((double)a[u][v].x, rd[v][0], acc), acc1 = fma((double)a[u][v].y, rd[v][1], acc1);
            acc = fma((double)a[u][v].z, rd[v][2], acc), acc1 = fma((double)a[u][v].w, rd[v][3], acc1);
          }
          acc += acc1;
        }
#pragma unroll
        for (int off = 1; off < 32; off <<= 1)
          if (off < lanes_per_head) acc += __shfl_xor_sync(FULL, acc, off);      // uniform condition
        const int64_t eid = __shfl_sync(FULL, my_eid, e[u] & 31);
        if (e[u] < n && writer) z[eid * H + my_head] = (float)acc;
      }
    }
  }
}

template <int LPR, int NV>
static int launch_u_dot_v_csc(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx, const int32_t *eidx,
                              int64_t n_rows, int64_t heads, int64_t fv, int64_t dv, const float *l, const float *r,
                              float *z, cudaStream_t stream) {
  const int64_t n_items = plan ? plan->n_items : n_rows;
  if (n_items == 0) return GPHL_OK;
  const unsigned grid = (unsigned)((n_items + 7) / 8);
  const Item *items = plan ? plan->items : nullptr;
  const float4 *l4 = reinterpret_cast<const float4 *>(l), *r4 = reinterpret_cast<const float4 *>(r);
  if (knob("GPHL_DOT_MIX", 0))
    u_dot_v_csc_kernel<LPR, NV, true><<<grid, 256, 0, stream>>>(items, n_items, pointer, idx, eidx, (int32_t)heads,
                                                                 (int32_t)fv, (int32_t)dv, l4, r4, z);
  else
    u_dot_v_csc_kernel<LPR, NV, false><<<grid, 256, 0, stream>>>(items, n_items, pointer, idx, eidx, (int32_t)heads,
                                                                  (int32_t)fv, (int32_t)dv, l4, r4, z);
  return launched("u_dot_v_csc_kernel");
}

static unsigned grid_for(int64_t total, int block) {
  int64_t g = (total + block - 1) / block;
  const int64_t cap = 148LL * 64;  // grid-stride beyond a few waves of the 148 SMs
  return (unsigned)(g < cap ? (g > 0 ? g : 1) : cap);
}

template <typename I>
static int u_add_v(const I *src, const I *dst, int64_t n_edges, int64_t feat, const float *l, const float *r, float *z,
                   void *stream_) {
  GPHL_REQUIRE(n_edges >= 0 && feat >= 0 && feat < (1 << 20), "bad sizes");
  if (n_edges == 0 || feat == 0) return GPHL_OK;
  GPHL_REQUIRE(src && dst && l && r && z, "null pointer argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (feat % 4 == 0 && aligned16(l) && aligned16(r) && aligned16(z)) {
    const int32_t fv = (int32_t)(feat / 4), lanes = std::min(fv, 256);
    const int64_t per_block = 256 / lanes;
    u_add_v_vec_kernel<I><<<grid_for((n_edges + per_block - 1) / per_block * 256, 256), 256, 0, stream>>>(
        src, dst, n_edges, fv, lanes, reinterpret_cast<const float4 *>(l), reinterpret_cast<const float4 *>(r),
        reinterpret_cast<float4 *>(z));
    return launched("u_add_v_vec_kernel");
  }
  u_add_v_scalar_kernel<I><<<grid_for(n_edges * feat, 256), 256, 0, stream>>>(src, dst, n_edges, (int32_t)feat, l, r, z);
  return launched("u_add_v_scalar_kernel");
}

template <typename I>
static int u_dot_v(const I *src, const I *dst, int64_t n_edges, int64_t heads, int64_t dim, const float *l,
                   const float *r, float *z, void *stream_) {
  GPHL_REQUIRE(n_edges >= 0 && heads >= 1 && dim >= 1 && heads * dim < (1 << 20), "bad sizes");
  if (n_edges == 0) return GPHL_OK;
  GPHL_REQUIRE(src && dst && l && r && z, "null pointer argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int64_t total = n_edges * heads;
  const int64_t dv = dim / 4, fv = heads * dim / 4;
  if (dim % 4 == 0 && (dv & (dv - 1)) == 0 && dv <= 32 && fv <= 128 && (dim >= 32 || fv >= 64) && aligned16(l) &&
      aligned16(r)) {
    // coalesced path for wide rows / wide heads (measured: at 512-byte rows with 64-byte heads the thread-per-head
    // kernel below is faster, its reads are still sector-sized): whole rows as 16-byte vectors, heads reduced
    // across lanes
    const int64_t lpr = fv <= 1 ? 1 : fv <= 2 ? 2 : fv <= 4 ? 4 : fv <= 8 ? 8 : fv <= 16 ? 16 : 32;
    const int64_t nv = fv <= 32 ? 1 : fv <= 64 ? 2 : 4;       // vectors per lane; a lane must stay inside one head
    if (dv % nv == 0 && dv / nv <= lpr) {
      switch (lpr) {
        case 1: return launch_u_dot_v_rows<I, 1, 1>(src, dst, n_edges, heads, fv, dv, l, r, z, stream);
        case 2: return launch_u_dot_v_rows<I, 2, 1>(src, dst, n_edges, heads, fv, dv, l, r, z, stream);
        case 4: return launch_u_dot_v_rows<I, 4, 1>(src, dst, n_edges, heads, fv, dv, l, r, z, stream);
        case 8: return launch_u_dot_v_rows<I, 8, 1>(src, dst, n_edges, heads, fv, dv, l, r, z, stream);
        case 16: return launch_u_dot_v_rows<I, 16, 1>(src, dst, n_edges, heads, fv, dv, l, r, z, stream);
        default:
          if (fv <= 32) return launch_u_dot_v_rows<I, 32, 1>(src, dst, n_edges, heads, fv, dv, l, r, z, stream);
          if (fv <= 64) return launch_u_dot_v_rows<I, 32, 2>(src, dst, n_edges, heads, fv, dv, l, r, z, stream);
          return launch_u_dot_v_rows<I, 32, 4>(src, dst, n_edges, heads, fv, dv, l, r, z, stream);
      }
    }
  }
  const int64_t per_block = 256 / std::min<int64_t>(heads, 256);
  const unsigned grid = grid_for((n_edges + per_block - 1) / per_block * 256, 256);
  if (dim % 4 == 0 && aligned16(l) && aligned16(r)) {
    u_dot_v_kernel<I, true><<<grid, 256, 0, stream>>>(src, dst, n_edges, (int32_t)heads, (int32_t)dim, l, r, z);
  } else {
    u_dot_v_kernel<I, false><<<grid, 256, 0, stream>>>(src, dst, n_edges, (int32_t)heads, (int32_t)dim, l, r, z);
  }
  return launched("u_dot_v_kernel");
}

}  // namespace gphl

using namespace gphl;

extern "C" int gphl_sddmm_u_add_v_f32_i64(const int64_t *src, const int64_t *dst, int64_t n_edges, int64_t feat,
                                          const float *l, const float *r, float *z, void *stream) {
  return u_add_v<int64_t>(src, dst, n_edges, feat, l, r, z, stream);
}
extern "C" int gphl_sddmm_u_add_v_f32_i32(const int32_t *src, const int32_t *dst, int64_t n_edges, int64_t feat,
                                          const float *l, const float *r, float *z, void *stream) {
  return u_add_v<int32_t>(src, dst, n_edges, feat, l, r, z, stream);
}
extern "C" int gphl_sddmm_u_dot_v_f32_i64(const int64_t *src, const int64_t *dst, int64_t n_edges, int64_t heads,
                                          int64_t dim, const float *l, const float *r, float *z, void *stream) {
  return u_dot_v<int64_t>(src, dst, n_edges, heads, dim, l, r, z, stream);
}
extern "C" int gphl_sddmm_u_dot_v_f32_i32(const int32_t *src, const int32_t *dst, int64_t n_edges, int64_t heads,
                                          int64_t dim, const float *l, const float *r, float *z, void *stream) {
  return u_dot_v<int32_t>(src, dst, n_edges, heads, dim, l, r, z, stream);
}

// Destination-row order: out[eid[i], h] = sum_d l[idx[i], h, d] * r[v, h, d] for every position i of row v.
// Returns GPHL_ERR_UNSUPPORTED for shapes the row kernel does not cover (the caller then uses the COO form).
extern "C" int gphl_sddmm_u_dot_v_csc_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx,
                                          const int32_t *eidx, int64_t n_rows, int64_t heads, int64_t dim, const float *l,
                                          const float *r, float *z, void *stream_) {
  GPHL_REQUIRE(n_rows >= 0 && n_rows < INT32_MAX && heads >= 1 && dim >= 1 && heads * dim < (1 << 20), "bad sizes");
  if (n_rows == 0) return GPHL_OK;
  GPHL_REQUIRE(pointer && idx && l && r && z, "null pointer argument");
  GPHL_REQUIRE(!plan || plan->n_rows == n_rows, "plan was built for a different row count");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int64_t dv = dim / 4, fv = heads * dim / 4;
  if (!(dim % 4 == 0 && (dv & (dv - 1)) == 0 && dv <= 32 && fv <= 128 && aligned16(l) && aligned16(r)))
    return fail(GPHL_ERR_UNSUPPORTED, "u_dot_v (row order) needs 16-byte aligned rows of at most 512 columns and heads of "
                "4, 8, ..., 128 columns");
  const int64_t lpr = fv <= 1 ? 1 : fv <= 2 ? 2 : fv <= 4 ? 4 : fv <= 8 ? 8 : fv <= 16 ? 16 : 32;
  const int64_t nv = fv <= 32 ? 1 : fv <= 64 ? 2 : 4;
  if (dv % nv != 0 || dv / nv > lpr)
    return fail(GPHL_ERR_UNSUPPORTED, "u_dot_v (row order): a head of %lld columns does not fit the lane layout", (long long)dim);
#define GPHL_CSC(L, V) return launch_u_dot_v_csc<L, V>(plan, pointer, idx, eidx, n_rows, heads, fv, dv, l, r, z, stream)
  switch (lpr) {
    case 1: GPHL_CSC(1, 1);
    case 2: GPHL_CSC(2, 1);
    case 4: GPHL_CSC(4, 1);
    case 8: GPHL_CSC(8, 1);
    case 16: GPHL_CSC(16, 1);
    default:
      if (nv == 1) GPHL_CSC(32, 1);
      if (nv == 2) GPHL_CSC(32, 2);
      GPHL_CSC(32, 4);
  }
#undef GPHL_CSC
}

// ---- attention scores per node and head: el[n,h] = sum_d z[n,h,d] a_src[h,d], er likewise with a_dst ----
// The dense prologue of the GAT layer (the reference computes it as mm(z, attn_weight) after its split pass,
// examples/GAT/GAT.py:25-31).  One thread per (node, head) reads the head's slice of the row once with 16-byte loads
// and produces both scores from exact products.
namespace gphl {

__global__ void head_scores_kernel(const float *__restrict__ z, const float *__restrict__ a_src,
                                   const float *__restrict__ a_dst, int64_t n, int32_t H, int32_t D,
                                   float *__restrict__ el, float *__restrict__ er) {
  // one thread per (node, head): D is small (8..64) and consecutive threads read consecutive heads of a row
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n * H) return;
  const int h = (int)(t % H);
  const float *row = z + t * D;                      // (n*H + h) * D
  const float *as = a_src + (int64_t)h * D, *ad = a_dst + (int64_t)h * D;
  // both dot products exact to the last rounding, one on each floating-point pipe: el in double (exact products),
  // er as packed fp32 products with their rounding errors in a compensated pair
  double s = 0.0;
  if ((D & 3) == 0 && aligned16_dev(row) && aligned16_dev(as) && aligned16_dev(ad)) {
    Acc2 d2{0, 0};
    for (int k = 0; k < D; k += 4) {
      const float4 v = __ldg(reinterpret_cast<const float4 *>(row + k));
      const float4 p = __ldg(reinterpret_cast<const float4 *>(as + k));
      const float4 q = __ldg(reinterpret_cast<const float4 *>(ad + k));
      s = fma((double)v.x, (double)p.x, s), s = fma((double)v.y, (double)p.y, s);
      s = fma((double)v.z, (double)p.z, s), s = fma((double)v.w, (double)p.w, s);
      d2.fma_exact(pack2(v.x, v.y), pack2(q.x, q.y));
      d2.fma_exact(pack2(v.z, v.w), pack2(q.z, q.w));
    }
    float h0, h1, l0, l1;
    unpack2(d2.hi, h0, h1);
    unpack2(d2.lo, l0, l1);
    el[t] = (float)s;
    er[t] = (float)(((double)h0 + (double)h1) + ((double)l0 + (double)l1));
  } else {
    double d = 0.0;
    for (int k = 0; k < D; ++k) {
      const double v = (double)__ldg(row + k);
      s = fma(v, (double)__ldg(as + k), s);
      d = fma(v, (double)__ldg(ad + k), d);
    }
    el[t] = (float)s;
    er[t] = (float)d;
  }
}

// The same scores with coalesced row reads, for rows of up to 128 vectors whose heads are a power-of-two number of
// vectors: a group of LPR lanes reads a node's row as consecutive 16-byte vectors (NV per lane, all of one head), keeps
// its columns of the two attention vectors in registers, and the lanes of a head reduce with shuffles.  The thread-per-
// head kernel above reads 128-byte slices at a 128-byte stride between lanes and reaches a quarter of the bandwidth.
template <int LPR, int NV>
__global__ void __launch_bounds__(256) head_scores_rows_kernel(const float4 *__restrict__ z, const float4 *__restrict__ a_src,
                                                               const float4 *__restrict__ a_dst, int64_t n, int32_t H,
                                                               int32_t FV, int32_t DV, float *__restrict__ el,
                                                               float *__restrict__ er) {
  constexpr int G = 32 / LPR, U = (NV >= 2) ? 2 : 4;
  const int lane = threadIdx.x & 31, g = lane / LPR, ll = lane % LPR;
  const int cv0 = ll * NV;
  const bool cok = cv0 < FV;
  const int lanes_per_head = DV / NV;
  const bool writer = cok && (ll % lanes_per_head) == 0;     // hoisted: integer division by a run-time value is dear
  const int my_head = cv0 / DV;
  double ps[NV][4];                                      // this lane's columns of a_src, widened once
  float4 pd[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const float4 p = cok ? __ldg(a_src + cv0 + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    ps[v][0] = (double)p.x, ps[v][1] = (double)p.y, ps[v][2] = (double)p.z, ps[v][3] = (double)p.w;
    pd[v] = cok ? __ldg(a_dst + cv0 + v) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp_id * (G * U); base < n; base += n_warps * (G * U)) {
    float4 a[U][NV];
    int64_t r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      r[u] = base + u * G + g;
      const bool ok = r[u] < n && cok;
#pragma unroll
      for (int v = 0; v < NV; ++v) a[u][v] = ok ? __ldg(z + r[u] * FV + cv0 + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      double s = 0.0;                                    // el: exact products in double
      Acc2 d2{0, 0};                                     // er: packed fp32 products with their rounding errors
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        s = fma((double)a[u][v].x, ps[v][0], s), s = fma((double)a[u][v].y, ps[v][1], s);
        s = fma((double)a[u][v].z, ps[v][2], s), s = fma((double)a[u][v].w, ps[v][3], s);
        d2.fma_exact(pack2(a[u][v].x, a[u][v].y), pack2(pd[v].x, pd[v].y));
        d2.fma_exact(pack2(a[u][v].z, a[u][v].w), pack2(pd[v].z, pd[v].w));
      }
      float h0, h1, l0, l1;
      unpack2(d2.hi, h0, h1);
      unpack2(d2.lo, l0, l1);
      double d = ((double)h0 + (double)h1) + ((double)l0 + (double)l1);
      for (int off = 1; off < lanes_per_head; off <<= 1) {     // a power of two <= LPR
        s += __shfl_xor_sync(FULL, s, off);
        d += __shfl_xor_sync(FULL, d, off);
      }
      if (r[u] < n && writer) {
        el[r[u] * H + my_head] = (float)s;
        er[r[u] * H + my_head] = (float)d;
      }
    }
  }
}

template <int LPR, int NV>
static int launch_head_scores_rows(const float *z, const float *a_src, const float *a_dst, int64_t n, int64_t heads,
                                   int64_t fv, int64_t dv, float *el, float *er, cudaStream_t stream) {
  constexpr int per_warp = (32 / LPR) * ((NV >= 2) ? 2 : 4);
  const int64_t warps = (n + per_warp - 1) / per_warp;
  const int64_t blocks = std::min<int64_t>((warps + 7) / 8, 148LL * 32);
  head_scores_rows_kernel<LPR, NV><<<(unsigned)blocks, 256, 0, stream>>>(
      reinterpret_cast<const float4 *>(z), reinterpret_cast<const float4 *>(a_src), reinterpret_cast<const float4 *>(a_dst),
      n, (int32_t)heads, (int32_t)fv, (int32_t)dv, el, er);
  return launched("head_scores_rows_kernel");
}

}  // namespace gphl

extern "C" int gphl_gat_head_scores_f32(const float *z, const float *attn_src, const float *attn_dst, int64_t n_nodes,
                                        int64_t heads, int64_t dim, float *el, float *er, void *stream_) {
  GPHL_REQUIRE(n_nodes >= 0 && heads >= 1 && dim >= 1 && heads * dim < (1 << 20), "bad sizes");
  if (n_nodes == 0) return GPHL_OK;
  GPHL_REQUIRE(z && attn_src && attn_dst && el && er, "null pointer argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int64_t dv = dim / 4, fv = heads * dim / 4;
  if (dim % 4 == 0 && (dv & (dv - 1)) == 0 && dv <= 32 && fv <= 128 && gphl::aligned16(z) && gphl::aligned16(attn_src) &&
      gphl::aligned16(attn_dst)) {
    const int64_t nv = fv <= 32 ? 1 : fv <= 64 ? 2 : 4;       // vectors per lane; a lane must stay inside one head
    if (dv % nv == 0) {
      using namespace gphl;
      if (nv == 4) return launch_head_scores_rows<32, 4>(z, attn_src, attn_dst, n_nodes, heads, fv, dv, el, er, stream);
      if (nv == 2) return launch_head_scores_rows<32, 2>(z, attn_src, attn_dst, n_nodes, heads, fv, dv, el, er, stream);
      if (fv <= 1) return launch_head_scores_rows<1, 1>(z, attn_src, attn_dst, n_nodes, heads, fv, dv, el, er, stream);
      if (fv <= 2) return launch_head_scores_rows<2, 1>(z, attn_src, attn_dst, n_nodes, heads, fv, dv, el, er, stream);
      if (fv <= 4) return launch_head_scores_rows<4, 1>(z, attn_src, attn_dst, n_nodes, heads, fv, dv, el, er, stream);
      if (fv <= 8) return launch_head_scores_rows<8, 1>(z, attn_src, attn_dst, n_nodes, heads, fv, dv, el, er, stream);
      if (fv <= 16) return launch_head_scores_rows<16, 1>(z, attn_src, attn_dst, n_nodes, heads, fv, dv, el, er, stream);
      return launch_head_scores_rows<32, 1>(z, attn_src, attn_dst, n_nodes, heads, fv, dv, el, er, stream);
    }
  }
  const int64_t total = n_nodes * heads;
  gphl::head_scores_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      z, attn_src, attn_dst, n_nodes, (int32_t)heads, (int32_t)dim, el, er);
  return gphl::launched("head_scores_kernel");
}
