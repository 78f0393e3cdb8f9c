// Row-gather SpMM family for sm_100a: copy_u_sum / copy_e_sum, u_mul_e_sum (per-head edge
// weights) and the aggregation half of the fused attention operator.
//
// Work decomposition: one warp per work item (a whole row, or one `chunk`-entry piece of a
// hub row).  A feature row is read as 16-byte vectors; rows narrower than 512 B are read by
// sub-warp groups so that one warp streams 32/LPR neighbour rows at a time.  Each warp first
// loads 32 neighbour indices with one coalesced access, (for the weighted modes) stages the
// 32 x H edge weights in shared memory, then issues U independent 16-byte loads per lane
// before accumulating, which keeps >= U KB per warp in flight.  Sums are compensated
// (two-sum) fp32 in a fixed order; pieces of a cut row are combined in ascending order by a
// second small kernel, so the result does not depend on the split or on the GPU count.
#include "common.cuh"

namespace gphl {

enum Mode { COPY = 0, MUL_E = 1, GAT = 2 };

struct GatherArgs {
  const Item *items;
  int64_t n_items;
  const int32_t *pointer;
  const int32_t *idx;    // neighbour row per position (node id, or edge id for copy_e)
  const int32_t *eidx;   // edge id per position (NULL: position == edge id)
  const void *x;
  void *y;
  const float *w;        // MUL_E: (n_edges, H)
  const float *el, *er;  // GAT: (n_src, H), (n_rows, H)
  const float *stats;    // GAT: (n_rows, H, 2) = row maximum, reciprocal of the exp-sum
  float *alpha_out;      // GAT: optional (n_edges, H)
  float *scratch;
  int64_t plane;         // floats per scratch plane row (plan->max_feat)
  const float *dst_scale;  // optional per-row factor applied to the finished sum (epilogue)
  float slope;
  int32_t relu;          // epilogue: max(., 0)
  int32_t exact;         // 1: compensated accumulation (default), 0: plain fp32 adds
  int32_t wvec;          // per-head arrays (w | el, er, stats) can be read four heads at a time
  int64_t n_long;        // items [0, n_long) are longer than GPHL_SHORT_ITEM positions; -1: unknown (no plan)
  int32_t F, FV, H, DV;  // columns, 16-byte vectors per row, heads, vectors per head
};

constexpr int WARPS = 8;

// Raw 16-byte vector of a row; elements are widened to fp32 pairs only when they are accumulated, so
// loads in flight cost four registers each whatever the storage type.
template <typename T>
__device__ __forceinline__ void unpack_pairs(const uint4 &r, uint64_t (&v)[VecOf<T>::N / 2]);
template <>
__device__ __forceinline__ void unpack_pairs<float>(const uint4 &r, uint64_t (&v)[2]) {
  v[0] = pack2(__uint_as_float(r.x), __uint_as_float(r.y));
  v[1] = pack2(__uint_as_float(r.z), __uint_as_float(r.w));
}
template <>
__device__ __forceinline__ void unpack_pairs<__nv_bfloat16>(const uint4 &r, uint64_t (&v)[4]) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = pack2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
}

// Accumulator kinds, all on packed pairs of columns.  1: compensated (two-sum) fp32, the library's contract.
// 0: plain fp32 adds (opt-in; the same arithmetic as the reference's kernels, a third of the instructions).
// 2: one double per column (the sum of fp32 terms in double is exact to 2^-53 per addition, and products of two
// fp32 values are exact in double): the same contract as 1 on the fp64 pipe.  `hi` / `lo` then hold the bit
// patterns of the two doubles, so that zeroing, shuffling and merging read the same as for kind 1.
template <int KIND>
struct AccT;
template <>
struct AccT<1> : Acc2 {
  using Acc2::add;
  using Acc2::fma_exact;
  using Acc2::merge;
  using Acc2::value;
  __device__ __forceinline__ void add(uint64_t v, int) { Acc2::add(v); }
  __device__ __forceinline__ void fma_exact(uint64_t p, uint64_t q, int) { Acc2::fma_exact(p, q); }
  __device__ __forceinline__ void fma_w(uint64_t p, float w, double, int) { Acc2::fma_exact(p, pack2(w, w)); }
  __device__ __forceinline__ void merge(uint64_t ohi, uint64_t olo, int) { Acc2::merge(ohi, olo); }
  __device__ __forceinline__ uint64_t value(int) const { return Acc2::value(); }
  __device__ __forceinline__ void planes(float &h0, float &h1, float &l0, float &l1, int = 0) const {
    unpack2(hi, h0, h1);
    unpack2(lo, l0, l1);
  }
};
template <>
struct AccT<0> {
  uint64_t hi;
  static constexpr uint64_t lo = 0;
  __device__ __forceinline__ void add(uint64_t v, int = 0) { hi = fadd2(hi, v); }
  __device__ __forceinline__ void fma_exact(uint64_t a, uint64_t b, int = 0) { hi = ffma2(a, b, hi); }
  __device__ __forceinline__ void fma_w(uint64_t a, float w, double, int = 0) { hi = ffma2(a, pack2(w, w), hi); }
  __device__ __forceinline__ void merge(uint64_t ohi, uint64_t, int = 0) { hi = fadd2(hi, ohi); }
  __device__ __forceinline__ uint64_t value(int = 0) const { return hi; }
  __device__ __forceinline__ void planes(float &h0, float &h1, float &l0, float &l1, int = 0) const {
    unpack2(hi, h0, h1);
    l0 = l1 = 0.f;
  }
};
template <>
struct AccT<2> {
  uint64_t hi, lo;                    // bits of the even and the odd column's double
  static __device__ __forceinline__ double d(uint64_t b) { return __longlong_as_double((long long)b); }
  static __device__ __forceinline__ uint64_t b(double v) { return (uint64_t)__double_as_longlong(v); }
  __device__ __forceinline__ void add(uint64_t v, int = 0) {
    float x, y;
    unpack2(v, x, y);
    hi = b(d(hi) + (double)x), lo = b(d(lo) + (double)y);
  }
  __device__ __forceinline__ void fma_exact(uint64_t p, uint64_t q, int = 0) {
    float px, py, qx, qy;
    unpack2(p, px, py);
    unpack2(q, qx, qy);
    hi = b(fma((double)px, (double)qx, d(hi))), lo = b(fma((double)py, (double)qy, d(lo)));
  }
  // both columns of the pair times one weight that was widened once (the conversions run on the slowest pipe)
  __device__ __forceinline__ void fma_w(uint64_t p, float, double wd, int = 0) {
    float px, py;
    unpack2(p, px, py);
    hi = b(fma((double)px, wd, d(hi))), lo = b(fma((double)py, wd, d(lo)));
  }
  __device__ __forceinline__ void merge(uint64_t ohi, uint64_t olo, int = 0) {
    hi = b(d(hi) + d(ohi)), lo = b(d(lo) + d(olo));
  }
  __device__ __forceinline__ uint64_t value(int = 0) const { return pack2((float)d(hi), (float)d(lo)); }
  __device__ __forceinline__ void planes(float &h0, float &h1, float &l0, float &l1, int = 0) const {
    h0 = (float)d(hi), h1 = (float)d(lo);
    l0 = (float)(d(hi) - (double)h0), l1 = (float)(d(lo) - (double)h1);
  }
};

// 3: kind 2 for every second column pair of a lane and kind 1 for the others, so that the fp64 and the fp32 pipe
// each carry half of the accumulation (measured against one pair in four and three in four: 6.0 ms against 6.5 and
// 6.4 on the 62 M-edge, 256-column gather).  `k` numbers the pairs a lane holds (a constant after unrolling).
template <>
struct AccT<3> {
  uint64_t hi, lo;
  static __device__ __forceinline__ bool in_double(int k) { return (k & 1) == 0; }
  __device__ __forceinline__ void add(uint64_t v, int k) {
    if (in_double(k)) {
      AccT<2> t{hi, lo};
      t.add(v);
      hi = t.hi, lo = t.lo;
    } else {
      Acc2 t{hi, lo};
      t.add(v);
      hi = t.hi, lo = t.lo;
    }
  }
  __device__ __forceinline__ void fma_exact(uint64_t p, uint64_t q, int k) {
    if (in_double(k)) {
      AccT<2> t{hi, lo};
      t.fma_exact(p, q);
      hi = t.hi, lo = t.lo;
    } else {
      Acc2 t{hi, lo};
      t.fma_exact(p, q);
      hi = t.hi, lo = t.lo;
    }
  }
  __device__ __forceinline__ void fma_w(uint64_t p, float w, double wd, int k) {
    if (in_double(k)) {
      AccT<2> t{hi, lo};
      t.fma_w(p, w, wd);
      hi = t.hi, lo = t.lo;
    } else {
      Acc2 t{hi, lo};
      t.fma_exact(p, pack2(w, w));
      hi = t.hi, lo = t.lo;
    }
  }
  __device__ __forceinline__ void merge(uint64_t ohi, uint64_t olo, int k) {
    if (in_double(k)) {
      AccT<2> t{hi, lo};
      t.merge(ohi, olo);
      hi = t.hi, lo = t.lo;
    } else {
      Acc2 t{hi, lo};
      t.merge(ohi, olo);
      hi = t.hi, lo = t.lo;
    }
  }
  __device__ __forceinline__ uint64_t value(int k) const {
    if (in_double(k)) return AccT<2>{hi, lo}.value();
    return Acc2{hi, lo}.value();
  }
  __device__ __forceinline__ void planes(float &h0, float &h1, float &l0, float &l1, int k) const {
    if (in_double(k)) {
      AccT<2>{hi, lo}.planes(h0, h1, l0, l1);
    } else {
      unpack2(hi, h0, h1);
      unpack2(lo, l0, l1);
    }
  }
};
// Register budget: the kernel hides gather latency with resident warps, so for fp32 rows of up to 64 vectors the
// allocation is capped where it was measured best - five blocks per SM for the unweighted sum (<= 51 registers), four
// for the weighted ones (<= 64).  The other shapes (more vectors per lane, bf16 unpacking) would spill under that cap.
template <typename T, int NV, int MODE>
constexpr int gather_min_blocks() {
  return (sizeof(T) == 4 && NV <= 2) ? (MODE == COPY ? 5 : 4) : 0;      // 0: no minimum, the compiler's own choice
}
template <typename T, int LPR, int NV, int MODE, int EXACT>
__global__ void __launch_bounds__(WARPS * 32, gather_min_blocks<T, NV, MODE>()) gather_sum_kernel(GatherArgs a) {
  constexpr int VEC = VecOf<T>::N;
  constexpr int G = 32 / LPR;              // neighbour rows streamed concurrently by one warp
  constexpr int U = (NV >= 4) ? 1 : 4 / NV;  // rows in flight per group: four 16-byte loads per lane (more costs occupancy)
  extern __shared__ float smem_w[];        // WARPS x 32 x H staged edge weights

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item_id = (int64_t)blockIdx.x * WARPS + warp;
  if (item_id >= a.n_items) return;
  const Item it = fetch_item(a.items, a.pointer, item_id);
  const int g = lane / LPR, l = lane % LPR;
  const int tile0 = blockIdx.y * (LPR * NV);

  int cv[NV];
  bool cok[NV];
  int head[NV];
  bool cols_full = true;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    cv[v] = tile0 + v * LPR + l;
    cok[v] = cv[v] < a.FV;
    cols_full = cols_full && cok[v];
    head[v] = (MODE == COPY || !cok[v]) ? 0 : cv[v] / a.DV;
    if (!cok[v]) cv[v] = 0;                // keep addresses in range; the value is discarded
  }
  cols_full = __all_sync(FULL, cols_full);

  constexpr int VP = VEC / 2;              // packed column pairs per 16-byte vector
  AccT<EXACT> acc[NV][VP];
#pragma unroll
  for (int v = 0; v < NV; ++v)
#pragma unroll
    for (int k = 0; k < VP; ++k) {
      acc[v][k].hi = 0;
      if constexpr (EXACT) acc[v][k].lo = 0;
    }

  // one multiply-add per edge forms a row's address: the lane's byte offset is folded into the base once, the second
  // and later vectors of a lane lie at compile-time distances (LPR vectors apart)
  const char *xb = static_cast<const char *>(a.x) + (size_t)(tile0 + l) * 16;
  const uint32_t row_bytes = (uint32_t)a.FV * 16u;
  float *wsm = smem_w + (size_t)warp * 32 * a.H;

  int next_idx = 0;
  if (it.begin + lane < it.end) next_idx = __ldg(a.idx + it.begin + lane);
  for (int base = it.begin; base < it.end; base += 32) {
    const int n = min(32, it.end - base);
    const int my_idx = next_idx;
    if (base + 32 + lane < it.end) next_idx = __ldg(a.idx + base + 32 + lane);   // prefetch the next batch
    if (MODE != COPY) {
      __syncwarp();
      if (lane < n) {
        const int eid = a.eidx ? __ldg(a.eidx + base + lane) : base + lane;
        if (MODE == MUL_E) {
          if (a.wvec) {                                     // H % 4 == 0, 16-byte aligned arrays: four heads per access
            for (int h = 0; h < a.H; h += 4)
              *reinterpret_cast<float4 *>(wsm + lane * a.H + h) =
                  __ldg(reinterpret_cast<const float4 *>(a.w + (int64_t)eid * a.H + h));
          } else {
            for (int h = 0; h < a.H; ++h) wsm[lane * a.H + h] = __ldg(a.w + (int64_t)eid * a.H + h);
          }
        } else if (a.wvec) {
#pragma unroll 1
          for (int h = 0; h < a.H; h += 4) {
            const float4 el4 = __ldg(reinterpret_cast<const float4 *>(a.el + (int64_t)my_idx * a.H + h));
            const float4 er4 = __ldg(reinterpret_cast<const float4 *>(a.er + (int64_t)it.row * a.H + h));
            const float4 *st = reinterpret_cast<const float4 *>(a.stats + 2 * ((int64_t)it.row * a.H + h));
            const float4 s01 = __ldg(st), s23 = __ldg(st + 1);       // (max, 1/sum) of heads h, h+1 | h+2, h+3
            float4 wv;
            wv.x = exp_neg(leaky(el4.x + er4.x, a.slope) - s01.x) * s01.y;
            wv.y = exp_neg(leaky(el4.y + er4.y, a.slope) - s01.z) * s01.w;
            wv.z = exp_neg(leaky(el4.z + er4.z, a.slope) - s23.x) * s23.y;
            wv.w = exp_neg(leaky(el4.w + er4.w, a.slope) - s23.z) * s23.w;
            *reinterpret_cast<float4 *>(wsm + lane * a.H + h) = wv;
            if (a.alpha_out && blockIdx.y == 0) {
              float *ao = a.alpha_out + (int64_t)eid * a.H + h;
              ao[0] = wv.x, ao[1] = wv.y, ao[2] = wv.z, ao[3] = wv.w;
            }
          }
        } else {
#pragma unroll 1
          for (int h = 0; h < a.H; ++h) {
            const float2 st = __ldg(reinterpret_cast<const float2 *>(a.stats) + (int64_t)it.row * a.H + h);
            float e = leaky(__ldg(a.el + (int64_t)my_idx * a.H + h) + __ldg(a.er + (int64_t)it.row * a.H + h), a.slope);
            float wgt = exp_neg(e - st.x) * st.y;
            wsm[lane * a.H + h] = wgt;
            if (a.alpha_out && blockIdx.y == 0) a.alpha_out[(int64_t)eid * a.H + h] = wgt;
          }
        }
      }
      __syncwarp();
    }
#pragma unroll 1
    for (int jj = 0; jj < n; jj += G * U) {
      uint4 raw[U][NV];
      int e[U];
      if (jj + G * U <= n && cols_full) {
        // whole group of G*U neighbours present: no predicates on the loads
#pragma unroll
        for (int u = 0; u < U; ++u) {
          e[u] = jj + u * G + g;
          const int src = __shfl_sync(FULL, my_idx, e[u]);
          const char *row = xb + (uint64_t)(uint32_t)src * row_bytes;
#pragma unroll
          for (int v = 0; v < NV; ++v) raw[u][v] = __ldg(reinterpret_cast<const uint4 *>(row + v * (LPR * 16)));
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          e[u] = jj + u * G + g;
          const bool ok = e[u] < n;
          const int src = __shfl_sync(FULL, my_idx, e[u] & 31);
          const char *row = xb + (uint64_t)(uint32_t)src * row_bytes;
#pragma unroll
          for (int v = 0; v < NV; ++v)
            raw[u][v] = (ok && cok[v]) ? __ldg(reinterpret_cast<const uint4 *>(row + v * (LPR * 16))) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          uint64_t val[VP];
          unpack_pairs<T>(raw[u][v], val);
          if (MODE == COPY) {
#pragma unroll
            for (int k = 0; k < VP; ++k) acc[v][k].add(val[k], v * VP + k);
          } else {
            const float wgt = (e[u] < n) ? wsm[e[u] * a.H + head[v]] : 0.f;
            const uint64_t w2 = pack2(wgt, wgt);
            const double wd = (double)wgt;                  // widened once per (edge, vector), not once per product
#pragma unroll
            for (int k = 0; k < VP; ++k) {
              // attention weights are softmax probabilities: the rounded products sum to at most max|x| in
              // magnitude, so their rounding (<= eps/2 of that) is far below tolerance and only the sum is
              // compensated; arbitrary edge weights (u_mul_e_sum) keep the exact product
              if (MODE == GAT) acc[v][k].add(fmul2(val[k], w2), v * VP + k);
              else acc[v][k].fma_w(val[k], wgt, wd, v * VP + k);
            }
          }
        }
      }
    }
  }

  // combine the G sub-warp groups in a fixed order
#pragma unroll
  for (int off = LPR; off < 32; off <<= 1) {
#pragma unroll
    for (int v = 0; v < NV; ++v)
#pragma unroll
      for (int k = 0; k < VP; ++k) {
        const uint64_t ohi = __shfl_xor_sync(FULL, (unsigned long long)acc[v][k].hi, off);
        const uint64_t olo = EXACT ? __shfl_xor_sync(FULL, (unsigned long long)acc[v][k].lo, off) : 0ull;
        // both partners add in the same order (lower group first) and so hold identical values
        if ((lane & off) == 0) {
          acc[v][k].merge(ohi, olo, v * VP + k);
        } else {
          AccT<EXACT> t;
          t.hi = ohi;
          if constexpr (EXACT) t.lo = olo;
          t.merge(acc[v][k].hi, acc[v][k].lo, v * VP + k);
          acc[v][k] = t;
        }
      }
  }
  if (g != 0) return;

  if (it.slot < 0) {
    T *y = static_cast<T *>(a.y) + (int64_t)it.row * a.F;
    const float scale = a.dst_scale ? __ldg(a.dst_scale + it.row) : 1.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (!cok[v]) continue;
      float o[VEC];
#pragma unroll
      for (int k = 0; k < VP; ++k) unpack2(acc[v][k].value(v * VP + k), o[2 * k], o[2 * k + 1]);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        if (a.dst_scale) o[k] = __fmul_rn(o[k], scale);
        if (a.relu) o[k] = fmaxf(o[k], 0.f);
      }
      VecOf<T>::store(y + (int64_t)cv[v] * VEC, o);
    }
  } else {
    float *hi = a.scratch + (int64_t)(2 * it.slot) * a.plane;
    float *lo = hi + a.plane;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (!cok[v]) continue;
#pragma unroll
      for (int k = 0; k < VP; ++k) {
        float h0, h1, l0, l1;
        acc[v][k].planes(h0, h1, l0, l1, v * VP + k);
        hi[cv[v] * VEC + 2 * k] = h0, hi[cv[v] * VEC + 2 * k + 1] = h1;
        lo[cv[v] * VEC + 2 * k] = l0, lo[cv[v] * VEC + 2 * k + 1] = l1;
      }
    }
  }
}

// ---- short items of narrow features ----------------------------------------------------------------
// Rows of at most 8 vectors (32 fp32 columns): a warp per item would leave most lanes idle on a low-degree row, so
// LPR lanes take one item and a warp serves 32 / LPR items.  The lanes walk the item's positions in order, four rows in
// flight, with no exchange between lanes.  The plan orders items by length, so the groups of a warp finish together.
template <typename T, int LPR, int MODE, int EXACT>
__global__ void __launch_bounds__(256) gather_sum_rows_kernel(GatherArgs a, int64_t first_item) {
  constexpr int VEC = VecOf<T>::N, VP = VEC / 2;
  const int l = threadIdx.x % LPR;
  const int64_t item_id = first_item + ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
  if (item_id >= a.n_items) return;
  const Item it = fetch_item(a.items, a.pointer, item_id);
  const bool cok = (int)blockIdx.y * LPR + l < a.FV;      // blockIdx.y: column slice of LPR vectors (one slice for narrow rows)
  const int cv = cok ? (int)blockIdx.y * LPR + l : 0;
  const int head = (MODE == COPY) ? 0 : cv / a.DV;
  AccT<EXACT> acc[VP];
#pragma unroll
  for (int k = 0; k < VP; ++k) {
    acc[k].hi = 0;
    if constexpr (EXACT) acc[k].lo = 0;
  }
  float erv = 0.f, mx = 0.f, inv = 0.f;
  if (MODE == GAT) {
    erv = __ldg(a.er + (int64_t)it.row * a.H + head);
    const float2 st = __ldg(reinterpret_cast<const float2 *>(a.stats) + (int64_t)it.row * a.H + head);
    mx = st.x, inv = st.y;
  }
  const char *xb = static_cast<const char *>(a.x) + (size_t)cv * 16;     // one multiply-add per row address
  const uint32_t row_bytes = (uint32_t)a.FV * 16u;
  auto weight = [&](int i, int src) {
    if (MODE == MUL_E) {
      const int eid = a.eidx ? __ldg(a.eidx + i) : i;
      return __ldg(a.w + (int64_t)eid * a.H + head);
    }
    return exp_neg(leaky(__ldg(a.el + (int64_t)src * a.H + head) + erv, a.slope) - mx) * inv;
  };
  auto accumulate = [&](const uint4 &raw, float wgt) {
    uint64_t val[VP];
    unpack_pairs<T>(raw, val);
    const uint64_t w2 = pack2(wgt, wgt);
#pragma unroll
    for (int k = 0; k < VP; ++k) {
      if (MODE == COPY) acc[k].add(val[k], k);
      else if (MODE == GAT) acc[k].add(fmul2(val[k], w2), k);
      else acc[k].fma_exact(val[k], w2, k);
    }
  };
  int i = it.begin;
  for (; i + 3 < it.end; i += 4) {
    int src[4];
    uint4 raw[4];
    float wgt[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) src[u] = __ldg(a.idx + i + u);
#pragma unroll
    for (int u = 0; u < 4; ++u) raw[u] = __ldg(reinterpret_cast<const uint4 *>(xb + (uint64_t)(uint32_t)src[u] * row_bytes));
#pragma unroll
    for (int u = 0; u < 4; ++u) wgt[u] = (MODE == COPY) ? 1.f : weight(i + u, src[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u) accumulate(raw[u], wgt[u]);
  }
  for (; i < it.end; ++i) {
    const int src = __ldg(a.idx + i);
    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(xb + (uint64_t)(uint32_t)src * row_bytes));
    accumulate(raw, (MODE == COPY) ? 1.f : weight(i, src));
  }
  if (!cok) return;
  if (it.slot < 0) {
    T *y = static_cast<T *>(a.y) + (int64_t)it.row * a.F;
    const float scale = a.dst_scale ? __ldg(a.dst_scale + it.row) : 1.f;
    float o[VEC];
#pragma unroll
    for (int k = 0; k < VP; ++k) unpack2(acc[k].value(k), o[2 * k], o[2 * k + 1]);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      if (a.dst_scale) o[k] = __fmul_rn(o[k], scale);
      if (a.relu) o[k] = fmaxf(o[k], 0.f);
    }
    VecOf<T>::store(y + (int64_t)cv * VEC, o);
  } else {
    float *hi = a.scratch + (int64_t)(2 * it.slot) * a.plane;
    float *lo = hi + a.plane;
#pragma unroll
    for (int k = 0; k < VP; ++k) {
      float h0, h1, l0, l1;
      acc[k].planes(h0, h1, l0, l1, k);
      hi[cv * VEC + 2 * k] = h0, hi[cv * VEC + 2 * k + 1] = h1;
      lo[cv * VEC + 2 * k] = l0, lo[cv * VEC + 2 * k + 1] = l1;
    }
  }
}

// ---- column-sliced unweighted sum for matrices far larger than the L2 cache ----------------------------
// A feature matrix of gigabytes gathered ~26 times per row is served from the 126 MB L2 only for its most popular
// rows; everything else comes from DRAM once per edge.  Cutting the columns into slices of LPR 16-byte vectors and
// running the slices one after the other (blockIdx.y, the slow grid dimension) shrinks the bytes a source row
// occupies in the cache by the number of slices, so the cache holds that many more distinct sources, at the cost of
// one more pass over the index array per slice.  A warp takes one work item and one slice: its 32 / LPR lane groups
// walk the item's positions round-robin (group g takes positions g, g + G, ...), each lane holding one 16-byte
// vector of the slice, U rows in flight per group, the next U indices fetched while the current rows are summed.
// The groups' partial sums are merged in a fixed order, so the result depends only on the item and on LPR.
template <typename T, int LPR, int EXACT>
__global__ void __launch_bounds__(WARPS * 32) gather_sum_sliced_kernel(GatherArgs a) {
  constexpr int VEC = VecOf<T>::N, VP = VEC / 2, G = 32 / LPR, U = 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item_id = (int64_t)blockIdx.x * WARPS + warp;
  if (item_id >= a.n_items) return;
  const Item it = fetch_item(a.items, a.pointer, item_id);
  const int g = lane / LPR, l = lane % LPR;
  int cv = blockIdx.y * LPR + l;
  const bool cok = cv < a.FV;
  if (!cok) cv = 0;

  AccT<EXACT> acc[VP];
#pragma unroll
  for (int k = 0; k < VP; ++k) {
    acc[k].hi = 0;
    if constexpr (EXACT) acc[k].lo = 0;
  }
  const char *xb = static_cast<const char *>(a.x) + (size_t)cv * 16;
  const uint32_t row_bytes = (uint32_t)a.FV * 16u;
  const int32_t *ip = a.idx + it.begin + g;
  const int cnt = (it.end - it.begin - g + G - 1) / G;      // positions of this lane group
  auto add_row = [&](const uint4 &raw) {
    uint64_t val[VP];
    unpack_pairs<T>(raw, val);
#pragma unroll
    for (int k = 0; k < VP; ++k) acc[k].add(val[k], k);
  };
  int i = 0;
  int s[U];
  if (U <= cnt) {
#pragma unroll
    for (int u = 0; u < U; ++u) s[u] = __ldg(ip + u * G);
  }
#pragma unroll 1
  for (; i + U <= cnt; i += U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) raw[u] = __ldg(reinterpret_cast<const uint4 *>(xb + (uint64_t)(uint32_t)s[u] * row_bytes));
    if (i + 2 * U <= cnt) {
#pragma unroll
      for (int u = 0; u < U; ++u) s[u] = __ldg(ip + (i + U + u) * G);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) add_row(raw[u]);
  }
  for (; i < cnt; ++i) {
    const uint32_t src = (uint32_t)__ldg(ip + i * G);
    add_row(__ldg(reinterpret_cast<const uint4 *>(xb + (uint64_t)src * row_bytes)));
  }
  __syncwarp();

  // combine the G lane groups in a fixed order (both partners add lower group first and hold identical values)
#pragma unroll
  for (int off = LPR; off < 32; off <<= 1) {
#pragma unroll
    for (int k = 0; k < VP; ++k) {
      const uint64_t ohi = __shfl_xor_sync(FULL, (unsigned long long)acc[k].hi, off);
      const uint64_t olo = EXACT ? __shfl_xor_sync(FULL, (unsigned long long)acc[k].lo, off) : 0ull;
      if ((lane & off) == 0) {
        acc[k].merge(ohi, olo, k);
      } else {
        AccT<EXACT> t;
        t.hi = ohi;
        if constexpr (EXACT) t.lo = olo;
        t.merge(acc[k].hi, acc[k].lo, k);
        acc[k] = t;
      }
    }
  }
  if (g != 0 || !cok) return;

  if (it.slot < 0) {
    T *y = static_cast<T *>(a.y) + (int64_t)it.row * a.F;
    const float scale = a.dst_scale ? __ldg(a.dst_scale + it.row) : 1.f;
    float o[VEC];
#pragma unroll
    for (int k = 0; k < VP; ++k) unpack2(acc[k].value(k), o[2 * k], o[2 * k + 1]);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      if (a.dst_scale) o[k] = __fmul_rn(o[k], scale);
      if (a.relu) o[k] = fmaxf(o[k], 0.f);
    }
    VecOf<T>::store(y + (int64_t)cv * VEC, o);
  } else {
    float *hi = a.scratch + (int64_t)(2 * it.slot) * a.plane;
    float *lo = hi + a.plane;
#pragma unroll
    for (int k = 0; k < VP; ++k) {
      float h0, h1, l0, l1;
      acc[k].planes(h0, h1, l0, l1, k);
      hi[cv * VEC + 2 * k] = h0, hi[cv * VEC + 2 * k + 1] = h1;
      lo[cv * VEC + 2 * k] = l0, lo[cv * VEC + 2 * k + 1] = l1;
    }
  }
}

template <typename T, int LPR>
static int launch_sliced(const GatherArgs &a, cudaStream_t stream) {
  // long items: a warp per (item, slice); short items: LPR lanes per (item, slice)
  const int64_t n_warp = (a.n_long >= 0 && knob("GPHL_SLICE_ROWS", 1)) ? a.n_long : a.n_items;
  const unsigned slices = (unsigned)((a.FV + LPR - 1) / LPR);
  if (n_warp > 0) {
    GatherArgs w = a;
    w.n_items = n_warp;
    dim3 grid((unsigned)((n_warp + WARPS - 1) / WARPS), slices);
    if (a.exact) gather_sum_sliced_kernel<T, LPR, 3><<<grid, WARPS * 32, 0, stream>>>(w);
    else gather_sum_sliced_kernel<T, LPR, 0><<<grid, WARPS * 32, 0, stream>>>(w);
    int rc = launched("gather_sum_sliced_kernel");
    if (rc != GPHL_OK) return rc;
  }
  if (n_warp < a.n_items) {
    const int64_t threads = (a.n_items - n_warp) * LPR;
    dim3 grid((unsigned)((threads + 255) / 256), slices);
    if (a.exact) gather_sum_rows_kernel<T, LPR, COPY, 3><<<grid, 256, 0, stream>>>(a, n_warp);
    else gather_sum_rows_kernel<T, LPR, COPY, 0><<<grid, 256, 0, stream>>>(a, n_warp);
    return launched("gather_sum_rows_kernel");
  }
  return GPHL_OK;
}

// Which unweighted sums take the sliced kernels (slice width in 16-byte vectors; 0 = the general kernel, one pass
// over whole rows).  Measured on the 62 M-edge graph with 256 columns.  fp32 (1 KB rows): one pass 6.0 ms, two slices
// of 32 vectors 6.0-6.4 ms, four of 16 6.1 ms, eight of 8 9.2 ms: the better cache hit rate of narrow slices is paid
// for with one more pass over the index array and one more fixed cost per short row and slice, so fp32 stays on the
// general kernel.  bf16 storage (512-byte rows = one slice of 32 vectors): 4.1 ms against 5.1 ms, because the sliced
// pair (a warp per long item, a plain per-row loop for short items, indices read directly instead of exchanged by
// shuffle) spends fewer instructions per row; it is the default there (smaller graphs: 0.41 against 0.49 ms on a tenth
// of that graph, 0.11 against 0.13 ms at 1.5 M edges, 0.17 against 0.16 ms at 1.3 M edges of degree 8).  The choice depends on the storage type and the
// row width only, never on the number of rows, so that a shard of any size takes the same kernel and sums in the
// same order.  Measurement builds choose the width with GPHL_SLICE_LPR (-1: never).
template <typename T>
static int slice_lanes(int32_t FV) {
  const int forced = knob("GPHL_SLICE_LPR", 0);
  if (forced) return forced < 0 ? 0 : forced;
  return (sizeof(T) == 2 && FV == 32) ? 32 : 0;
}

// Any shape / alignment: one thread per (item, column), serial over the piece.
template <typename T, int MODE>
__global__ void gather_sum_scalar_kernel(GatherArgs a, int32_t D) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= a.n_items * a.F) return;
  const int64_t item_id = t / a.F;
  const int f = (int)(t % a.F);
  const Item it = fetch_item(a.items, a.pointer, item_id);
  const int h = (MODE == COPY) ? 0 : f / D;
  const T *x = static_cast<const T *>(a.x);
  Acc acc{0.f, 0.f};
  float m = 0.f, inv = 0.f, erv = 0.f;
  if (MODE == GAT) {
    m = a.stats[((int64_t)it.row * a.H + h) * 2];
    inv = a.stats[((int64_t)it.row * a.H + h) * 2 + 1];
    erv = a.er[(int64_t)it.row * a.H + h];
  }
  for (int i = it.begin; i < it.end; ++i) {
    const int src = a.idx[i];
    const float v = to_f32(x[(int64_t)src * a.F + f]);
    if (MODE == COPY) {
      acc.add(v);
    } else {
      const int eid = a.eidx ? a.eidx[i] : i;
      float wgt;
      if (MODE == MUL_E) {
        wgt = a.w[(int64_t)eid * a.H + h];
      } else {
        wgt = exp_neg(leaky(a.el[(int64_t)src * a.H + h] + erv, a.slope) - m) * inv;
        if (a.alpha_out && f == h * D) a.alpha_out[(int64_t)eid * a.H + h] = wgt;
      }
      acc.fma_exact(v, wgt);
    }
  }
  if (it.slot < 0) {
    float o = acc.value();
    if (a.dst_scale) o = __fmul_rn(o, a.dst_scale[it.row]);
    if (a.relu) o = fmaxf(o, 0.f);
    from_f32(static_cast<T *>(a.y)[(int64_t)it.row * a.F + f], o);
  } else {
    a.scratch[(int64_t)(2 * it.slot) * a.plane + f] = acc.hi;
    a.scratch[(int64_t)(2 * it.slot + 1) * a.plane + f] = acc.lo;
  }
}

// Combines the pieces of every cut row, ascending, one thread per (cut row, column).
template <typename T>
__global__ void split_reduce_kernel(const int32_t *split_rows, const int32_t *split_ptr, int64_t n_split,
                                    const float *scratch, int64_t plane, int32_t F, const float *dst_scale,
                                    int32_t relu, T *y) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_split * F) return;
  const int64_t r = t / F;
  const int f = (int)(t % F);
  Acc acc{0.f, 0.f};
  for (int s = split_ptr[r]; s < split_ptr[r + 1]; ++s)
    acc.merge(scratch[(int64_t)(2 * s) * plane + f], scratch[(int64_t)(2 * s + 1) * plane + f]);
  float o = acc.value();
  if (dst_scale) o = __fmul_rn(o, dst_scale[split_rows[r]]);
  if (relu) o = fmaxf(o, 0.f);
  from_f32(y[(int64_t)split_rows[r] * F + f], o);
}

template <typename T, int MODE, int LPR, int NV, int EXACT>
static int launch_vec_e(const GatherArgs &a, cudaStream_t stream) {
  const int tiles = (a.FV + LPR * NV - 1) / (LPR * NV);
  dim3 grid((unsigned)((a.n_items + WARPS - 1) / WARPS), (unsigned)tiles);
  const size_t smem = (MODE == COPY) ? 0 : sizeof(float) * WARPS * 32 * a.H;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gather_sum_kernel<T, LPR, NV, MODE, EXACT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(GPHL_ERR_CUDA, "gather_sum: shared memory opt-in: %s", cudaGetErrorString(e));
  }
  gather_sum_kernel<T, LPR, NV, MODE, EXACT><<<grid, WARPS * 32, smem, stream>>>(a);
  return launched("gather_sum_kernel");
}

template <typename T, int MODE, int LPR, int EXACT>
static int launch_rows_e(const GatherArgs &a, int64_t first_item, cudaStream_t stream) {
  const int64_t threads = (a.n_items - first_item) * LPR;
  gather_sum_rows_kernel<T, LPR, MODE, EXACT><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(a, first_item);
  return launched("gather_sum_rows_kernel");
}

// Narrow rows (FV <= LPR <= 8): the first n_long items (the long ones) go a warp each, the short ones a lane group each.
template <typename T, int MODE, int LPR, int NV>
static int launch_vec(const GatherArgs &a, cudaStream_t stream) {
  // plain accumulation is offered for the unweighted sum and the fused attention aggregate
  const bool exact = !(MODE != MUL_E && !a.exact);
  if constexpr (LPR <= 8 && NV == 1) {
    if (a.n_long >= 0 && a.n_long < a.n_items && !(MODE == GAT && a.alpha_out)) {
      int rc = GPHL_OK;
      if (a.n_long > 0) {
        GatherArgs w = a;
        w.n_items = a.n_long;
        rc = exact ? launch_vec_e<T, MODE, LPR, NV, true>(w, stream) : launch_vec_e<T, MODE, LPR, NV, false>(w, stream);
        if (rc != GPHL_OK) return rc;
      }
      return exact ? launch_rows_e<T, MODE, LPR, true>(a, a.n_long, stream)
                   : launch_rows_e<T, MODE, LPR, false>(a, a.n_long, stream);
    }
  }
  if (!exact) return launch_vec_e<T, MODE, LPR, NV, 0>(a, stream);
  // Which exact accumulator: measured on the 62 M-edge, 256-column gather, the unweighted sum is fastest with the
  // columns split between the fp64 and the fp32 pipe (5.9 ms; two-sum alone 6.7, double alone 6.4), the edge-weighted
  // sum with doubles alone (7.8 ms against 9.4: its exact product is one fused multiply-add in double and ten
  // operations in fp32); the attention aggregate does not care (it waits on its per-edge weights).  
  const int forced = knob("GPHL_ACC", 0);            // measurement builds: 1 two-sum, 2 double, 3 mixed
  const int kind = forced ? forced : (MODE == MUL_E ? 2 : 3);
  if (kind == 1) return launch_vec_e<T, MODE, LPR, NV, 1>(a, stream);
  if (kind == 2) return launch_vec_e<T, MODE, LPR, NV, 2>(a, stream);
  return launch_vec_e<T, MODE, LPR, NV, 3>(a, stream);
}

template <typename T, int MODE>
static int dispatch(const gphl_plan *plan, GatherArgs a, int32_t D, cudaStream_t stream) {
  constexpr int VEC = VecOf<T>::N;
  if (a.n_items == 0 || a.F == 0) return GPHL_OK;
  a.n_long = -1;
  if (plan) {
    a.items = plan->items;
    a.n_items = plan->n_items;
    a.n_long = plan->n_long_items;
    a.scratch = plan->scratch;
    a.plane = plan->max_feat;
    if (plan->n_pieces > 0 && a.F > plan->max_feat)
      return fail(GPHL_ERR_TOO_LARGE, "feature width %d exceeds the plan's scratch width %lld", a.F,
                  (long long)plan->max_feat);
  }
  const bool vec_ok = (a.F % VEC == 0) && aligned16(a.x) && aligned16(a.y) && (MODE == COPY || D % VEC == 0) &&
                      (MODE == COPY || a.H <= 64);
  int rc;
  if (vec_ok) {
    a.FV = a.F / VEC;
    a.DV = (MODE == COPY) ? a.FV : D / VEC;
    a.wvec = 0;
    if (MODE == MUL_E) a.wvec = a.H % 4 == 0 && aligned16(a.w);
    if (MODE == GAT) a.wvec = a.H % 4 == 0 && aligned16(a.el) && aligned16(a.er) && aligned16(a.stats);
    const int slice = (MODE == COPY) ? slice_lanes<T>(a.FV) : 0;
    if (MODE == COPY && slice > 0) {
      if (slice >= 32) rc = launch_sliced<T, 32>(a, stream);
      else if (slice >= 16) rc = launch_sliced<T, 16>(a, stream);
      else if (slice >= 8) rc = launch_sliced<T, 8>(a, stream);
      else rc = launch_sliced<T, 4>(a, stream);
    } else
    if (a.FV <= 1) rc = launch_vec<T, MODE, 1, 1>(a, stream);
    else if (a.FV <= 2) rc = launch_vec<T, MODE, 2, 1>(a, stream);
    else if (a.FV <= 4) rc = launch_vec<T, MODE, 4, 1>(a, stream);
    else if (a.FV <= 8) rc = launch_vec<T, MODE, 8, 1>(a, stream);
    else if (a.FV <= 16) rc = launch_vec<T, MODE, 16, 1>(a, stream);
    else if (a.FV <= 32) rc = launch_vec<T, MODE, 32, 1>(a, stream);
    else if (a.FV <= 64) rc = launch_vec<T, MODE, 32, 2>(a, stream);
    else rc = launch_vec<T, MODE, 32, 4>(a, stream);
  } else {
    const int64_t total = a.n_items * a.F;
    gather_sum_scalar_kernel<T, MODE><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a, D);
    rc = launched("gather_sum_scalar_kernel");
  }
  if (rc != GPHL_OK) return rc;
  if (plan && plan->n_split_rows > 0) {
    const int64_t total = plan->n_split_rows * a.F;
    split_reduce_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        plan->split_rows, plan->split_ptr, plan->n_split_rows, plan->scratch, plan->max_feat, a.F, a.dst_scale,
        a.relu, static_cast<T *>(a.y));
    rc = launched("split_reduce_kernel");
  }
  return rc;
}

static int check_common(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx, int64_t n_rows, int64_t feat,
                        const void *x, const void *y) {
  GPHL_REQUIRE(n_rows >= 0 && feat >= 0, "negative size");
  GPHL_REQUIRE(n_rows < INT32_MAX && feat < (1 << 20), "row count or feature width out of range");
  if (n_rows == 0 || feat == 0) return GPHL_OK;
  GPHL_REQUIRE(pointer && idx && x && y, "null pointer argument");
  GPHL_REQUIRE(!plan || plan->n_rows == n_rows, "plan was built for a different row count");
  return GPHL_OK;
}

}  // namespace gphl

using namespace gphl;

extern "C" int gphl_spmm_gather_sum_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx, int64_t n_rows,
                                        int64_t feat, const float *x, float *y, void *stream) {
  int rc = check_common(plan, pointer, idx, n_rows, feat, x, y);
  if (rc != GPHL_OK) return rc;
  GatherArgs a{};
  a.exact = 1;
  a.n_items = n_rows, a.pointer = pointer, a.idx = idx, a.x = x, a.y = y, a.F = (int32_t)feat, a.H = 1;
  return dispatch<float, COPY>(plan, a, (int32_t)feat, static_cast<cudaStream_t>(stream));
}

extern "C" int gphl_spmm_gather_sum_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx, int64_t n_rows,
                                         int64_t feat, const void *x, void *y, void *stream) {
  int rc = check_common(plan, pointer, idx, n_rows, feat, x, y);
  if (rc != GPHL_OK) return rc;
  GatherArgs a{};
  a.exact = 1;
  a.n_items = n_rows, a.pointer = pointer, a.idx = idx, a.x = x, a.y = y, a.F = (int32_t)feat, a.H = 1;
  return dispatch<__nv_bfloat16, COPY>(plan, a, (int32_t)feat, static_cast<cudaStream_t>(stream));
}

template <typename T>
static int gather_sum_ex(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx, int64_t n_rows, int64_t feat,
                         const void *x, const float *dst_scale, int32_t flags, void *y, void *stream) {
  int rc = check_common(plan, pointer, idx, n_rows, feat, x, y);
  if (rc != GPHL_OK) return rc;
  GPHL_REQUIRE((flags & ~(GPHL_ACCUM_FAST | GPHL_EPILOGUE_RELU)) == 0, "unknown flag bits");
  GatherArgs a{};
  a.n_items = n_rows, a.pointer = pointer, a.idx = idx, a.x = x, a.y = y, a.F = (int32_t)feat, a.H = 1;
  a.exact = (flags & GPHL_ACCUM_FAST) ? 0 : 1;
  a.relu = (flags & GPHL_EPILOGUE_RELU) ? 1 : 0;
  a.dst_scale = dst_scale;
  return dispatch<T, COPY>(plan, a, (int32_t)feat, static_cast<cudaStream_t>(stream));
}

extern "C" int gphl_spmm_gather_sum_ex_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx,
                                           int64_t n_rows, int64_t feat, const float *x, const float *dst_scale,
                                           int32_t flags, float *y, void *stream) {
  return gather_sum_ex<float>(plan, pointer, idx, n_rows, feat, x, dst_scale, flags, y, stream);
}

extern "C" int gphl_spmm_gather_sum_ex_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx,
                                            int64_t n_rows, int64_t feat, const void *x, const float *dst_scale,
                                            int32_t flags, void *y, void *stream) {
  return gather_sum_ex<__nv_bfloat16>(plan, pointer, idx, n_rows, feat, x, dst_scale, flags, y, stream);
}

extern "C" int gphl_spmm_u_mul_e_sum_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                                         const int32_t *edge_idx, int64_t n_rows, int64_t heads, int64_t dim,
                                         const float *x, const float *w, float *y, void *stream) {
  GPHL_REQUIRE(heads >= 1 && dim >= 1, "heads and dim must be >= 1");
  int rc = check_common(plan, pointer, node_idx, n_rows, heads * dim, x, y);
  if (rc != GPHL_OK) return rc;
  if (n_rows == 0) return GPHL_OK;
  GPHL_REQUIRE(w != nullptr, "null weight pointer");
  GatherArgs a{};
  a.exact = 1;
  a.n_items = n_rows, a.pointer = pointer, a.idx = node_idx, a.eidx = edge_idx, a.x = x, a.y = y, a.w = w;
  a.F = (int32_t)(heads * dim), a.H = (int32_t)heads;
  return dispatch<float, MUL_E>(plan, a, (int32_t)dim, static_cast<cudaStream_t>(stream));
}

// Aggregation half of the fused attention operator (the statistics half lives in softmax.cu).
namespace gphl {
int gat_aggregate_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx, const int32_t *edge_idx,
                      int64_t n_rows, int64_t heads, int64_t dim, const float *el, const float *er, const float *z,
                      float slope, float *out, float *alpha_out, const float *stats, int32_t flags, cudaStream_t stream) {
  GatherArgs a{};
  a.exact = (flags & GPHL_ACCUM_FAST) ? 0 : 1;
  a.n_items = n_rows, a.pointer = pointer, a.idx = node_idx, a.eidx = edge_idx, a.x = z, a.y = out;
  a.el = el, a.er = er, a.stats = stats, a.alpha_out = alpha_out, a.slope = slope;
  a.F = (int32_t)(heads * dim), a.H = (int32_t)heads;
  return dispatch<float, GAT>(plan, a, (int32_t)dim, stream);
}
int gat_aggregate_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx, int64_t n_rows,
                       int64_t heads, int64_t dim, const float *el, const float *er, const void *z, float slope,
                       void *out, const float *stats, int32_t flags, cudaStream_t stream) {
  GatherArgs a{};
  a.exact = (flags & GPHL_ACCUM_FAST) ? 0 : 1;
  a.n_items = n_rows, a.pointer = pointer, a.idx = node_idx, a.x = z, a.y = out;
  a.el = el, a.er = er, a.stats = stats, a.slope = slope;
  a.F = (int32_t)(heads * dim), a.H = (int32_t)heads;
  return dispatch<__nv_bfloat16, GAT>(plan, a, (int32_t)dim, stream);
}
}  // namespace gphl
