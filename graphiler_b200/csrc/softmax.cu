// Per-destination (segment) softmax for sm_100a, multi-head, and the statistics half of the
// fused attention operator.
//
// Pass 1 (stats): one warp per work item; lanes are laid out as (edge sub-batch x head group) so
// that the H logits of one edge are one coalesced access (16-byte loads of four heads when H is
// a multiple of four); every lane keeps online (maximum, exp-sum) pairs, initialised at -inf,
// and the sub-batches are merged with shuffles.  An item that is a whole row then writes
// exp(x - max) / sum in a second sweep over the logits it has just read.  Pieces of cut rows
// leave partial pairs in the plan's scratch, a merge kernel combines them in ascending order and
// pass 2 (normalise) writes their outputs.  The fused attention operator uses pass 1 only and
// replaces the rest by the weighted gather in spmm.cu.
#include <mutex>

#include "common.cuh"

namespace gphl {

int gat_aggregate_f32(const gphl_plan *, const int32_t *, const int32_t *, const int32_t *, int64_t, int64_t, int64_t,
                      const float *, const float *, const float *, float, float *, float *, const float *, int32_t,
                      cudaStream_t);
int gat_aggregate_bf16(const gphl_plan *, const int32_t *, const int32_t *, int64_t, int64_t, int64_t, const float *,
                       const float *, const void *, float, void *, const float *, int32_t, cudaStream_t);

struct StatsArgs {
  const Item *items;
  int64_t n_items;
  const int32_t *pointer;
  const int32_t *idx;   // GAT: source node per position
  const int32_t *eidx;  // logits mode: edge id per position (NULL: position)
  const float *x;       // logits mode: (n_edges, H)
  const float *el, *er; // GAT
  float slope;
  float *stats;         // (n_rows, H, 2)
  float *scratch;       // (n_pieces, H, 2) partial pairs
  float *y;             // normalise pass output
  int32_t H, Hp;        // heads, lanes per edge (power of two >= min(H, 32))
};

constexpr int SW = 8;  // warps per block

// V consecutive heads of one edge per lane: V = 4 turns the H logits of an edge into 16-byte accesses
// (heads % 4 == 0 and 16-byte aligned arrays), V = 1 is the general layout.
template <int V>
struct HeadVec {
  float v[V];
};
template <int V>
__device__ __forceinline__ HeadVec<V> load_heads(const float *p) {
  HeadVec<V> r;
  if constexpr (V == 4) {
    const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    r.v[0] = t.x, r.v[1] = t.y, r.v[2] = t.z, r.v[3] = t.w;
  } else {
    r.v[0] = __ldg(p);
  }
  return r;
}
template <int V>
__device__ __forceinline__ void store_heads(float *p, const HeadVec<V> &r) {
  if constexpr (V == 4) *reinterpret_cast<float4 *>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  else *p = r.v[0];
}

// Pass 1.  NORMALIZE (logits mode only): an item that is a whole row also writes its outputs in
// a second sweep over the row, which the warp has just pulled through L2, so that pass 2 is
// left with the pieces of cut rows.
template <bool GAT_LOGITS, int V, bool NORMALIZE>
__global__ void __launch_bounds__(SW * 32) segment_stats_kernel(StatsArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item_id = (int64_t)blockIdx.x * SW + warp;
  if (item_id >= a.n_items) return;
  const Item it = fetch_item(a.items, a.pointer, item_id);
  const int hl = lane % a.Hp, eg = lane / a.Hp, epw = 32 / a.Hp;
  for (int h0 = 0; h0 < a.H; h0 += a.Hp * V) {
    const int h = h0 + hl * V;
    const bool hok = h < a.H;
    MaxSum ms[V];
#pragma unroll
    for (int v = 0; v < V; ++v) ms[v].init();
    HeadVec<V> erv;
#pragma unroll
    for (int v = 0; v < V; ++v) erv.v[v] = 0.f;
    if (GAT_LOGITS && hok) erv = load_heads<V>(a.er + (int64_t)it.row * a.H + h);
    auto logit = [&](int i) {
      if (GAT_LOGITS) {
        const int src = __ldg(a.idx + i);
        HeadVec<V> r = load_heads<V>(a.el + (int64_t)src * a.H + h);
#pragma unroll
        for (int v = 0; v < V; ++v) r.v[v] = leaky(r.v[v] + erv.v[v], a.slope);
        return r;
      }
      const int eid = a.eidx ? __ldg(a.eidx + i) : i;
      return load_heads<V>(a.x + (int64_t)eid * a.H + h);
    };
    if (hok) {
      int i = it.begin + eg;
      for (; i + 3 * epw < it.end; i += 4 * epw) {        // four dependent index -> value chains in flight
        const HeadVec<V> v0 = logit(i), v1 = logit(i + epw), v2 = logit(i + 2 * epw), v3 = logit(i + 3 * epw);
#pragma unroll
        for (int v = 0; v < V; ++v) ms[v].push4(v0.v[v], v1.v[v], v2.v[v], v3.v[v]);
      }
      for (; i < it.end; i += epw) {
        const HeadVec<V> v0 = logit(i);
#pragma unroll
        for (int v = 0; v < V; ++v) ms[v].push(v0.v[v]);
      }
    }
    __syncwarp();
    // combine the sub-batches: common maximum, rescale each lane's sum to it, add (the butterfly leaves the same
    // pair on every lane of a head group)
#pragma unroll
    for (int v = 0; v < V; ++v) {
      float mr = ms[v].m;
      for (int off = a.Hp; off < 32; off <<= 1) mr = fmaxf(mr, __shfl_xor_sync(FULL, mr, off));
      float sc = ms[v].s > 0.f ? ms[v].s * exp_neg(ms[v].m - mr) : 0.f;
      for (int off = a.Hp; off < 32; off <<= 1) sc += __shfl_xor_sync(FULL, sc, off);
      ms[v].m = mr, ms[v].s = sc;
    }
    if (!hok) continue;
    if (it.slot >= 0) {
      if (eg == 0) {
#pragma unroll
        for (int v = 0; v < V; ++v)
          reinterpret_cast<float2 *>(a.scratch)[(int64_t)it.slot * a.H + h + v] = make_float2(ms[v].m, ms[v].s);
      }
      continue;
    }
    HeadVec<V> mx, inv;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const bool any = ms[v].s > 0.f;
      mx.v[v] = any ? ms[v].m : 0.f, inv.v[v] = any ? 1.f / ms[v].s : 0.f;
    }
    if (eg == 0) {
#pragma unroll
      for (int v = 0; v < V; ++v)
        reinterpret_cast<float2 *>(a.stats)[(int64_t)it.row * a.H + h + v] = make_float2(mx.v[v], inv.v[v]);
    }
    if (NORMALIZE) {                                       // every lane of a head group holds the row's pair
      auto emit = [&](int i, const HeadVec<V> &x) {
        const int eid = a.eidx ? __ldg(a.eidx + i) : i;
        HeadVec<V> y;
#pragma unroll
        for (int v = 0; v < V; ++v) y.v[v] = exp_neg(x.v[v] - mx.v[v]) * inv.v[v];
        store_heads<V>(a.y + (int64_t)eid * a.H + h, y);
      };
      int i = it.begin + eg;
      for (; i + 3 * epw < it.end; i += 4 * epw) {
        const HeadVec<V> v0 = logit(i), v1 = logit(i + epw), v2 = logit(i + 2 * epw), v3 = logit(i + 3 * epw);
        emit(i, v0), emit(i + epw, v1), emit(i + 2 * epw, v2), emit(i + 3 * epw, v3);
      }
      for (; i < it.end; i += epw) emit(i, logit(i));
    }
  }
}

// Pass 1 for short items (at most GPHL_SHORT_ITEM positions), which are most rows of a sparse graph: one thread
// per (item, group of V heads) walks the item's positions, so a warp serves 32 / (H / V) items and the per-item
// bookkeeping is shared by as many.  The plan orders items by length, so the threads of a warp run equally long.
// Same arithmetic per (row, head) as the warp kernel up to the order in which positions are combined.
template <bool GAT_LOGITS, int V, bool NORMALIZE>
__global__ void __launch_bounds__(256) segment_stats_rows_kernel(StatsArgs a, int64_t first_item, int32_t units) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t item_id = first_item + t / units;
  if (item_id >= a.n_items) return;
  const int h = (int)(t % units) * V;
  const Item it = fetch_item(a.items, a.pointer, item_id);
  MaxSum ms[V];
#pragma unroll
  for (int v = 0; v < V; ++v) ms[v].init();
  HeadVec<V> erv;
#pragma unroll
  for (int v = 0; v < V; ++v) erv.v[v] = 0.f;
  if (GAT_LOGITS) erv = load_heads<V>(a.er + (int64_t)it.row * a.H + h);
  auto logit = [&](int i) {
    if (GAT_LOGITS) {
      const int src = __ldg(a.idx + i);
      HeadVec<V> r = load_heads<V>(a.el + (int64_t)src * a.H + h);
#pragma unroll
      for (int v = 0; v < V; ++v) r.v[v] = leaky(r.v[v] + erv.v[v], a.slope);
      return r;
    }
    const int eid = a.eidx ? __ldg(a.eidx + i) : i;
    return load_heads<V>(a.x + (int64_t)eid * a.H + h);
  };
  int i = it.begin;
  for (; i + 3 < it.end; i += 4) {
    const HeadVec<V> v0 = logit(i), v1 = logit(i + 1), v2 = logit(i + 2), v3 = logit(i + 3);
#pragma unroll
    for (int v = 0; v < V; ++v) ms[v].push4(v0.v[v], v1.v[v], v2.v[v], v3.v[v]);
  }
  for (; i < it.end; ++i) {
    const HeadVec<V> v0 = logit(i);
#pragma unroll
    for (int v = 0; v < V; ++v) ms[v].push(v0.v[v]);
  }
  if (it.slot >= 0) {
#pragma unroll
    for (int v = 0; v < V; ++v)
      reinterpret_cast<float2 *>(a.scratch)[(int64_t)it.slot * a.H + h + v] = make_float2(ms[v].m, ms[v].s);
    return;
  }
  HeadVec<V> mx, inv;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const bool any = ms[v].s > 0.f;
    mx.v[v] = any ? ms[v].m : 0.f, inv.v[v] = any ? 1.f / ms[v].s : 0.f;
    reinterpret_cast<float2 *>(a.stats)[(int64_t)it.row * a.H + h + v] = make_float2(mx.v[v], inv.v[v]);
  }
  if (NORMALIZE) {
    auto emit = [&](int j, const HeadVec<V> &x) {
      const int eid = a.eidx ? __ldg(a.eidx + j) : j;
      HeadVec<V> y;
#pragma unroll
      for (int v = 0; v < V; ++v) y.v[v] = exp_neg(x.v[v] - mx.v[v]) * inv.v[v];
      store_heads<V>(a.y + (int64_t)eid * a.H + h, y);
    };
    i = it.begin;
    for (; i + 3 < it.end; i += 4) {
      const HeadVec<V> v0 = logit(i), v1 = logit(i + 1), v2 = logit(i + 2), v3 = logit(i + 3);
      emit(i, v0), emit(i + 1, v1), emit(i + 2, v2), emit(i + 3, v3);
    }
    for (; i < it.end; ++i) emit(i, logit(i));
  }
}

// Combines the partial pairs of a cut row: one warp per (cut row, head), lanes striding over the row's pieces.
__global__ void __launch_bounds__(256) stats_merge_kernel(const int32_t *split_rows, const int32_t *split_ptr,
                                                         int64_t n_split, int32_t H, const float *scratch,
                                                         float *stats) {
  const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= n_split * H) return;
  const int64_t r = w / H;
  const int h = (int)(w % H);
  MaxSum ms;
  ms.init();
  for (int s = split_ptr[r] + lane; s < split_ptr[r + 1]; s += 32) {
    const float2 p = reinterpret_cast<const float2 *>(scratch)[(int64_t)s * H + h];
    ms.merge(p.x, p.y);
  }
  float mr = ms.m;
  for (int off = 1; off < 32; off <<= 1) mr = fmaxf(mr, __shfl_xor_sync(FULL, mr, off));
  float sc = ms.s > 0.f ? ms.s * exp_neg(ms.m - mr) : 0.f;
  for (int off = 1; off < 32; off <<= 1) sc += __shfl_xor_sync(FULL, sc, off);
  if (lane == 0) {
    float2 o = sc > 0.f ? make_float2(mr, 1.f / sc) : make_float2(0.f, 0.f);
    reinterpret_cast<float2 *>(stats)[(int64_t)split_rows[r] * H + h] = o;
  }
}

// Pass 2 for the cut rows (the others were finished by pass 1): one block per piece, so that a hub row of 10^5
// positions is spread over hundreds of blocks.  Pieces of a cut row are `chunk` positions each (the last one
// shorter) and their scratch slots are consecutive, so the slot number gives the row (search in split_ptr) and
// the position range.
template <int V>
__global__ void __launch_bounds__(256) softmax_normalize_kernel(StatsArgs a, const int32_t *split_rows,
                                                               const int32_t *split_ptr, int32_t n_split,
                                                               int32_t chunk) {
  __shared__ int s_row, s_begin, s_end;
  if (threadIdx.x == 0) {
    const int slot = blockIdx.x;
    int lo = 0, hi = n_split - 1;                       // last r with split_ptr[r] <= slot
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (__ldg(split_ptr + mid) <= slot) lo = mid;
      else hi = mid - 1;
    }
    const int row = __ldg(split_rows + lo);
    const int begin = __ldg(a.pointer + row) + (slot - __ldg(split_ptr + lo)) * chunk;
    s_row = row, s_begin = begin, s_end = min(begin + chunk, __ldg(a.pointer + row + 1));
  }
  __syncthreads();
  const int row = s_row, begin = s_begin, end = s_end;
  const int units = a.H / V;
  const int total = (end - begin) * units;
  for (int t = threadIdx.x; t < total; t += blockDim.x) {
    const int i = begin + t / units, h = (t % units) * V;
    const int eid = a.eidx ? __ldg(a.eidx + i) : i;
    const HeadVec<V> x = load_heads<V>(a.x + (int64_t)eid * a.H + h);
    HeadVec<V> y;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const float2 st = __ldg(reinterpret_cast<const float2 *>(a.stats) + (int64_t)row * a.H + h + v);
      y.v[v] = exp_neg(x.v[v] - st.x) * st.y;
    }
    store_heads<V>(a.y + (int64_t)eid * a.H + h, y);
  }
}

static int lanes_per_edge(int64_t units) {
  int hp = 1;
  while (hp < units && hp < 32) hp <<= 1;
  return hp;
}

// Statistics of every row; with NORMALIZE also the outputs of the rows that were not cut.
template <bool GAT_LOGITS, bool NORMALIZE>
static int run_stats(const gphl_plan *plan, StatsArgs a, int64_t n_rows, cudaStream_t stream) {
  if (plan) {
    a.items = plan->items, a.n_items = plan->n_items, a.scratch = plan->scratch;
    if (plan->n_pieces > 0 && a.H > plan->max_feat)
      return fail(GPHL_ERR_TOO_LARGE, "head count %d exceeds the plan's scratch width %lld", a.H,
                  (long long)plan->max_feat);
  } else {
    a.n_items = n_rows;
  }
  const bool vec = a.H % 4 == 0 && (GAT_LOGITS ? aligned16(a.el) && aligned16(a.er) : aligned16(a.x) && aligned16(a.y));
  a.Hp = lanes_per_edge(vec ? a.H / 4 : a.H);
  // long items: a warp each; short items (the plan puts them last): a thread per (item, head group)
  const int64_t n_warp_items = plan ? plan->n_long_items : a.n_items;
  int rc = GPHL_OK;
  if (n_warp_items > 0) {
    StatsArgs w = a;
    w.n_items = n_warp_items;
    const unsigned grid = (unsigned)((n_warp_items + SW - 1) / SW);
    if (vec) segment_stats_kernel<GAT_LOGITS, 4, NORMALIZE><<<grid, SW * 32, 0, stream>>>(w);
    else segment_stats_kernel<GAT_LOGITS, 1, NORMALIZE><<<grid, SW * 32, 0, stream>>>(w);
    rc = launched("segment_stats_kernel");
    if (rc != GPHL_OK) return rc;
  }
  if (a.n_items > n_warp_items) {
    const int32_t units = vec ? a.H / 4 : a.H;
    const int64_t threads = (a.n_items - n_warp_items) * units;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    if (vec) segment_stats_rows_kernel<GAT_LOGITS, 4, NORMALIZE><<<grid, 256, 0, stream>>>(a, n_warp_items, units);
    else segment_stats_rows_kernel<GAT_LOGITS, 1, NORMALIZE><<<grid, 256, 0, stream>>>(a, n_warp_items, units);
    rc = launched("segment_stats_rows_kernel");
    if (rc != GPHL_OK) return rc;
  }
  if (plan && plan->n_split_rows > 0) {
    const int64_t total = plan->n_split_rows * a.H * 32;
    stats_merge_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(plan->split_rows, plan->split_ptr,
                                                                          plan->n_split_rows, a.H, plan->scratch, a.stats);
    rc = launched("stats_merge_kernel");
    if (rc != GPHL_OK || !NORMALIZE) return rc;
    const unsigned pieces = (unsigned)plan->n_pieces;
    if (vec)
      softmax_normalize_kernel<4><<<pieces, 256, 0, stream>>>(a, plan->split_rows, plan->split_ptr,
                                                               (int32_t)plan->n_split_rows, plan->chunk);
    else
      softmax_normalize_kernel<1><<<pieces, 256, 0, stream>>>(a, plan->split_rows, plan->split_ptr,
                                                               (int32_t)plan->n_split_rows, plan->chunk);
    rc = launched("softmax_normalize_kernel");
  }
  return rc;
}

}  // namespace gphl

using namespace gphl;

extern "C" int gphl_segment_softmax_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *edge_idx,
                                        int64_t n_rows, int64_t heads, const float *x, float *y, float *stats,
                                        void *stream_) {
  GPHL_REQUIRE(n_rows >= 0 && heads >= 1 && n_rows < INT32_MAX && heads < (1 << 20), "bad sizes");
  if (n_rows == 0) return GPHL_OK;
  GPHL_REQUIRE(pointer && x && y && stats, "null pointer argument");
  GPHL_REQUIRE(!plan || plan->n_rows == n_rows, "plan was built for a different row count");
  GPHL_REQUIRE((reinterpret_cast<uintptr_t>(stats) & 7u) == 0, "stats must be 8-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  StatsArgs a{};
  a.pointer = pointer, a.eidx = edge_idx, a.x = x, a.y = y, a.stats = stats, a.H = (int32_t)heads;
  return run_stats<false, true>(plan, a, n_rows, stream);
}

static int gat_check(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx, int64_t n_rows,
                     int64_t heads, int64_t dim, const void *el, const void *er, const void *z, const void *out,
                     const void *stats) {
  GPHL_REQUIRE(n_rows >= 0 && heads >= 1 && dim >= 1 && n_rows < INT32_MAX && heads * dim < (1 << 20), "bad sizes");
  if (n_rows == 0) return GPHL_OK;
  GPHL_REQUIRE(pointer && node_idx && el && er && z && out && stats, "null pointer argument");
  GPHL_REQUIRE(!plan || plan->n_rows == n_rows, "plan was built for a different row count");
  GPHL_REQUIRE((reinterpret_cast<uintptr_t>(stats) & 7u) == 0, "stats must be 8-byte aligned");
  return GPHL_OK;
}

extern "C" int gphl_gat_fused_ex_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                                     const int32_t *edge_idx, int64_t n_rows, int64_t heads, int64_t dim,
                                     const float *el, const float *er, const float *z, float slope, int32_t flags,
                                     float *out, float *alpha_out, float *stats, void *stream_) {
  GPHL_REQUIRE((flags & ~GPHL_ACCUM_FAST) == 0, "unknown flag bits");
  int rc = gat_check(plan, pointer, node_idx, n_rows, heads, dim, el, er, z, out, stats);
  if (rc != GPHL_OK || n_rows == 0) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  StatsArgs a{};
  a.pointer = pointer, a.idx = node_idx, a.el = el, a.er = er, a.slope = slope, a.stats = stats, a.H = (int32_t)heads;
  rc = run_stats<true, false>(plan, a, n_rows, stream);
  if (rc != GPHL_OK) return rc;
  return gat_aggregate_f32(plan, pointer, node_idx, edge_idx, n_rows, heads, dim, el, er, z, slope, out, alpha_out,
                           stats, flags, stream);
}

extern "C" int gphl_gat_fused_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                                  const int32_t *edge_idx, int64_t n_rows, int64_t heads, int64_t dim, const float *el,
                                  const float *er, const float *z, float slope, float *out, float *alpha_out,
                                  float *stats, void *stream) {
  return gphl_gat_fused_ex_f32(plan, pointer, node_idx, edge_idx, n_rows, heads, dim, el, er, z, slope, 0, out,
                               alpha_out, stats, stream);
}

extern "C" int gphl_gat_fused_ex_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                                      int64_t n_rows, int64_t heads, int64_t dim, const float *el, const float *er,
                                      const void *z, float slope, int32_t flags, void *out, float *stats,
                                      void *stream_) {
  GPHL_REQUIRE((flags & ~GPHL_ACCUM_FAST) == 0, "unknown flag bits");
  int rc = gat_check(plan, pointer, node_idx, n_rows, heads, dim, el, er, z, out, stats);
  if (rc != GPHL_OK || n_rows == 0) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  StatsArgs a{};
  a.pointer = pointer, a.idx = node_idx, a.el = el, a.er = er, a.slope = slope, a.stats = stats, a.H = (int32_t)heads;
  rc = run_stats<true, false>(plan, a, n_rows, stream);
  if (rc != GPHL_OK) return rc;
  return gat_aggregate_bf16(plan, pointer, node_idx, n_rows, heads, dim, el, er, z, slope, out, stats, flags, stream);
}

extern "C" int gphl_gat_fused_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                                   int64_t n_rows, int64_t heads, int64_t dim, const float *el, const float *er,
                                   const void *z, float slope, void *out, float *stats, void *stream) {
  return gphl_gat_fused_ex_bf16(plan, pointer, node_idx, n_rows, heads, dim, el, er, z, slope, 0, out, stats, stream);
}

// ---- segment softmax for callers that must not allocate ---------------------------------------
//
// The row statistics (maximum, reciprocal exp-sum per row and head) normally live in scratch the
// caller hands in.  Some callers have no way to provide device scratch: a host process that gave
// all device memory to its own pool at start-up and forbids cudaMalloc afterwards (cudaMalloc
// synchronises the device and its latency is unbounded), or a plugin inside a framework that owns
// the allocator and offers plugins no allocation hook.  For them the statistics live in the
// fixed array below, which is part of the library image: every GPU that loads the library holds
// these 8 MiB until the process exits.
//
// In host code `g_softmax_stats` is only a handle for the runtime, not a device address; the
// address is looked up once per device with cudaGetSymbolAddress and cached.
static __device__ __align__(256) float g_softmax_stats[2 * GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
float *g_noalloc_stats[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int gphl_segment_softmax_noalloc_f32(const int32_t *pointer, const int32_t *edge_idx, int64_t n_rows,
                                                int64_t heads, const float *x, float *y, void *stream) {
  GPHL_REQUIRE(n_rows >= 0 && heads >= 1, "bad sizes");
  // the documented limit, checked without forming a product that could overflow: n_rows * heads <= capacity, and the
  // head count itself below the regular entry point's limit (2^20), so that what passes here passes there too
  if (heads >= GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS || (n_rows > 0 && n_rows > GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS / heads))
    return fail(GPHL_ERR_TOO_LARGE,
                "segment_softmax_noalloc: %lld rows x %lld heads exceed the built-in scratch of %d (row, head) pairs "
                "(and fewer than %d heads); use gphl_segment_softmax_f32 with caller-provided scratch",
                (long long)n_rows, (long long)heads, GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS, GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS);
  int dev = 0;
  GPHL_CUDA(cudaGetDevice(&dev));
  GPHL_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal out of range");
  float *stats = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_stats[dev] == nullptr) {
      // set-up for this device (it is the current one): resolve the array's device address
      void *p = nullptr;
      GPHL_CUDA(cudaGetSymbolAddress(&p, g_softmax_stats));
      g_noalloc_stats[dev] = static_cast<float *>(p);
    }
    stats = g_noalloc_stats[dev];
  }
  // Pass 1 writes the pair of every (row, head) that pass 2 reads, so nothing left behind by an
  // earlier call is ever consumed and the array needs no clearing.
  return gphl_segment_softmax_f32(nullptr, pointer, edge_idx, n_rows, heads, x, y, stats, stream);
}
