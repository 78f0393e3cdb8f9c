// Per-destination (segment) softmax for sm_100a, multi-head, and the statistics half of the
// fused attention operator.
//
// Pass 1 (stats): one warp per work item; lanes are laid out as (edge sub-batch x head) so
// that the H logits of one edge are one coalesced access; every lane keeps an online
// (maximum, exp-sum) pair, initialised at -inf, and the sub-batches are merged with
// shuffles.  Pieces of cut rows leave partial pairs in the plan's scratch and a merge
// kernel combines them in ascending order.  Pass 2 (normalise) writes exp(x - max) / sum at
// every edge id.  The fused operator replaces pass 2 by the weighted gather in spmm.cu.
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

template <bool GAT_LOGITS>
__global__ void __launch_bounds__(SW * 32) segment_stats_kernel(StatsArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item_id = (int64_t)blockIdx.x * SW + warp;
  if (item_id >= a.n_items) return;
  const Item it = fetch_item(a.items, a.pointer, item_id);
  const int hl = lane % a.Hp, eg = lane / a.Hp, epw = 32 / a.Hp;
  for (int h0 = 0; h0 < a.H; h0 += a.Hp) {
    const int h = h0 + hl;
    const bool hok = h < a.H;
    MaxSum ms;
    ms.init();
    const float erv = (GAT_LOGITS && hok) ? __ldg(a.er + (int64_t)it.row * a.H + h) : 0.f;
    if (hok) {
      auto logit = [&](int i) {
        if (GAT_LOGITS) {
          const int src = __ldg(a.idx + i);
          return leaky(__ldg(a.el + (int64_t)src * a.H + h) + erv, a.slope);
        }
        const int eid = a.eidx ? __ldg(a.eidx + i) : i;
        return __ldg(a.x + (int64_t)eid * a.H + h);
      };
      int i = it.begin + eg;
      for (; i + 3 * epw < it.end; i += 4 * epw) {        // four dependent index -> value chains in flight
        const float v0 = logit(i), v1 = logit(i + epw), v2 = logit(i + 2 * epw), v3 = logit(i + 3 * epw);
        ms.push(v0), ms.push(v1), ms.push(v2), ms.push(v3);
      }
      for (; i < it.end; i += epw) ms.push(logit(i));
    }
    __syncwarp();
    for (int off = a.Hp; off < 32; off <<= 1) {
      const float om = __shfl_xor_sync(FULL, ms.m, off);
      const float os = __shfl_xor_sync(FULL, ms.s, off);
      // identical on both partners: merge the lower sub-batch first
      if ((lane & off) == 0) {
        ms.merge(om, os);
      } else {
        MaxSum t{om, os};
        t.merge(ms.m, ms.s);
        ms = t;
      }
    }
    if (eg == 0 && hok) {
      if (it.slot < 0) {
        float2 o = ms.s > 0.f ? make_float2(ms.m, 1.f / ms.s) : make_float2(0.f, 0.f);
        reinterpret_cast<float2 *>(a.stats)[(int64_t)it.row * a.H + h] = o;
      } else {
        reinterpret_cast<float2 *>(a.scratch)[(int64_t)it.slot * a.H + h] = make_float2(ms.m, ms.s);
      }
    }
  }
}

__global__ void stats_merge_kernel(const int32_t *split_rows, const int32_t *split_ptr, int64_t n_split, int32_t H,
                                   const float *scratch, float *stats) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_split * H) return;
  const int64_t r = t / H;
  const int h = (int)(t % H);
  MaxSum ms;
  ms.init();
  for (int s = split_ptr[r]; s < split_ptr[r + 1]; ++s) {
    const float2 p = reinterpret_cast<const float2 *>(scratch)[(int64_t)s * H + h];
    ms.merge(p.x, p.y);
  }
  float2 o = ms.s > 0.f ? make_float2(ms.m, 1.f / ms.s) : make_float2(0.f, 0.f);
  reinterpret_cast<float2 *>(stats)[(int64_t)split_rows[r] * H + h] = o;
}

__global__ void __launch_bounds__(SW * 32) softmax_normalize_kernel(StatsArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item_id = (int64_t)blockIdx.x * SW + warp;
  if (item_id >= a.n_items) return;
  const Item it = fetch_item(a.items, a.pointer, item_id);
  const int hl = lane % a.Hp, eg = lane / a.Hp, epw = 32 / a.Hp;
  for (int h0 = 0; h0 < a.H; h0 += a.Hp) {
    const int h = h0 + hl;
    if (h >= a.H) continue;
    const float2 st = __ldg(reinterpret_cast<const float2 *>(a.stats) + (int64_t)it.row * a.H + h);
    for (int i = it.begin + eg; i < it.end; i += epw) {
      const int eid = a.eidx ? __ldg(a.eidx + i) : i;
      const int64_t o = (int64_t)eid * a.H + h;
      a.y[o] = expf(__ldg(a.x + o) - st.x) * st.y;
    }
  }
}

static int lanes_per_edge(int64_t H) {
  int hp = 1;
  while (hp < H && hp < 32) hp <<= 1;
  return hp;
}

template <bool GAT_LOGITS>
static int run_stats(const gphl_plan *plan, StatsArgs a, int64_t n_rows, cudaStream_t stream) {
  if (plan) {
    a.items = plan->items, a.n_items = plan->n_items, a.scratch = plan->scratch;
    if (plan->n_pieces > 0 && a.H > plan->max_feat)
      return fail(GPHL_ERR_TOO_LARGE, "head count %d exceeds the plan's scratch width %lld", a.H,
                  (long long)plan->max_feat);
  } else {
    a.n_items = n_rows;
  }
  a.Hp = lanes_per_edge(a.H);
  segment_stats_kernel<GAT_LOGITS><<<(unsigned)((a.n_items + SW - 1) / SW), SW * 32, 0, stream>>>(a);
  int rc = launched("segment_stats_kernel");
  if (rc != GPHL_OK) return rc;
  if (plan && plan->n_split_rows > 0) {
    const int64_t total = plan->n_split_rows * a.H;
    stats_merge_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(plan->split_rows, plan->split_ptr,
                                                                          plan->n_split_rows, a.H, plan->scratch, a.stats);
    rc = launched("stats_merge_kernel");
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
  int rc = run_stats<false>(plan, a, n_rows, stream);
  if (rc != GPHL_OK) return rc;
  if (plan) a.items = plan->items, a.n_items = plan->n_items;
  else a.n_items = n_rows;
  a.Hp = lanes_per_edge(heads);
  softmax_normalize_kernel<<<(unsigned)((a.n_items + SW - 1) / SW), SW * 32, 0, stream>>>(a);
  return launched("softmax_normalize_kernel");
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
  rc = run_stats<true>(plan, a, n_rows, stream);
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
  rc = run_stats<true>(plan, a, n_rows, stream);
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
  if (n_rows > 0 && (heads > GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS || n_rows > GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS / heads))
    return fail(GPHL_ERR_TOO_LARGE,
                "segment_softmax_noalloc: n_rows * heads = %lld exceeds the built-in scratch of %d (row, head) pairs; "
                "use gphl_segment_softmax_f32 with caller-provided scratch",
                (long long)(n_rows * heads), GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS);
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
