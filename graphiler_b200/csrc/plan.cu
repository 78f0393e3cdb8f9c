// Host side of the library: error state, launch counter and the row-split plan.
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace gphl {

static thread_local std::string t_error;
std::atomic<int64_t> g_launches{0};

void set_error(const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_error = buf;
}

#ifdef GPHL_MEASURE
int knob(const char *name, int dflt) {
  const char *e = getenv(name);
  return e ? atoi(e) : dflt;
}
#endif

}  // namespace gphl

using namespace gphl;

extern "C" const char *gphl_last_error(void) { return t_error.c_str(); }
extern "C" int gphl_version(void) { return (0 << 16) | 1; }
extern "C" int64_t gphl_launch_count(void) { return g_launches.load(); }

extern "C" int gphl_plan_create(const int32_t *pointer, int64_t n_rows, int32_t chunk, int64_t max_feat,
                                void *stream_, gphl_plan **out_plan) {
  GPHL_REQUIRE(out_plan != nullptr, "plan_create: out_plan is NULL");
  *out_plan = nullptr;
  GPHL_REQUIRE(pointer != nullptr && n_rows >= 0, "plan_create: bad pointer array");
  GPHL_REQUIRE(chunk >= 32 && chunk % 32 == 0, "plan_create: chunk must be a positive multiple of 32");
  GPHL_REQUIRE(max_feat >= 0, "plan_create: max_feat must be >= 0");
  GPHL_REQUIRE(n_rows < INT32_MAX, "plan_create: row count must fit int32");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  std::vector<int32_t> ptr(n_rows + 1);
  GPHL_CUDA(cudaMemcpyAsync(ptr.data(), pointer, sizeof(int32_t) * (n_rows + 1), cudaMemcpyDeviceToHost, stream));
  GPHL_CUDA(cudaStreamSynchronize(stream));

  std::vector<Item> items;
  items.reserve(n_rows + n_rows / 8 + 16);
  std::vector<int32_t> split_rows, split_ptr;
  split_ptr.push_back(0);
  int32_t slot = 0;
  int64_t n_long = 0;
  for (int64_t v = 0; v < n_rows; ++v) {
    const int32_t b = ptr[v], e = ptr[v + 1];
    if (e < b) return fail(GPHL_ERR_INVALID_ARGUMENT, "plan_create: pointer array decreases at row %lld", (long long)v);
    if (e - b <= chunk) {
      items.push_back(Item{(int32_t)v, b, e, -1});
    } else {
      for (int32_t s = b; s < e; s += chunk) items.push_back(Item{(int32_t)v, s, std::min(e, s + chunk), slot++});
      split_rows.push_back((int32_t)v);
      split_ptr.push_back(slot);
    }
  }

  // Launch order: longest pieces first (stable counting sort on the piece length), so that the
  // warps of one block finish together and no long piece is left for the tail of the launch.
  // Scratch slots were assigned in row order above and do not move.
  {
    std::vector<int64_t> start((size_t)chunk + 2, 0);
    for (const Item &it : items) start[(size_t)(chunk - (it.end - it.begin)) + 1]++;
    for (size_t i = 1; i < start.size(); ++i) start[i] += start[i - 1];
    // buckets are ordered by falling length: the long items are those in front of the first short bucket
    const int32_t short_item = std::max(0, knob("GPHL_SHORT_ITEM", GPHL_SHORT_ITEM));
    n_long = chunk > short_item ? start[(size_t)(chunk - short_item)] : 0;
    std::vector<Item> sorted(items.size());
    for (const Item &it : items) sorted[(size_t)start[(size_t)(chunk - (it.end - it.begin))]++] = it;
    items.swap(sorted);
  }

  gphl_plan *p = new gphl_plan();
  p->n_rows = n_rows;
  p->chunk = chunk;
  p->n_items = (int64_t)items.size();
  p->n_split_rows = (int64_t)split_rows.size();
  p->n_pieces = slot;
  p->n_long_items = n_long;
  // rows are padded to a multiple of 8 columns so that 16-byte accesses to scratch stay aligned
  p->max_feat = (max_feat + 7) / 8 * 8;
  p->scratch_bytes = (int64_t)sizeof(float) * 2 * p->n_pieces * p->max_feat;

  auto upload = [&](void **dst, const void *src, size_t bytes) -> cudaError_t {
    *dst = nullptr;
    if (bytes == 0) return cudaSuccess;
    cudaError_t e = cudaMalloc(dst, bytes);
    if (e != cudaSuccess) return e;
    return cudaMemcpyAsync(*dst, src, bytes, cudaMemcpyHostToDevice, stream);
  };
  cudaError_t e = upload((void **)&p->items, items.data(), sizeof(Item) * items.size());
  if (e == cudaSuccess) e = upload((void **)&p->split_rows, split_rows.data(), sizeof(int32_t) * split_rows.size());
  if (e == cudaSuccess && p->n_split_rows > 0)
    e = upload((void **)&p->split_ptr, split_ptr.data(), sizeof(int32_t) * split_ptr.size());
  if (e == cudaSuccess && p->scratch_bytes > 0) e = cudaMalloc((void **)&p->scratch, p->scratch_bytes);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);  // the host vectors die with this frame
  if (e != cudaSuccess) {
    gphl_plan_destroy(p);
    return fail(GPHL_ERR_CUDA, "plan_create: %s", cudaGetErrorString(e));
  }
  *out_plan = p;
  return GPHL_OK;
}

extern "C" void gphl_plan_destroy(gphl_plan *p) {
  if (!p) return;
  cudaFree(p->items);
  cudaFree(p->split_rows);
  cudaFree(p->split_ptr);
  if (p->owns_scratch) cudaFree(p->scratch);
  delete p;
}

// Scratch handed in by the caller (2 * num_pieces * round_up(max_feat, 8) floats, 16-byte aligned) in place of scratch
// the plan owns: a plan created with max_feat = 0 owns none, and a caller with its own allocator binds a buffer wide
// enough for the next calls.  Not thread-safe against calls that use the plan at the same time.
extern "C" int gphl_plan_bind_scratch(gphl_plan *p, void *scratch, int64_t max_feat) {
  GPHL_REQUIRE(p != nullptr && max_feat >= 0, "plan_bind_scratch: bad arguments");
  GPHL_REQUIRE(p->n_pieces == 0 || max_feat == 0 || (scratch != nullptr && aligned16(scratch)),
               "plan_bind_scratch: scratch must be a 16-byte aligned device buffer");
  if (p->owns_scratch && p->scratch) GPHL_CUDA(cudaFree(p->scratch));
  p->owns_scratch = false;
  p->scratch = static_cast<float *>(scratch);
  p->max_feat = (max_feat + 7) / 8 * 8;
  p->scratch_bytes = (int64_t)sizeof(float) * 2 * p->n_pieces * p->max_feat;
  return GPHL_OK;
}
extern "C" int64_t gphl_plan_num_pieces(const gphl_plan *p) { return p ? p->n_pieces : 0; }
extern "C" int64_t gphl_plan_num_items(const gphl_plan *p) { return p ? p->n_items : 0; }
extern "C" int64_t gphl_plan_num_split_rows(const gphl_plan *p) { return p ? p->n_split_rows : 0; }
extern "C" int64_t gphl_plan_scratch_bytes(const gphl_plan *p) { return p ? p->scratch_bytes : 0; }

// ---- index validation ------------------------------------------------------------------------------------------------
// The kernels trust the graph arrays (an index out of range is an out-of-bounds read).  These entry points check them
// once per graph, where the arrays enter the library: the reference checks nothing (src/dglgraph.cpp:5-24) and a
// memory checker cannot be assumed at the caller's site.  Each runs one pass over the array, synchronises the stream
// and returns GPHL_ERR_INVALID_ARGUMENT with a message that names the first kind of violation found.
namespace gphl {
__device__ int g_check_flags[4];

__global__ void check_pointer_kernel(const int32_t *__restrict__ ptr, int64_t n_rows, int64_t total, int *flags) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_rows && ptr[i + 1] < ptr[i]) flags[0] = 1;
  if (i == 0 && (ptr[0] != 0 || (int64_t)ptr[n_rows] != total)) flags[1] = 1;
}
template <typename I>
__global__ void check_range_kernel(const I *__restrict__ a, int64_t n, int64_t limit, int *flag) {
  bool bad = false;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    bad |= a[i] < 0 || (int64_t)a[i] >= limit;
  if (bad) *flag = 1;
}
static std::mutex g_check_mutex;

template <typename I>
static void launch_range(const I *a, int64_t n, int64_t limit, int *flag, cudaStream_t stream) {
  if (n == 0 || a == nullptr) return;
  const unsigned grid = (unsigned)std::min<int64_t>((n + 255) / 256, 148 * 16);
  check_range_kernel<I><<<grid, 256, 0, stream>>>(a, n, limit, flag);
}
}  // namespace gphl

extern "C" int gphl_validate_csr(const int32_t *pointer, int64_t n_rows, int64_t n_entries, const int32_t *idx,
                                 int64_t idx_limit, const int32_t *eidx, int64_t eidx_limit, void *stream_) {
  GPHL_REQUIRE(n_rows >= 0 && n_entries >= 0 && n_rows < INT32_MAX && n_entries < INT32_MAX, "validate: sizes out of range");
  GPHL_REQUIRE(pointer != nullptr, "validate: pointer array is NULL");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  std::lock_guard<std::mutex> lock(g_check_mutex);
  int *flags = nullptr;
  GPHL_CUDA(cudaGetSymbolAddress((void **)&flags, g_check_flags));
  GPHL_CUDA(cudaMemsetAsync(flags, 0, sizeof(int) * 4, stream));
  check_pointer_kernel<<<(unsigned)(n_rows / 256 + 1), 256, 0, stream>>>(pointer, n_rows, n_entries, flags);
  launch_range<int32_t>(idx, n_entries, idx_limit, flags + 2, stream);
  launch_range<int32_t>(eidx, n_entries, eidx_limit, flags + 3, stream);
  int h[4] = {0, 0, 0, 0};
  GPHL_CUDA(cudaMemcpyAsync(h, flags, sizeof(h), cudaMemcpyDeviceToHost, stream));
  GPHL_CUDA(cudaStreamSynchronize(stream));
  GPHL_CUDA(cudaGetLastError());
  if (h[0]) return fail(GPHL_ERR_INVALID_ARGUMENT, "validate: the pointer array decreases somewhere");
  if (h[1]) return fail(GPHL_ERR_INVALID_ARGUMENT, "validate: the pointer array must start at 0 and end at %lld", (long long)n_entries);
  if (h[2]) return fail(GPHL_ERR_INVALID_ARGUMENT, "validate: a neighbour index lies outside [0, %lld)", (long long)idx_limit);
  if (h[3]) return fail(GPHL_ERR_INVALID_ARGUMENT, "validate: an edge index lies outside [0, %lld)", (long long)eidx_limit);
  return GPHL_OK;
}

extern "C" int gphl_validate_index_i64(const int64_t *a, int64_t n, int64_t limit, void *stream_) {
  GPHL_REQUIRE(n >= 0 && (a != nullptr || n == 0), "validate: bad arguments");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  std::lock_guard<std::mutex> lock(g_check_mutex);
  int *flags = nullptr;
  GPHL_CUDA(cudaGetSymbolAddress((void **)&flags, g_check_flags));
  GPHL_CUDA(cudaMemsetAsync(flags, 0, sizeof(int) * 4, stream));
  launch_range<int64_t>(a, n, limit, flags, stream);
  int h = 0;
  GPHL_CUDA(cudaMemcpyAsync(&h, flags, sizeof(int), cudaMemcpyDeviceToHost, stream));
  GPHL_CUDA(cudaStreamSynchronize(stream));
  GPHL_CUDA(cudaGetLastError());
  if (h) return fail(GPHL_ERR_INVALID_ARGUMENT, "validate: an index lies outside [0, %lld)", (long long)limit);
  return GPHL_OK;
}
