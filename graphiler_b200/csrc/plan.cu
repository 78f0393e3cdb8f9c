// Host side of the library: error state, launch counter and the row-split plan.
#include <cstdlib>
#include <cstring>
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
  GPHL_REQUIRE(max_feat >= 1, "plan_create: max_feat must be >= 1");
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

extern "C" int64_t gphl_plan_num_items(const gphl_plan *p) { return p ? p->n_items : 0; }
extern "C" int64_t gphl_plan_num_split_rows(const gphl_plan *p) { return p ? p->n_split_rows : 0; }
extern "C" int64_t gphl_plan_scratch_bytes(const gphl_plan *p) { return p ? p->scratch_bytes : 0; }
