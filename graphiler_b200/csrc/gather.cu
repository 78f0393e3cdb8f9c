// Broadcast operators for sm_100a: row gathers y[i,:] = x[idx[i],:] (optionally through a
// second index, y[i,:] = x[idx[idx2[i]],:]) for rows of any byte length, moved in 16-byte (or, for
// odd row lengths / alignments, 4- or 1-byte) units; consecutive threads move consecutive units of
// the same row.
#include <algorithm>

#include "common.cuh"

namespace gphl {

// Thread layout shared by the row movers: `lanes` = min(units per row, 256) threads walk one row together, a block
// holds 256 / lanes rows, and a thread's column and row slot are fixed for its whole life, so the only divisions are
// two 32-bit ones per thread (a 64-bit division per 16 bytes moved cost more than the move).
template <typename I, typename U>
__global__ void __launch_bounds__(256) gather_rows_kernel(const I *__restrict__ idx, const I *__restrict__ idx2, int64_t n_out,
                                                          int32_t units, int32_t lanes, const U *__restrict__ x,
                                                          U *__restrict__ y) {
  const int rows_per_block = 256 / lanes;
  const int slot = (int)threadIdx.x / lanes, c0 = (int)threadIdx.x - slot * lanes;
  if (slot >= rows_per_block) return;
  for (int64_t i = (int64_t)blockIdx.x * rows_per_block + slot; i < n_out; i += (int64_t)gridDim.x * rows_per_block) {
    int64_t row = idx2 ? (int64_t)__ldg(idx2 + i) : i;
    row = (int64_t)__ldg(idx + row);
    const U *src = x + row * units;
    U *dst = y + i * units;
    for (int c = c0; c < units; c += lanes) dst[c] = __ldg(src + c);
  }
}

template <typename I>
static int gather_rows(const I *idx, const I *idx2, int64_t n_out, int64_t row_bytes, const void *x, void *y,
                       void *stream_) {
  GPHL_REQUIRE(n_out >= 0 && row_bytes >= 0, "bad sizes");
  if (n_out == 0 || row_bytes == 0) return GPHL_OK;
  GPHL_REQUIRE(idx && x && y, "null pointer argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  auto launch = [&](auto unit_tag, int64_t units) {
    using U = decltype(unit_tag);
    const int lanes = (int)std::min<int64_t>(units, 256);
    const int64_t rows_per_block = 256 / lanes;
    const unsigned grid = (unsigned)std::min<int64_t>((n_out + rows_per_block - 1) / rows_per_block, 148LL * 64);
    gather_rows_kernel<I, U><<<grid, 256, 0, stream>>>(idx, idx2, n_out, (int32_t)units, lanes, static_cast<const U *>(x),
                                                     static_cast<U *>(y));
  };
  GPHL_REQUIRE(row_bytes < (int64_t)1 << 31, "rows of 2 GiB or more are not supported");
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | (uintptr_t)row_bytes;
  if ((bits & 15u) == 0) launch(uint4{}, row_bytes / 16);
  else if ((bits & 3u) == 0) launch(uint32_t{}, row_bytes / 4);
  else launch(uint8_t{}, row_bytes);
  return launched("gather_rows_kernel");
}

// ---- the sending side of the sparse exchange: rows to several receivers in one launch -----------------------------
// Receiver p gets rows x[idx[src_start[p] + k]] for k in [0, count[p]) at rows dst_start[p] + k of its buffer
// dst[p], which may live in another GPU's memory mapped into this process (plain stores over NVLink; loads are local).
// Work is dealt so that threads that run together write to different receivers: list position j of the launch is
// visited in the order (j mod P) * ceil(total / P) + j / P over the concatenated lists, which spreads every moment's
// stores over all links instead of filling one receiver after the other.
struct ScatterPeers {
  void *dst[GPHL_MAX_PEERS];
  int64_t src_start[GPHL_MAX_PEERS], dst_start[GPHL_MAX_PEERS], prefix[GPHL_MAX_PEERS + 1];
  int32_t n_peers;
};

__global__ void __launch_bounds__(256) scatter_rows_peers_kernel(const int64_t *__restrict__ idx, ScatterPeers p, int32_t units,
                                                                 int32_t lanes, const uint4 *__restrict__ x) {
  const int rows_per_block = 256 / lanes;
  const int slot = (int)threadIdx.x / lanes, c0 = (int)threadIdx.x - slot * lanes;
  if (slot >= rows_per_block) return;
  const uint32_t np = (uint32_t)p.n_peers;
  const int64_t total_rows = p.prefix[p.n_peers];
  const int64_t seg = (total_rows + np - 1) / np;
  const int64_t visits = seg * np;                          // positions past the end of the lists are skipped
  for (int64_t i = (int64_t)blockIdx.x * rows_per_block + slot; i < visits; i += (int64_t)gridDim.x * rows_per_block) {
    const uint32_t hi = (uint32_t)(i / np);                 // i < 2^31 * 16: one 64-bit division per row, not per 16 bytes
    const int64_t j = (int64_t)(uint32_t)(i - (int64_t)hi * np) * seg + hi;
    if (j >= total_rows) continue;
    int q = 0;
#pragma unroll
    for (int k = 1; k < GPHL_MAX_PEERS; ++k) q += (k < p.n_peers && j >= p.prefix[k]) ? 1 : 0;
    const int64_t k = j - p.prefix[q];
    const int64_t row = __ldg(idx + p.src_start[q] + k);
    const uint4 *src = x + row * units;
    uint4 *dst = static_cast<uint4 *>(p.dst[q]) + (p.dst_start[q] + k) * units;
    for (int c = c0; c < units; c += lanes) dst[c] = __ldg(src + c);
  }
}

}  // namespace gphl

extern "C" int gphl_gather_rows_i64(const int64_t *idx, const int64_t *idx2, int64_t n_out, int64_t row_bytes,
                                    const void *x, void *y, void *stream) {
  return gphl::gather_rows<int64_t>(idx, idx2, n_out, row_bytes, x, y, stream);
}
extern "C" int gphl_gather_rows_i32(const int32_t *idx, const int32_t *idx2, int64_t n_out, int64_t row_bytes,
                                    const void *x, void *y, void *stream) {
  return gphl::gather_rows<int32_t>(idx, idx2, n_out, row_bytes, x, y, stream);
}

extern "C" int gphl_scatter_rows_peers_i64(const int64_t *idx, int32_t n_peers, const int64_t *src_start,
                                           const int64_t *count, void *const *dst, const int64_t *dst_start,
                                           int64_t row_bytes, const void *x, void *stream_) {
  using namespace gphl;
  GPHL_REQUIRE(n_peers >= 1 && n_peers <= GPHL_MAX_PEERS, "scatter_rows_peers: between 1 and %d receivers", GPHL_MAX_PEERS);
  GPHL_REQUIRE(src_start && count && dst && dst_start && row_bytes >= 0, "scatter_rows_peers: null pointer argument");
  GPHL_REQUIRE(row_bytes % 16 == 0 && aligned16(x), "scatter_rows_peers: rows must be multiples of 16 bytes, 16-byte aligned");
  ScatterPeers p{};
  p.n_peers = n_peers;
  p.prefix[0] = 0;
  for (int i = 0; i < n_peers; ++i) {
    GPHL_REQUIRE(count[i] >= 0 && src_start[i] >= 0 && dst_start[i] >= 0, "scatter_rows_peers: negative count or offset");
    GPHL_REQUIRE(count[i] == 0 || (dst[i] != nullptr && aligned16(dst[i])), "scatter_rows_peers: receiver buffer missing or unaligned");
    p.dst[i] = dst[i], p.src_start[i] = src_start[i], p.dst_start[i] = dst_start[i];
    p.prefix[i + 1] = p.prefix[i] + count[i];
  }
  const int64_t total_rows = p.prefix[n_peers], units = row_bytes / 16;
  if (total_rows == 0 || units == 0) return GPHL_OK;
  GPHL_REQUIRE(idx && x, "scatter_rows_peers: null pointer argument");
  GPHL_REQUIRE(units < ((int64_t)1 << 27) && total_rows < ((int64_t)1 << 31), "scatter_rows_peers: sizes out of range");
  const int64_t seg = (total_rows + n_peers - 1) / n_peers;
  const int lanes = (int)std::min<int64_t>(units, 256);
  const int64_t rows_per_block = 256 / lanes;
  const int64_t blocks = std::min<int64_t>((seg * n_peers + rows_per_block - 1) / rows_per_block, 148LL * 64);
  scatter_rows_peers_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      idx, p, (int32_t)units, lanes, static_cast<const uint4 *>(x));
  return launched("scatter_rows_peers_kernel");
}
