// Broadcast operators for sm_100a: row gathers y[i,:] = x[idx[i],:] (optionally through a
// second index, y[i,:] = x[idx[idx2[i]],:]) for rows of any byte length.  One thread moves one
// 16-byte (or, for odd row lengths / alignments, 4- or 1-byte) unit; consecutive threads
// move consecutive units of the same row.
#include "common.cuh"

namespace gphl {

template <typename I, typename U>
__global__ void gather_rows_kernel(const I *__restrict__ idx, const I *__restrict__ idx2, int64_t n_out,
                                   int64_t units, const U *__restrict__ x, U *__restrict__ y) {
  const int64_t total = n_out * units;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t / units;
    const int64_t c = t - i * units;
    int64_t row = idx2 ? (int64_t)__ldg(idx2 + i) : i;
    row = (int64_t)__ldg(idx + row);
    y[t] = __ldg(x + row * units + c);
  }
}

template <typename I>
static int gather_rows(const I *idx, const I *idx2, int64_t n_out, int64_t row_bytes, const void *x, void *y,
                       void *stream_) {
  GPHL_REQUIRE(n_out >= 0 && row_bytes >= 0, "bad sizes");
  if (n_out == 0 || row_bytes == 0) return GPHL_OK;
  GPHL_REQUIRE(idx && x && y, "null pointer argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  auto grid = [](int64_t total) {
    int64_t g = (total + 255) / 256;
    const int64_t cap = 148LL * 64;
    return (unsigned)(g < cap ? g : cap);
  };
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | (uintptr_t)row_bytes;
  if ((bits & 15u) == 0) {
    const int64_t units = row_bytes / 16;
    gather_rows_kernel<I, uint4><<<grid(n_out * units), 256, 0, stream>>>(idx, idx2, n_out, units,
                                                                       static_cast<const uint4 *>(x), static_cast<uint4 *>(y));
  } else if ((bits & 3u) == 0) {
    const int64_t units = row_bytes / 4;
    gather_rows_kernel<I, uint32_t><<<grid(n_out * units), 256, 0, stream>>>(
        idx, idx2, n_out, units, static_cast<const uint32_t *>(x), static_cast<uint32_t *>(y));
  } else {
    gather_rows_kernel<I, uint8_t><<<grid(n_out * row_bytes), 256, 0, stream>>>(
        idx, idx2, n_out, row_bytes, static_cast<const uint8_t *>(x), static_cast<uint8_t *>(y));
  }
  return launched("gather_rows_kernel");
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
