// Edge-parallel SDDMM kernels for sm_100a: u_add_v and u_dot_v over the COO arrays.
//
// One thread produces one 16-byte output vector (u_add_v) or one (edge, head) dot product
// (u_dot_v); consecutive threads own consecutive outputs of the same edge, so the gathered
// reads of one endpoint row and the output writes are contiguous.  Dot products are
// accumulated with an exact-product compensated sum.
#include "common.cuh"

namespace gphl {

template <typename I>
__global__ void u_add_v_vec_kernel(const I *__restrict__ src, const I *__restrict__ dst, int64_t n_edges, int32_t FV,
                                   const float4 *__restrict__ l, const float4 *__restrict__ r, float4 *__restrict__ z) {
  const int64_t total = n_edges * FV;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = t / FV;
    const int c = (int)(t - e * FV);
    const float4 a = __ldg(l + (int64_t)__ldg(src + e) * FV + c);
    const float4 b = __ldg(r + (int64_t)__ldg(dst + e) * FV + c);
    z[t] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
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
  const int64_t total = n_edges * H;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = t / H;
    const int h = (int)(t - e * H);
    const float *a = l + ((int64_t)__ldg(src + e) * H + h) * D;
    const float *b = r + ((int64_t)__ldg(dst + e) * H + h) * D;
    Acc acc{0.f, 0.f};
    if (VEC4) {
      for (int d = 0; d < D; d += 4) {
        const float4 p = __ldg(reinterpret_cast<const float4 *>(a + d));
        const float4 q = __ldg(reinterpret_cast<const float4 *>(b + d));
        acc.fma_exact(p.x, q.x);
        acc.fma_exact(p.y, q.y);
        acc.fma_exact(p.z, q.z);
        acc.fma_exact(p.w, q.w);
      }
    } else {
      for (int d = 0; d < D; ++d) acc.fma_exact(__ldg(a + d), __ldg(b + d));
    }
    z[t] = acc.value();
  }
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
    const int64_t total = n_edges * (feat / 4);
    u_add_v_vec_kernel<I><<<grid_for(total, 256), 256, 0, stream>>>(
        src, dst, n_edges, (int32_t)(feat / 4), reinterpret_cast<const float4 *>(l), reinterpret_cast<const float4 *>(r),
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
  if (dim % 4 == 0 && aligned16(l) && aligned16(r)) {
    u_dot_v_kernel<I, true><<<grid_for(total, 256), 256, 0, stream>>>(src, dst, n_edges, (int32_t)heads, (int32_t)dim, l, r, z);
  } else {
    u_dot_v_kernel<I, false><<<grid_for(total, 256), 256, 0, stream>>>(src, dst, n_edges, (int32_t)heads, (int32_t)dim, l, r, z);
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
