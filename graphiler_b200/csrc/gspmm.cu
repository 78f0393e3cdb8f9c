// General g-SpMM: out[v, j] = reduce over the positions i of row v of  op(u[nid[i], uoff[j]], e[eid[i], eoff[j]])
// with op in {add, sub, mul, div, copy_lhs, copy_rhs}, reduce in {sum, max, min}, broadcasting through per-column
// offset tables and, for max / min, the arguments (neighbour id and edge id) that produced each output.
//
// This is the part of the sparse library that no registered operator of the reference reaches (its registered
// operators are copy_lhs / mul with sum, which have the tuned kernels of spmm.cu): it is here for completeness of
// the primitive set, parallelised as the reference's generic kernel is - one thread per (row, output column), serial
// over the row's positions - plus coalescing across columns.  Arithmetic: the binary operator is evaluated in fp32
// exactly as written (IEEE add / sub / mul / div, so max and min match an fp32 evaluation bit for bit and ties keep
// the first position), sums accumulate those fp32 terms in double and round once.
#include "common.cuh"

namespace gphl {

struct GspmmArgs {
  const int32_t *pointer, *nid, *eid;   // eid NULL: edge id == position
  const float *u, *e;
  const int64_t *uoff, *eoff;           // per output column; NULL: identity
  float *out;
  int32_t *arg_u, *arg_e;               // optional, max / min only
  int64_t n_rows, out_len, u_len, e_len;
};

template <int OP>
__device__ __forceinline__ float binary(float a, float b) {
  if (OP == GPHL_OP_ADD) return __fadd_rn(a, b);
  if (OP == GPHL_OP_SUB) return __fsub_rn(a, b);
  if (OP == GPHL_OP_MUL) return __fmul_rn(a, b);
  if (OP == GPHL_OP_DIV) return __fdiv_rn(a, b);
  if (OP == GPHL_OP_COPY_LHS) return a;
  return b;
}

template <int OP, int RED>
__global__ void gspmm_kernel(GspmmArgs a) {
  constexpr bool use_lhs = OP != GPHL_OP_COPY_RHS, use_rhs = OP != GPHL_OP_COPY_LHS;
  const int64_t total = a.n_rows * a.out_len;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t v = t / a.out_len, j = t - v * a.out_len;
    const int64_t lj = a.uoff ? a.uoff[j] : j, rj = a.eoff ? a.eoff[j] : j;
    double sum = 0.0;
    float best = RED == GPHL_REDUCE_MAX ? -INFINITY : INFINITY;
    int32_t bu = 0, be = 0;
    for (int32_t i = a.pointer[v]; i < a.pointer[v + 1]; ++i) {
      const int32_t c = a.nid[i], eidx = a.eid ? a.eid[i] : i;
      const float x = use_lhs ? __ldg(a.u + (int64_t)c * a.u_len + lj) : 0.f;
      const float y = use_rhs ? __ldg(a.e + (int64_t)eidx * a.e_len + rj) : 0.f;
      const float val = binary<OP>(x, y);
      if (RED == GPHL_REDUCE_SUM) sum += (double)val;
      else if (RED == GPHL_REDUCE_MAX ? best < val : best > val) best = val, bu = c, be = eidx;
    }
    a.out[t] = RED == GPHL_REDUCE_SUM ? (float)sum : best;
    if (RED != GPHL_REDUCE_SUM) {
      if (a.arg_u && use_lhs) a.arg_u[t] = bu;
      if (a.arg_e && use_rhs) a.arg_e[t] = be;
    }
  }
}

template <int OP>
static int launch_red(int32_t reduce, const GspmmArgs &a, cudaStream_t stream) {
  const int64_t total = a.n_rows * a.out_len;
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148LL * 64);
  if (reduce == GPHL_REDUCE_SUM) gspmm_kernel<OP, GPHL_REDUCE_SUM><<<grid, 256, 0, stream>>>(a);
  else if (reduce == GPHL_REDUCE_MAX) gspmm_kernel<OP, GPHL_REDUCE_MAX><<<grid, 256, 0, stream>>>(a);
  else gspmm_kernel<OP, GPHL_REDUCE_MIN><<<grid, 256, 0, stream>>>(a);
  return launched("gspmm_kernel");
}

}  // namespace gphl

using namespace gphl;

extern "C" int gphl_gspmm_f32(int32_t op, int32_t reduce, const int32_t *pointer, const int32_t *node_idx,
                              const int32_t *edge_idx, int64_t n_rows, int64_t out_len, const float *u, int64_t u_len,
                              const float *e, int64_t e_len, const int64_t *u_off, const int64_t *e_off, float *out,
                              int32_t *arg_u, int32_t *arg_e, void *stream_) {
  GPHL_REQUIRE(op >= GPHL_OP_ADD && op <= GPHL_OP_COPY_RHS, "gspmm: unknown binary operator %d", op);
  GPHL_REQUIRE(reduce >= GPHL_REDUCE_SUM && reduce <= GPHL_REDUCE_MIN, "gspmm: unknown reducer %d", reduce);
  GPHL_REQUIRE(n_rows >= 0 && out_len >= 0 && u_len >= 0 && e_len >= 0 && n_rows < INT32_MAX, "gspmm: bad sizes");
  if (n_rows == 0 || out_len == 0) return GPHL_OK;
  GPHL_REQUIRE(pointer && node_idx && out, "gspmm: null pointer argument");
  GPHL_REQUIRE(op == GPHL_OP_COPY_RHS || (u != nullptr && u_len >= 1), "gspmm: the operator reads u, which is NULL or empty");
  GPHL_REQUIRE(op == GPHL_OP_COPY_LHS || (e != nullptr && e_len >= 1), "gspmm: the operator reads e, which is NULL or empty");
  GPHL_REQUIRE((u_off != nullptr) == (e_off != nullptr), "gspmm: pass both offset tables or neither");
  if (!u_off) {
    GPHL_REQUIRE(op == GPHL_OP_COPY_RHS || u_len == out_len, "gspmm: without offset tables u must have out_len columns");
    GPHL_REQUIRE(op == GPHL_OP_COPY_LHS || e_len == out_len, "gspmm: without offset tables e must have out_len columns");
  }
  GspmmArgs a{pointer, node_idx, edge_idx, u, e, u_off, e_off, out, arg_u, arg_e, n_rows, out_len, u_len, e_len};
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  switch (op) {
    case GPHL_OP_ADD: return launch_red<GPHL_OP_ADD>(reduce, a, stream);
    case GPHL_OP_SUB: return launch_red<GPHL_OP_SUB>(reduce, a, stream);
    case GPHL_OP_MUL: return launch_red<GPHL_OP_MUL>(reduce, a, stream);
    case GPHL_OP_DIV: return launch_red<GPHL_OP_DIV>(reduce, a, stream);
    case GPHL_OP_COPY_LHS: return launch_red<GPHL_OP_COPY_LHS>(reduce, a, stream);
    default: return launch_red<GPHL_OP_COPY_RHS>(reduce, a, stream);
  }
}
