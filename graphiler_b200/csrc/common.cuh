// Shared device/host helpers of the sm_100a kernel library: error reporting, launch
// accounting, compensated fp32 arithmetic and the row-split work-item format.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/gphl.h"

namespace gphl {

// ---- host: errors and launch accounting ------------------------------------------------

void set_error(const char *fmt, ...);
extern std::atomic<int64_t> g_launches;

inline int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  set_error("%s", buf);
  return code;
}

// Checks the launch that was just issued (no synchronisation) and counts it.
inline int launched(const char *what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GPHL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return GPHL_OK;
}

#define GPHL_CUDA(call)                                                                   \
  do {                                                                                    \
    cudaError_t e_ = (call);                                                              \
    if (e_ != cudaSuccess)                                                                \
      return ::gphl::fail(GPHL_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_));        \
  } while (0)

#define GPHL_REQUIRE(cond, ...)                                                           \
  do {                                                                                    \
    if (!(cond)) return ::gphl::fail(GPHL_ERR_INVALID_ARGUMENT, __VA_ARGS__);             \
  } while (0)

// Integer tuning knobs.  The product library compiles every knob to its default; the measurement build
// (-DGPHL_MEASURE, lib/libgphl_measure.so, used only by the per-kernel timer) reads them from the environment at
// every call, so that variants of one kernel can be timed side by side in one process.
#ifdef GPHL_MEASURE
int knob(const char *name, int dflt);
#else
inline int knob(const char *, int dflt) { return dflt; }
#endif

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- work items ------------------------------------------------------------------------
// One item = one contiguous piece [begin, end) of one row's segment.  slot < 0: the piece
// is the whole row and its result goes straight to the output; slot >= 0: the row was cut
// and this piece's partial result goes to scratch slot `slot`.
struct Item {
  int32_t row, begin, end, slot;
};

}  // namespace gphl

// Items of at most this many positions are "short": kernels whose per-position work is a few bytes give a short
// item to a group of threads instead of a whole warp.
#define GPHL_SHORT_ITEM 64

struct gphl_plan {
  int64_t n_rows = 0;
  int32_t chunk = 0;
  int64_t n_items = 0;
  int64_t n_split_rows = 0;
  int64_t n_pieces = 0;
  int64_t n_long_items = 0;         // items longer than GPHL_SHORT_ITEM positions (they come first in `items`)
  int64_t max_feat = 0;
  gphl::Item *items = nullptr;      // device, n_items
  int32_t *split_rows = nullptr;    // device, n_split_rows: row id of each cut row
  int32_t *split_ptr = nullptr;     // device, n_split_rows + 1: first slot of each cut row
  float *scratch = nullptr;         // device, 2 * n_pieces * max_feat floats (hi plane, lo plane per slot)
  int64_t scratch_bytes = 0;
  bool owns_scratch = true;
};

namespace gphl {

#ifdef __CUDACC__

constexpr unsigned FULL = 0xffffffffu;

// s + err == a + b exactly (Knuth two-sum; no ordering requirement on |a|, |b|).
__device__ __forceinline__ void two_sum(float a, float b, float &s, float &err) {
  s = __fadd_rn(a, b);
  float bb = __fsub_rn(s, a);
  err = __fadd_rn(__fsub_rn(a, __fsub_rn(s, bb)), __fsub_rn(b, bb));
}

// Compensated accumulator: value = hi + lo, lo collects the rounding errors of hi.
struct Acc {
  float hi, lo;
  __device__ __forceinline__ void add(float v) {
    float s, e;
    two_sum(hi, v, s, e);
    hi = s;
    lo = __fadd_rn(lo, e);
  }
  // adds the exact product a*b
  __device__ __forceinline__ void fma_exact(float a, float b) {
    float p = __fmul_rn(a, b);
    float pe = __fmaf_rn(a, b, -p);
    float s, e;
    two_sum(hi, p, s, e);
    hi = s;
    lo = __fadd_rn(lo, __fadd_rn(e, pe));
  }
  __device__ __forceinline__ void merge(float ohi, float olo) {
    float s, e;
    two_sum(hi, ohi, s, e);
    hi = s;
    lo = __fadd_rn(lo, __fadd_rn(e, olo));
  }
  __device__ __forceinline__ float value() const { return __fadd_rn(hi, lo); }
};

// Packed pairs of fp32 (sm_100 add/sub/mul/fma.f32x2): one instruction issues two IEEE operations, which
// halves the issue slots of the compensated accumulation.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &a, float &b) {
  asm("mov.b64 {%0,%1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fsub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fneg2(uint64_t a) { return a ^ 0x8000000080000000ull; }

// Two compensated accumulators side by side (see Acc): the same operations, element-wise on a pair.
struct Acc2 {
  uint64_t hi, lo;
  __device__ __forceinline__ void add(uint64_t v) {
    const uint64_t s = fadd2(hi, v), bb = fsub2(s, hi);
    const uint64_t e = fadd2(fsub2(hi, fsub2(s, bb)), fsub2(v, bb));
    hi = s;
    lo = fadd2(lo, e);
  }
  __device__ __forceinline__ void fma_exact(uint64_t a, uint64_t b) {
    const uint64_t p = fmul2(a, b);
    const uint64_t pe = ffma2(a, b, fneg2(p));
    const uint64_t s = fadd2(hi, p), bb = fsub2(s, hi);
    const uint64_t e = fadd2(fsub2(hi, fsub2(s, bb)), fsub2(p, bb));
    hi = s;
    lo = fadd2(lo, fadd2(e, pe));
  }
  __device__ __forceinline__ void merge(uint64_t ohi, uint64_t olo) {
    const uint64_t s = fadd2(hi, ohi), bb = fsub2(s, hi);
    const uint64_t e = fadd2(fsub2(hi, fsub2(s, bb)), fsub2(ohi, bb));
    hi = s;
    lo = fadd2(lo, fadd2(e, olo));
  }
  __device__ __forceinline__ uint64_t value() const { return fadd2(hi, lo); }
};

__device__ __forceinline__ bool aligned16_dev(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ float leaky(float v, float slope) { return v >= 0.f ? v : v * slope; }

// Online-softmax pair (running maximum, sum of exp(x - maximum)).
// exp through the hardware base-2 exponential (ex2.approx after one multiplication).  Arguments here are
// x - max <= 0: the relative error is about 2^-22 + |x| * 2^-24, under 2e-6 wherever the result is not
// negligible, against an element tolerance of 1e-5 relative.  A quarter of the instructions of expf, which
// bounded the softmax kernels.
__device__ __forceinline__ float exp_neg(float x) { return __expf(x); }

struct MaxSum {
  float m, s;
  __device__ __forceinline__ void init() {
    m = -INFINITY;
    s = 0.f;
  }
  // reference point of the exponentials: the maximum, or 0 while everything seen is -inf (keeps inf - inf out)
  static __device__ __forceinline__ float ref_of(float mx) { return mx == -INFINITY ? 0.f : mx; }
  __device__ __forceinline__ void push(float x) {
    const float mn = fmaxf(m, x), r = ref_of(mn);
    s = s * exp_neg(m - r) + exp_neg(x - r);
    m = mn;
  }
  __device__ __forceinline__ void push4(float a, float b, float c, float d) {
    const float mn = fmaxf(fmaxf(m, fmaxf(a, b)), fmaxf(c, d)), r = ref_of(mn);
    s = s * exp_neg(m - r) + ((exp_neg(a - r) + exp_neg(b - r)) + (exp_neg(c - r) + exp_neg(d - r)));
    m = mn;
  }
  __device__ __forceinline__ void merge(float om, float os) {
    const float mn = fmaxf(m, om), r = ref_of(mn);
    s = s * exp_neg(m - r) + os * exp_neg(om - r);
    m = mn;
  }
};

// 16-byte vector views of a feature row.
template <typename T>
struct VecOf;
template <>
struct VecOf<float> {
  static constexpr int N = 4;
  __device__ __forceinline__ static void load(const float *p, float (&v)[4]) {
    float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
  }
  __device__ __forceinline__ static void store(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct VecOf<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void load(const __nv_bfloat16 *p, float (&v)[8]) {
    uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static void store(__nv_bfloat16 *p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t *>(&b);
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f32(float &d, float v) { d = v; }
__device__ __forceinline__ void from_f32(__nv_bfloat16 &d, float v) { d = __float2bfloat16_rn(v); }

__device__ __forceinline__ Item fetch_item(const Item *items, const int32_t *pointer, int64_t i) {
  if (items) {
    int4 t = __ldg(reinterpret_cast<const int4 *>(items) + i);
    return Item{t.x, t.y, t.z, t.w};
  }
  return Item{(int32_t)i, __ldg(pointer + i), __ldg(pointer + i + 1), -1};
}

#endif  // __CUDACC__

}  // namespace gphl
