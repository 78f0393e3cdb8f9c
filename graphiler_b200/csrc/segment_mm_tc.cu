// Typed linear on the 5th-generation tensor cores (tcgen05 + TMEM) for sm_100a:
//   y[p_t:p_{t+1}, :] = (x[p_t:p_{t+1}, :] or x[gather[...], :]) @ w[t]   (optionally * row_scale, relu)
//
// fp32 in, fp32 out, fp32-level accuracy: every operand is split into three bf16 terms
// (x = x1 + x2 + x3 to 2^-24) and six bf16 products x1w1 + x1w2 + x2w1 + x2w2 + x1w3 + x3w1 are
// accumulated in fp32 in tensor memory; the dropped terms are below 2^-24 relative.
//
// One block = one 128-row tile of one type (row tiles never straddle a type boundary; the block
// finds its tile by walking the device-resident type pointer) x one <=128-column slice of the
// output.  The reduction dimension is processed in slabs of 64: all threads load the slab of x
// (16-byte loads, optionally through a row index), split it and store the three bf16 copies into
// shared memory in the 128-byte-swizzled K-major layout the tensor core reads; the slab of the
// pre-split, pre-transposed weights arrives next to it by TMA (cp.async.bulk.tensor.2d with the 128-byte
// swizzle, from a tensor map over the weight workspace in this GPU's own memory; no multicast), one or two
// slabs ahead of the tensor core; one elected thread issues the 24 tcgen05.mma instructions of the slab
// and commits them to an mbarrier.  The next slab's loads of x
// are issued before that barrier is waited on, and two or three blocks share an SM, so loads,
// splitting and tensor work overlap.  The accumulator (128 lanes x <=128 columns) is read back
// with tcgen05.ld and stored with 16-byte stores.  Every wait is bounded: if a barrier does not
// complete, the block records it in a device flag, waits once more for what it issued, frees its
// tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

namespace gphl {

constexpr int TC_THREADS = 256;
constexpr int TC_M = 128;       // rows per tile = TMEM lanes
constexpr int TC_NMAX = 128;    // output columns per block = TMEM columns
constexpr int TC_SLAB = 64;     // bf16 elements per 128-byte swizzle row
constexpr int A_SPLIT_BYTES = TC_M * 128;          // one bf16 copy of the x slab
constexpr uint32_t WAIT_LIMIT = 1u << 22;          // try_wait polls before giving up
constexpr int FAN_CACHE = 256;                     // fan-out entries a warp keeps in shared memory at a time
static_assert(8 * 4096 + 8 * FAN_CACHE * 8 <= 3 * A_SPLIT_BYTES, "staging buffers and entry caches share the x slab");

__device__ int g_tc_wait_timeouts = 0;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// Bounded wait on phase `parity`; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One box of the tensor map (64 K-values x box rows, 128-byte swizzle) into shared memory; completion is counted in
// bytes on `bar`.  x is a multiple of 64 bf16 elements = 128 bytes, so the 16-byte alignment rule of the inner
// coordinate always holds.  The map covers the weight workspace of the launching GPU only.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
               : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);        // start address
  d |= (uint64_t)1 << 16;                         // leading-dimension offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride between 8-row groups
  d |= (uint64_t)1 << 46;                         // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
  return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

// 32 consecutive fp32 columns of this warp's 32 TMEM lanes -> one row of 32 values per thread.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
      "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// x = b1 + b2 + b3 (each bf16, round to nearest), packed two elements per word.
__device__ __forceinline__ void split3(float x0, float x1, uint32_t &p1, uint32_t &p2, uint32_t &p3) {
  __nv_bfloat162 h1 = __floats2bfloat162_rn(x0, x1);
  float r0 = x0 - __low2float(h1), r1 = x1 - __high2float(h1);
  __nv_bfloat162 h2 = __floats2bfloat162_rn(r0, r1);
  r0 -= __low2float(h2), r1 -= __high2float(h2);
  __nv_bfloat162 h3 = __floats2bfloat162_rn(r0, r1);
  p1 = *reinterpret_cast<uint32_t *>(&h1), p2 = *reinterpret_cast<uint32_t *>(&h2), p3 = *reinterpret_cast<uint32_t *>(&h3);
}

// Weights: w (T, K, N) fp32 -> ws (3, T, Npad, Kpad) bf16, transposed (K contiguous), zero padded.
__global__ void split_weights_kernel(const float *__restrict__ w, int32_t T, int32_t K, int32_t N, int32_t Kpad,
                                     int32_t Npad, __nv_bfloat16 *__restrict__ ws) {
  const int64_t total = (int64_t)T * Npad * Kpad;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int k = (int)(i % Kpad);
    const int n = (int)((i / Kpad) % Npad);
    const int t = (int)(i / ((int64_t)Kpad * Npad));
    float v = (k < K && n < N) ? w[((int64_t)t * K + k) * N + n] : 0.f;
    __nv_bfloat16 b1 = __float2bfloat16_rn(v);
    v -= __bfloat162float(b1);
    __nv_bfloat16 b2 = __float2bfloat16_rn(v);
    v -= __bfloat162float(b2);
    ws[i] = b1, ws[total + i] = b2, ws[2 * total + i] = __float2bfloat16_rn(v);
  }
}

struct TcArgs {
  const float *x;
  const __nv_bfloat16 *ws;   // (3, T, Npad, Kpad)
  const int32_t *ptr;
  const int64_t *gather;     // optional row index into x
  const float *row_scale;    // optional per-output-row factor
  float *y;
  int64_t m;
  int32_t T, K, N, Kpad, Npad, relu;
  // Optional fan-out of the finished rows (the sending side of a sparse exchange fused into the epilogue): output row
  // i is also stored at row (entry & 0xffffffffff) of receiver (entry >> 40)'s buffer, for every entry in
  // [fan_ptr[i], fan_ptr[i + 1]).  Receivers' buffers may be other GPUs' memory mapped into this process (plain stores).
  const int32_t *fan_ptr;
  const int64_t *fan_entry;
  float *fan_base[GPHL_MAX_PEERS];
  int32_t stages;            // weight slabs in shared memory (1 or 2)
  int32_t box_rows;          // rows of one TMA box = min(128, Npad)
};

// Which (type, 128-row tile) is row tile `b`?  Run by one warp: 32 types per step - tile counts, warp prefix sum, one
// hit - and written to *seg, *row0, *rows (shared memory; *rows is left alone when b lies beyond the last tile).
__device__ __forceinline__ void tile_lookup(const TcArgs &a, int64_t b, int lane, int *seg, int *row0, int *rows) {
  int64_t base = 0;
  for (int t0 = 0; t0 < a.T; t0 += 32) {
    const int t = t0 + lane;
    const int lo = t < a.T ? __ldg(a.ptr + t) : 0, hi = t < a.T ? __ldg(a.ptr + t + 1) : lo;
    const int nt = (hi - lo + TC_M - 1) / TC_M;
    int incl = nt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(FULL, incl, d);
      if (lane >= d) incl += v;
    }
    const bool hit = t < a.T && b >= base + incl - nt && b < base + incl;
    if (hit) {
      const int first = lo + (int)(b - (base + incl - nt)) * TC_M;
      *seg = t, *row0 = first, *rows = min(TC_M, hi - first);
    }
    if (__any_sync(FULL, hit)) break;
    base += __shfl_sync(FULL, incl, 31);
  }
}

// Accumulators -> global memory for one tile: the two TMEM accumulators are added, scaled / clamped, and leave as
// whole 128-byte row segments through a swizzled staging buffer in the x slab's shared memory.
__device__ __forceinline__ void tile_epilogue(const TcArgs &a, uint32_t tmem, uint32_t acc_cols, int rows, int row0, int n0,
                                              int ncols, uint8_t *sA, int warp, int lane) {
  // epilogue: warp w reads lanes 32*(w%4).., warps 0-3 the first half of the columns, 4-7 the second
  const int r = (warp & 3) * 32 + lane;
  const int chalf = ((ncols + 63) / 64) * 32;            // columns per warp group, multiple of 32
  const int cbeg = (warp >> 2) * chalf;
  const float scale = (a.row_scale && r < rows) ? __ldg(a.row_scale + row0 + r) : 1.f;
  // fan-out: the entries of the warp's 32 rows are one contiguous range [e0, e1) of fan_entry; they are brought into
  // shared memory with coalesced loads, FAN_CACHE at a time (behind the staging buffers in the x slab's memory),
  // each tagged in bits 56.. with the row of the warp that owns it
  int p0 = 0, p1 = 0, e0 = 0, e1 = 0, cached = -1;
  uint64_t *ent = reinterpret_cast<uint64_t *>(sA + 8 * 4096 + warp * (FAN_CACHE * 8));
  if (a.fan_ptr) {
    p0 = __ldg(a.fan_ptr + row0 + min(r, rows));
    p1 = __ldg(a.fan_ptr + row0 + min(r + 1, rows));
    e0 = __shfl_sync(FULL, p0, 0), e1 = __shfl_sync(FULL, p1, 31);
  }
  for (int c0 = cbeg; c0 < min(cbeg + chalf, ncols); c0 += 32) {
    uint32_t v[32], u[32];
    const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)c0;
    tmem_ld32(taddr, v);
    tmem_ld32(taddr + acc_cols, u);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int q = 0; q < 32; ++q) v[q] = __float_as_uint(__fadd_rn(__uint_as_float(v[q]), __uint_as_float(u[q])));
    // A thread holds 32 columns of its own row; storing them directly would make every store instruction touch
    // 32 different rows.  The 32 x 32 block goes through a swizzled staging buffer (the x slab's shared memory
    // is free by now) and leaves as whole 128-byte row segments: 8 lanes per row, 4 rows per instruction.
    uint8_t *stg = sA + warp * 4096;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[e] = __uint_as_float(v[q * 4 + e]);
        if (a.row_scale) o[e] = __fmul_rn(o[e], scale);
        if (a.relu) o[e] = fmaxf(o[e], 0.f);
      }
      *reinterpret_cast<float4 *>(stg + lane * 128 + ((q ^ (lane & 7)) << 4)) = make_float4(o[0], o[1], o[2], o[3]);
    }
    __syncwarp();
    const int ch = lane & 7;
    const bool vec = ((a.N & 3) == 0);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int rr = (lane >> 3) + 4 * j;
      const float4 o = *reinterpret_cast<const float4 *>(stg + rr * 128 + ((ch ^ (rr & 7)) << 4));
      const int grow = (warp & 3) * 32 + rr, col = n0 + c0 + ch * 4;
      if (grow < rows) {
        const float oo[4] = {o.x, o.y, o.z, o.w};
        if (a.y) {
          float *dst = a.y + (int64_t)(row0 + grow) * a.N + col;
          if (vec && col + 3 < a.N) {
            __stcs(reinterpret_cast<float4 *>(dst), o);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (col + e < a.N) dst[e] = oo[e];
          }
        }
      }
    }
    if (a.fan_ptr) {
      // every (row, receiver) entry of the warp's rows is one unit of work for a group of 8 lanes: the groups stay
      // busy whatever the rows' fan-outs are, and no global load sits between two stores
      const int ecol = n0 + c0 + ch * 4;
      for (int cb = e0; cb < e1; cb += FAN_CACHE) {
        const int n = min(e1 - cb, FAN_CACHE);
        if (cb != cached) {
          __syncwarp();                                          // the previous piece has been read by every lane
          for (int i = lane; i < n; i += 32) ent[i] = (uint64_t)__ldg(a.fan_entry + cb + i);
          __syncwarp();
          for (int f = max(p0, cb); f < min(p1, cb + n); ++f) ent[f - cb] |= (uint64_t)lane << 56;   // owner row
          __syncwarp();
          cached = cb;
        }
        for (int i = lane >> 3; i < n; i += 4) {
          const uint64_t en = ent[i];
          const int rl = (int)(en >> 56);
          const float4 o = *reinterpret_cast<const float4 *>(stg + rl * 128 + ((ch ^ (rl & 7)) << 4));
          float *dst = a.fan_base[(en >> 40) & 0xffff] + (int64_t)(en & 0xffffffffffULL) * a.N + ecol;
          if (vec && ecol + 3 < a.N) {
            *reinterpret_cast<float4 *>(dst) = o;
          } else {
            const float oo[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (ecol + e < a.N) dst[e] = oo[e];
          }
        }
      }
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(TC_THREADS) segment_mm_tc_kernel(TcArgs a, const __grid_constant__ CUtensorMap wmap) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t s_bar;
  __shared__ uint64_t s_full[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_seg, s_row0, s_rows, s_failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // tile lookup (rows) and column slice
  const int n_slices = (a.Npad + TC_NMAX - 1) / TC_NMAX;
  if (warp == 0) {
    if (lane == 0) s_rows = 0, s_failed = 0;
    __syncwarp();
    tile_lookup(a, blockIdx.x / n_slices, lane, &s_seg, &s_row0, &s_rows);   // column slices of one row tile are neighbours
  }
  __syncthreads();
  const int rows = s_rows;
  if (rows == 0) return;                                   // uniform: no barrier or TMEM touched yet
  const int seg = s_seg, row0 = s_row0;
  const int n0 = (int)(blockIdx.x % n_slices) * TC_NMAX;
  const int ncols = min(TC_NMAX, a.Npad - n0);             // multiple of 16
  // two accumulators side by side: [0, acc_cols) the leading products x1w1, [acc_cols, 2 acc_cols) the five
  // correction products.  The tensor core truncates when it adds into an fp32 accumulator, an error that scales
  // with the accumulator's magnitude; keeping the small terms apart makes 5/6 of those additions harmless.
  const uint32_t acc_cols = ncols <= 32 ? 32 : (ncols <= 64 ? 64 : 128);
  const uint32_t tmem_cols = 2 * acc_cols;

  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t *sA = smem;                                      // 3 x (128 rows x 128 B)
  uint8_t *sB = smem + 3 * A_SPLIT_BYTES;                  // stages x 3 x (box_rows rows x 128 B)
  const int b_split_bytes = a.box_rows * 128;              // a box is always whole; rows beyond ncols are not multiplied
  const int b_stage_bytes = 3 * b_split_bytes;
  const uint32_t bar = smem_u32(&s_bar);
  const uint32_t full0 = smem_u32(&s_full[0]);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    if (lane == 0) {
      mbar_init(bar, 1);
      mbar_init(full0, 1);
      mbar_init(full0 + 8, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;

  // each thread owns 4 (row, 16-byte output chunk) pairs of the x slab: chunk c = 8 k-values
  const int c = tid & 7;
  const float *xrow[4];
  bool rok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = (tid >> 3) + 32 * i;
    rok[i] = r < rows;
    const int64_t src = rok[i] ? (a.gather ? __ldg(a.gather + row0 + r) : (int64_t)(row0 + r)) : 0;
    xrow[i] = a.x + src * a.K;
  }
  float4 pre[4][2];
  auto load_slab = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + c * 8;
      pre[i][0] = (rok[i] && k < a.K) ? __ldg(reinterpret_cast<const float4 *>(xrow[i] + k)) : make_float4(0, 0, 0, 0);
      pre[i][1] = (rok[i] && k + 4 < a.K) ? __ldg(reinterpret_cast<const float4 *>(xrow[i] + k + 4)) : make_float4(0, 0, 0, 0);
    }
  };

  const int nslabs = a.Kpad / TC_SLAB;
  const uint32_t idesc = umma_idesc(ncols);
  // weight slabs: slab j goes to stage j % S; with S = 2 the copy of slab s + 1 is issued as soon as the tensor core
  // has finished slab s - 1, and runs while slab s is split, stored and multiplied
  const int S = a.stages, L = S - 1;
  const int wrow0 = seg * a.Npad + n0, wplane = a.T * a.Npad;      // row of this tile in split 0; rows per split
  int issued = 0, consumed = 0;                                     // thread 0 only
  auto issue_weights = [&](int j) {
    const uint32_t fb = full0 + 8 * (j % S);
    const uint32_t dst = smem_u32(sB) + (uint32_t)((j % S) * b_stage_bytes);
    mbar_expect_tx(fb, (uint32_t)b_stage_bytes);
#pragma unroll
    for (int sp = 0; sp < 3; ++sp) tma_load_2d(dst + sp * b_split_bytes, &wmap, j * TC_SLAB, sp * wplane + wrow0, fb);
    ++issued;
  };
  if (tid == 0)
    for (int j = 0; j < L && j < nslabs; ++j) issue_weights(j);
  load_slab(0);
  for (int s = 0; s < nslabs; ++s) {
    // the tensor core must be done reading the previous slab before it is overwritten; a wait that runs
    // out is recorded and acted on by all threads together after the next block-wide barrier
    if (s > 0 && !mbar_wait(bar, (uint32_t)((s - 1) & 1))) s_failed = 1;
    if (tid == 0 && s + L < nslabs && !s_failed) issue_weights(s + L);
    // x slab: split and store the three bf16 copies (swizzled: 16-byte chunk c of row r goes to chunk c ^ (r % 8))
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = (tid >> 3) + 32 * i;
      uint4 o1, o2, o3;
      split3(pre[i][0].x, pre[i][0].y, o1.x, o2.x, o3.x);
      split3(pre[i][0].z, pre[i][0].w, o1.y, o2.y, o3.y);
      split3(pre[i][1].x, pre[i][1].y, o1.z, o2.z, o3.z);
      split3(pre[i][1].z, pre[i][1].w, o1.w, o2.w, o3.w);
      const int off = (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4);
      *reinterpret_cast<uint4 *>(sA + off) = o1;
      *reinterpret_cast<uint4 *>(sA + A_SPLIT_BYTES + off) = o2;
      *reinterpret_cast<uint4 *>(sA + 2 * A_SPLIT_BYTES + off) = o3;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // make the stores visible to the tensor core
    if (s + 1 < nslabs) load_slab((s + 1) * TC_SLAB);              // in flight while the tensor core works
    __syncthreads();
    if (s_failed) break;                                           // uniform: written before the barrier
    if (tid == 0) {
      const bool arrived = mbar_wait(full0 + 8 * (s % S), (uint32_t)((s / S) & 1));   // this slab's weights
      ++consumed;
      if (!arrived) s_failed = 1;                                  // seen by everyone after the next barrier
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t aA = smem_u32(sA), aB = smem_u32(sB) + (uint32_t)((s % S) * b_stage_bytes);
      // corrections (smallest first) x1w3, x3w1, x2w2, x1w2, x2w1 into the second accumulator, x1w1 into the first
      const int pa[6] = {0, 2, 1, 0, 1, 0}, pb[6] = {2, 0, 1, 1, 0, 0};
      if (arrived) {
#pragma unroll
        for (int p = 0; p < 6; ++p) {
#pragma unroll
          for (int kk = 0; kk < TC_SLAB / 16; ++kk) {
            const uint64_t da = umma_desc(aA + pa[p] * A_SPLIT_BYTES + kk * 32);
            const uint64_t db = umma_desc(aB + pb[p] * b_split_bytes + kk * 32);
            if (p < 5) umma_bf16(tmem + acc_cols, da, db, idesc, (s > 0 || p > 0 || kk > 0) ? 1u : 0u);
            else umma_bf16(tmem, da, db, idesc, (s > 0 || kk > 0) ? 1u : 0u);
          }
        }
      }
      // committed in either case, so that the other threads' wait for this slab ends
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }
  }
  // copies that were issued but never waited for (only after a failed wait) must land before the block leaves
  if (tid == 0)
    for (int j = consumed; j < issued; ++j) mbar_wait(full0 + 8 * (j % S), (uint32_t)((j / S) & 1));
  // wait for the last committed slab (bounded); on a timeout, count it once per block
  if (!mbar_wait(bar, (uint32_t)((nslabs - 1) & 1))) s_failed = 1;
  __syncthreads();
  const bool ok = (s_failed == 0);
  if (!ok && tid == 0) atomicAdd(&g_tc_wait_timeouts, 1);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  if (ok) {
    tile_epilogue(a, tmem, acc_cols, rows, row0, n0, ncols, sA, warp, lane);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

}  // namespace gphl

using namespace gphl;

extern "C" int64_t gphl_segment_mm_tc_workspace_bytes(int64_t n_types, int64_t k, int64_t n) {
  if (n_types <= 0 || k <= 0 || n <= 0) return 0;
  const int64_t kpad = (k + TC_SLAB - 1) / TC_SLAB * TC_SLAB, npad = (n + 15) / 16 * 16;
  return 3 * n_types * npad * kpad * (int64_t)sizeof(__nv_bfloat16);
}

// Tensor map over the split weights: a (3 * T * Npad) x Kpad matrix of bf16, K contiguous; one box = 64 K-values
// (128 bytes, the swizzle span) x box_rows rows.  cuTensorMapEncodeTiled is reached through the runtime's driver
// entry-point query, so the library does not link against the driver.
namespace gphl {
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
}  // namespace gphl

// Splits and transposes the weights into `workspace` (gphl_segment_mm_tc_workspace_bytes): the part of the typed
// linear that depends on the weights alone.  A caller whose weights are constants of a layer does it once and calls
// gphl_segment_mm_tc_prepared_f32 afterwards.
extern "C" int gphl_segment_mm_tc_prepare_weights(const float *w, int64_t n_types, int64_t k, int64_t n, void *workspace,
                                                  void *stream_) {
  GPHL_REQUIRE(n_types >= 0 && k >= 0 && n >= 0, "negative size");
  GPHL_REQUIRE(k < (1 << 16) && n < (1 << 16) && n_types < (1 << 20), "size out of range");
  if (n == 0 || n_types == 0 || k == 0) return GPHL_OK;
  GPHL_REQUIRE(w && workspace && aligned16(workspace), "null or unaligned pointer argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int32_t kpad = (int32_t)((k + TC_SLAB - 1) / TC_SLAB * TC_SLAB), npad = (int32_t)((n + 15) / 16 * 16);
  const int64_t total = n_types * (int64_t)npad * kpad;
  split_weights_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, 148 * 16), 256, 0, stream>>>(
      w, (int32_t)n_types, (int32_t)k, (int32_t)n, kpad, npad, static_cast<__nv_bfloat16 *>(workspace));
  return launched("split_weights_kernel");
}

static int tc_prepared(const float *x, const void *workspace, const int32_t *type_pointer, int64_t n_types, int64_t m,
                       int64_t k, int64_t n, const int64_t *gather_idx, const float *row_scale, int32_t relu, float *y,
                       int32_t n_peers, void *const *peer_base, const int32_t *fan_ptr, const int64_t *fan_entry,
                       void *stream_) {
  GPHL_REQUIRE(n_types >= 0 && m >= 0 && k >= 0 && n >= 0, "negative size");
  GPHL_REQUIRE(m < INT32_MAX && k < (1 << 16) && n < (1 << 16) && n_types < (1 << 20), "size out of range");
  if (m == 0 || n == 0 || n_types == 0) return GPHL_OK;
  GPHL_REQUIRE(x && type_pointer && workspace && (y || fan_ptr), "null pointer argument");
  GPHL_REQUIRE(!fan_ptr || (fan_entry && peer_base && n_peers >= 1 && n_peers <= GPHL_MAX_PEERS),
               "segment_mm_tc: fan-out needs entries and between 1 and %d receiver buffers", GPHL_MAX_PEERS);
  if (k % 4 != 0 || k == 0 || !aligned16(x) || !aligned16(workspace) || !aligned16(y))
    return fail(GPHL_ERR_UNSUPPORTED, "segment_mm_tc needs k %% 4 == 0 and 16-byte aligned x, y and workspace");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int32_t kpad = (int32_t)((k + TC_SLAB - 1) / TC_SLAB * TC_SLAB), npad = (int32_t)((n + 15) / 16 * 16);
  TcArgs a{};
  a.x = x, a.ws = static_cast<const __nv_bfloat16 *>(workspace), a.ptr = type_pointer, a.gather = gather_idx;
  a.row_scale = row_scale, a.y = y, a.m = m, a.T = (int32_t)n_types, a.K = (int32_t)k, a.N = (int32_t)n;
  a.Kpad = kpad, a.Npad = npad, a.relu = relu;
  a.fan_ptr = fan_ptr, a.fan_entry = fan_entry;
  if (fan_ptr)
    for (int i = 0; i < n_peers; ++i) {
      GPHL_REQUIRE(peer_base[i] == nullptr || aligned16(peer_base[i]), "segment_mm_tc: receiver buffers must be 16-byte aligned");
      a.fan_base[i] = static_cast<float *>(peer_base[i]);
    }
  a.box_rows = std::min<int>(TC_NMAX, npad);
  // two weight slabs in shared memory where two blocks still share an SM (boxes of at most 64 rows: 1 + 48 + 2 x 24
  // KB); with 128-row boxes a second slab would leave one block per SM, and two blocks with one slab each overlap
  // their phases better (measured)
  const size_t stage_bytes = 3 * (size_t)a.box_rows * 128;
  const int forced = knob("GPHL_TC_STAGES", 0);
  a.stages = forced ? std::min(2, std::max(1, forced)) : (a.box_rows <= 64 ? 2 : 1);
  const size_t smem = 1024 + 3 * (size_t)A_SPLIT_BYTES + a.stages * stage_bytes;

  EncodeTiledFn enc = encode_tiled();
  if (!enc) return fail(GPHL_ERR_CUDA, "segment_mm_tc: cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap wmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)kpad, (cuuint64_t)(3 * n_types * npad)};
  const cuuint64_t gstride[1] = {(cuuint64_t)kpad * sizeof(__nv_bfloat16)};
  const cuuint32_t box[2] = {(cuuint32_t)TC_SLAB, (cuuint32_t)a.box_rows};
  const cuuint32_t estride[2] = {1, 1};
  const CUresult cr = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(workspace), gdim, gstride, box, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(GPHL_ERR_CUDA, "segment_mm_tc: cuTensorMapEncodeTiled failed (%d)", (int)cr);
  {
    // the opt-in is a per-device attribute of the function: set it on every call (a process may use several GPUs)
    cudaError_t e = cudaFuncSetAttribute(segment_mm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         1024 + 3 * A_SPLIT_BYTES + 2 * 3 * TC_NMAX * 128);
    if (e != cudaSuccess) return fail(GPHL_ERR_CUDA, "segment_mm_tc: shared memory opt-in: %s", cudaGetErrorString(e));
  }
  const int64_t row_tiles = (m + TC_M - 1) / TC_M + n_types;
  const int64_t blocks = row_tiles * ((npad + TC_NMAX - 1) / TC_NMAX);
  GPHL_REQUIRE(blocks <= 2147483647LL, "too many tiles");
  segment_mm_tc_kernel<<<(unsigned)blocks, TC_THREADS, smem, stream>>>(a, wmap);
  return launched("segment_mm_tc_kernel");
}

extern "C" int gphl_segment_mm_tc_prepared_f32(const float *x, const void *workspace, const int32_t *type_pointer,
                                               int64_t n_types, int64_t m, int64_t k, int64_t n, const int64_t *gather_idx,
                                               const float *row_scale, int32_t relu, float *y, void *stream_) {
  GPHL_REQUIRE(y != nullptr || m == 0 || n == 0 || n_types == 0, "null pointer argument");
  return tc_prepared(x, workspace, type_pointer, n_types, m, k, n, gather_idx, row_scale, relu, y, 0, nullptr, nullptr, nullptr,
                     stream_);
}

// The typed linear with the sending side of a sparse row exchange fused into its epilogue: every finished 128-row
// tile is stored, 128-byte row segment by row segment, to the rows of the receivers' buffers that read it (`y` may be
// NULL when nobody needs the rows locally).  One kernel computes and sends; the receivers synchronise afterwards.
extern "C" int gphl_segment_mm_tc_fanout_f32(const float *x, const void *workspace, const int32_t *type_pointer,
                                             int64_t n_types, int64_t m, int64_t k, int64_t n, const float *row_scale,
                                             int32_t relu, float *y, int32_t n_peers, void *const *peer_base,
                                             const int32_t *fan_ptr, const int64_t *fan_entry, void *stream_) {
  GPHL_REQUIRE(fan_ptr != nullptr || m == 0, "segment_mm_tc_fanout: fan_ptr is NULL");
  return tc_prepared(x, workspace, type_pointer, n_types, m, k, n, nullptr, row_scale, relu, y, n_peers, peer_base, fan_ptr,
                     fan_entry, stream_);
}

extern "C" int gphl_segment_mm_tc_f32(const float *x, const float *w, const int32_t *type_pointer, int64_t n_types,
                                      int64_t m, int64_t k, int64_t n, const int64_t *gather_idx, const float *row_scale,
                                      int32_t relu, void *workspace, float *y, void *stream_) {
  if (m == 0 || n == 0 || n_types == 0) return GPHL_OK;
  GPHL_REQUIRE(w != nullptr, "null pointer argument");
  if (k % 4 != 0 || k <= 0 || !aligned16(x) || !aligned16(workspace) || !aligned16(y))
    return fail(GPHL_ERR_UNSUPPORTED, "segment_mm_tc needs k %% 4 == 0 and 16-byte aligned x, y and workspace");
  int rc = gphl_segment_mm_tc_prepare_weights(w, n_types, k, n, workspace, stream_);
  if (rc != GPHL_OK) return rc;
  return gphl_segment_mm_tc_prepared_f32(x, workspace, type_pointer, n_types, m, k, n, gather_idx, row_scale, relu, y, stream_);
}

// Self-test of the bounded wait: one warp waits, with a short poll limit, on an mbarrier that nothing ever
// completes; the wait must give up, count the timeout and return, leaving the context usable.
namespace gphl {
__global__ void wait_selftest_kernel(uint32_t polls) {
  __shared__ uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  bool done = false;
  for (uint32_t i = 0; i < polls && !done; ++i) {
    uint32_t d;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(d)
        : "r"(b), "r"(0u)
        : "memory");
    done = d != 0;
  }
  if (!done && threadIdx.x == 0) atomicAdd(&g_tc_wait_timeouts, 1);
}
}  // namespace gphl

extern "C" int gphl_debug_wait_selftest(int32_t polls, void *stream) {
  GPHL_REQUIRE(polls >= 1 && polls <= (1 << 20), "polls must be in [1, 2^20]");
  gphl::wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>((uint32_t)polls);
  return gphl::launched("wait_selftest_kernel");
}

extern "C" int gphl_debug_reset_wait_timeouts(void) {
  const int zero = 0;
  GPHL_CUDA(cudaMemcpyToSymbol(gphl::g_tc_wait_timeouts, &zero, sizeof(int)));
  return GPHL_OK;
}

// Number of barrier waits that ran out in tensor-core kernels since the library was loaded
// (0 in a healthy process).  Synchronises the device.
extern "C" int gphl_tc_wait_timeouts(int *count) {
  GPHL_REQUIRE(count != nullptr, "null pointer argument");
  GPHL_CUDA(cudaMemcpyFromSymbol(count, g_tc_wait_timeouts, sizeof(int)));
  return GPHL_OK;
}
