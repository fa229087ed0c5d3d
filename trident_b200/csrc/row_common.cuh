// Launch planning and register-resident row access shared by the HBM-bound row kernels
// (LayerNorm, RMSNorm, Softmax, MaskedSoftmax).
//
// Fast path ("row_vec"): every row is read once into registers with 16-byte loads and
// written once with 16-byte stores. Rows of up to 32*MAXC vectors are owned by one warp
// (shuffle reductions only); longer rows are owned by a whole CTA of 128..512 threads
// (one shared-memory exchange per reduction). Thread t of a row owns vectors
// t, t+R, t+2R, ... (R = threads per row) so that every load instruction of a warp
// covers one contiguous 512-byte span.
//
// Generic path ("row_generic"): one warp per row, scalar strided accesses, the row is
// re-read from L1/L2 for each pass. It covers widths that are not a multiple of the
// vector width, unaligned bases, strided (dim=0) softmax and very long rows.
#pragma once

#include <type_traits>

#include "attn_math.cuh"
#include "common.cuh"

namespace tb200 {

struct RowPlan {
  bool vec = false;     // false: generic path
  bool cta_row = false; // true: a CTA per row, false: a warp per row
  int chunks = 1;       // 16-byte vectors per thread (power of two)
  int threads = 256;    // block size
  int rows_per_cta = 8;
};

template <typename T>
constexpr int max_chunks() { return sizeof(T) == 4 ? 8 : 4; }

static inline int next_pow2(int64_t v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

// `ptrs_ok`: every tensor base is 16-byte aligned and every row pitch is a multiple of
// the vector width. `cta_max_chunks` bounds the vectors per thread of CTA-per-row plans
// (kernels that also carry per-column accumulators ask for fewer to stay in registers).
template <typename T>
static inline RowPlan plan_rows(int64_t cols, bool ptrs_ok, int cta_max_chunks = max_chunks<T>()) {
  RowPlan p;
  constexpr int VEC = Traits<T>::VEC;
  constexpr int MAXC = max_chunks<T>();
  if (!ptrs_ok || cols % VEC != 0 || cols <= 0) return p;
  const int64_t vecs = cols / VEC;
  // A warp owns a row only while two vectors per lane cover it: wider rows in one warp need so
  // many registers that a single 8-warp CTA fits on an SM and too few rows are in flight
  // (measured: 1024 fp32 columns per warp reached 2.9 TB/s, the same row split over a
  // 128-thread CTA behaves like the softmax kernels, which run at the HBM roofline).
  (void)MAXC;
  if (vecs <= 64) {
    p.vec = true;
    p.cta_row = false;
    p.chunks = next_pow2(ceil_div(vecs, 32));
    p.threads = 256;
    p.rows_per_cta = 8;
    return p;
  }
  int threads = next_pow2(ceil_div(vecs, cta_max_chunks));
  if (threads < 128) threads = 128;
  if (threads > 512) return p;
  p.vec = true;
  p.cta_row = true;
  p.threads = threads;
  p.chunks = next_pow2(ceil_div(vecs, threads));
  p.rows_per_cta = 1;
  return p;
}

template <int C>
using IntC = std::integral_constant<int, C>;
template <bool B>
using BoolC = std::integral_constant<bool, B>;

// Calls fn(IntC<chunks>, BoolC<cta_row>) for the plan's compile-time shape.
template <typename T, typename Fn>
static inline int dispatch_plan(const RowPlan& p, Fn&& fn) {
  if (p.cta_row) {
    switch (p.chunks) {
      case 1: return fn(IntC<1>{}, BoolC<true>{});
      case 2: return fn(IntC<2>{}, BoolC<true>{});
      case 4: return fn(IntC<4>{}, BoolC<true>{});
      case 8:
        if constexpr (max_chunks<T>() >= 8) return fn(IntC<8>{}, BoolC<true>{});
    }
  } else {
    switch (p.chunks) {
      case 1: return fn(IntC<1>{}, BoolC<false>{});
      case 2: return fn(IntC<2>{}, BoolC<false>{});
      case 4: return fn(IntC<4>{}, BoolC<false>{});
      case 8:
        if constexpr (max_chunks<T>() >= 8) return fn(IntC<8>{}, BoolC<false>{});
    }
  }
  set_error("internal: bad row plan (chunks=%d)", p.chunks);
  return TB200_ERR_INVALID;
}

// A 16-byte vector of T as fp32 pairs packed in 64-bit registers, for the two-lane fp32
// instructions (fma/mul/add .f32x2): they halve the arithmetic instruction count of the row
// kernels, which are close to issue-bound once their loads are in flight.
template <typename T>
__device__ inline void unpack2(const uint4& raw, uint64_t (&out)[Traits<T>::VEC / 2]);
template <>
__device__ inline void unpack2<float>(const uint4& raw, uint64_t (&out)[2]) {
  out[0] = am::pack2u(raw.x, raw.y);
  out[1] = am::pack2u(raw.z, raw.w);
}
template <>
__device__ inline void unpack2<__nv_bfloat16>(const uint4& raw, uint64_t (&out)[4]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = am::pack2u(w[i] << 16, w[i] & 0xffff0000u);
}
template <>
__device__ inline void unpack2<__half>(const uint4& raw, uint64_t (&out)[4]) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    out[i] = am::pack2f(f.x, f.y);
  }
}
template <typename T>
__device__ inline uint4 pack2(const uint64_t (&in)[Traits<T>::VEC / 2]) {
  uint4 r;
  uint32_t* w = reinterpret_cast<uint32_t*>(&r);
  if constexpr (sizeof(T) == 4) {
    float a, b;
    am::unpack2f(in[0], a, b);
    w[0] = __float_as_uint(a);
    w[1] = __float_as_uint(b);
    am::unpack2f(in[1], a, b);
    w[2] = __float_as_uint(a);
    w[3] = __float_as_uint(b);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a, b;
      am::unpack2f(in[i], a, b);
      w[i] = am::cvt_pair<T>(a, b);
    }
  }
  return r;
}
__device__ inline uint64_t splat2(float v) { return am::pack2f(v, v); }
__device__ inline float hsum2(uint64_t v) {
  float a, b;
  am::unpack2f(v, a, b);
  return a + b;
}

// Position of the calling thread inside the row decomposition.
template <bool CTA_ROW>
struct RowThread {
  int row_threads, tid, rows_per_cta, local_row;
  __device__ RowThread() {
    if constexpr (CTA_ROW) {
      row_threads = blockDim.x;
      tid = threadIdx.x;
      rows_per_cta = 1;
      local_row = 0;
    } else {
      row_threads = 32;
      tid = threadIdx.x & 31;
      rows_per_cta = blockDim.x >> 5;
      local_row = threadIdx.x >> 5;
    }
  }
  __device__ int64_t first_row() const { return (int64_t)blockIdx.x * rows_per_cta + local_row; }
  __device__ int64_t row_step() const { return (int64_t)gridDim.x * rows_per_cta; }
  // first column of chunk c
  template <int VEC>
  __device__ int col(int c) const { return (c * row_threads + tid) * VEC; }
};

// Loads CHUNKS vectors of one row into floats; out-of-range vectors read as `fill`.
template <typename T, int CHUNKS, bool CTA_ROW, bool STREAM = true>
__device__ inline void load_row(float (&dst)[CHUNKS][Traits<T>::VEC], const T* row_ptr, int cols,
                                const RowThread<CTA_ROW>& rt, float fill = 0.f) {
  constexpr int VEC = Traits<T>::VEC;
  uint4 raw[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = rt.template col<VEC>(c);
    if (col < cols) raw[c] = STREAM ? ld_stream(row_ptr + col) : ld_cached(row_ptr + col);
  }
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = rt.template col<VEC>(c);
    if (col < cols) {
      unpack<T>(raw[c], dst[c]);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) dst[c][i] = fill;
    }
  }
}

template <typename T, int CHUNKS, bool CTA_ROW>
__device__ inline void store_row(T* row_ptr, const float (&src)[CHUNKS][Traits<T>::VEC], int cols,
                                 const RowThread<CTA_ROW>& rt) {
  constexpr int VEC = Traits<T>::VEC;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = rt.template col<VEC>(c);
    if (col < cols) st_stream(row_ptr + col, pack<T>(src[c]));
  }
}

// Grid for kernels that write one partial column-sum row per CTA: a bounded, SM-sized
// grid. `ctas_per_sm` is 2 for warp-per-row plans and for small CTAs.
static inline int64_t persistent_grid(const RowPlan& p, int64_t rows) {
  const int64_t want = ceil_div(rows, p.rows_per_cta);
  int per_sm = p.cta_row ? (p.threads <= 256 ? 4 : 2) : 2;
  const int64_t cap = (int64_t)sm_count() * per_sm;
  return want < cap ? want : cap;
}

// Column partial sums: partial[p][which][col], p < nparts, which < gridDim.y (1 or 2),
// reduced by this kernel into out_a (which = 0) and out_b (which = 1); null outputs are
// skipped. Block (32, 32):
// threadIdx.x walks columns (coalesced), threadIdx.y splits the partial rows.
template <typename T>
__global__ void colsum_finalize_kernel(T* out_a, T* out_b, const float* partial, int nparts,
                                       int cols) {
  __shared__ float tile[32][33];
  const int which = blockIdx.y;
  T* out = which == 0 ? out_a : out_b;
  if (out == nullptr) return;
  const int col = blockIdx.x * 32 + threadIdx.x;
  float acc = 0.f;
  if (col < cols) {
    // eight independent loads per trip: the kernel is a chain of load latencies otherwise
    for (int p0 = threadIdx.y; p0 < nparts; p0 += 32 * 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int p = p0 + 32 * j;
        v[j] = p < nparts ? __ldg(partial + ((int64_t)p * gridDim.y + which) * cols + col) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += v[j];
    }
  }
  tile[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < cols) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) s += tile[i][threadIdx.x];
    out[col] = Traits<T>::from_f(s);
  }
}

// Adds this thread's per-column accumulators into the CTA's partial row of the
// workspace. Warp-per-row plans first fold the CTA's warps together (fixed order, so
// the result does not depend on scheduling).
template <int CHUNKS, int VEC, bool CTA_ROW>
__device__ inline void write_col_partials(float* partial_row /*[2][cols]*/, int cols,
                                          const float (&acc_a)[CHUNKS][VEC],
                                          const float (&acc_b)[CHUNKS][VEC],
                                          const RowThread<CTA_ROW>& rt, float* smem /*2*cols or null*/) {
  if constexpr (CTA_ROW) {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      if (col < cols) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
          *reinterpret_cast<float4*>(partial_row + col + i) =
              make_float4(acc_a[c][i], acc_a[c][i + 1], acc_a[c][i + 2], acc_a[c][i + 3]);
          *reinterpret_cast<float4*>(partial_row + cols + col + i) =
              make_float4(acc_b[c][i], acc_b[c][i + 1], acc_b[c][i + 2], acc_b[c][i + 3]);
        }
      }
    }
  } else {
    const int nwarps = blockDim.x >> 5;
    for (int w = 0; w < nwarps; ++w) {
      if (rt.local_row == w) {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const int col = rt.template col<VEC>(c);
          if (col < cols) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
              if (w == 0) {
                smem[col + i] = acc_a[c][i];
                smem[cols + col + i] = acc_b[c][i];
              } else {
                smem[col + i] += acc_a[c][i];
                smem[cols + col + i] += acc_b[c][i];
              }
            }
          }
        }
      }
      __syncthreads();
    }
    for (int i = threadIdx.x * 4; i < 2 * cols; i += blockDim.x * 4)
      *reinterpret_cast<float4*>(partial_row + i) = *reinterpret_cast<const float4*>(smem + i);
  }
}

}  // namespace tb200
