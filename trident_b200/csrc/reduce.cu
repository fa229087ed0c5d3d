// Row reductions Sum, Mean, Var and VarMean of a 2-D tensor along either dimension, forward and
// backward, as single-pass HBM-bound kernels (the reference launches one Triton program per
// output element: trident/kernel/sum.py:35-92, mean.py, var.py, var_mean.py, with the block
// reductions of trident/language/sum.py, mean.py, var.py).
//
// The problem is described as the reference's util.size_and_stride does (trident/util/util.py:
// 65-76): `y_size` outputs, each reducing `x_size` elements, x[y * y_stride + i * x_stride].
//
//   sum      a = sum_i x_i                     dx_i = da
//   mean     a = sum_i x_i / n                 dx_i = da / n
//   var      a = sum_i (x_i - m)^2 / (n - c)   dx_i = da * 2 (x_i - m) / (n - c)
//   var_mean a = var, b = m                    dx_i = da * 2 (x_i - m) / (n - c) + db / n
//
// Fast path (x_stride == 1, 16-byte aligned rows of a multiple of the vector width): the row is
// read once into registers; variance is the two-pass form (mean, then centred squares) on those
// registers. Algorithmic bytes: forward N*e, backward N*e (sum, mean: a pure write) or 2*N*e.
// Generic path (any strides, in particular reductions down the columns): a CTA of 32 x 8 threads
// owns 32 adjacent outputs, coalesced when y_stride == 1; the data are read once per pass.
#include "row_common.cuh"

namespace tb200 {

enum ReduceKind { RK_SUM = 0, RK_MEAN = 1, RK_VAR = 2, RK_VAR_MEAN = 3 };

// Sums two values over the threads of a row with one shared-memory exchange (slot: [2][32] pairs).
template <bool CTA_ROW>
__device__ inline void row_reduce2(float& a, float& b, float* slot, int& phase) {
  a = warp_sum(a);
  b = warp_sum(b);
  if constexpr (CTA_ROW) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float* s = slot + phase * 32;
    phase ^= 1;
    if (lane == 0) {
      s[warp] = a;
      s[16 + warp] = b;
    }
    __syncthreads();
    a = warp_sum(lane < nwarps ? s[lane] : 0.f);
    b = warp_sum(lane < nwarps ? s[16 + lane] : 0.f);
  }
}

template <typename T, int CHUNKS, bool CTA_ROW, int KIND>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256)
    reduce_fwd_vec(T* __restrict__ out_a, T* __restrict__ out_b, const T* __restrict__ x, int64_t rows,
                   int cols, int64_t row_stride, float correction) {
  constexpr int VEC = Traits<T>::VEC;
  constexpr int PAIRS = VEC / 2;
  __shared__ float slot[64];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  const float n = (float)cols;
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    uint4 raw[CHUNKS];
    const T* xr = x + row * row_stride;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      raw[c] = col < cols ? ld_stream(xr + col) : make_uint4(0, 0, 0, 0);
    }
    if constexpr (KIND == RK_SUM || KIND == RK_MEAN) {
      uint64_t s2 = 0ull;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        uint64_t t[PAIRS];
        unpack2<T>(raw[c], t);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) s2 = am::add2(s2, t[i]);
      }
      const float s = row_reduce<CTA_ROW, false>(hsum2(s2), slot, phase);
      if (rt.tid == 0) out_a[row] = Traits<T>::from_f(KIND == RK_SUM ? s : s / n);
    } else {
      // Variance in one pass over the registers and one exchange: sums of d = x - c and of d^2 with
      // the shift c = a sample of the row (so d is of the order of the spread and the subtraction
      // below does not cancel): mean = c + S1/n, var = (S2 - S1^2/n)/(n-k).
      // (the median of three samples, so that a single outlier cannot become the shift)
      const float q0 = Traits<T>::to_f(__ldg(xr)), q1 = Traits<T>::to_f(__ldg(xr + cols / 2)),
                  q2 = Traits<T>::to_f(__ldg(xr + cols - 1));
      const float shift = fmaxf(fminf(q0, q1), fminf(fmaxf(q0, q1), q2));
      const uint64_t nshift2 = splat2(-shift);
      uint64_t s1 = 0ull, s2 = 0ull;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        if (rt.template col<VEC>(c) < cols) {
          uint64_t t[PAIRS];
          unpack2<T>(raw[c], t);
#pragma unroll
          for (int i = 0; i < PAIRS; ++i) {
            const uint64_t d = am::add2(t[i], nshift2);
            s1 = am::add2(s1, d);
            s2 = am::fma2(d, d, s2);
          }
        }
      }
      float a1 = hsum2(s1), a2 = hsum2(s2);
      row_reduce2<CTA_ROW>(a1, a2, slot, phase);
      if (rt.tid == 0) {
        out_a[row] = Traits<T>::from_f((a2 - a1 * a1 / n) / (n - correction));
        if constexpr (KIND == RK_VAR_MEAN) out_b[row] = Traits<T>::from_f(shift + a1 / n);
      }
    }
  }
}

template <typename T, int CHUNKS, bool CTA_ROW, int KIND>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256)
    reduce_bwd_vec(T* __restrict__ dx, const T* __restrict__ da, const T* __restrict__ db,
                   const T* __restrict__ x, int64_t rows, int cols, int64_t row_stride, float correction) {
  constexpr int VEC = Traits<T>::VEC;
  constexpr int PAIRS = VEC / 2;
  __shared__ float slot[64];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  const float n = (float)cols;
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    T* dr = dx + row * row_stride;
    const float ga = Traits<T>::to_f(da[row]);
    if constexpr (KIND == RK_SUM || KIND == RK_MEAN) {
      uint64_t g[PAIRS];
#pragma unroll
      for (int i = 0; i < PAIRS; ++i) g[i] = splat2(KIND == RK_SUM ? ga : ga / n);
      const uint4 packed = pack2<T>(g);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = rt.template col<VEC>(c);
        if (col < cols) st_stream(dr + col, packed);
      }
    } else {
      uint4 raw[CHUNKS];
      const T* xr = x + row * row_stride;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = rt.template col<VEC>(c);
        raw[c] = col < cols ? ld_stream(xr + col) : make_uint4(0, 0, 0, 0);
      }
      uint64_t s2 = 0ull;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        uint64_t t[PAIRS];
        unpack2<T>(raw[c], t);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) s2 = am::add2(s2, t[i]);
      }
      const float mu = row_reduce<CTA_ROW, false>(hsum2(s2), slot, phase) / n;
      // dx = k (x - mu) + add, k = 2 da / (n - c), add = db / n (var_mean only)
      const float k = 2.f * ga / (n - correction);
      const float add = (KIND == RK_VAR_MEAN && db) ? Traits<T>::to_f(db[row]) / n : 0.f;
      const uint64_t k2 = splat2(k), off2 = splat2(add - k * mu);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = rt.template col<VEC>(c);
        if (col < cols) {
          uint64_t t[PAIRS];
          unpack2<T>(raw[c], t);
#pragma unroll
          for (int i = 0; i < PAIRS; ++i) t[i] = am::fma2(t[i], k2, off2);
          st_stream(dr + col, pack2<T>(t));
        }
      }
    }
  }
}

// Generic path: block (32, 8); threadIdx.x picks one of 32 adjacent outputs, threadIdx.y splits the
// reduced range. Sums over threadIdx.y go through shared memory in a fixed order.
__device__ inline float fold8(float v, float (*red)[33]) {
  red[threadIdx.y][threadIdx.x] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s += red[j][threadIdx.x];
  __syncthreads();
  return s;
}

template <typename T>
__global__ void __launch_bounds__(256)
    reduce_fwd_generic(T* out_a, T* out_b, const T* x, int64_t y_size, int64_t x_size, int64_t y_stride,
                       int64_t x_stride, int kind, float correction) {
  __shared__ float red[8][33];
  const int64_t y = (int64_t)blockIdx.x * 32 + threadIdx.x;
  const bool live = y < y_size;
  const T* base = x + (live ? y : 0) * y_stride;
  const float n = (float)x_size;
  float s = 0.f;
  if (live)
    for (int64_t i = threadIdx.y; i < x_size; i += 8) s += Traits<T>::to_f(base[i * x_stride]);
  s = fold8(s, red);
  float a = s, mu = s / n;
  if (kind == RK_MEAN) a = mu;
  if (kind >= RK_VAR) {
    float v = 0.f;
    if (live)
      for (int64_t i = threadIdx.y; i < x_size; i += 8) {
        const float d = Traits<T>::to_f(base[i * x_stride]) - mu;
        v = fmaf(d, d, v);
      }
    a = fold8(v, red) / (n - correction);
  }
  if (live && threadIdx.y == 0) {
    out_a[y] = Traits<T>::from_f(a);
    if (kind == RK_VAR_MEAN) out_b[y] = Traits<T>::from_f(mu);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
    reduce_bwd_generic(T* dx, const T* da, const T* db, const T* x, int64_t y_size, int64_t x_size,
                       int64_t y_stride, int64_t x_stride, int kind, float correction) {
  __shared__ float red[8][33];
  const int64_t y = (int64_t)blockIdx.x * 32 + threadIdx.x;
  const bool live = y < y_size;
  const int64_t off = (live ? y : 0) * y_stride;
  const float n = (float)x_size;
  const float ga = live ? Traits<T>::to_f(da[y]) : 0.f;
  if (kind <= RK_MEAN) {
    const T g = Traits<T>::from_f(kind == RK_SUM ? ga : ga / n);
    if (live)
      for (int64_t i = threadIdx.y; i < x_size; i += 8) dx[off + i * x_stride] = g;
    return;
  }
  float s = 0.f;
  if (live)
    for (int64_t i = threadIdx.y; i < x_size; i += 8) s += Traits<T>::to_f(x[off + i * x_stride]);
  const float mu = fold8(s, red) / n;
  const float k = 2.f * ga / (n - correction);
  const float add = (kind == RK_VAR_MEAN && db && live) ? Traits<T>::to_f(db[y]) / n : 0.f;
  if (live)
    for (int64_t i = threadIdx.y; i < x_size; i += 8)
      dx[off + i * x_stride] = Traits<T>::from_f(fmaf(Traits<T>::to_f(x[off + i * x_stride]) - mu, k, add));
}

template <typename Fn>
static int dispatch_kind(int kind, Fn&& fn) {
  switch (kind) {
    case RK_SUM: return fn(IntC<RK_SUM>{});
    case RK_MEAN: return fn(IntC<RK_MEAN>{});
    case RK_VAR: return fn(IntC<RK_VAR>{});
    case RK_VAR_MEAN: return fn(IntC<RK_VAR_MEAN>{});
  }
  set_error("unknown reduction kind %d", kind);
  return TB200_ERR_INVALID;
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_reduce_fwd(void* out_a, void* out_b, const void* x, int64_t y_size, int64_t x_size,
                                int64_t y_stride, int64_t x_stride, int kind, float correction, int dtype,
                                void* stream) {
  TB200_REQUIRE(kind >= RK_SUM && kind <= RK_VAR_MEAN, TB200_ERR_INVALID, "reduce_fwd: unknown kind %d", kind);
  TB200_REQUIRE(y_size >= 0 && x_size > 0, TB200_ERR_INVALID, "reduce_fwd: bad shape");
  if (y_size == 0) return 0;
  TB200_REQUIRE(out_a && x, TB200_ERR_INVALID, "reduce_fwd: null pointer");
  TB200_REQUIRE(kind != RK_VAR_MEAN || out_b, TB200_ERR_INVALID, "reduce_fwd: var_mean needs two outputs");
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Traits<T>::VEC;
    const bool ok = aligned16(x) && x_stride == 1 && y_stride % VEC == 0 && y_stride >= x_size && x_size < (1 << 30);
    RowPlan p = plan_rows<T>(x_size, ok);
    if (p.vec) {
      const int64_t grid = ceil_div(y_size, p.rows_per_cta);
      int rc = dispatch_kind(kind, [&](auto k) -> int {
        return dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
          reduce_fwd_vec<T, decltype(c)::value, decltype(cta)::value, decltype(k)::value>
              <<<(unsigned)grid, p.threads, 0, st>>>((T*)out_a, (T*)out_b, (const T*)x, y_size, (int)x_size,
                                                     y_stride, correction);
          return launch_status("reduce_fwd_vec");
        });
      });
      if (rc == 0) note_kernel("row_vec", 1);
      return rc;
    }
    reduce_fwd_generic<T><<<(unsigned)ceil_div(y_size, 32), dim3(32, 8), 0, st>>>(
        (T*)out_a, (T*)out_b, (const T*)x, y_size, x_size, y_stride, x_stride, kind, correction);
    int rc = launch_status("reduce_fwd_generic");
    if (rc == 0) note_kernel("row_generic", 1);
    return rc;
  });
}

extern "C" int tb200_reduce_bwd(void* dx, const void* dout_a, const void* dout_b, const void* x, int64_t y_size,
                                int64_t x_size, int64_t y_stride, int64_t x_stride, int kind, float correction,
                                int dtype, void* stream) {
  TB200_REQUIRE(kind >= RK_SUM && kind <= RK_VAR_MEAN, TB200_ERR_INVALID, "reduce_bwd: unknown kind %d", kind);
  TB200_REQUIRE(y_size >= 0 && x_size > 0, TB200_ERR_INVALID, "reduce_bwd: bad shape");
  if (y_size == 0) return 0;
  TB200_REQUIRE(dx && dout_a, TB200_ERR_INVALID, "reduce_bwd: null pointer");
  TB200_REQUIRE(kind < RK_VAR || x, TB200_ERR_INVALID, "reduce_bwd: the variance gradient needs the input");
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Traits<T>::VEC;
    const bool ok = aligned16(dx) && (kind < RK_VAR || aligned16(x)) && x_stride == 1 && y_stride % VEC == 0 &&
                    y_stride >= x_size && x_size < (1 << 30);
    RowPlan p = plan_rows<T>(x_size, ok);
    if (p.vec) {
      const int64_t grid = ceil_div(y_size, p.rows_per_cta);
      int rc = dispatch_kind(kind, [&](auto k) -> int {
        return dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
          reduce_bwd_vec<T, decltype(c)::value, decltype(cta)::value, decltype(k)::value>
              <<<(unsigned)grid, p.threads, 0, st>>>((T*)dx, (const T*)dout_a, (const T*)dout_b, (const T*)x,
                                                     y_size, (int)x_size, y_stride, correction);
          return launch_status("reduce_bwd_vec");
        });
      });
      if (rc == 0) note_kernel("row_vec", 1);
      return rc;
    }
    reduce_bwd_generic<T><<<(unsigned)ceil_div(y_size, 32), dim3(32, 8), 0, st>>>(
        (T*)dx, (const T*)dout_a, (const T*)dout_b, (const T*)x, y_size, x_size, y_stride, x_stride, kind,
        correction);
    int rc = launch_status("reduce_bwd_generic");
    if (rc == 0) note_kernel("row_generic", 1);
    return rc;
  });
}
