// LayerNorm and RMSNorm, forward and backward, as single-pass HBM-bound row kernels.
//
// Math (all reductions and statistics in fp32, outputs rounded once):
//   LayerNorm  fwd: mu = mean(x); var = mean((x-mu)^2); rstd = rsqrt(var+eps);
//                   y = (x-mu)*rstd*w + b                       (w, b optional)
//              bwd: g = dy*w; c1 = mean(g*xhat); c2 = mean(g);
//                   dx = rstd*(g - xhat*c1 - c2); dw = sum_rows dy*xhat; db = sum_rows dy
//     (restates trident/kernel/layer_norm.py:72-126 and :188-246 plus the torch.sum
//      calls of trident/operation/layer_norm.py:112-122)
//   RMSNorm    fwd: rms = sqrt(sum_{i<P} x_i^2 / P); y = x/(rms+eps)*w (+ b)
//              bwd: g = dy*w; s = sum_i g_i*x_i;
//                   dx_i = g_i/(rms+eps) - [i<P] x_i*s / (P*rms*(rms+eps)^2);
//                   dw = sum_rows dy*x/(rms+eps); db = sum_rows dy
//     (restates trident/kernel/rms_norm.py:74-117 and :190-232, with the exact derivative
//      of the forward expression; eps sits outside the square root as in
//      tests/test_rms_norm.py:22-39)
//
// Algorithmic HBM bytes per element of the [rows, cols] problem: forward 2*e (read x,
// write y), backward 3*e (read x and dy, write dx); the weight-gradient column sums add
// one fp32 partial row per CTA (grid bounded by the SM count), reduced by a second small
// kernel.
#include <cooperative_groups.h>

#include <type_traits>

#include "row_common.cuh"

namespace tb200 {

// Grouped backward kernels (defined at the end of this file): they take rows of up to 1024
// vectors; *handled tells the caller whether they launched.
int try_layer_norm_bwd_grouped(void* dx, void* dweight, void* dbias, const void* dy, const void* x,
                               const void* weight, const float* mean, const float* rstd, void* workspace,
                               size_t workspace_bytes, int64_t rows, int64_t cols, int dtype, cudaStream_t st,
                               bool* handled, bool allow_fused);
int try_rms_norm_bwd_grouped(void* dx, void* dweight, void* dbias, const void* dy, const void* x,
                             const void* weight, const float* rms, void* workspace, size_t workspace_bytes,
                             int64_t rows, int64_t cols, int64_t row_stride, int64_t col_stride,
                             int64_t partial_cols, float eps, int dtype, cudaStream_t st, bool* handled);

// ------------------------------------------------------------------ LayerNorm fwd
// The row stays packed in registers (16-byte vectors as loaded) and is unpacked once per
// pass (sum, centred squares, output): for 16-bit rows that halves the live registers, which
// is what decides how many rows an SM keeps in flight.
template <typename T, int CHUNKS, bool CTA_ROW>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256, CTA_ROW ? 2 : 4)
    ln_fwd_vec(T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd,
               const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
               int64_t rows, int cols, float eps) {
  constexpr int VEC = Traits<T>::VEC;
  __shared__ float slot[64];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  const float inv_n = 1.f / (float)cols;
  pdl_wait();     // (programmatic dependent launch: nothing is read before the previous kernel is done)
  pdl_release();  // the next kernel of the stream may be scheduled
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    uint4 raw[CHUNKS];
    const T* xr = x + row * cols;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      raw[c] = col < cols ? ld_stream(xr + col) : make_uint4(0, 0, 0, 0);
    }
    // weight and bias are requested before the reductions, so that their (L2) latency hides
    // behind the row's own load instead of following the second barrier
    // (only while the registers allow it)
    constexpr bool EARLY = CHUNKS == 1 || (CHUNKS == 2 && sizeof(T) == 4);
    uint4 wraw[EARLY ? CHUNKS : 1], braw[EARLY ? CHUNKS : 1];
    if constexpr (EARLY) {
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = rt.template col<VEC>(c);
        wraw[c] = (w && col < cols) ? ld_cached(w + col) : make_uint4(0, 0, 0, 0);
        braw[c] = (b && col < cols) ? ld_cached(b + col) : make_uint4(0, 0, 0, 0);
      }
    }
    constexpr int PAIRS = VEC / 2;  // arithmetic on fp32 pairs (two-lane instructions)
    uint64_t s2 = 0ull;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      uint64_t t[PAIRS];
      unpack2<T>(raw[c], t);
#pragma unroll
      for (int i = 0; i < PAIRS; ++i) s2 = am::add2(s2, t[i]);
    }
    const float mu = row_reduce<CTA_ROW, false>(hsum2(s2), slot, phase) * inv_n;
    const uint64_t nmu2 = splat2(-mu);
    uint64_t v2 = 0ull;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      if (rt.template col<VEC>(c) < cols) {
        uint64_t t[PAIRS];
        unpack2<T>(raw[c], t);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
          const uint64_t d = am::add2(t[i], nmu2);
          v2 = am::fma2(d, d, v2);
        }
      }
    }
    const float var = row_reduce<CTA_ROW, false>(hsum2(v2), slot, phase) * inv_n;
    const float rs = rsqrtf(var + eps);
    const uint64_t rs2 = splat2(rs);
    T* yr = y + row * cols;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      if (col < cols) {
        uint64_t t[PAIRS], ws[PAIRS], bs[PAIRS];
        unpack2<T>(raw[c], t);
        if (w) unpack2<T>(EARLY ? wraw[EARLY ? c : 0] : ld_cached(w + col), ws);
        if (b) unpack2<T>(EARLY ? braw[EARLY ? c : 0] : ld_cached(b + col), bs);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
          uint64_t o = am::mul2(am::add2(t[i], nmu2), rs2);
          if (w) o = b ? am::fma2(o, ws[i], bs[i]) : am::mul2(o, ws[i]);
          else if (b) o = am::add2(o, bs[i]);
          t[i] = o;
        }
        st_stream(yr + col, pack2<T>(t));
      }
    }
    if (rt.tid == 0) {
      mean[row] = mu;
      rstd[row] = rs;
    }
  }
}

template <typename T>
__global__ void ln_fwd_generic(T* y, float* mean, float* rstd, const T* x, const T* w, const T* b,
                               int64_t rows, int64_t cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * cols;
  float s = 0.f;
  for (int64_t i = lane; i < cols; i += 32) s += Traits<T>::to_f(xr[i]);
  const float mu = warp_sum(s) / (float)cols;
  float v = 0.f;
  for (int64_t i = lane; i < cols; i += 32) {
    const float d = Traits<T>::to_f(xr[i]) - mu;
    v += d * d;
  }
  const float rs = rsqrtf(warp_sum(v) / (float)cols + eps);
  T* yr = y + row * cols;
  for (int64_t i = lane; i < cols; i += 32) {
    float o = (Traits<T>::to_f(xr[i]) - mu) * rs;
    if (w) o *= Traits<T>::to_f(w[i]);
    if (b) o += Traits<T>::to_f(b[i]);
    yr[i] = Traits<T>::from_f(o);
  }
  if (lane == 0) {
    mean[row] = mu;
    rstd[row] = rs;
  }
}

// ------------------------------------------------------------------ LayerNorm bwd
template <typename T, int CHUNKS, bool CTA_ROW>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256)
    ln_bwd_vec(T* __restrict__ dx, float* __restrict__ partial, const T* __restrict__ dy,
               const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ mean,
               const float* __restrict__ rstd, int64_t rows, int cols, int want_cols) {
  constexpr int VEC = Traits<T>::VEC;
  __shared__ float slot[64];
  __shared__ __align__(16) float colbuf[CTA_ROW ? 4 : 2 * 1024];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  const float inv_n = 1.f / (float)cols;
  float acc_w[CHUNKS][VEC], acc_b[CHUNKS][VEC], ws[CHUNKS][VEC];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = rt.template col<VEC>(c);
    if (w && col < cols) unpack<T>(ld_cached(w + col), ws[c]);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      acc_w[c][i] = 0.f;
      acc_b[c][i] = 0.f;
      if (!w || col >= cols) ws[c][i] = 1.f;
    }
  }
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    float xs[CHUNKS][VEC], gs[CHUNKS][VEC];
    load_row<T, CHUNKS, CTA_ROW>(xs, x + row * cols, cols, rt);
    load_row<T, CHUNKS, CTA_ROW>(gs, dy + row * cols, cols, rt);
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const bool in = rt.template col<VEC>(c) < cols;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float xh = in ? (xs[c][i] - mu) * rs : 0.f;
        const float d = gs[c][i];
        acc_w[c][i] += d * xh;
        acc_b[c][i] += d;
        const float g = d * ws[c][i];
        xs[c][i] = xh;
        gs[c][i] = g;
        s1 += g * xh;
        s2 += g;
      }
    }
    const float c1 = row_reduce<CTA_ROW, false>(s1, slot, phase) * inv_n;
    const float c2 = row_reduce<CTA_ROW, false>(s2, slot, phase) * inv_n;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) xs[c][i] = rs * (gs[c][i] - xs[c][i] * c1 - c2);
    store_row<T, CHUNKS, CTA_ROW>(dx + row * cols, xs, cols, rt);
  }
  if (want_cols)
    write_col_partials<CHUNKS, VEC, CTA_ROW>(partial + (int64_t)blockIdx.x * 2 * cols, cols, acc_w,
                                             acc_b, rt, colbuf);
}

template <typename T>
__global__ void ln_bwd_dx_generic(T* dx, const T* dy, const T* x, const T* w, const float* mean,
                                  const float* rstd, int64_t rows, int64_t cols) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * cols;
  const T* gr = dy + row * cols;
  const float mu = mean[row], rs = rstd[row];
  float s1 = 0.f, s2 = 0.f;
  for (int64_t i = lane; i < cols; i += 32) {
    const float xh = (Traits<T>::to_f(xr[i]) - mu) * rs;
    const float g = Traits<T>::to_f(gr[i]) * (w ? Traits<T>::to_f(w[i]) : 1.f);
    s1 += g * xh;
    s2 += g;
  }
  const float c1 = warp_sum(s1) / (float)cols, c2 = warp_sum(s2) / (float)cols;
  for (int64_t i = lane; i < cols; i += 32) {
    const float xh = (Traits<T>::to_f(xr[i]) - mu) * rs;
    const float g = Traits<T>::to_f(gr[i]) * (w ? Traits<T>::to_f(w[i]) : 1.f);
    dx[row * cols + i] = Traits<T>::from_f(rs * (g - xh * c1 - c2));
  }
}

// One thread per column walks all rows (coalesced across the warp). `scale_kind`:
// 0 = LayerNorm (xhat = (x-mean)*rstd), 1 = RMSNorm (xhat = x/(rms+eps)).
template <typename T>
__global__ void norm_bwd_cols_generic(T* dw, T* db, const T* dy, const T* x, const float* stat_a,
                                      const float* stat_b, int64_t rows, int64_t cols,
                                      int64_t x_rs, int64_t x_cs, float eps, int scale_kind) {
  const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  float aw = 0.f, ab = 0.f;
  for (int64_t r = 0; r < rows; ++r) {
    const float d = Traits<T>::to_f(dy[r * cols + col]);
    const float xv = Traits<T>::to_f(x[r * x_rs + col * x_cs]);
    const float xh = scale_kind == 0 ? (xv - stat_a[r]) * stat_b[r] : xv / (stat_a[r] + eps);
    aw += d * xh;
    ab += d;
  }
  if (dw) dw[col] = Traits<T>::from_f(aw);
  if (db) db[col] = Traits<T>::from_f(ab);
}

// ------------------------------------------------------------------ RMSNorm fwd
// (two 512-thread CTAs per SM: the register cap roughly doubles the rows in flight)
template <typename T, int CHUNKS, bool CTA_ROW>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256, CTA_ROW ? 2 : 4)
    rms_fwd_vec(T* __restrict__ y, float* __restrict__ rms, const T* __restrict__ x,
                const T* __restrict__ w, const T* __restrict__ b, int64_t rows, int cols,
                int64_t row_stride, int partial, float eps) {
  constexpr int VEC = Traits<T>::VEC;
  __shared__ float slot[64];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  pdl_wait();     // (programmatic dependent launch: nothing is read before the previous kernel is done)
  pdl_release();  // the next kernel of the stream may be scheduled
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    constexpr bool EARLY = CHUNKS <= 4;  // as far as the registers allow
    uint4 raw[CHUNKS], wraw[EARLY ? CHUNKS : 1];
    const T* xr = x + row * row_stride;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      raw[c] = col < cols ? ld_stream(xr + col) : make_uint4(0, 0, 0, 0);
    }
    // the weight is requested before the reduction: its latency hides behind the row's own load
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      if constexpr (EARLY) wraw[c] = col < cols ? ld_cached(w + col) : make_uint4(0, 0, 0, 0);
    }
    constexpr int PAIRS = VEC / 2;  // arithmetic on fp32 pairs (two-lane instructions)
    uint64_t s2 = 0ull;
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      if (col + VEC <= partial) {
        uint64_t t[PAIRS];
        unpack2<T>(raw[c], t);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) s2 = am::fma2(t[i], t[i], s2);
      } else if (col < partial) {
        float t[VEC];
        unpack<T>(raw[c], t);
#pragma unroll
        for (int i = 0; i < VEC; ++i) s += (col + i < partial) ? t[i] * t[i] : 0.f;
      }
    }
    const float r = sqrtf(row_reduce<CTA_ROW, false>(s + hsum2(s2), slot, phase) / (float)partial);
    const float inv = 1.f / (r + eps);
    const uint64_t inv2 = splat2(inv);
    T* yr = y + row * cols;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      if (y && col < cols) {  // y == null: only the row statistic is wanted
        uint64_t t[PAIRS], ws[PAIRS], bs[PAIRS];
        unpack2<T>(raw[c], t);
        unpack2<T>(EARLY ? wraw[EARLY ? c : 0] : ld_cached(w + col), ws);
        if (b) unpack2<T>(ld_cached(b + col), bs);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
          const uint64_t o = am::mul2(t[i], am::mul2(ws[i], inv2));
          t[i] = b ? am::add2(o, bs[i]) : o;
        }
        st_stream(yr + col, pack2<T>(t));
      }
    }
    if (rt.tid == 0) rms[row] = r;
  }
}

template <typename T>
__global__ void rms_fwd_generic(T* y, float* rms, const T* x, const T* w, const T* b, int64_t rows,
                                int64_t cols, int64_t rs_, int64_t cs_, int64_t partial, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * rs_;
  float s = 0.f;
  for (int64_t i = lane; i < partial; i += 32) {
    const float v = Traits<T>::to_f(xr[i * cs_]);
    s += v * v;
  }
  const float r = sqrtf(warp_sum(s) / (float)partial);
  const float inv = 1.f / (r + eps);
  for (int64_t i = lane; y && i < cols; i += 32) {  // y == null: only the row statistic is wanted
    float o = Traits<T>::to_f(xr[i * cs_]) * inv * Traits<T>::to_f(w[i]);
    if (b) o += Traits<T>::to_f(b[i]);
    y[row * cols + i] = Traits<T>::from_f(o);
  }
  if (lane == 0) rms[row] = r;
}

// ------------------------------------------------------------------ RMSNorm bwd
template <typename T, int CHUNKS, bool CTA_ROW>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256)
    rms_bwd_vec(T* __restrict__ dx, float* __restrict__ partial_ws, const T* __restrict__ dy,
                const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ rms,
                int64_t rows, int cols, int64_t row_stride, int partial, float eps) {
  constexpr int VEC = Traits<T>::VEC;
  __shared__ float slot[64];
  __shared__ __align__(16) float colbuf[CTA_ROW ? 4 : 2 * 1024];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  float acc_w[CHUNKS][VEC], acc_b[CHUNKS][VEC], ws[CHUNKS][VEC];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = rt.template col<VEC>(c);
    if (col < cols) unpack<T>(ld_cached(w + col), ws[c]);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      acc_w[c][i] = 0.f;
      acc_b[c][i] = 0.f;
      if (col >= cols) ws[c][i] = 0.f;
    }
  }
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    float xs[CHUNKS][VEC], gs[CHUNKS][VEC];
    load_row<T, CHUNKS, CTA_ROW>(xs, x + row * row_stride, cols, rt);
    load_row<T, CHUNKS, CTA_ROW>(gs, dy + row * cols, cols, rt);
    const float r = rms[row];
    const float inv = 1.f / (r + eps);
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float d = gs[c][i];
        acc_w[c][i] += d * xs[c][i] * inv;
        acc_b[c][i] += d;
        const float g = d * ws[c][i];
        gs[c][i] = g;
        s += g * xs[c][i];
      }
    s = row_reduce<CTA_ROW, false>(s, slot, phase);
    // second term vanishes for an all-zero row (rms == 0)
    const float k = r > 0.f ? s * inv * inv / ((float)partial * r) : 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
#pragma unroll
      for (int i = 0; i < VEC; ++i)
        xs[c][i] = gs[c][i] * inv - ((col + i < partial) ? xs[c][i] * k : 0.f);
    }
    store_row<T, CHUNKS, CTA_ROW>(dx + row * cols, xs, cols, rt);
  }
  write_col_partials<CHUNKS, VEC, CTA_ROW>(partial_ws + (int64_t)blockIdx.x * 2 * cols, cols, acc_w,
                                           acc_b, rt, colbuf);
}

template <typename T>
__global__ void rms_bwd_dx_generic(T* dx, const T* dy, const T* x, const T* w, const float* rms,
                                   int64_t rows, int64_t cols, int64_t rs_, int64_t cs_,
                                   int64_t partial, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * rs_;
  const float r = rms[row];
  const float inv = 1.f / (r + eps);
  float s = 0.f;
  for (int64_t i = lane; i < cols; i += 32)
    s += Traits<T>::to_f(dy[row * cols + i]) * Traits<T>::to_f(w[i]) * Traits<T>::to_f(xr[i * cs_]);
  s = warp_sum(s);
  const float k = r > 0.f ? s * inv * inv / ((float)partial * r) : 0.f;
  for (int64_t i = lane; i < cols; i += 32) {
    const float g = Traits<T>::to_f(dy[row * cols + i]) * Traits<T>::to_f(w[i]);
    const float xv = Traits<T>::to_f(xr[i * cs_]);
    dx[row * cols + i] = Traits<T>::from_f(g * inv - (i < partial ? xv * k : 0.f));
  }
}

// ------------------------------------------------------------------ host side
static size_t col_partial_bytes(int64_t cols) {
  // one [2, cols] fp32 row per CTA of the bounded grid (at most 4 CTAs per SM)
  return (size_t)sm_count() * 4 * 2 * (size_t)cols * sizeof(float);
}

template <typename T>
static int finalize_cols(T* da, T* db, const float* partial, int nparts, int64_t cols,
                         cudaStream_t st, int sets = 2) {
  // `sets`: 2 for partial rows [2][cols] (weight, bias), 1 for [cols] (weight only)
  dim3 grid((unsigned)ceil_div(cols, 32), (unsigned)sets), block(32, 32);
  colsum_finalize_kernel<T><<<grid, block, 0, st>>>(da, db, partial, nparts, (int)cols);
  return launch_status("colsum_finalize");
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_layer_norm_fwd(void* y, float* mean, float* rstd, const void* x,
                                    const void* weight, const void* bias, int64_t rows,
                                    int64_t cols, float eps, int dtype, void* stream) {
  TB200_REQUIRE(rows >= 0 && cols > 0, TB200_ERR_INVALID, "layer_norm_fwd: bad shape %lld x %lld",
                (long long)rows, (long long)cols);
  if (rows == 0) return 0;  // (empty tensors may come with null pointers)
  TB200_REQUIRE(y && mean && rstd && x, TB200_ERR_INVALID, "layer_norm_fwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    const bool ok = aligned16(y) && aligned16(x) && (!weight || aligned16(weight)) &&
                    (!bias || aligned16(bias)) && cols < (1 << 30);
    RowPlan p = plan_rows<T>(cols, ok);
    if (p.vec) {
      const int64_t grid = ceil_div(rows, p.rows_per_cta);
      int rc = dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
        cudaError_t e = launch_pdl(ln_fwd_vec<T, decltype(c)::value, decltype(cta)::value>, dim3((unsigned)grid),
                                   dim3(p.threads), 0, st, false, (T*)y, mean, rstd, (const T*)x, (const T*)weight,
                                   (const T*)bias, rows, (int)cols, eps);
        (void)e;  // picked up by launch_status
        return launch_status("ln_fwd_vec");
      });
      if (rc == 0) note_kernel("row_vec", 1);
      return rc;
    }
    ln_fwd_generic<T><<<(unsigned)ceil_div(rows, 4), 128, 0, st>>>(
        (T*)y, mean, rstd, (const T*)x, (const T*)weight, (const T*)bias, rows, cols, eps);
    int rc = launch_status("ln_fwd_generic");
    if (rc == 0) note_kernel("row_generic", 1);
    return rc;
  });
}

extern "C" size_t tb200_layer_norm_bwd_workspace(int64_t rows, int64_t cols) {
  (void)rows;
  return cols > 0 ? col_partial_bytes(cols) : 0;
}

extern "C" int tb200_layer_norm_bwd(void* dx, void* dweight, void* dbias, const void* dy,
                                    const void* x, const void* weight, const float* mean,
                                    const float* rstd, void* workspace, size_t workspace_bytes,
                                    int64_t rows, int64_t cols, int dtype, void* stream) {
  TB200_REQUIRE(rows >= 0 && cols > 0, TB200_ERR_INVALID, "layer_norm_bwd: bad shape");
  cudaStream_t st = (cudaStream_t)stream;
  if (rows == 0) {  // sums over no rows
    if (int rc = zero_fill(dweight, (size_t)cols * dtype_size(dtype), st, "layer_norm_bwd")) return rc;
    return zero_fill(dbias, (size_t)cols * dtype_size(dtype), st, "layer_norm_bwd");
  }
  TB200_REQUIRE(dx && dy && x && mean && rstd, TB200_ERR_INVALID, "layer_norm_bwd: null pointer");
  const bool want_cols = dweight || dbias;
  {
    bool handled = false;
    int rc = try_layer_norm_bwd_grouped(dx, dweight, dbias, dy, x, weight, mean, rstd, workspace, workspace_bytes,
                                        rows, cols, dtype, st, &handled, /*allow_fused=*/true);
    if (rc || handled) return rc;
  }
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    const bool ok = aligned16(dx) && aligned16(dy) && aligned16(x) &&
                    (!weight || aligned16(weight)) && cols < (1 << 30) &&
                    (!want_cols || (workspace && aligned16(workspace)));
    RowPlan p = plan_rows<T>(cols, ok, max_chunks<T>() / 2);
    if (p.vec && rows > 0) {
      const int64_t grid = persistent_grid(p, rows);
      if (want_cols)
        TB200_REQUIRE(workspace_bytes >= (size_t)grid * 2 * cols * sizeof(float),
                      TB200_ERR_WORKSPACE, "layer_norm_bwd: workspace too small");
      int rc = dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
        ln_bwd_vec<T, decltype(c)::value, decltype(cta)::value>
            <<<(unsigned)grid, p.threads, 0, st>>>((T*)dx, (float*)workspace, (const T*)dy,
                                                   (const T*)x, (const T*)weight, mean, rstd, rows,
                                                   (int)cols, want_cols ? 1 : 0);
        return launch_status("ln_bwd_vec");
      });
      if (rc) return rc;
      if (want_cols) {
        rc = finalize_cols<T>((T*)dweight, (T*)dbias, (const float*)workspace, (int)grid, cols, st);
        if (rc) return rc;
      }
      note_kernel("row_vec", want_cols ? 2 : 1);
      return 0;
    }
    int launches = 0;
    if (rows > 0) {
      ln_bwd_dx_generic<T><<<(unsigned)ceil_div(rows, 4), 128, 0, st>>>(
          (T*)dx, (const T*)dy, (const T*)x, (const T*)weight, mean, rstd, rows, cols);
      int rc = launch_status("ln_bwd_dx_generic");
      if (rc) return rc;
      ++launches;
    }
    if (want_cols) {
      norm_bwd_cols_generic<T><<<(unsigned)ceil_div(cols, 128), 128, 0, st>>>(
          (T*)dweight, (T*)dbias, (const T*)dy, (const T*)x, mean, rstd, rows, cols, cols, 1, 0.f,
          0);
      int rc = launch_status("norm_bwd_cols_generic");
      if (rc) return rc;
      ++launches;
    }
    note_kernel("row_generic", launches);
    return 0;
  });
}

extern "C" int tb200_rms_norm_fwd(void* y, float* rms, const void* x, const void* weight,
                                  const void* bias, int64_t rows, int64_t cols, int64_t row_stride,
                                  int64_t col_stride, int64_t partial_cols, float eps, int dtype,
                                  void* stream) {
  TB200_REQUIRE(rows >= 0 && cols > 0, TB200_ERR_INVALID, "rms_norm_fwd: bad shape");
  TB200_REQUIRE(partial_cols > 0 && partial_cols <= cols, TB200_ERR_INVALID,
                "rms_norm_fwd: partial_cols %lld outside (0, %lld]", (long long)partial_cols,
                (long long)cols);
  if (rows == 0) return 0;
  TB200_REQUIRE(rms && x && weight, TB200_ERR_INVALID, "rms_norm_fwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Traits<T>::VEC;
    const bool ok = (!y || aligned16(y)) && aligned16(x) && aligned16(weight) &&
                    (!bias || aligned16(bias)) && col_stride == 1 && row_stride % VEC == 0 &&
                    row_stride >= cols && cols < (1 << 30);
    RowPlan p = plan_rows<T>(cols, ok);
    if (p.vec) {
      const int64_t grid = ceil_div(rows, p.rows_per_cta);
      int rc = dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
        cudaError_t e = launch_pdl(rms_fwd_vec<T, decltype(c)::value, decltype(cta)::value>, dim3((unsigned)grid),
                                   dim3(p.threads), 0, st, false, (T*)y, rms, (const T*)x, (const T*)weight,
                                   (const T*)bias, rows, (int)cols, row_stride, (int)partial_cols, eps);
        (void)e;  // picked up by launch_status
        return launch_status("rms_fwd_vec");
      });
      if (rc == 0) note_kernel("row_vec", 1);
      return rc;
    }
    rms_fwd_generic<T><<<(unsigned)ceil_div(rows, 4), 128, 0, st>>>(
        (T*)y, rms, (const T*)x, (const T*)weight, (const T*)bias, rows, cols, row_stride,
        col_stride, partial_cols, eps);
    int rc = launch_status("rms_fwd_generic");
    if (rc == 0) note_kernel("row_generic", 1);
    return rc;
  });
}

extern "C" size_t tb200_rms_norm_bwd_workspace(int64_t rows, int64_t cols) {
  (void)rows;
  return cols > 0 ? col_partial_bytes(cols) : 0;
}

extern "C" int tb200_rms_norm_bwd(void* dx, void* dweight, void* dbias, const void* dy,
                                  const void* x, const void* weight, const float* rms,
                                  void* workspace, size_t workspace_bytes, int64_t rows,
                                  int64_t cols, int64_t row_stride, int64_t col_stride,
                                  int64_t partial_cols, float eps, int dtype, void* stream) {
  TB200_REQUIRE(rows >= 0 && cols > 0, TB200_ERR_INVALID, "rms_norm_bwd: bad shape");
  TB200_REQUIRE(partial_cols > 0 && partial_cols <= cols, TB200_ERR_INVALID,
                "rms_norm_bwd: partial_cols outside (0, cols]");
  cudaStream_t st = (cudaStream_t)stream;
  if (rows == 0) {  // sums over no rows
    if (int rc = zero_fill(dweight, (size_t)cols * dtype_size(dtype), st, "rms_norm_bwd")) return rc;
    return zero_fill(dbias, (size_t)cols * dtype_size(dtype), st, "rms_norm_bwd");
  }
  TB200_REQUIRE(dx && dweight && dy && x && weight && rms, TB200_ERR_INVALID,
                "rms_norm_bwd: null pointer");
  {
    bool handled = false;
    int rc = try_rms_norm_bwd_grouped(dx, dweight, dbias, dy, x, weight, rms, workspace, workspace_bytes, rows,
                                      cols, row_stride, col_stride, partial_cols, eps, dtype, st, &handled);
    if (rc || handled) return rc;
  }
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Traits<T>::VEC;
    const bool ok = aligned16(dx) && aligned16(dy) && aligned16(x) && aligned16(weight) &&
                    col_stride == 1 && row_stride % VEC == 0 && row_stride >= cols &&
                    cols < (1 << 30) && workspace && aligned16(workspace);
    RowPlan p = plan_rows<T>(cols, ok, max_chunks<T>() / 2);
    if (p.vec && rows > 0) {
      const int64_t grid = persistent_grid(p, rows);
      TB200_REQUIRE(workspace_bytes >= (size_t)grid * 2 * cols * sizeof(float), TB200_ERR_WORKSPACE,
                    "rms_norm_bwd: workspace too small");
      int rc = dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
        rms_bwd_vec<T, decltype(c)::value, decltype(cta)::value>
            <<<(unsigned)grid, p.threads, 0, st>>>((T*)dx, (float*)workspace, (const T*)dy,
                                                   (const T*)x, (const T*)weight, rms, rows,
                                                   (int)cols, row_stride, (int)partial_cols, eps);
        return launch_status("rms_bwd_vec");
      });
      if (rc) return rc;
      rc = finalize_cols<T>((T*)dweight, (T*)dbias, (const float*)workspace, (int)grid, cols, st);
      if (rc) return rc;
      note_kernel("row_vec", 2);
      return 0;
    }
    int launches = 0;
    if (rows > 0) {
      rms_bwd_dx_generic<T><<<(unsigned)ceil_div(rows, 4), 128, 0, st>>>(
          (T*)dx, (const T*)dy, (const T*)x, (const T*)weight, rms, rows, cols, row_stride,
          col_stride, partial_cols, eps);
      int rc = launch_status("rms_bwd_dx_generic");
      if (rc) return rc;
      ++launches;
    }
    norm_bwd_cols_generic<T><<<(unsigned)ceil_div(cols, 128), 128, 0, st>>>(
        (T*)dweight, (T*)dbias, (const T*)dy, (const T*)x, rms, nullptr, rows, cols, row_stride,
        col_stride, eps, 1);
    int rc = launch_status("norm_bwd_cols_generic");
    if (rc) return rc;
    note_kernel("row_generic", launches + 1);
    return 0;
  });
}

// ---------------------------------------------------------------------------
// LayerNorm backward without any caller-provided or allocated scratch.
//
// The regular entry point above needs a workspace for the per-CTA column partials of the
// weight and bias gradients, which the caller sizes with a query and allocates. Some callers
// cannot do that: a server that handed every byte of device memory to its own arena at
// start-up has nothing left to allocate from, and a caller bound to a "no cudaMalloc on the
// request path" rule (cudaMalloc stalls the whole device) may not allocate at all. For them
// the partials live in the fixed array below, which every GPU that loads the library holds
// from load to exit.
// ---------------------------------------------------------------------------
#include <mutex>

namespace tb200 {

constexpr size_t LN_STATIC_SCRATCH_FLOATS = 512 * 1024;  // 2 MiB per device
constexpr int64_t LN_STATIC_MAX_COLS = 8192;             // leaves room for at least 32 partial rows

static __device__ __align__(256) float g_ln_bwd_scratch[LN_STATIC_SCRATCH_FLOATS];

// Device address of the array above on the current device. In host code the array's name is
// only a handle, not an address a kernel could use, so it is resolved once per device (with
// that device current) and remembered.
static int ln_static_scratch(float** out) {
  static std::mutex mu;
  static float* resolved[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("layer_norm_bwd_static: no current CUDA device (%s)", cudaGetErrorString(e));
    return e != cudaSuccess ? (int)e : TB200_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (resolved[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_ln_bwd_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("layer_norm_bwd_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : TB200_ERR_UNSUPPORTED;
    }
    resolved[dev] = p;
  }
  *out = resolved[dev];
  return 0;
}

}  // namespace tb200

extern "C" int tb200_layer_norm_bwd_static(void* dx, void* dweight, void* dbias, const void* dy,
                                           const void* x, const void* weight, const float* mean,
                                           const float* rstd, int64_t rows, int64_t cols, int dtype,
                                           void* stream) {
  TB200_REQUIRE(rows >= 0 && cols > 0, TB200_ERR_INVALID, "layer_norm_bwd_static: bad shape");
  TB200_REQUIRE(cols <= LN_STATIC_MAX_COLS, TB200_ERR_UNSUPPORTED,
                "layer_norm_bwd_static: %lld columns exceed the built-in scratch (at most %lld); use "
                "tb200_layer_norm_bwd with a workspace",
                (long long)cols, (long long)LN_STATIC_MAX_COLS);
  cudaStream_t st = (cudaStream_t)stream;
  if (rows == 0) {  // sums over no rows, exactly as tb200_layer_norm_bwd (data pointers may be null)
    if (int rc = zero_fill(dweight, (size_t)cols * dtype_size(dtype), st, "layer_norm_bwd_static")) return rc;
    return zero_fill(dbias, (size_t)cols * dtype_size(dtype), st, "layer_norm_bwd_static");
  }
  TB200_REQUIRE(dx && dy && x && mean && rstd, TB200_ERR_INVALID,
                "layer_norm_bwd_static: null pointer");
  const bool want_cols = dweight || dbias;
  float* scratch = nullptr;
  if (want_cols) {
    if (int rc = ln_static_scratch(&scratch)) return rc;
  }
  {
    // same kernel choice as tb200_layer_norm_bwd, with the built-in array as the workspace
    bool handled = false;
    int rc = try_layer_norm_bwd_grouped(dx, dweight, dbias, dy, x, weight, mean, rstd, scratch,
                                        LN_STATIC_SCRATCH_FLOATS * sizeof(float), rows, cols, dtype, st,
                                        &handled, /*allow_fused=*/false);
    if (rc || handled) return rc;
  }
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    const bool ok = aligned16(dx) && aligned16(dy) && aligned16(x) && (!weight || aligned16(weight));
    RowPlan p = plan_rows<T>(cols, ok, max_chunks<T>() / 2);
    if (p.vec && rows > 0) {
      int64_t grid = persistent_grid(p, rows);
      const int64_t fit = (int64_t)(LN_STATIC_SCRATCH_FLOATS / (size_t)(2 * cols));
      if (grid > fit) grid = fit;  // fewer, longer-running CTAs: one [2, cols] partial row each
      int rc = dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
        ln_bwd_vec<T, decltype(c)::value, decltype(cta)::value>
            <<<(unsigned)grid, p.threads, 0, st>>>((T*)dx, scratch, (const T*)dy, (const T*)x,
                                                   (const T*)weight, mean, rstd, rows, (int)cols,
                                                   want_cols ? 1 : 0);
        return launch_status("ln_bwd_vec (static scratch)");
      });
      if (rc) return rc;
      if (want_cols) {
        rc = finalize_cols<T>((T*)dweight, (T*)dbias, scratch, (int)grid, cols, st);
        if (rc) return rc;
      }
      note_kernel("row_vec", want_cols ? 2 : 1);
      return 0;
    }
    // widths the vector kernel does not take need no scratch at all
    int launches = 0;
    if (rows > 0) {
      ln_bwd_dx_generic<T><<<(unsigned)ceil_div(rows, 4), 128, 0, st>>>(
          (T*)dx, (const T*)dy, (const T*)x, (const T*)weight, mean, rstd, rows, cols);
      int rc = launch_status("ln_bwd_dx_generic");
      if (rc) return rc;
      ++launches;
    }
    if (want_cols) {
      norm_bwd_cols_generic<T><<<(unsigned)ceil_div(cols, 128), 128, 0, st>>>(
          (T*)dweight, (T*)dbias, (const T*)dy, (const T*)x, mean, rstd, rows, cols, cols, 1, 0.f,
          0);
      int rc = launch_status("norm_bwd_cols_generic");
      if (rc) return rc;
      ++launches;
    }
    note_kernel("row_generic", launches);
    return 0;
  });
}

// ---------------------------------------------------------------------------
// Grouped backward kernel for LayerNorm and RMSNorm (rows of up to 1024 vectors).
//
// A 512-thread CTA is split into 512/TPR groups of TPR threads; every group owns one row at
// a time, so a CTA keeps 512/TPR rows (x and dy) in flight and two CTAs fit on an SM. The grid
// is bounded by twice the SM count, which bounds the fp32 [2, cols] partial rows of the
// weight/bias gradients (one per CTA, folded over the CTA's groups in shared memory in a fixed
// order). Each thread holds at most two 16-byte vectors per tensor, which keeps the register
// footprint small enough for that occupancy.
// ---------------------------------------------------------------------------
namespace tb200 {

template <int TPR>
__device__ inline void group_barrier(int group) {
  if constexpr (TPR > 32) asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(TPR) : "memory");
}

// Sums NV (1 or 2) values over the TPR threads of a group. `slots` holds [2 phases][16 warps][2];
// the per-warp sums are read back with 16-byte loads.
template <int TPR, int NV>
__device__ inline void group_sum(float& a, float& b, float* slots, int& phase, int group) {
  a = warp_sum(a);
  if constexpr (NV == 2) b = warp_sum(b);
  if constexpr (TPR > 32) {
    constexpr int WPG = TPR / 32;  // warps per group: 2, 4, 8 or 16
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* s = slots + phase * 32;
    phase ^= 1;
    if constexpr (NV == 2) {
      if (lane == 0) *reinterpret_cast<float2*>(s + warp * 2) = make_float2(a, b);
      group_barrier<TPR>(group);
      const float4* v = reinterpret_cast<const float4*>(s + group * WPG * 2);
      float ra = 0.f, rb = 0.f;
#pragma unroll
      for (int w = 0; w < WPG / 2; ++w) {
        const float4 t = v[w];
        ra += t.x + t.z;
        rb += t.y + t.w;
      }
      a = ra;
      b = rb;
    } else {
      if (lane == 0) s[warp] = a;
      group_barrier<TPR>(group);
      float ra = 0.f;
      if constexpr (WPG >= 4) {
        const float4* v = reinterpret_cast<const float4*>(s + group * WPG);
#pragma unroll
        for (int w = 0; w < WPG / 4; ++w) {
          const float4 t = v[w];
          ra += (t.x + t.y) + (t.z + t.w);
        }
      } else {
        const float2 t = *reinterpret_cast<const float2*>(s + group * WPG);
        ra = t.x + t.y;
      }
      a = ra;
    }
  }
}

// DEPTH rows are in flight per group: a group requests the rows up to DEPTH-1 iterations
// ahead before it works on the current one (a ring of register buffers, the loop unrolled over
// the ring so that no register is copied).
template <typename T, int CHUNKS, int TPR, bool RMS, bool WANT_B, int DEPTH, int MINB>
__global__ void __launch_bounds__(512, MINB)
    norm_bwd_grouped(T* __restrict__ dx, float* __restrict__ partial, const T* __restrict__ dy,
                     const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ stat_a,
                     const float* __restrict__ stat_b, int64_t rows, int cols, int64_t x_row_stride,
                     int partial_cols, float eps, int want_cols, T* __restrict__ dw_out,
                     T* __restrict__ db_out, int fused_slab) {
  constexpr int VEC = Traits<T>::VEC;
  constexpr int GROUPS = 512 / TPR;
  extern __shared__ __align__(16) float colbuf[];  // [2][cols], used after the row loop
  __shared__ __align__(16) float slots[64];
  int phase = 0;
  const int group = threadIdx.x / TPR, tid = threadIdx.x % TPR;
  const float inv_n = 1.f / (float)cols;
  // A row (x and dy) stays packed in registers as loaded and is unpacked once per pass. A
  // thread always works on the same columns, so with one vector per thread its weights are
  // loaded once, packed; with two they are re-read per pass (L1 hits).
  constexpr bool W_REGS = CHUNKS == 1 || MINB == 1;
  constexpr int PAIRS = VEC / 2;  // arithmetic runs on fp32 pairs (two-lane instructions)
  pdl_wait();     // (programmatic dependent launch: nothing is read before the previous kernel is done)
  pdl_release();  // the next kernel of the stream may be scheduled
  uint64_t acc_w[CHUNKS][PAIRS], acc_b[WANT_B ? CHUNKS : 1][PAIRS];
  uint4 wreg[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * TPR + tid) * VEC;
    wreg[c] = (W_REGS && w && col < cols) ? ld_cached(w + col) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < PAIRS; ++i) {
      acc_w[c][i] = 0ull;
      if constexpr (WANT_B) acc_b[c][i] = 0ull;
    }
  }
  const bool has_w = w != nullptr;
  auto get_w = [&](uint64_t (&dst)[PAIRS], int c) {
    const int col = (c * TPR + tid) * VEC;
    if (has_w && (W_REGS || col < cols)) {
      // out-of-range columns: zeros, and dy is zero there as well
      unpack2<T>(W_REGS ? wreg[c] : ld_cached(w + col), dst);
    } else {
#pragma unroll
      for (int i = 0; i < PAIRS; ++i) dst[i] = splat2(1.f);
    }
  };
  struct RowRegs {
    uint4 x[CHUNKS], g[CHUNKS];
    float sa, sb;
  };
  // Rows are taken last to first: when this kernel follows the forward pass directly, the rows
  // the forward touched last are the ones still in L2 (measured: bf16 [8192, 4096] forward +
  // backward 65.0 -> 63.7 us).
  auto request = [&](RowRegs& r, int64_t row) {
    if (row < rows) {
      row = rows - 1 - row;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = (c * TPR + tid) * VEC;
        if (col < cols) {
          r.x[c] = ld_stream(x + row * x_row_stride + col);
          r.g[c] = ld_stream(dy + row * cols + col);
        } else {
          r.x[c] = make_uint4(0, 0, 0, 0);
          r.g[c] = make_uint4(0, 0, 0, 0);
        }
      }
      r.sa = __ldg(stat_a + row);
      r.sb = RMS ? 0.f : __ldg(stat_b + row);
    }
  };
  auto process = [&](const RowRegs& r, int64_t row) {
    row = rows - 1 - row;
    const float sa = r.sa, sb = r.sb;
    if constexpr (!RMS) {
      // LayerNorm: sa = mean, sb = rstd; xh = (x - mean) * rstd.
      // Out-of-range columns hold x = dy = 0: their xh is finite and every product with dy is 0.
      const uint64_t nsa2 = splat2(-sa), sb2 = splat2(sb);
      uint64_t s1 = 0ull, s2 = 0ull;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        uint64_t xs[PAIRS], gs[PAIRS], wv[PAIRS];
        unpack2<T>(r.x[c], xs);
        unpack2<T>(r.g[c], gs);
        get_w(wv, c);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
          const uint64_t xh = am::mul2(am::add2(xs[i], nsa2), sb2);
          acc_w[c][i] = am::fma2(gs[i], xh, acc_w[c][i]);
          if constexpr (WANT_B) acc_b[c][i] = am::add2(acc_b[c][i], gs[i]);
          const uint64_t g = am::mul2(gs[i], wv[i]);
          s1 = am::fma2(g, xh, s1);
          s2 = am::add2(s2, g);
        }
      }
      float t1 = hsum2(s1), t2 = hsum2(s2);
      group_sum<TPR, 2>(t1, t2, slots, phase, group);
      // dx = rstd * (g - xh * c1 - c2) with g = dy * w, c1 = mean(g * xh), c2 = mean(g)
      const uint64_t k1 = splat2(-sb * t1 * inv_n), k2 = splat2(-sb * t2 * inv_n);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = (c * TPR + tid) * VEC;
        uint64_t xs[PAIRS], gs[PAIRS], wv[PAIRS];
        unpack2<T>(r.x[c], xs);
        unpack2<T>(r.g[c], gs);
        get_w(wv, c);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
          const uint64_t xh = am::mul2(am::add2(xs[i], nsa2), sb2);
          xs[i] = am::fma2(am::mul2(gs[i], wv[i]), sb2, am::fma2(xh, k1, k2));
        }
        if (col < cols) st_stream(dx + row * cols + col, pack2<T>(xs));
      }
    } else {
      // RMSNorm: sa = rms
      const float inv = 1.f / (sa + eps);
      const uint64_t inv2 = splat2(inv);
      uint64_t s = 0ull;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        uint64_t xs[PAIRS], gs[PAIRS], wv[PAIRS];
        unpack2<T>(r.x[c], xs);
        unpack2<T>(r.g[c], gs);
        get_w(wv, c);
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
          const uint64_t t = am::mul2(gs[i], xs[i]);
          acc_w[c][i] = am::fma2(t, inv2, acc_w[c][i]);
          if constexpr (WANT_B) acc_b[c][i] = am::add2(acc_b[c][i], gs[i]);
          s = am::fma2(t, wv[i], s);
        }
      }
      float t1 = hsum2(s), unused = 0.f;
      group_sum<TPR, 1>(t1, unused, slots, phase, group);
      const float k = sa > 0.f ? t1 * inv * inv / ((float)partial_cols * sa) : 0.f;
      const uint64_t nk2 = splat2(-k);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = (c * TPR + tid) * VEC;
        uint64_t xs[PAIRS], gs[PAIRS], wv[PAIRS];
        unpack2<T>(r.x[c], xs);
        unpack2<T>(r.g[c], gs);
        get_w(wv, c);
        if (col + VEC <= partial_cols) {
#pragma unroll
          for (int i = 0; i < PAIRS; ++i)
            xs[i] = am::fma2(gs[i], am::mul2(wv[i], inv2), am::mul2(xs[i], nk2));
        } else {
#pragma unroll
          for (int i = 0; i < PAIRS; ++i) {
            float x0, x1;
            am::unpack2f(xs[i], x0, x1);
            const uint64_t xk = am::pack2f(col + 2 * i < partial_cols ? -k * x0 : 0.f,
                                           col + 2 * i + 1 < partial_cols ? -k * x1 : 0.f);
            xs[i] = am::fma2(gs[i], am::mul2(wv[i], inv2), xk);
          }
        }
        if (col < cols) st_stream(dx + row * cols + col, pack2<T>(xs));
      }
    }
  };
  // Each group walks its own rows (the group barrier only involves the group's threads, and
  // the trip count is uniform within a group).
  const int64_t row_step = (int64_t)gridDim.x * GROUPS;
  int64_t row = (int64_t)blockIdx.x * GROUPS + group;
  RowRegs ring[DEPTH];
#pragma unroll
  for (int d = 0; d + 1 < DEPTH; ++d) request(ring[d], row + d * row_step);
  while (row < rows) {
#pragma unroll
    for (int k = 0; k < DEPTH; ++k) {
      if (row < rows) {
        request(ring[(k + DEPTH - 1) % DEPTH], row + (DEPTH - 1) * row_step);
        process(ring[k], row);
        row += row_step;
      }
    }
  }
  // partial rows are [2][cols] (weight, bias), or [cols] when no bias gradient is kept
  constexpr int NSETS = WANT_B ? 2 : 1;
  if (want_cols) {
    // fold the groups of this CTA in a fixed order, then write its partial row
    for (int g = 0; g < GROUPS; ++g) {
      if (group == g) {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const int col = (c * TPR + tid) * VEC;
          if (col < cols) {
            // 16-byte shared-memory accesses (col is a multiple of VEC, VEC of 4)
            float vw[VEC], vb[VEC];
#pragma unroll
            for (int i = 0; i < VEC; i += 2) {
              am::unpack2f(acc_w[c][i >> 1], vw[i], vw[i + 1]);
              if constexpr (WANT_B) am::unpack2f(acc_b[c][i >> 1], vb[i], vb[i + 1]);
            }
#pragma unroll
            for (int i = 0; i < VEC; i += 4) {
              float4* pw4 = reinterpret_cast<float4*>(colbuf + col + i);
              float4 a = make_float4(vw[i], vw[i + 1], vw[i + 2], vw[i + 3]);
              if (g != 0) {
                const float4 o = *pw4;
                a = make_float4(o.x + a.x, o.y + a.y, o.z + a.z, o.w + a.w);
              }
              *pw4 = a;
              if constexpr (WANT_B) {
                float4* pb4 = reinterpret_cast<float4*>(colbuf + cols + col + i);
                float4 b4 = make_float4(vb[i], vb[i + 1], vb[i + 2], vb[i + 3]);
                if (g != 0) {
                  const float4 o = *pb4;
                  b4 = make_float4(o.x + b4.x, o.y + b4.y, o.z + b4.z, o.w + b4.w);
                }
                *pb4 = b4;
              }
            }
          }
        }
      }
      __syncthreads();
    }
    float* out = partial + (int64_t)blockIdx.x * NSETS * cols;
    for (int i = threadIdx.x * 4; i < NSETS * cols; i += 512 * 4)
      *reinterpret_cast<float4*>(out + i) = *reinterpret_cast<const float4*>(colbuf + i);
  }
  if (fused_slab > 0) {
    // Cooperative launch: after a grid-wide barrier the CTAs share the column sums of the
    // partial rows among themselves, `fused_slab` adjacent columns of the flattened [2][cols]
    // row per CTA and step, 512 / fused_slab threads walking the partial rows of each column.
    // The summation order is fixed, so the result does not depend on scheduling.
    cooperative_groups::this_grid().sync();
    __shared__ float red[512];
    const int nparts = gridDim.x;
    const int lanes = 512 / fused_slab;
    const int cl = threadIdx.x % fused_slab, j = threadIdx.x / fused_slab;
    const int limit = (WANT_B && db_out) ? 2 * cols : cols;
    for (int base = blockIdx.x * fused_slab; base < limit; base += gridDim.x * fused_slab) {
      const int cc = base + cl;
      float acc = 0.f;
      if (cc < limit) {
        // sixteen independent loads per trip: one round trip to L2 covers up to 16 * lanes partial rows
        for (int p0 = j; p0 < nparts; p0 += lanes * 16) {
          float v[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const int p = p0 + lanes * u;
            v[u] = p < nparts ? __ldcg(partial + (int64_t)p * NSETS * cols + cc) : 0.f;
          }
#pragma unroll
          for (int u = 0; u < 16; ++u) acc += v[u];
        }
      }
      red[j * fused_slab + cl] = acc;
      __syncthreads();
      if (threadIdx.x < fused_slab && cc < limit) {
        float sum = 0.f;
        for (int jj = 0; jj < lanes; ++jj) sum += red[jj * fused_slab + cl];
        T* o = cc < cols ? dw_out : db_out;
        if (o) o[cc < cols ? cc : cc - cols] = Traits<T>::from_f(sum);
      }
      __syncthreads();
    }
  }
}

struct GroupedPlan {
  bool ok = false;
  int tpr = 32, chunks = 1, depth = 1, minb = 2;
};

// Plan of the grouped kernel, from measurements on bf16 [8192, 4096] and fp32 [4096, 1024]:
// rows of up to 256 vectors put one vector on a thread, two CTAs per SM (64 registers) and
// request one row ahead (none for 16-bit rows with a bias gradient, whose second set of
// accumulators leaves no registers for it); wider rows put two vectors on a thread, one CTA
// per SM (128 registers), one row ahead. Fat threads matter because the kernel is close to
// issue-bound: the per-row overhead (addresses, shuffles, barrier) is paid per thread.
template <typename T>
static GroupedPlan plan_grouped(int64_t cols, bool ptrs_ok, bool want_b) {
  GroupedPlan p;
  constexpr int VEC = Traits<T>::VEC;
  if (!ptrs_ok || cols <= 0 || cols % VEC != 0) return p;
  const int64_t vecs = cols / VEC;
  if (vecs > 1024) return p;
  p.ok = true;
  if (vecs <= 256) {
    p.tpr = vecs <= 32 ? 32 : vecs <= 128 ? 128 : 256;
    p.chunks = 1;
    p.depth = (sizeof(T) == 2 && want_b) ? 1 : 2;
    p.minb = 2;
  } else {
    p.tpr = vecs <= 512 ? 256 : 512;
    p.chunks = 2;
    p.depth = 2;
    p.minb = 1;
  }
  return p;
}

// Test hook of the calling thread (see tb200_set_norm_fused_finalize): thread-local, so one
// thread's setting never changes another thread's dispatch.
static thread_local int g_norm_fused_finalize = 1;

// Launches the grouped kernel; returns the number of partial rows written (the grid size) in
// *nparts. `grid_cap` bounds the grid (the workspace of the caller must hold that many rows).
// With `fuse` the launch is cooperative and the kernel also folds the partial rows into
// dw_out/db_out after a grid barrier; *fused reports whether that happened (when the grid
// cannot be co-resident the plain launch is used and the caller runs the finalize kernel).
template <typename T, bool RMS, bool WANT_B>
static int launch_grouped(const GroupedPlan& gp, T* dx, float* partial, const T* dy, const T* x, const T* w,
                          const float* stat_a, const float* stat_b, int64_t rows, int64_t cols,
                          int64_t x_row_stride, int64_t partial_cols, float eps, bool want_cols,
                          int64_t grid_cap, int* nparts, cudaStream_t st, bool fuse = false, T* dw_out = nullptr,
                          T* db_out = nullptr, bool* fused = nullptr) {
  const int groups = 512 / gp.tpr;
  int64_t grid = ceil_div(rows, groups);
  if (grid > grid_cap) grid = grid_cap;
  if (grid < 1) grid = 1;
  *nparts = (int)grid;
  if (fused) *fused = false;
  const size_t smem = want_cols ? (size_t)2 * cols * sizeof(float) : 0;
  auto go = [&](auto kern) -> int {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) {
        set_error("norm_bwd_grouped: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
        return (int)e;
      }
    }
    int cols_i = (int)cols, pc_i = (int)partial_cols, wc_i = want_cols ? 1 : 0, slab = 0;
    if (fuse && want_cols && g_norm_fused_finalize) {
      // The occupancy of a kernel at a block size depends on the kernel, the shared-memory size
      // and the device: the last answer is cached under all three (this lambda is shared by every
      // instantiation with the same pointer type, so the kernel is part of the key).
      static thread_local const void* cached_kern = nullptr;
      static thread_local size_t cached_smem = ~size_t(0);
      static thread_local int cached_dev = -1;
      static thread_local int cached_per_sm = 0;
      int dev = -1;
      if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        dev = -1;
      }
      if (cached_kern != (const void*)kern || cached_smem != smem || cached_dev != dev || dev < 0) {
        int q = 0;
        cached_per_sm = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kern, 512, smem) == cudaSuccess ? q : 0;
        cached_kern = (const void*)kern;
        cached_smem = smem;
        cached_dev = dev;
      }
      const int per_sm = cached_per_sm;
      if ((int64_t)per_sm * sm_count() >= grid) {
        const int64_t limit = db_out ? 2 * cols : cols;
        slab = 16;
        while (slab < 64 && ceil_div(limit, slab) > grid) slab *= 2;
      }
    }
    if (slab > 0) {
      // cooperative, and allowed to be scheduled during the tail of the previous kernel
      cudaError_t e = launch_pdl(kern, dim3((unsigned)grid), dim3(512), smem, st, true, dx, partial, dy, x, w, stat_a,
                                 stat_b, rows, cols_i, x_row_stride, pc_i, eps, wc_i, dw_out, db_out, slab);
      if (e != cudaSuccess) {  // the combination of attributes is refused: cooperative alone
        (void)cudaGetLastError();
        void* args[] = {&dx, &partial, &dy, &x, &w, &stat_a, &stat_b, &rows, &cols_i, &x_row_stride,
                        &pc_i, &eps, &wc_i, &dw_out, &db_out, &slab};
        e = cudaLaunchCooperativeKernel((const void*)kern, dim3((unsigned)grid), dim3(512), args, smem, st);
      }
      if (e == cudaSuccess) {
        if (fused) *fused = true;
        return launch_status("norm_bwd_grouped");
      }
      (void)cudaGetLastError();  // fall through to the plain launch
      slab = 0;
    }
    cudaError_t e = launch_pdl(kern, dim3((unsigned)grid), dim3(512), smem, st, false, dx, partial, dy, x, w, stat_a,
                               stat_b, rows, cols_i, x_row_stride, pc_i, eps, wc_i, (T*)nullptr, (T*)nullptr, 0);
    (void)e;  // picked up by launch_status
    return launch_status("norm_bwd_grouped");
  };
#define TB200_GROUPED_CASE(C, R, D, M)                                                      \
  if (gp.chunks == C && gp.tpr == R && gp.depth == D && gp.minb == M)                       \
    return go(norm_bwd_grouped<T, C, R, RMS, WANT_B, D, M>);
  if constexpr (sizeof(T) == 2 && WANT_B) {
    TB200_GROUPED_CASE(1, 32, 1, 2)
    TB200_GROUPED_CASE(1, 128, 1, 2)
    TB200_GROUPED_CASE(1, 256, 1, 2)
  } else {
    TB200_GROUPED_CASE(1, 32, 2, 2)
    TB200_GROUPED_CASE(1, 128, 2, 2)
    TB200_GROUPED_CASE(1, 256, 2, 2)
  }
  TB200_GROUPED_CASE(2, 256, 2, 1)
  TB200_GROUPED_CASE(2, 512, 2, 1)
#undef TB200_GROUPED_CASE
  set_error("internal: bad grouped plan");
  return TB200_ERR_INVALID;
}

int try_layer_norm_bwd_grouped(void* dx, void* dweight, void* dbias, const void* dy, const void* x,
                               const void* weight, const float* mean, const float* rstd, void* workspace,
                               size_t workspace_bytes, int64_t rows, int64_t cols, int dtype, cudaStream_t st,
                               bool* handled, bool allow_fused) {
  *handled = false;
  const bool want_cols = dweight || dbias;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    const bool ok = aligned16(dx) && aligned16(dy) && aligned16(x) && (!weight || aligned16(weight)) &&
                    (!want_cols || (workspace && aligned16(workspace))) && rows > 0;
    GroupedPlan gp = plan_grouped<T>(cols, ok, true);
    if (!gp.ok) return 0;
    int64_t cap = (int64_t)sm_count() * gp.minb;
    if (want_cols) {
      const int64_t fit = (int64_t)(workspace_bytes / ((size_t)2 * cols * sizeof(float)));
      if (fit < 1) return 0;
      if (cap > fit) cap = fit;
    }
    int nparts = 0;
    bool fused = false;
    int rc = launch_grouped<T, false, true>(gp, (T*)dx, (float*)workspace, (const T*)dy, (const T*)x, (const T*)weight,
                                      mean, rstd, rows, cols, cols, cols, 0.f, want_cols, cap, &nparts, st,
                                      allow_fused, (T*)dweight, (T*)dbias, &fused);
    if (rc) return rc;
    if (want_cols && !fused) {
      rc = finalize_cols<T>((T*)dweight, (T*)dbias, (const float*)workspace, nparts, cols, st);
      if (rc) return rc;
    }
    note_kernel("row_vec", want_cols && !fused ? 2 : 1);
    *handled = true;
    return 0;
  });
}

int try_rms_norm_bwd_grouped(void* dx, void* dweight, void* dbias, const void* dy, const void* x,
                             const void* weight, const float* rms, void* workspace, size_t workspace_bytes,
                             int64_t rows, int64_t cols, int64_t row_stride, int64_t col_stride,
                             int64_t partial_cols, float eps, int dtype, cudaStream_t st, bool* handled) {
  *handled = false;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Traits<T>::VEC;
    const bool ok = aligned16(dx) && aligned16(dy) && aligned16(x) && aligned16(weight) && col_stride == 1 &&
                    row_stride % VEC == 0 && row_stride >= cols && workspace && aligned16(workspace) && rows > 0;
    GroupedPlan gp = plan_grouped<T>(cols, ok, dbias != nullptr);
    if (!gp.ok) return 0;
    int64_t cap = (int64_t)sm_count() * gp.minb;
    const int64_t fit = (int64_t)(workspace_bytes / ((size_t)2 * cols * sizeof(float)));
    if (fit < 1) return 0;
    if (cap > fit) cap = fit;
    int nparts = 0;
    bool fused = false;
    int rc = dbias ? launch_grouped<T, true, true>(gp, (T*)dx, (float*)workspace, (const T*)dy, (const T*)x,
                                                   (const T*)weight, rms, nullptr, rows, cols, row_stride,
                                                   partial_cols, eps, true, cap, &nparts, st, true, (T*)dweight,
                                                   (T*)dbias, &fused)
                   : launch_grouped<T, true, false>(gp, (T*)dx, (float*)workspace, (const T*)dy, (const T*)x,
                                                    (const T*)weight, rms, nullptr, rows, cols, row_stride,
                                                    partial_cols, eps, true, cap, &nparts, st, true, (T*)dweight,
                                                    (T*)dbias, &fused);
    if (rc) return rc;
    if (!fused) {
      rc = finalize_cols<T>((T*)dweight, (T*)dbias, (const float*)workspace, nparts, cols, st, dbias ? 2 : 1);
      if (rc) return rc;
    }
    note_kernel("row_vec", fused ? 1 : 2);
    *handled = true;
    return 0;
  });
}

}  // namespace tb200

extern "C" int tb200_set_norm_fused_finalize(int on) {
  const int old = tb200::g_norm_fused_finalize;
  tb200::g_norm_fused_finalize = on;
  return old;
}
