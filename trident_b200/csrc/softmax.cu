// Softmax and MaskedSoftmax, forward and backward, as single-pass HBM-bound row kernels.
//
//   fwd: z = mask ? -inf : x; m = max(z); y = exp(z-m) / sum(exp(z-m))
//   bwd: delta = sum(dy*y); dx = y*(dy - delta)          (same for the masked variant)
// (restates trident/kernel/softmax.py:64-106,160-178,223-238 and
//  trident/kernel/masked_softmax.py:64-81; the reference's separate backward_delta and
//  backward launches are one kernel here, and the forward reads x once.)
//
// Algorithmic HBM bytes per element: forward 2*e (+1 for the byte mask), backward 3*e.
#include "row_common.cuh"

namespace tb200 {

template <typename T, int CHUNKS, bool CTA_ROW, bool MASKED>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256)
    softmax_fwd_vec(T* __restrict__ y, const T* __restrict__ x, const uint8_t* __restrict__ mask,
                    int64_t rows, int cols, int64_t row_stride, int64_t mask_row_stride) {
  constexpr int VEC = Traits<T>::VEC;
  __shared__ float slot[64];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  pdl_wait();     // (programmatic dependent launch: nothing is read before the previous kernel is done)
  pdl_release();  // the next kernel of the stream may be scheduled
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    float xs[CHUNKS][VEC];
    load_row<T, CHUNKS, CTA_ROW>(xs, x + row * row_stride, cols, rt, -INFINITY);
    if constexpr (MASKED) {
      const uint8_t* mr = mask + row * mask_row_stride;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = rt.template col<VEC>(c);
        if (col < cols) {
          // VEC mask bytes: one 4- or 8-byte load
          uint32_t mw[VEC / 4];
          if constexpr (VEC == 8) {
            const uint2 t = __ldg(reinterpret_cast<const uint2*>(mr + col));
            mw[0] = t.x;
            mw[1] = t.y;
          } else {
            mw[0] = __ldg(reinterpret_cast<const uint32_t*>(mr + col));
          }
#pragma unroll
          for (int i = 0; i < VEC; ++i)
            if ((mw[i >> 2] >> (8 * (i & 3))) & 0xffu) xs[c][i] = -INFINITY;
        }
      }
    }
    float m = -INFINITY;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) m = fmaxf(m, xs[c][i]);
    m = row_reduce<CTA_ROW, true>(m, slot, phase);
    // a fully masked row has m = -inf: (x - m) would be NaN, as in the eager oracle
    float s = 0.f;
    constexpr float LOG2E = 1.4426950408889634f;
    const float mb = m * LOG2E;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float e = exp2f(fmaf(xs[c][i], LOG2E, -mb));
        xs[c][i] = e;
        s += e;
      }
    s = row_reduce<CTA_ROW, false>(s, slot, phase);
    const float inv = 1.f / s;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) xs[c][i] *= inv;
    store_row<T, CHUNKS, CTA_ROW>(y + row * row_stride, xs, cols, rt);
  }
}

template <typename T>
__global__ void softmax_fwd_generic(T* y, const T* x, const uint8_t* mask, int64_t rows,
                                    int64_t cols, int64_t rs_, int64_t cs_, int64_t mrs,
                                    int64_t mcs) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * rs_;
  const uint8_t* mr = mask ? mask + row * mrs : nullptr;
  float m = -INFINITY;
  for (int64_t i = lane; i < cols; i += 32) {
    const float v = (mr && mr[i * mcs]) ? -INFINITY : Traits<T>::to_f(xr[i * cs_]);
    m = fmaxf(m, v);
  }
  m = warp_max(m);
  float s = 0.f;
  for (int64_t i = lane; i < cols; i += 32) {
    const float v = (mr && mr[i * mcs]) ? -INFINITY : Traits<T>::to_f(xr[i * cs_]);
    s += expf(v - m);
  }
  s = warp_sum(s);
  const float inv = 1.f / s;
  T* yr = y + row * rs_;
  for (int64_t i = lane; i < cols; i += 32) {
    const float v = (mr && mr[i * mcs]) ? -INFINITY : Traits<T>::to_f(xr[i * cs_]);
    yr[i * cs_] = Traits<T>::from_f(expf(v - m) * inv);
  }
}

template <typename T, int CHUNKS, bool CTA_ROW>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256)
    softmax_bwd_vec(T* __restrict__ dx, const T* __restrict__ dy, const T* __restrict__ y,
                    int64_t rows, int cols, int64_t row_stride) {
  constexpr int VEC = Traits<T>::VEC;
  __shared__ float slot[64];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  pdl_wait();     // (programmatic dependent launch: nothing is read before the previous kernel is done)
  pdl_release();  // the next kernel of the stream may be scheduled
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    float ys[CHUNKS][VEC], gs[CHUNKS][VEC];
    load_row<T, CHUNKS, CTA_ROW>(ys, y + row * row_stride, cols, rt);
    load_row<T, CHUNKS, CTA_ROW>(gs, dy + row * row_stride, cols, rt);
    float d = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) d = fmaf(ys[c][i], gs[c][i], d);
    d = row_reduce<CTA_ROW, false>(d, slot, phase);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int i = 0; i < VEC; ++i) ys[c][i] = ys[c][i] * (gs[c][i] - d);
    store_row<T, CHUNKS, CTA_ROW>(dx + row * row_stride, ys, cols, rt);
  }
}

template <typename T>
__global__ void softmax_bwd_generic(T* dx, const T* dy, const T* y, int64_t rows, int64_t cols,
                                    int64_t rs_, int64_t cs_) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t base = row * rs_;
  float d = 0.f;
  for (int64_t i = lane; i < cols; i += 32)
    d += Traits<T>::to_f(y[base + i * cs_]) * Traits<T>::to_f(dy[base + i * cs_]);
  d = warp_sum(d);
  for (int64_t i = lane; i < cols; i += 32) {
    const float yv = Traits<T>::to_f(y[base + i * cs_]);
    dx[base + i * cs_] = Traits<T>::from_f(yv * (Traits<T>::to_f(dy[base + i * cs_]) - d));
  }
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_softmax_fwd(void* y, const void* x, const uint8_t* mask, int64_t rows,
                                 int64_t cols, int64_t row_stride, int64_t col_stride,
                                 int64_t mask_row_stride, int64_t mask_col_stride, int dtype,
                                 void* stream) {
  TB200_REQUIRE(rows >= 0 && cols > 0, TB200_ERR_INVALID, "softmax_fwd: bad shape");
  if (rows == 0) return 0;
  TB200_REQUIRE(y && x, TB200_ERR_INVALID, "softmax_fwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Traits<T>::VEC;
    bool ok = aligned16(y) && aligned16(x) && col_stride == 1 && row_stride % VEC == 0 &&
              row_stride >= cols && cols < (1 << 30);
    if (mask)
      ok = ok && mask_col_stride == 1 && mask_row_stride % VEC == 0 &&
           (reinterpret_cast<uintptr_t>(mask) % VEC) == 0;
    RowPlan p = plan_rows<T>(cols, ok);
    if (p.vec) {
      const int64_t grid = ceil_div(rows, p.rows_per_cta);
      int rc = dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
        constexpr int C = decltype(c)::value;
        constexpr bool R = decltype(cta)::value;
        cudaError_t e;
        if (mask)
          e = launch_pdl(softmax_fwd_vec<T, C, R, true>, dim3((unsigned)grid), dim3(p.threads), 0, st, false, (T*)y,
                         (const T*)x, mask, rows, (int)cols, row_stride, mask_row_stride);
        else
          e = launch_pdl(softmax_fwd_vec<T, C, R, false>, dim3((unsigned)grid), dim3(p.threads), 0, st, false, (T*)y,
                         (const T*)x, (const uint8_t*)nullptr, rows, (int)cols, row_stride, (int64_t)0);
        (void)e;  // picked up by launch_status
        return launch_status("softmax_fwd_vec");
      });
      if (rc == 0) note_kernel("row_vec", 1);
      return rc;
    }
    softmax_fwd_generic<T><<<(unsigned)ceil_div(rows, 4), 128, 0, st>>>(
        (T*)y, (const T*)x, mask, rows, cols, row_stride, col_stride, mask_row_stride,
        mask_col_stride);
    int rc = launch_status("softmax_fwd_generic");
    if (rc == 0) note_kernel("row_generic", 1);
    return rc;
  });
}

extern "C" int tb200_softmax_bwd(void* dx, const void* dy, const void* y, int64_t rows,
                                 int64_t cols, int64_t row_stride, int64_t col_stride, int dtype,
                                 void* stream) {
  TB200_REQUIRE(rows >= 0 && cols > 0, TB200_ERR_INVALID, "softmax_bwd: bad shape");
  if (rows == 0) return 0;
  TB200_REQUIRE(dx && dy && y, TB200_ERR_INVALID, "softmax_bwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Traits<T>::VEC;
    const bool ok = aligned16(dx) && aligned16(dy) && aligned16(y) && col_stride == 1 &&
                    row_stride % VEC == 0 && row_stride >= cols && cols < (1 << 30);
    RowPlan p = plan_rows<T>(cols, ok);
    if (p.vec) {
      const int64_t grid = ceil_div(rows, p.rows_per_cta);
      int rc = dispatch_plan<T>(p, [&](auto c, auto cta) -> int {
        cudaError_t e = launch_pdl(softmax_bwd_vec<T, decltype(c)::value, decltype(cta)::value>, dim3((unsigned)grid),
                                   dim3(p.threads), 0, st, false, (T*)dx, (const T*)dy, (const T*)y, rows, (int)cols,
                                   row_stride);
        (void)e;  // picked up by launch_status
        return launch_status("softmax_bwd_vec");
      });
      if (rc == 0) note_kernel("row_vec", 1);
      return rc;
    }
    softmax_bwd_generic<T><<<(unsigned)ceil_div(rows, 4), 128, 0, st>>>(
        (T*)dx, (const T*)dy, (const T*)y, rows, cols, row_stride, col_stride);
    int rc = launch_status("softmax_bwd_generic");
    if (rc == 0) note_kernel("row_generic", 1);
    return rc;
  });
}
