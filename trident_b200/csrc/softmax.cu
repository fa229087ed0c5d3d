// Softmax and MaskedSoftmax, forward and backward, as single-pass HBM-bound row kernels.
//
//   fwd: z = mask ? -inf : x; m = max(z); y = exp(z-m) / sum(exp(z-m))
//   bwd: delta = sum(dy*y); dx = y*(dy - delta)          (same for the masked variant)
// (restates trident/kernel/softmax.py:64-106,160-178,223-238 and
//  trident/kernel/masked_softmax.py:64-81; the reference's separate backward_delta and
//  backward launches are one kernel here, and the forward reads x once.)
//
// Algorithmic HBM bytes per element: forward 2*e (+1 for the byte mask), backward 3*e.
#include <type_traits>

#include "row_common.cuh"

namespace tb200 {

// -inf in every element of a packed 32-bit word of T
template <typename T>
__device__ inline uint32_t neg_inf_word() {
  if constexpr (std::is_same<T, float>::value) return 0xff800000u;
  else if constexpr (std::is_same<T, __half>::value) return 0xfc00fc00u;
  else return 0xff80ff80u;
}

// 0xff in every byte of `m` that is not zero
__device__ inline uint32_t nonzero_bytes(uint32_t m) {
  const uint32_t high = (m | ((m & 0x7f7f7f7fu) + 0x7f7f7f7fu)) & 0x80808080u;
  return (high >> 7) * 0xffu;
}

// The row stays packed in registers as loaded; masking is done on the packed words (a masked
// element becomes the bit pattern of -inf), the arithmetic runs on fp32 pairs (two-lane
// instructions). The kernel issues about 7 instructions per element where a scalar formulation
// took 11, which matters because the masked forward was at 60 % issue utilisation.
template <typename T, int CHUNKS, bool CTA_ROW, bool MASKED>
__global__ void __launch_bounds__(CTA_ROW ? 512 : 256)
    softmax_fwd_vec(T* __restrict__ y, const T* __restrict__ x, const uint8_t* __restrict__ mask,
                    int64_t rows, int cols, int64_t row_stride, int64_t mask_row_stride) {
  constexpr int VEC = Traits<T>::VEC;
  constexpr int PAIRS = VEC / 2;
  __shared__ float slot[64];
  int phase = 0;
  RowThread<CTA_ROW> rt;
  pdl_wait();     // (programmatic dependent launch: nothing is read before the previous kernel is done)
  pdl_release();  // the next kernel of the stream may be scheduled
  constexpr float LOG2E = 1.4426950408889634f;
  const uint32_t ninf = neg_inf_word<T>();
  for (int64_t row = rt.first_row(); row < rows; row += rt.row_step()) {
    uint4 raw[CHUNKS];
    const T* xr = x + row * row_stride;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      raw[c] = col < cols ? ld_stream(xr + col) : make_uint4(ninf, ninf, ninf, ninf);
    }
    if constexpr (MASKED) {
      // every mask load is issued before the first one is used (no mask bytes = nothing masked)
      const uint8_t* mr = mask + row * mask_row_stride;
      uint32_t mw[CHUNKS][VEC / 4];
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = rt.template col<VEC>(c);
        if constexpr (VEC == 8) {
          const uint2 t = col < cols ? __ldg(reinterpret_cast<const uint2*>(mr + col)) : make_uint2(0u, 0u);
          mw[c][0] = t.x;
          mw[c][1] = t.y;
        } else {
          mw[c][0] = col < cols ? __ldg(reinterpret_cast<const uint32_t*>(mr + col)) : 0u;
        }
      }
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        uint32_t* w = reinterpret_cast<uint32_t*>(&raw[c]);
        if constexpr (VEC == 8) {  // 8 mask bytes, 4 words of two 16-bit elements
          const uint32_t m0 = nonzero_bytes(mw[c][0]), m1 = nonzero_bytes(mw[c][1]);
          const uint32_t k0 = __byte_perm(m0, 0, 0x1100), k1 = __byte_perm(m0, 0, 0x3322);
          const uint32_t k2 = __byte_perm(m1, 0, 0x1100), k3 = __byte_perm(m1, 0, 0x3322);
          w[0] = (w[0] & ~k0) | (ninf & k0);
          w[1] = (w[1] & ~k1) | (ninf & k1);
          w[2] = (w[2] & ~k2) | (ninf & k2);
          w[3] = (w[3] & ~k3) | (ninf & k3);
        } else {  // 4 mask bytes, 4 fp32 elements
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if ((mw[c][0] >> (8 * i)) & 0xffu) w[i] = ninf;
        }
      }
    }
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      uint64_t t[PAIRS];
      unpack2<T>(raw[c], t);
#pragma unroll
      for (int i = 0; i < PAIRS; i += 2) {
        float a0, a1, b0, b1;
        am::unpack2f(t[i], a0, a1);
        am::unpack2f(t[i + 1], b0, b1);
        m0 = am::max3(m0, a0, a1);
        m1 = am::max3(m1, b0, b1);
      }
    }
    const float m = row_reduce<CTA_ROW, true>(fmaxf(m0, m1), slot, phase);
    // a fully masked row has m = -inf: (x - m) is NaN, as in the eager oracle
    const uint64_t log2e2 = splat2(LOG2E), nmb2 = splat2(-m * LOG2E);
    uint64_t e[CHUNKS][PAIRS];
    uint64_t s2 = 0ull;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      uint64_t t[PAIRS];
      unpack2<T>(raw[c], t);
#pragma unroll
      for (int i = 0; i < PAIRS; ++i) {
        float x0, x1;
        am::unpack2f(am::fma2(t[i], log2e2, nmb2), x0, x1);
        e[c][i] = am::pack2f(exp2f(x0), exp2f(x1));
        s2 = am::add2(s2, e[c][i]);
      }
    }
    const float sum = row_reduce<CTA_ROW, false>(hsum2(s2), slot, phase);
    const uint64_t inv2 = splat2(1.f / sum);
    T* yr = y + row * row_stride;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = rt.template col<VEC>(c);
      if (col < cols) {
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) e[c][i] = am::mul2(e[c][i], inv2);
        st_stream(yr + col, pack2<T>(e[c]));
      }
    }
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
  // Rows are taken last to first: after a forward pass over the same rows, the probabilities it
  // wrote last are the ones still in L2.
  for (int64_t it = rt.first_row(); it < rows; it += rt.row_step()) {
    const int64_t row = rows - 1 - it;
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
