// CUDA-core GEMM for the shapes the tensor-core kernel does not take (fp32 operands,
// permuted/unaligned operands such as K=100 rows of 16-bit data), the GEGLU elementwise
// kernels, and the bias-gradient column sum.
//
//   gemm_simt:  C[b,m,n] = sum_{r,k} A[b,r,m,k] * B[b,r,n,k] (+ bias[n]), fp32 accumulate,
//               every operand addressed through element strides, so the same kernel
//               serves Linear forward (A=x, B=w), input gradient (A=dy, B=w^T) and
//               weight gradient (A=dy^T, B=x^T, r = batch folded into the reduction).
#include <algorithm>

#include "common.cuh"
#include "gemm_simt.cuh"
#include "row_common.cuh"

namespace tb200 {

template <typename T>
__global__ void __launch_bounds__(256)
    gemm_simt_kernel(T* __restrict__ C, const T* __restrict__ A, const T* __restrict__ Bm,
                     const T* __restrict__ bias, SimtGemmArgs g) {
  __shared__ float As[16][65];
  __shared__ float Bs[16][65];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
  const int64_t batch = blockIdx.z;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int64_t r = 0; r < g.R; ++r) {
    const T* Ab = A + batch * g.a_sb + r * g.a_sr;
    const T* Bb = Bm + batch * g.b_sb + r * g.b_sr;
    for (int64_t k0 = 0; k0 < g.K; k0 += 16) {
      if (g.a_sk == 1 || g.a_sm != 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = threadIdx.x + i * 256;
          const int kk = idx & 15, mm = idx >> 4;
          const int64_t m = m0 + mm, k = k0 + kk;
          As[kk][mm] = (m < g.M && k < g.K) ? Traits<T>::to_f(Ab[m * g.a_sm + k * g.a_sk]) : 0.f;
        }
      } else {  // m is the contiguous index: walk it fastest
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = threadIdx.x + i * 256;
          const int mm = idx & 63, kk = idx >> 6;
          const int64_t m = m0 + mm, k = k0 + kk;
          As[kk][mm] = (m < g.M && k < g.K) ? Traits<T>::to_f(Ab[m * g.a_sm + k * g.a_sk]) : 0.f;
        }
      }
      if (g.b_sk == 1 || g.b_sn != 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = threadIdx.x + i * 256;
          const int kk = idx & 15, nn = idx >> 4;
          const int64_t n = n0 + nn, k = k0 + kk;
          Bs[kk][nn] = (n < g.N && k < g.K) ? Traits<T>::to_f(Bb[n * g.b_sn + k * g.b_sk]) : 0.f;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = threadIdx.x + i * 256;
          const int nn = idx & 63, kk = idx >> 6;
          const int64_t n = n0 + nn, k = k0 + kk;
          Bs[kk][nn] = (n < g.N && k < g.K) ? Traits<T>::to_f(Bb[n * g.b_sn + k * g.b_sk]) : 0.f;
        }
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (bias) v += Traits<T>::to_f(bias[n]);
      C[batch * g.c_sb + m * g.c_sm + n * g.c_sn] = Traits<T>::from_f(v);
    }
  }
}

int launch_gemm_simt(void* C, const void* A, const void* Bm, const void* bias,
                     const SimtGemmArgs& g, int dtype, cudaStream_t st) {
  if (g.M == 0 || g.N == 0 || g.batches == 0) return 0;
  TB200_REQUIRE(ceil_div(g.M, 64) <= 65535 && g.batches <= 65535, TB200_ERR_UNSUPPORTED,
                "gemm_simt: grid too large (M=%lld, batches=%lld)", (long long)g.M,
                (long long)g.batches);
  dim3 grid((unsigned)ceil_div(g.N, 64), (unsigned)ceil_div(g.M, 64), (unsigned)g.batches);
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    gemm_simt_kernel<T><<<grid, 256, 0, st>>>((T*)C, (const T*)A, (const T*)Bm, (const T*)bias, g);
    return launch_status("gemm_simt");
  });
}

// ---------------------------------------------------------------------------
// GELU (exact erf form and tanh approximation) and its derivative
// ---------------------------------------------------------------------------
__device__ inline float gelu_f(float g, bool tanh_form) {
  if (tanh_form) {
    const float a = tanhf(0.7978845608028654f * g * (1.f + 0.044715f * g * g));
    return 0.5f * g * (1.f + a);
  }
  return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
}
// GELU and its derivative together (the backward needs both, and they share their transcendentals).
// For 16-bit tensors the erf form takes the normal CDF from one exponential and one reciprocal
// (Abramowitz & Stegun 7.1.26, |error| <= 1.5e-7, far below the output's rounding step); the
// exponential e^(-g*g/2) is the one the derivative needs. fp32 tensors use erff.
template <typename T>
__device__ inline void gelu_value_grad(float g, bool tanh_form, float& gel, float& grad) {
  if (tanh_form) {
    const float a = tanhf(0.7978845608028654f * g * (1.f + 0.044715f * g * g));
    gel = 0.5f * g * (1.f + a);
    grad = 0.5f * (1.f + a + g * (1.f - a * a) * (0.7978845608028654f + 0.1070322244089f * g * g));
    return;
  }
  float cdf, pdf_e;
  if constexpr (sizeof(T) == 2) {
    const float t = __frcp_rn(fmaf(0.3275911f * 0.7071067811865476f, fabsf(g), 1.f));
    pdf_e = exp2f(-0.7213475204444817f * g * g);
    float poly = fmaf(t, 1.061405429f, -1.453152027f);
    poly = fmaf(t, poly, 1.421413741f);
    poly = fmaf(t, poly, -0.284496736f);
    poly = fmaf(t, poly, 0.254829592f);
    const float h = 0.5f * poly * t * pdf_e;  // the smaller tail
    cdf = g < 0.f ? h : 1.f - h;
  } else {
    cdf = fmaf(0.5f, erff(g * 0.7071067811865476f), 0.5f);
    pdf_e = __expf(-0.5f * g * g);
  }
  gel = g * cdf;
  grad = fmaf(g * 0.3989422804014327f, pdf_e, cdf);
}

// out[r, j] = state * gelu(gate), from the already rounded state_gate [rows, 2X]
template <typename T, int V>
__global__ void geglu_fwd_elementwise_kernel(T* __restrict__ out, const T* __restrict__ sg,
                                             int64_t rows, int64_t X, int tanh_form) {
  const int64_t per_row = X / V;
  const int64_t total = rows * per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / per_row, j = (idx % per_row) * V;
    const T* s = sg + r * 2 * X + j;
    float sv[V], gv[V];
    if constexpr (V > 1) {
      unpack<T>(ld_stream(s), sv);
      unpack<T>(ld_stream(s + X), gv);
    } else {
      sv[0] = Traits<T>::to_f(s[0]);
      gv[0] = Traits<T>::to_f(s[X]);
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
      // gelu rounded to T first, then the product: the rounding points of the eager oracle
      const float ge = Traits<T>::to_f(Traits<T>::from_f(gelu_f(gv[i], tanh_form)));
      sv[i] = sv[i] * ge;
    }
    if constexpr (V > 1)
      st_stream(out + r * X + j, pack<T>(sv));
    else
      out[r * X + j] = Traits<T>::from_f(sv[0]);
  }
}

template <typename T, int V>
__global__ void geglu_bwd_elementwise_kernel(T* __restrict__ dsg, const T* __restrict__ dout,
                                             const T* __restrict__ sg, int64_t rows, int64_t X,
                                             int tanh_form) {
  const int64_t per_row = X / V;
  const int64_t total = rows * per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / per_row, j = (idx % per_row) * V;
    const T* s = sg + r * 2 * X + j;
    float sv[V], gv[V], dv[V];
    if constexpr (V > 1) {
      unpack<T>(ld_stream(s), sv);
      unpack<T>(ld_stream(s + X), gv);
      unpack<T>(ld_stream(dout + r * X + j), dv);
    } else {
      sv[0] = Traits<T>::to_f(s[0]);
      gv[0] = Traits<T>::to_f(s[X]);
      dv[0] = Traits<T>::to_f(dout[r * X + j]);
    }
    float ds[V], dg[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float gel, grad;
      gelu_value_grad<T>(gv[i], tanh_form, gel, grad);
      ds[i] = dv[i] * gel;
      dg[i] = dv[i] * sv[i] * grad;
    }
    T* d = dsg + r * 2 * X + j;
    if constexpr (V > 1) {
      st_stream(d, pack<T>(ds));
      st_stream(d + X, pack<T>(dg));
    } else {
      d[0] = Traits<T>::from_f(ds[0]);
      d[X] = Traits<T>::from_f(dg[0]);
    }
  }
}

// GEGLU backward elementwise step fused with the bias gradient: a CTA owns 32 * V adjacent
// columns of the state half (and the same columns of the gate half) and a slab of rows; every
// thread keeps fp32 column sums of what it writes, and the CTA leaves one partial row
// [2X] per slab for colsum_finalize_kernel. GELU and its derivative share one erf.
template <typename T, int V>
__global__ void __launch_bounds__(256)
    geglu_bwd_bias_kernel(T* __restrict__ dsg, float* __restrict__ partial, const T* __restrict__ dout,
                          const T* __restrict__ sg, int64_t rows, int64_t X, int64_t rows_per_slab,
                          int tanh_form) {
  __shared__ float red[8][2][32 * V + 1];
  const int64_t j = ((int64_t)blockIdx.x * 32 + threadIdx.x) * V;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
  const int64_t r1 = min(rows, r0 + rows_per_slab);
  float acc_s[V], acc_g[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc_s[i] = acc_g[i] = 0.f;
  if (j < X) {
    auto row_step = [&](int64_t r, const uint4& sraw, const uint4& graw, const uint4& draw) {
      float sv[V], gv[V], dv[V], ds[V], dg[V];
      unpack<T>(sraw, sv);
      unpack<T>(graw, gv);
      unpack<T>(draw, dv);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float gel, grad;
        gelu_value_grad<T>(gv[i], tanh_form, gel, grad);
        ds[i] = dv[i] * gel;
        dg[i] = dv[i] * sv[i] * grad;
        acc_s[i] += ds[i];
        acc_g[i] += dg[i];
      }
      T* d = dsg + r * 2 * X + j;
      st_stream(d, pack<T>(ds));
      st_stream(d + X, pack<T>(dg));
    };
    for (int64_t r = r0 + threadIdx.y; r < r1; r += 8) {
      const T* s0 = sg + r * 2 * X + j;
      const uint4 a0 = ld_stream(s0), a1 = ld_stream(s0 + X), a2 = ld_stream(dout + r * X + j);
      row_step(r, a0, a1, a2);
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) {
    red[threadIdx.y][0][threadIdx.x * V + i] = acc_s[i];
    red[threadIdx.y][1][threadIdx.x * V + i] = acc_g[i];
  }
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;
  for (int c = t; c < 2 * 32 * V; c += 256) {
    const int which = c / (32 * V), cc = c % (32 * V);
    const int64_t gc = (int64_t)blockIdx.x * 32 * V + cc;
    if (gc < X) {
      float sum = 0.f;
#pragma unroll
      for (int y = 0; y < 8; ++y) sum += red[y][which][cc];
      partial[(int64_t)blockIdx.y * 2 * X + (int64_t)which * X + gc] = sum;
    }
  }
}

int launch_geglu_fwd_elementwise(void* out, const void* sg, int64_t rows, int64_t X, int tanh_form,
                                 int dtype, cudaStream_t st) {
  if (rows == 0 || X == 0) return 0;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int V = Traits<T>::VEC;
    const bool vec = X % V == 0 && aligned16(out) && aligned16(sg);
    const int64_t total = rows * (vec ? X / V : X);
    const int64_t cap = (int64_t)sm_count() * 16;
    const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(total, 256), cap);
    if (vec)
      geglu_fwd_elementwise_kernel<T, V><<<grid, 256, 0, st>>>((T*)out, (const T*)sg, rows, X,
                                                               tanh_form);
    else
      geglu_fwd_elementwise_kernel<T, 1><<<grid, 256, 0, st>>>((T*)out, (const T*)sg, rows, X,
                                                               tanh_form);
    return launch_status("geglu_fwd_elementwise");
  });
}

// ---------------------------------------------------------------------------
// bias gradient: column sums of dy [rows, N]
// ---------------------------------------------------------------------------
// Block (32, 8): threadIdx.x owns V adjacent columns, threadIdx.y splits the rows of the
// CTA's row slab; grid.y slabs write fp32 partials [slab][N].
template <typename T, int V>
__global__ void __launch_bounds__(256)
    colsum_partial_kernel(float* __restrict__ partial, const T* __restrict__ dy, int64_t rows,
                          int64_t N, int64_t rows_per_slab) {
  __shared__ float red[8][32 * V + 1];
  const int64_t col = ((int64_t)blockIdx.x * 32 + threadIdx.x) * V;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
  const int64_t r1 = min(rows, r0 + rows_per_slab);
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (col < N) {
    for (int64_t r = r0 + threadIdx.y; r < r1; r += 8) {
      float v[V];
      if constexpr (V > 1)
        unpack<T>(ld_stream(dy + r * N + col), v);
      else
        v[0] = Traits<T>::to_f(dy[r * N + col]);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] += v[i];
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) red[threadIdx.y][threadIdx.x * V + i] = acc[i];
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;
  for (int c = t; c < 32 * V; c += 256) {
    const int64_t gc = (int64_t)blockIdx.x * 32 * V + c;
    if (gc < N) {
      float s = 0.f;
#pragma unroll
      for (int y = 0; y < 8; ++y) s += red[y][c];
      partial[(int64_t)blockIdx.y * N + gc] = s;
    }
  }
}

static int64_t bias_slabs(int64_t rows, int64_t N) {
  const int64_t col_ctas = std::max<int64_t>(1, ceil_div(N, 256));
  int64_t slabs = std::max<int64_t>(1, ((int64_t)sm_count() * 8) / col_ctas);
  slabs = std::min<int64_t>(slabs, std::max<int64_t>(1, ceil_div(rows, 64)));
  return std::min<int64_t>(slabs, 1024);
}

}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_linear_bwd_bias_workspace(int64_t rows, int64_t N) {
  if (rows <= 0 || N <= 0) return 0;
  return (size_t)bias_slabs(rows, N) * (size_t)N * sizeof(float);
}

extern "C" int tb200_linear_bwd_bias(void* dbias, const void* dy, void* workspace,
                                     size_t workspace_bytes, int64_t rows, int64_t N, int dtype,
                                     void* stream) {
  TB200_REQUIRE(rows >= 0 && N > 0, TB200_ERR_INVALID, "linear_bwd_bias: bad shape");
  if (rows == 0)  // a sum over no rows
    return zero_fill(dbias, (size_t)N * dtype_size(dtype), (cudaStream_t)stream, "linear_bwd_bias");
  TB200_REQUIRE(dbias && dy && workspace, TB200_ERR_INVALID, "linear_bwd_bias: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t slabs = bias_slabs(rows, N);
  TB200_REQUIRE(workspace_bytes >= (size_t)slabs * N * sizeof(float), TB200_ERR_WORKSPACE,
                "linear_bwd_bias: workspace too small");
  const int64_t rows_per_slab = std::max<int64_t>(1, ceil_div(rows, slabs));
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int V = Traits<T>::VEC;
    const bool vec = N % V == 0 && aligned16(dy);
    dim3 block(32, 8);
    if (vec) {
      dim3 grid((unsigned)ceil_div(N, 32 * V), (unsigned)slabs);
      colsum_partial_kernel<T, V><<<grid, block, 0, st>>>((float*)workspace, (const T*)dy, rows, N,
                                                          rows_per_slab);
    } else {
      dim3 grid((unsigned)ceil_div(N, 32), (unsigned)slabs);
      colsum_partial_kernel<T, 1><<<grid, block, 0, st>>>((float*)workspace, (const T*)dy, rows, N,
                                                          rows_per_slab);
    }
    int rc = launch_status("colsum_partial");
    if (rc) return rc;
    dim3 fgrid((unsigned)ceil_div(N, 32), 1), fblock(32, 32);
    colsum_finalize_kernel<T><<<fgrid, fblock, 0, st>>>((T*)dbias, nullptr, (const float*)workspace,
                                                        (int)slabs, (int)N);
    rc = launch_status("colsum_finalize");
    if (rc == 0) note_kernel("colsum", 2);
    return rc;
  });
}

extern "C" int tb200_geglu_bwd_elementwise(void* d_state_gate, const void* dout,
                                           const void* state_gate, int64_t rows, int64_t N,
                                           int gelu_tanh, int dtype, void* stream) {
  TB200_REQUIRE(rows >= 0 && N > 0 && N % 2 == 0, TB200_ERR_INVALID,
                "geglu_bwd_elementwise: N must be even and positive");
  if (rows == 0) return 0;
  TB200_REQUIRE(d_state_gate && dout && state_gate, TB200_ERR_INVALID,
                "geglu_bwd_elementwise: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t X = N / 2;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int V = Traits<T>::VEC;
    const bool vec =
        X % V == 0 && aligned16(d_state_gate) && aligned16(dout) && aligned16(state_gate);
    const int64_t total = rows * (vec ? X / V : X);
    const int64_t cap = (int64_t)sm_count() * 16;
    const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(total, 256), cap);
    if (vec)
      geglu_bwd_elementwise_kernel<T, V><<<grid, 256, 0, st>>>(
          (T*)d_state_gate, (const T*)dout, (const T*)state_gate, rows, X, gelu_tanh);
    else
      geglu_bwd_elementwise_kernel<T, 1><<<grid, 256, 0, st>>>(
          (T*)d_state_gate, (const T*)dout, (const T*)state_gate, rows, X, gelu_tanh);
    int rc = launch_status("geglu_bwd_elementwise");
    if (rc == 0) note_kernel("elementwise", 1);
    return rc;
  });
}


extern "C" int tb200_geglu_bwd_elementwise_bias(void* d_state_gate, void* dbias, const void* dout,
                                                const void* state_gate, void* workspace,
                                                size_t workspace_bytes, int64_t rows, int64_t N,
                                                int gelu_tanh, int dtype, void* stream) {
  TB200_REQUIRE(rows >= 0 && N > 0 && N % 2 == 0, TB200_ERR_INVALID,
                "geglu_bwd_elementwise_bias: N must be even and positive");
  if (rows == 0)  // a sum over no rows
    return zero_fill(dbias, (size_t)N * dtype_size(dtype), (cudaStream_t)stream, "geglu_bwd_elementwise_bias");
  TB200_REQUIRE(d_state_gate && dbias && dout && state_gate && workspace, TB200_ERR_INVALID,
                "geglu_bwd_elementwise_bias: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t X = N / 2;
  const int64_t slabs = bias_slabs(rows, N);
  TB200_REQUIRE(workspace_bytes >= (size_t)slabs * N * sizeof(float), TB200_ERR_WORKSPACE,
                "geglu_bwd_elementwise_bias: workspace too small");
  const int64_t rows_per_slab = std::max<int64_t>(1, ceil_div(rows, slabs));
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int V = Traits<T>::VEC;
    const bool vec = X % V == 0 && aligned16(d_state_gate) && aligned16(dout) && aligned16(state_gate) &&
                     aligned16(workspace) && rows > 0;
    if (!vec) {
      // widths the vector kernel does not take: the two separate steps
      int rc = tb200_geglu_bwd_elementwise(d_state_gate, dout, state_gate, rows, N, gelu_tanh, dtype, stream);
      if (rc) return rc;
      return tb200_linear_bwd_bias(dbias, d_state_gate, workspace, workspace_bytes, rows, N, dtype, stream);
    }
    dim3 block(32, 8), grid((unsigned)ceil_div(X, 32 * V), (unsigned)slabs);
    geglu_bwd_bias_kernel<T, V><<<grid, block, 0, st>>>((T*)d_state_gate, (float*)workspace, (const T*)dout,
                                                        (const T*)state_gate, rows, X, rows_per_slab, gelu_tanh);
    int rc = launch_status("geglu_bwd_bias");
    if (rc) return rc;
    dim3 fgrid((unsigned)ceil_div(N, 32), 1), fblock(32, 32);
    colsum_finalize_kernel<T><<<fgrid, fblock, 0, st>>>((T*)dbias, nullptr, (const float*)workspace, (int)slabs,
                                                        (int)N);
    rc = launch_status("colsum_finalize");
    if (rc == 0) note_kernel("elementwise", 2);
    return rc;
  });
}
