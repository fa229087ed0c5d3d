// CUDA-core attention, forward and backward: the kernels for everything the tensor-core
// path does not take (fp32 operands, head sizes 16/32, sequences shorter than a tile,
// the dense mask gradient). One warp owns one query row (forward, dq) or one key row
// (dk, dv); scores are recomputed from q, k and the saved log-sum-exp in backward.
//
//   fwd:  s_j = scale*q.k_j + M_j;  o = sum_j softmax(s)_j v_j;  lse = log sum_j exp(s_j)
//   bwd:  delta = o.do;  p_j = exp(s_j - lse);  dv_j += p_j do;  dp_j = do.v_j;
//         ds_j = p_j (dp_j - delta);  dq += scale ds_j k_j;  dk_j += scale ds_j q;  dM_j = ds_j
// (restates trident/kernel/attention.py:115-165 and :283-339 in fp32.)
#include "attention.cuh"
#include "common.cuh"

namespace tb200 {

template <typename T>
__device__ inline float ldf(const T* p) { return Traits<T>::to_f(*p); }

template <typename T, int D>
__global__ void __launch_bounds__(128)
    attn_fwd_simt(T* __restrict__ out, float* __restrict__ lse, const T* __restrict__ q,
                  const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ mask,
                  AttnArgs a) {
  constexpr int DL = (D + 31) / 32;  // output dims per lane
  __shared__ float qs[4][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  const int64_t b = blockIdx.y / a.H, h = blockIdx.y % a.H;
  if (row >= a.S) return;
  const T* qr = q + b * a.qs[0] + h * a.qs[1] + row * a.qs[2];
  for (int d = lane; d < D; d += 32) qs[warp][d] = ldf(qr + d * a.qs[3]) * a.scale;
  __syncwarp();
  const T* kb = k + b * a.ks[0] + h * a.ks[1];
  const T* vb = v + b * a.vs[0] + h * a.vs[1];
  const T* mr = mask ? mask + b * a.ms[0] + h * a.ms[1] + row * a.ms[2] : nullptr;
  float m = -INFINITY, l = 0.f, o[DL];
#pragma unroll
  for (int i = 0; i < DL; ++i) o[i] = 0.f;
  const int64_t kend = a.causal ? row + 1 : a.S;
  for (int64_t kc = 0; kc < kend; kc += 32) {
    const int64_t key = kc + lane;
    float s = -INFINITY;
    if (key < kend) {
      const T* kr = kb + key * a.ks[2];
      float acc = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) acc = fmaf(qs[warp][d], ldf(kr + d * a.ks[3]), acc);
      s = acc;
      if (mr) s += ldf(mr + key * a.ms[3]);
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = s == -INFINITY ? 0.f : expf(s - m_new);
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < DL; ++i) o[i] *= corr;
    const int nk = (int)min((int64_t)32, kend - kc);
    for (int j = 0; j < nk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const T* vr = vb + (kc + j) * a.vs[2];
#pragma unroll
      for (int i = 0; i < DL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) o[i] = fmaf(pj, ldf(vr + d * a.vs[3]), o[i]);
      }
    }
    m = m_new;
  }
  T* orow = out + b * a.os[0] + h * a.os[1] + row * a.os[2];
#pragma unroll
  for (int i = 0; i < DL; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d * a.os[3]] = Traits<T>::from_f(o[i] / l);
  }
  if (lane == 0) lse[(b * a.H + h) * a.S + row] = m + logf(l);
}

// delta[b,h,s] = sum_d out*dout. dout is contiguous [B,H,S,D]; out is strided.
template <typename T>
__global__ void attn_delta_kernel(float* __restrict__ delta, const T* __restrict__ out,
                                  const T* __restrict__ dout, AttnArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t total = a.B * a.H * a.S;
  if (r >= total) return;
  const int64_t s = r % a.S, h = (r / a.S) % a.H, b = r / (a.S * a.H);
  const T* orow = out + b * a.os[0] + h * a.os[1] + s * a.os[2];
  const T* drow = dout + r * a.D;
  float acc = 0.f;
  for (int d = lane; d < a.D; d += 32) acc += ldf(orow + d * a.os[3]) * ldf(drow + d);
  acc = warp_sum(acc);
  if (lane == 0) delta[r] = acc;
}

template <typename T, int D>
__global__ void __launch_bounds__(128)
    attn_bwd_dq_simt(T* __restrict__ dq, T* __restrict__ dmask, const T* __restrict__ dout,
                     const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                     const float* __restrict__ lse, const float* __restrict__ delta,
                     const T* __restrict__ mask, AttnArgs a) {
  constexpr int DL = (D + 31) / 32;
  __shared__ float qs[4][D];
  __shared__ float gs[4][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  const int64_t b = blockIdx.y / a.H, h = blockIdx.y % a.H;
  if (row >= a.S) return;
  const int64_t bh = b * a.H + h;
  const T* qr = q + b * a.qs[0] + h * a.qs[1] + row * a.qs[2];
  const T* gr = dout + (bh * a.S + row) * D;
  for (int d = lane; d < D; d += 32) {
    qs[warp][d] = ldf(qr + d * a.qs[3]) * a.scale;
    gs[warp][d] = ldf(gr + d);
  }
  __syncwarp();
  const T* kb = k + b * a.ks[0] + h * a.ks[1];
  const T* vb = v + b * a.vs[0] + h * a.vs[1];
  const T* mr = mask ? mask + b * a.ms[0] + h * a.ms[1] + row * a.ms[2] : nullptr;
  T* dmr = dmask ? dmask + (bh * a.S + row) * a.S : nullptr;
  const float L = lse[bh * a.S + row], dl = delta[bh * a.S + row];
  float acc[DL];
#pragma unroll
  for (int i = 0; i < DL; ++i) acc[i] = 0.f;
  const int64_t kend = a.causal ? row + 1 : a.S;
  for (int64_t kc = 0; kc < kend; kc += 32) {
    const int64_t key = kc + lane;
    float ds = 0.f;
    if (key < kend) {
      const T* kr = kb + key * a.ks[2];
      const T* vr = vb + key * a.vs[2];
      float s = 0.f, dp = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) {
        s = fmaf(qs[warp][d], ldf(kr + d * a.ks[3]), s);
        dp = fmaf(gs[warp][d], ldf(vr + d * a.vs[3]), dp);
      }
      if (mr) s += ldf(mr + key * a.ms[3]);
      const float p = s == -INFINITY ? 0.f : expf(s - L);
      ds = p * (dp - dl);
      if (dmr) dmr[key] = Traits<T>::from_f(ds);
    }
    const int nk = (int)min((int64_t)32, kend - kc);
    for (int j = 0; j < nk; ++j) {
      const float dj = __shfl_sync(0xffffffffu, ds, j);
      const T* kr = kb + (kc + j) * a.ks[2];
#pragma unroll
      for (int i = 0; i < DL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(dj, ldf(kr + d * a.ks[3]), acc[i]);
      }
    }
  }
  T* dqr = dq + (bh * a.S + row) * D;
#pragma unroll
  for (int i = 0; i < DL; ++i) {
    const int d = lane + 32 * i;
    if (d < D) dqr[d] = Traits<T>::from_f(acc[i] * a.scale);
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(128)
    attn_bwd_dkv_simt(T* __restrict__ dk, T* __restrict__ dv, const T* __restrict__ dout,
                      const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      const float* __restrict__ lse, const float* __restrict__ delta,
                      const T* __restrict__ mask, AttnArgs a) {
  constexpr int DL = (D + 31) / 32;
  __shared__ float ks_[4][D];
  __shared__ float vs_[4][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t key = (int64_t)blockIdx.x * 4 + warp;
  const int64_t b = blockIdx.y / a.H, h = blockIdx.y % a.H;
  if (key >= a.S) return;
  const int64_t bh = b * a.H + h;
  const T* kr = k + b * a.ks[0] + h * a.ks[1] + key * a.ks[2];
  const T* vr = v + b * a.vs[0] + h * a.vs[1] + key * a.vs[2];
  for (int d = lane; d < D; d += 32) {
    ks_[warp][d] = ldf(kr + d * a.ks[3]) * a.scale;
    vs_[warp][d] = ldf(vr + d * a.vs[3]);
  }
  __syncwarp();
  const T* qb = q + b * a.qs[0] + h * a.qs[1];
  const T* gb = dout + bh * a.S * D;
  const T* mb = mask ? mask + b * a.ms[0] + h * a.ms[1] + key * a.ms[3] : nullptr;
  float acck[DL], accv[DL];
#pragma unroll
  for (int i = 0; i < DL; ++i) acck[i] = accv[i] = 0.f;
  const int64_t qbeg = a.causal ? (key / 32) * 32 : 0;
  for (int64_t qc = qbeg; qc < a.S; qc += 32) {
    const int64_t qi = qc + lane;
    float p = 0.f, ds = 0.f;
    if (qi < a.S && (!a.causal || qi >= key)) {
      const T* qr = qb + qi * a.qs[2];
      const T* gr = gb + qi * D;
      float s = 0.f, dp = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) {
        s = fmaf(ks_[warp][d], ldf(qr + d * a.qs[3]), s);
        dp = fmaf(vs_[warp][d], ldf(gr + d), dp);
      }
      if (mb) s += ldf(mb + qi * a.ms[2]);
      p = s == -INFINITY ? 0.f : expf(s - lse[bh * a.S + qi]);
      ds = p * (dp - delta[bh * a.S + qi]);
    }
    const int nq = (int)min((int64_t)32, a.S - qc);
    for (int j = 0; j < nq; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const float dj = __shfl_sync(0xffffffffu, ds, j);
      const T* qr = qb + (qc + j) * a.qs[2];
      const T* gr = gb + (qc + j) * D;
#pragma unroll
      for (int i = 0; i < DL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) {
          accv[i] = fmaf(pj, ldf(gr + d), accv[i]);
          acck[i] = fmaf(dj, ldf(qr + d * a.qs[3]), acck[i]);
        }
      }
    }
  }
  T* dkr = dk + (bh * a.S + key) * D;
  T* dvr = dv + (bh * a.S + key) * D;
#pragma unroll
  for (int i = 0; i < DL; ++i) {
    const int d = lane + 32 * i;
    if (d < D) {
      dkr[d] = Traits<T>::from_f(acck[i] * a.scale);
      dvr[d] = Traits<T>::from_f(accv[i]);
    }
  }
}

template <typename T, typename Fn>
static int dispatch_head(int64_t D, Fn&& fn) {
  switch (D) {
    case 16: return fn(IntD<16>{});
    case 32: return fn(IntD<32>{});
    case 64: return fn(IntD<64>{});
    case 128: return fn(IntD<128>{});
  }
  set_error("attention: head size %lld not in {16,32,64,128}", (long long)D);
  return TB200_ERR_UNSUPPORTED;
}

int launch_attn_fwd_simt(void* out, float* lse, const void* q, const void* k, const void* v,
                         const void* mask, const AttnArgs& a, int dtype, cudaStream_t st) {
  TB200_REQUIRE(a.B * a.H <= 65535, TB200_ERR_UNSUPPORTED,
                "attention (CUDA-core path): batch*heads %lld exceeds 65535",
                (long long)(a.B * a.H));
  dim3 grid((unsigned)ceil_div(a.S, 4), (unsigned)(a.B * a.H));
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    return dispatch_head<T>(a.D, [&](auto d) -> int {
      attn_fwd_simt<T, decltype(d)::value><<<grid, 128, 0, st>>>(
          (T*)out, lse, (const T*)q, (const T*)k, (const T*)v, (const T*)mask, a);
      return launch_status("attn_fwd_simt");
    });
  });
}

int launch_attn_delta(float* delta, const void* out, const void* dout, const AttnArgs& a,
                      int dtype, cudaStream_t st) {
  const int64_t total = a.B * a.H * a.S;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    attn_delta_kernel<T><<<(unsigned)ceil_div(total, 8), 256, 0, st>>>(delta, (const T*)out,
                                                                      (const T*)dout, a);
    return launch_status("attn_delta");
  });
}

int launch_attn_bwd_simt(void* dq, void* dk, void* dv, void* dmask, const void* dout,
                         const void* q, const void* k, const void* v, const float* lse,
                         const float* delta, const void* mask, const AttnArgs& a, int dtype,
                         cudaStream_t st) {
  TB200_REQUIRE(a.B * a.H <= 65535, TB200_ERR_UNSUPPORTED,
                "attention (CUDA-core path): batch*heads %lld exceeds 65535",
                (long long)(a.B * a.H));
  dim3 grid((unsigned)ceil_div(a.S, 4), (unsigned)(a.B * a.H));
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    return dispatch_head<T>(a.D, [&](auto d) -> int {
      constexpr int D = decltype(d)::value;
      attn_bwd_dq_simt<T, D><<<grid, 128, 0, st>>>((T*)dq, (T*)dmask, (const T*)dout, (const T*)q,
                                                   (const T*)k, (const T*)v, lse, delta,
                                                   (const T*)mask, a);
      int rc = launch_status("attn_bwd_dq_simt");
      if (rc) return rc;
      attn_bwd_dkv_simt<T, D><<<grid, 128, 0, st>>>((T*)dk, (T*)dv, (const T*)dout, (const T*)q,
                                                    (const T*)k, (const T*)v, lse, delta,
                                                    (const T*)mask, a);
      return launch_status("attn_bwd_dkv_simt");
    });
  });
}

}  // namespace tb200
