// Shared host/device helpers for the tb200 kernels: status plumbing, dtype traits,
// 128-bit vector access, warp/block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/tb200.h"

namespace tb200 {

// ---------------------------------------------------------------------------
// host side: error text, dispatch record, device attributes
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);
void note_kernel(const char* family, int launches);
void add_launches(int launches);
int sm_count();       // SMs of the current device (cached per device)

#define TB200_REQUIRE(cond, code, ...)     \
  do {                                     \
    if (!(cond)) {                         \
      ::tb200::set_error(__VA_ARGS__);     \
      return (code);                       \
    }                                      \
  } while (0)

// Returns the launch error (cudaError_t as a positive int) without synchronising.
static inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// Driver-API entry points (tensor-map encoding) need the primary context bound to the calling
// thread; a thread that has not yet made a runtime call (an autograd worker) may not have it.
static inline void bind_primary_context() {
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
}

// An empty problem (no rows) launches nothing; outputs that are sums over the rows are zero.
static inline int zero_fill(void* p, size_t bytes, cudaStream_t st, const char* who) {
  if (!p || bytes == 0) return 0;
  cudaError_t e = cudaMemsetAsync(p, 0, bytes, st);
  if (e != cudaSuccess) {
    set_error("%s: cudaMemsetAsync failed: %s", who, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// Programmatic dependent launch: the kernel may be scheduled while the previous kernel of the
// stream is still running (its launch latency and the start of its CTAs then overlap that
// kernel's tail). A kernel launched this way must execute pdl_wait() before its first access to
// global memory: the wait returns once the previous kernel has completed and its writes are
// visible (and immediately when there is no such dependency). pdl_release() lets the next kernel
// of the stream be scheduled early in the same way.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     bool cooperative, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cooperative ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Opt-in of a kernel to more than 48 KB of dynamic shared memory. The attribute belongs to the
// (kernel, device) pair, so it is set once per device: `done` holds one bit per device ordinal
// and lives beside the kernel (one static per template instantiation).
static inline cudaError_t smem_optin_per_device(std::atomic<unsigned long long>& done, const void* kern, int bytes) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    dev = -1;
  }
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && (done.load(std::memory_order_acquire) >> dev) & 1ull) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && tracked) done.fetch_or(1ull << dev, std::memory_order_release);
  return e;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t dtype_size(int dtype) { return dtype == TB200_F32 ? 4 : 2; }

// ---------------------------------------------------------------------------
// device side
// ---------------------------------------------------------------------------
template <typename T>
struct Traits;
template <>
struct Traits<float> {
  static constexpr int VEC = 4;  // elements per 16-byte vector
  __device__ static inline float to_f(float v) { return v; }
  __device__ static inline float from_f(float v) { return v; }
};
template <>
struct Traits<__half> {
  static constexpr int VEC = 8;
  __device__ static inline float to_f(__half v) { return __half2float(v); }
  __device__ static inline __half from_f(float v) { return __float2half_rn(v); }
};
template <>
struct Traits<__nv_bfloat16> {
  static constexpr int VEC = 8;
  __device__ static inline float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static inline __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// A 16-byte vector of T viewed as floats.
template <typename T>
struct Vec {
  static constexpr int N = Traits<T>::VEC;
  float v[N];
};

template <typename T>
__device__ inline void unpack(const uint4& raw, float* out);
template <>
__device__ inline void unpack<float>(const uint4& raw, float* out) {
  out[0] = __uint_as_float(raw.x);
  out[1] = __uint_as_float(raw.y);
  out[2] = __uint_as_float(raw.z);
  out[3] = __uint_as_float(raw.w);
}
template <>
__device__ inline void unpack<__half>(const uint4& raw, float* out) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
template <>
__device__ inline void unpack<__nv_bfloat16>(const uint4& raw, float* out) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename T>
__device__ inline uint4 pack(const float* in);
template <>
__device__ inline uint4 pack<float>(const float* in) {
  return make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]),
                    __float_as_uint(in[3]));
}
template <>
__device__ inline uint4 pack<__half>(const float* in) {
  uint4 r;
  __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
  return r;
}
template <>
__device__ inline uint4 pack<__nv_bfloat16>(const float* in) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
  return r;
}

__device__ inline void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ inline void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Streaming 16-byte accesses: data is touched once, keep it out of L1.
__device__ inline uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ inline void st_stream(void* p, const uint4& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ inline uint4 ld_cached(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ inline float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum (or max) over the threads that share a row. ROW_THREADS == 32: one warp per row,
// shuffles only. ROW_THREADS == blockDim.x: the whole CTA shares one row; `slot` is a
// shared array of 2*32 floats used alternately so that one __syncthreads per call is
// enough (`phase` flips on every call).
template <bool CTA_ROW, bool IS_MAX>
__device__ inline float row_reduce(float v, float* slot, int& phase) {
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  if constexpr (CTA_ROW) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float* s = slot + phase * 32;
    phase ^= 1;
    if (lane == 0) s[warp] = v;
    __syncthreads();
    float r = lane < nwarps ? s[lane] : (IS_MAX ? -INFINITY : 0.f);
    v = IS_MAX ? warp_max(r) : warp_sum(r);
  }
  return v;
}

template <typename Fn>
static inline int dispatch_dtype(int dtype, Fn&& fn) {
  switch (dtype) {
    case TB200_F32: return fn(float{});
    case TB200_F16: return fn(__half{});
    case TB200_BF16: return fn(__nv_bfloat16{});
    default: set_error("unknown dtype %d", dtype); return TB200_ERR_INVALID;
  }
}

}  // namespace tb200
