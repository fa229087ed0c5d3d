// Argument block and launch entry points shared by the attention kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace tb200 {

template <int D>
using IntD = std::integral_constant<int, D>;

// Strides are in elements, ordered (batch, head, sequence, feature); mask strides are
// (batch, head, query, key) with 0 for a broadcast dimension.
struct AttnArgs {
  int64_t B = 0, H = 0, S = 0, D = 0;
  int64_t qs[4] = {0, 0, 0, 0}, ks[4] = {0, 0, 0, 0}, vs[4] = {0, 0, 0, 0}, os[4] = {0, 0, 0, 0};
  int64_t ms[4] = {0, 0, 0, 0};
  int causal = 0;
  float scale = 1.f;
};

// CUDA-core kernels (attention_simt.cu)
int launch_attn_fwd_simt(void* out, float* lse, const void* q, const void* k, const void* v,
                         const void* mask, const AttnArgs& a, int dtype, cudaStream_t st);
int launch_attn_delta(float* delta, const void* out, const void* dout, const AttnArgs& a,
                      int dtype, cudaStream_t st);
int launch_attn_bwd_simt(void* dq, void* dk, void* dv, void* dmask, const void* dout,
                         const void* q, const void* k, const void* v, const float* lse,
                         const float* delta, const void* mask, const AttnArgs& a, int dtype,
                         cudaStream_t st);

}  // namespace tb200

namespace tb200 {
// tcgen05 kernels (attention_fwd_tc.cu, attention_bwd_tc.cu): 16-bit operands, head size 64
// or 128, sequence length a multiple of 128, unit innermost strides, 16-byte aligned rows.
bool attn_tc_supported(const AttnArgs& a, int dtype, const void* q, const void* k, const void* v,
                       const void* out);
int launch_attn_fwd_tc(void* out, float* lse, const void* q, const void* k, const void* v,
                       const void* mask, const AttnArgs& a, int dtype, cudaStream_t st);
}  // namespace tb200

namespace tb200 {
// row_scratch: 2 * B*H*S floats (-delta and -lse*log2e, written by a first small kernel);
// dq_acc: fp32 scratch of B*H*S*D elements.
int launch_attn_bwd_tc(void* dq, void* dk, void* dv, void* dmask, const void* dout, const void* q, const void* k,
                       const void* v, const void* out, const float* lse, float* row_scratch,
                       float* dq_acc, const void* mask, const AttnArgs& a, int dtype, cudaStream_t st);
}  // namespace tb200
