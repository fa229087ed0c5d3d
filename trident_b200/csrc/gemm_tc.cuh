// Interface of the tcgen05 (5th-generation tensor core) GEMM used by Linear and GEGLU.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {

// C[m,n] = sum_k A(m,k) * B(n,k) (+ bias[n]), 16-bit operands, fp32 accumulation in
// tensor memory, one rounding to the operand type on the way out.
//   a_kmajor: A is stored [M, K] with K contiguous (leading dimension a_ld);
//             otherwise A is stored [K, M] with M contiguous (an "MN-major" operand).
//   b_kmajor: B is stored [N, K] with K contiguous; otherwise [K, N] with N contiguous.
// GEGLU mode (geglu_out != null): N is the width of state_gate; the kernel pairs column
// j (state) with column N/2 + j (gate) in one accumulator, writes state_gate into c and
// state * gelu(gate) into geglu_out [M, N/2].
struct TcGemmArgs {
  int64_t M = 0, N = 0, K = 0;
  const void* a = nullptr;
  int64_t a_ld = 0;
  bool a_kmajor = true;
  const void* b = nullptr;
  int64_t b_ld = 0;
  bool b_kmajor = true;
  void* c = nullptr;
  int64_t c_ld = 0;
  const void* bias = nullptr;
  void* geglu_out = nullptr;
  int gelu_tanh = 0;
  const float* row_scale = nullptr;  // [M]: the accumulator row is multiplied by it before the bias
};

bool tc_gemm_supported(const TcGemmArgs& g, int dtype);
int launch_gemm_tc(const TcGemmArgs& g, int dtype, cudaStream_t st);

}  // namespace tb200
