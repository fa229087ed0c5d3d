// Interface of the CUDA-core GEMM and of the GEGLU elementwise helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {

// C[b,m,n] = sum_{r<R} sum_{k<K} A[b,r,m,k] * B[b,r,n,k] (+ bias[n]); strides in elements.
struct SimtGemmArgs {
  int64_t batches = 1, M = 0, N = 0, K = 0, R = 1;
  int64_t a_sb = 0, a_sr = 0, a_sm = 0, a_sk = 0;
  int64_t b_sb = 0, b_sr = 0, b_sn = 0, b_sk = 0;
  int64_t c_sb = 0, c_sm = 0, c_sn = 0;
};

int launch_gemm_simt(void* C, const void* A, const void* Bm, const void* bias,
                     const SimtGemmArgs& g, int dtype, cudaStream_t st);
int launch_geglu_fwd_elementwise(void* out, const void* state_gate, int64_t rows, int64_t X,
                                 int tanh_form, int dtype, cudaStream_t st);

}  // namespace tb200
