#include "gemm_tc.cuh"
#include "common.cuh"
namespace tb200 {
bool tc_gemm_supported(const TcGemmArgs&, int) { return false; }
int launch_gemm_tc(const TcGemmArgs&, int, cudaStream_t) {
  set_error("gemm_tc: not built");
  return TB200_ERR_UNSUPPORTED;
}
}  // namespace tb200
