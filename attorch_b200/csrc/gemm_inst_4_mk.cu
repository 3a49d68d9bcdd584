// Instantiates the tcgen05 GEMM kernels for 4-byte elements, A MN-major, B K-major.
#include "gemm_launch.cuh"

namespace ab200 {
int launch_tc_4_mk(const TcProblem& p, int bn, cudaStream_t stream) {
  return launch_family<4, true, false>(p, bn, stream);
}
}  // namespace ab200
