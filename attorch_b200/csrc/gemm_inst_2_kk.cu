// Instantiates the tcgen05 GEMM kernels for 2-byte elements, A K-major, B K-major.
#include "gemm_launch.cuh"

namespace ab200 {
int launch_tc_2_kk(const TcProblem& p, int bn, cudaStream_t stream) {
  return launch_family<2, false, false>(p, bn, stream);
}
}  // namespace ab200
