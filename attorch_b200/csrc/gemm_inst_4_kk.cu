// Instantiates the tcgen05 GEMM kernels for 4-byte elements, A K-major, B K-major.
#include "gemm_launch.cuh"

namespace ab200 {
int launch_tc_4_kk(const TcProblem& p, int bn, cudaStream_t stream) {
  return launch_family<4, false, false>(p, bn, stream);
}
}  // namespace ab200
