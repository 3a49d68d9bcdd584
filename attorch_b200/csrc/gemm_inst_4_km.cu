// Instantiates the tcgen05 GEMM kernels for 4-byte elements, A K-major, B MN-major.
#include "gemm_launch.cuh"

namespace ab200 {
int launch_tc_4_km(const TcProblem& p, int bn, cudaStream_t stream) {
  return launch_family<4, false, true>(p, bn, stream);
}
}  // namespace ab200
