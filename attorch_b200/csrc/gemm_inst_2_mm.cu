// Instantiates the tcgen05 GEMM kernels for 2-byte elements, A MN-major, B MN-major.
#include "gemm_launch.cuh"

namespace ab200 {
int launch_tc_2_mm(const TcProblem& p, int bn, cudaStream_t stream) {
  return launch_family<2, true, true>(p, bn, stream);
}
}  // namespace ab200
