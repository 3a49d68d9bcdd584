// Host-side launchers of the layer-normalisation kernels (layer_norm.cu); arguments are validated by the
// C-ABI functions that call them.
#pragma once
#include <cuda_runtime.h>

namespace ab200 {

// Number of partial rows ([parts, F] floats each for weight and bias gradient) that the backward pass of
// a [rows, F] problem writes.
long long layer_norm_parts(long long rows, long long F);

// Both return the number of kernels launched, or a negative Status.  status: device word for a bounded wait
// that ran out, or NULL (then rows are not staged in shared memory).
int launch_layer_norm_forward(const void* x, long long ldx, const void* w, const void* b, int param_dtype,
                              float* mean, float* inv_std, void* y, long long ldy, long long rows, int F,
                              int x_dtype, int y_dtype, float eps, cudaStream_t stream);
int launch_layer_norm_backward(const void* dy, long long lddy, const void* x, long long ldx, const float* mean,
                               const float* inv_std, const void* w, int param_dtype, void* dx, long long lddx,
                               float* weight_grad, float* bias_grad, float* workspace, long long rows, int F,
                               int dy_dtype, int x_dtype, int dx_dtype, int* status, cudaStream_t stream);

}  // namespace ab200
