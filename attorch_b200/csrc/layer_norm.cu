// Dispatch of the layer-normalisation kernels over element types, row width and alignment.
#include "layer_norm.cuh"

#include <cstdint>

#include "gemm_launch.cuh"
#include "layer_norm_launch.cuh"

namespace ab200 {
namespace {

// Threads that share one row.
int group_threads(int F) { return F <= 32 * kLnCache ? 32 : (F <= 256 * kLnCache ? 256 : 512); }

bool aligned16(const void* p, long long ld, int elt) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld * elt) % 16 == 0;
}

long long row_blocks(long long rows, int R) {
  const int per_block = R < 256 ? 256 / R : 1;
  return (rows + per_block - 1) / per_block;
}

// Blocks of the backward grid: at most two per SM, so that the partial rows stay few.
long long backward_blocks(long long rows, int R) {
  const long long cap = 2ll * sm_count();
  const long long nb = row_blocks(rows, R);
  return nb < cap ? nb : cap;
}

constexpr long long kParamChunks = 256;   // row chunks of ln_param_grad_kernel

template <class TIn, class TOut>
int forward_typed(const void* x, long long ldx, const void* w, const void* b, int pdt, float* mean, float* inv_std,
                  void* y, long long ldy, long long rows, int F, float eps, cudaStream_t stream) {
  const int R = group_threads(F);
  const bool vec = R > 32 && F % 8 == 0 && aligned16(x, ldx, sizeof(TIn)) && aligned16(y, ldy, sizeof(TOut));
  long long nb = row_blocks(rows, R);
  const long long cap = 8ll * sm_count();
  if (nb > cap) nb = cap;
#define AB200_LN_FWD(RR, VEC)                                                                              \
  ln_forward_kernel<TIn, TOut, RR, VEC><<<static_cast<unsigned>(nb), (RR) < 256 ? 256 : (RR), 0, stream>>>( \
      static_cast<const TIn*>(x), ldx, w, b, pdt, mean, inv_std, static_cast<TOut*>(y), ldy, rows, F, eps)
  if (R == 32) AB200_LN_FWD(32, false);
  else if (R == 256 && vec) AB200_LN_FWD(256, true);
  else if (R == 256) AB200_LN_FWD(256, false);
  else if (vec) AB200_LN_FWD(512, true);
  else AB200_LN_FWD(512, false);
#undef AB200_LN_FWD
  return cudaGetLastError() == cudaSuccess ? 1 : ERR_LAUNCH;
}

template <class TIn, class TDy, class TDx>
int backward_typed(const void* dy, long long lddy, const void* x, long long ldx, const float* mean,
                   const float* inv_std, const void* w, int pdt, void* dx, long long lddx, float* weight_grad,
                   float* bias_grad, float* workspace, long long rows, int F, cudaStream_t stream) {
  const int R = group_threads(F);
  const bool vec = R > 32 && F % 8 == 0 && aligned16(x, ldx, sizeof(TIn)) && aligned16(dy, lddy, sizeof(TDy)) &&
                   aligned16(dx, lddx, sizeof(TDx));
  const bool want_params = weight_grad != nullptr;
  const bool in_registers = want_params && F <= R * kLnCache;
  const long long nb = backward_blocks(rows, R);
  const long long parts = layer_norm_parts(rows, F);
  float* wpart = workspace;
  float* bpart = bias_grad != nullptr ? workspace + parts * F : nullptr;
  int launches = 0;
#define AB200_LN_BWD(RR, VEC, PAR)                                                                          \
  ln_backward_kernel<TIn, TDy, TDx, RR, VEC, PAR>                                                           \
      <<<static_cast<unsigned>(nb), (RR) < 256 ? 256 : (RR), 0, stream>>>(                                  \
          static_cast<const TDy*>(dy), lddy, static_cast<const TIn*>(x), ldx, mean, inv_std, w, pdt,          \
          static_cast<TDx*>(dx), lddx, wpart, bpart, rows, F)
#define AB200_LN_BWD_P(RR, VEC)          \
  do {                                   \
    if (in_registers) AB200_LN_BWD(RR, VEC, true); \
    else AB200_LN_BWD(RR, VEC, false);   \
  } while (0)
  if (R == 32) AB200_LN_BWD_P(32, false);
  else if (R == 256 && vec) AB200_LN_BWD_P(256, true);
  else if (R == 256) AB200_LN_BWD_P(256, false);
  else if (vec) AB200_LN_BWD_P(512, true);
  else AB200_LN_BWD_P(512, false);
#undef AB200_LN_BWD_P
#undef AB200_LN_BWD
  ++launches;
  if (cudaGetLastError() != cudaSuccess) return ERR_LAUNCH;
  if (!want_params) return launches;
  if (!in_registers) {
    const long long per_chunk = (rows + parts - 1) / parts;
    ln_param_grad_kernel<TIn, TDy><<<dim3((F + 255) / 256, static_cast<unsigned>(parts)), 256, 0, stream>>>(
        static_cast<const TDy*>(dy), lddy, static_cast<const TIn*>(x), ldx, mean, inv_std, wpart, bpart, rows, F,
        per_chunk);
    ++launches;
    if (cudaGetLastError() != cudaSuccess) return ERR_LAUNCH;
  }
  ln_param_finish_kernel<<<dim3((F + 255) / 256, 2), 256, 0, stream>>>(wpart, bpart, static_cast<int>(parts), F,
                                                                      weight_grad, bias_grad);
  ++launches;
  return cudaGetLastError() == cudaSuccess ? launches : ERR_LAUNCH;
}

}  // namespace

long long layer_norm_parts(long long rows, long long F) {
  if (rows <= 0 || F <= 0) return 0;
  const int R = group_threads(static_cast<int>(F));
  if (F > static_cast<long long>(R) * kLnCache) return rows < kParamChunks ? rows : kParamChunks;
  return backward_blocks(rows, R) * (R < 256 ? 256 / R : 1);
}

int launch_layer_norm_forward(const void* x, long long ldx, const void* w, const void* b, int pdt, float* mean,
                              float* inv_std, void* y, long long ldy, long long rows, int F, int xdt, int ydt,
                              float eps, cudaStream_t stream) {
#define AB200_LN(TI, TO) \
  return forward_typed<TI, TO>(x, ldx, w, b, pdt, mean, inv_std, y, ldy, rows, F, eps, stream)
  if (xdt == DT_F32 && ydt == DT_F32) AB200_LN(float, float);
  if (xdt == DT_F16 && ydt == DT_F16) AB200_LN(__half, __half);
  if (xdt == DT_BF16 && ydt == DT_BF16) AB200_LN(__nv_bfloat16, __nv_bfloat16);
  if (xdt == DT_F16 && ydt == DT_F32) AB200_LN(__half, float);
  if (xdt == DT_BF16 && ydt == DT_F32) AB200_LN(__nv_bfloat16, float);
  if (xdt == DT_F32 && ydt == DT_F16) AB200_LN(float, __half);
  if (xdt == DT_F32 && ydt == DT_BF16) AB200_LN(float, __nv_bfloat16);
#undef AB200_LN
  return ERR_BAD_DTYPE;
}

int launch_layer_norm_backward(const void* dy, long long lddy, const void* x, long long ldx, const float* mean,
                               const float* inv_std, const void* w, int pdt, void* dx, long long lddx,
                               float* weight_grad, float* bias_grad, float* workspace, long long rows, int F,
                               int dydt, int xdt, int dxdt, cudaStream_t stream) {
#define AB200_LN(TI, TG, TD)                                                                                   \
  return backward_typed<TI, TG, TD>(dy, lddy, x, ldx, mean, inv_std, w, pdt, dx, lddx, weight_grad, bias_grad, \
                                    workspace, rows, F, stream)
  if (xdt == DT_F32 && dydt == DT_F32 && dxdt == DT_F32) AB200_LN(float, float, float);
  if (xdt == DT_F16 && dydt == DT_F16 && dxdt == DT_F16) AB200_LN(__half, __half, __half);
  if (xdt == DT_BF16 && dydt == DT_BF16 && dxdt == DT_BF16) AB200_LN(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  if (xdt == DT_F16 && dydt == DT_F32 && dxdt == DT_F32) AB200_LN(__half, float, float);
  if (xdt == DT_BF16 && dydt == DT_F32 && dxdt == DT_F32) AB200_LN(__nv_bfloat16, float, float);
  if (xdt == DT_F32 && dydt == DT_F16 && dxdt == DT_F32) AB200_LN(float, __half, float);
  if (xdt == DT_F32 && dydt == DT_BF16 && dxdt == DT_F32) AB200_LN(float, __nv_bfloat16, float);
#undef AB200_LN
  return ERR_BAD_DTYPE;
}

}  // namespace ab200
