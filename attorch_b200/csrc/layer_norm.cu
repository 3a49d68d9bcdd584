// Dispatch of the layer-normalisation kernels over element types, row width and alignment.
#include "layer_norm.cuh"

#include <atomic>
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

// Blocks of Kernel that one SM holds at a time (at least 1), looked up once per kernel.
template <auto Kernel>
int resident_per_sm(int threads) {
  static std::atomic<int> cached{0};
  int n = cached.load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, Kernel, threads, 0) != cudaSuccess || n < 1) n = 1;
    cached.store(n, std::memory_order_relaxed);
  }
  return n;
}

// Blocks loop over rows: the grid is what the GPU holds at a time, so that no second, partly filled wave
// follows, and in backward so that the partial rows stay few (at most kMaxBackwardPerSm blocks per SM).
constexpr int kMaxBackwardPerSm = 2;

long long grid_blocks(long long rows, int R, int per_sm) {
  const long long cap = static_cast<long long>(per_sm) * sm_count();
  const long long nb = row_blocks(rows, R);
  return nb < cap ? nb : cap;
}

constexpr long long kParamChunks = 256;   // row chunks of ln_param_grad_kernel
constexpr long long kStageBudget = 200 * 1024;   // bytes of shared memory for staged rows

template <class TIn, class TOut>
int forward_typed(const void* x, long long ldx, const void* w, const void* b, int pdt, float* mean, float* inv_std,
                  void* y, long long ldy, long long rows, int F, float eps, cudaStream_t stream) {
  const int R = group_threads(F);
  const bool vec = R > 32 && F % 8 == 0 && aligned16(x, ldx, sizeof(TIn)) && aligned16(y, ldy, sizeof(TOut));
#define AB200_LN_FWD(RR, VEC)                                                                               \
  do {                                                                                                      \
    constexpr int threads = (RR) < 256 ? 256 : (RR);                                                        \
    const long long nb =                                                                                    \
        grid_blocks(rows, RR, resident_per_sm<ln_forward_kernel<TIn, TOut, RR, VEC>>(threads));             \
    ln_forward_kernel<TIn, TOut, RR, VEC><<<static_cast<unsigned>(nb), threads, 0, stream>>>(              \
        static_cast<const TIn*>(x), ldx, w, b, pdt, mean, inv_std, static_cast<TOut*>(y), ldy, rows, F, eps); \
  } while (0)
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
                   float* bias_grad, float* workspace, long long rows, int F, int* status, cudaStream_t stream) {
  const int R = group_threads(F);
  const bool vec = R > 32 && F % 8 == 0 && aligned16(x, ldx, sizeof(TIn)) && aligned16(dy, lddy, sizeof(TDy)) &&
                   aligned16(dx, lddx, sizeof(TDx));
  const bool want_params = weight_grad != nullptr;
  const bool in_registers = want_params && F <= R * kLnCache;
  // Partial rows actually written: one per row group of the grid, or one per row chunk of the column kernel.
  long long parts = in_registers ? 0 : layer_norm_parts(rows, F);
  float* wpart = workspace;
  float* bpart = nullptr;
  int launches = 0;

  // Rows staged in shared memory by bulk copies: wide, aligned rows that the block's registers cover.
  const long long stage_bytes = static_cast<long long>(F) * (sizeof(TIn) + sizeof(TDy));
  // Rows of up to 4096 elements: 256 threads and, when each still gets three stages, two blocks per SM,
  // whose row-sum barriers then overlap; wider rows: 512 threads, one block.
  const int staged_threads = F <= 256 * kLnCache ? 256 : 512;
  const int per_sm = staged_threads == 256 && kStageBudget / 2 / stage_bytes >= 3 ? 2 : 1;
  long long stages = kStageBudget / per_sm / stage_bytes;
  if (stages > kLnMaxStages) stages = kLnMaxStages;
  const bool staged = status != nullptr && vec && F > 32 * kLnCache && F <= 512 * kLnCache && stages >= 2 &&
                      (!want_params || in_registers);
  if (staged) {
    const int smem = static_cast<int>(stages * stage_bytes);
    bool ok = true;
    // The grid is the number of blocks the GPU holds at a time (asked of the runtime after the kernel has been
    // given its shared memory): a block that had to wait for an SM would double the run time.
#define AB200_LN_STAGED(RR, PAR)                                                                                  \
  do {                                                                                                            \
    auto kernel = ln_backward_staged_kernel<TIn, TDy, TDx, RR, PAR>;                                              \
    int fit = 0;                                                                                                  \
    ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&        \
         cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,                             \
                              cudaSharedmemCarveoutMaxShared) == cudaSuccess &&                                   \
         cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fit, kernel, RR, smem) == cudaSuccess && fit >= 1;        \
    if (ok) {                                                                                                     \
      const long long cap = static_cast<long long>(fit < per_sm ? fit : per_sm) * sm_count();                     \
      const long long nb = rows < cap ? rows : cap;                                                               \
      if (want_params) parts = nb;                                                                                \
      bpart = bias_grad != nullptr ? workspace + parts * F : nullptr;                                             \
      kernel<<<static_cast<unsigned>(nb), RR, smem, stream>>>(                                                    \
          static_cast<const TDy*>(dy), lddy, static_cast<const TIn*>(x), ldx, mean, inv_std, w, pdt,                \
          static_cast<TDx*>(dx), lddx, wpart, bpart, rows, F, static_cast<int>(stages), status);                  \
    }                                                                                                             \
  } while (0)
    if (staged_threads == 512 && want_params) AB200_LN_STAGED(512, true);
    else if (staged_threads == 512) AB200_LN_STAGED(512, false);
    else if (want_params) AB200_LN_STAGED(256, true);
    else AB200_LN_STAGED(256, false);
#undef AB200_LN_STAGED
    if (!ok || cudaGetLastError() != cudaSuccess) return ERR_LAUNCH;
    ++launches;
    if (!want_params) return launches;
    ln_param_finish_kernel<<<dim3((F + kLnFinishCols - 1) / kLnFinishCols, 2), kLnFinishCols * kLnFinishSlices, 0, stream>>>(wpart, bpart, static_cast<int>(parts), F,
                                                                        weight_grad, bias_grad);
    ++launches;
    return cudaGetLastError() == cudaSuccess ? launches : ERR_LAUNCH;
  }
#define AB200_LN_BWD(RR, VEC, PAR)                                                                          \
  do {                                                                                                      \
    constexpr int threads = (RR) < 256 ? 256 : (RR);                                                        \
    int per_sm = resident_per_sm<ln_backward_kernel<TIn, TDy, TDx, RR, VEC, PAR>>(threads);                 \
    if (per_sm > kMaxBackwardPerSm) per_sm = kMaxBackwardPerSm;                                             \
    const long long nb = grid_blocks(rows, RR, per_sm);                                                     \
    if (PAR) parts = nb * (threads / (RR));                                                                 \
    bpart = bias_grad != nullptr ? workspace + parts * F : nullptr;                                         \
    ln_backward_kernel<TIn, TDy, TDx, RR, VEC, PAR><<<static_cast<unsigned>(nb), threads, 0, stream>>>(    \
        static_cast<const TDy*>(dy), lddy, static_cast<const TIn*>(x), ldx, mean, inv_std, w, pdt,            \
        static_cast<TDx*>(dx), lddx, wpart, bpart, rows, F);                                                \
  } while (0)
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
  ln_param_finish_kernel<<<dim3((F + kLnFinishCols - 1) / kLnFinishCols, 2), kLnFinishCols * kLnFinishSlices, 0, stream>>>(wpart, bpart, static_cast<int>(parts), F,
                                                                      weight_grad, bias_grad);
  ++launches;
  return cudaGetLastError() == cudaSuccess ? launches : ERR_LAUNCH;
}

}  // namespace

long long layer_norm_parts(long long rows, long long F) {
  if (rows <= 0 || F <= 0) return 0;
  const int R = group_threads(static_cast<int>(F));
  if (F > static_cast<long long>(R) * kLnCache) return rows < kParamChunks ? rows : kParamChunks;
  return grid_blocks(rows, R, kMaxBackwardPerSm) * (R < 256 ? 256 / R : 1);     // an upper bound
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
                               int dydt, int xdt, int dxdt, int* status, cudaStream_t stream) {
#define AB200_LN(TI, TG, TD)                                                                                   \
  return backward_typed<TI, TG, TD>(dy, lddy, x, ldx, mean, inv_std, w, pdt, dx, lddx, weight_grad, bias_grad, \
                                    workspace, rows, F, status, stream)
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
