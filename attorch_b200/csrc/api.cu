// C-ABI entry points of libattorch_b200.so (declared in include/attorch_b200.h): argument checks,
// kernel selection, TMA tensor-map construction and launches.  No torch types, no allocation.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "../../include/attorch_b200.h"
#include "common.cuh"
#include "gemm_launch.cuh"
#include "kernels_misc.cuh"
#include "act_elementwise.cuh"
#include "glu.cuh"
#include "cross_entropy.cuh"
#include "layer_norm_launch.cuh"

namespace ab200 {

int launch_hybrid_finish(const GemmArgs& g, int first_tile, int count, int workers, int tile_m, int bn,
                         cudaStream_t stream) {
  HybridFinishArgs a{};
  a.partial = g.partial;
  a.first_tile = first_tile; a.tail_tiles = count; a.workers = workers; a.k_blocks = g.k_blocks;
  a.tiles_m = g.tiles_m; a.tiles_n = g.tiles_n; a.group_m = g.group_m;
  a.tile_m = tile_m; a.bn = bn;
  a.M = g.M; a.N = g.N;
  a.bias = g.bias; a.bias_dtype = g.bias_dtype;
  a.aux = g.aux; a.ld_aux = g.ld_aux;
  a.out = g.out; a.ld_out = g.ld_out; a.out_dtype = g.out_dtype;
  a.act = g.act; a.act_param = g.act_param; a.save_grad = g.save_grad; a.grad_dtype = g.grad_dtype;
  a.residual = g.residual; a.ld_res = g.ld_res;
  // 16 blocks per tile: enough parallelism for a handful of tiles.
  hybrid_finish_kernel<<<dim3(count, 16), 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}

namespace {

thread_local int g_last_path = 0;
std::atomic<int64_t> g_launches{0};   // all host threads: backward runs on autograd's threads

bool valid_dtype(int dt) { return dt == DT_F32 || dt == DT_F16 || dt == DT_BF16; }
bool valid_act(int act) { return act >= 0 && act < ACT_COUNT; }
bool valid_backward_act(int act) { return valid_act(act) || act == ACT_SAVED_DERIVATIVE || act == ACT_SAVED_DERIVATIVE_F16; }

// Can TMA address this matrix: unit inner stride, 16-byte aligned base and row pitch?
bool tma_ok(const void* p, long long pitch_elems, long long unit_stride, int elt) {
  if (unit_stride != 1) return false;
  if (reinterpret_cast<uintptr_t>(p) & 15) return false;
  if (pitch_elems <= 0 || (pitch_elems * elt) % 16 != 0) return false;
  return true;
}

// A forward pass with at most 128 rows is a stream of W through the SMs, bound by HBM.  When W is wide
// enough that its 256-column blocks give at least 60 % of the SMs one whole tile each, that single
// wave of whole tiles (fused epilogue, no workspace, X re-read once per 256 columns) is the fastest
// schedule measured: 76-81 us for M = 8 ... 128 on 8192 -> 28672 fp16 (6.0-6.2 TB/s), against 90-137 us
// for the swap-AB stream-K kernel, which stays for narrower outputs and for fewer than 8 rows (86 us;
// whole tiles take 97 us there, and 82 us when the CTAs start at spread-out k-blocks: not understood).
bool few_rows_wide_output(long long M, long long N) {
  return M >= 8 && M <= 128 && ((N + 255) / 256) * 10 >= static_cast<long long>(sm_count()) * 6;
}

// Widest tile that still gives every SM work; otherwise the narrowest that covers N.
int pick_bn(long long M, long long N) {
  const long long tm = (M + 127) / 128;
  const int sms = sm_count();
  if (few_rows_wide_output(M, N)) return 256;
  if (N > 128 && tm * ((N + 255) / 256) >= sms) return 256;
  if (N > 64 && tm * ((N + 127) / 128) >= sms) return 128;
  if (N > 128) return 256;
  if (N > 64) return 128;
  if (N > 32) return 64;
  return 32;
}

int launch_any(const AnyGemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return OK;
  dim3 grid((a.N + 63) / 64, (a.M + 63) / 64);
  gemm_any_kernel<<<grid, 256, 0, stream>>>(a);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}

bool fits_int(int64_t v) { return v >= 0 && v < (1ll << 31); }

// CTA pairs (cta_group::2) are used unless the call's flags or AB200_CTA_PAIR=0 say otherwise.
bool pair_allowed(int flags) {
  static const bool env_on = []() {
    const char* e = std::getenv("AB200_CTA_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  return env_on && !(flags & AB200_FLAG_NO_PAIR);
}

int launch_tc_counted(const TcProblem& p, int bn, cudaStream_t stream) {
  const int rc = launch_tc(p, bn, stream);
  if (rc == OK) ++g_launches;
  return rc;
}

int launch_finish(float* partial, const GemmArgs& e, long long M, long long N, cudaStream_t stream) {
  const long long total = M * N;
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  streamk_finish_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      partial, N, static_cast<int>(M), static_cast<int>(N), e.bias, e.bias_dtype, e.aux, e.ld_aux, e.out,
      e.ld_out, e.out_dtype, e.act, e.act_param, e.save_grad, e.grad_dtype, e.residual, e.ld_res);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}

// Should a GEMM with this output and reduction length be run as equal (tile, k-block) ranges over
// all SMs instead of whole tiles?  Yes when whole tiles would leave at least half of the SMs idle
// and the reduction is long enough to share: every CTA then still gets at least 4 k-blocks.
bool want_split(long long rows, long long cols, long long reduction, int elt) {
  const int bn = pick_bn(rows, cols);
  const long long tiles = ((rows + 127) / 128) * ((cols + bn - 1) / bn);
  const long long k_blocks = (reduction + 128 / elt - 1) / (128 / elt);
  const int sms = sm_count();
  return tiles * 2 <= sms && tiles * k_blocks >= 4ll * sms;
}

// Runs p as whole tiles with the fused epilogue, or, if the shape calls for it and the caller
// supplied enough workspace, as stream-K partial sums plus the finishing kernel.  p.g holds the
// epilogue in both cases.
int run_tiles_or_split(TcProblem& p, void* workspace, int64_t workspace_bytes, cudaStream_t stream,
                       int flags) {
  GemmArgs& g = p.g;
  p.allow_pair = pair_allowed(flags);
  p.allow_tma_store = !(flags & AB200_FLAG_NO_TMA_STORE);
  p.reserve_sms = (flags >> AB200_FLAG_RESERVE_SMS_SHIFT) & 0xFF;
  const int bn = pick_bn(g.M, g.N);
  const int64_t need = static_cast<int64_t>(g.M) * g.N * 4;
  if (want_split(g.M, g.N, g.K, dtype_size(p.op_dtype)) && workspace != nullptr && workspace_bytes >= need) {
    if (cudaMemsetAsync(workspace, 0, need, stream) != cudaSuccess) return ERR_LAUNCH;
    g.stream_k = 1;
    g.partial = static_cast<float*>(workspace);
    g.ld_partial = g.N;
    g.partial_transposed = 0;
    g_last_path = AB200_PATH_STREAMK;
    const int rc = launch_tc_counted(p, bn, stream);
    if (rc != OK) return rc;
    return launch_finish(g.partial, g, g.M, g.N, stream);
  }
  g.stream_k = 0;
  // Scratch for sharing out a mostly idle last round of tiles (summed in a fixed order).
  if (!(flags & AB200_FLAG_WHOLE_TILES)) {
    p.tail_workspace = workspace;
    p.tail_workspace_bytes = workspace_bytes;
    p.allow_split_tail = true;
  }
  g_last_path = AB200_PATH_TCGEN05;
  return launch_tc_counted(p, bn, stream);
}

}  // namespace
}  // namespace ab200

using namespace ab200;

extern "C" {

int ab200_version(void) { return 1000; }

const char* ab200_error_string(int code) {
  switch (code) {
    case OK: return "ok";
    case ERR_NULL_POINTER: return "a required pointer is NULL";
    case ERR_BAD_SHAPE: return "negative or inconsistent shape";
    case ERR_BAD_DTYPE: return "unsupported element type";
    case ERR_BAD_ACT: return "unknown activation id";
    case ERR_BAD_STRIDE: return "operand strides or alignment not addressable by the requested kernel";
    case ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case ERR_TENSOR_MAP: return "cuTensorMapEncodeTiled rejected the operand";
    case ERR_LAUNCH: return "kernel launch failed";
    case ERR_TOO_LARGE: return "a dimension exceeds 2^31 - 1";
    case ERR_DRIVER: return "CUDA driver entry point or symbol address unavailable";
    case ERR_BAD_PROBABILITY: return "dropout probability outside [0, 1]";
    case ERR_STATIC_SCRATCH_TOO_SMALL:
      return "shape needs more scratch than the built-in array of ab200_act_backward_static holds";
    case DEV_TIMEOUT_PRODUCER: return "device: TMA producer gave up waiting for a free stage";
    case DEV_TIMEOUT_MMA: return "device: MMA issuer gave up waiting for operands or an accumulator";
    case DEV_TIMEOUT_EPILOGUE: return "device: epilogue gave up waiting for an accumulator";
    case DEV_TIMEOUT_COLLECTIVE: return "device: all-reduce gave up waiting for another rank";
    case DEV_TIMEOUT_ROW_COPY: return "device: layer normalisation gave up waiting for a row copy into shared memory";
    default: return "unknown code";
  }
}

int ab200_last_path(void) { return g_last_path; }
int ab200_last_schedule(void) { return last_schedule(); }
int ab200_set_gemm_cta_limit(int ctas) {
  const int previous = gemm_cta_limit();
  set_gemm_cta_limit(ctas);
  return previous;
}
int64_t ab200_launch_count(void) { return g_launches.load(); }

int64_t ab200_forward_workspace_bytes(int64_t M, int64_t K, int64_t N, int flags) {
  if (M <= 0 || N <= 0) return 0;
  if ((M <= 128 && !few_rows_wide_output(M, N) && !(flags & AB200_FLAG_NO_STREAMK)) ||
      (flags & AB200_FLAG_FORCE_STREAMK))
    return M * N * 4;
  // One wave of whole tiles: nothing to share out, no scratch.
  if (few_rows_wide_output(M, N) && (N + 255) / 256 <= sm_count()) return 0;
  return ab200_gemm_workspace_bytes(M, N, K);
}

int64_t ab200_gemm_workspace_bytes(int64_t rows, int64_t cols, int64_t reduction) {
  if (rows <= 0 || cols <= 0 || reduction <= 0) return 0;
  // The narrower element type gives the fewer k-blocks; a caller that sizes for it is safe for both.
  int64_t need = (want_split(rows, cols, reduction, 2) || want_split(rows, cols, reduction, 4)) ? rows * cols * 4 : 0;
  // Sharing out a partial last round of 256 x 256 (pair) or 128 x 256 tiles: fewer tiles than workers.
  const int64_t tiles = ((rows + 127) / 128) * ((cols + 255) / 256);
  const int64_t tail = 2 * static_cast<int64_t>(sm_count()) * 128 * 256 * 4;   // two slots per worker
  if (tiles > sm_count() / 2 && reduction >= 1024 && tail > need) need = tail;
  return need;
}

int ab200_linear_forward(const void* x, const void* w, const void* bias, void* pre_act, void* out,
                         int64_t M, int64_t K, int64_t N, int64_t x_stride_m, int64_t x_stride_k,
                         int64_t w_stride_k, int64_t w_stride_n, int64_t ld_pre, int64_t ld_out,
                         int op_dtype, int out_dtype, int bias_dtype, int act, float act_param,
                         void* workspace, int64_t workspace_bytes, int* status, void* stream_,
                         int flags) {
  return ab200_linear_forward_residual(x, w, bias, pre_act, out, nullptr, M, K, N, x_stride_m, x_stride_k,
                                       w_stride_k, w_stride_n, ld_pre, ld_out, 0, op_dtype, out_dtype,
                                       bias_dtype, act, act_param, workspace, workspace_bytes, status, stream_,
                                       flags);
}

int ab200_linear_forward_residual(const void* x, const void* w, const void* bias, void* pre_act, void* out,
                                  const void* residual, int64_t M, int64_t K, int64_t N, int64_t x_stride_m,
                                  int64_t x_stride_k, int64_t w_stride_k, int64_t w_stride_n, int64_t ld_pre,
                                  int64_t ld_out, int64_t ld_res, int op_dtype, int out_dtype, int bias_dtype,
                                  int act, float act_param, void* workspace, int64_t workspace_bytes,
                                  int* status, void* stream_, int flags) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || K < 0 || N < 0) return ERR_BAD_SHAPE;
  if (residual != nullptr && ld_res < N) return ERR_BAD_STRIDE;
  if (!fits_int(M) || !fits_int(K) || !fits_int(N)) return ERR_TOO_LARGE;
  if (!valid_dtype(op_dtype) || !valid_dtype(out_dtype) || (bias && !valid_dtype(bias_dtype)))
    return ERR_BAD_DTYPE;
  if (!valid_act(act)) return ERR_BAD_ACT;
  if (M == 0 || N == 0) return OK;
  if (!out || (K > 0 && (!x || !w))) return ERR_NULL_POINTER;
  if (ld_out < N || (pre_act && ld_pre < N)) return ERR_BAD_STRIDE;
  const int save_grad = (flags & AB200_FLAG_SAVE_DERIVATIVE) && act != ACT_NONE ? 1 : 0;
  // The saved derivative of a bf16 layer may be stored as fp16 (same size, three more mantissa bits;
  // activation derivatives are of order one, far inside fp16's range): the product dY * act'(Z) then
  // differs from one formed with the unrounded derivative by 1 part in 4000 instead of 1 in 500.
  const int grad_dtype = (save_grad && out_dtype == DT_BF16 && (flags & AB200_FLAG_DERIVATIVE_FP16)) ? DT_F16 : out_dtype;

  const int elt = dtype_size(op_dtype);
  const bool tc_ok = K > 0 && tma_ok(x, x_stride_m, x_stride_k, elt) && tma_ok(w, w_stride_k, w_stride_n, elt) &&
                     x_stride_m >= K && w_stride_k >= N;
  if ((flags & AB200_FLAG_FORCE_TCGEN05) && !tc_ok) return ERR_BAD_STRIDE;
  const bool use_tc = tc_ok && !(flags & AB200_FLAG_FORCE_GENERIC) && status != nullptr;

  if (!use_tc) {
    AnyGemmArgs a{};
    a.a = x; a.sam = x_stride_m; a.sak = x_stride_k; a.a_dtype = op_dtype;
    a.b = w; a.sbk = w_stride_k; a.sbn = w_stride_n; a.b_dtype = op_dtype;
    a.M = static_cast<int>(M); a.N = static_cast<int>(N); a.K = static_cast<int>(K);
    a.out = out; a.ld_out = ld_out; a.out_dtype = out_dtype;
    a.aux = pre_act; a.ld_aux = ld_pre;
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.act = act; a.act_param = act_param;
    a.save_grad = save_grad;
    a.grad_dtype = grad_dtype;
    a.residual = residual; a.ld_res = ld_res;
    g_last_path = AB200_PATH_GENERIC;
    return launch_any(a, stream);
  }

  TcProblem p{};
  p.op_dtype = op_dtype;
  GemmArgs& g = p.g;
  g.status = status;
  const bool skinny = ((M <= 128 && !few_rows_wide_output(M, N) && !(flags & AB200_FLAG_NO_STREAMK)) ||
                       (flags & AB200_FLAG_FORCE_STREAMK));
  if (skinny) {
    // Swap-AB: D'[N, M] = W^T[N, K] * X^T[K, M].  A = W (MN-major), B = X (K-major).  The fp32
    // partial sums land in workspace as [M, N] (coalesced along N) and a finishing kernel applies
    // bias and activation.
    const int64_t need = M * N * 4;
    if (workspace == nullptr || workspace_bytes < need) return ERR_WORKSPACE_TOO_SMALL;
    if (cudaMemsetAsync(workspace, 0, need, stream) != cudaSuccess) return ERR_LAUNCH;
    p.a = w; p.a_mn = true; p.a_pitch = w_stride_k;
    p.b = x; p.b_mn = false; p.b_pitch = x_stride_m;
    g.M = static_cast<int>(N); g.N = static_cast<int>(M); g.K = static_cast<int>(K);
    g.stream_k = 1;
    g.partial = static_cast<float*>(workspace);
    g.ld_partial = N;
    g.partial_transposed = 1;
    const int bn = M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256));
    g_last_path = AB200_PATH_STREAMK;
    int rc = launch_tc_counted(p, bn, stream);
    if (rc != OK) return rc;
    GemmArgs e{};
    e.bias = bias; e.bias_dtype = bias_dtype; e.aux = pre_act; e.ld_aux = ld_pre;
    e.out = out; e.ld_out = ld_out; e.out_dtype = out_dtype; e.act = act; e.act_param = act_param;
    e.save_grad = save_grad;
    e.grad_dtype = grad_dtype;
    e.residual = residual; e.ld_res = ld_res;
    return launch_finish(static_cast<float*>(workspace), e, M, N, stream);
  }

  p.a = x; p.a_mn = false; p.a_pitch = x_stride_m;
  p.b = w; p.b_mn = true; p.b_pitch = w_stride_k;
  g.M = static_cast<int>(M); g.N = static_cast<int>(N); g.K = static_cast<int>(K);
  g.out = out; g.ld_out = ld_out; g.out_dtype = out_dtype;
  g.aux = pre_act; g.ld_aux = ld_pre;
  g.bias = bias; g.bias_dtype = bias_dtype;
  g.act = act; g.act_param = act_param;
  g.save_grad = save_grad;
  g.grad_dtype = grad_dtype;
  g.residual = residual; g.ld_res = ld_res;
  return run_tiles_or_split(p, workspace, workspace_bytes, stream, flags);
}

int ab200_gated_linear_forward(const void* x, const void* w, const void* bias, void* pre_act, void* out, int64_t M,
                               int64_t K, int64_t H, int64_t x_stride_m, int64_t x_stride_k, int64_t w_stride_k,
                               int64_t w_stride_n, int64_t ld_pre, int64_t ld_out, int op_dtype, int out_dtype,
                               int bias_dtype, int act, float act_param, int* status, void* stream_, int flags) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || K < 0 || H < 0) return ERR_BAD_SHAPE;
  if (!fits_int(M) || !fits_int(K) || !fits_int(2 * H)) return ERR_TOO_LARGE;
  if (!valid_dtype(op_dtype) || !valid_dtype(out_dtype) || (bias && !valid_dtype(bias_dtype))) return ERR_BAD_DTYPE;
  if (!valid_act(act)) return ERR_BAD_ACT;
  if (M == 0 || H == 0) return OK;
  if (!out || !x || !w || !status) return ERR_NULL_POINTER;
  if (ld_out < H || (pre_act && ld_pre < 2 * H)) return ERR_BAD_STRIDE;
  const int elt = dtype_size(op_dtype);
  // Tensor-core path only: operands TMA can address, a reduction, and a second half that starts on a
  // 16-byte boundary in W, in the saved pre-activation and in the bias.
  if (K <= 0 || !tma_ok(x, x_stride_m, x_stride_k, elt) || !tma_ok(w, w_stride_k, w_stride_n, elt) ||
      x_stride_m < K || w_stride_k < 2 * H || (H * elt) % 16 != 0 || (H * dtype_size(out_dtype)) % 16 != 0)
    return ERR_BAD_STRIDE;
  TcProblem p{};
  p.op_dtype = op_dtype;
  p.a = x; p.a_mn = false; p.a_pitch = x_stride_m;
  p.b = w; p.b_mn = true; p.b_pitch = w_stride_k;
  p.allow_pair = pair_allowed(flags);
  p.allow_tma_store = !(flags & AB200_FLAG_NO_TMA_STORE);
  p.reserve_sms = (flags >> AB200_FLAG_RESERVE_SMS_SHIFT) & 0xFF;
  GemmArgs& g = p.g;
  g.status = status;
  g.M = static_cast<int>(M); g.N = static_cast<int>(H); g.K = static_cast<int>(K);
  g.gate_cols = static_cast<int>(H);
  g.out = out; g.ld_out = ld_out; g.out_dtype = out_dtype; g.grad_dtype = out_dtype;
  g.aux = pre_act; g.ld_aux = ld_pre;
  g.bias = bias; g.bias_dtype = bias_dtype;
  g.act = act; g.act_param = act_param;
  g.stream_k = 0;
  g_last_path = AB200_PATH_TCGEN05;
  return launch_tc_counted(p, 256, stream);
}

extern "C++" {
namespace {
// Rows per block of act_backward_kernel for an M x N problem whose blocks are cols_per_block wide:
// kActRows, or more where that makes the grid a whole number of waves of resident blocks (a grid of
// 1.7 waves costs as much as one of 2).  Never fewer, so ceil(M / kActRows) partial rows always suffice.
int act_rows_per_block(int64_t M, int64_t N, int cols_per_block) {
  static const int resident = []() {
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, act_backward_kernel<__nv_bfloat16, true, 32>, 256, 0) !=
            cudaSuccess || blocks <= 0)
      blocks = 4;
    return blocks;
  }();
  const int64_t gx = (N + cols_per_block - 1) / cols_per_block;
  const int64_t max_gy = (M + kActRows - 1) / kActRows;
  const int64_t slots = static_cast<int64_t>(sm_count()) * resident;
  const int64_t waves = gx * max_gy / slots;
  if (waves < 1) return kActRows;
  const int64_t gy = waves * slots / gx;
  if (gy < 1 || gy > max_gy) return kActRows;
  int64_t rows = (M + gy - 1) / gy;
  rows = (rows + 7) / 8 * 8;
  return static_cast<int>(rows < kActRows ? kActRows : rows);
}
}  // namespace
}  // extern "C++"

int64_t ab200_act_backward_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  return ((M + kActRows - 1) / kActRows) * N * 4;
}

int ab200_act_backward(const void* dy, const void* z, void* dz, void* db, int64_t M, int64_t N,
                       int64_t ld_dy, int64_t ld_z, int64_t ld_dz, int dtype, int db_dtype, int act,
                       float act_param, void* workspace, int64_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || N < 0) return ERR_BAD_SHAPE;
  if (!fits_int(M) || !fits_int(N)) return ERR_TOO_LARGE;
  if (!valid_dtype(dtype) || (db && !valid_dtype(db_dtype))) return ERR_BAD_DTYPE;
  if (!valid_backward_act(act)) return ERR_BAD_ACT;
  if (N == 0) return OK;
  if (M > 0 && (!dy || (act != ACT_NONE && !z))) return ERR_NULL_POINTER;
  if (dz == nullptr && db == nullptr) return OK;
  if (ld_dy < N || (z && ld_z < N) || (dz && ld_dz < N)) return ERR_BAD_STRIDE;
  const int rows_per_block = act_rows_per_block(M, N, 256);
  const int chunks = static_cast<int>((M + rows_per_block - 1) / rows_per_block);
  float* partial = nullptr;
  if (db != nullptr) {
    if (M == 0) {
      // Empty sum.
      return cudaMemsetAsync(db, 0, N * dtype_size(db_dtype), stream) == cudaSuccess ? OK : ERR_LAUNCH;
    }
    if (!workspace || workspace_bytes < ab200_act_backward_workspace_bytes(M, N)) return ERR_WORKSPACE_TOO_SMALL;
    partial = static_cast<float*>(workspace);
  }
  if (M == 0) return OK;
  const int elt = dtype_size(dtype);
  auto aligned = [&](const void* p, long long ld) {
    return p == nullptr || ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld * elt) % 16 == 0);
  };
  const bool vec = (N % 8 == 0) && aligned(dy, ld_dy) && aligned(z, ld_z) && aligned(dz, ld_dz);
  // 32 threads side by side on a row and 8 row lanes measured faster than 256 x 1 on B200 for
  // every width tried, so the wide layout is kept for experiments only.
  const bool wide = false;
  const int cols_per_block = wide ? 2048 : 256;
  dim3 grid(static_cast<unsigned>((N + cols_per_block - 1) / cols_per_block), static_cast<unsigned>(chunks));
  const int Mi = static_cast<int>(M), Ni = static_cast<int>(N);
#define AB200_LAUNCH_ACT_V(T, V, C)                                                                  \
  act_backward_kernel<T, V, C><<<grid, 256, 0, stream>>>(static_cast<const T*>(dy), ld_dy,           \
      static_cast<const T*>(z), ld_z, static_cast<T*>(dz), ld_dz, partial, Mi, Ni, act, act_param,     \
      rows_per_block)
#define AB200_LAUNCH_ACT(T)                                                  \
  do {                                                                       \
    if (vec && wide) AB200_LAUNCH_ACT_V(T, true, 256);                       \
    else if (vec) AB200_LAUNCH_ACT_V(T, true, 32);                           \
    else if (wide) AB200_LAUNCH_ACT_V(T, false, 256);                        \
    else AB200_LAUNCH_ACT_V(T, false, 32);                                   \
  } while (0)
  if (dtype == DT_F32) AB200_LAUNCH_ACT(float);
  else if (dtype == DT_F16) AB200_LAUNCH_ACT(__half);
  else AB200_LAUNCH_ACT(__nv_bfloat16);
#undef AB200_LAUNCH_ACT_V
#undef AB200_LAUNCH_ACT
  ++g_launches;
  if (cudaGetLastError() != cudaSuccess) return ERR_LAUNCH;
  if (db != nullptr) {
    colsum_finish_kernel<<<(Ni + 31) / 32, 256, 0, stream>>>(partial, chunks, Ni, db, db_dtype);
    ++g_launches;
    if (cudaGetLastError() != cudaSuccess) return ERR_LAUNCH;
  }
  return OK;
}

// ------------------------------------------------------------------------------------------------
// Activation backward for callers that must not allocate.
//
// The column-sum partials live in this file-scope device array instead of a caller-supplied
// workspace.  Every GPU that loads the library holds these 4 MiB until the process exits.  In host
// code the array's name is only a handle for cudaGetSymbolAddress; the address a kernel needs is
// looked up once per device (with that device current) and cached.
// ------------------------------------------------------------------------------------------------
constexpr int64_t kStaticScratchFloats = 1 << 20;
static __device__ __align__(256) float g_static_colsum_scratch[kStaticScratchFloats];

namespace {
constexpr int kMaxDevices = 64;
std::atomic<float*> g_static_scratch_ptr[kMaxDevices];

// Device address of g_static_colsum_scratch on the current device, or nullptr with *rc set.
float* static_scratch_for_current_device(int* rc) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *rc = ERR_LAUNCH;
    return nullptr;
  }
  float* ptr = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_static_colsum_scratch) != cudaSuccess || sym == nullptr) {
      *rc = ERR_DRIVER;
      return nullptr;
    }
    ptr = static_cast<float*>(sym);
    g_static_scratch_ptr[dev].store(ptr, std::memory_order_release);
  }
  return ptr;
}
}  // namespace

int64_t ab200_act_backward_static_max_floats(void) { return kStaticScratchFloats; }

int ab200_act_backward_static(const void* dy, const void* z, void* dz, void* db, int64_t M, int64_t N,
                              int64_t ld_dy, int64_t ld_z, int64_t ld_dz, int dtype, int db_dtype,
                              int act, float act_param, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || N < 0) return ERR_BAD_SHAPE;
  if (!fits_int(M) || !fits_int(N)) return ERR_TOO_LARGE;
  if (!valid_dtype(dtype) || (db && !valid_dtype(db_dtype))) return ERR_BAD_DTYPE;
  if (!valid_backward_act(act)) return ERR_BAD_ACT;
  if (N == 0) return OK;
  if (M > 0 && (!dy || (act != ACT_NONE && !z))) return ERR_NULL_POINTER;
  if (dz == nullptr && db == nullptr) return OK;
  if (ld_dy < N || (z && ld_z < N) || (dz && ld_dz < N)) return ERR_BAD_STRIDE;
  // One fp32 per (row block, column): reject shapes the built-in array cannot hold (by the documented
  // bound, ceil(M / 128) * N; the grid may use fewer, taller row blocks).
  if (db != nullptr && (M + kActRows - 1) / kActRows * N > kStaticScratchFloats) return ERR_STATIC_SCRATCH_TOO_SMALL;
  const int rows_per_block = act_rows_per_block(M, N, 256);
  const int64_t chunks = (M + rows_per_block - 1) / rows_per_block;
  if (M == 0) {
    if (db == nullptr) return OK;
    return cudaMemsetAsync(db, 0, N * dtype_size(db_dtype), stream) == cudaSuccess ? OK : ERR_LAUNCH;
  }
  float* partial = nullptr;
  if (db != nullptr) {
    int rc = OK;
    partial = static_scratch_for_current_device(&rc);
    if (partial == nullptr) return rc;
  }
  const int elt = dtype_size(dtype);
  auto aligned = [&](const void* p, long long ld) {
    return p == nullptr || ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld * elt) % 16 == 0);
  };
  const bool vec = (N % 8 == 0) && aligned(dy, ld_dy) && aligned(z, ld_z) && aligned(dz, ld_dz);
  dim3 grid(static_cast<unsigned>((N + 255) / 256), static_cast<unsigned>(chunks));
  const int Mi = static_cast<int>(M), Ni = static_cast<int>(N);
  // Each block overwrites its own row of partials for every column below N, and the finishing
  // kernel reads only those, so nothing left in the array by an earlier call is ever read.
#define AB200_LAUNCH_ACT_STATIC(T)                                                                     \
  do {                                                                                                 \
    if (vec)                                                                                           \
      act_backward_kernel<T, true, 32><<<grid, 256, 0, stream>>>(static_cast<const T*>(dy), ld_dy,     \
          static_cast<const T*>(z), ld_z, static_cast<T*>(dz), ld_dz, partial, Mi, Ni, act, act_param, \
          rows_per_block);                                                                             \
    else                                                                                               \
      act_backward_kernel<T, false, 32><<<grid, 256, 0, stream>>>(static_cast<const T*>(dy), ld_dy,    \
          static_cast<const T*>(z), ld_z, static_cast<T*>(dz), ld_dz, partial, Mi, Ni, act, act_param, \
          rows_per_block);                                                                             \
  } while (0)
  if (dtype == DT_F32) AB200_LAUNCH_ACT_STATIC(float);
  else if (dtype == DT_F16) AB200_LAUNCH_ACT_STATIC(__half);
  else AB200_LAUNCH_ACT_STATIC(__nv_bfloat16);
#undef AB200_LAUNCH_ACT_STATIC
  ++g_launches;
  if (cudaGetLastError() != cudaSuccess) return ERR_LAUNCH;
  if (db != nullptr) {
    colsum_finish_kernel<<<(Ni + 31) / 32, 256, 0, stream>>>(partial, static_cast<int>(chunks), Ni, db, db_dtype);
    ++g_launches;
    if (cudaGetLastError() != cudaSuccess) return ERR_LAUNCH;
  }
  return OK;
}

int ab200_linear_backward_input(const void* dz, const void* w, void* dx, int64_t M, int64_t K,
                                int64_t N, int64_t dz_stride_m, int64_t dz_stride_n,
                                int64_t w_stride_k, int64_t w_stride_n, int64_t ld_dx, int op_dtype,
                                int dx_dtype, void* workspace, int64_t workspace_bytes, int* status,
                                void* stream_, int flags) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || K < 0 || N < 0) return ERR_BAD_SHAPE;
  if (!fits_int(M) || !fits_int(K) || !fits_int(N)) return ERR_TOO_LARGE;
  if (!valid_dtype(op_dtype) || !valid_dtype(dx_dtype)) return ERR_BAD_DTYPE;
  if (M == 0 || K == 0) return OK;
  if (!dx || (N > 0 && (!dz || !w))) return ERR_NULL_POINTER;
  if (ld_dx < K) return ERR_BAD_STRIDE;
  const int elt = dtype_size(op_dtype);
  // dX[M, K] = dZ[M, N] * W^T: the reduction runs over N, contiguous in both dZ rows and W rows.
  const bool tc_ok = N > 0 && tma_ok(dz, dz_stride_m, dz_stride_n, elt) && tma_ok(w, w_stride_k, w_stride_n, elt) &&
                     dz_stride_m >= N && w_stride_k >= N;
  if ((flags & AB200_FLAG_FORCE_TCGEN05) && !tc_ok) return ERR_BAD_STRIDE;
  if (tc_ok && !(flags & AB200_FLAG_FORCE_GENERIC) && status != nullptr) {
    TcProblem p{};
    p.op_dtype = op_dtype;
    p.a = dz; p.a_mn = false; p.a_pitch = dz_stride_m;
    p.b = w; p.b_mn = false; p.b_pitch = w_stride_k;
    GemmArgs& g = p.g;
    g.status = status;
    g.M = static_cast<int>(M); g.N = static_cast<int>(K); g.K = static_cast<int>(N);
    g.out = dx; g.ld_out = ld_dx; g.out_dtype = dx_dtype;
    g.act = ACT_NONE;
    return run_tiles_or_split(p, workspace, workspace_bytes, stream, flags);
  }
  AnyGemmArgs a{};
  a.a = dz; a.sam = dz_stride_m; a.sak = dz_stride_n; a.a_dtype = op_dtype;
  a.b = w; a.sbk = w_stride_n; a.sbn = w_stride_k; a.b_dtype = op_dtype;   // B[n, k] = W[k, n]
  a.M = static_cast<int>(M); a.N = static_cast<int>(K); a.K = static_cast<int>(N);
  a.out = dx; a.ld_out = ld_dx; a.out_dtype = dx_dtype;
  a.act = ACT_NONE;
  g_last_path = AB200_PATH_GENERIC;
  return launch_any(a, stream);
}

int ab200_linear_backward_weight(const void* x, const void* dz, void* dw, int64_t M, int64_t K,
                                 int64_t N, int64_t x_stride_m, int64_t x_stride_k,
                                 int64_t dz_stride_m, int64_t dz_stride_n, int64_t ld_dw,
                                 int op_dtype, int dw_dtype, void* workspace, int64_t workspace_bytes,
                                 int* status, void* stream_, int flags) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || K < 0 || N < 0) return ERR_BAD_SHAPE;
  if (!fits_int(M) || !fits_int(K) || !fits_int(N)) return ERR_TOO_LARGE;
  if (!valid_dtype(op_dtype) || !valid_dtype(dw_dtype)) return ERR_BAD_DTYPE;
  if (K == 0 || N == 0) return OK;
  if (!dw || (M > 0 && (!x || !dz))) return ERR_NULL_POINTER;
  if (ld_dw < N) return ERR_BAD_STRIDE;
  const int elt = dtype_size(op_dtype);
  // dW[K, N] = X^T[K, M] * dZ[M, N]: the reduction runs over M, the strided dimension of both.
  const bool tc_ok = M > 0 && tma_ok(x, x_stride_m, x_stride_k, elt) && tma_ok(dz, dz_stride_m, dz_stride_n, elt) &&
                     x_stride_m >= K && dz_stride_m >= N;
  if ((flags & AB200_FLAG_FORCE_TCGEN05) && !tc_ok) return ERR_BAD_STRIDE;
  if (tc_ok && !(flags & AB200_FLAG_FORCE_GENERIC) && status != nullptr) {
    TcProblem p{};
    p.op_dtype = op_dtype;
    p.a = x; p.a_mn = true; p.a_pitch = x_stride_m;
    p.b = dz; p.b_mn = true; p.b_pitch = dz_stride_m;
    GemmArgs& g = p.g;
    g.status = status;
    g.M = static_cast<int>(K); g.N = static_cast<int>(N); g.K = static_cast<int>(M);
    g.out = dw; g.ld_out = ld_dw; g.out_dtype = dw_dtype;
    g.act = ACT_NONE;
    return run_tiles_or_split(p, workspace, workspace_bytes, stream, flags);
  }
  AnyGemmArgs a{};
  a.a = x; a.sam = x_stride_k; a.sak = x_stride_m; a.a_dtype = op_dtype;   // A[k_feat, m] = X[m, k_feat]
  a.b = dz; a.sbk = dz_stride_m; a.sbn = dz_stride_n; a.b_dtype = op_dtype;
  a.M = static_cast<int>(K); a.N = static_cast<int>(N); a.K = static_cast<int>(M);
  a.out = dw; a.ld_out = ld_dw; a.out_dtype = dw_dtype;
  a.act = ACT_NONE;
  g_last_path = AB200_PATH_GENERIC;
  return launch_any(a, stream);
}

extern "C++" {
namespace {
template <bool kBackward>
int launch_act_elementwise(const void* x, const void* dy, void* out, int64_t n, int dtype, int act,
                           float act_param, float drop_p, uint32_t seed, cudaStream_t stream, int flags) {
  if (n < 0) return ERR_BAD_SHAPE;
  if (!valid_dtype(dtype)) return ERR_BAD_DTYPE;
  if (!valid_act(act)) return ERR_BAD_ACT;
  if (!(drop_p >= 0.0f && drop_p <= 1.0f)) return ERR_BAD_PROBABILITY;
  if (n == 0) return OK;
  if (!x || !out || (kBackward && !dy)) return ERR_NULL_POINTER;
  if (drop_p == 1.0f) {
    // Every element is dropped (the uniform numbers lie in [0, 1)): the reference's
    // tl.where(random < 1, 0, ...) gives zeros in both directions (attorch/dropout_kernels.py:12-46).
    return cudaMemsetAsync(out, 0, static_cast<size_t>(n) * dtype_size(dtype), stream) == cudaSuccess ? OK : ERR_LAUNCH;
  }
  const int dropout = drop_p > 0.0f ? ((flags & AB200_FLAG_DROPOUT_PACKED) ? DROPOUT_PACKED : DROPOUT_REFERENCE)
                                    : DROPOUT_OFF;
  const uint32_t threshold = dropout ? dropout_threshold(drop_p, dropout) : 0u;
  const long long groups = (n + 7) / 8;
  long long blocks = (groups + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
#define AB200_ACT_EW(T)                                                                                 \
  act_elementwise_kernel<T, kBackward><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(              \
      static_cast<const T*>(x), static_cast<const T*>(dy), static_cast<T*>(out), n, act, act_param,     \
      drop_p, seed, dropout, threshold)
  if (dtype == DT_F32) AB200_ACT_EW(float);
  else if (dtype == DT_F16) AB200_ACT_EW(__half);
  else AB200_ACT_EW(__nv_bfloat16);
#undef AB200_ACT_EW
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}
}  // namespace
}  // extern "C++"

int ab200_act_forward(const void* x, void* y, int64_t n, int dtype, int act, float act_param, float drop_p,
                      uint32_t seed, void* stream, int flags) {
  return launch_act_elementwise<false>(x, nullptr, y, n, dtype, act, act_param, drop_p, seed,
                                       static_cast<cudaStream_t>(stream), flags);
}

int ab200_act_input_grad(const void* dy, const void* x, void* dx, int64_t n, int dtype, int act,
                         float act_param, float drop_p, uint32_t seed, void* stream, int flags) {
  return launch_act_elementwise<true>(x, dy, dx, n, dtype, act, act_param, drop_p, seed,
                                      static_cast<cudaStream_t>(stream), flags);
}

extern "C++" {
namespace {
template <bool kBackward>
int launch_glu(const void* x, const void* dy, void* out, int64_t outer, int64_t inner, int dtype, int act,
               float act_param, cudaStream_t stream) {
  if (outer < 0 || inner < 0) return ERR_BAD_SHAPE;
  if (!valid_dtype(dtype)) return ERR_BAD_DTYPE;
  if (!valid_act(act)) return ERR_BAD_ACT;
  if (outer == 0 || inner == 0) return OK;
  if (!x || !out || (kBackward && !dy)) return ERR_NULL_POINTER;
  if (outer > (1ll << 40) / (inner > 0 ? inner : 1)) return ERR_TOO_LARGE;   // 2 * outer * inner must index safely
  const auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int vec = inner % 8 == 0 && aligned(x) && aligned(out) && (!kBackward || aligned(dy)) ? 1 : 0;
  const long long groups_per_row = (inner + 7) / 8;
  const long long groups = outer * groups_per_row;
  long long blocks = (groups + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
#define AB200_GLU(T)                                                                                          \
  glu_kernel<T, kBackward><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                              \
      static_cast<const T*>(x), static_cast<const T*>(dy), static_cast<T*>(out), outer, inner, groups_per_row, \
      act, act_param, vec)
  if (dtype == DT_F32) AB200_GLU(float);
  else if (dtype == DT_F16) AB200_GLU(__half);
  else AB200_GLU(__nv_bfloat16);
#undef AB200_GLU
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}
}  // namespace
}  // extern "C++"

int ab200_glu_forward(const void* x, void* y, int64_t outer, int64_t inner, int dtype, int act, float act_param,
                      void* stream) {
  return launch_glu<false>(x, nullptr, y, outer, inner, dtype, act, act_param, static_cast<cudaStream_t>(stream));
}

int ab200_glu_backward(const void* dy, const void* x, void* dx, int64_t outer, int64_t inner, int dtype, int act,
                       float act_param, void* stream) {
  return launch_glu<true>(x, dy, dx, outer, inner, dtype, act, act_param, static_cast<cudaStream_t>(stream));
}

int64_t ab200_cross_entropy_workspace_bytes(int64_t M) { return M > 0 ? (4 * M + 1) * 4 : 4; }

int ab200_cross_entropy_forward(const void* logits, const int64_t* target, const void* weight, void* loss,
                                float* lse, int64_t M, int64_t V, int64_t stride_m, int64_t stride_v, int dtype,
                                int weight_dtype, int loss_dtype, void* workspace, int64_t workspace_bytes,
                                void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || V <= 0) return ERR_BAD_SHAPE;
  if (!fits_int(M) || !fits_int(V)) return ERR_TOO_LARGE;
  if (!valid_dtype(dtype) || !valid_dtype(loss_dtype) || (weight && !valid_dtype(weight_dtype))) return ERR_BAD_DTYPE;
  if (!loss || !workspace || (M > 0 && (!logits || !target || !lse))) return ERR_NULL_POINTER;
  if (workspace_bytes < ab200_cross_entropy_workspace_bytes(M)) return ERR_WORKSPACE_TOO_SMALL;
  // Workspace: per row the weighted loss, the weight, the maximum and log(sum exp(x - maximum)); then
  // the denominator of the mean.
  float* row_loss = static_cast<float*>(workspace);
  float* row_weight = row_loss + M;
  float* row_max = row_weight + M;
  float* row_logsum = row_max + M;
  float* denominator = row_logsum + M;
  if (M > 0) {
    const unsigned grid = static_cast<unsigned>(M);
    const long long* t = reinterpret_cast<const long long*>(target);
    if (dtype == DT_F32)
      ce_forward_kernel<float><<<grid, kCeThreads, 0, stream>>>(static_cast<const float*>(logits), stride_m, stride_v, t,
                                                             weight, weight_dtype, row_loss, row_weight, row_max, row_logsum, lse, static_cast<int>(V));
    else if (dtype == DT_F16)
      ce_forward_kernel<__half><<<grid, kCeThreads, 0, stream>>>(static_cast<const __half*>(logits), stride_m, stride_v, t,
                                                              weight, weight_dtype, row_loss, row_weight, row_max, row_logsum, lse, static_cast<int>(V));
    else
      ce_forward_kernel<__nv_bfloat16><<<grid, kCeThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), stride_m,
                                                                     stride_v, t, weight, weight_dtype, row_loss,
                                                                     row_weight, row_max, row_logsum, lse,
                                                                     static_cast<int>(V));
    ++g_launches;
    if (cudaGetLastError() != cudaSuccess) return ERR_LAUNCH;
  }
  ce_finish_kernel<<<1, 1024, 0, stream>>>(row_loss, row_weight, M, weight != nullptr ? 1 : 0, loss, loss_dtype, denominator);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}

int ab200_cross_entropy_backward(const void* loss_grad, int loss_grad_dtype, const void* logits, const int64_t* target,
                                 const void* weight, const float* lse, const void* workspace, void* logits_grad,
                                 int64_t M, int64_t V, int64_t stride_m, int64_t stride_v, int64_t ld_grad, int dtype,
                                 int weight_dtype, int grad_dtype, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || V <= 0) return ERR_BAD_SHAPE;
  if (!fits_int(M) || !fits_int(V)) return ERR_TOO_LARGE;
  if (!valid_dtype(dtype) || !valid_dtype(grad_dtype) || !valid_dtype(loss_grad_dtype) ||
      (weight && !valid_dtype(weight_dtype)))
    return ERR_BAD_DTYPE;
  // The gradient has the input's type, or fp32 for 16-bit logits (the loss's type under autocast).
  if (grad_dtype != dtype && grad_dtype != DT_F32) return ERR_BAD_DTYPE;
  if (M == 0) return OK;
  if (!loss_grad || !logits || !target || !lse || !workspace || !logits_grad) return ERR_NULL_POINTER;
  if (ld_grad < V) return ERR_BAD_STRIDE;
  const float* row_max = static_cast<const float*>(workspace) + 2 * M;
  const float* row_logsum = row_max + M;
  const float* denominator = row_logsum + M;
  const unsigned grid = static_cast<unsigned>(M);
  const long long* t = reinterpret_cast<const long long*>(target);
#define AB200_CE_BWD(T, G)                                                                                          \
  ce_backward_kernel<T, G><<<grid, kCeThreads, 0, stream>>>(static_cast<const T*>(logits), stride_m, stride_v, t, weight, \
                                                          weight_dtype, row_max, row_logsum, denominator, loss_grad,  \
                                                          loss_grad_dtype,                                           \
                                                          static_cast<G*>(logits_grad), ld_grad, static_cast<int>(V))
  if (dtype == DT_F32) AB200_CE_BWD(float, float);
  else if (dtype == DT_F16 && grad_dtype == DT_F16) AB200_CE_BWD(__half, __half);
  else if (dtype == DT_F16) AB200_CE_BWD(__half, float);
  else if (grad_dtype == DT_BF16) AB200_CE_BWD(__nv_bfloat16, __nv_bfloat16);
  else AB200_CE_BWD(__nv_bfloat16, float);
#undef AB200_CE_BWD
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}

int ab200_layer_norm_forward(const void* x, const void* weight, const void* bias, float* mean, float* inv_std, void* y,
                             int64_t rows, int64_t feat, int64_t ldx, int64_t ldy, int x_dtype, int param_dtype,
                             int y_dtype, float eps, void* stream_) {
  if (rows < 0 || feat <= 0) return ERR_BAD_SHAPE;
  if (!fits_int(rows) || !fits_int(feat)) return ERR_TOO_LARGE;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype) || (weight && !valid_dtype(param_dtype))) return ERR_BAD_DTYPE;
  // y has x's type, or fp32 for a 16-bit x, or a 16-bit type for an fp32 x.
  if (x_dtype != y_dtype && x_dtype != DT_F32 && y_dtype != DT_F32) return ERR_BAD_DTYPE;
  if (rows == 0) return OK;
  if (!x || !y || (bias && !weight) || ((mean == nullptr) != (inv_std == nullptr))) return ERR_NULL_POINTER;
  if (ldx < feat || ldy < feat) return ERR_BAD_STRIDE;
  const int rc = launch_layer_norm_forward(x, ldx, weight, weight ? bias : nullptr, param_dtype, mean, inv_std, y, ldy,
                                           rows, static_cast<int>(feat), x_dtype, y_dtype, eps,
                                           static_cast<cudaStream_t>(stream_));
  if (rc < 0) return rc;
  g_launches += rc;
  return OK;
}

int64_t ab200_layer_norm_workspace_bytes(int64_t rows, int64_t feat) {
  const long long parts = layer_norm_parts(rows, feat);
  return parts > 0 ? 2 * parts * feat * 4 : 4;
}

int ab200_layer_norm_backward(const void* dy, const void* x, const float* mean, const float* inv_std,
                              const void* weight, void* dx, float* weight_grad, float* bias_grad, int64_t rows,
                              int64_t feat, int64_t lddy, int64_t ldx, int64_t lddx, int dy_dtype, int x_dtype,
                              int param_dtype, int dx_dtype, void* workspace, int64_t workspace_bytes, int* status,
                              void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows < 0 || feat <= 0) return ERR_BAD_SHAPE;
  if (!fits_int(rows) || !fits_int(feat)) return ERR_TOO_LARGE;
  if (!valid_dtype(x_dtype) || !valid_dtype(dy_dtype) || !valid_dtype(dx_dtype) || (weight && !valid_dtype(param_dtype)))
    return ERR_BAD_DTYPE;
  // dy has the forward output's type; dx the wider of that and x's.
  const bool same = x_dtype == dy_dtype && x_dtype == dx_dtype;
  const bool widened = x_dtype != DT_F32 && dy_dtype == DT_F32 && dx_dtype == DT_F32;
  const bool narrowed = x_dtype == DT_F32 && dy_dtype != DT_F32 && dx_dtype == DT_F32;
  if (!same && !widened && !narrowed) return ERR_BAD_DTYPE;
  if ((weight_grad && !weight) || (bias_grad && !weight_grad)) return ERR_NULL_POINTER;
  if (rows == 0) {
    // No rows: the parameter gradients are sums over nothing.
    if (weight_grad && cudaMemsetAsync(weight_grad, 0, feat * 4, stream) != cudaSuccess) return ERR_LAUNCH;
    if (bias_grad && cudaMemsetAsync(bias_grad, 0, feat * 4, stream) != cudaSuccess) return ERR_LAUNCH;
    return OK;
  }
  if (!dy || !x || !mean || !inv_std || !dx) return ERR_NULL_POINTER;
  if (lddy < feat || ldx < feat || lddx < feat) return ERR_BAD_STRIDE;
  if (weight_grad) {
    if (!workspace) return ERR_NULL_POINTER;
    if (workspace_bytes < ab200_layer_norm_workspace_bytes(rows, feat)) return ERR_WORKSPACE_TOO_SMALL;
    if (reinterpret_cast<uintptr_t>(workspace) & 3) return ERR_BAD_STRIDE;
  }
  const int rc = launch_layer_norm_backward(dy, lddy, x, ldx, mean, inv_std, weight, param_dtype, dx, lddx, weight_grad,
                                            bias_grad, static_cast<float*>(workspace), rows, static_cast<int>(feat),
                                            dy_dtype, x_dtype, dx_dtype, status, stream);
  if (rc < 0) return rc;
  g_launches += rc;
  return OK;
}

uint32_t ab200_dropout_threshold(float drop_p, int flags) {
  return dropout_threshold(drop_p, (flags & AB200_FLAG_DROPOUT_PACKED) ? DROPOUT_PACKED : DROPOUT_REFERENCE);
}

float ab200_dropout_uniform(uint32_t seed, uint64_t index, int flags) {
  return dropout_uniform(seed, index, (flags & AB200_FLAG_DROPOUT_PACKED) ? DROPOUT_PACKED : DROPOUT_REFERENCE);
}

int ab200_cast_2d(const void* src, void* dst, int64_t rows, int64_t cols, int64_t src_stride_r,
                  int64_t src_stride_c, int src_dtype, int dst_dtype, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows < 0 || cols < 0) return ERR_BAD_SHAPE;
  if (!valid_dtype(src_dtype) || !valid_dtype(dst_dtype)) return ERR_BAD_DTYPE;
  if (rows == 0 || cols == 0) return OK;
  if (!src || !dst) return ERR_NULL_POINTER;
  const bool vec = src_stride_c == 1 && cols % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(dst) & 15) == 0 &&
                   (src_stride_r * dtype_size(src_dtype)) % 16 == 0;
  const long long work = vec ? rows * (cols / 8) : rows * cols;
  long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
#define AB200_CAST(S, D)                                                                             \
  do {                                                                                               \
    if (vec)                                                                                         \
      cast_kernel<S, D, true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                  \
          static_cast<const S*>(src), src_stride_r, src_stride_c, static_cast<D*>(dst), rows, cols); \
    else                                                                                             \
      cast_kernel<S, D, false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                 \
          static_cast<const S*>(src), src_stride_r, src_stride_c, static_cast<D*>(dst), rows, cols); \
  } while (0)
#define AB200_CAST_TO(S)                                    \
  do {                                                      \
    if (dst_dtype == DT_F32) AB200_CAST(S, float);          \
    else if (dst_dtype == DT_F16) AB200_CAST(S, __half);    \
    else AB200_CAST(S, __nv_bfloat16);                      \
  } while (0)
  if (src_dtype == DT_F32) AB200_CAST_TO(float);
  else if (src_dtype == DT_F16) AB200_CAST_TO(__half);
  else AB200_CAST_TO(__nv_bfloat16);
#undef AB200_CAST_TO
#undef AB200_CAST
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}

}  // extern "C"
