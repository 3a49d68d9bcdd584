/*
 * attorch_b200 -- C ABI of the B200-native (sm_100a) fused linear layer.
 *
 * The reference (BobMcDear/attorch) is pure Python + Triton and has no FFI of its own; its
 * boundary for this path is the Python call LinearAutoGrad.apply(input, weight, bias, act_func)
 * (attorch/linear_layer.py:19-161).  Each entry point below replaces one device-side step of that
 * function; the Python module attorch_b200.linear_layer binds them with ctypes.
 *
 * Conventions
 *   - Every pointer is a device pointer owned by the caller.  Except where an entry point says
 *     otherwise the library allocates no device memory and keeps no pointer after it returns.
 *   - Matrices are row-major; "ld" arguments are row pitches in ELEMENTS.
 *   - The weight has the reference's layout [in_features, out_features] (attorch/linear_layer.py:200).
 *   - Calls are asynchronous on `stream` (a cudaStream_t passed as void*), never synchronise, and
 *     may be made from any host thread with the right device current.
 *   - The return value is 0 on success or a negative AB200_ERR_* code for an argument the host
 *     rejected before launching anything.  A kernel that gives up on a bounded wait writes a
 *     positive AB200_DEV_* code to `*status` (a device int the caller zeroes and reads when it
 *     next synchronises); the outputs of that call are then undefined.
 */
#ifndef ATTORCH_B200_H_
#define ATTORCH_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types. */
#define AB200_F32 0
#define AB200_F16 1
#define AB200_BF16 2

/* Host-side return codes. */
#define AB200_OK 0
#define AB200_ERR_NULL_POINTER (-1)
#define AB200_ERR_BAD_SHAPE (-2)
#define AB200_ERR_BAD_DTYPE (-3)
#define AB200_ERR_BAD_ACT (-4)
#define AB200_ERR_BAD_STRIDE (-5)
#define AB200_ERR_WORKSPACE_TOO_SMALL (-6)
#define AB200_ERR_TENSOR_MAP (-7)
#define AB200_ERR_LAUNCH (-8)
#define AB200_ERR_TOO_LARGE (-9)
#define AB200_ERR_DRIVER (-10)
#define AB200_ERR_STATIC_SCRATCH_TOO_SMALL (-11)
#define AB200_ERR_BAD_PROBABILITY (-12)

/* Device-side status codes (written to *status). */
#define AB200_DEV_OK 0
#define AB200_DEV_TIMEOUT_PRODUCER 1
#define AB200_DEV_TIMEOUT_MMA 2
#define AB200_DEV_TIMEOUT_EPILOGUE 3
#define AB200_DEV_TIMEOUT_COLLECTIVE 4
#define AB200_DEV_TIMEOUT_ROW_COPY 5

/* Activation ids: the act_func strings of attorch/linear_layer.py:42-49 in the order of the
 * dispatcher attorch/act_kernels.py:654-727.  Ids 17..21 take `act_param`. */
#define AB200_ACT_NONE 0
#define AB200_ACT_SIGMOID 1
#define AB200_ACT_LOGSIGMOID 2
#define AB200_ACT_TANH 3
#define AB200_ACT_RELU 4
#define AB200_ACT_GELU 5
#define AB200_ACT_GELUAPPROX 6
#define AB200_ACT_SILU 7
#define AB200_ACT_RELU6 8
#define AB200_ACT_HARDSIGMOID 9
#define AB200_ACT_HARDTANH 10
#define AB200_ACT_HARDSWISH 11
#define AB200_ACT_SELU 12
#define AB200_ACT_MISH 13
#define AB200_ACT_SOFTPLUS 14
#define AB200_ACT_SOFTSIGN 15
#define AB200_ACT_TANHSHRINK 16
#define AB200_ACT_LEAKY_RELU 17
#define AB200_ACT_ELU 18
#define AB200_ACT_CELU 19
#define AB200_ACT_HARDSHRINK 20
#define AB200_ACT_SOFTSHRINK 21
#define AB200_ACT_COUNT 22
/* ab200_act_backward only: `z` already holds act'(Z), written by a forward call that had
 * AB200_FLAG_SAVE_DERIVATIVE set; dZ = dY * z. */
#define AB200_ACT_SAVED_DERIVATIVE 22
/* Same, for a forward call that also had AB200_FLAG_DERIVATIVE_FP16 set: `z` holds act'(Z) as fp16
 * whatever `dtype` is (2-byte types only). */
#define AB200_ACT_SAVED_DERIVATIVE_F16 23

/* Flags (bit set) accepted by the GEMM entry points. */
#define AB200_FLAG_FORCE_GENERIC 1  /* use the any-shape CUDA-core kernel                      */
#define AB200_FLAG_FORCE_TCGEN05 2  /* fail with AB200_ERR_BAD_STRIDE instead of falling back   */
#define AB200_FLAG_FORCE_STREAMK 4  /* forward only: use the swap-AB stream-K kernel            */
#define AB200_FLAG_NO_STREAMK 8     /* forward only: never use the swap-AB stream-K kernel      */
#define AB200_FLAG_NO_PAIR 16       /* one CTA per tile: no cta_group::2 kernels                */
#define AB200_FLAG_NO_TMA_STORE 32  /* epilogue stores from registers, not through TMA           */
#define AB200_FLAG_SAVE_DERIVATIVE 64 /* forward: pre_act receives act'(Z) instead of Z            */
#define AB200_FLAG_WHOLE_TILES 128  /* never share out or halve a partial last round of tiles   */
#define AB200_FLAG_DROPOUT_PACKED 256 /* activation layers: the cheaper dropout stream (see below) */
#define AB200_FLAG_DERIVATIVE_FP16 512 /* forward with SAVE_DERIVATIVE and a bf16 output: act'(Z) is stored
                                        * as fp16 (same size, 3 more mantissa bits; derivatives are O(1)), so
                                        * that dZ = dY * act'(Z) is in effect rounded once, as the reference's */
/* Bits 16-23 of the flags of a GEMM entry point: the number of SMs (0-255) the persistent kernel of
 * that call leaves free, for a collective that runs beside it (same purpose as
 * ab200_set_gemm_cta_limit, but per call instead of process-wide). */
#define AB200_FLAG_RESERVE_SMS_SHIFT 16
#define AB200_FLAG_RESERVE_SMS(n) (((n) & 0xFF) << AB200_FLAG_RESERVE_SMS_SHIFT)

/* Which kernel the last call on this host thread chose: 1 tcgen05 tile-parallel, 2 tcgen05
 * swap-AB stream-K, 3 generic CUDA-core.  For tests and benchmarks. */
#define AB200_PATH_TCGEN05 1
#define AB200_PATH_STREAMK 2
#define AB200_PATH_GENERIC 3

/* Library version, major * 1000 + minor. */
int ab200_version(void);

/* Text for a host return code or a device status code. */
const char* ab200_error_string(int code);

/* Kernel chosen by the last GEMM entry point called on this host thread (AB200_PATH_*). */
int ab200_last_path(void);

/*
 * How the last tensor-core GEMM launched from this host thread divided its work: 0 whole tiles;
 * 1 equal (tile, k-block) shares added atomically (stream-K); 2 whole tiles, the partial last round
 * shared out and summed in a fixed order; 3 whole tiles, the partial last round as half-width tiles.
 */
int ab200_last_schedule(void);

/*
 * Limits the CTAs (= SMs) the persistent GEMM kernels launch with, process-wide; 0 restores "all".
 * Returns the previous limit.  For callers that overlap a GEMM with a collective (NCCL needs SMs of
 * its own, and a GEMM that already holds every SM would make it wait until the GEMM ends).
 */
int ab200_set_gemm_cta_limit(int ctas);

/* Number of kernels this library has launched (all host threads) since it was loaded. */
int64_t ab200_launch_count(void);

/*
 * Forward:  Z = X * W (+ bias);  pre_act <- Z (if not NULL);  out <- act(Z).
 * Replaces linear_forward_kernel (attorch/linear_kernels.py:59-188) as launched at
 * attorch/linear_layer.py:88-98.
 *   x        [M, K], element strides (x_stride_m, x_stride_k), type op_dtype
 *   w        [K, N], element strides (w_stride_k, w_stride_n), type op_dtype
 *   bias     [N] of bias_dtype, or NULL; rounded to out_dtype before it is added when out_dtype is
 *            16-bit (attorch/linear_kernels.py:171-172)
 *   pre_act  [M, N] of out_dtype, row pitch ld_pre, or NULL: the value before the activation,
 *            rounded to out_dtype (what backward differentiates through).  With
 *            AB200_FLAG_SAVE_DERIVATIVE it receives act'(Z) instead (piecewise derivatives taken at
 *            the rounded Z, exactly where the reference takes them), which turns the activation
 *            backward into one multiply per element: pass it to ab200_act_backward as `z` with
 *            act = AB200_ACT_SAVED_DERIVATIVE
 *   out      [M, N] of out_dtype, row pitch ld_out
 * Accumulation is fp32; fp32 operands are multiplied as TF32 on the tensor cores
 * (attorch/linear_kernels.py:57,165).  The activation is evaluated on the unrounded fp32 value
 * (attorch/linear_kernels.py:183).
 * Operands with unit inner stride and 16-byte aligned base and row pitch run on the tcgen05
 * kernels; anything else runs on the generic kernel.  M <= 128 uses the swap-AB stream-K kernel,
 * which needs workspace_bytes >= ab200_forward_workspace_bytes(M, K, N, flags); the workspace is
 * cleared by the call itself.
 */
int ab200_linear_forward(const void* x, const void* w, const void* bias, void* pre_act, void* out,
                         int64_t M, int64_t K, int64_t N, int64_t x_stride_m, int64_t x_stride_k,
                         int64_t w_stride_k, int64_t w_stride_n, int64_t ld_pre, int64_t ld_out,
                         int op_dtype, int out_dtype, int bias_dtype, int act, float act_param,
                         void* workspace, int64_t workspace_bytes, int* status, void* stream,
                         int flags);

/*
 * ab200_linear_forward with a residual added after the activation:
 *     Y = act(X W + b) + R
 * R: [M, N] in out_dtype with row pitch ld_res elements (>= N), or NULL (then this is
 * ab200_linear_forward).  pre_act still receives Z (or act'(Z)), which does not involve R, so the
 * backward entry points are unchanged; the gradient of R is the upstream gradient itself.  No
 * counterpart in the reference, whose callers add the residual in a separate pass over Y
 * (examples/wikitext-2/gpt.py:82).
 */
int ab200_linear_forward_residual(const void* x, const void* w, const void* bias, void* pre_act, void* out,
                                  const void* residual, int64_t M, int64_t K, int64_t N, int64_t x_stride_m,
                                  int64_t x_stride_k, int64_t w_stride_k, int64_t w_stride_n, int64_t ld_pre,
                                  int64_t ld_out, int64_t ld_res, int op_dtype, int out_dtype, int bias_dtype,
                                  int act, float act_param, void* workspace, int64_t workspace_bytes,
                                  int* status, void* stream, int flags);

/*
 * Projection followed by a gated linear unit, in one kernel:
 *     [X1 | X2] = X * W (+ bias),   pre_act <- [X1 | X2] (if not NULL),   out <- X1 * act(X2)
 * with W [K, 2H], bias [2H], pre_act [M, 2H] (row pitch ld_pre >= 2H), out [M, H].  It replaces
 * linear_forward_kernel without activation (attorch/linear_kernels.py:59-188) followed by
 * glu_forward_kernel over its output (attorch/glu_kernels.py:13-53, with the two copies of the halves
 * attorch/glu_layer.py:58-60 makes), i.e. attorch.GLU(act_func)(attorch.Linear(K, 2H)(x)), and saves
 * the read of [M, 2H] between the two.  The halves are multiplied as they are stored (rounded to
 * out_dtype), so the result equals the two-kernel sequence bit for bit.  Backward is the existing
 * sequence: ab200_glu_backward on pre_act, then the bias sum and the two products.
 * Tensor-core path only: returns AB200_ERR_BAD_STRIDE where x or w are not TMA-addressable or H is not a
 * multiple of 16 bytes' worth of elements (callers then run the two kernels).  flags: AB200_FLAG_NO_PAIR,
 * AB200_FLAG_NO_TMA_STORE, AB200_FLAG_RESERVE_SMS(n).
 */
int ab200_gated_linear_forward(const void* x, const void* w, const void* bias, void* pre_act, void* out, int64_t M,
                               int64_t K, int64_t H, int64_t x_stride_m, int64_t x_stride_k, int64_t w_stride_k,
                               int64_t w_stride_n, int64_t ld_pre, int64_t ld_out, int op_dtype, int out_dtype,
                               int bias_dtype, int act, float act_param, int* status, void* stream, int flags);

/* Workspace the forward call may use for this shape and these flags (0 when it needs none). */
int64_t ab200_forward_workspace_bytes(int64_t M, int64_t K, int64_t N, int flags);

/*
 * Workspace a GEMM entry point may use for an output of rows x cols elements and the given reduction
 * length (0 when it needs none).  Outputs too small to occupy half of the SMs with whole tiles,
 * e.g. the weight gradient of a narrow layer over a long batch, are computed as equal shares of the
 * reduction on all SMs, accumulated in fp32 in the workspace and rounded by a finishing kernel.
 * Large outputs whose last round of tiles would leave most SMs idle (256 tiles on 74 CTA pairs,
 * say) share out just that round the same way.  Without the workspace the call still succeeds, on
 * whole tiles.
 */
int64_t ab200_gemm_workspace_bytes(int64_t rows, int64_t cols, int64_t reduction);

/*
 * Backward, step 1:  dZ = dY * act'(Z)  and  db[n] = sum_m dZ[m, n].
 * Replaces act_func_backward_kernel (attorch/act_kernels.py:883-927, launched at
 * attorch/linear_layer.py:143-146) and pre_act_grad.sum(dim=0) (attorch/linear_layer.py:156).
 *   dy, z, dz  [M, N] of `dtype`; z may be NULL iff act == AB200_ACT_NONE; dz may be NULL when
 *              only db is wanted (act == NONE, where dZ is dY itself)
 *   db         [N] of db_dtype or NULL; summed in fp32 in a fixed order, rounded once
 *   workspace  needed iff db != NULL: ab200_act_backward_workspace_bytes(M, N) bytes
 */
int ab200_act_backward(const void* dy, const void* z, void* dz, void* db, int64_t M, int64_t N,
                       int64_t ld_dy, int64_t ld_z, int64_t ld_dz, int dtype, int db_dtype, int act,
                       float act_param, void* workspace, int64_t workspace_bytes, void* stream);

int64_t ab200_act_backward_workspace_bytes(int64_t M, int64_t N);

/*
 * Backward, step 1, for callers that cannot allocate device memory.  (No counterpart in the
 * reference: it allocates freely through PyTorch.)
 *
 * Same computation and same results as ab200_act_backward, but the scratch for the bias-gradient
 * column sums is a fixed 4 MiB array inside the library, so the caller passes only inputs and
 * outputs and the call never runs cudaMalloc, cudaFree or any allocating routine.  It is meant for
 * code that runs where allocation is forbidden or impossible: inside a memory pool that has been
 * frozen for the step, in a latency-critical serving loop that must not touch the allocator, or in
 * a host thread that owns no allocator at all (for instance a plain C or Go caller of this ABI).
 *
 *   - Limit: ceil(M / 128) * N must not exceed ab200_act_backward_static_max_floats() (1 Mi fp32),
 *     e.g. M = 8192 with N up to 16384; larger shapes return AB200_ERR_STATIC_SCRATCH_TOO_SMALL and
 *     launch nothing.  The limit applies only when db is wanted; without db no scratch is used.
 *   - The first call on each device looks up the array's device address (with that device current)
 *     and remembers it; make that first call before any stream capture begins.
 *   - Every call on a device shares the one array.  Calls that may overlap on the GPU (different
 *     streams, or different processes' threads on one context) race on it: serialise them.
 *     Nothing has to be zeroed between calls; each call overwrites every entry it later reads.
 *   - Every GPU that loads the library keeps the 4 MiB reserved until the process exits.
 */
int ab200_act_backward_static(const void* dy, const void* z, void* dz, void* db, int64_t M, int64_t N,
                              int64_t ld_dy, int64_t ld_z, int64_t ld_dz, int dtype, int db_dtype,
                              int act, float act_param, void* stream);

/* Capacity of the built-in scratch of ab200_act_backward_static, in fp32 elements. */
int64_t ab200_act_backward_static_max_floats(void);

/*
 * Backward, step 2:  dX[M, K] = dZ[M, N] * W^T.   Replaces `pre_act_grad @ weight.T`
 * (attorch/linear_layer.py:153).  dz and w are of op_dtype, dx of dx_dtype.  workspace: optional,
 * ab200_gemm_workspace_bytes(M, K, N) bytes.
 */
int ab200_linear_backward_input(const void* dz, const void* w, void* dx, int64_t M, int64_t K,
                                int64_t N, int64_t dz_stride_m, int64_t dz_stride_n,
                                int64_t w_stride_k, int64_t w_stride_n, int64_t ld_dx, int op_dtype,
                                int dx_dtype, void* workspace, int64_t workspace_bytes, int* status,
                                void* stream, int flags);

/*
 * Backward, step 3:  dW[K, N] = X^T * dZ.   Replaces `flattened_input.T @ pre_act_grad`
 * (attorch/linear_layer.py:154-155).  x and dz are of op_dtype, dw of dw_dtype (pass AB200_F32 to
 * keep the fp32 accumulator unrounded, e.g. for fp32 master weights or an fp32 all-reduce bucket).
 * workspace: optional, ab200_gemm_workspace_bytes(K, N, M) bytes.
 */
int ab200_linear_backward_weight(const void* x, const void* dz, void* dw, int64_t M, int64_t K,
                                 int64_t N, int64_t x_stride_m, int64_t x_stride_k,
                                 int64_t dz_stride_m, int64_t dz_stride_n, int64_t ld_dw,
                                 int op_dtype, int dw_dtype, void* workspace, int64_t workspace_bytes,
                                 int* status, void* stream, int flags);

/*
 * Standalone activation layer with fused dropout, forward:  y[i] = keep_i ? act(x[i]) / (1 - p) : 0.
 * Replaces act_func_forward_kernel (attorch/act_kernels.py:840-880, launched at
 * attorch/act_layers.py:66-73) with apply_dropout (attorch/dropout_kernels.py:12-28).  x, y: n
 * contiguous elements of `dtype`; act != AB200_ACT_NONE is not required (identity + dropout works).
 * drop_p = 0 switches dropout off and drop_p = 1 drops every element (zeros, as the reference's
 * tl.where(random < 1, 0, ...) gives); otherwise element i is dropped iff
 * ab200_dropout_uniform(seed, i, flags) < drop_p.  flags: 0 or AB200_FLAG_DROPOUT_PACKED.
 */
int ab200_act_forward(const void* x, void* y, int64_t n, int dtype, int act, float act_param, float drop_p,
                      uint32_t seed, void* stream, int flags);

/*
 * Its backward:  dx[i] = (keep_i ? dy[i] / (1 - p) : 0) * act'(x[i]), same mask as forward for the
 * same seed and flags.  Replaces act_func_backward_kernel (attorch/act_kernels.py:883-927, launched
 * at attorch/act_layers.py:106-110) with apply_dropout_grad (attorch/dropout_kernels.py:31-46).
 */
int ab200_act_input_grad(const void* dy, const void* x, void* dx, int64_t n, int dtype, int act,
                         float act_param, float drop_p, uint32_t seed, void* stream, int flags);

/*
 * The uniform number in [0, 1) the dropout mask compares with drop_p (host function).
 * flags = 0: the number the reference draws for the same seed and element, tl.rand(seed, offset)
 * (attorch/dropout_kernels.py:26) - Philox 4x32-10 with key (seed, 0) and counter
 * (uint32(index), 0, 0, 0); the first output word w as int32, mirrored (w < 0 ? -w - 1 : w),
 * converted to fp32 and multiplied by 4.6566127342e-10 - so that a given seed drops the same
 * elements here and there.  AB200_FLAG_DROPOUT_PACKED: counter index / 4, word index % 4, top 24
 * bits: a quarter of the integer work (one block per four elements), a different mask.
 */
float ab200_dropout_uniform(uint32_t seed, uint64_t index, int flags);

/*
 * The integer form of "ab200_dropout_uniform(...) < drop_p" the kernels use (host function; no
 * counterpart in the reference): element i is dropped iff m < ab200_dropout_threshold(drop_p, flags),
 * m being the Philox word of element i - mirrored (w < 0 ? -w - 1 : w) with flags = 0, as it is with
 * AB200_FLAG_DROPOUT_PACKED.  Exact, because the word -> fp32 conversions are monotonic.
 */
uint32_t ab200_dropout_threshold(float drop_p, int flags);

/*
 * Gated linear unit with an arbitrary activation, forward:  y = x1 * act(x2), x1 and x2 being the two
 * halves of the input along the gated dimension.  Replaces glu_forward_kernel
 * (attorch/glu_kernels.py:13-53, launched at attorch/glu_layer.py:58-79) together with the two
 * .contiguous() copies of the halves made there: x is the contiguous input seen as
 * [outer, 2 * inner] (outer = product of the dimensions before the gated one, inner = half the gated
 * extent times the product of the dimensions after it), y is [outer, inner].  act = AB200_ACT_NONE
 * gives the bilinear unit x1 * x2.
 */
int ab200_glu_forward(const void* x, void* y, int64_t outer, int64_t inner, int dtype, int act, float act_param,
                      void* stream);

/*
 * Its backward:  dx1 = dy * act(x2),  dx2 = dy * x1 * act'(x2), written into dx in the layout of x
 * (no concatenation pass).  Replaces glu_backward_kernel (attorch/glu_kernels.py:56-105, launched at
 * attorch/glu_layer.py:101-116).
 */
int ab200_glu_backward(const void* dy, const void* x, void* dx, int64_t outer, int64_t inner, int dtype, int act,
                       float act_param, void* stream);

/*
 * dst[r, c] (contiguous, dst_dtype) = src[r * src_stride_r + c * src_stride_c] (src_dtype).
 * The operand casts that autocast implies (attorch/linear_kernels.py:161-163 casts in registers;
 * torch.autocast casts before its matmuls, attorch/linear_layer.py:152) and the copy that makes a
 * strided input addressable by TMA.
 */
int ab200_cast_2d(const void* src, void* dst, int64_t rows, int64_t cols, int64_t src_stride_r,
                  int64_t src_stride_c, int src_dtype, int dst_dtype, void* stream);

/*
 * Cross-entropy loss of a logits matrix against class indices, the loss the final projection of a
 * language model feeds.  Forward replaces cross_entropy_loss_forward_kernel
 * (attorch/cross_entropy_loss_kernels.py:13-88, launched at attorch/cross_entropy_loss_layer.py:67-80)
 * together with the sums and the division that follow it there (lines 75-79):
 *     L = sum_i w[t_i] * (log sum_j exp(x_ij) - x_{i,t_i}) / (weight ? sum_i w[t_i] : M)
 *   logits  [M, V] of `dtype`, element strides (stride_m, stride_v); evaluated in fp32
 *   target  [M] int64 class indices in [0, V)
 *   weight  [V] class weights of weight_dtype, or NULL
 *   loss    one element of loss_dtype (the reference: fp32 under autocast, else the logits' type)
 *   lse     [M] fp32, receives log-sum-exp of every row (for callers that want it)
 *   workspace  ab200_cross_entropy_workspace_bytes(M) bytes; it must reach the backward call intact:
 *           it holds every row's maximum and log(sum exp(x - maximum)), with which backward needs
 *           one exponential per element instead of a second maximum / sum pass (the reference
 *           recomputes both), and the denominator of the mean
 * M = 0 gives a loss of 0.  Row sums are added in a fixed order.
 */
int ab200_cross_entropy_forward(const void* logits, const int64_t* target, const void* weight, void* loss,
                                float* lse, int64_t M, int64_t V, int64_t stride_m, int64_t stride_v, int dtype,
                                int weight_dtype, int loss_dtype, void* workspace, int64_t workspace_bytes,
                                void* stream);

int64_t ab200_cross_entropy_workspace_bytes(int64_t M);

/*
 * Its backward:  dx_ij = dL * s_i * (softmax(x_i)_j - [j == t_i]),  s_i = w[t_i] / sum_i w[t_i]  or
 * 1 / M.  Replaces cross_entropy_loss_backward_kernel (attorch/cross_entropy_loss_kernels.py:91-173,
 * launched at attorch/cross_entropy_loss_layer.py:107-114).  loss_grad: one element of loss_grad_dtype
 * (device memory); logits_grad: [M, V] of grad_dtype (the logits' type, or fp32), row pitch ld_grad.
 */
int ab200_cross_entropy_backward(const void* loss_grad, int loss_grad_dtype, const void* logits, const int64_t* target,
                                 const void* weight, const float* lse, const void* workspace, void* logits_grad,
                                 int64_t M, int64_t V, int64_t stride_m, int64_t stride_v, int64_t ld_grad, int dtype,
                                 int weight_dtype, int grad_dtype, void* stream);

/*
 * Input gradient with the activation gradient formed in the operand path, as one kernel:
 *     dx[M, K] = (dy[M, N] (.) derivative[M, N]) * w[K, N]^T
 * where `derivative` is act'(Z) as ab200_linear_forward stored it (AB200_FLAG_SAVE_DERIVATIVE).  It
 * stands for act_func_backward_kernel followed by `pre_act_grad @ weight.T` (attorch/linear_layer.py:
 * 136-153) without the pass that writes pre_act_grad: the products are rounded to bf16 as that pass
 * rounds them, written to tensor memory and read from there as the A operand of tcgen05.mma (see
 * csrc/dx_fused.cu).  The bias gradient is not part of it.  The layer's backward does not use this entry
 * point: it was measured slower than the two kernels it replaces; it is kept so that the measurement can
 * be repeated (bench.py --workload dxfused).
 *   dy          [M, N] bf16, row pitch ld_dy;  derivative [M, N] fp16 or bf16 (derivative_dtype), pitch ld_d
 *   w           [K, N] bf16 (the layer's [in, out] weight), pitch ld_w
 *   dx          [M, K] bf16 or fp32 (dx_dtype), pitch ld_dx
 *   N a multiple of 64; dy, derivative and w 16-byte aligned with pitches that are multiples of 8 elements
 *   status      device word, required (bounded waits report AB200_DEV_TIMEOUT_* there)
 */
int ab200_linear_backward_input_fused(const void* dy, const void* derivative, const void* w, void* dx, int64_t M,
                                      int64_t K, int64_t N, int64_t ld_dy, int64_t ld_d, int64_t ld_w,
                                      int64_t ld_dx, int derivative_dtype, int dx_dtype, int* status, void* stream);

/*
 * Layer normalisation over the rows of [rows, feat], the step in front of a transformer block's first
 * projection (the caller: examples/wikitext-2/gpt.py:82).  Replaces layer_norm_forward_kernel
 * (attorch/layer_norm_kernels.py:14-103, launched at attorch/layer_norm_layer.py:74-82):
 *     y_ij = (x_ij - mean_i) * rsqrt(var_i + eps) [* weight_j [+ bias_j]],  var_i the biased variance
 *   x       [rows, feat] of x_dtype, unit inner stride, row pitch ldx (elements)
 *   weight, bias  [feat] of param_dtype, or NULL (bias only together with weight)
 *   mean, inv_std  [rows] fp32, receive the row statistics for backward; both NULL when not wanted
 *   y       [rows, feat] of y_dtype, row pitch ldy.  y_dtype is x_dtype, or fp32 for a 16-bit x (the
 *           reference's autocast_to_fp32, attorch/layer_norm_layer.py:55-57), or a 16-bit type for an
 *           fp32 x: the operand type of the projection that follows under autocast, which then needs no
 *           cast pass of its own.  Values are computed in fp32 and rounded once by the store.
 * One pass over x: each row is held in registers between the sums and the store.
 */
int ab200_layer_norm_forward(const void* x, const void* weight, const void* bias, float* mean, float* inv_std, void* y,
                             int64_t rows, int64_t feat, int64_t ldx, int64_t ldy, int x_dtype, int param_dtype,
                             int y_dtype, float eps, void* stream);

/* Bytes of workspace ab200_layer_norm_backward needs when it is asked for parameter gradients. */
int64_t ab200_layer_norm_workspace_bytes(int64_t rows, int64_t feat);

/*
 * Its backward.  Replaces layer_norm_backward_kernel (attorch/layer_norm_kernels.py:106-221, launched at
 * attorch/layer_norm_layer.py:134-144) and the sums over its per-program partial rows (lines 146-149):
 *     p_ij = (x_ij - mean_i) * inv_std_i,  g_ij = weight_j * dy_ij (dy_ij without weight)
 *     dx_ij = inv_std_i * (g_ij - (p_ij * sum_j(p_ij g_ij) / feat + sum_j g_ij / feat))
 *     weight_grad_j = sum_i dy_ij p_ij,  bias_grad_j = sum_i dy_ij      (fp32, fixed order of addition)
 *   dy      [rows, feat] of dy_dtype (the forward's y_dtype), row pitch lddy
 *   dx      [rows, feat] of dx_dtype, row pitch lddx: the wider of x_dtype and dy_dtype (the reference
 *           stores it in the forward's output type and the autograd engine casts, layer_norm_layer.py:117)
 *   weight_grad, bias_grad  [feat] fp32 or NULL (bias_grad only together with weight_grad; weight_grad
 *           needs weight); with them, workspace of ab200_layer_norm_workspace_bytes(rows, feat) bytes
 *   status  device word as for the GEMM entry points, or NULL.  With it, aligned rows of 520 ... 8192
 *           elements are staged in shared memory by bulk copies that wait on mbarriers with a time limit;
 *           a wait that runs out stores AB200_DEV_TIMEOUT_ROW_COPY.  Without it they go through registers.
 * One pass over x and dy for rows of up to 8192 elements: the parameter-gradient sums of a thread's
 * columns stay in its registers over all rows of its block.
 */
int ab200_layer_norm_backward(const void* dy, const void* x, const float* mean, const float* inv_std,
                              const void* weight, void* dx, float* weight_grad, float* bias_grad, int64_t rows,
                              int64_t feat, int64_t lddy, int64_t ldx, int64_t lddx, int dy_dtype, int x_dtype,
                              int param_dtype, int dx_dtype, void* workspace, int64_t workspace_bytes, int* status,
                              void* stream);

/*
 * In-place SUM all-reduce of a gradient bucket over the GPUs of one NVSwitch domain (one process per
 * GPU), through NVLink multicast: the switch adds the ranks' copies (multimem.ld_reduce) and writes the
 * sums back to all of them (multimem.st); see csrc/allreduce_multimem.cu.  No counterpart in the
 * reference, which has no distributed code; it serves the data-parallel step, where dW / db of every
 * layer are summed over the ranks that share a batch (what `torch.distributed.all_reduce` would do).
 *   multicast_ptr  the multicast address of the buffer: `numel` elements of `dtype`, 16-byte aligned,
 *                  numel * element size a multiple of 16 bytes.  Every rank has bound its own buffer of
 *                  that size to one multicast object and calls with the same arguments but `rank`.
 *   flag_blocks    DEVICE array of world_size pointers: entry r is rank r's flag block as mapped into
 *                  this rank's address space (peer-accessible memory of ab200_collective_flag_bytes()
 *                  bytes, zeroed once before the first call and then left to the library).
 *   ctas           CTAs (= SMs) the kernel uses, at most AB200_COLLECTIVE_MAX_CTAS; <= 0 picks 8.  The
 *                  additions run in the switch, so few are enough; every rank must pass the same value.
 *   status         device word as for the GEMMs: a rank that waits longer than 2 s for another stores
 *                  AB200_DEV_TIMEOUT_COLLECTIVE there and returns.
 * Every rank must make the same sequence of calls on the same flag blocks (the barriers count
 * launches), and the buffer's contents must be final on the calling stream before the call.  All ranks
 * end with bit-identical sums.  world_size == 1 returns at once.
 */
#define AB200_COLLECTIVE_MAX_CTAS 32
#define AB200_COLLECTIVE_MAX_RANKS 16
int ab200_multimem_all_reduce(void* multicast_ptr, int64_t numel, int dtype, int rank, int world_size,
                              void* const* flag_blocks, int ctas, int* status, void* stream);

/* Size in bytes of one rank's flag block for ab200_multimem_all_reduce. */
int64_t ab200_collective_flag_bytes(void);

#ifdef __cplusplus
}
#endif
#endif /* ATTORCH_B200_H_ */
