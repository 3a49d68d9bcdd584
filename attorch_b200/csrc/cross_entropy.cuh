// Cross-entropy loss over the rows of a logits matrix, forward and backward: the loss the final
// projection of a language model feeds (reference: attorch/cross_entropy_loss_kernels.py:13-173,
// launched from attorch/cross_entropy_loss_layer.py:20-121).
//
//   forward   loss_i = log(sum_j exp(x_ij)) - x_{i, t_i}          (t_i = target class of row i)
//             L = sum_i loss_i / M                                 or, with class weights w,
//             L = sum_i w_{t_i} loss_i / sum_i w_{t_i}
//   backward  dx_ij = dL * s_i * (softmax(x_i)_j - [j == t_i]),    s_i = 1 / M  or  w_{t_i} / sum_i w_{t_i}
//
// Both kernels are bound by HBM: forward reads the logits once (one pass: running maximum and running
// sum of exponentials per thread, merged across the block), backward reads them once and writes the
// gradient.  Forward also stores each row's maximum and log(sum exp(x - maximum)) (8 bytes), so backward
// is one exponential per element instead of a second maximum / sum pass - the reference recomputes both
// there.  (The two are kept apart rather than added: for logits of large magnitude their sum, the
// log-sum-exp, has too coarse an fp32 spacing to subtract from.)  Everything
// is evaluated in fp32, as in the reference (it widens the loaded logits to fp32, lines 74-76, 150-154).
// Row sums are added in a fixed order: results do not depend on scheduling.
#pragma once
#include <cfloat>

#include "common.cuh"

namespace ab200 {

constexpr int kCeThreads = 256;

// Merges two (maximum, sum of exp(x - maximum)) pairs.
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  const float mx = fmaxf(m, m2);
  // exp(-inf - -inf) must not appear: an empty partial has s = 0 and m = -inf.
  const float a = (m == -INFINITY) ? 0.0f : s * __expf(m - mx);
  const float b = (m2 == -INFINITY) ? 0.0f : s2 * __expf(m2 - mx);
  m = mx;
  s = a + b;
}

// One block per row.  row_loss[i] = w_i * loss_i (w_i = 1 without class weights), row_weight[i] = w_i,
// row_max[i] and row_logsum[i] as above, lse[i] = their sum, the log-sum-exp of row i.
template <class T>
__global__ void __launch_bounds__(kCeThreads)
ce_forward_kernel(const T* __restrict__ x, long long stride_m, long long stride_v, const long long* __restrict__ target,
                  const void* __restrict__ weight, int weight_dtype, float* __restrict__ row_loss,
                  float* __restrict__ row_weight, float* __restrict__ row_max, float* __restrict__ row_logsum,
                  float* __restrict__ lse, int V) {
  const long long row = blockIdx.x;
  const T* xr = x + row * stride_m;
  float m = -INFINITY, s = 0.0f;
  const bool vec = stride_v == 1 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0;
  constexpr int kPer = 16 / sizeof(T);       // elements per 16-byte load
  const int whole = vec ? V / kPer : 0;
  // (Four loads in flight per thread and trip measured no faster: 183 vs 175 us on [8192, 50304] bf16.
  // With one exponential, one maximum and one addition per element the forward pass is bound by
  // instruction issue at about 4.7 TB/s, below the HBM limit that the backward pass reaches.)
  for (int g = threadIdx.x; g < whole; g += kCeThreads) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(xr) + g);
    const T* e = reinterpret_cast<const T*>(&q);
    float v[kPer];
    float gm = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      v[i] = to_f32<T>(e[i]);
      gm = fmaxf(gm, v[i]);
    }
    if (gm > m) {
      s = (m == -INFINITY) ? 0.0f : s * __expf(m - gm);
      m = gm;
    }
    if (m != -INFINITY) {
#pragma unroll
      for (int i = 0; i < kPer; ++i) s += __expf(v[i] - m);
    }
  }
  for (int c = whole * kPer + threadIdx.x; c < V; c += kCeThreads) {
    const float v = to_f32<T>(xr[static_cast<long long>(c) * stride_v]);
    if (v > m) {
      s = (m == -INFINITY) ? 0.0f : s * __expf(m - v);
      m = v;
    }
    if (m != -INFINITY) s += __expf(v - m);
  }
  // Warp, then block: fixed order.
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float m2 = __shfl_xor_sync(0xFFFFFFFFu, m, off);
    const float s2 = __shfl_xor_sync(0xFFFFFFFFu, s, off);
    lse_merge(m, s, m2, s2);
  }
  __shared__ float sm[kCeThreads / 32], ss[kCeThreads / 32];
  if ((threadIdx.x & 31) == 0) {
    sm[threadIdx.x >> 5] = m;
    ss[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = sm[0], bs = ss[0];
#pragma unroll
    for (int w = 1; w < kCeThreads / 32; ++w) lse_merge(bm, bs, sm[w], ss[w]);
    const float ls = logf(bs);
    const long long t = target[row];
    const bool in_range = t >= 0 && t < V;
    const float pred = in_range ? to_f32<T>(xr[t * stride_v]) : 0.0f;
    const float w = (weight != nullptr && in_range) ? load_as_f32(weight, weight_dtype, t) : 1.0f;
    lse[row] = bm + ls;
    row_max[row] = bm;
    row_logsum[row] = ls;
    row_loss[row] = w * (ls - pred + bm);      // the reference's order of operations (line 78)
    row_weight[row] = w;
  }
}

// L = sum(row_loss) / (weighted ? sum(row_weight) : M), rounded once to the output type; the
// denominator is also written to *denominator (fp32) for backward.  One block; lane sums in a fixed
// order.
__global__ void __launch_bounds__(1024)
ce_finish_kernel(const float* __restrict__ row_loss, const float* __restrict__ row_weight, long long M, int weighted,
                 void* out, int out_dtype, float* denominator) {
  __shared__ double sl[1024], sw[1024];
  double l = 0.0, w = 0.0;
  for (long long i = threadIdx.x; i < M; i += 1024) {
    l += row_loss[i];
    w += row_weight[i];
  }
  sl[threadIdx.x] = l;
  sw[threadIdx.x] = w;
  __syncthreads();
  for (int off = 512; off > 0; off >>= 1) {
    if (threadIdx.x < off) {
      sl[threadIdx.x] += sl[threadIdx.x + off];
      sw[threadIdx.x] += sw[threadIdx.x + off];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const double denom = weighted ? sw[0] : static_cast<double>(M);
    *denominator = static_cast<float>(denom);
    store_from_f32(out, out_dtype, 0, M > 0 ? static_cast<float>(sl[0] / denom) : 0.0f);
  }
}

// dx_ij = dL * s_i * (exp((x_ij - max_i) - logsum_i) - [j == t_i]), one block per row.
template <class T, class G>
__global__ void __launch_bounds__(kCeThreads)
ce_backward_kernel(const T* __restrict__ x, long long stride_m, long long stride_v, const long long* __restrict__ target,
                   const void* __restrict__ weight, int weight_dtype, const float* __restrict__ row_max,
                   const float* __restrict__ row_logsum, const float* __restrict__ denominator, const void* __restrict__ out_grad, int out_grad_dtype,
                   G* __restrict__ dx, long long ld_dx, int V) {
  const long long row = blockIdx.x;
  const T* xr = x + row * stride_m;
  G* dr = dx + row * ld_dx;
  const long long t = target[row];
  const bool in_range = t >= 0 && t < V;
  const float w = (weight != nullptr && in_range) ? load_as_f32(weight, weight_dtype, t) : 1.0f;
  const float scale = load_as_f32(out_grad, out_grad_dtype, 0) * w / *denominator;
  const float mx = row_max[row], ls = row_logsum[row];
  constexpr int kPer = 16 / sizeof(T);
  const bool vec = stride_v == 1 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(dr) & (kPer * sizeof(G) - 1)) == 0;
  const int whole = vec ? V / kPer : 0;
  for (int g = threadIdx.x; g < whole; g += kCeThreads) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(xr) + g);
    const T* e = reinterpret_cast<const T*>(&q);
    alignas(16) G o[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int c = g * kPer + i;
      const float p = __expf((to_f32<T>(e[i]) - mx) - ls);
      o[i] = from_f32<G>(scale * (p - (c == t ? 1.0f : 0.0f)));
    }
    if constexpr (kPer * sizeof(G) == 16) {
      reinterpret_cast<uint4*>(dr)[g] = *reinterpret_cast<const uint4*>(o);
    } else {   // a 16-bit input with an fp32 gradient: 32 bytes
      reinterpret_cast<uint4*>(dr)[2 * g] = reinterpret_cast<const uint4*>(o)[0];
      reinterpret_cast<uint4*>(dr)[2 * g + 1] = reinterpret_cast<const uint4*>(o)[1];
    }
  }
  for (int c = whole * kPer + threadIdx.x; c < V; c += kCeThreads) {
    const float p = __expf((to_f32<T>(xr[static_cast<long long>(c) * stride_v]) - mx) - ls);
    dr[c] = from_f32<G>(scale * (p - (c == t ? 1.0f : 0.0f)));
  }
}

}  // namespace ab200
