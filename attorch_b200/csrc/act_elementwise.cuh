// Standalone activation layers with fused dropout (the reference's act_func_forward_kernel and
// act_func_backward_kernel, attorch/act_kernels.py:840-927, with apply_dropout /
// apply_dropout_grad, attorch/dropout_kernels.py:12-46): flat, HBM-bound, 8 elements per thread.
//
//   forward    y  = keep ? act(x) / (1 - p) : 0          keep = (u(seed, index) >= p)
//   backward   dx = (keep ? dy / (1 - p) : 0) * act'(x)
//
// u(seed, index) is a counter-based generator (Philox 4x32 with 10 rounds, key = (seed, 0), counter
// = (index / 4, 0, 0, 0), word index % 4, top 24 bits -> [0, 1)), so forward and backward see the
// same mask without storing it, as in the reference; the stream itself is this library's own (the
// reference's comes from Triton's tl.rand and is not reproduced bit for bit).
#pragma once
#include "act_math.cuh"
#include "common.cuh"

namespace ab200 {

__host__ __device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                      uint32_t k0, uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = static_cast<uint32_t>(p0);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Uniform number in [0, 1) for element `index` of the stream `seed`.
__host__ __device__ __forceinline__ float dropout_uniform(uint32_t seed, uint64_t index) {
  uint32_t r[4];
  philox4x32_10(static_cast<uint32_t>(index >> 2), static_cast<uint32_t>(index >> 34), 0u, 0u, seed, 0u, r);
  return static_cast<float>(r[index & 3] >> 8) * (1.0f / 16777216.0f);
}

// kBackward = false: y = dropout(act(x));  true: dx = dropout_grad(dy) * act'(x).
template <class T, bool kBackward>
__global__ void __launch_bounds__(256)
act_elementwise_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out, long long n,
                       int act, float param, float drop_p, uint32_t seed, int dropout) {
  const float keep_scale = dropout ? 1.0f / (1.0f - drop_p) : 1.0f;
  const long long groups = (n + 7) / 8;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                       (!kBackward || (reinterpret_cast<uintptr_t>(dy) & 15) == 0);
  constexpr int kWords = sizeof(T) * 8 / 16;
  for (long long gidx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; gidx < groups;
       gidx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long base = gidx * 8;
    const bool full = aligned && base + 8 <= n;
    float xv[8], gv[8];
    if (full) {
      uint4 xq[kWords], gq[kWords];
#pragma unroll
      for (int w = 0; w < kWords; ++w) xq[w] = __ldg(reinterpret_cast<const uint4*>(x + base) + w);
      if constexpr (kBackward) {
#pragma unroll
        for (int w = 0; w < kWords; ++w) gq[w] = __ldg(reinterpret_cast<const uint4*>(dy + base) + w);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xv[i] = to_f32<T>(reinterpret_cast<const T*>(xq)[i]);
        gv[i] = kBackward ? to_f32<T>(reinterpret_cast<const T*>(gq)[i]) : 0.0f;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool in = base + i < n;
        xv[i] = in ? to_f32<T>(x[base + i]) : 0.0f;
        gv[i] = (kBackward && in) ? to_f32<T>(dy[base + i]) : 0.0f;
      }
    }
    float res[8];
    if constexpr (kBackward) {
#pragma unroll
      for (int i = 0; i < 8; ++i) res[i] = gv[i];
      act_grad_mul(res, xv, act, param);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) res[i] = xv[i];
      act_fwd_inplace(res, act, param);
    }
    if (dropout) {
      // Two Philox blocks cover the 8 consecutive indices of this group.
      uint32_t r[8];
      uint32_t a[4], b[4];
      const uint64_t blk = static_cast<uint64_t>(base) >> 2;
      philox4x32_10(static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32), 0u, 0u, seed, 0u, a);
      philox4x32_10(static_cast<uint32_t>(blk + 1), static_cast<uint32_t>((blk + 1) >> 32), 0u, 0u, seed, 0u, b);
#pragma unroll
      for (int i = 0; i < 4; ++i) { r[i] = a[i]; r[4 + i] = b[i]; }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float u = static_cast<float>(r[i] >> 8) * (1.0f / 16777216.0f);
        res[i] = (u < drop_p) ? 0.0f : res[i] * keep_scale;
      }
    }
    if (full) {
      alignas(16) T o[8];
      pack8<T>(res, o);
#pragma unroll
      for (int w = 0; w < kWords; ++w) reinterpret_cast<uint4*>(out + base)[w] = reinterpret_cast<const uint4*>(o)[w];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (base + i < n) out[base + i] = from_f32<T>(res[i]);
    }
  }
}

}  // namespace ab200
