// Standalone activation layers with fused dropout (the reference's act_func_forward_kernel and
// act_func_backward_kernel, attorch/act_kernels.py:840-927, with apply_dropout /
// apply_dropout_grad, attorch/dropout_kernels.py:12-46): flat, HBM-bound, 8 elements per thread.
//
//   forward    y  = keep ? act(x) / (1 - p) : 0          keep = (u(seed, index) >= p)
//   backward   dx = (keep ? dy / (1 - p) : 0) * act'(x)
//
// u(seed, index) comes from a counter-based generator (Philox 4x32 with 10 rounds, key = (seed, 0)),
// so forward and backward see the same mask without storing it.  Two streams:
//
//   reference (default)  the numbers Triton's tl.rand(seed, offset) yields, which the reference draws
//                        (attorch/dropout_kernels.py:26): counter (uint32(index), 0, 0, 0), first output
//                        word w, as int32 mirrored onto [0, 2^31) (w < 0 ? -w - 1 : w), converted to
//                        fp32 and scaled by 4.6566127342e-10.  Same seed, same mask as the reference.
//                        One Philox block per element: 17 32x32->64-bit multiplies, which makes the
//                        2-byte kernels ALU-bound rather than HBM-bound.
//   packed               counter (index / 4, 0, 0, 0), word index % 4, top 24 bits -> [0, 1): one block
//                        per four elements, a quarter of the integer work; a different mask.
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

enum DropoutStream : int { DROPOUT_OFF = 0, DROPOUT_REFERENCE = 1, DROPOUT_PACKED = 2 };

// A word taken as int32 and mirrored onto [0, 2^31): w < 0 ? -w - 1 : w.
__host__ __device__ __forceinline__ uint32_t mirrored_word(uint32_t w) {
  return w ^ static_cast<uint32_t>(static_cast<int32_t>(w) >> 31);
}

__host__ __device__ __forceinline__ float reference_uniform_of(uint32_t mirrored) {
  return static_cast<float>(static_cast<int32_t>(mirrored)) * 4.6566127342e-10f;
}

// First output word of the block with counter (c0, 0, 0, 0) -> uniform fp32 in [0, 1), as tl.rand does it.
__host__ __device__ __forceinline__ float reference_uniform(uint32_t seed, uint32_t c0) {
  uint32_t r[4];
  philox4x32_10(c0, 0u, 0u, 0u, seed, 0u, r);
  return reference_uniform_of(mirrored_word(r[0]));
}

__host__ __device__ __forceinline__ float packed_uniform(uint32_t word) {
  return static_cast<float>(word >> 8) * (1.0f / 16777216.0f);
}

// Uniform number in [0, 1) for element `index` of the stream `seed`.
__host__ __device__ __forceinline__ float dropout_uniform(uint32_t seed, uint64_t index, int stream) {
  if (stream == DROPOUT_PACKED) {
    uint32_t r[4];
    philox4x32_10(static_cast<uint32_t>(index >> 2), static_cast<uint32_t>(index >> 34), 0u, 0u, seed, 0u, r);
    return packed_uniform(r[index & 3]);
  }
  return reference_uniform(seed, static_cast<uint32_t>(index));
}

// The integer t with  u < drop_p  <=>  m < t, where m is the mirrored word (reference stream) or the
// raw word (packed stream) u is made from: both conversions are monotonic in m, so the float
// comparison has an exact integer form.  0 <= drop_p < 1.
inline uint32_t dropout_threshold(float drop_p, int stream) {
  if (stream == DROPOUT_PACKED) {
    // float(word >> 8) / 2^24 < p  <=>  (word >> 8) < ceil(p 2^24)  <=>  word < ceil(p 2^24) << 8.
    const double scaled = static_cast<double>(drop_p) * 16777216.0;
    uint64_t t = static_cast<uint64_t>(scaled);
    if (static_cast<double>(t) < scaled) ++t;
    return static_cast<uint32_t>(t << 8);
  }
  // Smallest m in [0, 2^31] with float(m) * scale >= drop_p, by bisection.
  uint64_t lo = 0, hi = 1ull << 31;   // invariant: u(m) < p for m < lo, u(m) >= p for m >= hi
  while (lo < hi) {
    const uint64_t mid = (lo + hi) / 2;
    if (reference_uniform_of(static_cast<uint32_t>(mid)) < drop_p) lo = mid + 1; else hi = mid;
  }
  return static_cast<uint32_t>(lo);
}

// The arithmetic of one group of 8 elements: res = act(xv) or gv * act'(xv), then the dropout mask of
// elements base .. base + 7.
template <bool kBackward>
__device__ __forceinline__ void act_group(const float (&xv)[8], const float (&gv)[8], float (&res)[8],
                                          long long base, int act, float param, float keep_scale,
                                          uint32_t seed, int dropout, uint32_t threshold) {
  if constexpr (kBackward) {
#pragma unroll
    for (int i = 0; i < 8; ++i) res[i] = gv[i];
    act_grad_mul(res, xv, act, param);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) res[i] = xv[i];
    act_fwd_inplace(res, act, param);
  }
  // "u < drop_p" as an integer comparison with dropout_threshold(): no int -> float conversion.
  if (dropout == DROPOUT_REFERENCE) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t r[4];
      philox4x32_10(static_cast<uint32_t>(base + i), 0u, 0u, 0u, seed, 0u, r);
      res[i] = (mirrored_word(r[0]) < threshold) ? 0.0f : res[i] * keep_scale;
    }
  } else if (dropout == DROPOUT_PACKED) {
    // Two Philox blocks cover the 8 consecutive indices of this group.
    uint32_t a[4], b[4];
    const uint64_t blk = static_cast<uint64_t>(base) >> 2;
    philox4x32_10(static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32), 0u, 0u, seed, 0u, a);
    philox4x32_10(static_cast<uint32_t>(blk + 1), static_cast<uint32_t>((blk + 1) >> 32), 0u, 0u, seed, 0u, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      res[i] = (a[i] < threshold) ? 0.0f : res[i] * keep_scale;
      res[4 + i] = (b[i] < threshold) ? 0.0f : res[4 + i] * keep_scale;
    }
  }
}

// kBackward = false: y = dropout(act(x));  true: dx = dropout_grad(dy) * act'(x).
// Whole, 16-byte aligned groups go two per thread and trip with every load issued before the
// arithmetic (the kernel is bound by memory latency unless the dropout generator dominates); the
// ragged tail and unaligned tensors take the element-wise path.
template <class T, bool kBackward>
__global__ void __launch_bounds__(256)
act_elementwise_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out, long long n,
                       int act, float param, float drop_p, uint32_t seed, int dropout, uint32_t threshold) {
  const float keep_scale = dropout ? 1.0f / (1.0f - drop_p) : 1.0f;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                       (!kBackward || (reinterpret_cast<uintptr_t>(dy) & 15) == 0);
  constexpr int kWords = sizeof(T) * 8 / 16;
  const long long whole = aligned ? n / 8 : 0;             // groups handled 16 bytes at a time
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (long long g0 = first; g0 < whole; g0 += 2 * stride) {
    const long long g1 = g0 + stride < whole ? g0 + stride : g0;   // the last trip may repeat g0
    const long long gs[2] = {g0, g1};
    uint4 xq[2][kWords], gq[2][kWords];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
#pragma unroll
      for (int w = 0; w < kWords; ++w) xq[u][w] = __ldg(reinterpret_cast<const uint4*>(x + gs[u] * 8) + w);
      if constexpr (kBackward) {
#pragma unroll
        for (int w = 0; w < kWords; ++w) gq[u][w] = __ldg(reinterpret_cast<const uint4*>(dy + gs[u] * 8) + w);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && g1 == g0) break;
      float xv[8], gv[8], res[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xv[i] = to_f32<T>(reinterpret_cast<const T*>(xq[u])[i]);
        gv[i] = kBackward ? to_f32<T>(reinterpret_cast<const T*>(gq[u])[i]) : 0.0f;
      }
      act_group<kBackward>(xv, gv, res, gs[u] * 8, act, param, keep_scale, seed, dropout, threshold);
      alignas(16) T o[8];
      pack8<T>(res, o);
#pragma unroll
      for (int w = 0; w < kWords; ++w)
        reinterpret_cast<uint4*>(out + gs[u] * 8)[w] = reinterpret_cast<const uint4*>(o)[w];
    }
  }
  // Element-wise remainder: everything if the tensors are not 16-byte aligned, else the last n % 8.
  const long long groups = (n + 7) / 8;
  for (long long g = whole + first; g < groups; g += stride) {
    const long long base = g * 8;
    float xv[8], gv[8], res[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool in = base + i < n;
      xv[i] = in ? to_f32<T>(x[base + i]) : 0.0f;
      gv[i] = (kBackward && in) ? to_f32<T>(dy[base + i]) : 0.0f;
    }
    act_group<kBackward>(xv, gv, res, base, act, param, keep_scale, seed, dropout, threshold);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (base + i < n) out[base + i] = from_f32<T>(res[i]);
  }
}

}  // namespace ab200
