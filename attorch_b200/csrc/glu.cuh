// Gated linear unit with an arbitrary activation (the reference's glu_forward_kernel and
// glu_backward_kernel, attorch/glu_kernels.py:13-105, as launched by attorch/glu_layer.py:58-116):
//
//   forward    y  = x1 * act(x2)
//   backward   dx1 = dy * act(x2),   dx2 = dy * x1 * act'(x2)
//
// where x1, x2 are the halves of the input along the gated dimension.  The reference first copies
// both halves into contiguous tensors, runs a flat kernel and, in backward, concatenates the two
// gradients again.  Here the input is addressed in place as [outer, 2 * inner] (outer = product of
// the dimensions before the gated one, inner = half its extent times the product of the dimensions
// after it): x1 is the first `inner` elements of a row, x2 the rest, y is [outer, inner], and dx is
// written straight into its [outer, 2 * inner] layout.  HBM-bound: 3 n e bytes forward and 5 n e
// backward for n output elements of e bytes (the reference's data flow moves 7 n e and 9 n e).
#pragma once
#include "act_math.cuh"
#include "common.cuh"

namespace ab200 {

template <class T>
struct Raw8 {                      // 8 elements as loaded: one or two 16-byte words
  static constexpr int kWords = sizeof(T) * 8 / 16;
  uint4 q[kWords];
  __device__ __forceinline__ void load(const T* p) {
#pragma unroll
    for (int w = 0; w < kWords; ++w) q[w] = __ldg(reinterpret_cast<const uint4*>(p) + w);
  }
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f32<T>(reinterpret_cast<const T*>(q)[i]);
  }
};

template <class T>
__device__ __forceinline__ void load8(const T* p, bool vec, long long left, float (&v)[8]) {
  if (vec) {
    Raw8<T> r;
    r.load(p);
    r.unpack(v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = i < left ? to_f32<T>(p[i]) : 0.0f;
  }
}

template <class T>
__device__ __forceinline__ void store8(T* p, bool vec, long long left, const float (&v)[8]) {
  constexpr int kWords = sizeof(T) * 8 / 16;
  if (vec) {
    alignas(16) T o[8];
    pack8<T>(v, o);
#pragma unroll
    for (int w = 0; w < kWords; ++w) reinterpret_cast<uint4*>(p)[w] = reinterpret_cast<const uint4*>(o)[w];
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < left) p[i] = from_f32<T>(v[i]);
  }
}

// The arithmetic of one group of 8 elements: a = x1, b = x2, gy = dy (backward only).
template <class T, bool kBackward>
__device__ __forceinline__ void glu_group(float (&a)[8], float (&b)[8], const float (&gy)[8], T* out, long long row,
                                          long long col, long long inner, bool vec, long long left, int act,
                                          float param) {
  if constexpr (!kBackward) {
    act_fwd_inplace(b, act, param);
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] *= b[i];
    store8<T>(out + row * inner + col, vec, left, a);
  } else {
    float g1[8], g2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      g1[i] = b[i];
      g2[i] = gy[i] * a[i];
    }
    act_fwd_inplace(g1, act, param);
#pragma unroll
    for (int i = 0; i < 8; ++i) g1[i] *= gy[i];
    act_grad_mul(g2, b, act, param);
    T* d1 = out + row * 2 * inner + col;
    store8<T>(d1, vec, left, g1);
    store8<T>(d1 + inner, vec, left, g2);
  }
}

// One thread handles 8 consecutive elements of one row's half.  groups_per_row = ceil(inner / 8).
// `vec` (uniform): inner is a multiple of 8 and every base pointer is 16-byte aligned, so that all
// accesses are whole 16-byte words; then a thread takes two groups per trip and issues the loads of
// both before any arithmetic (the kernel is bound by memory latency, not by its instruction count).
template <class T, bool kBackward>
__global__ void __launch_bounds__(256)
glu_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out, long long outer,
           long long inner, long long groups_per_row, int act, float param, int vec) {
  const long long groups = outer * groups_per_row;
  const bool narrow = groups < (1ll << 32) && groups_per_row < (1ll << 32);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  auto locate = [&](long long g, long long& row, long long& col) {
    if (narrow) {      // 32-bit division where the sizes allow it
      const unsigned r = static_cast<unsigned>(g) / static_cast<unsigned>(groups_per_row);
      row = r;
      col = (static_cast<unsigned>(g) - r * static_cast<unsigned>(groups_per_row)) * 8ll;
    } else {
      row = g / groups_per_row;
      col = (g - row * groups_per_row) * 8;
    }
  };
  const long long first = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (vec) {
    for (long long g0 = first; g0 < groups; g0 += 2 * stride) {
      const long long g1 = g0 + stride < groups ? g0 + stride : g0;   // the last trip may repeat g0
      long long row[2], col[2];
      locate(g0, row[0], col[0]);
      locate(g1, row[1], col[1]);
      Raw8<T> ra[2], rb[2], rg[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const T* x1 = x + row[u] * 2 * inner + col[u];
        ra[u].load(x1);
        rb[u].load(x1 + inner);
        if constexpr (kBackward) rg[u].load(dy + row[u] * inner + col[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u == 1 && g1 == g0) break;
        float a[8], b[8], gy[8] = {};
        ra[u].unpack(a);
        rb[u].unpack(b);
        if constexpr (kBackward) rg[u].unpack(gy);
        glu_group<T, kBackward>(a, b, gy, out, row[u], col[u], inner, true, 8, act, param);
      }
    }
  } else {
    for (long long g = first; g < groups; g += stride) {
      long long row, col;
      locate(g, row, col);
      const long long left = inner - col;
      const T* x1 = x + row * 2 * inner + col;
      float a[8], b[8], gy[8] = {};
      load8<T>(x1, false, left, a);
      load8<T>(x1 + inner, false, left, b);
      if constexpr (kBackward) load8<T>(dy + row * inner + col, false, left, gy);
      glu_group<T, kBackward>(a, b, gy, out, row, col, inner, false, left, act, param);
    }
  }
}

}  // namespace ab200
