// Layer normalisation over the rows of a matrix, forward and backward: the step in front of the first
// projection of a transformer block (reference: attorch/layer_norm_kernels.py:14-221, launched from
// attorch/layer_norm_layer.py:19-157; the caller is examples/wikitext-2/gpt.py:82).
//
//   forward   mean_i = sum_j x_ij / F,  d_ij = x_ij - mean_i,  inv_std_i = rsqrt(sum_j d_ij^2 / F + eps)
//             y_ij = d_ij * inv_std_i [* w_j [+ b_j]]
//   backward  p_ij = (x_ij - mean_i) * inv_std_i,  g_ij = w_j * dy_ij
//             dx_ij = inv_std_i * (g_ij - (p_ij * sum_j(p_ij g_ij) / F + sum_j g_ij / F))
//             dw_j = sum_i dy_ij p_ij,  db_j = sum_i dy_ij
//
// Both kernels are bound by HBM and touch every element once: a row is loaded into registers (16 elements
// per thread, 16-byte loads), both row sums are taken from the registers, and the result is written from
// them.  A row belongs to a group of R threads: one warp for rows of up to 512 elements (eight rows per
// block), 256 threads up to 4096, 512 threads beyond; elements past 16 * R are read again (from L2) in
// the second and third pass.  Blocks loop over rows, so weight and bias are loaded once per block, and
// in backward each thread keeps the weight- and bias-gradient sums of its own columns in registers over
// all rows of its block; one partial row per row group goes to the workspace, and ln_param_finish_kernel
// adds the partials in a fixed order.  (The reference re-reads x and dy in a second pass over the same
// data for these sums only when its programs hold several rows; it writes one partial per program.)
//
// The stored type of y may differ from x's: fp32 for a 16-bit x (the reference's autocast_to_fp32), or
// a 16-bit y for an fp32 x - the operand type of the projection that follows, which saves that layer's
// cast pass over the activations.  Every value is computed in fp32 and rounded once by the store, as in
// the reference (it widens the loaded row, line 84, and the store narrows, line 102).  All sums have a
// fixed order: results do not depend on scheduling.
#pragma once
#include <type_traits>

#include "act_math.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace ab200 {

constexpr int kLnCache = 16;   // elements of a row that one thread keeps in registers

// V elements of T as loaded: one scalar, or an 8- or 16-byte word.
template <class T, int V>
struct LnRawType {
  static_assert(V * sizeof(T) == 8 || V * sizeof(T) == 16, "an 8- or 16-byte access");
  using type = std::conditional_t<V * sizeof(T) == 16, uint4, uint2>;
};
template <class T>
struct LnRawType<T, 1> {
  using type = T;
};
template <class T, int V>
using LnRaw = typename LnRawType<T, V>::type;

// V elements of T starting at p, which is aligned to V * sizeof(T) bytes, as one access.
template <class T, int V>
__device__ __forceinline__ LnRaw<T, V> ln_load_raw(const T* p) {
  return *reinterpret_cast<const LnRaw<T, V>*>(p);
}

template <class T, int V>
__device__ __forceinline__ LnRaw<T, V> ln_zero_raw() {
  if constexpr (V == 1) return from_f32<T>(0.0f);
  else if constexpr (V * sizeof(T) == 16) return make_uint4(0u, 0u, 0u, 0u);
  else return make_uint2(0u, 0u);
}

template <class T, int V>
__device__ __forceinline__ void ln_unpack(const LnRaw<T, V>& q, float* v) {
  const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
  for (int i = 0; i < V; ++i) v[i] = to_f32<T>(e[i]);
}

template <class T, int V>
__device__ __forceinline__ void ln_load(const T* p, float* v) {
  const LnRaw<T, V> q = ln_load_raw<T, V>(p);
  ln_unpack<T, V>(q, v);
}

template <class T, int V>
__device__ __forceinline__ void ln_store(T* p, const float* v) {
  constexpr int kBytes = V * static_cast<int>(sizeof(T));
  if constexpr (V == 1) {
    *p = from_f32<T>(v[0]);
  } else if constexpr (kBytes == 16) {
    uint4 q;
    T* e = reinterpret_cast<T*>(&q);
#pragma unroll
    for (int i = 0; i < V; ++i) e[i] = from_f32<T>(v[i]);
    *reinterpret_cast<uint4*>(p) = q;
  } else {
    uint2 q;
    T* e = reinterpret_cast<T*>(&q);
#pragma unroll
    for (int i = 0; i < V; ++i) e[i] = from_f32<T>(v[i]);
    *reinterpret_cast<uint2*>(p) = q;
  }
}

// Sums a and b over the R threads of a row group; every thread of the block must call it.  Groups of
// more than one warp go through shared memory (two buffers, used in turn, so one barrier per call).
template <int R, int kThreads>
__device__ __forceinline__ float2 ln_group_sum(float a, float b, float2 (*scratch)[kThreads / 32], int& phase) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    a += __shfl_xor_sync(0xFFFFFFFFu, a, off);
    b += __shfl_xor_sync(0xFFFFFFFFu, b, off);
  }
  if constexpr (R > 32) {
    static_assert(R == kThreads, "a row group larger than a warp is the whole block");
    if ((threadIdx.x & 31) == 0) scratch[phase][threadIdx.x >> 5] = make_float2(a, b);
    __syncthreads();
    a = 0.0f;
    b = 0.0f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) {
      a += scratch[phase][w].x;
      b += scratch[phase][w].y;
    }
    phase ^= 1;
  }
  return make_float2(a, b);
}

template <int A, int B>
struct LnMax {
  static constexpr int value = A > B ? A : B;
};

template <class TIn, class TOut, int R, bool kVec>
__global__ void __launch_bounds__(R < 256 ? 256 : R)
ln_forward_kernel(const TIn* __restrict__ x, long long ldx, const void* __restrict__ w, const void* __restrict__ b,
                  int param_dtype, float* __restrict__ mean, float* __restrict__ inv_std, TOut* __restrict__ y,
                  long long ldy, long long rows, int F, float eps) {
  constexpr int kThreads = R < 256 ? 256 : R;
  constexpr int kRowsPerBlock = kThreads / R;
  constexpr int V = kVec ? 16 / LnMax<sizeof(TIn), sizeof(TOut)>::value : 1;
  constexpr int kG = kLnCache / V;          // groups of V elements each thread keeps
  __shared__ float2 scratch[2][kThreads / 32];
  int phase = 0;
  const int t = threadIdx.x % R, slot = threadIdx.x / R;
  const int groups = F / V;
  const float feat = static_cast<float>(F);

  float wc[kLnCache], bc[kLnCache];
#pragma unroll
  for (int i = 0; i < kG; ++i) {
    const int g = t + i * R;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const bool in = g < groups;
      wc[i * V + j] = (w != nullptr && in) ? load_as_f32(w, param_dtype, g * V + j) : 1.0f;
      bc[i * V + j] = (b != nullptr && in) ? load_as_f32(b, param_dtype, g * V + j) : 0.0f;
    }
  }

  const long long row_blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  // The part of row block rb that this thread keeps, as loaded; zeros past the end of the problem.
  auto fetch = [&](long long rb, LnRaw<TIn, V> (&dst)[kG]) {
    const long long r = rb * kRowsPerBlock + slot;
    const bool ok = rb < row_blocks && r < rows;
    const TIn* p = x + (ok ? r : 0) * ldx;
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      const int g = t + i * R;
      dst[i] = (ok && g < groups) ? ln_load_raw<TIn, V>(p + g * V) : ln_zero_raw<TIn, V>();
    }
  };
  LnRaw<TIn, V> cur[kG], nxt[kG];
  fetch(blockIdx.x, cur);
  for (long long rb = blockIdx.x; rb < row_blocks; rb += gridDim.x) {
    // The next row's loads are in flight while this row is summed, normalised and stored.
    fetch(rb + gridDim.x, nxt);
    const long long row = rb * kRowsPerBlock + slot;
    const bool live = row < rows;
    const TIn* xr = x + (live ? row : 0) * ldx;
    TOut* yr = y + (live ? row : 0) * ldy;

    float xc[kLnCache];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      ln_unpack<TIn, V>(cur[i], &xc[i * V]);
#pragma unroll
      for (int j = 0; j < V; ++j) s += xc[i * V + j];
    }
    if (live) {
      for (int g = t + kG * R; g < groups; g += R) {
        float v[V];
        ln_load<TIn, V>(xr + g * V, v);
#pragma unroll
        for (int j = 0; j < V; ++j) s += v[j];
      }
    }
    const float mu = ln_group_sum<R, kThreads>(s, 0.0f, scratch, phase).x / feat;

    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      const bool in = t + i * R < groups;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float d = in ? xc[i * V + j] - mu : 0.0f;
        xc[i * V + j] = d;
        q += d * d;
      }
    }
    if (live) {
      for (int g = t + kG * R; g < groups; g += R) {
        float v[V];
        ln_load<TIn, V>(xr + g * V, v);
#pragma unroll
        for (int j = 0; j < V; ++j) q += (v[j] - mu) * (v[j] - mu);
      }
    }
    const float rs = rsqrtf(ln_group_sum<R, kThreads>(q, 0.0f, scratch, phase).x / feat + eps);
    if (live && t == 0 && mean != nullptr) {
      mean[row] = mu;
      inv_std[row] = rs;
    }
    if (live) {
#pragma unroll
      for (int i = 0; i < kG; ++i) {
        const int g = t + i * R;
        if (g < groups) {
          float o[V];
#pragma unroll
          for (int j = 0; j < V; ++j) o[j] = xc[i * V + j] * rs * wc[i * V + j] + bc[i * V + j];
          ln_store<TOut, V>(yr + g * V, o);
        }
      }
      for (int g = t + kG * R; g < groups; g += R) {
        float v[V], o[V];
        ln_load<TIn, V>(xr + g * V, v);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float wj = w != nullptr ? load_as_f32(w, param_dtype, g * V + j) : 1.0f;
          const float bj = b != nullptr ? load_as_f32(b, param_dtype, g * V + j) : 0.0f;
          o[j] = (v[j] - mu) * rs * wj + bj;
        }
        ln_store<TOut, V>(yr + g * V, o);
      }
    }
#pragma unroll
    for (int i = 0; i < kG; ++i) cur[i] = nxt[i];
  }
}

// kParams: also accumulate the weight- and bias-gradient sums of this thread's columns (requires
// F <= kLnCache * R, so that every column is one that a thread keeps).  wpart / bpart: one row of F
// floats per row group of the grid, [gridDim.x * rows per block, F].
template <class TIn, class TDy, class TDx, int R, bool kVec, bool kParams>
__global__ void __launch_bounds__(R < 256 ? 256 : R)
ln_backward_kernel(const TDy* __restrict__ dy, long long lddy, const TIn* __restrict__ x, long long ldx,
                   const float* __restrict__ mean, const float* __restrict__ inv_std, const void* __restrict__ w,
                   int param_dtype, TDx* __restrict__ dx, long long lddx, float* __restrict__ wpart,
                   float* __restrict__ bpart, long long rows, int F) {
  constexpr int kThreads = R < 256 ? 256 : R;
  constexpr int kRowsPerBlock = kThreads / R;
  constexpr int V =
      kVec ? 16 / LnMax<LnMax<sizeof(TIn), sizeof(TDy)>::value, sizeof(TDx)>::value : 1;
  constexpr int kG = kLnCache / V;
  __shared__ float2 scratch[2][kThreads / 32];
  int phase = 0;
  const int t = threadIdx.x % R, slot = threadIdx.x / R;
  const int groups = F / V;
  const float feat = static_cast<float>(F);

  float wc[kLnCache];
#pragma unroll
  for (int i = 0; i < kG; ++i) {
    const int g = t + i * R;
#pragma unroll
    for (int j = 0; j < V; ++j)
      wc[i * V + j] = (w != nullptr && g < groups) ? load_as_f32(w, param_dtype, g * V + j) : 1.0f;
  }
  float wacc[kParams ? kLnCache : 1], bacc[kParams ? kLnCache : 1];
  if constexpr (kParams) {
#pragma unroll
    for (int i = 0; i < kLnCache; ++i) wacc[i] = bacc[i] = 0.0f;
  }

  const long long row_blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  // The parts of x and dy of row block rb that this thread keeps, as loaded; zeros past the end.
  auto fetch = [&](long long rb, LnRaw<TIn, V> (&xdst)[kG], LnRaw<TDy, V> (&gdst)[kG]) {
    const long long r = rb * kRowsPerBlock + slot;
    const bool ok = rb < row_blocks && r < rows;
    const TIn* px = x + (ok ? r : 0) * ldx;
    const TDy* pg = dy + (ok ? r : 0) * lddy;
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      const int g = t + i * R;
      const bool in = ok && g < groups;
      xdst[i] = in ? ln_load_raw<TIn, V>(px + g * V) : ln_zero_raw<TIn, V>();
      gdst[i] = in ? ln_load_raw<TDy, V>(pg + g * V) : ln_zero_raw<TDy, V>();
    }
  };
  // With 512 threads (at most 128 registers each) the sums of the parameter gradients leave no room for
  // a second row.
  constexpr bool kPrefetch = !(R == 512 && kParams);
  LnRaw<TIn, V> xcur[kG], xnxt[kPrefetch ? kG : 1];
  LnRaw<TDy, V> gcur[kG], gnxt[kPrefetch ? kG : 1];
  fetch(blockIdx.x, xcur, gcur);
  for (long long rb = blockIdx.x; rb < row_blocks; rb += gridDim.x) {
    // The next row's loads are in flight while this row is reduced and its gradient stored.
    if constexpr (kPrefetch) fetch(rb + gridDim.x, xnxt, gnxt);
    const long long row = rb * kRowsPerBlock + slot;
    const bool live = row < rows;
    const TIn* xr = x + (live ? row : 0) * ldx;
    const TDy* gr = dy + (live ? row : 0) * lddy;
    TDx* dr = dx + (live ? row : 0) * lddx;
    const float mu = live ? mean[row] : 0.0f;
    const float rs = live ? inv_std[row] : 0.0f;

    float pc[kLnCache], gc[kLnCache];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      const int g = t + i * R;
      ln_unpack<TIn, V>(xcur[i], &pc[i * V]);
      ln_unpack<TDy, V>(gcur[i], &gc[i * V]);
      if (live && g < groups) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const int e = i * V + j;
          const float p = (pc[e] - mu) * rs;
          pc[e] = p;
          if constexpr (kParams) {
            wacc[e] += gc[e] * p;
            bacc[e] += gc[e];
          }
          gc[e] *= wc[e];
          s1 += p * gc[e];
          s2 += gc[e];
        }
      }
    }
    if (live) {
      for (int g = t + kG * R; g < groups; g += R) {
        float xv[V], gv[V];
        ln_load<TIn, V>(xr + g * V, xv);
        ln_load<TDy, V>(gr + g * V, gv);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float wj = w != nullptr ? load_as_f32(w, param_dtype, g * V + j) : 1.0f;
          const float p = (xv[j] - mu) * rs;
          s1 += p * (wj * gv[j]);
          s2 += wj * gv[j];
        }
      }
    }
    const float2 sums = ln_group_sum<R, kThreads>(s1, s2, scratch, phase);
    const float c1 = sums.x / feat, c2 = sums.y / feat;
    if (live) {
#pragma unroll
      for (int i = 0; i < kG; ++i) {
        const int g = t + i * R;
        if (g < groups) {
          float o[V];
#pragma unroll
          for (int j = 0; j < V; ++j) o[j] = rs * (gc[i * V + j] - (pc[i * V + j] * c1 + c2));
          ln_store<TDx, V>(dr + g * V, o);
        }
      }
      for (int g = t + kG * R; g < groups; g += R) {
        float xv[V], gv[V], o[V];
        ln_load<TIn, V>(xr + g * V, xv);
        ln_load<TDy, V>(gr + g * V, gv);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float wj = w != nullptr ? load_as_f32(w, param_dtype, g * V + j) : 1.0f;
          const float p = (xv[j] - mu) * rs;
          o[j] = rs * (wj * gv[j] - (p * c1 + c2));
        }
        ln_store<TDx, V>(dr + g * V, o);
      }
    }
    if constexpr (kPrefetch) {
#pragma unroll
      for (int i = 0; i < kG; ++i) {
        xcur[i] = xnxt[i];
        gcur[i] = gnxt[i];
      }
    } else {
      fetch(rb + gridDim.x, xcur, gcur);
    }
  }

  if constexpr (kParams) {
    const long long part = static_cast<long long>(blockIdx.x) * kRowsPerBlock + slot;
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      const int g = t + i * R;
      if (g < groups) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          wpart[part * F + g * V + j] = wacc[i * V + j];
          if (bpart != nullptr) bpart[part * F + g * V + j] = bacc[i * V + j];
        }
      }
    }
  }
}

constexpr int kLnMaxStages = 16;     // rows in flight per block of the staged backward kernel
constexpr int kLnStatChunk = 64;     // row statistics fetched at a time

// The backward pass with rows staged in shared memory: one or two blocks of R threads per SM; one thread keeps
// `stages` rows of x and dy (the rows blockIdx.x, blockIdx.x + gridDim.x, ...) in flight as untiled bulk
// copies, each pair completing on its stage's mbarrier, so the bytes in flight do not depend on how many
// registers or warps the block has - the register variant above, with one row ahead, stops near half of
// the HBM bandwidth.  Every thread then takes its columns of the row from shared memory; the arithmetic
// and the order of every sum are those of ln_backward_kernel.  The block barrier inside the row sums
// doubles as the signal that a stage has been read and may be refilled.  Requires 16-byte aligned rows,
// F % 8 == 0 and F <= kLnCache * R.  A wait on a stage has a time limit; when it runs out the block stores
// DEV_TIMEOUT_ROW_COPY in *status, waits (with the same limit) for its copies still in flight and returns.
template <class TIn, class TDy, class TDx, int R, bool kParams>
__global__ void __launch_bounds__(R, R <= 256 ? 2 : 1)
ln_backward_staged_kernel(const TDy* __restrict__ dy, long long lddy, const TIn* __restrict__ x, long long ldx,
                          const float* __restrict__ mean, const float* __restrict__ inv_std,
                          const void* __restrict__ w, int param_dtype, TDx* __restrict__ dx, long long lddx,
                          float* __restrict__ wpart, float* __restrict__ bpart, long long rows, int F, int stages,
                          int* status) {
  constexpr int V = 16 / LnMax<LnMax<sizeof(TIn), sizeof(TDy)>::value, sizeof(TDx)>::value;
  constexpr int kG = kLnCache / V;
  extern __shared__ __align__(128) unsigned char ln_stage_smem[];
  __shared__ __align__(8) uint64_t full[kLnMaxStages];
  __shared__ float2 scratch[2][R / 32];
  __shared__ float stat_mean[kLnStatChunk], stat_rs[kLnStatChunk];
  int phase = 0;
  const int t = threadIdx.x;
  const int groups = F / V;
  const float feat = static_cast<float>(F);
  const uint32_t xbytes = static_cast<uint32_t>(F) * sizeof(TIn), gbytes = static_cast<uint32_t>(F) * sizeof(TDy);
  const uint32_t stage_bytes = xbytes + gbytes;
  // Rows of this block: blockIdx.x + k * gridDim.x, k < n (the grid has at most `rows` blocks).
  const long long n = (rows - blockIdx.x + gridDim.x - 1) / gridDim.x;

  if (t == 0) {
    for (int s = 0; s < stages; ++s) ptx::mbar_init(ptx::smem_u32(&full[s]), 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](long long k, int s) {
    const long long row = blockIdx.x + k * gridDim.x;
    const uint32_t bar = ptx::smem_u32(&full[s]);
    const uint32_t dst = ptx::smem_u32(ln_stage_smem + static_cast<size_t>(s) * stage_bytes);
    ptx::mbar_arrive_expect_tx(bar, stage_bytes);
    ptx::bulk_load(dst, x + row * ldx, xbytes, bar);
    ptx::bulk_load(dst + xbytes, dy + row * lddy, gbytes, bar);
  };
  // A wait with a time limit.
  auto wait = [&](int s, uint32_t parity) -> bool {
    const uint32_t bar = ptx::smem_u32(&full[s]);
    uint32_t spins = 0;
    uint64_t t0 = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
      if ((++spins & 0x3FFu) == 0) {
        const uint64_t now = ptx::globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > ptx::kWaitLimitNs) return false;
      }
    }
    return true;
  };
  if (t == 0) {
    for (int k = 0; k < stages && k < n; ++k) issue(k, k);
  }

  float wc[kLnCache];
#pragma unroll
  for (int i = 0; i < kG; ++i) {
    const int g = t + i * R;
#pragma unroll
    for (int j = 0; j < V; ++j)
      wc[i * V + j] = (w != nullptr && g < groups) ? load_as_f32(w, param_dtype, g * V + j) : 1.0f;
  }
  // Two elements per instruction throughout (packed fp32: same roundings as the one-element forms).
  float2 wacc[kParams ? kLnCache / 2 : 1], bacc[kParams ? kLnCache / 2 : 1];
  if constexpr (kParams) {
#pragma unroll
    for (int i = 0; i < kLnCache / 2; ++i) wacc[i] = bacc[i] = make_float2(0.0f, 0.0f);
  }

  long long failed_at = -1;
  int stage_index = 0, stat_index = 0;       // k % stages, k % kLnStatChunk
  uint32_t stage_parity = 0;                  // (k / stages) & 1
  for (long long k = 0; k < n; ++k) {
    if (stat_index == 0) {
      // Every thread read its statistics of the previous chunk before the last row-sum barrier.
      for (int i = t; i < kLnStatChunk && k + i < n; i += R) {
        const long long r = blockIdx.x + (k + i) * gridDim.x;
        stat_mean[i] = mean[r];
        stat_rs[i] = inv_std[r];
      }
      __syncthreads();
    }
    const long long row = blockIdx.x + k * gridDim.x;
    const float mu = stat_mean[stat_index], rs = stat_rs[stat_index];
    const bool ok = wait(stage_index, stage_parity);
    const unsigned char* stage = ln_stage_smem + static_cast<size_t>(stage_index) * stage_bytes;

    float2 pc[kLnCache / 2], gc[kLnCache / 2];
    float2 s1p = make_float2(0.0f, 0.0f), s2p = make_float2(0.0f, 0.0f);
    const float2 neg_mu = actm::both(-mu), rs2 = actm::both(rs);
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      const int g = t + i * R;
      if (g < groups) {
        const LnRaw<TIn, V> xq = *reinterpret_cast<const LnRaw<TIn, V>*>(stage + static_cast<size_t>(g) * V * sizeof(TIn));
        const LnRaw<TDy, V> gq =
            *reinterpret_cast<const LnRaw<TDy, V>*>(stage + xbytes + static_cast<size_t>(g) * V * sizeof(TDy));
        float xv[V], gv[V];
        ln_unpack<TIn, V>(xq, xv);
        ln_unpack<TDy, V>(gq, gv);
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          const int e = (i * V + j) / 2;
          const float2 p = actm::mul2(actm::add2(make_float2(xv[j], xv[j + 1]), neg_mu), rs2);
          float2 gg = make_float2(gv[j], gv[j + 1]);
          if constexpr (kParams) {
            wacc[e] = actm::fma2(gg, p, wacc[e]);
            bacc[e] = actm::add2(bacc[e], gg);
          }
          gg = actm::mul2(gg, make_float2(wc[i * V + j], wc[i * V + j + 1]));
          s1p = actm::fma2(p, gg, s1p);
          s2p = actm::add2(s2p, gg);
          pc[e] = p;
          gc[e] = gg;
        }
      } else {
#pragma unroll
        for (int j = 0; j < V; j += 2) pc[(i * V + j) / 2] = gc[(i * V + j) / 2] = make_float2(0.0f, 0.0f);
      }
    }
    float s1 = s1p.x + s1p.y, s2 = s2p.x + s2p.y;
    // Row sums over the block; the barrier also tells whether any thread's wait ran out.
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, off);
      s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, off);
    }
    if ((t & 31) == 0) scratch[phase][t >> 5] = make_float2(s1, s2);
    if (__syncthreads_or(ok ? 0 : 1)) {
      failed_at = k;
      break;
    }
    s1 = 0.0f;
    s2 = 0.0f;
#pragma unroll
    for (int wi = 0; wi < R / 32; ++wi) {
      s1 += scratch[phase][wi].x;
      s2 += scratch[phase][wi].y;
    }
    phase ^= 1;
    // All threads have read this stage: refill it.
    if (t == 0 && k + stages < n) issue(k + stages, stage_index);
    const float2 c1 = actm::both(s1 / feat), c2 = actm::both(s2 / feat);
    TDx* dr = dx + row * lddx;
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      const int g = t + i * R;
      if (g < groups) {
        float o[V];
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          const int e = (i * V + j) / 2;
          // rs * (g - (p c1 + c2))
          const float2 r = actm::mul2(rs2, actm::fma2(actm::fma2(pc[e], c1, c2), actm::both(-1.0f), gc[e]));
          o[j] = r.x;
          o[j + 1] = r.y;
        }
        ln_store<TDx, V>(dr + g * V, o);
      }
    }
    stat_index = stat_index + 1 == kLnStatChunk ? 0 : stat_index + 1;
    if (++stage_index == stages) {
      stage_index = 0;
      stage_parity ^= 1u;
    }
  }

  if (failed_at >= 0 && t == 0) {
    atomicCAS(status, 0, DEV_TIMEOUT_ROW_COPY);
    // Copies issued and not consumed: rows failed_at ... failed_at + stages - 1 (those below n), in the
    // stages from stage_index on.
    for (long long k = failed_at; k < failed_at + stages && k < n; ++k) {
      wait(stage_index, stage_parity);
      if (++stage_index == stages) {
        stage_index = 0;
        stage_parity ^= 1u;
      }
    }
  }
  if constexpr (kParams) {
#pragma unroll
    for (int i = 0; i < kG; ++i) {
      const int g = t + i * R;
      if (g < groups) {
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          const int e = (i * V + j) / 2;
          float* wp = wpart + static_cast<long long>(blockIdx.x) * F + g * V + j;
          wp[0] = wacc[e].x;
          wp[1] = wacc[e].y;
          if (bpart != nullptr) {
            float* bp = bpart + static_cast<long long>(blockIdx.x) * F + g * V + j;
            bp[0] = bacc[e].x;
            bp[1] = bacc[e].y;
          }
        }
      }
    }
  }
}

// Weight- and bias-gradient partial sums for rows wider than the register variant holds: one thread per
// column, gridDim.y chunks of rows; partial row blockIdx.y of wpart / bpart.
template <class TIn, class TDy>
__global__ void __launch_bounds__(256)
ln_param_grad_kernel(const TDy* __restrict__ dy, long long lddy, const TIn* __restrict__ x, long long ldx,
                     const float* __restrict__ mean, const float* __restrict__ inv_std, float* __restrict__ wpart,
                     float* __restrict__ bpart, long long rows, int F, long long rows_per_chunk) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col >= F) return;
  const long long begin = blockIdx.y * rows_per_chunk;
  const long long end = begin + rows_per_chunk < rows ? begin + rows_per_chunk : rows;
  float wa = 0.0f, ba = 0.0f;
  for (long long r = begin; r < end; ++r) {
    const float g = to_f32<TDy>(dy[r * lddy + col]);
    const float p = (to_f32<TIn>(x[r * ldx + col]) - mean[r]) * inv_std[r];
    wa += g * p;
    ba += g;
  }
  wpart[static_cast<long long>(blockIdx.y) * F + col] = wa;
  if (bpart != nullptr) bpart[static_cast<long long>(blockIdx.y) * F + col] = ba;
}

// weight_grad[j] = sum over the partial rows of wpart[., j]; the same for the bias (blockIdx.y = 1).
// A block takes 32 columns; its 32 warps each add every 32nd partial row (four interleaved sums, so four
// loads in flight), then one warp adds the 32 results in order.  The order is fixed.
constexpr int kLnFinishCols = 32, kLnFinishSlices = 32;

__global__ void __launch_bounds__(kLnFinishCols * kLnFinishSlices)
ln_param_finish_kernel(const float* __restrict__ wpart, const float* __restrict__ bpart, int parts, int F,
                       float* __restrict__ weight_grad, float* __restrict__ bias_grad) {
  __shared__ float red[kLnFinishSlices][kLnFinishCols + 1];
  const float* src = blockIdx.y == 0 ? wpart : bpart;
  float* dst = blockIdx.y == 0 ? weight_grad : bias_grad;
  if (dst == nullptr) return;
  const int c = threadIdx.x % kLnFinishCols, slice = threadIdx.x / kLnFinishCols;
  const int col = blockIdx.x * kLnFinishCols + c;
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
  if (col < F) {
    int p = slice;
    for (; p + 3 * kLnFinishSlices < parts; p += 4 * kLnFinishSlices) {
      a0 += src[static_cast<long long>(p) * F + col];
      a1 += src[static_cast<long long>(p + kLnFinishSlices) * F + col];
      a2 += src[static_cast<long long>(p + 2 * kLnFinishSlices) * F + col];
      a3 += src[static_cast<long long>(p + 3 * kLnFinishSlices) * F + col];
    }
    for (; p < parts; p += kLnFinishSlices) a0 += src[static_cast<long long>(p) * F + col];
  }
  red[slice][c] = (a0 + a1) + (a2 + a3);
  __syncthreads();
  if (slice == 0 && col < F) {
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < kLnFinishSlices; ++i) total += red[i][c];
    dst[col] = total;
  }
}

}  // namespace ab200
