// The memory-bound and the any-shape kernels around the tcgen05 GEMM:
//   * act_backward_kernel   dZ = dY * act'(Z) with the bias-gradient column sums fused in
//                           (reference: act_func_backward_kernel, attorch/act_kernels.py:883-927,
//                           and pre_act_grad.sum(dim=0), attorch/linear_layer.py:156)
//   * colsum_finish_kernel  fixed-order reduction of the per-row-block column sums -> db
//   * streamk_finish_kernel fp32 partial sums -> bias, pre-activation, activation, output
//   * cast_kernel           strided 2-D copy with element-type conversion (autocast operand casts)
//   * gemm_any_kernel       CUDA-core GEMM for shapes the TMA path cannot address (row pitches that
//                           are not multiples of 16 bytes, arbitrary element strides)
#pragma once
#include "act_math.cuh"
#include "common.cuh"
#include "gemm_tcgen05.cuh"

namespace ab200 {

// ------------------------------------------------------------------------------------------------
// dZ = dY * act'(Z), plus per-row-block column sums of dZ.
// A block of 256 threads covers kColThreads * 8 columns and kActRows rows; kColThreads threads sit
// side by side on one row and 256 / kColThreads row lanes take alternate rows.  With
// kColThreads = 256 (wide matrices) every row pass reads 4 KB (2-byte types) of one row
// contiguously, which keeps DRAM pages open, and a thread owns its 8 columns for all rows of the
// block, so the column sums need no exchange; with kColThreads = 32 (narrow matrices) the row
// lanes' sums meet in shared memory.  partial is [gridDim.y][N] fp32.  A block takes rows_per_block
// consecutive rows: at least kActRows (which bounds the partial sums a caller must provide room for)
// and otherwise as many as make the grid a whole number of waves of resident blocks.
// ------------------------------------------------------------------------------------------------
constexpr int kActRows = 128;

template <class T, bool kVec, int kColThreads>
__global__ void __launch_bounds__(256)
act_backward_kernel(const T* __restrict__ dy, long long ld_dy, const T* __restrict__ z, long long ld_z,
                    T* __restrict__ dz, long long ld_dz, float* __restrict__ partial, int M, int N,
                    int act, float act_param, int rows_per_block) {
  constexpr int kRowLanes = 256 / kColThreads;
  // Rows in flight per thread.  Four rows were slower on B200 (45.7 vs 40.5 us on 8192 x 4096 bf16):
  // at 124 registers only two blocks fit an SM, so no more loads are in flight than with two rows.
  constexpr int kUnroll = kRowLanes == 1 ? 4 : 2;
  constexpr int kWords = sizeof(T) * 8 / 16;   // 16-byte words per 8 elements
  const int ct = threadIdx.x % kColThreads;
  const int rl = threadIdx.x / kColThreads;
  const int col0 = (blockIdx.x * kColThreads + ct) * 8;
  const int row_begin = blockIdx.y * rows_per_block;
  const int row_end = min(M, row_begin + rows_per_block);
  float sum[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sum[i] = 0.0f;
  // The saved derivative of a bf16 layer may have been stored as fp16 (same size): see api.cu.
  const bool z_is_half = sizeof(T) == 2 && act == ACT_SAVED_DERIVATIVE_F16;

  if (col0 < N) {
    for (int r0 = row_begin + rl; r0 < row_end; r0 += kRowLanes * kUnroll) {
      uint4 gq[kUnroll][kWords], zq[kUnroll][kWords];
      float g[kUnroll][8], zz[kUnroll][8];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int r = r0 + kRowLanes * u;
        if (r >= row_end) continue;
        if constexpr (kVec) {
          const uint4* gp = reinterpret_cast<const uint4*>(dy + r * ld_dy + col0);
#pragma unroll
          for (int w = 0; w < kWords; ++w) gq[u][w] = __ldg(gp + w);
          if (z != nullptr) {
            const uint4* zp = reinterpret_cast<const uint4*>(z + r * ld_z + col0);
#pragma unroll
            for (int w = 0; w < kWords; ++w) zq[u][w] = __ldg(zp + w);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const bool in = col0 + i < N;
            g[u][i] = in ? to_f32<T>(dy[r * ld_dy + col0 + i]) : 0.0f;
            if (z_is_half)
              zz[u][i] = in ? __half2float(reinterpret_cast<const __half*>(z)[r * ld_z + col0 + i]) : 0.0f;
            else
              zz[u][i] = (in && z != nullptr) ? to_f32<T>(z[r * ld_z + col0 + i]) : 0.0f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int r = r0 + kRowLanes * u;
        if (r >= row_end) continue;
        if constexpr (kVec) {
          const T* ge = reinterpret_cast<const T*>(gq[u]);
          const T* ze = reinterpret_cast<const T*>(zq[u]);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            g[u][i] = to_f32<T>(ge[i]);
            if (z_is_half) zz[u][i] = __half2float(reinterpret_cast<const __half*>(zq[u])[i]);
            else zz[u][i] = (z != nullptr) ? to_f32<T>(ze[i]) : 0.0f;
          }
        }
        alignas(16) T o[8];
        if constexpr (kVec && sizeof(T) == 2) {
          if (act == ACT_SAVED_DERIVATIVE) {
            // dZ = dY * act'(Z) on packed pairs: one multiply with a single rounding to the 16-bit
            // type, which is what the fp32 route gives too (the product of two 16-bit values is exact
            // in fp32), at a fraction of its unpack / convert instructions.
            using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
            const T2* ga = reinterpret_cast<const T2*>(gq[u]);
            const T2* za = reinterpret_cast<const T2*>(zq[u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<T2*>(o)[i] = __hmul2(ga[i], za[i]);
          } else {
            act_grad_mul(g[u], zz[u], act, act_param);
            pack8<T>(g[u], o);
          }
        } else {
          act_grad_mul(g[u], zz[u], act, act_param);
          // The stored dZ is rounded to the element type; the column sums use the rounded values,
          // as a sum over the stored dZ would.
          pack8<T>(g[u], o);
        }
        if (partial != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; ++i) sum[i] += to_f32<T>(o[i]);
        }
        if (dz != nullptr) {
          if constexpr (kVec) {
            uint4* op = reinterpret_cast<uint4*>(dz + r * ld_dz + col0);
#pragma unroll
            for (int w = 0; w < kWords; ++w) op[w] = reinterpret_cast<const uint4*>(o)[w];
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (col0 + i < N) dz[r * ld_dz + col0 + i] = o[i];
          }
        }
      }
    }
  }

  if (partial != nullptr) {
    float* dst = partial + static_cast<long long>(blockIdx.y) * N;
    if constexpr (kRowLanes == 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (col0 + i < N) dst[col0 + i] = sum[i];
    } else {
      __shared__ float red[kRowLanes][kColThreads * 8 + 8];
#pragma unroll
      for (int i = 0; i < 8; ++i) red[rl][ct * 8 + i] = sum[i];
      __syncthreads();
      for (int c = threadIdx.x; c < kColThreads * 8; c += 256) {
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < kRowLanes; ++j) s += red[j][c];
        const int col = blockIdx.x * kColThreads * 8 + c;
        if (col < N) dst[col] = s;
      }
    }
  }
}

// db[n] = sum over row blocks of partial[c][n], rounded once to the output type.  A block of 256
// threads handles 32 columns with 8 lanes per column; lane j adds blocks j, j + 8, ... in order and
// the 8 lane sums are added in lane order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256)
colsum_finish_kernel(const float* __restrict__ partial, int chunks, int N, void* db, int db_dtype) {
  __shared__ float red[8][33];
  const int cl = threadIdx.x & 31;
  const int lane = threadIdx.x >> 5;
  const int n = blockIdx.x * 32 + cl;
  float s = 0.0f;
  if (n < N) {
    for (int c = lane; c < chunks; c += 8) s += partial[static_cast<long long>(c) * N + n];
  }
  red[lane][cl] = s;
  __syncthreads();
  if (lane == 0 && n < N) {
    float t = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += red[j][cl];
    store_from_f32(db, db_dtype, n, t);
  }
}

// ------------------------------------------------------------------------------------------------
// Finishing pass of the stream-K GEMM: partial[M, N] fp32 -> (+bias) -> aux -> act -> out.
// Clears the partial sums behind itself so that the workspace is zero again for the next call.
// ------------------------------------------------------------------------------------------------
__global__ void streamk_finish_kernel(float* __restrict__ partial, long long ld_partial, int M, int N,
                                      const void* bias, int bias_dtype, void* aux, long long ld_aux,
                                      void* out, long long ld_out, int out_dtype, int act,
                                      float act_param, int save_grad, int grad_dtype, const void* residual,
                                      long long ld_res) {
  // Four consecutive columns per thread where the row pitch allows 16-byte accesses.
  const bool vec = (N % 4 == 0) && (ld_partial % 4 == 0);
  const int width = vec ? 4 : 1;
  const long long groups_per_row = N / width;
  const long long total = static_cast<long long>(M) * groups_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = i / groups_per_row;
    const long long n0 = (i - m * groups_per_row) * width;
    float* pp = partial + m * ld_partial + n0;
    float vals[4];
    if (vec) {
      const float4 p = *reinterpret_cast<const float4*>(pp);
      *reinterpret_cast<float4*>(pp) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      vals[0] = p.x; vals[1] = p.y; vals[2] = p.z; vals[3] = p.w;
    } else {
      vals[0] = *pp;
      *pp = 0.0f;
    }
    for (int e = 0; e < width; ++e) {
      const long long n = n0 + e;
      float v[1] = {vals[e]};
      if (bias != nullptr) v[0] += round_through(load_as_f32(bias, bias_dtype, n), out_dtype);
      if (aux != nullptr && save_grad) {
        float zr[1] = {round_through(v[0], out_dtype)}, g[1];
        act_fwd_grad(v, zr, g, act, act_param);
        store_from_f32(aux, grad_dtype, m * ld_aux + n, g[0]);
      } else {
        if (aux != nullptr) store_from_f32(aux, out_dtype, m * ld_aux + n, v[0]);
        act_fwd_inplace(v, act, act_param);
      }
      if (residual != nullptr) v[0] += load_as_f32(residual, out_dtype, m * ld_res + n);
      store_from_f32(out, out_dtype, m * ld_out + n, v[0]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Finishing pass of the hybrid GEMM.  Shared-out tile t (blockIdx.x) received pieces from the workers
// whose share of the (tile, k-block) units overlaps it; worker w wrote them to slot 2w (if the tile
// is the first its share touches) or 2w + 1.  The pieces are summed in worker order and go through
// the same epilogue as everywhere.
// ------------------------------------------------------------------------------------------------
struct HybridFinishArgs {
  const float* partial;
  int first_tile, tail_tiles, workers, k_blocks;
  int tiles_m, tiles_n, group_m, tile_m, bn;
  int M, N;
  const void* bias; int bias_dtype;
  void* aux; long long ld_aux;
  void* out; long long ld_out; int out_dtype;
  int act; float act_param; int save_grad; int grad_dtype;
  const void* residual; long long ld_res;
};


__global__ void __launch_bounds__(256) hybrid_finish_kernel(const HybridFinishArgs a) {
  // Slots of the pieces of this tile, in worker order.
  __shared__ int slots[kMaxTailPieces];
  __shared__ int piece_slot[kMaxTailPieces];   // per worker: its slot for this tile, or -1
  __shared__ int n_slots;
  {
    const long long total = static_cast<long long>(a.tail_tiles) * a.k_blocks;
    const long long t0 = static_cast<long long>(blockIdx.x) * a.k_blocks, t1 = t0 + a.k_blocks;
    for (int w = threadIdx.x; w < a.workers && w < kMaxTailPieces; w += blockDim.x) {
      const long long u0 = total * w / a.workers, u1 = total * (w + 1) / a.workers;
      piece_slot[w] = (u0 < t1 && u1 > t0 && u1 > u0) ? 2 * w + ((u0 / a.k_blocks == blockIdx.x) ? 0 : 1) : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int n = 0;
      for (int w = 0; w < a.workers && w < kMaxTailPieces; ++w)
        if (piece_slot[w] >= 0) slots[n++] = piece_slot[w];
      n_slots = n;
    }
  }
  __syncthreads();
  int m_blk, n_blk;
  tile_to_blocks(a.first_tile + blockIdx.x, a.tiles_m, a.tiles_n, a.group_m, m_blk, n_blk);
  const int elems = a.tile_m * a.bn;
  const int pieces = n_slots;
  // Four consecutive columns per thread (bn is a multiple of 32).
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < elems; i += gridDim.y * blockDim.x * 4) {
    const int r = i / a.bn, c = i - r * a.bn;
    const long long m = static_cast<long long>(m_blk) * a.tile_m + r;
    const long long n0 = static_cast<long long>(n_blk) * a.bn + c;
    if (m >= a.M || n0 >= a.N) continue;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int j = 0; j < pieces; ++j) {
      const float4 p = *reinterpret_cast<const float4*>(a.partial + static_cast<long long>(slots[j]) * elems + i);
      acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const long long n = n0 + e;
      if (n >= a.N) break;
      float v[1] = {vals[e]};
      if (a.bias != nullptr) v[0] += round_through(load_as_f32(a.bias, a.bias_dtype, n), a.out_dtype);
      if (a.aux != nullptr && a.save_grad) {
        float zr[1] = {round_through(v[0], a.out_dtype)}, g[1];
        act_fwd_grad(v, zr, g, a.act, a.act_param);
        store_from_f32(a.aux, a.grad_dtype, m * a.ld_aux + n, g[0]);
      } else {
        if (a.aux != nullptr) store_from_f32(a.aux, a.out_dtype, m * a.ld_aux + n, v[0]);
        act_fwd_inplace(v, a.act, a.act_param);
      }
      if (a.residual != nullptr) v[0] += load_as_f32(a.residual, a.out_dtype, m * a.ld_res + n);
      store_from_f32(a.out, a.out_dtype, m * a.ld_out + n, v[0]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// dst[r, c] (contiguous) = convert(src[r * sr + c * sc])
// ------------------------------------------------------------------------------------------------
template <class S, class D, bool kVec>
__global__ void cast_kernel(const S* __restrict__ src, long long sr, long long sc, D* __restrict__ dst,
                            long long rows, long long cols) {
  if constexpr (kVec) {
    // cols % 8 == 0, sc == 1, both sides 16-byte aligned: 8 elements per 16-byte access, four such
    // groups per thread and trip with every load issued before the conversions (latency-bound).
    constexpr int kUnroll = 4;
    constexpr int kSw = sizeof(S) * 8 / 16, kDw = sizeof(D) * 8 / 16;
    const long long groups_per_row = cols / 8;
    const long long total = rows * groups_per_row;
    const bool narrow = total < (1ll << 32);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total;
         i0 += kUnroll * stride) {
      uint4 in[kUnroll][kSw];
      long long dst_off[kUnroll];
      bool live[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = i0 + u * stride;
        live[u] = i < total;
        const long long j = live[u] ? i : i0;
        long long r, c;
        if (narrow) {
          const unsigned q = static_cast<unsigned>(j) / static_cast<unsigned>(groups_per_row);
          r = q;
          c = (static_cast<unsigned>(j) - q * static_cast<unsigned>(groups_per_row)) * 8ll;
        } else {
          r = j / groups_per_row;
          c = (j - r * groups_per_row) * 8;
        }
        dst_off[u] = r * cols + c;
        const uint4* sp = reinterpret_cast<const uint4*>(src + r * sr + c);
#pragma unroll
        for (int w = 0; w < kSw; ++w) in[u][w] = __ldg(sp + w);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (!live[u]) continue;
        uint4 outv[kDw];
        const S* se = reinterpret_cast<const S*>(in[u]);
        D* de = reinterpret_cast<D*>(outv);
#pragma unroll
        for (int k = 0; k < 8; ++k) de[k] = from_f32<D>(to_f32<S>(se[k]));
        uint4* dp = reinterpret_cast<uint4*>(dst + dst_off[u]);
#pragma unroll
        for (int w = 0; w < kDw; ++w) dp[w] = outv[w];
      }
    }
  } else {
    const long long total = rows * cols;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long r = i / cols;
      const long long c = i - r * cols;
      dst[i] = from_f32<D>(to_f32<S>(src[r * sr + c * sc]));
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Any-shape GEMM on CUDA cores: C[m, n] = sum_k A[m * sam + k * sak] * B[k * sbk + n * sbn], fp32
// accumulation, same fused epilogue as the tensor-core kernel.  64 x 64 tile, 256 threads, 4 x 4
// outputs per thread.
// ------------------------------------------------------------------------------------------------
struct AnyGemmArgs {
  const void* a; long long sam, sak; int a_dtype;
  const void* b; long long sbk, sbn; int b_dtype;
  int M, N, K;
  void* out; long long ld_out; int out_dtype;
  void* aux; long long ld_aux;
  const void* bias; int bias_dtype;
  int act; float act_param;
  int save_grad;          // aux receives act'(Z) instead of Z
  int grad_dtype;         // ... stored in this element type
  const void* residual; long long ld_res;   // optional [M, N] in the output dtype, added after the activation
};

__global__ void __launch_bounds__(256) gemm_any_kernel(const AnyGemmArgs g) {
  constexpr int T = 64, KS = 16;
  __shared__ float As[KS][T + 4];
  __shared__ float Bs[KS][T + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * T, n0 = blockIdx.x * T;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < g.K; k0 += KS) {
    // 64 x 16 elements of each operand, 4 per thread.
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;
      {
        const int mm = idx % T, kk = idx / T;   // consecutive threads -> consecutive m
        const int m = m0 + mm, k = k0 + kk;
        float v = 0.0f;
        if (m < g.M && k < g.K) {
          v = load_as_f32(g.a, g.a_dtype, m * g.sam + k * g.sak);
        }
        As[kk][mm] = v;
      }
      {
        const int nn = idx % T, kk = idx / T;
        const int n = n0 + nn, k = k0 + kk;
        float v = 0.0f;
        if (n < g.N && k < g.K) {
          v = load_as_f32(g.b, g.b_dtype, k * g.sbk + n * g.sbn);
        }
        Bs[kk][nn] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v[1] = {acc[i][j]};
      if (g.bias != nullptr) v[0] += round_through(load_as_f32(g.bias, g.bias_dtype, n), g.out_dtype);
      if (g.aux != nullptr && g.save_grad) {
        float zr[1] = {round_through(v[0], g.out_dtype)}, d[1];
        act_fwd_grad(v, zr, d, g.act, g.act_param);
        store_from_f32(g.aux, g.grad_dtype, m * g.ld_aux + n, d[0]);
      } else {
        if (g.aux != nullptr) store_from_f32(g.aux, g.out_dtype, m * g.ld_aux + n, v[0]);
        act_fwd_inplace(v, g.act, g.act_param);
      }
      if (g.residual != nullptr) v[0] += load_as_f32(g.residual, g.out_dtype, m * g.ld_res + n);
      store_from_f32(g.out, g.out_dtype, m * g.ld_out + n, v[0]);
    }
  }
}

}  // namespace ab200
