// Input gradient of the fused linear layer with the activation gradient formed in the operand path:
//     dX[M, K] = (dY[M, N] (.) D[M, N]) * W[K, N]^T,        D = act'(Z) as the forward pass stored it,
// instead of a separate pass that writes dZ = dY (.) D for the product to read (the reference's
// act_func_backward_kernel, attorch/linear_layer.py:136-146, followed by its matmul, line 153).
//
// tcgen05 takes the A operand of an MMA from shared memory or from tensor memory.  Here it comes from
// tensor memory: TMA brings the dY tile, the D tile and the W tile of a k-block into shared memory; four
// transform warps (one thread per row of the 128-row tile) multiply their 64 dY and D values, round the
// products to bf16 exactly as the separate pass does, and tcgen05.st them into a 32-column slot of tensor
// memory; the MMA warp then issues four K = 16 MMAs whose A operand is that slot and whose B operand is the
// W tile in shared memory.  One CTA per SM works on whole 128 x 256 tiles: the fp32 accumulator takes 256
// of the 512 tensor-memory columns, three A slots take 96, so the accumulator is not double-buffered and
// the epilogue of a tile does not overlap the next tile's MMAs.
//
// This kernel exists to measure that route against the two-kernel path it would replace (see
// bench.py --workload dxfused); the layer's backward does not call it.
//
// Every wait has a time limit; a waiter that gives up stores its role's code in *status, raises the
// CTA's abort flag so that the other roles stop too, and the kernel returns.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/attorch_b200.h"
#include "common.cuh"
#include "gemm_launch.cuh"
#include "ptx.cuh"

namespace ab200 {
namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 3;
constexpr int kRowTileBytes = kBM * 128;                        // 128 rows of 64 two-byte elements
constexpr int kWTileBytes = kBN * 128;
constexpr int kStageBytes = 2 * kRowTileBytes + kWTileBytes;    // dY + D + W: 64 KB
constexpr int kThreads = 320;                                   // producer, MMA, 4 transform, 4 epilogue warps
constexpr int kAccCols = 256, kSlotCols = 32, kTmemCols = 512;
constexpr int kGroupM = 8;                                      // row tiles that share their W tiles in L2
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;

struct DxFusedArgs {
  void* dx;
  long long ld_dx;
  int dx_dtype, d_is_half;
  int M, K, N;
  int tiles_m, tiles_n;
  int* status;
};

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}

__global__ void __launch_bounds__(kThreads, 1)
dx_fused_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_d,
                const __grid_constant__ CUtensorMap tmap_w, const DxFusedArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* smem = smem_raw + pad;                 // 1024-byte aligned: the 128-byte swizzle needs it
  const uint32_t smem_base = raw_addr + pad;
  uint8_t* bar_region = smem + kStages * kStageBytes;
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  // Barriers (8 bytes each): full[s], empty[s], a_full[s], acc_full, acc_empty.
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto a_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  const uint32_t acc_full_bar = bar_base + 8u * (3 * kStages);
  const uint32_t acc_empty_bar = bar_base + 8u * (3 * kStages + 1);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_region + 8 * (3 * kStages + 2));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);        // the producer's arrive.expect_tx
      ptx::mbar_init(empty_bar(s), 5);       // four transform warps (dY, D read) + one tcgen05.commit (W, slot read)
      ptx::mbar_init(a_full_bar(s), 4);      // four transform warps (slot written)
    }
    ptx::mbar_init(acc_full_bar, 1);         // one tcgen05.commit
    ptx::mbar_init(acc_empty_bar, 4);        // four epilogue warps
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&tmap_dy);
    ptx::prefetch_tmap(&tmap_d);
    ptx::prefetch_tmap(&tmap_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  auto wait = [&](uint32_t bar, uint32_t parity, int code) -> bool {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
      if ((++spins & 0x3FFu) == 0) {
        if (*abort_flag) return false;
        const uint64_t now = ptx::globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > ptx::kWaitLimitNs) {
          *abort_flag = 1;
          atomicCAS(args.status, 0, code);
          return false;
        }
      }
    }
    return true;
  };

  const int tiles = args.tiles_m * args.tiles_n;
  const int k_blocks = args.N / kBK;
  // Tile t: groups of kGroupM row tiles; within a group the row tile varies fastest, so the tiles that
  // run at the same time share a few dY / D slabs and all of W in L2.
  auto decode = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = kGroupM * args.tiles_n;
    const int g = t / per_group, r = t % per_group;
    const int rows_here = args.tiles_m - g * kGroupM < kGroupM ? args.tiles_m - g * kGroupM : kGroupM;
    m_blk = g * kGroupM + r % rows_here;
    n_blk = r / rows_here;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        int m_blk, n_blk;
        decode(t, m_blk, n_blk);
        const int m0 = m_blk * kBM, n0 = n_blk * kBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!wait(empty_bar(s), ph ^ 1u, DEV_TIMEOUT_PRODUCER)) { ok = false; break; }
          const uint32_t full = full_bar(s);
          ptx::mbar_arrive_expect_tx(full, kStageBytes);
          const uint32_t dst = smem_base + s * kStageBytes;
          const int k0 = kb * kBK;
          ptx::tma_load_2d(dst, &tmap_dy, full, k0, m0);
          ptx::tma_load_2d(dst + kRowTileBytes, &tmap_d, full, k0, m0);
          ptx::tma_load_2d(dst + 2 * kRowTileBytes, &tmap_w, full, k0, n0);
          ptx::tma_load_2d(dst + 2 * kRowTileBytes + kWTileBytes / 2, &tmap_w, full, k0, n0 + kBN / 2);
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc(1, 0, 0, kBM, kBN);     // bf16, both K-major
      int s = 0;
      uint32_t ph = 0, n_acc = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        if (!wait(acc_empty_bar, (n_acc & 1u) ^ 1u, DEV_TIMEOUT_MMA)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!wait(a_full_bar(s), ph, DEV_TIMEOUT_MMA) || !wait(full_bar(s), ph, DEV_TIMEOUT_MMA)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t w_addr = smem_base + s * kStageBytes + 2 * kRowTileBytes;
          const uint32_t slot = tmem_base + kAccCols + s * kSlotCols;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // K = 16 per MMA: 8 columns of the slot, the next 32 bytes of every 128-byte W row.
            const uint64_t b_desc = ptx::make_smem_desc(w_addr + k * 32, 16, 1024);
            ptx::umma_a_tmem(tmem_base, slot + k * 8, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          ptx::umma_commit(empty_bar(s));      // W tile and slot reusable once these MMAs have read them
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(acc_full_bar);
        ++n_acc;
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ transform (warps 2..5)
    const int q = warp & 3;                       // tensor-memory lane quarter this warp may access
    const int row = q * 32 + lane;                // row of the tile
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!wait(full_bar(s), ph, DEV_TIMEOUT_EPILOGUE)) { ok = false; break; }
        const uint8_t* ty = smem + s * kStageBytes + row * 128;
        const uint8_t* td = ty + kRowTileBytes;
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          // 128-byte swizzle: 16-byte chunk c of row `row` sits at chunk c ^ (row % 8).
          const int pc = c ^ (row & 7);
          const uint4 y = *reinterpret_cast<const uint4*>(ty + pc * 16);
          const uint4 d = *reinterpret_cast<const uint4*>(td + pc * 16);
          const uint32_t yw[4] = {y.x, y.y, y.z, y.w};
          const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 yf = unpack_bf16x2(yw[j]);
            const float2 df = args.d_is_half ? __half22float2(*reinterpret_cast<const __half2*>(&dw[j]))
                                             : unpack_bf16x2(dw[j]);
            const __nv_bfloat162 p = __floats2bfloat162_rn(yf.x * df.x, yf.y * df.y);
            r[4 * c + j] = *reinterpret_cast<const uint32_t*>(&p);
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(empty_bar(s));          // this warp has read its rows of dY and D
        ptx::tmem_st_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + kAccCols + s * kSlotCols, r);
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(a_full_bar(s));
        if (++s == kStages) { s = 0; ph ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 6..9)
    const int q = warp & 3;
    uint32_t n_acc = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
      int m_blk, n_blk;
      decode(t, m_blk, n_blk);
      if (!wait(acc_full_bar, n_acc & 1u, DEV_TIMEOUT_EPILOGUE)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const int row = m_blk * kBM + q * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c * 32, r);
        ptx::tmem_ld_wait();
        const int col = n_blk * kBN + c * 32;
        if (row < args.M) {
          const long long off = static_cast<long long>(row) * args.ld_dx + col;
          if (args.dx_dtype == DT_F32) {
            float* o = static_cast<float*>(args.dx) + off;
            if (col + 32 <= args.K && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<uint4*>(o)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
            } else {
              for (int i = 0; i < 32; ++i)
                if (col + i < args.K) o[i] = __uint_as_float(r[i]);
            }
          } else {
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(args.dx) + off;
            if (col + 32 <= args.K && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * j]),
                                                                 __uint_as_float(r[8 * i + 2 * j + 1]));
                  w[j] = *reinterpret_cast<const uint32_t*>(&p);
                }
                reinterpret_cast<uint4*>(o)[i] = make_uint4(w[0], w[1], w[2], w[3]);
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col + i < args.K) o[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
            }
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty_bar);
      ++n_acc;
    }
  }

  if (warp == 0 && lane == 0 && *abort_flag) {
    // Gave up: the copies this CTA issued may still be landing in its shared memory; give them time.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) {
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

}  // namespace
}  // namespace ab200

using namespace ab200;

extern "C" int ab200_linear_backward_input_fused(const void* dy, const void* derivative, const void* w, void* dx,
                                                 int64_t M, int64_t K, int64_t N, int64_t ld_dy, int64_t ld_d,
                                                 int64_t ld_w, int64_t ld_dx, int derivative_dtype, int dx_dtype,
                                                 int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || K <= 0 || N <= 0 || N % kBK != 0) return ERR_BAD_SHAPE;
  if (M >= (1ll << 31) || K >= (1ll << 31) || N >= (1ll << 31)) return ERR_TOO_LARGE;
  if ((derivative_dtype != DT_F16 && derivative_dtype != DT_BF16) || (dx_dtype != DT_F32 && dx_dtype != DT_BF16))
    return ERR_BAD_DTYPE;
  if (M == 0) return OK;
  if (!dy || !derivative || !w || !dx || !status) return ERR_NULL_POINTER;
  auto tma_ok = [](const void* p, int64_t ld, int64_t inner) {
    return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && ld >= inner && (ld * 2) % 16 == 0;
  };
  if (!tma_ok(dy, ld_dy, N) || !tma_ok(derivative, ld_d, N) || !tma_ok(w, ld_w, N) || ld_dx < K) return ERR_BAD_STRIDE;
  CUtensorMap tdy, td, tw;
  int rc = encode_2d(&tdy, DT_BF16, dy, N, M, ld_dy * 2, kBK, kBM);
  if (rc == OK) rc = encode_2d(&td, derivative_dtype, derivative, N, M, ld_d * 2, kBK, kBM);
  if (rc == OK) rc = encode_2d(&tw, DT_BF16, w, N, K, ld_w * 2, kBK, kBN / 2);
  if (rc != OK) return rc;
  DxFusedArgs a{};
  a.dx = dx; a.ld_dx = ld_dx; a.dx_dtype = dx_dtype; a.d_is_half = derivative_dtype == DT_F16 ? 1 : 0;
  a.M = static_cast<int>(M); a.K = static_cast<int>(K); a.N = static_cast<int>(N);
  a.tiles_m = static_cast<int>((M + kBM - 1) / kBM);
  a.tiles_n = static_cast<int>((K + kBN - 1) / kBN);
  a.status = status;
  if (cudaFuncSetAttribute(dx_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return ERR_LAUNCH;
  const long long tiles = static_cast<long long>(a.tiles_m) * a.tiles_n;
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  dx_fused_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tdy, td, tw, a);
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}
