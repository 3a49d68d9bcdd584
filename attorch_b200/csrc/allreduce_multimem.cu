// In-place SUM all-reduce of the gradient bucket over the GPUs of one NVSwitch domain, for the
// data-parallel step of the fused linear layer (the reference has no distributed code; this is the
// one collective the path needs: dW / db summed over the ranks that share a batch).
//
// Every rank maps the same buffer through an NVLink multicast object ("symmetric memory"; the caller
// sets that up, e.g. with torch.distributed._symmetric_memory).  The kernel then is the two-step
// NVSwitch all-reduce: rank r owns the r-th slice of the buffer;
//   multimem.ld_reduce  makes the switch fetch that slice from every rank and add the copies
//                       (fp32 accumulation for the 16-bit types), 16 bytes per instruction,
//   multimem.st         writes the sum back into every rank's copy,
// between two barriers over all ranks (flags in peer-mapped memory, release / acquire at system
// scope).  The additions happen in the switch, so the SMs only move addresses: a handful of CTAs
// saturate the links, which is what lets the all-reduce run beside a GEMM that keeps the other SMs.
// Every rank receives bit-identical sums.
//
// Each wait has a time limit; a waiter that gives up stores DEV_TIMEOUT_COLLECTIVE in the caller's
// status word and the kernel returns (its results are then undefined).  Nothing spins forever.
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/attorch_b200.h"
#include "common.cuh"
#include "ptx.cuh"

namespace ab200 {
namespace {

constexpr int kThreads = 1024;
constexpr int kUnroll = 8;

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Sum over all ranks of the 16 bytes at `addr` (a multicast address), as packed elements of kDtype.
template <int kDtype>
__device__ __forceinline__ uint4 multimem_ld_reduce(uint64_t addr) {
  uint4 v;
  if constexpr (kDtype == DT_BF16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr) : "memory");
  } else if constexpr (kDtype == DT_F16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr) : "memory");
  } else {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr) : "memory");
  }
  return v;
}

// Writes 16 bytes to `addr` in every rank's copy.
__device__ __forceinline__ void multimem_st(uint64_t addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}

// Barrier over all ranks for the CTAs with this block index.  flags[r] is rank r's flag block as
// mapped into this rank's address space: AB200_COLLECTIVE_MAX_CTAS x AB200_COLLECTIVE_MAX_RANKS words
// that peers write, then one epoch counter per CTA that only the owner touches.  Rank s signals CTA b
// of rank r by storing `value` to flags[r][b][s]; values only ever grow, so nothing is reset.
__device__ __forceinline__ bool rank_barrier(uint32_t* const* flags, int rank, int world, uint32_t value, int* status) {
  __syncthreads();   // this CTA's earlier writes are ordered before the signalling threads' release
  bool ok = true;
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    st_release_sys(flags[peer] + blockIdx.x * AB200_COLLECTIVE_MAX_RANKS + rank, value);
    const uint32_t* mine = flags[rank] + blockIdx.x * AB200_COLLECTIVE_MAX_RANKS + peer;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    // Signed difference: correct across the wrap of the 32-bit counter.
    while (static_cast<int32_t>(ld_acquire_sys(mine) - value) < 0) {
      if ((++spins & 0xFFu) == 0) {
        const uint64_t now = ptx::globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > ptx::kWaitLimitNs) {
          atomicCAS(status, 0, DEV_TIMEOUT_COLLECTIVE);
          ok = false;
          break;
        }
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

template <int kDtype>
__global__ void __launch_bounds__(kThreads)
multimem_all_reduce_kernel(uint64_t mc_base, long long units, int rank, int world, uint32_t* const* flags, int* status) {
  __shared__ uint32_t s_epoch;
  uint32_t* epoch_slot = flags[rank] + AB200_COLLECTIVE_MAX_CTAS * AB200_COLLECTIVE_MAX_RANKS + blockIdx.x;
  if (threadIdx.x == 0) s_epoch = *epoch_slot;
  __syncthreads();
  const uint32_t epoch = s_epoch;     // launches so far; equal on every rank, which run the same sequence

  // Every rank's buffer is complete (the kernels before this one on each rank's stream have ended).
  if (rank_barrier(flags, rank, world, 2 * epoch + 1, status)) {
    // This rank's slice, in 16-byte units, shared out over the CTAs.
    const long long per_rank = (units + world - 1) / world;
    const long long begin = per_rank * rank;
    const long long end = begin + per_rank < units ? begin + per_rank : units;
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    for (long long i = begin + static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < end; i += kUnroll * stride) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < end) v[u] = multimem_ld_reduce<kDtype>(mc_base + static_cast<uint64_t>(i + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < end) multimem_st(mc_base + static_cast<uint64_t>(i + u * stride) * 16, v[u]);
    }
    // Every rank has written its slice everywhere.
    rank_barrier(flags, rank, world, 2 * epoch + 2, status);
  }
  if (threadIdx.x == 0) *epoch_slot = epoch + 1;
}

}  // namespace
}  // namespace ab200

using namespace ab200;

extern "C" {

int64_t ab200_collective_flag_bytes(void) {
  return (static_cast<int64_t>(AB200_COLLECTIVE_MAX_CTAS) * AB200_COLLECTIVE_MAX_RANKS + AB200_COLLECTIVE_MAX_CTAS) * 4;
}

int ab200_multimem_all_reduce(void* multicast_ptr, int64_t numel, int dtype, int rank, int world_size,
                              void* const* flag_blocks, int ctas, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (numel < 0 || world_size < 1 || rank < 0 || rank >= world_size) return ERR_BAD_SHAPE;
  if (world_size > AB200_COLLECTIVE_MAX_RANKS) return ERR_TOO_LARGE;
  if (dtype != DT_F32 && dtype != DT_F16 && dtype != DT_BF16) return ERR_BAD_DTYPE;
  if (numel == 0 || world_size == 1) return OK;
  if (!multicast_ptr || !flag_blocks || !status) return ERR_NULL_POINTER;
  const int64_t bytes = numel * dtype_size(dtype);
  if ((reinterpret_cast<uintptr_t>(multicast_ptr) & 15) != 0 || bytes % 16 != 0) return ERR_BAD_STRIDE;
  if (ctas <= 0) ctas = 8;
  if (ctas > AB200_COLLECTIVE_MAX_CTAS) ctas = AB200_COLLECTIVE_MAX_CTAS;
  const long long units = bytes / 16;
  const uint64_t base = reinterpret_cast<uint64_t>(multicast_ptr);
  uint32_t* const* flags = reinterpret_cast<uint32_t* const*>(flag_blocks);
  if (dtype == DT_BF16)
    multimem_all_reduce_kernel<DT_BF16><<<ctas, kThreads, 0, stream>>>(base, units, rank, world_size, flags, status);
  else if (dtype == DT_F16)
    multimem_all_reduce_kernel<DT_F16><<<ctas, kThreads, 0, stream>>>(base, units, rank, world_size, flags, status);
  else
    multimem_all_reduce_kernel<DT_F32><<<ctas, kThreads, 0, stream>>>(base, units, rank, world_size, flags, status);
  return cudaGetLastError() == cudaSuccess ? OK : ERR_LAUNCH;
}

}  // extern "C"
