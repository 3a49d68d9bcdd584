// Types shared by the kernels and the C-ABI layer.
#pragma once
#include <cstdint>
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace ab200 {

// Element types (same numbering as include/attorch_b200.h).
enum DType : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };

__host__ __device__ inline int dtype_size(int dt) { return dt == DT_F32 ? 4 : 2; }

// Return codes of the C-ABI (same numbering as include/attorch_b200.h).
enum Status : int {
  OK = 0,
  ERR_NULL_POINTER = -1,
  ERR_BAD_SHAPE = -2,
  ERR_BAD_DTYPE = -3,
  ERR_BAD_ACT = -4,
  ERR_BAD_STRIDE = -5,
  ERR_WORKSPACE_TOO_SMALL = -6,
  ERR_TENSOR_MAP = -7,
  ERR_LAUNCH = -8,
  ERR_TOO_LARGE = -9,
  ERR_DRIVER = -10,
  ERR_STATIC_SCRATCH_TOO_SMALL = -11,
  ERR_BAD_PROBABILITY = -12,
};

// Codes a kernel writes to the caller's device status word when a bounded wait runs out.
enum DeviceStatus : int {
  DEV_OK = 0,
  DEV_TIMEOUT_PRODUCER = 1,
  DEV_TIMEOUT_MMA = 2,
  DEV_TIMEOUT_EPILOGUE = 3,
  DEV_TIMEOUT_COLLECTIVE = 4,
  DEV_TIMEOUT_ROW_COPY = 5,
};

template <class T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Loads element i of an array whose element type is only known at run time.
__device__ __forceinline__ float load_as_f32(const void* p, int dt, long long i) {
  if (dt == DT_F32) return static_cast<const float*>(p)[i];
  if (dt == DT_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void store_from_f32(void* p, int dt, long long i, float v) {
  if (dt == DT_F32)
    static_cast<float*>(p)[i] = v;
  else if (dt == DT_F16)
    static_cast<__half*>(p)[i] = __float2half_rn(v);
  else
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// Rounds an fp32 value to the given storage type and back (what a store followed by a load does).
__device__ __forceinline__ float round_through(float v, int dt) {
  if (dt == DT_F16) return __half2float(__float2half_rn(v));
  if (dt == DT_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}

// round_through for two values with one conversion instruction.
__device__ __forceinline__ void round_through2(float& a, float& b, int dt) {
  if (dt == DT_BF16) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&p);
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xFFFF0000u);
  } else if (dt == DT_F16) {
    const float2 f = __half22float2(__floats2half2_rn(a, b));
    a = f.x;
    b = f.y;
  }
}

// Rounds eight fp32 values to T, packed in order into 16 (2-byte T) or 32 (fp32) bytes; two values
// per conversion instruction for the 2-byte types.
template <class T>
__device__ __forceinline__ void pack8(const float (&v)[8], T (&o)[8]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = v[i];
  } else if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) {
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<__half2*>(o)[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<__nv_bfloat162*>(o)[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  }
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int dt) {
  if (dt == DT_F16) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&b);
}

}  // namespace ab200
