// Shared by every kernel file: element types, conversions, reductions, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define VIPERA_API extern "C" __attribute__((visibility("default")))

// Element type codes of the C interface.
enum ViperaDtype { VIPERA_F32 = 0, VIPERA_BF16 = 1 };

// Return codes of the launchers: 0, a cudaError_t (positive), or one of these.
enum ViperaStatus {
  VIPERA_OK = 0,
  VIPERA_BAD_DTYPE = -1,
  VIPERA_BAD_SHAPE = -2,
  VIPERA_BAD_ARGUMENT = -3,
  VIPERA_NO_DRIVER_ENTRY = -4,
};

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  Every thread
// gets the total.  The order of the additions is fixed by the block size alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = lane < warps ? scratch[lane] : 0.0f;
  return warp_sum(total);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = lane < warps ? scratch[lane] : -INFINITY;
  return warp_max(total);
}

static inline int vipera_launch_status() {
  cudaError_t error = cudaGetLastError();
  return error == cudaSuccess ? VIPERA_OK : static_cast<int>(error);
}

// Text for a return code of any launcher.
static inline const char* vipera_status_text(int status) {
  switch (status) {
    case VIPERA_OK: return "ok";
    case VIPERA_BAD_DTYPE: return "unsupported element type";
    case VIPERA_BAD_SHAPE: return "a size this kernel does not take";
    case VIPERA_BAD_ARGUMENT: return "bad argument";
    case VIPERA_NO_DRIVER_ENTRY: return "the CUDA driver gave no entry point for tensor maps";
    default: return status > 0 ? cudaGetErrorString(static_cast<cudaError_t>(status)) : "unknown status";
  }
}
