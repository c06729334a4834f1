// Shared by every kernel file: element types, conversions, reductions, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <utility>

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

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch: a kernel may be started while the kernel before it on the
// stream is still running.  It then runs its own set-up (and reads of memory no earlier
// kernel writes, such as weights) at once, and calls pdl_wait() before it touches anything
// an earlier kernel produced; pdl_wait() returns when the earlier kernels have finished and
// their writes are visible.  pdl_launch_dependents() lets the kernel after this one start
// in the same way.  Every kernel of this package calls both, so a chain of them overlaps
// each launch and prologue with the tail of the kernel before.  VIPERA_PDL=0 in the
// environment turns the launch attribute off; the calls are then no-ops.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool vipera_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* value = std::getenv("VIPERA_PDL");
    enabled = (value && value[0] == '0') ? 0 : 1;
  }
  return enabled == 1;
}

// Launch `kernel` on `stream`, allowed to start before the kernel ahead of it has finished.
template <typename... KernelArgs, typename... Args>
static inline int vipera_launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared_bytes,
                                cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = vipera_pdl_enabled() ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  cudaError_t error = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(std::forward<Args>(args))...);
  return error == cudaSuccess ? 0 : static_cast<int>(error);
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
