// Shared device helpers for the sm_100a kernels of this engine.
//
// Every kernel file exports plain C launchers (extern "C", returning a cudaError_t as
// int) so that the host side can load the library without any binding generator.
// Storage types are float (the true 32-bit path) and __nv_bfloat16 (the serving path);
// arithmetic inside every kernel here is 32-bit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TLIE_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the host wrappers
#define TLIE_F32 0
#define TLIE_BF16 1

namespace tlie {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 2^x in one instruction (ex2.approx: relative error about 2^-22, results below 2^-126 become zero, 2^-inf = 0).  exp2f()
// without fast-math wraps the same instruction in a rescaling for denormal results, which a softmax weight does not need;
// in the attention kernels' inner loops that wrapper was a third of the instructions per score.
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

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

// Sum over a block of up to 1024 threads.  The order of additions depends only on the
// block size, so a row's result does not depend on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = (lane < warps) ? scratch[lane] : 0.0f;
  total = warp_sum(total);
  return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = (lane < warps) ? scratch[lane] : -INFINITY;
  total = warp_max(total);
  return total;
}

}  // namespace tlie

// --- programmatic dependent launch -----------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while its
// predecessor in the stream still runs.  It must call grid_dependency_wait() before it reads
// anything the predecessor wrote (weights and other constants may be fetched earlier), and it
// lets its own successor start early with grid_launch_dependents().  Without the attribute both
// are no-ops.
namespace tlie {
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
}  // namespace tlie

#ifdef __CUDACC__
#include <cstdlib>
namespace tlie {
// Streaming multiprocessors of the current device (asked once; 148 on a B200).  Grids of persistent CTAs are sized from it.
static inline int device_sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0, found = 0;
    if (cudaGetDevice(&device) == cudaSuccess && cudaDeviceGetAttribute(&found, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && found > 0)
      count = found;
    else
      count = 148;
  }
  return count;
}

// Launch with programmatic dependent launch unless TLIE_PDL=0 is set in the environment.
template <typename... KernelArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
  static const bool enabled = [] {
    const char* v = std::getenv("TLIE_PDL");
    return !(v && v[0] == '0');
  }();
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = enabled ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}
}  // namespace tlie
#endif
