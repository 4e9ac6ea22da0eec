// Shared helpers of the sm_100a kernels: element types, conversions, reductions,
// launch-error reporting.  Every entry point of the library is `extern "C"`, takes
// raw device pointers and the stream to launch on, and returns a cudaError_t as int.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rl {

// Element type tags shared with the Python side.
enum DType : int { kF32 = 0, kBF16 = 1 };

// Bits of the device-side fault word (`int* fault`).  Kernels that index with
// values they were handed (token ids, page ids, positions) clamp or skip the access
// and set a bit instead of reading out of bounds; the host checks the word after a step.
enum Fault : int {
  kFaultTokenId = 1,    // a token id outside [0, vocab)
  kFaultPageId = 2,     // a page id outside [0, num_pages)
  kFaultPosition = 4,   // a position outside the rotary table or the block table
  kFaultSlot = 8,       // a slot outside the block table
  kFaultWaitLimit = 16  // a bounded wait inside a kernel ran out
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
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

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  Every thread
// gets the result.  The tree is fixed, so the value does not depend on timing.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = (lane < warps) ? scratch[lane] : 0.0f;
  total = warp_sum(total);
  return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = (lane < warps) ? scratch[lane] : -INFINITY;
  total = warp_max(total);
  return total;
}

// Loads of 8 consecutive elements as floats (16 bytes of bf16, 32 bytes of f32).
__device__ __forceinline__ void load8(const float* p, float (&out)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&out)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

// ---- programmatic dependent launch -------------------------------------------------------
// A kernel launched with `pdl` may start while the kernel before it in the stream is still
// running.  Every kernel of this library therefore follows one discipline: it lets its own
// successor start early (pdl_trigger, first thing), touches before pdl_wait() only memory
// that no kernel of a step writes (weights, tables, the step's uploaded metadata), and calls
// pdl_wait() — which returns once the preceding kernel has finished and its writes are
// visible — before it reads an activation or writes anything at all.  Because every kernel
// waits before it finishes, "the kernel before me is done" implies that all earlier ones
// are.  Both instructions do nothing in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launches `kernel`; with `pdl` as a programmatic dependent of the stream's previous kernel.
template <typename... Params, typename... Args>
inline int launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = pdl ? 1 : 0;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...));
}

}  // namespace rl

// Calls `fn<float>` or `fn<__nv_bfloat16>` by a DType tag; returns cudaErrorInvalidValue otherwise.
#define RL_DISPATCH_DTYPE(dtype, ...)                            \
  do {                                                           \
    if ((dtype) == rl::kF32) {                                   \
      using scalar_t = float;                                    \
      __VA_ARGS__                                                \
    } else if ((dtype) == rl::kBF16) {                           \
      using scalar_t = __nv_bfloat16;                            \
      __VA_ARGS__                                                \
    } else {                                                     \
      return static_cast<int>(cudaErrorInvalidValue);            \
    }                                                            \
  } while (0)
