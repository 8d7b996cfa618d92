// Shared helpers of the hand-written sm_100a kernels.
//
// Every launcher is an extern "C" function that takes raw device pointers, sizes and a
// cudaStream_t, launches on that stream and returns 0 or a negative NV_ERR_* / positive
// cudaError_t code.  Nothing here allocates device memory: the caller owns every buffer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#define NV_DT_F32 0
#define NV_DT_BF16 1

#define NV_OK 0
#define NV_ERR_BAD_DTYPE (-2)
#define NV_ERR_BAD_SIZE (-3)
#define NV_ERR_UNSUPPORTED (-4)

#define NV_API extern "C" __attribute__((visibility("default")))

#define NV_RETURN_LAST()                          \
  do {                                            \
    cudaError_t e__ = cudaGetLastError();         \
    return e__ == cudaSuccess ? NV_OK : (int)e__; \
  } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Load / store with a run-time dtype code: the plain kernels take it where a template
// parameter would multiply instantiations without making anything faster that matters.
__device__ __forceinline__ float ld_dt(const void* p, int dt, size_t i) {
  return dt == NV_DT_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}
__device__ __forceinline__ void st_dt(void* p, int dt, size_t i, float v) {
  if (dt == NV_DT_F32) ((float*)p)[i] = v;
  else ((bf16*)p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// SiLU(g) * u exactly as the reference writes it: g / (1 + expf(-g)) * u  (src/hip_ops.hip:419-429).
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute may start
// while the kernel before it in the stream still runs; what it reads of that kernel's results, and whatever it
// writes, must come after grid_dep_wait(), which returns once the earlier kernel has finished and its writes
// are visible.  grid_dep_launch() in the earlier kernel says "my dependents may be scheduled now" (once every
// CTA has said so or exited); without it they are scheduled as its CTAs exit.  Both are no-ops for kernels
// launched the ordinary way.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launches `kernel` as a programmatic dependent of the kernel before it on the stream (an ordinary launch
// when nv_set_dependent_launch(0) was called).  Such a kernel must call grid_dep_wait() before it reads anything
// an earlier kernel of the step wrote and before it writes anything, and calls grid_dep_launch() right after,
// so that at most one kernel is ever set up ahead of the one that runs: everything older has finished by then.
// Grids of more than NV_DEP_MAX_BLOCKS blocks are launched the ordinary way: their waiting blocks would crowd
// the multiprocessors on which the kernel before them is still finishing (measured: a prompt of 2,048 tokens
// ran 7 % slower with every kernel a dependent), and a launch latency is nothing beside such a kernel's time.
constexpr unsigned NV_DEP_MAX_BLOCKS = 2048;
extern int g_nv_dependent_launch;
template <typename... Exp, typename... Act>
static inline cudaError_t launch_dep(void (*kernel)(Exp...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Act&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  const unsigned long long blocks = (unsigned long long)grid.x * grid.y * grid.z;
  attr[0].val.programmaticStreamSerializationAllowed = (g_nv_dependent_launch && blocks <= NV_DEP_MAX_BLOCKS) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Exp>(args)...);
}
#define NV_RETURN_IF(e)                            \
  do {                                             \
    cudaError_t e2__ = (e);                        \
    if (e2__ != cudaSuccess) return (int)e2__;     \
  } while (0)

static inline int dt_ok(int dt) { return dt == NV_DT_F32 || dt == NV_DT_BF16; }
