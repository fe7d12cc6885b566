// Shared helpers of the sm_100a kernels: element types, conversions, reductions and the
// launch-status convention.  Every exported launcher is `extern "C" int zk_*(..., stream)`
// and returns 0 or a cudaError_t value; argument errors are negative (ZK_EINVAL).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ZK_EINVAL (-22)

// dtype codes shared with the Python side
#define ZK_F32 0
#define ZK_BF16 1

#define ZK_LAUNCH_STATUS() ((int)cudaGetLastError())

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a thread block of up to 1024 threads; every thread gets the result.
// `scratch` is 32 floats of shared memory.  The order of the additions is fixed by the
// thread layout only, so the same row gives the same sum whatever else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

static inline int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

// ------------------------------------------------------------------------------ dependent launches
// A kernel launched with zk_launch_dependent may start while the kernel before it in the stream is
// still running: its blocks take the places of blocks that have ended, do whatever needs nothing
// of that kernel (index arithmetic, the first loads of weights), and then call zk_wait_prior(),
// which returns when every kernel before it is complete and its memory is visible.  NOTHING that
// an earlier kernel writes may be read, and nothing may be written, before zk_wait_prior().
// zk_let_next_start() lets the kernel after this one be launched in the same way; with no call
// it starts when this kernel's blocks have ended.  Both are no-ops in a kernel launched plainly.
__device__ __forceinline__ void zk_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void zk_let_next_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline int zk_launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
