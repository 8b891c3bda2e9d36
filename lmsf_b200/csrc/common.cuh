// Shared helpers of the lmsf_b200 kernels (sm_100a only).
//
// Conventions of every launcher in this folder:
//   * C ABI, returns 0 on success, a cudaError_t (> 0) from the launch, or LMSF_EBADARG (-1)
//     when a size or option is outside what the kernel was written for; the text of the last
//     refusal of this library is returned by <file>_last_error().
//   * dtype codes: 0 = float32, 1 = bfloat16.  Reductions, softmax, rotation angles and
//     residual sums are always float32 whatever the storage type.
//   * all index tensors are int32 and live on the device; `stream` is a cudaStream_t.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#if !defined(__CUDA_ARCH__) || __CUDA_ARCH__ >= 1000
#else
#error "lmsf_b200 kernels are written for sm_100a only"
#endif

#define LMSF_API extern "C" __attribute__((visibility("default")))
#define LMSF_EBADARG (-1)
#define LMSF_F32 0
#define LMSF_BF16 1

#define LMSF_DEFINE_LAST_ERROR(prefix)                                              \
  static thread_local char g_last_error[512] = "";                                  \
  LMSF_API const char* prefix##_last_error() { return g_last_error; }

#define LMSF_REFUSE(...)                                                            \
  do {                                                                              \
    snprintf(g_last_error, sizeof(g_last_error), __VA_ARGS__);                      \
    return LMSF_EBADARG;                                                            \
  } while (0)

#define LMSF_LAUNCH_STATUS() ((int)cudaGetLastError())

namespace lmsf {

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

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
// The order of additions depends only on blockDim, never on the data or on other blocks.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// One rotated pair (x, y) -> (x c - y s, y c + x s), every product and sum rounded on its own (no fused
// multiply-add), so that every kernel that rotates gives the same bits.
__device__ __forceinline__ float rot_first(float x, float y, float c, float s) { return __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s)); }
__device__ __forceinline__ float rot_second(float x, float y, float c, float s) { return __fadd_rn(__fmul_rn(y, c), __fmul_rn(x, s)); }

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch -------------------------------------------------------------------
// A kernel launched through launch_pdl may start while the kernel before it in the stream is still
// draining: everything it does before pdl_wait() overlaps that kernel's tail.  Rules for such kernels:
// before pdl_wait() read only data that no kernel of the step writes (weights, constants) and write
// nothing to global memory; call pdl_launch_dependents() once the block has started, so that the next
// kernel may be scheduled as soon as every block of this one is resident.
// LMSF_PDL=0 in the environment turns the overlap off (plain stream order).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline int pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LMSF_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v;
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace lmsf
