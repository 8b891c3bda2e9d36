// Gated activation of the feed-forward: out[t, i] = act(x[t, i]) * x[t, d + i].
// Counterpart in the reference: silu_and_mul_kernel, vllm/kernels/activation_kernels.cu:26-41
// (gelu variants :13-24, :44-51).  Here both factors are taken to float32 and the product is
// rounded once.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_activation)

namespace lmsf {

enum { kActSilu = 0, kActGeluTanh = 1 };

__device__ __forceinline__ float act_silu(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float act_gelu_tanh(float g) {
  const float k = 0.7978845608028654f;  // sqrt(2 / pi)
  return 0.5f * g * (1.0f + tanhf(k * (g + 0.044715f * g * g * g)));
}

template <typename T, int ACT>
__global__ void gated_act_kernel(T* __restrict__ out, const T* __restrict__ in, int d, long long in_stride) {
  const T* row = in + (size_t)blockIdx.x * in_stride;
  T* o = out + (size_t)blockIdx.x * d;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x) {
    const float g = to_f32(row[i]), u = to_f32(row[d + i]);
    o[i] = from_f32<T>((ACT == kActSilu ? act_silu(g) : act_gelu_tanh(g)) * u);
  }
}

// 8 bfloat16 values per thread and pass (16-byte loads); d % 8 == 0, in_stride % 8 == 0, aligned pointers.
template <int ACT>
__global__ void gated_act_vec_kernel(bf16* __restrict__ out, const bf16* __restrict__ in, int d, long long in_stride) {
  const bf16* row = in + (size_t)blockIdx.x * in_stride;
  bf16* o = out + (size_t)blockIdx.x * d;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < d; i += gridDim.y * blockDim.x * 8) {
    uint4 gr = *reinterpret_cast<const uint4*>(row + i), ur = *reinterpret_cast<const uint4*>(row + d + i), r;
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur);
    __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
      r2[e] = __floats2bfloat162_rn((ACT == kActSilu ? act_silu(g.x) : act_gelu_tanh(g.x)) * u.x,
                                    (ACT == kActSilu ? act_silu(g.y) : act_gelu_tanh(g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(o + i) = r;
  }
}

// x[t, i] += bias[i], the sum taken in float32 and rounded once to x's type.
template <typename T>
__global__ void bias_add_kernel(T* __restrict__ x, const T* __restrict__ bias, int d, long long stride) {
  T* row = x + (size_t)blockIdx.x * stride;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x)
    row[i] = from_f32<T>(to_f32(row[i]) + to_f32(bias[i]));
}

}  // namespace lmsf

// x: [n, d] with `stride` elements between rows, bias: [d] of x's type; in place.  The projections of a model whose
// config.json asks for biases (attention_bias, mlp_bias) add them with this kernel after the product; the
// reference's linear layer does the same as a separate broadcast add (core/src/model_executor/layers/linear.rs:100-104).
LMSF_API int lmsf_bias_add(void* x, const void* bias, int n, int d, long long stride, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (d <= 0 || stride < d) LMSF_REFUSE("bias_add: d=%d, stride=%lld", d, stride);
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("bias_add: unknown dtype code %d", dtype);
  int gy = ceil_div(d, 256 * 4);
  if (gy > 64) gy = 64;
  dim3 grid(n, gy);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) bias_add_kernel<float><<<grid, 256, 0, s>>>((float*)x, (const float*)bias, d, stride);
  else bias_add_kernel<bf16><<<grid, 256, 0, s>>>((bf16*)x, (const bf16*)bias, d, stride);
  return LMSF_LAUNCH_STATUS();
}

// in: [n, 2 * d] with `in_stride` elements between rows (gate first, up second); out: [n, d].
LMSF_API int lmsf_gated_act(void* out, const void* in, int n, int d, long long in_stride, int act, int dtype,
                            void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (d <= 0 || in_stride < 2LL * d) LMSF_REFUSE("gated_act: d=%d, in_stride=%lld", d, in_stride);
  if (act != kActSilu && act != kActGeluTanh) LMSF_REFUSE("gated_act: unknown activation code %d", act);
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("gated_act: unknown dtype code %d", dtype);
  const int threads = 256;
  int gy = ceil_div(d, threads * 4);
  if (gy > 64) gy = 64;
  dim3 grid(n, gy);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_BF16 && d % 8 == 0 && in_stride % 8 == 0 && ((uintptr_t)out | (uintptr_t)in) % 16 == 0) {
    int vy = ceil_div(d, 256 * 8);
    if (vy > 64) vy = 64;
    dim3 vgrid(n, vy);
    if (act == kActSilu) gated_act_vec_kernel<kActSilu><<<vgrid, 256, 0, s>>>((bf16*)out, (const bf16*)in, d, in_stride);
    else gated_act_vec_kernel<kActGeluTanh><<<vgrid, 256, 0, s>>>((bf16*)out, (const bf16*)in, d, in_stride);
    return LMSF_LAUNCH_STATUS();
  }
#define LMSF_GA(T, A) gated_act_kernel<T, A><<<grid, threads, 0, s>>>((T*)out, (const T*)in, d, in_stride)
  if (dtype == LMSF_F32) { if (act == kActSilu) LMSF_GA(float, kActSilu); else LMSF_GA(float, kActGeluTanh); }
  else { if (act == kActSilu) LMSF_GA(bf16, kActSilu); else LMSF_GA(bf16, kActGeluTanh); }
#undef LMSF_GA
  return LMSF_LAUNCH_STATUS();
}
