// RMSNorm, alone or fused with the residual add that precedes it.
// Counterparts in the reference: rms_norm_kernel and fused_add_rms_norm_kernel,
// vllm/kernels/layernorm_kernels.cu:13-68.  Differences: the residual stream is kept in
// float32 whatever the activation type, and the normalised value is rounded once, after the
// multiplication by the weight.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_rmsnorm)

namespace lmsf {

// mode 0: h = norm(x) * w                        (res untouched, may be null)
// mode 1: res = float(x);        h = norm(res) * w
// mode 2: res = res + float(x);  h = norm(res) * w
// One block per row.  The row is kept in shared memory as float32 between the two passes
// when `cache_row` is set (hidden * 4 bytes of dynamic shared memory), else re-read.
template <typename T, typename WT>
__global__ void add_rmsnorm_kernel(T* __restrict__ h_out, const T* __restrict__ x, float* __restrict__ res,
                                   const WT* __restrict__ w, int hidden, float eps, int mode, int cache_row) {
  extern __shared__ float row_cache[];
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f32(x[base + i]);
    if (mode == 2) v += res[base + i];
    if (mode != 0) res[base + i] = v;
    if (cache_row) row_cache[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v;
    if (cache_row) v = row_cache[i];
    else if (mode == 0) v = to_f32(x[base + i]);
    else v = res[base + i];
    h_out[base + i] = from_f32<T>((v * inv) * to_f32(w[i]));
  }
}

// Vectorised variant: the row is read once, 8 elements per thread and pass (16-byte loads of x, two of the
// residual), kept in registers between the sum of squares and the scaling.  hidden % 8 == 0, pointers
// 16-byte aligned, hidden <= 8 * ITERS * blockDim.  Same results as the kernel above up to the order of the
// partial sums, which depends on hidden only.
template <typename T> struct Vec8;
template <> struct Vec8<bf16> {
  uint4 raw;
  __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void get(float (&v)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ __forceinline__ void set(const float (&v)[8]) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  }
};
template <> struct Vec8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4);
  }
  __device__ __forceinline__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = a; *reinterpret_cast<float4*>(p + 4) = b;
  }
  __device__ __forceinline__ void get(float (&v)[8]) const {
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  __device__ __forceinline__ void set(const float (&v)[8]) {
    a = make_float4(v[0], v[1], v[2], v[3]); b = make_float4(v[4], v[5], v[6], v[7]);
  }
};

template <typename T, typename WT, int ITERS>
__global__ void add_rmsnorm_vec_kernel(T* __restrict__ h_out, const T* __restrict__ x, float* __restrict__ res,
                                       const WT* __restrict__ w, int hidden, float eps, int mode) {
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * hidden;
  float v[ITERS][8];
  float ss = 0.f;
  pdl_launch_dependents();
  pdl_wait();
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 8;
    if (i < hidden) {
      Vec8<T> xv;
      xv.load(x + base + i);
      xv.get(v[it]);
      if (mode == 2) {
        Vec8<float> rv;
        rv.load(res + base + i);
        float r[8];
        rv.get(r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[it][e] += r[e];
      }
      if (mode != 0) {
        Vec8<float> rv;
        rv.set(v[it]);
        rv.store(res + base + i);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[it][e], v[it][e], ss);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 8;
    if (i < hidden) {
      Vec8<WT> wv;
      wv.load(w + i);
      float wf[8], o[8];
      wv.get(wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[it][e] * inv) * wf[e];
      Vec8<T> ov;
      ov.set(o);
      ov.store(h_out + base + i);
    }
  }
}

// The second half of an RMSNorm whose first half another kernel did (the residual form of the weight-streaming
// product): h = (res / rms) * w, the row's sum of squares given as `parts` partial sums.  One block per row.
template <typename T, typename WT>
__global__ void finish_rmsnorm_kernel(T* __restrict__ h_out, const float* __restrict__ res, const float* __restrict__ sumsq,
                                      int parts, long long ld, const WT* __restrict__ w, int hidden, float eps) {
  __shared__ float scratch[33];
  float ss = 0.f;
  for (int p = threadIdx.x; p < parts; p += blockDim.x) ss += sumsq[(size_t)blockIdx.x * ld + p];
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  const size_t base = (size_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    h_out[base + i] = from_f32<T>((res[base + i] * inv) * to_f32(w[i]));
}

template <typename T, typename WT>
static int launch(void* h, const void* x, float* res, const void* w, int n, int hidden, float eps, int mode,
                  cudaStream_t s) {
  const bool aligned = hidden % 8 == 0 && ((uintptr_t)h | (uintptr_t)x | (uintptr_t)res | (uintptr_t)w) % 16 == 0;
  if (aligned && hidden <= 8 * 2 * 1024) {
    const int vecs = hidden / 8;
    if (vecs <= 1024) {
      const int threads = ((vecs + 31) / 32) * 32;
      return launch_pdl(add_rmsnorm_vec_kernel<T, WT, 1>, dim3(n), dim3(threads), 0, s, (T*)h, (const T*)x, res,
                        (const WT*)w, hidden, eps, mode);
    }
    return launch_pdl(add_rmsnorm_vec_kernel<T, WT, 2>, dim3(n), dim3(1024), 0, s, (T*)h, (const T*)x, res,
                      (const WT*)w, hidden, eps, mode);
  }
  int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
  const size_t smem = (size_t)hidden * 4;
  const int cache_row = smem <= 40 * 1024;
  add_rmsnorm_kernel<T, WT><<<n, threads, cache_row ? smem : 0, s>>>((T*)h, (const T*)x, res, (const WT*)w, hidden,
                                                                     eps, mode, cache_row);
  return LMSF_LAUNCH_STATUS();
}

}  // namespace lmsf

// x, h: [n, hidden] of `dtype`; res: [n, hidden] float32 (modes 1, 2); w: [hidden] of `w_dtype`.
// h may alias x.
LMSF_API int lmsf_add_rmsnorm(void* h, const void* x, float* res, const void* w, int n, int hidden, float eps,
                              int mode, int dtype, int w_dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (hidden <= 0) LMSF_REFUSE("rmsnorm: hidden=%d must be positive", hidden);
  if (mode < 0 || mode > 2) LMSF_REFUSE("rmsnorm: unknown mode %d", mode);
  if (mode != 0 && res == nullptr) LMSF_REFUSE("rmsnorm: mode %d needs a residual buffer", mode);
  if (!(eps > 0.f)) LMSF_REFUSE("rmsnorm: eps must be positive");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32 && w_dtype == LMSF_F32) return launch<float, float>(h, x, res, w, n, hidden, eps, mode, s);
  if (dtype == LMSF_BF16 && w_dtype == LMSF_BF16) return launch<bf16, bf16>(h, x, res, w, n, hidden, eps, mode, s);
  if (dtype == LMSF_BF16 && w_dtype == LMSF_F32) return launch<bf16, float>(h, x, res, w, n, hidden, eps, mode, s);
  LMSF_REFUSE("rmsnorm: unsupported dtype pair (x %d, w %d)", dtype, w_dtype);
}

// h: [n, hidden] of `dtype` = (res / rms) * w, where sumsq[m * ld + 0 .. parts) add up to the sum of squares of row m
// of res (float32 [n, hidden]).
LMSF_API int lmsf_finish_rmsnorm(void* h, const float* res, const float* sumsq, int parts, long long ld, const void* w,
                                 int n, int hidden, float eps, int dtype, int w_dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (hidden <= 0 || parts <= 0 || ld < parts) LMSF_REFUSE("finish_rmsnorm: hidden=%d parts=%d", hidden, parts);
  if (!(eps > 0.f)) LMSF_REFUSE("finish_rmsnorm: eps must be positive");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_BF16 && w_dtype == LMSF_BF16)
    finish_rmsnorm_kernel<bf16, bf16><<<n, 256, 0, s>>>((bf16*)h, res, sumsq, parts, ld, (const bf16*)w, hidden, eps);
  else if (dtype == LMSF_BF16 && w_dtype == LMSF_F32)
    finish_rmsnorm_kernel<bf16, float><<<n, 256, 0, s>>>((bf16*)h, res, sumsq, parts, ld, (const float*)w, hidden, eps);
  else LMSF_REFUSE("finish_rmsnorm: unsupported dtype pair (h %d, w %d)", dtype, w_dtype);
  return LMSF_LAUNCH_STATUS();
}
