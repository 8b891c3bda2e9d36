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

template <typename T, typename WT>
static int launch(void* h, const void* x, float* res, const void* w, int n, int hidden, float eps, int mode,
                  cudaStream_t s) {
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
