// Token sampling from float32 logits: greedy (argmax, lowest index wins ties) and temperature
// sampling as an exponential race, argmax_v(softmax(logits / T)_v / q_v) with q_v ~ Exp(1),
// which is argmax_v(logits_v / T - log q_v).
// Counterparts in the reference: greedy_sample and multinomial in
// core/src/model_executor/layers/sampler.rs:326-384 with the exponential noise of
// tops/csrc/tops/oneflow/kernel/distribution/exponential_distribution.cu:80-155.  Difference: the
// noise is a pure function of (request seed, index of the output token, vocabulary id) through
// Philox-4x32-10, so a draw does not depend on which requests share the batch, on how prompts
// were cut or on a recomputation after preemption.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_sampling)

namespace lmsf {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// -log(q), q = -log(u), u = (r + 1) / 2^32 in (0, 1]
__device__ __forceinline__ double neg_log_exponential(uint32_t seed_lo, uint32_t seed_hi, uint32_t step, uint32_t v) {
  uint32_t r[4];
  philox4x32_10(v, step, 0u, 0u, seed_lo, seed_hi, r);
  const double u = ((double)r[0] + 1.0) * (1.0 / 4294967296.0);
  return -log(-log(u));
}

struct Best { double score; int index; };
__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.score > a.score || (b.score == a.score && b.index < a.index)) return b;
  return a;
}

// One block per row.  temperature < 1e-5 selects greedy (core/src/common/sampling_params.rs:156-164).
__global__ void sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long long row_stride, int vocab,
                              const float* __restrict__ temperature, const unsigned long long* __restrict__ seed,
                              const int* __restrict__ step) {
  __shared__ Best sh[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const float T = temperature ? temperature[r] : 0.f;
  const bool greedy = T < 1e-5f;
  const uint32_t slo = seed ? (uint32_t)(seed[r] & 0xffffffffull) : 0u, shi = seed ? (uint32_t)(seed[r] >> 32) : 0u;
  const uint32_t st = step ? (uint32_t)step[r] : 0u;
  Best b{-INFINITY, 0x7fffffff};
  for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
    const float x = row[v];
    if (x != x) continue;  // a NaN never wins
    double s = (double)x;
    if (!greedy) s = s / (double)T + neg_log_exponential(slo, shi, st, (uint32_t)v);
    b = better(b, Best{s, v});
  }
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, b.score, o), __shfl_xor_sync(0xffffffffu, b.index, o)};
    b = better(b, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = b;
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    b = lane < nw ? sh[lane] : Best{-INFINITY, 0x7fffffff};
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, b.score, o), __shfl_xor_sync(0xffffffffu, b.index, o)};
      b = better(b, other);
    }
    if (lane == 0) out[r] = b.index == 0x7fffffff ? 0 : b.index;
  }
}

}  // namespace lmsf

// logits: [rows, vocab] float32; temperature [rows] float32, seed [rows] uint64, step [rows] int32
// (all three may be null: greedy).  out: [rows] int32.
LMSF_API int lmsf_sample(int* out, const float* logits, long long row_stride, int rows, int vocab,
                         const float* temperature, const unsigned long long* seed, const int* step, void* stream) {
  using namespace lmsf;
  if (rows <= 0) return 0;
  if (vocab <= 0 || row_stride < vocab) LMSF_REFUSE("sample: vocab=%d, row_stride=%lld", vocab, row_stride);
  const int threads = vocab >= 8192 ? 1024 : 256;
  sample_kernel<<<rows, threads, 0, (cudaStream_t)stream>>>(out, logits, row_stride, vocab, temperature, seed, step);
  return LMSF_LAUNCH_STATUS();
}
