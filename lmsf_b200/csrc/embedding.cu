// Embedding gather: out[t, :] = table[ids[t], :].
// Counterpart in the reference: index_select in
// core/src/model_executor/layers/vocab_parallel_embedding.rs:28-37.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_embedding)

namespace lmsf {

// One block per token.  Rows are copied as 16-byte words when the row size allows it.
// An id outside [0, vocab) writes a row of zeros and raises *error_flag (never reads outside the table).
template <typename W>
__global__ void embedding_kernel(W* __restrict__ out, const W* __restrict__ table, const int* __restrict__ ids,
                                 int row_words, int vocab, int* __restrict__ error_flag) {
  const int t = blockIdx.x;
  const int id = ids[t];
  W* dst = out + (size_t)t * row_words;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
    W zero;
    memset(&zero, 0, sizeof(W));
    for (int i = threadIdx.x; i < row_words; i += blockDim.x) dst[i] = zero;
    return;
  }
  const W* src = table + (size_t)id * row_words;
  for (int i = threadIdx.x; i < row_words; i += blockDim.x) dst[i] = src[i];
}

// The same with every value multiplied by `scale` (float32 product, rounded once): the embedding scale that some
// architectures apply to their input (sqrt of the width, for one).
template <typename T>
__global__ void embedding_scaled_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                        int hidden, int vocab, float scale, int* __restrict__ error_flag) {
  const int t = blockIdx.x;
  const int id = ids[t];
  T* dst = out + (size_t)t * hidden;
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? from_f32<T>(to_f32(src[i]) * scale) : from_f32<T>(0.f);
}

// token_ids[dst[i]] = source[src[i]] for every i with dst[i] >= 0: puts tokens that were sampled on the device
// into the next step's input without a round trip to the host.
__global__ void patch_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ dst, const int* __restrict__ src,
                                    const int* __restrict__ source, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && dst[i] >= 0) token_ids[dst[i]] = source[src[i]];
}

}  // namespace lmsf

LMSF_API int lmsf_patch_tokens(int* token_ids, const int* dst, const int* src, const int* source, int n, void* stream) {
  if (n <= 0) return 0;
  lmsf::patch_tokens_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(token_ids, dst, src, source, n);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_embedding(void* out, const void* table, const int* ids, int n_tokens, int hidden, int vocab,
                            int dtype, int* error_flag, void* stream) {
  using namespace lmsf;
  if (n_tokens <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) LMSF_REFUSE("embedding: hidden=%d vocab=%d must be positive", hidden, vocab);
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("embedding: unknown dtype code %d", dtype);
  const size_t row_bytes = (size_t)hidden * (dtype == LMSF_F32 ? 4 : 2);
  cudaStream_t s = (cudaStream_t)stream;
  const bool aligned16 = row_bytes % 16 == 0 && ((uintptr_t)out % 16 == 0) && ((uintptr_t)table % 16 == 0);
  if (aligned16) {
    const int words = (int)(row_bytes / 16);
    const int threads = words >= 256 ? 256 : (words >= 64 ? 64 : 32);
    embedding_kernel<uint4><<<n_tokens, threads, 0, s>>>((uint4*)out, (const uint4*)table, ids, words, vocab,
                                                          error_flag);
  } else if (dtype == LMSF_F32) {
    embedding_kernel<float><<<n_tokens, 128, 0, s>>>((float*)out, (const float*)table, ids, hidden, vocab, error_flag);
  } else {
    embedding_kernel<unsigned short><<<n_tokens, 128, 0, s>>>((unsigned short*)out, (const unsigned short*)table, ids,
                                                               hidden, vocab, error_flag);
  }
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_embedding_scaled(void* out, const void* table, const int* ids, int n_tokens, int hidden, int vocab,
                                   float scale, int dtype, int* error_flag, void* stream) {
  using namespace lmsf;
  if (n_tokens <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) LMSF_REFUSE("embedding: hidden=%d vocab=%d must be positive", hidden, vocab);
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("embedding: unknown dtype code %d", dtype);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == LMSF_F32)
    embedding_scaled_kernel<float><<<n_tokens, threads, 0, s>>>((float*)out, (const float*)table, ids, hidden, vocab, scale, error_flag);
  else
    embedding_scaled_kernel<bf16><<<n_tokens, threads, 0, s>>>((bf16*)out, (const bf16*)table, ids, hidden, vocab, scale, error_flag);
  return LMSF_LAUNCH_STATUS();
}
