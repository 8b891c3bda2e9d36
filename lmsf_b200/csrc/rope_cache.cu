// Rotary position encoding of q and k fused with the write of k and v into the paged cache.
// Counterparts in the reference: rotary_embedding_kernel (vllm/kernels/pos_encoding_kernels.cu:12-77)
// followed by reshape_and_cache_kernel (vllm/kernels/cache_kernels.cu:190-232).  Differences: the
// angle is position * inv_freq in float32 and the rotation is done in float32 (the reference reads
// a cos/sin table rounded to the model type and rotates in that type); the page of a token is
// looked up in the request's block table here rather than through a precomputed slot mapping; k
// goes to the cache only (attention always reads keys from pages).
//
// Cache layout of one layer: [page][2 (k, v)][kv_head][slot][head_dim].
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_rope_cache)

namespace lmsf {

struct RopeCacheArgs {
  void* q; const void* k; const void* v;       // rows of n_q_heads*hd, n_kv_heads*hd, n_kv_heads*hd
  long long q_stride, k_stride, v_stride;      // elements between tokens
  const int* positions;                        // [n_tokens]
  const int* token_seq;                        // [n_tokens] -> row of block_table
  const int* block_table;                      // [n_seqs, max_blocks], -1 = no page
  int max_blocks, block_size;
  void* cache;                                 // null: rotate q only
  long long page_stride;                       // elements between pages of this layer
  const float* inv_freq;                       // [rot_dim / 2], null: no rotation
  int rot_dim, is_neox;
  int n_q_heads, n_kv_heads, head_dim;
  int* error_flag;
};

template <typename T>
__global__ void rope_cache_kernel(RopeCacheArgs a) {
  extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
  const int t = blockIdx.x;
  const int pos = a.positions[t];
  const int half = a.rot_dim / 2;
  if (a.inv_freq) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float ang = (float)pos * a.inv_freq[i];
      float s, c;
      sincosf(ang, &s, &c);
      cs[i] = c;
      cs[half + i] = s;
    }
  }
  __syncthreads();

  const int hd = a.head_dim;
  T* kc = nullptr;
  T* vc = nullptr;
  if (a.cache) {
    const int seq = a.token_seq[t];
    const int page = a.block_table[(size_t)seq * a.max_blocks + pos / a.block_size];
    if (page < 0) {
      if (threadIdx.x == 0 && a.error_flag) atomicExch(a.error_flag, 2);
    } else {
      const int slot = pos % a.block_size;
      kc = (T*)a.cache + (size_t)page * a.page_stride + (size_t)slot * hd;
      vc = kc + (size_t)a.n_kv_heads * a.block_size * hd;
    }
  }
  T* q = (T*)a.q + (size_t)t * a.q_stride;
  const T* k = (const T*)a.k + (size_t)t * a.k_stride;
  const T* v = (const T*)a.v + (size_t)t * a.v_stride;
  const size_t head_pitch = (size_t)a.block_size * hd;  // between kv heads inside a page

  // rotated pairs of q (in place) and k (to the cache)
  const int n_rot_heads = a.inv_freq ? a.n_q_heads + (a.k ? a.n_kv_heads : 0) : 0;
  for (int w = threadIdx.x; w < n_rot_heads * half; w += blockDim.x) {
    const int head = w / half, i = w % half;
    const int ix = a.is_neox ? i : 2 * i;
    const int iy = a.is_neox ? i + half : 2 * i + 1;
    const float c = cs[i], s = cs[half + i];
    if (head < a.n_q_heads) {
      T* p = q + (size_t)head * hd;
      const float x = to_f32(p[ix]), y = to_f32(p[iy]);
      p[ix] = from_f32<T>(x * c - y * s);
      p[iy] = from_f32<T>(y * c + x * s);
    } else if (kc) {
      const int g = head - a.n_q_heads;
      const T* p = k + (size_t)g * hd;
      const float x = to_f32(p[ix]), y = to_f32(p[iy]);
      T* d = kc + g * head_pitch;
      d[ix] = from_f32<T>(x * c - y * s);
      d[iy] = from_f32<T>(y * c + x * s);
    }
  }
  if (!kc) return;
  // the part of k that is not rotated, and v
  const int rot = a.inv_freq ? a.rot_dim : 0;
  const int tail = hd - rot;
  for (int w = threadIdx.x; w < a.n_kv_heads * tail; w += blockDim.x) {
    const int g = w / tail, i = rot + w % tail;
    kc[g * head_pitch + i] = k[(size_t)g * hd + i];
  }
  for (int w = threadIdx.x; w < a.n_kv_heads * hd; w += blockDim.x) {
    const int g = w / hd, i = w % hd;
    vc[g * head_pitch + i] = v[(size_t)g * hd + i];
  }
}

}  // namespace lmsf

LMSF_API int lmsf_rope_cache_write(void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                   long long v_stride, const int* positions, const int* token_seq,
                                   const int* block_table, int max_blocks, int block_size, void* cache,
                                   long long page_stride, const float* inv_freq, int rot_dim, int is_neox,
                                   int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int dtype,
                                   int* error_flag, void* stream) {
  using namespace lmsf;
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || n_q_heads < 0 || n_kv_heads < 0) LMSF_REFUSE("rope_cache: bad head sizes");
  if (inv_freq && (rot_dim <= 0 || rot_dim % 2 || rot_dim > head_dim))
    LMSF_REFUSE("rope_cache: rot_dim=%d must be even and at most head_dim=%d", rot_dim, head_dim);
  if (cache && (!k || !v || !block_table || !token_seq || block_size <= 0 || max_blocks <= 0))
    LMSF_REFUSE("rope_cache: a cache write needs k, v, a block table and the block size");
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("rope_cache: unknown dtype code %d", dtype);
  RopeCacheArgs a{q, k, v, q_stride, k_stride, v_stride, positions, token_seq, block_table, max_blocks, block_size,
                  cache, page_stride, inv_freq, rot_dim, is_neox, n_q_heads, n_kv_heads, head_dim, error_flag};
  const int work = (n_q_heads + 2 * n_kv_heads) * head_dim / 2;
  const int threads = work >= 1024 ? 256 : (work >= 256 ? 128 : 64);
  const size_t smem = inv_freq ? (size_t)rot_dim * sizeof(float) : 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) rope_cache_kernel<float><<<n_tokens, threads, smem, s>>>(a);
  else rope_cache_kernel<bf16><<<n_tokens, threads, smem, s>>>(a);
  return LMSF_LAUNCH_STATUS();
}
