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
#include <type_traits>

LMSF_DEFINE_LAST_ERROR(lmsf_rope_cache)

#ifndef LMSF_ROPE_ONE_BLOCK_TOKENS
#define LMSF_ROPE_ONE_BLOCK_TOKENS 256
#endif

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
      p[ix] = from_f32<T>(rot_first(x, y, c, s));
      p[iy] = from_f32<T>(rot_second(x, y, c, s));
    } else if (kc) {
      const int g = head - a.n_q_heads;
      const T* p = k + (size_t)g * hd;
      const float x = to_f32(p[ix]), y = to_f32(p[iy]);
      T* d = kc + g * head_pitch;
      d[ix] = from_f32<T>(rot_first(x, y, c, s));
      d[iy] = from_f32<T>(rot_second(x, y, c, s));
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

// Vectorised variant for NeoX pairing: work items of 16 bytes (VEC elements), spread over gridDim.y blocks
// per token.  Needs rot_dim / 2, head_dim - rot_dim and all row strides to be multiples of VEC and 16-byte
// aligned pointers.  Same arithmetic as the kernel above, element by element.
template <typename T, int VEC>
__global__ void rope_cache_vec_kernel(RopeCacheArgs a) {
  extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
  const int t = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = a.positions[t];
  const int half = a.inv_freq ? a.rot_dim / 2 : 0;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * a.inv_freq[i], &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  __syncthreads();
  const int hd = a.head_dim;
  T* kc = nullptr;
  T* vc = nullptr;
  if (a.cache) {
    const int page = a.block_table[(size_t)a.token_seq[t] * a.max_blocks + pos / a.block_size];
    if (page < 0) {
      if (threadIdx.x == 0 && blockIdx.y == 0 && a.error_flag) atomicExch(a.error_flag, 2);
    } else {
      kc = (T*)a.cache + (size_t)page * a.page_stride + (size_t)(pos % a.block_size) * hd;
      vc = kc + (size_t)a.n_kv_heads * a.block_size * hd;
    }
  }
  T* q = (T*)a.q + (size_t)t * a.q_stride;
  const T* k = (const T*)a.k + (size_t)t * a.k_stride;
  const T* v = (const T*)a.v + (size_t)t * a.v_stride;
  const size_t head_pitch = (size_t)a.block_size * hd;
  const int rot = 2 * half, hv = half / VEC, tail_v = (hd - rot) / VEC, hd_v = hd / VEC;
  const int n_qrot = a.n_q_heads * hv;
  const int n_krot = kc ? a.n_kv_heads * hv : 0;
  const int n_ktail = kc ? a.n_kv_heads * tail_v : 0;
  const int n_v = kc ? a.n_kv_heads * hd_v : 0;
  const int total = n_qrot + n_krot + n_ktail + n_v;
  typedef typename std::conditional<VEC == 8, uint4, float4>::type Raw;
  for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < total; w += gridDim.y * blockDim.x) {
    if (w < n_qrot + n_krot) {
      const bool is_q = w < n_qrot;
      const int u = is_q ? w : w - n_qrot;
      const int head = u / hv, i0 = (u % hv) * VEC;
      const T* src = is_q ? q + (size_t)head * hd : k + (size_t)head * hd;
      T* dst = is_q ? q + (size_t)head * hd : kc + head * head_pitch;
      Raw xr = *reinterpret_cast<const Raw*>(src + i0), yr = *reinterpret_cast<const Raw*>(src + half + i0);
      T* xe = reinterpret_cast<T*>(&xr);
      T* ye = reinterpret_cast<T*>(&yr);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float c = cs[i0 + e], s = cs[half + i0 + e];
        const float x = to_f32(xe[e]), y = to_f32(ye[e]);
        xe[e] = from_f32<T>(rot_first(x, y, c, s));
        ye[e] = from_f32<T>(rot_second(x, y, c, s));
      }
      *reinterpret_cast<Raw*>(dst + i0) = xr;
      *reinterpret_cast<Raw*>(dst + half + i0) = yr;
    } else if (w < n_qrot + n_krot + n_ktail) {
      const int u = w - n_qrot - n_krot;
      const int g = u / tail_v, i0 = rot + (u % tail_v) * VEC;
      *reinterpret_cast<Raw*>(kc + g * head_pitch + i0) = *reinterpret_cast<const Raw*>(k + (size_t)g * hd + i0);
    } else {
      const int u = w - n_qrot - n_krot - n_ktail;
      const int g = u / hd_v, i0 = (u % hd_v) * VEC;
      *reinterpret_cast<Raw*>(vc + g * head_pitch + i0) = *reinterpret_cast<const Raw*>(v + (size_t)g * hd + i0);
    }
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
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = inv_freq ? (size_t)rot_dim * sizeof(float) : 0;
  const int vec = dtype == LMSF_F32 ? 4 : 8;
  const int rot = inv_freq ? rot_dim : 0;
  const bool vec_ok = (is_neox || !inv_freq) && (rot / 2) % vec == 0 && (head_dim - rot) % vec == 0 &&
                      q_stride % vec == 0 && (!cache || (k_stride % vec == 0 && v_stride % vec == 0 && page_stride % vec == 0)) &&
                      ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)cache) % 16 == 0;
  if (vec_ok) {
    const int items = (n_q_heads * (rot / 2) + (cache ? n_kv_heads * (rot / 2 + (head_dim - rot) + head_dim) : 0)) / vec;
    int gy = ceil_div(items > 0 ? items : 1, 128);
    if (gy > 8) gy = 8;
    // Every block of a token computes the token's angles and looks its page up before it moves a byte: with many
    // tokens (a prompt portion) one block of 256 threads per token does that once; with few (a decode step) the
    // token's work is spread over several blocks so that the device is not left empty.
    int threads = 128;
    if (n_tokens >= LMSF_ROPE_ONE_BLOCK_TOKENS) { gy = 1; threads = 256; }
    dim3 grid(n_tokens, gy);
    if (dtype == LMSF_F32) return launch_pdl(rope_cache_vec_kernel<float, 4>, grid, dim3(threads), smem, s, a);
    return launch_pdl(rope_cache_vec_kernel<bf16, 8>, grid, dim3(threads), smem, s, a);
  }
  const int work = (n_q_heads + 2 * n_kv_heads) * head_dim / 2;
  const int threads = work >= 1024 ? 256 : (work >= 256 ? 128 : 64);
  if (dtype == LMSF_F32) rope_cache_kernel<float><<<n_tokens, threads, smem, s>>>(a);
  else rope_cache_kernel<bf16><<<n_tokens, threads, smem, s>>>(a);
  return LMSF_LAUNCH_STATUS();
}
