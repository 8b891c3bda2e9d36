// Causal attention of any mix of prompt portions and decoded tokens over the paged cache:
// the plain twin of the fast kernels, and the kernel of the float32 path.
//
// Counterparts in the reference: the dense prompt attention of
// core/src/model_executor/layers/attention.rs:106-159 and paged_attention_v1_kernel,
// vllm/kernels/attention/attention_kernels.cu:82-414.  Differences: one kernel serves prompt
// portions and decoded tokens alike (every query token reads its keys from pages, its own key
// included, which the cache write has stored before); the softmax is exact (no 1e-6 in the
// denominator, expf rather than __expf); any head size that is a multiple of 16 up to 256.
//
// One block of 4 warps per (query token, query head).  Keys are walked in tiles of 32 that are
// aligned to absolute positions; tile j belongs to warp j % 4; every warp keeps a running
// (max, sum, accumulator) and the four are merged in a fixed order.  The order of every
// floating-point operation therefore depends on the token's position only, not on how the
// tokens were cut into steps, which requests share the batch or which pages hold the keys.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_attention_generic)

namespace lmsf {

constexpr int kMaxHeadDim = 256;
constexpr int kWarps = 4;

struct GenericAttnArgs {
  const void* q; long long q_stride;           // [n_tokens, n_q_heads, hd]
  void* out; long long out_stride;             // [n_tokens, n_q_heads, hd]
  const void* cache; long long page_stride;    // [page][2][kv_head][slot][hd]
  const int* block_table; int max_blocks; int block_size;
  const int* token_seq; const int* positions;
  float scale; int window;                     // window <= 0: all keys
  int n_q_heads, n_kv_heads, head_dim;
  float softcap;                               // > 0: scores become softcap * tanh(score / softcap) before the softmax
  const float* slopes;                         // [n_q_heads] or null: slope * (key position - query position) is added to the scores
};

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) attention_generic_kernel(GenericAttnArgs a) {
  __shared__ float qs[kMaxHeadDim];
  __shared__ float part_acc[kWarps][kMaxHeadDim];
  __shared__ float part_m[kWarps], part_l[kWarps];

  const int t = blockIdx.x, head = blockIdx.y;
  const int hd = a.head_dim;
  const int kvh = head / (a.n_q_heads / a.n_kv_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = a.positions[t];
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int* table = a.block_table + (size_t)a.token_seq[t] * a.max_blocks;

  const T* q = (const T*)a.q + (size_t)t * a.q_stride + (size_t)head * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = to_f32(q[d]);
  __syncthreads();

  const size_t head_off = (size_t)kvh * a.block_size * hd;
  const size_t v_off = (size_t)a.n_kv_heads * a.block_size * hd;
  const int nd = (hd + 31) / 32;

  float m = -INFINITY, l = 0.f;
  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.f;

  for (int tile = lo / 32 + ((warp - lo / 32) % kWarps + kWarps) % kWarps; tile * 32 <= pos; tile += kWarps) {
    const int key = tile * 32 + lane;
    const bool valid = key >= lo && key <= pos;
    long long row = -1;  // element offset of this lane's key row inside the layer's cache
    float s = -INFINITY;
    if (valid) {
      const int page = table[key / a.block_size];
      if (page >= 0) {  // a key without a page (a fault of the caller) is left out, never read
        row = (long long)page * a.page_stride + head_off + (size_t)(key % a.block_size) * hd;
        const T* kr = (const T*)a.cache + row;
        float dot = 0.f;
        for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
        s = dot * a.scale;
        if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
        if (a.slopes) s = fmaf(a.slopes[head], (float)(key - pos), s);
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;  // nothing seen yet (uniform over the warp)
    const float p = row >= 0 ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);  // m = -inf on the first tile gives 0
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= alpha;
    for (int j = 0; j < 32; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long rj = __shfl_sync(0xffffffffu, row, j);
      if (rj < 0) continue;  // same for the whole warp
      const T* vr = (const T*)a.cache + rj + v_off;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (i < nd && d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
    m = m_new;
  }

  if (lane == 0) { part_m[warp] = m; part_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int d = lane + 32 * i;
    if (i < nd && d < hd) part_acc[warp][d] = acc[i];
  }
  __syncthreads();

  float M = part_m[0];
  for (int w = 1; w < kWarps; ++w) M = fmaxf(M, part_m[w]);
  float L = 0.f;
  float f[kWarps];
  for (int w = 0; w < kWarps; ++w) {
    f[w] = part_m[w] == -INFINITY ? 0.f : expf(part_m[w] - M);
    L = fmaf(part_l[w], f[w], L);
  }
  T* o = (T*)a.out + (size_t)t * a.out_stride + (size_t)head * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float v = 0.f;
    for (int w = 0; w < kWarps; ++w) v = fmaf(part_acc[w][d], f[w], v);
    o[d] = from_f32<T>(v / L);
  }
}

}  // namespace lmsf

// Two changes to the scores that some architectures make and only this kernel takes.  softcap > 0: the scaled scores
// are capped smoothly, softcap * tanh(score / softcap).  slopes ([n_q_heads] float32, may be null): a position encoding
// by a bias that grows with distance, slope[head] * (key position - query position), added to the scaled score as the
// reference's decode kernel adds it (vllm/kernels/attention/attention_kernels.cu:144-145, :232-234).
LMSF_API int lmsf_attention_generic_scores(const void* q, long long q_stride, void* out, long long out_stride,
                                           const void* cache, long long page_stride, const int* block_table, int max_blocks,
                                           int block_size, const int* token_seq, const int* positions, float scale,
                                           float softcap, const float* slopes, int window, int n_tokens, int n_q_heads,
                                           int n_kv_heads, int head_dim, int dtype, void* stream) {
  using namespace lmsf;
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim > kMaxHeadDim || head_dim % 16)
    LMSF_REFUSE("attention: head_dim=%d must be a multiple of 16 between 16 and %d", head_dim, kMaxHeadDim);
  if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    LMSF_REFUSE("attention: %d query heads cannot be grouped over %d kv heads", n_q_heads, n_kv_heads);
  if (n_q_heads > 65535) LMSF_REFUSE("attention: more than 65535 query heads");
  if (block_size <= 0 || max_blocks <= 0) LMSF_REFUSE("attention: bad block table geometry");
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("attention: unknown dtype code %d", dtype);
  GenericAttnArgs a{q, q_stride, out, out_stride, cache, page_stride, block_table, max_blocks, block_size,
                    token_seq, positions, scale, window, n_q_heads, n_kv_heads, head_dim, softcap > 0.f ? softcap : 0.f, slopes};
  dim3 grid(n_tokens, n_q_heads);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) attention_generic_kernel<float><<<grid, kWarps * 32, 0, s>>>(a);
  else attention_generic_kernel<bf16><<<grid, kWarps * 32, 0, s>>>(a);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_attention_generic(const void* q, long long q_stride, void* out, long long out_stride,
                                    const void* cache, long long page_stride, const int* block_table, int max_blocks,
                                    int block_size, const int* token_seq, const int* positions, float scale,
                                    int window, int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int dtype,
                                    void* stream) {
  return lmsf_attention_generic_scores(q, q_stride, out, out_stride, cache, page_stride, block_table, max_blocks, block_size,
                                       token_seq, positions, scale, 0.f, nullptr, window, n_tokens, n_q_heads, n_kv_heads,
                                       head_dim, dtype, stream);
}
