// Prefill half of attention_mma.cu (included there: it shares HD, the stages and the fragment helpers).
#pragma once

namespace lmsf {
namespace fa {

struct PrefillArgs {
  const bf16* q; long long q_stride;         // [n_tokens][n_q_heads * HD]
  bf16* out; long long out_stride;
  PagedKV kv;
  const int* block_table; int max_blocks;
  const int* tile_seq;                       // [grid.x] request of each 64-token query tile
  const int* tile_q0;                        // [grid.x] first token of the tile, counted inside the request's portion
  const int* cu_q; const int* ctx_len;
  float scale; int window;
  int n_q_heads, group;
};

// One block: 64 query tokens (16 per warp) of one head.  Query i of a portion of n tokens of a request
// that holds ctx keys after this step sits at position ctx - n + i and sees keys lo..position.
__global__ void __launch_bounds__(kThreads) prefill_kernel(PrefillArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  // blocks start in the order (all heads of tile 0, all heads of tile 1, ...); the caller lists the tiles that
  // see the most keys first
  const int seq = a.tile_seq[blockIdx.y], q0 = a.tile_q0[blockIdx.y];
  const int head = blockIdx.x, kvh = head / a.group;
  const int tok0 = a.cu_q[seq], n = a.cu_q[seq + 1] - tok0, ctx = a.ctx_len[seq];
  const int start = ctx - n;                                    // position of the portion's first token
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g4 = lane >> 2, t4 = lane & 3;
  const int rows_valid = min(kTileKeys, n - q0);                // query rows of this tile that exist
  const int hi = start + q0 + rows_valid;                       // keys < hi are visible to the tile's last row
  const int lo = a.window > 0 ? max(0, start + q0 - a.window + 1) : 0;
  const int* table = a.block_table + (size_t)seq * a.max_blocks;

  // this thread's two rows
  int pos[2];
  bool row_ok[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g4 + h * 8;
    row_ok[h] = r < rows_valid;
    pos[h] = start + q0 + min(r, rows_valid - 1);
  }
  const int warp_last_pos = start + q0 + min(warp * 16 + 15, rows_valid - 1);
  const int warp_first_pos = start + q0 + min(warp * 16, rows_valid - 1);
  const int warp_lo = a.window > 0 ? max(0, warp_first_pos - a.window + 1) : 0;

  uint32_t qf[kKSteps][4];
#pragma unroll
  for (int ks = 0; ks < kKSteps; ++ks)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int h = r & 1, col = ks * 16 + t4 * 2 + (r >> 1) * 8;
      const int row = warp * 16 + g4 + h * 8;
      qf[ks][r] = row_ok[h] ? *reinterpret_cast<const uint32_t*>(
                                  a.q + (size_t)(tok0 + q0 + row) * a.q_stride + (size_t)head * HD + col) : 0u;
    }

  const int tile_begin = lo / kTileKeys, tile_end = (hi + kTileKeys - 1) / kTileKeys;
  const int n_tiles = tile_end - tile_begin;
  const uint32_t smem_base = smem_u32(smem);
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_tiles) load_stage<HD>(smem_base + s * St::kBytes, a.kv, table, kvh, (tile_begin + s) * kTileKeys, lo, hi);
    cp_async_commit();
  }

  RowState st{{-INFINITY, -INFINITY}, {0.f, 0.f}};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const float sl2 = a.scale * kLog2e;

  for (int i = 0; i < n_tiles; ++i) {
    cp_async_wait<kStages - 2>();
    __syncthreads();
    {
      const int nxt = i + kStages - 1;
      if (nxt < n_tiles)
        load_stage<HD>(smem_base + (nxt % kStages) * St::kBytes, a.kv, table, kvh, (tile_begin + nxt) * kTileKeys, lo, hi);
      cp_async_commit();
    }
    const int key0 = (tile_begin + i) * kTileKeys;
    if (key0 > warp_last_pos || key0 + kTileKeys <= warp_lo) continue;   // all masked for this warp
    const uint32_t kbase = smem_base + (i % kStages) * St::kBytes;
    const uint32_t vbase = kbase + kTileKeys * St::kRowBytes;

    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {            // 16 keys per ldmatrix
        uint32_t b[4];
        const int mi = lane >> 3, r = lane & 7;
        ldmatrix_x4(b, kbase + St::off(kb * 16 + (mi >> 1) * 8 + r, ks * 2 + (mi & 1)));
        mma_16816(s[2 * kb], qf[ks], b[0], b[1]);
        mma_16816(s[2 * kb + 1], qf[ks], b[2], b[3]);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + j * 8 + t4 * 2 + (e & 1), h = e >> 1;
        const bool ok = key <= pos[h] && (a.window <= 0 || key > pos[h] - a.window);
        const float v = ok ? s[j][e] * sl2 : -INFINITY;
        s[j][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(st.m[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;      // a row that has seen no key yet
      alpha[h] = exp2f(st.m[h] - m_use[h]);
      st.m[h] = m_new;
      st.l[h] *= alpha[h];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[j][e] = exp2f(s[j][e] - m_use[e >> 1]);
        st.l[e >> 1] += s[j][e];
      }
#pragma unroll
    for (int nn = 0; nn < HD / 8; ++nn) {
      o[nn][0] *= alpha[0]; o[nn][1] *= alpha[0];
      o[nn][2] *= alpha[1]; o[nn][3] *= alpha[1];
    }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      uint32_t pf[4];
      pf[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
      pf[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
      pf[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
      pf[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
      for (int n2 = 0; n2 < kKSteps; ++n2) {
        uint32_t b[4];
        const int mi = lane >> 3, r = lane & 7;
        ldmatrix_x4_trans(b, vbase + St::off(kb * 16 + (mi & 1) * 8 + r, n2 * 2 + (mi >> 1)));
        mma_16816(o[2 * n2], pf, b[0], b[1]);
        mma_16816(o[2 * n2 + 1], pf, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!row_ok[h]) continue;
    const int row = warp * 16 + g4 + h * 8;
    const float inv = 1.0f / st.l[h];
    bf16* dst = a.out + (size_t)(tok0 + q0 + row) * a.out_stride + (size_t)head * HD + t4 * 2;
#pragma unroll
    for (int nn = 0; nn < HD / 8; ++nn)
      *reinterpret_cast<uint32_t*>(dst + nn * 8) = pack_bf16(o[nn][2 * h] * inv, o[nn][2 * h + 1] * inv);
  }
}

}  // namespace fa
}  // namespace lmsf

// Portions of prompts: tile_seq / tile_q0 list one entry per 64 query tokens (built by the caller).
LMSF_API int lmsf_attention_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                                    const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                    const int* block_table, int max_blocks, const int* tile_seq, const int* tile_q0,
                                    int n_tiles, const int* cu_q, const int* ctx_len, float scale, int window,
                                    int n_q_heads, int head_dim, void* stream) {
  using namespace lmsf;
  using namespace lmsf::fa;
  if (n_tiles <= 0) return 0;
  if (head_dim != HD) LMSF_REFUSE("attention_prefill: built for head_dim=%d, called with %d", HD, head_dim);
  if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    LMSF_REFUSE("attention_prefill: %d query heads cannot be grouped over %d kv heads", n_q_heads, n_kv_heads);
  if (n_tiles > 65535) LMSF_REFUSE("attention_prefill: more than 65535 query tiles in one launch");
  if (block_size <= 0 || max_blocks <= 0) LMSF_REFUSE("attention_prefill: bad block table geometry");
  PrefillArgs a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  if (!make_paged_kv(a.kv, cache, page_stride, block_size, n_kv_heads))
    LMSF_REFUSE("attention: block_size=%d must be a power of two", block_size);
  a.block_table = block_table; a.max_blocks = max_blocks; a.tile_seq = tile_seq; a.tile_q0 = tile_q0;
  a.cu_q = cu_q; a.ctx_len = ctx_len; a.scale = scale; a.window = window; a.n_q_heads = n_q_heads;
  a.group = n_q_heads / n_kv_heads;
  const int smem = kStages * St::kBytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  prefill_kernel<<<dim3(n_q_heads, n_tiles), kThreads, smem, (cudaStream_t)stream>>>(a);
  return LMSF_LAUNCH_STATUS();
}
