// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, float32 scores,
// softmax and accumulators), compiled for one head size: -DLMSF_HEAD_DIM=<multiple of 16, 16..128>.
//
//   decode  : one query token per request; a block serves the query heads that share one kv head
//             (rows of the product = heads), the keys are split over blocks (grid.x); up to 8 splits add
//             up through the shared memory of their cluster, more through scratch memory, where the block
//             that delivers last adds them.  Counterpart in the reference:
//             paged_attention_v2_kernel + reduce, vllm/kernels/attention/attention_kernels.cu:441-572.
//   prefill : portions of prompts (any number of query tokens per request, at any position); a block
//             serves 64 query tokens of one head and walks the keys 0..position from pages.
//             Counterpart in the reference: the dense prompt attention of
//             core/src/model_executor/layers/attention.rs:106-159, which materialises all scores.
//
// Keys and values are brought into shared memory in stages of 64 keys with cp.async (three stages in
// flight); both kernels read them with ldmatrix.  The softmax is exact (no constant in the denominator).
#include "attention_mma.cuh"

#ifndef LMSF_HEAD_DIM
#error "compile with -DLMSF_HEAD_DIM=<head size>"
#endif

LMSF_DEFINE_LAST_ERROR(lmsf_attention_mma)

namespace lmsf {
namespace fa {

constexpr int HD = LMSF_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head size must be a multiple of 16 between 16 and 128");
// stages of 64 keys in flight per block
#ifdef LMSF_KV_STAGES
constexpr int kStages = LMSF_KV_STAGES;
#else
// head size 64: three stages of 16 KB leave room for four blocks on an SM, so that 64 requests x 8 kv heads run in
// one wave (with four stages and three blocks per SM they took 72 us a layer in two waves)
constexpr int kStages = HD < 64 ? 4 : 3;
#endif
constexpr int kKSteps = HD / 16;   // k-steps of q k^T; also pairs of 8-wide output tiles of p v
constexpr float kLog2e = 1.4426950408889634f;
using St = Stage<HD>;                 // the prefill kernel's stages (64 keys)
// Decode blocks come in two widths, W = 4 or 2 warps; a warp takes 16 keys of a tile, so tiles hold 64 or 32 keys.
// Above head size 64 a stage of 64 keys is 35 KB and two blocks fit an SM: best for few requests, whose blocks
// are few and long.  With two warps and stages of 17 KB four blocks fit, and many requests (64 x 8 kv heads) run
// in one wave instead of two.

struct DecodeArgs {
  const bf16* q; long long q_stride;         // [n_tokens][n_q_heads * HD]
  bf16* out; long long out_stride;           // [n_tokens][n_q_heads * HD]
  float* part_o;                             // [n_seqs][n_q_heads][n_splits][HD] (n_splits > 1)
  float* part_lse;                           // [n_seqs][n_q_heads][n_splits]
  unsigned* counters;                        // [n_seqs][grid.y]: splits that have delivered; zero between launches
  PagedKV kv;
  const int* block_table; int max_blocks;
  const int* seq_ids;                        // [grid.z] requests served (null: 0, 1, 2, ...)
  const int* cu_q;                           // [n_seqs + 1] token offset of each request
  const int* ctx_len;                        // [n_seqs] keys of each request, the new token's included
  float scale; int window;
  int n_q_heads, group;                      // group = n_q_heads / n_kv_heads
  int n_splits;
  int cluster;                               // the splits of a request and group of heads form a thread-block cluster
  int rows;                                  // query heads a block holds at most: min(16, group); sizes the regions in which parts meet
  // Splits per request instead of one number for all: blockIdx.x is an entry of this list, {request, split, splits of
  // the request, splits of the requests before it}; a request of -1 is padding.  Null: every request has n_splits.
  const int4* items;
};

// Online-softmax state of the two rows (lane / 4 and lane / 4 + 8) that a thread holds.
struct RowState {
  float m[2], l[2];
};

// ------------------------------------------------------------------------------------------------ decode
constexpr int kMaxClusterSplits = 8;       // splits that add up through distributed shared memory
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// stores v at the same shared-memory offset as `local` in block `rank` of the cluster
__device__ __forceinline__ void st_cluster_f32(const float* local, unsigned rank, float v) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
constexpr int kTableCache = 512;           // block-table entries of a split that are kept in shared memory
constexpr int kMergeWeights = 4096;        // (heads of a block) x splits whose weights fit the shared memory used for adding up

// S: stages of the ring of key/value tiles (kStages; one more in the variant for launches of so few blocks that each
// has an SM to itself, below)
template <int W, int S = kStages>
__global__ void __launch_bounds__(32 * W) decode_kernel(DecodeArgs a) {
  constexpr int kDecWarps = W, kDecThreads = 32 * W, kDecTile = 16 * W;
  using DSt = Stage<HD, kDecTile>;
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_table[kTableCache];
  __shared__ int s_is_last;
  pdl_launch_dependents();
  int split = blockIdx.x, n_splits = a.n_splits, item_seq = 0, splits_before = 0;
  if (a.items) {
    // the list was written by a kernel of this step (the first attention layer's, before its own launch): it may be
    // read only after the dependency wait, so a launch with a list has no prologue that overlaps the kernel before
    pdl_wait();
    const int4 item = a.items[blockIdx.x];
    if (item.x < 0) return;
    item_seq = item.x; split = item.y; n_splits = item.z; splits_before = item.w;
  }
  // Until pdl_wait() only what no kernel of this step writes is read: the step's tables, and keys that were
  // cached before this step.  The kernel before this one writes the new token's key, value and query.
  const int chunks_per_kvh = (a.group + 15) / 16;
  const int kvh = blockIdx.y / chunks_per_kvh, hchunk = blockIdx.y % chunks_per_kvh;
  const int seq = a.items ? item_seq : (a.seq_ids ? a.seq_ids[blockIdx.z] : blockIdx.z);
  if (!a.items) splits_before = seq * n_splits;                // where the request's partial results start, in splits
  const int* table = a.block_table + (size_t)seq * a.max_blocks;
  // The head of the request's block table goes to shared memory at once, beside the loads of its lengths: for
  // contexts of up to kTableCache pages no copy of the loop waits for a table entry from global memory, and
  // the entries do not have to wait for the lengths either.
  const int n_head = min(a.max_blocks, kTableCache);
  for (int i = threadIdx.x; i < n_head; i += kDecThreads) s_table[i] = table[i];
  const int token = a.cu_q[seq];
  const int ctx = a.ctx_len[seq];
  const int lo = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g4 = lane >> 2, t4 = lane & 3;
  const int head0 = kvh * a.group + hchunk * 16;               // first query head of this block
  const int n_heads = min(16, a.group - hchunk * 16);          // valid rows

  // tiles of 64 keys aligned to absolute positions; this split's share of them
  const int tile_lo = lo / kDecTile, tile_hi = (ctx + kDecTile - 1) / kDecTile;
  const int per_split = (tile_hi - tile_lo + n_splits - 1) / n_splits;
  const int tile_begin = tile_lo + split * per_split;
  const int tile_end = min(tile_hi, tile_begin + per_split);
  const int n_tiles = max(0, tile_end - tile_begin);

  // a split beyond the cached head of the table copies its own slice (or, if that is too long, reads the table
  // in global memory)
  int table_off = 0;
  {
    const int blk0 = (tile_begin * kDecTile) >> a.kv.block_shift;
    const int blk1 = n_tiles > 0 ? min(a.max_blocks, ((min(ctx, tile_end * kDecTile) - 1) >> a.kv.block_shift) + 1) : 0;
    __syncthreads();
    if (blk1 <= n_head) {
      table = s_table;
    } else if (blk1 - blk0 <= kTableCache) {
      for (int i = threadIdx.x; i < blk1 - blk0; i += kDecThreads) s_table[i] = table[blk0 + i];
      __syncthreads();
      table = s_table;
      table_off = blk0;
    }
  }

  const uint32_t smem_base = smem_u32(smem);
  // first stages: tiles that end before the new token are requested now, the others after the wait
  const int safe_end = (ctx - 1) / kDecTile;                  // tiles below this index hold only older keys
  for (int s = 0; s < S - 1; ++s)
    if (s < n_tiles && tile_begin + s < safe_end)
      load_stage<HD, kDecTile, kDecThreads>(smem_base + s * DSt::kBytes, a.kv, table, kvh, (tile_begin + s) * kDecTile, lo, ctx, table_off);
  pdl_wait();
  for (int s = 0; s < S - 1; ++s) {
    if (s < n_tiles && tile_begin + s >= safe_end)
      load_stage<HD, kDecTile, kDecThreads>(smem_base + s * DSt::kBytes, a.kv, table, kvh, (tile_begin + s) * kDecTile, lo, ctx, table_off);
    cp_async_commit();
  }

  // q fragments: rows = heads (zero beyond n_heads), all k-steps
  uint32_t qf[kKSteps][4];
  {
    const bf16* qb = a.q + (size_t)token * a.q_stride + (size_t)head0 * HD;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = g4 + (r & 1) * 8, col = ks * 16 + t4 * 2 + (r >> 1) * 8;
        qf[ks][r] = row < n_heads ? *reinterpret_cast<const uint32_t*>(qb + (size_t)row * HD + col) : 0u;
      }
    }
  }

  RowState st{{-INFINITY, -INFINITY}, {0.f, 0.f}};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const float sl2 = a.scale * kLog2e;

  for (int i = 0; i < n_tiles; ++i) {
    cp_async_wait<S - 2>();
    __syncthreads();
    {
      const int nxt = i + S - 1;
      if (nxt < n_tiles)
        load_stage<HD, kDecTile, kDecThreads>(smem_base + (nxt % S) * DSt::kBytes, a.kv, table, kvh, (tile_begin + nxt) * kDecTile, lo, ctx, table_off);
      cp_async_commit();
    }
    const uint32_t kbase = smem_base + (i % S) * DSt::kBytes;       // this warp's rows are warp * 16 ..
    const uint32_t vbase = kbase + kDecTile * DSt::kRowBytes;
    const int key0 = (tile_begin + i) * kDecTile + warp * 16;   // first key of this warp's 16
    if (key0 >= ctx || key0 + 16 <= lo) continue;                // nothing valid (uniform over the warp)

    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      uint32_t b[4];
      const int mi = lane >> 3, r = lane & 7;
      ldmatrix_x4(b, kbase + DSt::off(warp * 16 + (mi >> 1) * 8 + r, ks * 2 + (mi & 1)));
      mma_16816(s[0], qf[ks], b[0], b[1]);
      mma_16816(s[1], qf[ks], b[2], b[3]);
    }
    // mask, running max, exponentials
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + j * 8 + t4 * 2 + (e & 1);
        const float v = (key >= lo && key < ctx) ? s[j][e] * sl2 : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(st.m[h], mx[h]);      // finite: at least one key of the 16 is valid
      alpha[h] = exp2f(st.m[h] - m_new);
      st.m[h] = m_new;
      st.l[h] *= alpha[h];
    }
    uint32_t pf[4];
    {
      float p[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[j][e] = exp2f(s[j][e] - st.m[e >> 1]);
          st.l[e >> 1] += p[j][e];
        }
      pf[0] = pack_bf16(p[0][0], p[0][1]);
      pf[1] = pack_bf16(p[0][2], p[0][3]);
      pf[2] = pack_bf16(p[1][0], p[1][1]);
      pf[3] = pack_bf16(p[1][2], p[1][3]);
    }
#pragma unroll
    for (int n2 = 0; n2 < kKSteps; ++n2) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        o[2 * n2 + h][0] *= alpha[0]; o[2 * n2 + h][1] *= alpha[0];
        o[2 * n2 + h][2] *= alpha[1]; o[2 * n2 + h][3] *= alpha[1];
      }
      uint32_t b[4];
      const int mi = lane >> 3, r = lane & 7;
      ldmatrix_x4_trans(b, vbase + DSt::off(warp * 16 + (mi & 1) * 8 + r, n2 * 2 + (mi >> 1)));
      mma_16816(o[2 * n2], pf, b[0], b[1]);
      mma_16816(o[2 * n2 + 1], pf, b[2], b[3]);
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  if (a.cluster) cluster_sync_all();        // the stages of every block of the cluster are free: split 0's will hold all parts

  // merge the warps through shared memory (the stages are free now)
  // (sized by the heads a block really holds, R = min(16, group): 4 for a group of 4, so that the region is a few
  // KB and the stages alone decide how many blocks an SM takes)
  constexpr int kOS = HD + 8;                                   // padded row: rows fall into different banks
  const int R = a.rows;
  float* sm_o = reinterpret_cast<float*>(smem);                 // [warps][R rows][kOS]
  float* sm_m = sm_o + kDecWarps * R * kOS;                     // [warps][16]
  float* sm_l = sm_m + kDecWarps * 16;                          // [warps][16]
  const int kPS = R * HD + 16;                                  // one split's part: R rows of HD values, 16 log-sum-exp
  float* sm_part = sm_l + kDecWarps * 16;                       // [splits][kPS], used in block 0 of a cluster
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
    if (t4 == 0) {
      sm_m[warp * 16 + g4 + h * 8] = st.m[h];
      sm_l[warp * 16 + g4 + h * 8] = st.l[h];
    }
  }
  // only the rows of heads that exist are written (4 of the 16 for a group of 4)
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    float* row0 = sm_o + (warp * R + g4) * kOS + n * 8 + t4 * 2;
    if (g4 < n_heads) *reinterpret_cast<float2*>(row0) = make_float2(o[n][0], o[n][1]);
    if (g4 + 8 < n_heads) *reinterpret_cast<float2*>(row0 + 8 * kOS) = make_float2(o[n][2], o[n][3]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_heads * HD; idx += kDecThreads) {
    const int row = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sm_m[w * 16 + row]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = sm_m[w * 16 + row];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += sm_l[w * 16 + row] * f;
      acc += sm_o[(w * R + row) * kOS + d] * f;
    }
    const int head = head0 + row;
    if (n_splits == 1) {
      a.out[(size_t)token * a.out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(acc / L);
    } else if (a.cluster) {
      st_cluster_f32(sm_part + split * kPS + row * HD + d, 0, L > 0.f ? acc / L : 0.f);
      if (d == 0) st_cluster_f32(sm_part + split * kPS + R * HD + row, 0, L > 0.f ? M + log2f(L) : -INFINITY);
    } else {
      const size_t pi = (size_t)splits_before * a.n_q_heads + (size_t)head * n_splits + split;
      a.part_o[pi * HD + d] = L > 0.f ? acc / L : 0.f;
      if (d == 0) a.part_lse[pi] = L > 0.f ? M + log2f(L) : -INFINITY;   // base-2 log-sum-exp
    }
  }
  if (n_splits == 1) return;
  if (a.cluster) {
    // all parts are in the shared memory of split 0, which adds them up in the order of the splits
    cluster_sync_all();
    if (split != 0) return;
    for (int idx = threadIdx.x; idx < n_heads * HD; idx += kDecThreads) {
      const int row = idx / HD, d = idx % HD;
      float M = -INFINITY;
      for (int s = 0; s < n_splits; ++s) M = fmaxf(M, sm_part[s * kPS + R * HD + row]);
      float acc = 0.f, L = 0.f;
      for (int s = 0; s < n_splits; ++s) {
        const float lse = sm_part[s * kPS + R * HD + row];
        const float f = lse == -INFINITY ? 0.f : exp2f(lse - M);
        L += f;
        acc += sm_part[s * kPS + row * HD + d] * f;
      }
      a.out[(size_t)token * a.out_stride + (size_t)(head0 + row) * HD + d] = __float2bfloat16_rn(acc / L);
    }
    return;
  }

  // The split that delivers last adds the splits up, always in the order of the splits:
  // out = sum_s part_o[s] 2^(lse_s - max) / sum_s 2^(lse_s - max).
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned* cnt = a.counters + (size_t)seq * gridDim.y + blockIdx.y;
    const unsigned before = atomicAdd(cnt, 1u);
    s_is_last = before == (unsigned)n_splits - 1;
    if (s_is_last) *cnt = 0;                 // every split has counted: the counter is left as it was found
  }
  __syncthreads();
  if (!s_is_last) return;
  __threadfence();
  const size_t base0 = (size_t)splits_before * a.n_q_heads + (size_t)head0 * n_splits;   // the block's heads are consecutive
  const int n_w = n_heads * n_splits;
  float* s_w = reinterpret_cast<float*>(smem);                                   // the stages are free
  if (n_w <= kMergeWeights) {
    // weights of all splits first (log-sum-exp values arrive together, not one after the other), then the sums
    for (int i = threadIdx.x; i < n_w; i += kDecThreads) s_w[i] = __ldcg(a.part_lse + base0 + i);
    __syncthreads();
    for (int row = warp; row < n_heads; row += kDecWarps) {
      float* w = s_w + row * n_splits;
      float M = -INFINITY;
      for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, w[s]);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
      float L = 0.f;
      for (int s = lane; s < n_splits; s += 32) {
        const float f = w[s] == -INFINITY ? 0.f : exp2f(w[s] - M);
        w[s] = f;
        L += f;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
      const float inv = 1.0f / L;
      for (int s = lane; s < n_splits; s += 32) w[s] *= inv;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_heads * HD; idx += kDecThreads) {
      const int row = idx / HD, d = idx % HD;
      const float* po = a.part_o + (base0 + (size_t)row * n_splits) * HD + d;
      const float* w = s_w + row * n_splits;
      float acc = 0.f;
      int s = 0;
      for (; s + 8 <= n_splits; s += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldcg(po + (size_t)(s + u) * HD);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc += v[u] * w[s + u];
      }
      for (; s < n_splits; ++s) acc += __ldcg(po + (size_t)s * HD) * w[s];
      a.out[(size_t)token * a.out_stride + (size_t)(head0 + row) * HD + d] = __float2bfloat16_rn(acc);
    }
    return;
  }
  for (int idx = threadIdx.x; idx < n_heads * HD; idx += kDecThreads) {
    const int row = idx / HD, d = idx % HD;
    const size_t base = base0 + (size_t)row * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, __ldcg(a.part_lse + base + s));
    float acc = 0.f, L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float lse = __ldcg(a.part_lse + base + s);
      const float f = lse == -INFINITY ? 0.f : exp2f(lse - M);
      L += f;
      acc += __ldcg(a.part_o + (base + s) * HD + d) * f;
    }
    a.out[(size_t)token * a.out_stride + (size_t)(head0 + row) * HD + d] = __float2bfloat16_rn(acc / L);
  }
}

// ---- splits per request ------------------------------------------------------------------------------------
// The list of work items of a decode launch whose requests differ much in length: request i gets
// s_i = round(keys_i / T) splits (1..kMaxItemSplits), with T the share of keys that a block would get if all keys
// were dealt evenly to the `slots` blocks that the device holds at a time (a multiple of 64 keys, at least 128).
// One warp: the requests are few.  items[k] for k >= sum of s_i is padding.
constexpr int kMaxItemSplits = 64;
struct ItemArgs {
  const int* ctx_len; const int* seq_ids; int n_served; int window;
  int blocks_per_split, slots, capacity;
  int4* items;
};
__global__ void __launch_bounds__(32) decode_items_kernel(ItemArgs a) {
  const int lane = threadIdx.x;
  auto keys_of = [&](int i) {
    const int seq = a.seq_ids ? a.seq_ids[i] : i;
    const int ctx = a.ctx_len[seq];
    return max(1, a.window > 0 ? min(ctx, a.window) : ctx);
  };
  auto warp_sum = [&](long long v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
  };
  long long total = 0;
  for (int i = lane; i < a.n_served; i += 32) total += keys_of(i);
  total = warp_sum(total);
  // A block's share if the keys were dealt evenly to the blocks that run at a time; a request is cut into pieces of
  // about that many keys (rounded to the nearest count, so a piece has at most 1.5 shares).  The pieces of all
  // requests are then at most slots / blocks_per_split + n_served / 2: short requests' blocks are over quickly, so
  // that the launch may hold more blocks than run at a time as long as none is long.
  const long long share = (total * a.blocks_per_split + a.slots - 1) / a.slots;
  const int Ti = (int)min(1ll << 30, max(128ll, (share + 63) / 64 * 64));
  auto splits_of = [&](int keys) { return max(1, min(kMaxItemSplits, (keys + Ti / 2) / Ti)); };
  int before = 0;                                        // splits of the requests before this pass
  for (int base = 0; base < a.n_served; base += 32) {
    const int i = base + lane;
    const int s_i = i < a.n_served ? splits_of(keys_of(i)) : 0;
    int incl = s_i;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    const int mine = before + incl - s_i;
    if (i < a.n_served) {
      const int seq = a.seq_ids ? a.seq_ids[i] : i;
      for (int j = 0; j < s_i; ++j)
        if (mine + j < a.capacity) a.items[mine + j] = make_int4(seq, j, s_i, mine);
    }
    before += __shfl_sync(0xffffffffu, incl, 31);
  }
  for (int k = before + lane; k < a.capacity; k += 32) a.items[k] = make_int4(-1, 0, 0, 0);
}

}  // namespace fa
}  // namespace lmsf

#include "attention_mma_prefill.cuh"

LMSF_API int lmsf_attention_mma_head_dim() { return LMSF_HEAD_DIM; }

// LMSF_DECODE_CLUSTER=0 in the environment sends every split count through global memory.
static int cluster_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LMSF_DECODE_CLUSTER");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v;
}

static int decode_rows(int group) { return group < 16 ? (group < 1 ? 1 : group) : 16; }

constexpr int kDeepStages = lmsf::fa::kStages + 1;      // the ring of the variant for few blocks

static int decode_smem_bytes(int group, int warps, int stages = lmsf::fa::kStages) {
  using namespace lmsf::fa;
  const int R = decode_rows(group);
  const int smem_stages = stages * (warps == 2 ? Stage<HD, 32>::kBytes : Stage<HD, 64>::kBytes);
  const int smem_merge = (warps * R * (HD + 8) + 2 * warps * 16) * (int)sizeof(float);
  const int smem_weights = kMergeWeights * (int)sizeof(float);     // weights of the splits when they are added up
  const int smem_cluster = smem_merge + kMaxClusterSplits * (R * HD + 16) * (int)sizeof(float);   // + the parts of a cluster
  int m = smem_stages > smem_merge ? smem_stages : smem_merge;
  if (smem_cluster > m) m = smem_cluster;
  return m > smem_weights ? m : smem_weights;
}

// Clusters of `cluster_size` blocks of the decode kernel (for query heads in groups of `group`) that the device holds
// at a time (0 on error): the splits of
// a request and kv head form a cluster, and a launch with more clusters than this runs in two waves.
// The decode kernel of a width is allowed as much dynamic shared memory as the largest request so far: the attribute is
// only ever raised (a query for a small group of heads must not lower what a launch for a large group was given).
typedef void (*DecodeKernel)(lmsf::fa::DecodeArgs);
static DecodeKernel decode_variant(int warps, bool deep) {
  using namespace lmsf::fa;
  if (warps == 2) return decode_kernel<2>;
  return deep ? (DecodeKernel)decode_kernel<4, kDeepStages> : (DecodeKernel)decode_kernel<4>;
}

static cudaError_t decode_allow_smem(int warps, int smem, bool deep = false) {
  static int allowed[3] = {0, 0, 0};
  const int v = warps == 2 ? 0 : (deep ? 2 : 1);
  if (smem <= allowed[v]) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(decode_variant(warps, deep), cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess) allowed[v] = smem;
  return e;
}

static int decode_max_clusters(int cluster_size, int group, int warps, bool deep) {
  using namespace lmsf::fa;
  if (cluster_size < 1 || cluster_size > kMaxClusterSplits || (warps != 2 && warps != 4)) return 0;
  const int smem = decode_smem_bytes(group, warps, deep ? kDeepStages : kStages);
  DecodeKernel kernel = decode_variant(warps, deep);
  if (decode_allow_smem(warps, smem, deep) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)cluster_size, 1024, 1);
  cfg.blockDim = dim3(32 * warps);
  cfg.dynamicSmemBytes = (size_t)smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster_size;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) return 0;
  return n;
}

LMSF_API int lmsf_attention_decode_max_clusters(int cluster_size, int group, int warps) {
  return decode_max_clusters(cluster_size, group, warps, false);
}

// Bytes of keys and values that a decode block of `warps` warps keeps in flight: what sets the rate at which one
// block streams (0 for a width that does not exist).
LMSF_API int lmsf_attention_decode_stream_bytes(int warps) {
  using namespace lmsf::fa;
  if (warps == 4) return (kStages - 1) * Stage<HD, 64>::kBytes;
  if (warps == 2) return (kStages - 1) * Stage<HD, 32>::kBytes;
  return 0;
}

// The width of the blocks when the caller names none: wide blocks (4 warps) while all (request, group of heads) pairs
// fit the device at once, narrow ones (2 warps) beyond that if more of them fit.  (The engine chooses the width together
// with the number of splits, kernels.decode_plan.)  LMSF_DECODE_WARPS=2 or 4 in the environment fixes the width of
// every launch, whatever the caller says.
static int forced_block_warps() {
  const char* e = getenv("LMSF_DECODE_WARPS");      // read at every call: tests switch it
  return (e && (e[0] == '2' || e[0] == '4') && e[1] == 0) ? e[0] - '0' : 0;
}
LMSF_API int lmsf_attention_decode_block_warps(int n_pairs, int group) {
  if (const int f = forced_block_warps()) return f;
  if (LMSF_HEAD_DIM <= 64) return 4;         // stages of 16 KB and less: four wide blocks fit already
  static int slots[17][2];                   // by rows of a block: blocks of each width that the device holds; 0: not asked yet
  const int R = decode_rows(group);
  if (slots[R][0] == 0) {
    slots[R][1] = lmsf_attention_decode_max_clusters(1, group, 2);
    slots[R][0] = lmsf_attention_decode_max_clusters(1, group, 4);
    if (slots[R][0] <= 0) slots[R][0] = 1 << 30;    // the occupancy cannot be read: stay wide
  }
  return (n_pairs > slots[R][0] && slots[R][1] > slots[R][0]) ? 2 : 4;
}

// Bytes of scratch that lmsf_attention_decode needs for the given sizes (0 when n_splits == 1): counters of
// the splits that have delivered (one per request and group of heads, always the first kDecodeCounterBytes,
// whatever the sizes of a call, so that calls of different sizes can share one buffer), then partial results.
constexpr long long kDecodeCounterSlots = 65536;
constexpr long long kDecodeCounterBytes = kDecodeCounterSlots * (long long)sizeof(unsigned);
LMSF_API long long lmsf_attention_decode_scratch_bytes(int n_seqs_total, int n_q_heads, int n_splits) {
  if (n_splits <= 1) return 0;
  return kDecodeCounterBytes + (long long)n_seqs_total * n_q_heads * n_splits * (lmsf::fa::HD + 1) * (long long)sizeof(float);
}

// One query token per served request.  seq_ids (may be null) lists the n_served requests among the
// n_seqs_total rows of block_table / cu_q / ctx_len.  scratch: lmsf_attention_decode_scratch_bytes(), zero when
// it is first used; a launch that completes leaves its counters zero again, so the same memory serves every call.
static int decode_launch(lmsf::fa::DecodeArgs& a, int gy, int grid_x, int grid_z, int warps, cudaStream_t s);

// block_warps: 4 or 2, the width of the blocks; 0: by the rule of lmsf_attention_decode_block_warps.
LMSF_API int lmsf_attention_decode_width(const void* q, long long q_stride, void* out, long long out_stride,
                                         const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                         const int* block_table, int max_blocks, const int* seq_ids, int n_served,
                                         int n_seqs_total, const int* cu_q, const int* ctx_len, float scale, int window,
                                         int n_q_heads, int head_dim, int n_splits, int block_warps, void* scratch,
                                         void* stream) {
  using namespace lmsf;
  using namespace lmsf::fa;
  if (n_served <= 0) return 0;
  if (head_dim != HD) LMSF_REFUSE("attention_decode: built for head_dim=%d, called with %d", HD, head_dim);
  if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    LMSF_REFUSE("attention_decode: %d query heads cannot be grouped over %d kv heads", n_q_heads, n_kv_heads);
  if (n_splits < 1 || n_splits > 65535) LMSF_REFUSE("attention_decode: n_splits=%d", n_splits);
  if (n_splits > 1 && !scratch) LMSF_REFUSE("attention_decode: %d splits need scratch memory", n_splits);
  if (!seq_ids && n_served > n_seqs_total)
    LMSF_REFUSE("attention_decode: n_served=%d exceeds n_seqs_total=%d, the rows the scratch was sized for", n_served,
                n_seqs_total);
  if (block_size <= 0 || max_blocks <= 0) LMSF_REFUSE("attention_decode: bad block table geometry");
  const int group = n_q_heads / n_kv_heads;
  const long long gy = (long long)n_kv_heads * ((group + 15) / 16);
  if (gy > 65535 || n_served > 65535) LMSF_REFUSE("attention_decode: too many heads or requests for one launch");
  DecodeArgs a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  if (n_splits > 1 && (long long)n_seqs_total * gy > kDecodeCounterSlots)
    LMSF_REFUSE("attention_decode: %d requests x %lld head groups exceed the %lld split counters; use n_splits=1",
                n_seqs_total, gy, kDecodeCounterSlots);
  a.counters = (unsigned*)scratch;
  a.part_o = scratch ? reinterpret_cast<float*>((unsigned char*)scratch + kDecodeCounterBytes) : nullptr;
  a.part_lse = a.part_o ? a.part_o + (size_t)n_seqs_total * n_q_heads * n_splits * HD : nullptr;
  if (!make_paged_kv(a.kv, cache, page_stride, block_size, n_kv_heads))
    LMSF_REFUSE("attention: block_size=%d must be a power of two", block_size);
  a.block_table = block_table; a.max_blocks = max_blocks; a.seq_ids = seq_ids; a.cu_q = cu_q; a.ctx_len = ctx_len;
  a.scale = scale; a.window = window; a.n_q_heads = n_q_heads; a.group = group; a.n_splits = n_splits;
  a.rows = decode_rows(group);
  if (block_warps != 0 && block_warps != 2 && block_warps != 4)
    LMSF_REFUSE("attention_decode: blocks have 2 or 4 warps, not %d", block_warps);
  int warps = forced_block_warps();
  if (!warps) warps = block_warps ? block_warps : lmsf_attention_decode_block_warps((int)(n_served * gy), group);
  a.items = nullptr;
  a.cluster = n_splits >= 2 && n_splits <= kMaxClusterSplits && cluster_enabled();
  return decode_launch(a, (int)gy, n_splits, n_served, warps, (cudaStream_t)stream);
}

// The launch itself: grid (grid_x, gy, grid_z) of blocks of `warps` warps; a.cluster: the grid_x blocks of a row form a
// thread-block cluster.
static int decode_launch(lmsf::fa::DecodeArgs& a, int gy, int grid_x, int grid_z, int warps, cudaStream_t s) {
  using namespace lmsf;
  using namespace lmsf::fa;
  // A launch of wide blocks that all run at once with one more stage each (one or two requests of Llama-3-8B's 8 kv
  // heads in 8 splits: 64 or 128 blocks on 148 SMs) gets that stage: more keys are asked for before the dependency
  // wait and more bytes are in flight (a decode step of one request 2.98 -> 2.90 ms, of two 2.98 -> 2.93).
  bool deep = false;
  if (warps == 4 && !a.items) {
    static int fit[kMaxClusterSplits + 1][17];             // by cluster size and rows of a block; 0: not asked yet
    const int cs = a.cluster ? grid_x : 1, R = decode_rows(a.group);
    if (fit[cs][R] == 0) {
      const int n = decode_max_clusters(cs, a.group, 4, true);
      fit[cs][R] = n > 0 ? n : -1;
    }
    const long long clusters = (long long)gy * grid_z * (a.cluster ? 1 : grid_x);
    deep = fit[cs][R] > 0 && clusters <= fit[cs][R];
  }
  DecodeKernel kernel = decode_variant(warps, deep);
  const int smem = decode_smem_bytes(a.group, warps, deep ? kDeepStages : kStages);
  if (const cudaError_t e = decode_allow_smem(warps, smem, deep)) return (int)e;
  if (!a.cluster) return launch_pdl(kernel, dim3(grid_x, (unsigned)gy, grid_z), dim3(32 * warps), smem, s, a);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid_x, (unsigned)gy, grid_z);
  cfg.blockDim = dim3(32 * warps);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = grid_x;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, kernel, a);
}

// ---- a launch with splits per request -----------------------------------------------------------------------
// lmsf_attention_decode_build_items writes the list (capacity entries of 4 ints) from the requests' context lengths;
// lmsf_attention_decode_items runs the attention over it.  slots: blocks of the chosen width that the device holds at
// a time (lmsf_attention_decode_max_clusters(1, group, warps)); capacity >= n_served.  Scratch of
// lmsf_attention_decode_items_scratch_bytes(capacity, n_q_heads), zero when first used.
LMSF_API int lmsf_attention_decode_build_items(const int* ctx_len, const int* seq_ids, int n_served, int window,
                                               int n_q_heads, int n_kv_heads, int slots, int capacity, void* items,
                                               void* stream) {
  using namespace lmsf::fa;
  if (n_served <= 0) return 0;
  if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    LMSF_REFUSE("attention_decode_build_items: %d query heads cannot be grouped over %d kv heads", n_q_heads, n_kv_heads);
  if (capacity < n_served || slots <= 0 || !items || ((uintptr_t)items & 15))
    LMSF_REFUSE("attention_decode_build_items: the list needs room for one entry per request (%d), 16-byte aligned", n_served);
  const int group = n_q_heads / n_kv_heads;
  ItemArgs a{ctx_len, seq_ids, n_served, window, n_kv_heads * ((group + 15) / 16), slots, capacity, (int4*)items};
  decode_items_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

LMSF_API long long lmsf_attention_decode_items_scratch_bytes(int capacity, int n_q_heads) {
  return kDecodeCounterBytes + (long long)capacity * n_q_heads * (lmsf::fa::HD + 1) * (long long)sizeof(float);
}

LMSF_API int lmsf_attention_decode_items(const void* q, long long q_stride, void* out, long long out_stride,
                                         const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                         const int* block_table, int max_blocks, const void* items, int capacity,
                                         int n_seqs_total, const int* cu_q, const int* ctx_len, float scale, int window,
                                         int n_q_heads, int head_dim, int block_warps, void* scratch, void* stream) {
  using namespace lmsf;
  using namespace lmsf::fa;
  if (capacity <= 0) return 0;
  if (head_dim != HD) LMSF_REFUSE("attention_decode: built for head_dim=%d, called with %d", HD, head_dim);
  if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    LMSF_REFUSE("attention_decode: %d query heads cannot be grouped over %d kv heads", n_q_heads, n_kv_heads);
  if (!items || !scratch) LMSF_REFUSE("attention_decode_items: the list of work items and scratch memory are needed");
  if (block_size <= 0 || max_blocks <= 0) LMSF_REFUSE("attention_decode: bad block table geometry");
  if (block_warps != 2 && block_warps != 4) LMSF_REFUSE("attention_decode_items: blocks have 2 or 4 warps, not %d", block_warps);
  const int group = n_q_heads / n_kv_heads;
  const long long gy = (long long)n_kv_heads * ((group + 15) / 16);
  if (gy > 65535) LMSF_REFUSE("attention_decode: too many heads for one launch");
  if ((long long)n_seqs_total * gy > kDecodeCounterSlots)
    LMSF_REFUSE("attention_decode_items: %d requests x %lld head groups exceed the %lld split counters", n_seqs_total, gy,
                kDecodeCounterSlots);
  DecodeArgs a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  a.counters = (unsigned*)scratch;
  a.part_o = reinterpret_cast<float*>((unsigned char*)scratch + kDecodeCounterBytes);
  a.part_lse = a.part_o + (size_t)capacity * n_q_heads * HD;
  if (!make_paged_kv(a.kv, cache, page_stride, block_size, n_kv_heads))
    LMSF_REFUSE("attention: block_size=%d must be a power of two", block_size);
  a.block_table = block_table; a.max_blocks = max_blocks; a.seq_ids = nullptr; a.cu_q = cu_q; a.ctx_len = ctx_len;
  a.scale = scale; a.window = window; a.n_q_heads = n_q_heads; a.group = group; a.n_splits = 1;
  a.rows = decode_rows(group);
  a.items = (const int4*)items;
  a.cluster = 0;
  int warps = forced_block_warps();
  if (!warps) warps = block_warps;
  return decode_launch(a, (int)gy, capacity, 1, warps, (cudaStream_t)stream);
}

LMSF_API int lmsf_attention_decode(const void* q, long long q_stride, void* out, long long out_stride,
                                   const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                   const int* block_table, int max_blocks, const int* seq_ids, int n_served,
                                   int n_seqs_total, const int* cu_q, const int* ctx_len, float scale, int window,
                                   int n_q_heads, int head_dim, int n_splits, void* scratch, void* stream) {
  return lmsf_attention_decode_width(q, q_stride, out, out_stride, cache, page_stride, block_size, n_kv_heads, block_table,
                                     max_blocks, seq_ids, n_served, n_seqs_total, cu_q, ctx_len, scale, window, n_q_heads,
                                     head_dim, n_splits, 0, scratch, stream);
}

// ------------------------------------------------------------------------------------------------
// The variant that allocates nothing (see attention_decode_static.h).
#include "attention_decode_static.h"

#include <mutex>

namespace {
constexpr long long kStaticScratchBytes = 8ll << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device
std::mutex g_static_scratch_mutex;
}  // namespace

LMSF_API long long lmsf_attention_decode_static_capacity() { return kStaticScratchBytes; }

LMSF_API int lmsf_attention_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                                          const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                          const int* block_table, int max_blocks, const int* seq_ids, int n_served,
                                          int n_seqs_total, const int* cu_q, const int* ctx_len, float scale,
                                          int window, int n_q_heads, int head_dim, int n_splits, void* stream) {
  if (n_seqs_total <= 0 || n_q_heads <= 0 || n_splits < 1)
    LMSF_REFUSE("attention_decode_static: n_seqs_total=%d n_q_heads=%d n_splits=%d", n_seqs_total, n_q_heads, n_splits);
  const long long need = lmsf_attention_decode_scratch_bytes(n_seqs_total, n_q_heads, n_splits);
  if (need > kStaticScratchBytes)
    LMSF_REFUSE("attention_decode_static: %d requests x %d heads x %d splits need %lld bytes of scratch, the static "
                "array holds %lld; use fewer splits or lmsf_attention_decode with scratch of your own",
                n_seqs_total, n_q_heads, n_splits, need, kStaticScratchBytes);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) LMSF_REFUSE("attention_decode_static: device ordinal %d is not supported", dev);
  void* scratch = nullptr;
  {
    // In host code the array's name is only a handle: the address a kernel can use has to be asked for,
    // once per device, with that device current.
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess) return (int)e;
      g_static_scratch_ptr[dev] = p;
    }
    scratch = g_static_scratch_ptr[dev];
  }
  return lmsf_attention_decode(q, q_stride, out, out_stride, cache, page_stride, block_size, n_kv_heads, block_table,
                               max_blocks, seq_ids, n_served, n_seqs_total, cu_q, ctx_len, scale, window, n_q_heads,
                               head_dim, n_splits, need > 0 ? scratch : nullptr, stream);
}
