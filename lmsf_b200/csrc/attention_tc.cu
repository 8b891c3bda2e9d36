// Prefill attention on the 5th-generation tensor cores: tcgen05.mma with both products' accumulators in
// tensor memory.  bfloat16, head size 64 or 128 (-DLMSF_HEAD_DIM), any mix of prompt portions over the
// paged cache; same interface and results (up to rounding) as lmsf_attention_prefill of attention_mma.cu.
//
// Counterpart in the reference: the dense float32 prompt attention of
// core/src/model_executor/layers/attention.rs:106-159.
//
// One block of 128 threads serves 128 query tokens of one head.  Per tile of 64 keys:
//   1. k and v rows are gathered from their pages into shared memory with cp.async, in the 128-byte
//      swizzled layout that the tensor core reads (k: K-major, v: MN-major); the next tile's rows are
//      requested while this tile's scores are computed;
//   2. one thread issues S = Q K^T (M 128, N 64, K head size) into tensor memory and commits to an mbarrier;
//   3. every thread owns one query row: it reads its 64 scores with tcgen05.ld, masks, updates the running
//      maximum (the accumulator is rescaled only when the maximum grew by more than 2^8, which keeps the
//      sums exact and saves most read-modify-writes of tensor memory), exponentiates in float32 and writes
//      P as bfloat16 into the shared memory that held the k tile;
//   4. one thread issues O += P V (M 128, N head size, K 64) and commits.
// Two blocks share an SM (96 KB of shared memory and 256 columns of tensor memory each), so one block's
// softmax overlaps the other's products.  Every wait on an mbarrier is bounded: when it runs out the
// block raises *error_flag (code 3), frees its tensor memory and returns.
#include "attention_mma.cuh"

#ifndef LMSF_HEAD_DIM
#error "compile with -DLMSF_HEAD_DIM=64 or 128"
#endif

LMSF_DEFINE_LAST_ERROR(lmsf_attention_tc)

namespace lmsf {
namespace tc {

using namespace lmsf::fa;

#ifdef LMSF_TC_TIMING
// Development aid: thread 127 of every block adds the cycles it spent in each phase of the loop.
__device__ long long* g_timing = nullptr;
#define LMSF_T(i) do { if (tid == 127) { const long long now_ = clock64(); tacc[i] += now_ - tlast; tlast = now_; } } while (0)
#else
#define LMSF_T(i) do {} while (0)
#endif

constexpr int HD = LMSF_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "the tcgen05 attention kernel takes head sizes 64 and 128");
constexpr int BM = 128;                    // query rows per block
constexpr int BN = 64;                     // keys per tile
constexpr int kHB = HD / 64;               // 64-wide blocks of the head dimension
constexpr int kQBytes = kHB * BM * 128;
constexpr int kKBytes = kHB * BN * 128;    // one k (or v) tile
constexpr int kPBytes = BM * 128;          // P: 128 rows x 64 keys, written over the k tile once S is done
constexpr int kKSlot = kKBytes > kPBytes ? kKBytes : kPBytes;
constexpr int kStageBytes = kKSlot + kKBytes;   // k (later P), then v
constexpr int kSmemBytes = kQBytes + 2 * kStageBytes + 1024;   // + slack for the 1024-byte alignment
constexpr uint32_t kTmemCols = 256;        // S: columns [0, 64), O: columns [128, 128 + HD)
constexpr uint32_t kOCol = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units
constexpr int kWaitLimit = 1 << 22;

struct Args {
  const bf16* q; long long q_stride;
  bf16* out; long long out_stride;
  PagedKV kv;
  const int* block_table; int max_blocks;
  const int* tile_seq; const int* tile_q0;   // one entry per 128 query tokens
  const int* cu_q; const int* ctx_len;
  float scale; int window;
  int n_q_heads, group;
  int* error_flag;
};

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;      // descriptor version of sm_100
  d |= (uint64_t)2 << 61;      // 128-byte swizzle
  return d;
}
// kind::f16, bfloat16 operands, float32 accumulator, A K-major
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
  uint32_t done = 0;
  for (int it = 0; it < kWaitLimit && !done; ++it)
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(mbar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
               "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
               : "=r"(r[0]),"=r"(r[1]),"=r"(r[2]),"=r"(r[3]),"=r"(r[4]),"=r"(r[5]),"=r"(r[6]),"=r"(r[7]),"=r"(r[8]),"=r"(r[9]),
                 "=r"(r[10]),"=r"(r[11]),"=r"(r[12]),"=r"(r[13]),"=r"(r[14]),"=r"(r[15]),"=r"(r[16]),"=r"(r[17]),"=r"(r[18]),
                 "=r"(r[19]),"=r"(r[20]),"=r"(r[21]),"=r"(r[22]),"=r"(r[23]),"=r"(r[24]),"=r"(r[25]),"=r"(r[26]),"=r"(r[27]),
                 "=r"(r[28]),"=r"(r[29]),"=r"(r[30]),"=r"(r[31])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
               "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
               ::"r"(taddr), "r"(r[0]),"r"(r[1]),"r"(r[2]),"r"(r[3]),"r"(r[4]),"r"(r[5]),"r"(r[6]),"r"(r[7]),"r"(r[8]),"r"(r[9]),
                 "r"(r[10]),"r"(r[11]),"r"(r[12]),"r"(r[13]),"r"(r[14]),"r"(r[15]),"r"(r[16]),"r"(r[17]),"r"(r[18]),
                 "r"(r[19]),"r"(r[20]),"r"(r[21]),"r"(r[22]),"r"(r[23]),"r"(r[24]),"r"(r[25]),"r"(r[26]),"r"(r[27]),
                 "r"(r[28]),"r"(r[29]),"r"(r[30]),"r"(r[31]) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {      // 2^x, 0 for -inf
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// k and v of keys [key0, key0 + 64) of kv head kvh into a stage: [64-wide block of the head][key][128 bytes],
// 16-byte chunk c of a row at chunk c ^ (key & 7).  Keys outside [lo, hi) or without a page are zero-filled.
constexpr int kNoPrefetch = -2;    // `page_hint` of load_kv_tile: look the page up now

// The page that holds the first row this thread copies of tile [key0, key0 + 64), or -1.  With a block size of
// at least the rows a thread copies (and both powers of two) all of a thread's rows of a tile share that page.
__device__ __forceinline__ int tile_page(const PagedKV& kv, const int* __restrict__ table, int key0, int lo, int hi) {
  constexpr int kChunks = HD / 8;
  constexpr int kRowsPerThread = BN * kChunks / 128;
  const int key = key0 + (threadIdx.x / kChunks) * kRowsPerThread;
  // a row range that straddles lo or hi still lies in one page; rows outside [lo, hi) are zero-filled anyway
  const int probe = min(max(key, lo), hi - 1);
  if (probe < key || probe >= key + kRowsPerThread) return -1;
  return table[probe >> kv.block_shift];
}

__device__ __forceinline__ void load_kv_tile(uint32_t stage, const PagedKV& kv, const int* __restrict__ table, int kvh,
                                             int key0, int lo, int hi, int page_hint) {
  constexpr int kChunks = HD / 8;                       // 16-byte chunks per row
  constexpr int kRowsPerThread = BN * kChunks / 128;    // consecutive rows per thread
  const size_t v_off = (size_t)kv.n_kv_heads * kv.block_size * HD;
  const size_t head_off = (size_t)kvh * kv.block_size * HD;
  const int mask = kv.block_size - 1;
  const int c = threadIdx.x % kChunks, row0 = (threadIdx.x / kChunks) * kRowsPerThread;
  const uint32_t col = (c / 8) * (BN * 128);
  const bf16* page_ptr = nullptr;
  bool have_page = false;
  if (page_hint != kNoPrefetch) {
    page_ptr = page_hint >= 0 ? kv.cache + (size_t)page_hint * kv.page_stride + head_off + c * 8 : nullptr;
    have_page = true;
    if (key0 >= lo && key0 + BN <= hi && page_ptr != nullptr) {
      // the common case: every key of the tile is wanted and this thread's rows sit in one page, one after
      // the other: the addresses are the first one plus constants
      const bf16* src = page_ptr + (size_t)((key0 + row0) & mask) * HD;
      const uint32_t dst = stage + col + row0 * 128;                   // row0 is a multiple of 8 or kRowsPerThread <= 8
#pragma unroll
      for (int it = 0; it < kRowsPerThread; ++it) {
        const uint32_t d = dst + it * 128 + (((c & 7) ^ ((row0 + it) & 7)) << 4);
        cp_async_16(d, src + it * HD, 16);
        cp_async_16(d + kKSlot, src + v_off + it * HD, 16);
      }
      return;
    }
  }
#pragma unroll
  for (int it = 0; it < kRowsPerThread; ++it) {
    const int row = row0 + it, key = key0 + row, slot = key & mask;
    const bool in_range = key >= lo && key < hi;
    if (page_hint == kNoPrefetch) {
      if (slot == 0) have_page = false;
      if (in_range && !have_page) {
        const int page = table[key >> kv.block_shift];
        page_ptr = page >= 0 ? kv.cache + (size_t)page * kv.page_stride + head_off + c * 8 : nullptr;
        have_page = true;
      }
    }
    const bool ok = in_range && page_ptr != nullptr;
    const bf16* src = ok ? page_ptr + (size_t)slot * HD : kv.cache;
    const uint32_t dst = stage + col + row * 128 + (((c & 7) ^ (row & 7)) << 4);
    cp_async_16(dst, src, ok ? 16 : 0);
    cp_async_16(dst + kKSlot, ok ? src + v_off : src, ok ? 16 : 0);
  }
}

__global__ void __launch_bounds__(128) prefill_tc_kernel(Args a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t mbar_s_mem, mbar_o_mem;
  __shared__ uint32_t tmem_base_mem;
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;     // the swizzle pattern is a function of the address
  const uint32_t sQ = smem, sStage0 = smem + kQBytes;
  const uint32_t mbar_s = smem_u32(&mbar_s_mem), mbar_o = smem_u32(&mbar_o_mem);
  const int tid = threadIdx.x, warp = tid >> 5;

  // blocks start in the order (all heads of tile 0, all heads of tile 1, ...); the caller lists the tiles that
  // see the most keys first, so the longest blocks are not left for the end
  const int tile = blockIdx.y;
  const int seq = a.tile_seq[tile], q0 = a.tile_q0[tile];
  const int head = blockIdx.x, kvh = head / a.group;
  const int tok0 = a.cu_q[seq], n = a.cu_q[seq + 1] - tok0, ctx = a.ctx_len[seq];
  const int start = ctx - n;
  const int rows_valid = min(BM, n - q0);
  const int hi = start + q0 + rows_valid;                       // keys < hi are visible to the tile's last row
  const int lo = a.window > 0 ? max(0, start + q0 - a.window + 1) : 0;
  const int* table = a.block_table + (size_t)seq * a.max_blocks;
  const bool row_ok = tid < rows_valid;
  const int pos = start + q0 + min(tid, rows_valid - 1);         // this thread's query position
  const int row_lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_s));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_o));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_mem)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }

  const int tile_begin = lo / BN, tile_end = (hi + BN - 1) / BN;
  const int n_tiles = tile_end - tile_begin;

  // Q tile: [64-wide block][row][128 bytes], rows beyond the portion are zero
  {
    constexpr int kChunks = HD / 8;
#pragma unroll
    for (int it = 0; it < BM * kChunks / 128; ++it) {
      const int idx = tid + it * 128;
      const int row = idx / kChunks, c = idx % kChunks;
      const bool ok = row < rows_valid;
      const bf16* src = ok ? a.q + (size_t)(tok0 + q0 + row) * a.q_stride + (size_t)head * HD + c * 8 : a.q;
      cp_async_16(sQ + (c / 8) * (BM * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4), src, ok ? 16 : 0);
    }
  }
  load_kv_tile(sStage0, a.kv, table, kvh, tile_begin * BN, lo, hi, kNoPrefetch);
  cp_async_commit();
  // Page numbers are looked up one tile ahead of the copies that use them, so that the copies of the loop
  // never wait on the block table.
  constexpr int kRowsPerThread = BN * (HD / 8) / 128;
  const bool prefetch_pages = a.kv.block_size >= kRowsPerThread;
  int next_page = (prefetch_pages && n_tiles > 1) ? tile_page(a.kv, table, (tile_begin + 1) * BN, lo, hi) : kNoPrefetch;

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_mem;
  const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);      // this warp's 32 lanes

  float m_run = -INFINITY, l_run = 0.f;
  const float sl2 = a.scale * kLog2e;
  bool failed = false;

#ifdef LMSF_TC_TIMING
  long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long tlast = clock64();
#endif
  for (int j = 0; j < n_tiles; ++j) {
    LMSF_T(7);
    const uint32_t stage = sStage0 + (j & 1) * kStageBytes;
    const uint32_t sK = stage, sV = stage + kKSlot, sP = stage;    // P takes the k tile's place once S is done
    // (a) this tile (and, the first time, Q) has landed
    cp_async_wait<0>();
    fence_async_smem();
    tc_fence_before();
    if (__syncthreads_or(failed)) { failed = true; break; }
    LMSF_T(0);
    // (b) S = Q K^T; it runs behind the previous tile's O += P V on the tensor pipe
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = instr_desc(BM, BN, 0);
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const uint32_t off_a = (ks / 4) * (BM * 128) + (ks % 4) * 32, off_b = (ks / 4) * (BN * 128) + (ks % 4) * 32;
        umma(tmem, smem_desc(sQ + off_a, 16, 1024), smem_desc(sK + off_b, 16, 1024), idesc, ks > 0);
      }
      umma_commit(mbar_s);
    }
    // (c) the product before this one has finished: O may be touched, the other stage may be overwritten
    if (j > 0 && !mbar_wait(mbar_o, (uint32_t)((j - 1) & 1))) failed = true;
    LMSF_T(1);
    // (d) next tile's loads, while S is being computed
    if (j + 1 < n_tiles)
      load_kv_tile(sStage0 + ((j + 1) & 1) * kStageBytes, a.kv, table, kvh, (tile_begin + j + 1) * BN, lo, hi, next_page);
    cp_async_commit();
    if (prefetch_pages && j + 2 < n_tiles) next_page = tile_page(a.kv, table, (tile_begin + j + 2) * BN, lo, hi);
    LMSF_T(2);
    // (e) softmax of this thread's row
    if (!mbar_wait(mbar_s, (uint32_t)(j & 1))) failed = true;
    tc_fence_after();
    LMSF_T(3);
    float s[BN];
    {
      uint32_t r[32];
      tmem_ld32(t_row, r);
#pragma unroll
      for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(r[i]);
      tmem_ld32(t_row + 32, r);
#pragma unroll
      for (int i = 0; i < 32; ++i) s[32 + i] = __uint_as_float(r[i]);
    }
    LMSF_T(4);
    const int key0 = (tile_begin + j) * BN;
    // Only tiles that reach past some row's position (the diagonal) or before its window need the mask;
    // the test is the same for the whole block.
    const bool need_mask = key0 + BN - 1 > start + q0 || (a.window > 0 && key0 < start + q0 + rows_valid - a.window);
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < BN; ++i) {
        const int key = key0 + i;
        if (key > pos || key < row_lo) s[i] = -INFINITY;
      }
    }
    float mx = s[0];
#pragma unroll
    for (int i = 1; i < BN; ++i) mx = fmaxf(mx, s[i]);
    mx *= sl2;                                                // scores enter the exponent as s * scale * log2(e)
    float alpha = 1.f;
    const bool grow = mx > m_run + kRescaleThreshold;         // also true for the first keys a row sees
    if (grow) {
      alpha = exp2f(m_run - mx);                              // 0 when m_run is -inf
      m_run = mx;
      l_run *= alpha;
    }
    if (j > 0 && __any_sync(0xffffffffu, grow)) {             // rescale this warp's rows of O
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(t_row + kOCol + c0, r);
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st32(t_row + kOCol + c0, r);
      }
    }
    const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
    {
      const int row = tid;
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int c = 0; c < BN / 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2_approx(fmaf(s[c * 8 + 2 * e], sl2, neg_m)), p1 = ex2_approx(fmaf(s[c * 8 + 2 * e + 1], sl2, neg_m));
          l0 += p0;
          l1 += p1;
          w[e] = pack_bf16(p0, p1);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sP + row * 128 + ((c ^ (row & 7)) << 4)),
                     "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
      }
      l_run += l0 + l1;
    }
    LMSF_T(5);
    fence_async_smem();
    tc_fence_before();
    if (__syncthreads_or(failed)) { failed = true; break; }
    LMSF_T(6);
    // (f) O += P V
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = instr_desc(BM, HD, 1);
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks)
        umma(tmem + kOCol, smem_desc(sP + ks * 32, 16, 1024), smem_desc(sV + ks * 16 * 128, BN * 128, 1024), idesc,
             (j > 0 || ks > 0) ? 1u : 0u);
      umma_commit(mbar_o);
    }
  }
  cp_async_wait<0>();
#ifdef LMSF_TC_TIMING
  if (tid == 127 && g_timing) {
    long long* t = g_timing + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * 9;
    for (int i = 0; i < 8; ++i) t[i] = tacc[i];
    t[8] = n_tiles;
  }
#endif

  if (!failed && n_tiles > 0 && !mbar_wait(mbar_o, (uint32_t)((n_tiles - 1) & 1))) failed = true;
  failed = __syncthreads_or(failed);
  tc_fence_after();
  if (!failed && n_tiles > 0) {
    const float inv = 1.0f / l_run;
    bf16* dst = a.out + (size_t)(tok0 + q0 + tid) * a.out_stride + (size_t)head * HD;
#pragma unroll
    for (int c0 = 0; c0 < HD; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(t_row + kOCol + c0, r);                       // every lane of the warp takes part
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + c0 + i) = v;
        }
      }
    }
  }
  if (failed && tid == 0 && a.error_flag) atomicExch(a.error_flag, 3);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}

}  // namespace tc
}  // namespace lmsf

LMSF_API int lmsf_attention_tc_head_dim() { return LMSF_HEAD_DIM; }

#ifdef LMSF_TC_TIMING
LMSF_API int lmsf_attention_tc_set_timing(long long* buf) {
  return (int)cudaMemcpyToSymbol(lmsf::tc::g_timing, &buf, sizeof(buf));
}
#endif

// tile_seq / tile_q0: one entry per 128 query tokens of each portion, best listed with the tiles that see the
// most keys first.  q and out rows must be 16-byte aligned.
LMSF_API int lmsf_attention_prefill_tc(const void* q, long long q_stride, void* out, long long out_stride,
                                       const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                       const int* block_table, int max_blocks, const int* tile_seq, const int* tile_q0,
                                       int n_tiles, const int* cu_q, const int* ctx_len, float scale, int window,
                                       int n_q_heads, int head_dim, int* error_flag, void* stream) {
  using namespace lmsf;
  using namespace lmsf::tc;
  if (n_tiles <= 0) return 0;
  if (head_dim != HD) LMSF_REFUSE("attention_prefill_tc: built for head_dim=%d, called with %d", HD, head_dim);
  if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    LMSF_REFUSE("attention_prefill_tc: %d query heads cannot be grouped over %d kv heads", n_q_heads, n_kv_heads);
  if (n_tiles > 65535) LMSF_REFUSE("attention_prefill_tc: more than 65535 query tiles in one launch");
  if (max_blocks <= 0) LMSF_REFUSE("attention_prefill_tc: bad block table geometry");
  if (q_stride % 8 || out_stride % 8 || ((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) % 16 || page_stride % 8)
    LMSF_REFUSE("attention_prefill_tc: q, out and the cache must be 16-byte aligned with row strides that are multiples of 8");
  Args a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  if (!make_paged_kv(a.kv, cache, page_stride, block_size, n_kv_heads))
    LMSF_REFUSE("attention_prefill_tc: block_size=%d must be a power of two", block_size);
  a.block_table = block_table; a.max_blocks = max_blocks; a.tile_seq = tile_seq; a.tile_q0 = tile_q0;
  a.cu_q = cu_q; a.ctx_len = ctx_len; a.scale = scale; a.window = window; a.n_q_heads = n_q_heads;
  a.group = n_q_heads / n_kv_heads; a.error_flag = error_flag;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  prefill_tc_kernel<<<dim3(n_q_heads, n_tiles), 128, kSmemBytes, (cudaStream_t)stream>>>(a);
  return LMSF_LAUNCH_STATUS();
}
