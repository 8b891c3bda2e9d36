// Prefill attention on the 5th-generation tensor cores: tcgen05.mma with both products' accumulators in
// tensor memory.  bfloat16, head size 64 or 128 (-DLMSF_HEAD_DIM), any mix of prompt portions over the
// paged cache; same interface and results (up to rounding) as lmsf_attention_prefill of attention_mma.cu.
//
// Counterpart in the reference: the dense float32 prompt attention of
// core/src/model_executor/layers/attention.rs:106-159.
//
// A unit of work is two items that share their keys: 128 query tokens of TWO query heads of one kv head, or, for a
// head that is left over (an odd group, or no grouping), two consecutive tiles of 128 query tokens of that head; so
// every k and v tile is fetched once for both.  The launch has at most one block per SM (a block holds all of an SM's
// tensor memory); block b of G takes the units b, 2G - 1 - b, 2G + b, ... of the list that the caller sorted longest
// first, so the blocks get nearly equal shares, and every mbarrier's phases run on from unit to unit.  The warps
// of a block have four roles:
//   * two producer warps, one for k and one for v, bring tiles of 128 keys from their pages into rings of
//     shared-memory stages with tensor-map copies (cp.async.bulk.tensor, one box per page and 64 head
//     elements, 128-byte swizzled by the copy engine; k is read K-major, v MN-major); the copies' bytes are
//     counted on mbarriers.  Pages of fewer than 8 keys are gathered with cp.async instead.  They run ahead into
//     the next unit's keys as far as the rings allow;
//   * a producer of the queries: the 128 x head-size tile of an item comes by tensor-map copies from the step's
//     [token][head x head size] matrix as soon as the item's last scores of the unit before are complete, i.e. while
//     that unit's last softmax, last P V and output are still under way; with the queries it leaves the softmax
//     warps a note of the unit's geometry in shared memory, so that no global load stands between two units;
//   * an issuing warp launches, for each item, S = Q K^T (M 128, N 128, K head size) into the item's score
//     buffer in tensor memory and, when the item's P is ready, O += P V (M 128, N head size, K 128) with P
//     read from tensor memory, in two halves of 64 keys: the first half's P V runs while the softmax still works
//     on the second half; completion goes to mbarriers through tcgen05.commit.  The two items take turns: one
//     item's products run while the other item's softmax is computed;
//   * two groups of four softmax warps, one per item, one query row per thread, with registers moved to them
//     from the other warps (setmaxnreg): tcgen05.ld of the row's 128 scores, mask where the tile needs one,
//     running maximum (the accumulator is rescaled only when the maximum grew by more than 2^8, which keeps the
//     sums exact and saves most read-modify-writes of tensor memory), exponentials in float32 with the packed
//     two-value arithmetic of sm_100 around them, P as bfloat16 pairs written over the first 64 columns of S
//     (tcgen05.st) and handed over in two halves.
// The kernel is launched as a programmatic dependent: barriers and tensor memory are set up while the kernel before
// it drains.  All 512 columns of tensor memory (S or P of two items, 128 each; O of two items, 128 each) and about
// 193 KB of shared memory (Q of two items, two stages of k, two of v).  Every wait on an mbarrier is bounded: when
// one runs out the block raises *error_flag (code 3), frees its tensor memory and returns.
#include <cstdlib>
#include <type_traits>

#include "attention_mma.cuh"
#include "tc_common.cuh"

#ifndef LMSF_HEAD_DIM
#error "compile with -DLMSF_HEAD_DIM=64 or 128"
#endif

LMSF_DEFINE_LAST_ERROR(lmsf_attention_tc)

namespace lmsf {
namespace tc {

using namespace lmsf::fa;

constexpr int HD = LMSF_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "the tcgen05 attention kernel takes head sizes 64 and 128");
constexpr int BM = 128;                    // query rows per item (a head and 128 tokens)
constexpr int BN = 128;                    // keys per tile
constexpr int kHB = HD / 64;               // 64-wide blocks of the head dimension
#ifndef LMSF_TC_STAGES
#define LMSF_TC_STAGES 2
#endif
constexpr int kStages = LMSF_TC_STAGES;    // k tiles in flight, and v tiles
constexpr int kQBytes = kHB * BM * 128;    // one item's queries
constexpr int kKBytes = kHB * BN * 128;    // one k (or v) tile
constexpr int kOffK = 2 * kQBytes, kOffV = kOffK + kStages * kKBytes;
constexpr int kSmemBytes = kOffV + kStages * kKBytes + 1024;   // + slack for the 1024-byte alignment
static_assert(kSmemBytes <= 227 * 1024, "too many stages for the shared memory of an SM");
// Tensor memory, 512 columns: S of item x in [128x, 128x + 128), and P (bfloat16 pairs) over its first 64
// columns once the scores are in registers; O of item x in [256 + 128x, +HD).
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kOCol = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units

struct Args {
  const bf16* q; long long q_stride;
  bf16* out; long long out_stride;
  PagedKV kv;
  const int* block_table; int max_blocks;
  const int* tile_seq; const int* tile_q0;   // one entry per 128 query tokens
  int n_q_tiles;
  const int* cu_q; const int* ctx_len;
  float scale; int window;
  int n_q_heads, group;
  int* error_flag;
  int use_tma;      // k and v tiles come by tensor-map copies (block_size >= 8), else by cp.async
  int rows_box;     // keys per tensor-map copy: min(block_size, 128)
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Registers move between warpgroups after the launch: the softmax warps hold a row of 128 scores each.
constexpr int kRegsSoftmax = 224, kRegsOther = 56;
__device__ __forceinline__ float ex2_approx(float x) {      // 2^x, 0 for -inf
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two float32 values in one 64-bit register, for the packed arithmetic of sm_100 (one instruction, two results).
__device__ __forceinline__ uint64_t pk2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// ---- roles ---------------------------------------------------------------------------------------------
// warps 0-3: softmax of the first item, one query row per thread (thread t owns lane t % 128 of tensor memory)
// warps 4-7: softmax of the second item
// warp 8   : producer of k tiles
// warp 9   : producer of v tiles
// warp 10  : issues the tensor-core products
// warp 11  : idle
constexpr int kSoftmaxThreads = 128;       // per item
constexpr int kThreadsTotal = 384;     // three warpgroups; warp 11 only gives its registers away

// Where pages are too small for tensor-map copies: the producer warp's cp.async gather of k (or v) of keys
// [key0, key0 + 128) of kv head kvh into a tile: [64-wide block of the head][key][128 bytes], 16-byte chunk c of
// a row at chunk c ^ (key & 7).  Keys outside [lo, hi) or without a page are zero-filled.
__device__ __forceinline__ void gather_tile(uint32_t dst_tile, const PagedKV& kv, const int* __restrict__ table, int max_blocks,
                                            int kvh, bool is_v, int key0, int lo, int hi, int lane) {
  constexpr int kChunks = HD / 8;
  constexpr int kRowsPerPass = 32 / kChunks;
  const size_t head_off = ((size_t)(is_v ? kv.n_kv_heads : 0) + kvh) * kv.block_size * HD;
  const int mask = kv.block_size - 1;
  const int c = lane % kChunks, r0 = lane / kChunks;
  const uint32_t col = (c / 8) * (BN * 128);
#pragma unroll 4
  for (int p = 0; p < BN / kRowsPerPass; ++p) {
    const int row = p * kRowsPerPass + r0, key = key0 + row, blk = key >> kv.block_shift;
    const int page = (key >= lo && key < hi && blk < max_blocks) ? table[blk] : -1;
    const bool ok = page >= 0;
    const bf16* src = ok ? kv.cache + (size_t)page * kv.page_stride + head_off + (size_t)(key & mask) * HD + c * 8 : kv.cache;
    cp_async_16(dst_tile + col + row * 128 + (((c & 7) ^ (row & 7)) << 4), src, ok ? 16 : 0);
  }
}

// A unit of work is a pair of items that share their keys.  First come the units of two query heads of one kv head:
// (a tile of 128 query tokens, a kv head, a pair of its heads), numbered with all heads of tile 0 first, then of tile
// 1, ...; the caller lists the tiles that see the most keys first.  Then, if a kv head has an odd number of query
// heads (or one: no grouping), the units of the head that is left over: it takes two consecutive tiles of 128 query
// tokens, so there is one unit for every tile that leads such a pair (q0 a multiple of 256) and kv head; the block
// lists the leading tiles in shared memory when it starts.
constexpr int kMaxLeadTiles = 4096;
struct UnitMap {
  int full_pairs, n_kv, units_full_per_tile, n_full, n_units;
  const unsigned short* lead;       // the tiles that lead a pair, in the order of the caller's list
};
struct Item { int head, q0, rows, hi, lo, tb, te; };   // a head and 128 query tokens; it sees the keys [lo, hi) in the tiles [tb, te)
struct Unit {
  int seq, kvh, head0, q0, tok0, n, start;
  bool two_heads, two, empty;
  int lo, hi, tile_begin, n_tiles;           // what either item sees
  __device__ __forceinline__ Item item(const Args& a, int x) const {
    Item i;
    i.head = head0 + (two_heads ? x : 0);
    i.q0 = q0 + (two_heads ? 0 : x * BM);
    i.rows = max(0, min(BM, n - i.q0));
    i.hi = start + i.q0 + i.rows;                               // keys < hi are visible to the item's last row
    i.lo = a.window > 0 ? max(0, start + i.q0 - a.window + 1) : 0;
    i.tb = i.lo / BN;
    i.te = (i.hi + BN - 1) / BN;
    return i;
  }
  // kLeft: the kernel is built twice, for even groups of heads (no unit of a head that is left over: the plain
  // numbering, which is also a little faster) and for odd ones
  template <bool kLeft>
  __device__ __forceinline__ void load(const Args& a, int unit, const UnitMap& m) {
    int tile, pair;
    if (!kLeft || unit < m.n_full) {
      tile = unit / m.units_full_per_tile;
      const int bx = unit % m.units_full_per_tile;
      kvh = bx / m.full_pairs;
      pair = bx % m.full_pairs;
    } else {
      const int j = unit - m.n_full;
      tile = m.lead[j / m.n_kv];
      kvh = j % m.n_kv;
      pair = m.full_pairs;
    }
    seq = a.tile_seq[tile];
    q0 = a.tile_q0[tile];
    head0 = kvh * a.group + 2 * pair;
    two_heads = 2 * pair + 1 < a.group;                         // the unit has a second head of the same kv head
    tok0 = a.cu_q[seq];
    n = a.cu_q[seq + 1] - tok0;
    start = a.ctx_len[seq] - n;
    // A head that is left over takes two query tiles: this one and the 128 tokens behind it.
    empty = !two_heads && (q0 & (2 * BM - 1)) != 0;
    two = two_heads || q0 + BM < n;                             // the unit has a second item
    const Item i0 = item(a, 0), i1 = item(a, 1);
    lo = i0.lo;                                                 // the second item is never behind the first
    hi = two ? i1.hi : i0.hi;
    tile_begin = i0.tb;
    n_tiles = (two ? i1.te : i0.te) - tile_begin;
    empty = empty || n_tiles <= 0;
  }
};

template <bool kLeft>
__global__ void __launch_bounds__(kThreadsTotal, 1) prefill_tc_kernel(const Args a, const __grid_constant__ CUtensorMap kv_map,
                                                                      const __grid_constant__ CUtensorMap q_map) {
  extern __shared__ unsigned char smem_raw[];
  // k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages], s_full[item], p_full[item][half of P],
  // o_done[item], q_full[item], q_free[item], taken[item]
  __shared__ __align__(8) uint64_t bars[4 * kStages + 14];
  __shared__ uint32_t tmem_base_mem;
  __shared__ int failed_mem;
  __shared__ unsigned short lead_tiles[kLeft ? kMaxLeadTiles : 1];
  __shared__ int n_lead_mem;
  // What the softmax warps of item x need to know of its next unit, written by the producer of the queries before it
  // announces the unit's queries on q_full[x]; two slots per item, used in turn.
  struct __align__(16) UnitNote { int head, q0, rows, tb, te, start, tok0, tile_begin, lo, hi, tiles_before, last; };
  __shared__ UnitNote notes[2][2];
  volatile int* failed = &failed_mem;
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;     // the swizzle pattern is a function of the address
  const uint32_t sQ = smem, sK = smem + kOffK, sV = smem + kOffV;
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto k_full = [&](int s) { return bar0 + 8u * s; };
  auto k_empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (3 * kStages + s); };
  auto s_full = [&](int x) { return bar0 + 8u * (4 * kStages + x); };
  auto p_full = [&](int x, int h) { return bar0 + 8u * (4 * kStages + 2 + 2 * x + h); };
  auto o_done = [&](int x) { return bar0 + 8u * (4 * kStages + 6 + x); };
  auto q_full = [&](int x) { return bar0 + 8u * (4 * kStages + 8 + x); };
  auto q_free = [&](int x) { return bar0 + 8u * (4 * kStages + 10 + x); };
  auto taken = [&](int x) { return bar0 + 8u * (4 * kStages + 12 + x); };
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // What needs nothing from global memory comes first, so that it overlaps the tail of the kernel before this
  // one (programmatic dependent launch): barriers, tensor memory.  Everything that kernel may have written
  // (q, the pages, the step's tables) is read after pdl_wait().
  pdl_launch_dependents();
  if (tid == 0) {
    // a tile is full after one arrival that announces the copies' bytes (tensor-map copies), or after one
    // arrival of each producer lane when its cp.async have landed
    for (int s = 0; s < kStages; ++s) {
      mbar_init(k_full(s), a.use_tma ? 1 : 32);
      mbar_init(v_full(s), a.use_tma ? 1 : 32);
      mbar_init(k_empty(s), 1);
      mbar_init(v_empty(s), 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(s_full(x), 1);
      mbar_init(p_full(x, 0), kSoftmaxThreads);
      mbar_init(p_full(x, 1), kSoftmaxThreads);
      mbar_init(o_done(x), 1);
      mbar_init(q_full(x), 1);
      mbar_init(q_free(x), 1);
      mbar_init(taken(x), kSoftmaxThreads);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    failed_mem = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_mem)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  if (kLeft && warp == 1) {
    // The tiles that lead a pair (the tile lists are inputs of the step: no kernel writes them, so they may be read
    // before the dependency wait).  The launcher takes no more tiles than the list holds.
    int count = 0;
    for (int base = 0; base < a.n_q_tiles; base += 32) {
      const int t = base + lane;
      const bool is_lead = t < a.n_q_tiles && (a.tile_q0[t] & (2 * BM - 1)) == 0;
      const unsigned mask = __ballot_sync(0xffffffffu, is_lead);
      const int pos = count + __popc(mask & ((1u << lane) - 1u));
      if (is_lead && pos < kMaxLeadTiles) lead_tiles[pos] = (unsigned short)t;
      count += __popc(mask);
    }
    if (lane == 0) n_lead_mem = min(count, kMaxLeadTiles);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_mem;
  pdl_wait();

  // The launch has at most one block per SM, and block b of G takes the units b, 2G - 1 - b, 2G + b, 4G - 1 - b,
  // ...: with a list sorted by length the blocks get nearly equal shares, a block pays for its barriers and tensor
  // memory once, and its producers fetch the next unit's first keys while the last unit is finished.  The
  // mbarriers' phases run on through the units, so every role counts what went before (all in the same way).
  UnitMap um;
  um.full_pairs = a.group / 2;
  um.n_kv = a.kv.n_kv_heads;
  um.units_full_per_tile = um.n_kv * um.full_pairs;
  um.n_full = um.units_full_per_tile * a.n_q_tiles;
  {
    um.lead = lead_tiles;
    um.n_units = um.n_full + (kLeft ? um.n_kv * n_lead_mem : 0);
  }
  const int n_units = um.n_units;
  const int G = gridDim.x;
  auto unit_of = [&](int pass) { return pass * G + ((pass & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x); };

  if (warp >= 8) {
  regs_dec<kRegsOther>();
  if (warp == 8 || warp == 9) {
    // ------------------------------------------------------------------ producers: warp 8 of k, warp 9 of v
    const bool is_v = warp == 9;
    auto full = [&](int s) { return is_v ? v_full(s) : k_full(s); };
    auto empty = [&](int s) { return is_v ? v_empty(s) : k_empty(s); };
    const uint32_t ring = is_v ? sV : sK;
    int tiles_before = 0;                                        // tiles of the block's earlier units
    int issued_total = 0;                                        // tiles whose copies were issued
    bool ok = true;
    for (int pass = 0; ok; ++pass) {
      const int unit = unit_of(pass);
      if (unit >= n_units) break;
      Unit u = {};
      u.template load<kLeft>(a, unit, um);
      if (u.empty) continue;
      const int* table = a.block_table + (size_t)u.seq * a.max_blocks;
      if (a.use_tma) {
        // Lane i copies box i of a tile: keys [i * rows_box, (i + 1) * rows_box), which lie in one page.  A key
        // range without a page (beyond the sequence, or before the window) is read from page 0 instead: all its
        // keys are masked, and the softmax warps clear those rows of v.
        const int n_box = BN / a.rows_box;
        const int head_row = (is_v ? a.kv.n_kv_heads : 0) + u.kvh;
        auto fetch_page = [&](int t) {
          const int blk = ((u.tile_begin + t) * BN + lane * a.rows_box) >> a.kv.block_shift;
          return (t < u.n_tiles && lane < n_box && blk < a.max_blocks) ? table[blk] : -1;
        };
        int page = fetch_page(0);
        for (int t = 0; t < u.n_tiles; ++t) {
          const int g = tiles_before + t, s = g % kStages;       // g: the tile counted over all units of the block
          const int slot0 = ((u.tile_begin + t) * BN + lane * a.rows_box) & (a.kv.block_size - 1);
          const uint32_t dst = ring + s * kKBytes + lane * a.rows_box * 128;
          if (g >= kStages && !mbar_wait_f(empty(s), (uint32_t)((g / kStages - 1) & 1), failed)) { ok = false; break; }
          const int next_page = fetch_page(t + 1);
          if (lane == 0) mbar_arrive_expect_tx(full(s), kKBytes);
          __syncwarp();
          if (lane < n_box) {
#pragma unroll
            for (int hb = 0; hb < kHB; ++hb)
              tma_load_box(dst + hb * (BN * 128), &kv_map, hb * 64, slot0, head_row, max(page, 0), full(s));
          }
          issued_total = g + 1;
          page = next_page;
        }
      } else {
        for (int t = 0; t < u.n_tiles; ++t) {
          const int g = tiles_before + t, s = g % kStages;
          if (g >= kStages && !mbar_wait_f(empty(s), (uint32_t)((g / kStages - 1) & 1), failed)) { ok = false; break; }
          gather_tile(ring + s * kKBytes, a.kv, table, a.max_blocks, u.kvh, is_v, (u.tile_begin + t) * BN, u.lo, u.hi, lane);
          cp_async_arrive(full(s));
        }
      }
      tiles_before += u.n_tiles;
    }
    // no copy of this block may be in flight when it ends, whichever way the loop was left
    if (a.use_tma) {
      for (int g = max(0, issued_total - kStages); g < issued_total; ++g) mbar_wait_drain(full(g % kStages), (uint32_t)((g / kStages) & 1));
    } else {
      cp_async_wait<0>();
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ tensor-core issue
    constexpr uint32_t idesc_s = instr_desc(BM, BN, 0), idesc_o = instr_desc(BM, HD, 1);
    const bool leader = elect_one();
    // descriptors of the first 16 head elements (S) or keys (P V) of each operand; a later slice of 16 adds
    // its byte offset / 16 to the address field
    const uint64_t dq0 = smem_desc(sQ, 16, 1024), dk0 = smem_desc(sK, 16, 1024), dv0 = smem_desc(sV, BN * 128, 1024);
    int tiles_before = 0;                                        // k (and v) tiles of the block's earlier units
    int item_tiles_before[2] = {0, 0};                           // tiles that item x has had in them
    int units_before[2] = {0, 0};                                // earlier units in which item x took part
    bool ok = true;
    for (int pass = 0; ok; ++pass) {
      const int unit = unit_of(pass);
      if (unit >= n_units) break;
      Unit u = {};
      u.template load<kLeft>(a, unit, um);
      if (u.empty) continue;
      const Item it0 = u.item(a, 0), it1 = u.item(a, 1);
      const int nx = u.two ? 2 : 1;
      const int n_tiles = u.n_tiles, tile_begin = u.tile_begin;
      auto active = [&](int x, int t) { return x == 0 ? (t >= it0.tb && t < it0.te) : (u.two && t >= it1.tb && t < it1.te); };
      // jx: how many tiles item x has had in this unit; j: tile counted from the unit's first
      auto issue_s = [&](int x, int j) {                          // S of item x and tile j
        const uint64_t dq = dq0 + (uint64_t)((x * kQBytes) >> 4);
        const uint64_t dk = dk0 + (uint64_t)((((tiles_before + j) % kStages) * kKBytes) >> 4);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off_a = (ks / 4) * (BM * 128) + (ks % 4) * 32, off_b = (ks / 4) * (BN * 128) + (ks % 4) * 32;
          umma(leader, tmem + x * BN, dq + (off_a >> 4), dk + (off_b >> 4), idesc_s, ks > 0);
        }
        umma_commit(leader, s_full(x));
        // the item's last scores of this unit: when they are complete its queries may be overwritten by the next unit's
        if (tile_begin + j == (x == 0 ? it0.te : it1.te) - 1) umma_commit(leader, q_free(x));
      };
      // O of item x += P V of tile j for the keys of half h (64 of the 128), P from tensor memory
      auto issue_pv = [&](int x, int j, int jx, int h) {
        const uint64_t dv = dv0 + (uint64_t)((((tiles_before + j) % kStages) * kKBytes) >> 4);
#pragma unroll
        for (int k4 = 0; k4 < BN / 32; ++k4) {
          const int ks = h * (BN / 32) + k4;
          umma_ts(leader, tmem + kOCol + x * 128, tmem + x * BN + ks * 8, dv + ((ks * 16 * 128) >> 4), idesc_o,
                  (jx > 0 || ks > 0) ? 1u : 0u);
        }
      };
      // the k tile of tile j is waited for once, before the first S that reads it
      int k_ready = -1;
      auto k_wait = [&](int j) {
        if (k_ready >= j) return true;
        const int g = tiles_before + j;
        if (!mbar_wait_f(k_full(g % kStages), (uint32_t)((g / kStages) & 1), failed)) return false;
        fence_async_smem();
        tc_fence_after();
        k_ready = j;
        return true;
      };
#pragma unroll
      for (int x = 0; x < 2; ++x)
        if (x < nx && ok) ok = mbar_wait_f(q_full(x), (uint32_t)(units_before[x] & 1), failed);
      if (ok) {
        fence_async_smem();
        ok = k_wait(0);
      }
      if (ok) {
#pragma unroll
        for (int x = 0; x < 2; ++x)
          if (x < nx && active(x, tile_begin)) issue_s(x, 0);
        umma_commit(leader, k_empty(tiles_before % kStages));
      }
      // The two items take turns: while one item's softmax runs, the tensor core works on the other item's
      // P V and on its next scores.  S of the next tile may overwrite P of this one because the products of one
      // thread are executed in the order of their issue.
      int jx[2] = {0, 0};
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int g = tiles_before + j, s = g % kStages, s1 = (g + 1) % kStages, t = tile_begin + j;
        const bool more = j + 1 < n_tiles;
        bool v_ready = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (x >= nx || !ok) continue;
          if (active(x, t)) {
            // the first 64 keys' P is handed over while the softmax still works on the other 64
            const uint32_t p_phase = (uint32_t)((item_tiles_before[x] + jx[x]) & 1);
            ok = mbar_wait_f(p_full(x, 0), p_phase, failed);
            if (ok && !v_ready) ok = mbar_wait_f(v_full(s), (uint32_t)((g / kStages) & 1), failed);
            if (!ok) continue;
            v_ready = true;
            fence_async_smem();
            tc_fence_after();
            issue_pv(x, j, jx[x], 0);
            ok = mbar_wait_f(p_full(x, 1), p_phase, failed);
            if (!ok) continue;
            tc_fence_after();
            issue_pv(x, j, jx[x], 1);
            ++jx[x];
            if (!active(x, t + 1)) umma_commit(leader, o_done(x));     // the item's last tile
          }
          if (more && active(x, t + 1)) {
            ok = k_wait(j + 1);
            if (!ok) continue;
            issue_s(x, j + 1);
          }
        }
        if (!ok) break;
        umma_commit(leader, v_empty(s));
        if (more) umma_commit(leader, k_empty(s1));
      }
      tiles_before += n_tiles;
      item_tiles_before[0] += it0.te - it0.tb;
      units_before[0] += 1;
      if (u.two) {
        item_tiles_before[1] += it1.te - it1.tb;
        units_before[1] += 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ producer of the queries (warp 11)
    // Q tile of an item: [64-wide block][row][128 bytes], 128-byte swizzled, one tensor-map copy per 64-wide block.
    // Rows beyond the portion hold the tokens that follow it in the step (zeros beyond the step's last token): their
    // results are never written.  The queries of a unit are requested as soon as the last scores of the unit before
    // are complete, so they arrive while that unit's last softmax, its last P V and its output are still under way.
    // This warp also reads the lists that describe a unit (it runs ahead of the others) and leaves the softmax warps
    // a note of what they need, so that no global load stands between two units on their path.
    int units_before[2] = {0, 0};
    int tiles_before = 0;
    bool ok = true;
    int issued[2] = {0, 0};
    for (int pass = 0; ok; ++pass) {
      const int unit = unit_of(pass);
      if (unit >= n_units) break;
      Unit u = {};
      u.template load<kLeft>(a, unit, um);
      if (u.empty) continue;
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        if (x == 1 && !u.two) continue;
        const Item me = u.item(a, x);
        // The item's scores of the unit before are complete: its queries may be overwritten.  And its softmax warps
        // have taken that unit's note: q_full[x] has two kinds of waiters, the issuing warp and the softmax warps, and
        // must not complete a second phase before both have seen the first (an item with a single tile in a unit
        // frees its queries before its softmax warps have even finished the unit before); the note of two units
        // ago is free as well then.
        if (units_before[x] > 0 && (!mbar_wait_f(q_free(x), (uint32_t)((units_before[x] - 1) & 1), failed) ||
                                    !mbar_wait_f(taken(x), (uint32_t)((units_before[x] - 1) & 1), failed))) { ok = false; break; }
        if (lane == 0) {
          notes[x][units_before[x] & 1] = UnitNote{me.head, me.q0, me.rows, me.tb, me.te, u.start, u.tok0, u.tile_begin, u.lo, u.hi,
                                                   tiles_before, 0};
          mbar_arrive_expect_tx(q_full(x), kQBytes);
#pragma unroll
          for (int hb = 0; hb < kHB; ++hb)
            tma_load_box_2d(sQ + x * kQBytes + hb * (BM * 128), &q_map, me.head * HD + hb * 64, u.tok0 + me.q0, q_full(x));
        }
        units_before[x] += 1;
        issued[x] = units_before[x];
      }
      tiles_before += u.n_tiles;
    }
    // no copy of this block may be in flight when it ends
    for (int x = 0; x < 2; ++x)
      if (issued[x] > 0) mbar_wait_drain(q_full(x), (uint32_t)((issued[x] - 1) & 1));
    // the note that ends the softmax warps' loop
    for (int x = 0; x < 2; ++x) {
      if (ok && units_before[x] > 0)
        ok = mbar_wait_f(q_free(x), (uint32_t)((units_before[x] - 1) & 1), failed) &&
             mbar_wait_f(taken(x), (uint32_t)((units_before[x] - 1) & 1), failed);
      if (lane == 0) {
        notes[x][units_before[x] & 1].last = 1;
        mbar_arrive(q_full(x));
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax of item x
    regs_inc<kRegsSoftmax>();
    const int x = warp >> 2, row = tid & 127;
    const uint32_t t_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 lanes of tensor memory
    const uint32_t t_s = t_row + x * BN, t_o = t_row + kOCol + x * 128;
    const float sl2 = a.scale * kLog2e;
    int my_tiles_before = 0;                                       // tiles that this item has had in the units before
    bool ok = true;
    for (int my_units_before = 0; ok; ++my_units_before) {         // the units in which this item takes part
      // the unit's queries are announced, and with them the note that describes the unit
      ok = mbar_wait_f(q_full(x), (uint32_t)(my_units_before & 1), failed);
      if (!ok) break;
      // the note stays as it is until this item's next unit but one is announced; what is needed once or seldom
      // is read where it is needed, so that it holds no register through the loop over the tiles
      const volatile UnitNote* note = &notes[x][my_units_before & 1];
      if (note->last) break;
      mbar_arrive(taken(x));
      struct { int rows, tb, te; } me = {note->rows, note->tb, note->te};
      const int q_pos0 = note->start + note->q0;                    // position of the item's first query
      const int stage0 = note->tiles_before + me.tb - note->tile_begin;   // the item's first tile counted over the block's units
      const int u_lo = note->lo, u_hi = note->hi;
      const bool row_ok = row < me.rows;
      const int pos = q_pos0 + min(row, me.rows - 1);                // this thread's query position
      const int row_lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
      float m_run = -INFINITY, l_run = 0.f;
      const int my_tiles = me.te - me.tb;
      for (int j = 0; j < my_tiles; ++j) {                           // j counts this item's tiles
        // S of the tile is complete, and with it every product issued before it: P V of the tile before too
        ok = mbar_wait_f(s_full(x), (uint32_t)((my_tiles_before + j) & 1), failed);
        if (!ok) break;
        tc_fence_after();
        const int key0 = (me.tb + j) * BN;
        const int ju = stage0 + j;                                   // the tile counted over the block's units: its stage
        // Only tiles that reach past some row's position (the diagonal) or before its window need the mask;
        // the test is the same for the whole group of warps.
        const bool need_mask = key0 + BN - 1 > q_pos0 || (a.window > 0 && key0 < q_pos0 + me.rows - a.window);
        // the row's 128 scores: four loads in flight, one wait
        float sc[BN];
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) tmem_ld32_issue(t_s + c0, sc + c0);
        tmem_wait_ld();
        if (need_mask) {      // keys that the row does not see become -inf; most tiles skip the test
#pragma unroll
          for (int i = 0; i < BN; ++i) {
            const int key = key0 + i;
            if ((key > pos) | (key < row_lo)) sc[i] = -INFINITY;
          }
        }
        // four chains of three-input maxima: 128 values in 16 dependent steps
        float mx0 = fmax3(sc[0], sc[1], sc[2]), mx1 = fmax3(sc[3], sc[4], sc[5]);
        float mx2 = fmax3(sc[6], sc[7], sc[8]), mx3 = fmax3(sc[9], sc[10], sc[11]);
#pragma unroll
        for (int i = 12; i + 7 < BN; i += 8) {
          mx0 = fmax3(mx0, sc[i], sc[i + 1]);
          mx1 = fmax3(mx1, sc[i + 2], sc[i + 3]);
          mx2 = fmax3(mx2, sc[i + 4], sc[i + 5]);
          mx3 = fmax3(mx3, sc[i + 6], sc[i + 7]);
        }
        float mx = fmaxf(fmax3(mx0, mx1, mx2), fmax3(mx3, sc[BN - 4], sc[BN - 3]));
        mx = fmax3(mx, sc[BN - 2], sc[BN - 1]);
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
            tmem_ld32(t_o + c0, r);
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(t_o + c0, r);
          }
        }
        if (key0 < u_lo || key0 + BN > u_hi) {
          // rows of v whose keys no query of the tile sees hold whatever their page holds: clear them, so that
          // their zero weights cannot meet a value that is not finite (both items' warps do, with the same zeros)
          const uint32_t v = sV + (ju % kStages) * kKBytes;
          const int r_lo = u_lo - key0, r_hi = u_hi - key0;
          ok = mbar_wait_f(v_full(ju % kStages), (uint32_t)((ju / kStages) & 1), failed);   // the tile's v has landed
          if (!ok) break;
          for (int idx = row; idx < kHB * BN * 8; idx += kSoftmaxThreads) {
            const int r = (idx >> 3) % BN;
            if (r < r_lo || r >= r_hi)
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v + (idx >> 3) * 128 + (idx & 7) * 16), "r"(0) : "memory");
          }
          fence_async_smem();
        }
        // P as bfloat16 pairs over the first 64 columns of S: keys 2c and 2c + 1 in column c
        const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
        // The scaling, the subtraction of the maximum and the row sums are packed (two values per instruction); the
        // exponentials come from the special-function unit.  (Tried and slower on this kernel: a share of the
        // exponentials by a polynomial on the FMA pipe, and exponentials of bfloat16 pairs; the softmax warps are
        // bound by the instructions they issue, not by that unit.)  The first 64 keys' P is handed to the issuing warp
        // while the other 64 are computed.
        const uint64_t sl2_2 = pk2(sl2, sl2), neg_m2 = pk2(neg_m, neg_m);
        uint64_t lsum = pk2(0.f, 0.f);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint64_t x2 = fma2(pk2(sc[h * 64 + 2 * i], sc[h * 64 + 2 * i + 1]), sl2_2, neg_m2);
            float p0, p1, x0, x1;
            upk2(x2, x0, x1);
            p0 = ex2_approx(x0);
            p1 = ex2_approx(x1);
            lsum = add2(lsum, pk2(p0, p1));
            w[i] = pack_bf16(p0, p1);
          }
          tmem_st32_issue(t_s + h * 32, w);
          if (h == 0) {
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(p_full(x, 0));
          }
        }
        tmem_wait_st();
        float l0, l1;
        upk2(lsum, l0, l1);
        l_run += l0 + l1;
        tc_fence_before();
        mbar_arrive(p_full(x, 1));
      }
      if (ok && my_tiles > 0) ok = mbar_wait_f(o_done(x), (uint32_t)(my_units_before & 1), failed);
      if (ok && my_tiles > 0) {
        tc_fence_after();
        const float inv = 1.0f / l_run;
        bf16* dst = a.out + (size_t)(note->tok0 + note->q0 + row) * a.out_stride + (size_t)note->head * HD;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_o + c0, r);                                 // every lane of the warp takes part
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
        // the next unit's first P V overwrites O: the reads above are complete (tmem_ld32 waits for them)
        tc_fence_before();
      }
      my_tiles_before += my_tiles;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*failed && tid == 0 && a.error_flag) atomicExch(a.error_flag, 3);
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}

// ---- tensor maps of the cache --------------------------------------------------------------------------
// One layer's cache is a 4-d tensor for the copy engine: (head element, slot, k heads then v heads, page).
// A box is 64 elements x rows_box slots; the engine writes it 128-byte swizzled.  cuTensorMapEncodeTiled is
// looked up in the driver at run time, so this library does not link against it.
// The map of a cache, made once per (address, geometry).  Returns nullptr and sets *why on failure.
inline const CUtensorMap* cache_tensor_map(const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                           long long n_pages, int rows_box, const char** why) {
  using Key = std::tuple<const void*, long long, int, int, long long>;
  static std::map<Key, CUtensorMap> maps;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key{cache, page_stride, block_size, n_kv_heads, n_pages};
  auto it = maps.find(key);
  if (it != maps.end()) return &it->second;
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) { *why = "the driver has no cuTensorMapEncodeTiled"; return nullptr; }
  const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)block_size, (cuuint64_t)(2 * n_kv_heads), (cuuint64_t)n_pages};
  const cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)block_size * HD * 2, (cuuint64_t)page_stride * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)rows_box, 1, 1};
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  CUtensorMap m;
  const CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled refused the cache's geometry"; return nullptr; }
  return &maps.emplace(key, m).first->second;
}

}  // namespace tc
}  // namespace lmsf

LMSF_API int lmsf_attention_tc_head_dim() { return LMSF_HEAD_DIM; }



// tile_seq / tile_q0: one entry per 128 query tokens of each portion, best listed with the tiles that see the
// most keys first.  q and out rows must be 16-byte aligned; q has n_tokens rows (all tokens of the step).
LMSF_API int lmsf_attention_prefill_tc(const void* q, long long q_stride, long long n_tokens, void* out, long long out_stride,
                                       const void* cache, long long page_stride, long long n_pages, int block_size,
                                       int n_kv_heads, const int* block_table, int max_blocks, const int* tile_seq, const int* tile_q0,
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
  if (n_tokens <= 0 || q_stride < (long long)n_q_heads * HD)
    LMSF_REFUSE("attention_prefill_tc: q must have a positive number of rows of at least heads x head size elements");
  if (q_stride % 8 || out_stride % 8 || ((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) % 16 || page_stride % 8)
    LMSF_REFUSE("attention_prefill_tc: q, out and the cache must be 16-byte aligned with row strides that are multiples of 8");
  Args a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  if (!make_paged_kv(a.kv, cache, page_stride, block_size, n_kv_heads))
    LMSF_REFUSE("attention_prefill_tc: block_size=%d must be a power of two", block_size);
  a.block_table = block_table; a.max_blocks = max_blocks; a.tile_seq = tile_seq; a.tile_q0 = tile_q0;
  a.cu_q = cu_q; a.ctx_len = ctx_len; a.scale = scale; a.window = window; a.n_q_heads = n_q_heads;
  a.group = n_q_heads / n_kv_heads; a.error_flag = error_flag; a.n_q_tiles = n_tiles;
  // pages of 8 keys and more come by tensor-map copies (a box of rows_box keys starts on a 1024-byte
  // boundary of the swizzled tile); smaller pages by cp.async
  a.rows_box = block_size < BN ? block_size : BN;
  a.use_tma = block_size >= 8 && n_pages > 0;
  CUtensorMap kv_map;
  memset(&kv_map, 0, sizeof(kv_map));
  if (a.use_tma) {
    const char* why = "";
    const CUtensorMap* m = cache_tensor_map(cache, page_stride, block_size, n_kv_heads, n_pages, a.rows_box, &why);
    if (!m) LMSF_REFUSE("attention_prefill_tc: %s", why);
    kv_map = *m;
  }
  // the queries as a 2-d tensor for the copy engine: (head x head size, token), a box of 64 elements x 128 tokens
  CUtensorMap q_map;
  {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) LMSF_REFUSE("attention_prefill_tc: the driver has no cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)n_q_heads * HD, (cuuint64_t)n_tokens};
    const cuuint64_t strides[1] = {(cuuint64_t)q_stride * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)BM};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) LMSF_REFUSE("attention_prefill_tc: cuTensorMapEncodeTiled refused the queries' geometry");
  }
  const bool left = (a.group & 1) != 0;          // a kv head has a query head that no other shares a unit with
  if (left && n_tiles > kMaxLeadTiles)
    LMSF_REFUSE("attention_prefill_tc: with an odd number of query heads per kv head a launch takes %d query tiles at most, not %d",
                kMaxLeadTiles, n_tiles);
  void (*kernel)(const Args, const CUtensorMap, const CUtensorMap) = left ? prefill_tc_kernel<true> : prefill_tc_kernel<false>;
  static bool configured[2] = {false, false};
  if (!configured[left]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured[left] = true;
  }
  // one block per SM at most (a block holds all of an SM's tensor memory); the blocks share the units out among them
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      LMSF_REFUSE("attention_prefill_tc: the device's number of SMs cannot be read");
    n_sms = v;
  }
  const long long n_units = (long long)n_kv_heads * ((a.group + 1) / 2) * n_tiles;
  long long n_blocks = n_units < n_sms ? n_units : n_sms;
  // LMSF_TC_MAX_BLOCKS=<n> launches fewer blocks, so that small inputs exercise blocks that take many units in turn
  if (const char* e = getenv("LMSF_TC_MAX_BLOCKS")) {
    const long long cap = atoll(e);
    if (cap > 0 && cap < n_blocks) n_blocks = cap;
  }
  return launch_pdl(kernel, dim3((unsigned)n_blocks), dim3(kThreadsTotal), kSmemBytes, (cudaStream_t)stream, a, kv_map, q_map);
}
