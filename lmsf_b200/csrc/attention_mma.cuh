// Building blocks of the bfloat16 tensor-core attention kernels: asynchronous copies of key/value
// rows from cache pages into shared memory, ldmatrix fragment loads and the m16n8k16 product.
#pragma once
#include "common.cuh"

namespace lmsf {
namespace fa {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16-byte asynchronous copy; src_bytes = 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// c (16x8, float32) += a (16x16 bf16, row) * b (16x8 bf16, col)
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kTileKeys = 64;   // keys per pipeline stage (prefill; decode blocks may take narrower tiles)
constexpr int kThreads = 128;   // 4 warps

// Geometry of one layer's cache and of one request's block table.  block_size is a power of two.
struct PagedKV {
  const bf16* cache;        // [page][2][kv_head][slot][HD]
  long long page_stride;    // elements between pages
  int block_size, block_shift;
  int n_kv_heads;
};

__host__ inline bool make_paged_kv(PagedKV& kv, const void* cache, long long page_stride, int block_size, int n_kv_heads) {
  if (block_size <= 0 || (block_size & (block_size - 1))) return false;
  int sh = 0;
  while ((1 << sh) < block_size) ++sh;
  kv = PagedKV{(const bf16*)cache, page_stride, block_size, sh, n_kv_heads};
  return true;
}

// Shared-memory stage: TILE rows of K then TILE rows of V.  Every row carries 16 bytes of padding, which
// makes the 8 rows of an ldmatrix fall into different banks for any HD.  Head size 64 is the exception: its rows
// are exactly 128 bytes and the 16-byte chunk c of row r sits at chunk c ^ (r & 7) instead, so that a stage is 16 KB
// and three stages leave room for four blocks on an SM (at head size 128 the same layout was measured slower than
// the padding: 108 us against 100 us for 64 requests of 2,048 keys).
template <int HD, int TILE = kTileKeys> struct Stage {
  static constexpr bool kSwizzled = HD == 64;
  static constexpr int kRowBytes = kSwizzled ? HD * 2 : HD * 2 + 16;
  static constexpr int kBytes = 2 * TILE * kRowBytes;
  static constexpr int kChunks = HD / 8;   // 16-byte chunks per row
  // byte offset of chunk `chunk` of row `row` inside the K (or the V) half of a stage
  __device__ static __forceinline__ uint32_t off(int row, int chunk) {
    return (uint32_t)(row * kRowBytes + ((kSwizzled ? (chunk ^ (row & 7)) : chunk) << 4));
  }
};

// Issues the copies of keys [key0, key0 + TILE) of kv head `kvh` into the stage at `stage_base`, by a block of THREADS.
// Keys outside [lo, hi) and keys whose page entry is negative are zero-filled, never read.
// A thread copies one 16-byte column of several CONSECUTIVE rows, so that it looks its page up once per
// page rather than once per row; a warp's copies of one pass cover whole rows (coalesced).
// `table` may be a copy of a slice of the request's block table: entry i of it is block i + table_off.
template <int HD, int TILE = kTileKeys, int THREADS = kThreads>
__device__ __forceinline__ void load_stage(uint32_t stage_base, const PagedKV& kv, const int* __restrict__ table, int kvh,
                                           int key0, int lo, int hi, int table_off = 0) {
  using S = Stage<HD, TILE>;
  const size_t v_off = (size_t)kv.n_kv_heads * kv.block_size * HD;
  const size_t head_off = (size_t)kvh * kv.block_size * HD;
  const int mask = kv.block_size - 1;
  if constexpr (THREADS % S::kChunks == 0) {
    constexpr int kRowsPerThread = TILE * S::kChunks / THREADS;   // = kChunks / 2
    const int c = threadIdx.x % S::kChunks, row0 = (threadIdx.x / S::kChunks) * kRowsPerThread;
    const bf16* page_ptr = nullptr;
    bool have_page = false;                         // page_ptr belongs to the page of the current row
#pragma unroll
    for (int it = 0; it < kRowsPerThread; ++it) {
      const int row = row0 + it, key = key0 + row, slot = key & mask;
      const bool in_range = key >= lo && key < hi;
      if (slot == 0) have_page = false;
      if (in_range && !have_page) {
        const int page = table[(key >> kv.block_shift) - table_off];
        page_ptr = page >= 0 ? kv.cache + (size_t)page * kv.page_stride + head_off + c * 8 : nullptr;
        have_page = true;
      }
      const bool ok = in_range && page_ptr != nullptr;
      const bf16* src = ok ? page_ptr + (size_t)slot * HD : kv.cache;
      const uint32_t dst = stage_base + S::off(row, c);
      cp_async_16(dst, src, ok ? 16 : 0);
      cp_async_16(dst + TILE * S::kRowBytes, ok ? src + v_off : src, ok ? 16 : 0);
    }
  } else {
    static_assert((TILE * S::kChunks) % THREADS == 0, "a stage's copies must divide evenly among the threads");
#pragma unroll
    for (int it = 0; it < (TILE * S::kChunks) / THREADS; ++it) {
      const int idx = threadIdx.x + it * THREADS;
      const int row = idx / S::kChunks, c = idx % S::kChunks;
      const int key = key0 + row;
      const bf16* src = kv.cache;
      int bytes = 0;
      if (key >= lo && key < hi) {
        const int page = table[(key >> kv.block_shift) - table_off];
        if (page >= 0) {
          src = kv.cache + (size_t)page * kv.page_stride + head_off + (size_t)(key & mask) * HD + c * 8;
          bytes = 16;
        }
      }
      const uint32_t dst = stage_base + S::off(row, c);
      cp_async_16(dst, src, bytes);
      cp_async_16(dst + TILE * S::kRowBytes, bytes ? src + v_off : src, bytes);
    }
  }
}

}  // namespace fa
}  // namespace lmsf
