// out[M, N] = x[M, K] * W[N, K]^T for 17 to 128 rows (bfloat16): the matrix product of a decode step with many
// requests, or of a short prompt portion.  As for fewer rows (gemm_skinny.cu) the time is the time to stream W
// from memory once; here the stream runs through the copy engine and the 5th-generation tensor cores.
//
// Counterpart in the reference: cublasLtMatmul for every M
// (tops/csrc/tops/tensorrt_llm/common/cublasMMWrapper.cpp:122-209).
//
// Shape of the kernel.  W is cut into tiles of 128 rows and K into blocks of 64; a unit of work is one block of
// one tile (16 KB of W).  The units, numbered tile by tile, are dealt out evenly and contiguously to one
// persistent block per SM, whatever the number of tiles, so every SM streams the same number of bytes.  A block
// has three roles:
//   * warp 0 requests a unit's 128 x 64 box of W and the matching rows x 64 box of x with cp.async.bulk.tensor
//     (128-byte swizzle) into a ring of stages; x comes from L2;
//   * warp 1 issues tcgen05.mma with the W box as the M side (128 output features), the x box as the N side
//     (the rows, padded to a multiple of 16) and float32 accumulators in tensor memory, two of them, so that
//     the next tile's products run while the last one is written out;
//   * warps 2-5 read an accumulator with tcgen05.ld.  If the block held all K blocks of the tile the values go
//     straight to `out`; else they go to the workspace as a partial sum (float32), a counter of the tile is
//     raised, and the block that raises it last adds the tile's partial sums in the order of k, always the
//     same order whoever is last, and writes `out`.
// Every wait on an mbarrier is bounded: when one runs out the block raises *error_flag (code 4), frees its
// tensor memory and returns.
#include "tc_common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_gemm_stream)

namespace lmsf {
namespace stream {

using namespace lmsf::tc;


constexpr int kTileN = 128;                // output features per tile (the M of the tensor-core product)
constexpr int kBlockK = 64;                // k per unit: 128 bytes of a row
constexpr int kWBytes = kTileN * 128;      // 16 KB
constexpr int kMaxRows = 128;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 256;        // two accumulators of up to 128 columns
constexpr int kIssueLanes = 4;
#ifndef LMSF_GS_RING_KB
#define LMSF_GS_RING_KB 200
#endif
constexpr int kRingBytes = LMSF_GS_RING_KB * 1024;     // shared memory of the stages: one block per SM
constexpr int kMaxParts = 64;              // blocks that may share one tile
constexpr int kMaxTiles = 1 << 16;         // counters at the start of the workspace

struct Args {
  void* out; long long ldo;
  float* workspace;                        // [n_ctas][2][rows_pad][128] partial sums
  unsigned* counters;                      // [n_tiles] parts of a shared tile that have been written; zero between launches
  int M, N, K;
  int rows_pad;                            // M rounded up to a multiple of 16
  int n_tiles, n_kblocks;
  int stages;
  int out_f32;
  int* error_flag;
};

// The units of block c: [first, last).
__host__ __device__ inline void units_of(long long total, int n_ctas, int c, long long& first, long long& last) {
  first = total * c / n_ctas;
  last = total * (c + 1) / n_ctas;
}

__global__ void __launch_bounds__(kThreads, 1) stream_kernel(const Args a, const __grid_constant__ CUtensorMap w_map,
                                                             const __grid_constant__ CUtensorMap x_map) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * 16 + 4];      // full[stages], empty[stages], acc_full[2], acc_empty[2]
  __shared__ uint32_t tmem_base_mem;
  __shared__ int failed_mem;
  __shared__ long long part_off[kMaxParts];      // where the parts of a shared tile lie in the workspace
  __shared__ int n_parts, is_last;
  volatile int* failed = &failed_mem;
  const uint32_t smem = (smem_addr(smem_raw) + 1023u) & ~1023u;
  const int x_bytes = a.rows_pad * 128;
  const int stage_bytes = kWBytes + x_bytes;
  const uint32_t bar0 = smem_addr(&bars[0]);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (16 + s); };
  auto acc_full = [&](int b) { return bar0 + 8u * (32 + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (34 + b); };
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  long long u0, u1;
  units_of((long long)a.n_tiles * a.n_kblocks, gridDim.x, blockIdx.x, u0, u1);

  if (tid == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    failed_mem = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_mem)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_mem;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // kIssueLanes lanes request kIssueLanes consecutive units in one instruction (a lane's request takes
    // several hundred cycles to issue; side by side they cost the same as one)
    const int count = (int)(u1 - u0);
    const int tile0 = (int)(u0 / a.n_kblocks), kb_first = (int)(u0 % a.n_kblocks);
    int issued = 0;                         // units requested so far (the same in every lane)
    bool ok = true;
    // W does not depend on the kernel before this one: the boxes of the first round of stages are requested
    // while that kernel may still run; x, its output, only after the wait.
    const int n_first = min(count, a.stages);
    auto coords = [&](int i, int& kb, int& row0) {
      const int k_lin = kb_first + i, t_off = k_lin / a.n_kblocks;
      kb = k_lin - t_off * a.n_kblocks;
      row0 = (tile0 + t_off) * kTileN;
    };
    if (lane < n_first) {
      int kb, row0;
      coords(lane, kb, row0);
      mbar_arrive_expect_tx(full(lane), (uint32_t)stage_bytes);
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(smem + lane * stage_bytes), "l"(&w_map), "r"(kb * kBlockK), "r"(row0), "r"(full(lane)) : "memory");
    }
    pdl_wait();
    if (lane < n_first) {
      int kb, row0;
      coords(lane, kb, row0);
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(smem + lane * stage_bytes + kWBytes), "l"(&x_map), "r"(kb * kBlockK), "r"(0), "r"(full(lane)) : "memory");
    }
    issued = n_first;
    for (int base = n_first; base < count && ok; base += kIssueLanes) {
      const int i = base + lane;
      const bool mine = lane < kIssueLanes && i < count;
      if (mine) {
        const int round = i / a.stages, s = i - round * a.stages;
        int kb, row0;
        coords(i, kb, row0);
        ok = mbar_wait_f(empty(s), (uint32_t)((round - 1) & 1), failed);
        if (ok) {
          const uint32_t dst = smem + s * stage_bytes;
          mbar_arrive_expect_tx(full(s), (uint32_t)stage_bytes);
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dst), "l"(&w_map), "r"(kb * kBlockK), "r"(row0), "r"(full(s)) : "memory");
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dst + kWBytes), "l"(&x_map), "r"(kb * kBlockK), "r"(0), "r"(full(s)) : "memory");
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) issued = min(count, base + kIssueLanes);
    }
    // no copy of this block may be in flight when it ends, whichever way the loop was left (a lane that gave up
    // has requested nothing for its unit; the units before `issued` have all been requested)
    for (int i = issued > a.stages ? issued - a.stages : 0; i < issued; ++i)
      mbar_wait_drain(full(i % a.stages), (uint32_t)((i / a.stages) & 1));
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor-core issue
    pdl_wait();
    const bool leader = elect_one();
    const uint32_t idesc = instr_desc(kTileN, a.rows_pad, 0);
    int seg = 0, s = 0;
    uint32_t phase = 0;                                        // parity of the ring's current round
    bool ok = true;
    int tile = (int)(u0 / a.n_kblocks), kb = (int)(u0 % a.n_kblocks);
    int left = (int)(u1 - u0);                                 // units still to do
    for (; left > 0 && ok; ++seg, ++tile, kb = 0) {
      const int n_seg = min(left, a.n_kblocks - kb);           // units of this segment
      const int buf = seg & 1;
      if (seg >= 2) {       // the accumulator was read out two segments ago
        ok = mbar_wait_f(acc_empty(buf), (uint32_t)((seg / 2 - 1) & 1), failed);
        if (!ok) break;
        tc_fence_after();
      }
      const uint32_t d = tmem + buf * kMaxRows;
      for (int i = 0; i < n_seg; ++i) {
        ok = mbar_wait_f(full(s), phase, failed);
        if (!ok) break;
        tc_fence_after();
        const uint32_t w = smem + s * stage_bytes;
        const uint64_t dw = smem_desc(w, 16, 1024), dx = smem_desc(w + kWBytes, 16, 1024);
#pragma unroll
        for (int ks = 0; ks < kBlockK / 16; ++ks)
          umma(leader, d, dw + (uint64_t)(ks * 2), dx + (uint64_t)(ks * 2), idesc, (i > 0 || ks > 0) ? 1u : 0u);
        umma_commit(leader, empty(s));
        if (++s == a.stages) { s = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(leader, acc_full(buf));
      left -= n_seg;
    }
  } else {
    // ------------------------------------------------------------------ epilogue: thread = one output feature of the tile
    pdl_wait();          // `out` and the workspace may still be read by the kernel before this one
    const int row = (warp & 3) * 32 + lane;                    // lane of tensor memory
    const uint32_t t_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    int seg = 0;
    bool ok = true;
    int tile = (int)(u0 / a.n_kblocks), kb = (int)(u0 % a.n_kblocks);
    int left = (int)(u1 - u0);
    for (; left > 0 && ok; ++seg, ++tile, kb = 0) {
      const int n_seg = min(left, a.n_kblocks - kb);
      const bool whole = n_seg == a.n_kblocks;
      const bool first = seg == 0;
      left -= n_seg;
      const int buf = seg & 1;
      ok = mbar_wait_f(acc_full(buf), (uint32_t)((seg / 2) & 1), failed);
      if (!ok) break;
      tc_fence_after();
      const int n = tile * kTileN + row;
      // a block's first segment may be the tail of a tile, its last one the head of a tile: slots 0 and 1
      float* part = a.workspace + ((size_t)blockIdx.x * 2 + (first ? 0 : 1)) * (size_t)a.rows_pad * kTileN;
      for (int c0 = 0; c0 < a.rows_pad; c0 += 16) {
        uint32_t r[16];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                     : "=r"(r[0]),"=r"(r[1]),"=r"(r[2]),"=r"(r[3]),"=r"(r[4]),"=r"(r[5]),"=r"(r[6]),"=r"(r[7]),"=r"(r[8]),
                       "=r"(r[9]),"=r"(r[10]),"=r"(r[11]),"=r"(r[12]),"=r"(r[13]),"=r"(r[14]),"=r"(r[15])
                     : "r"(t_row + buf * kMaxRows + c0));
        tmem_wait_ld();
        if (whole) {
          if (n < a.N) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int m = c0 + i;
              if (m < a.M) {
                if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + n] = __uint_as_float(r[i]);
                else reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + n] = __float2bfloat16_rn(__uint_as_float(r[i]));
              }
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) part[(size_t)(c0 + i) * kTileN + row] = __uint_as_float(r[i]);
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty(buf));
      if (whole) continue;
      // The tile is shared with other blocks: this block's part is counted, and the block that counts last adds
      // all parts up in the order of k (always the same order, whoever is last) and writes `out`.
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const long long total = (long long)a.n_tiles * a.n_kblocks;
        const long long t0 = (long long)tile * a.n_kblocks, t1 = t0 + a.n_kblocks;
        const int P = gridDim.x;
        int c = (int)(t0 * P / total);
        long long f, l;
        while (c > 0 && total * c / P > t0) --c;
        while (total * (c + 1) / P <= t0) ++c;
        int k = 0;
        for (; c < P && k < kMaxParts; ++c) {
          units_of(total, P, c, f, l);
          if (f >= t1) break;
          if (l <= f) continue;
          // the tile is block c's first segment if c starts inside it (or at its start), else its last
          part_off[k++] = (long long)(((size_t)c * 2 + (f >= t0 ? 0 : 1)) * (size_t)a.rows_pad * kTileN);
        }
        n_parts = k;
        const unsigned before = atomicAdd(a.counters + tile, 1u);
        is_last = before == (unsigned)k - 1;
        if (is_last) a.counters[tile] = 0;       // every part has been counted: the counter is left as it was found
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (is_last) {
        __threadfence();
        // thread: 4 neighbouring output features, every 4th row; 4 rows x all parts in flight at a time
        const int te = tid - 64, n4 = (te & 31) * 4, mg = te >> 5;
        const int nb = tile * kTileN + n4;
        for (int m0 = mg; m0 < a.M; m0 += 16) {
          float4 acc[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int k0 = 0; k0 < n_parts; k0 += 4) {          // 16 loads in flight, added in the order of k
            float4 v[4][4];
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const float* p = a.workspace + part_off[min(k0 + kk, n_parts - 1)] + n4;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int m = min(m0 + 4 * j, a.M - 1);
                v[kk][j] = __ldcg(reinterpret_cast<const float4*>(p + (size_t)m * kTileN));
              }
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              if (k0 + kk >= n_parts) break;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                acc[j].x += v[kk][j].x; acc[j].y += v[kk][j].y; acc[j].z += v[kk][j].z; acc[j].w += v[kk][j].w;
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int m = m0 + 4 * j;
            if (m >= a.M) continue;
            const float v[4] = {acc[j].x, acc[j].y, acc[j].z, acc[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (nb + e >= a.N) continue;
              if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + nb + e] = v[e];
              else reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + nb + e] = __float2bfloat16_rn(v[e]);
            }
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");        // part_off is free for the next segment
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*failed && tid == 0 && a.error_flag) atomicExch(a.error_flag, 4);
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}

inline bool make_map_2d(CUtensorMap& m, const void* p, long long inner, long long outer, long long ld_elems, int box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  const cuuint64_t strides[1] = {(cuuint64_t)ld_elems * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
  const cuuint32_t es[2] = {1, 1};
  return encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace stream
}  // namespace lmsf

// Floats of workspace that lmsf_gemm_stream needs for M rows on n_ctas blocks: counters (zero when the workspace is
// first used; a launch that completes leaves them zero), then the partial sums.
LMSF_API long long lmsf_gemm_stream_workspace_floats(int M, int n_ctas) {
  const int rows_pad = (M + 15) / 16 * 16;
  return lmsf::stream::kMaxTiles + (long long)n_ctas * 2 * rows_pad * lmsf::stream::kTileN;
}

// x: [M, K] bfloat16 (17 <= M <= 128 is what it is meant for; 1 <= M <= 128 is accepted), w: [N, K] bfloat16,
// out: [M, N] bfloat16 or float32.  K % 8 == 0, rows 16-byte aligned.  n_ctas: persistent blocks (the number of SMs).
LMSF_API int lmsf_gemm_stream(void* out, const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw,
                              long long ldo, int out_f32, float* workspace, long long workspace_floats, int n_ctas,
                              int* error_flag, void* stream) {
  using namespace lmsf;
  using namespace lmsf::stream;
  if (M <= 0 || N <= 0) return 0;
  if (M > kMaxRows) LMSF_REFUSE("gemm_stream: M=%d, this kernel takes at most %d rows", M, kMaxRows);
  if (K <= 0 || K % 8) LMSF_REFUSE("gemm_stream: K=%d must be a positive multiple of 8", K);
  if (ldx < K || ldw < K || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    LMSF_REFUSE("gemm_stream: the rows of x and w must be 16-byte aligned");
  if (ldo < N) LMSF_REFUSE("gemm_stream: ldo is smaller than the output row");
  if (n_ctas <= 0 || n_ctas > 1024) LMSF_REFUSE("gemm_stream: n_ctas=%d", n_ctas);
  if (workspace_floats < lmsf_gemm_stream_workspace_floats(M, n_ctas) || !workspace)
    LMSF_REFUSE("gemm_stream: the workspace holds %lld floats, %lld are needed", workspace_floats,
                lmsf_gemm_stream_workspace_floats(M, n_ctas));
  Args a;
  a.out = out; a.ldo = ldo; a.counters = reinterpret_cast<unsigned*>(workspace); a.workspace = workspace + kMaxTiles;
  a.M = M; a.N = N; a.K = K;
  a.rows_pad = (M + 15) / 16 * 16;
  a.n_tiles = (N + kTileN - 1) / kTileN;
  if (a.n_tiles > kMaxTiles) LMSF_REFUSE("gemm_stream: N=%d has more than %d tiles of %d", N, kMaxTiles, kTileN);
  a.n_kblocks = (K + kBlockK - 1) / kBlockK;
  a.out_f32 = out_f32; a.error_flag = error_flag;
  {
    // Fewer blocks for a small product: a block gets at least 4 units (64 KB of W), and at most kMaxParts - 2
    // blocks per tile, so that the partial sums of a tile stay within what the second kernel lists.
    const long long total = (long long)a.n_tiles * a.n_kblocks;
    long long n = n_ctas;
    if (n > total / 4) n = total / 4 > 0 ? total / 4 : 1;
    if (n > (long long)(kMaxParts - 2) * a.n_tiles) n = (long long)(kMaxParts - 2) * a.n_tiles;
    n_ctas = (int)n;
  }
  const int stage_bytes = kWBytes + a.rows_pad * 128;
  a.stages = kRingBytes / stage_bytes;
  if (a.stages > 16) a.stages = 16;
  if (a.stages < 2) a.stages = 2;
  CUtensorMap w_map, x_map;
  if (!make_map_2d(w_map, w, K, N, ldw, kTileN) || !make_map_2d(x_map, x, K, M, ldx, a.rows_pad))
    LMSF_REFUSE("gemm_stream: cuTensorMapEncodeTiled is missing or refused the operands");
  const int smem = a.stages * stage_bytes + 1024;
  static int configured_smem = 0;
  if (smem > configured_smem) {
    cudaError_t e = cudaFuncSetAttribute(stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured_smem = smem;
  }
  cudaStream_t s = (cudaStream_t)stream;
  return launch_pdl(stream_kernel, dim3(n_ctas), dim3(kThreads), (size_t)smem, s, a, w_map, x_map);
}
