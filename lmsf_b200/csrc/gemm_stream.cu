// out[M, N] = x[M, K] * W[N, K]^T for 17 to 128 rows (bfloat16): the matrix product of a decode step with many
// requests, or of a short prompt portion.  As for fewer rows (gemm_skinny.cu) the time is the time to stream W
// from memory once; here the stream runs through the copy engine and the 5th-generation tensor cores.
//
// Counterpart in the reference: cublasLtMatmul for every M
// (tops/csrc/tops/tensorrt_llm/common/cublasMMWrapper.cpp:122-209).
//
// Shape of the kernel.  W is cut into tiles of 128 rows (output features) and K into blocks of 64 (128 bytes of a
// row).  A thread block takes one tile and one contiguous share of its k blocks; the blocks that share a tile form
// a thread-block cluster (1, 2, 4 or 8 of them, the fewest that give every SM several blocks).  Blocks are small
// (a few hundred KB of W, at most ~100 KB of shared memory), so that several are resident per SM and the first
// copies of the next kernel's blocks, which do not depend on the kernel before, overlap that kernel's tail.
// A block has three roles:
//   * warp 0 requests a k block's 128 x 64 box of W and the matching rows x 64 box of x with cp.async.bulk.tensor
//     (128-byte swizzle) into a ring of stages; x comes from L2;
//   * warp 1 issues tcgen05.mma with the W box as the M side (128 output features), the x box as the N side
//     (the rows, padded to a multiple of 16) and a float32 accumulator in tensor memory;
//   * warps 2-5 read the accumulator with tcgen05.ld and put it, as float32, where the ring was.
// Then the cluster meets, and each block adds up a share of the rows over all blocks of the cluster, reading the
// others' shared memory in the order of k (always the same order), and writes that share of `out`.
// Every wait on an mbarrier is bounded: when one runs out the block raises *error_flag (code 4), still meets its
// cluster, frees its tensor memory and returns.
#include "tc_common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_gemm_stream)

namespace lmsf {
namespace stream {

using namespace lmsf::tc;

constexpr int kTileN = 128;                // output features per tile (the M of the tensor-core product)
constexpr int kBlockK = 64;                // k per stage: 128 bytes of a row
constexpr int kWBytes = kTileN * 128;      // 16 KB
constexpr int kMaxRows = 128;
constexpr int kThreads = 192;
constexpr int kIssueLanes = 4;
constexpr int kMaxSplits = 8;              // blocks of a cluster (the portable limit)
constexpr int kMaxStages = 8;
constexpr int kMinSmem = 56 * 1024;        // at most 4 blocks fit an SM: 4 x 128 columns of tensor memory are all there is

struct Args {
  void* out; long long ldo;
  int M, N, K;
  int rows_pad;                            // M rounded up to a multiple of 16
  int n_kblocks, n_splits;
  int stages;
  uint32_t tmem_cols;                      // a power of two >= rows_pad
  int out_f32;
  int* error_flag;
};

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// four floats at the same shared-memory offset as `local_addr` in block `rank` of the cluster
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, unsigned rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

__global__ void __launch_bounds__(kThreads) stream_kernel(const Args a, const __grid_constant__ CUtensorMap w_map,
                                                          const __grid_constant__ CUtensorMap x_map) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kMaxStages + 1];      // full[stages], empty[stages], acc_full
  __shared__ uint32_t tmem_base_mem;
  __shared__ int failed_mem;
  volatile int* failed = &failed_mem;
  const uint32_t smem = (smem_addr(smem_raw) + 1023u) & ~1023u;
  const int x_bytes = a.rows_pad * 128;
  const int stage_bytes = kWBytes + x_bytes;
  const uint32_t bar0 = smem_addr(&bars[0]);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
  const uint32_t acc_full = bar0 + 8u * (2 * kMaxStages);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, tile = blockIdx.y;               // split is also the block's rank in its cluster
  const int kb0 = (int)((long long)a.n_kblocks * split / a.n_splits);
  const int count = (int)((long long)a.n_kblocks * (split + 1) / a.n_splits) - kb0;     // >= 1: the host sees to it
  const int row0 = tile * kTileN;

  if (tid == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    failed_mem = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_mem)), "r"(a.tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_mem;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // W does not depend on the kernel before this one: the boxes of the first round of stages are requested
    // while that kernel may still run; x, its output, only after the wait.  Several lanes request side by side
    // (a lane's request takes several hundred cycles to issue; side by side they cost the same as one).
    const int n_first = min(count, a.stages);
    if (lane < n_first) {
      mbar_arrive_expect_tx(full(lane), (uint32_t)stage_bytes);
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(smem + lane * stage_bytes), "l"(&w_map), "r"((kb0 + lane) * kBlockK), "r"(row0), "r"(full(lane)) : "memory");
    }
    pdl_wait();
    if (lane < n_first) {
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(smem + lane * stage_bytes + kWBytes), "l"(&x_map), "r"((kb0 + lane) * kBlockK), "r"(0), "r"(full(lane)) : "memory");
    }
    int issued = n_first;                   // k blocks requested so far (the same in every lane)
    bool ok = true;
    // (never more lanes than stages: two requests for one stage in flight would pass the same wait)
    const int lanes = min(kIssueLanes, a.stages);
    for (int base = n_first; base < count && ok; base += lanes) {
      const int i = base + lane;
      if (lane < lanes && i < count) {
        const int round = i / a.stages, s = i - round * a.stages;
        ok = mbar_wait_f(empty(s), (uint32_t)((round - 1) & 1), failed);
        if (ok) {
          const uint32_t dst = smem + s * stage_bytes;
          mbar_arrive_expect_tx(full(s), (uint32_t)stage_bytes);
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dst), "l"(&w_map), "r"((kb0 + i) * kBlockK), "r"(row0), "r"(full(s)) : "memory");
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dst + kWBytes), "l"(&x_map), "r"((kb0 + i) * kBlockK), "r"(0), "r"(full(s)) : "memory");
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) issued = min(count, base + lanes);
    }
    // no copy of this block may be in flight when its ring is written over or it ends, whichever way the loop
    // was left (a lane that gave up has requested nothing; the k blocks before `issued` have all been requested)
    for (int i = issued > a.stages ? issued - a.stages : 0; i < issued; ++i)
      mbar_wait_drain(full(i % a.stages), (uint32_t)((i / a.stages) & 1));
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor-core issue
    const bool leader = elect_one();
    const uint32_t idesc = instr_desc(kTileN, a.rows_pad, 0);
    int s = 0;
    uint32_t phase = 0;                                        // parity of the ring's current round
    bool ok = true;
    for (int i = 0; i < count; ++i) {
      ok = mbar_wait_f(full(s), phase, failed);
      if (!ok) break;
      tc_fence_after();
      const uint32_t w = smem + s * stage_bytes;
      const uint64_t dw = smem_desc(w, 16, 1024), dx = smem_desc(w + kWBytes, 16, 1024);
#pragma unroll
      for (int ks = 0; ks < kBlockK / 16; ++ks)
        umma(leader, tmem, dw + (uint64_t)(ks * 2), dx + (uint64_t)(ks * 2), idesc, (i > 0 || ks > 0) ? 1u : 0u);
      umma_commit(leader, empty(s));
      if (++s == a.stages) { s = 0; phase ^= 1u; }
    }
    if (ok) umma_commit(leader, acc_full);
  } else {
    // ------------------------------------------------------------------ the accumulator goes where the ring was
    // thread = one output feature of the tile (a lane of tensor memory); part[m][feature], float32
    const int row = (warp & 3) * 32 + lane;
    const uint32_t t_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    float* part = reinterpret_cast<float*>(smem_raw + (smem - smem_addr(smem_raw)));
    if (mbar_wait_f(acc_full, 0u, failed)) {       // every product is done: every box has landed and been read
      tc_fence_after();
      for (int c0 = 0; c0 < a.rows_pad; c0 += 16) {
        uint32_t r[16];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                     : "=r"(r[0]),"=r"(r[1]),"=r"(r[2]),"=r"(r[3]),"=r"(r[4]),"=r"(r[5]),"=r"(r[6]),"=r"(r[7]),"=r"(r[8]),
                       "=r"(r[9]),"=r"(r[10]),"=r"(r[11]),"=r"(r[12]),"=r"(r[13]),"=r"(r[14]),"=r"(r[15])
                     : "r"(t_row + c0));
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) part[(c0 + i) * kTileN + row] = __uint_as_float(r[i]);
      }
    }
  }
  // Every block of the cluster has its part in place (a block whose wait ran out comes here too, so that the
  // others do not wait for it for ever; the launch is then reported as failed).
  tc_fence_before();
  if (a.n_splits > 1) cluster_sync_all();
  else __syncthreads();
  if (warp >= 2) {
    pdl_wait();          // `out` may still be read by the kernel before this one
    // this block's share of the rows; thread: 4 neighbouring features, every 4th row of the share
    const int m_lo = (int)((long long)a.M * split / a.n_splits), m_hi = (int)((long long)a.M * (split + 1) / a.n_splits);
    const int te = tid - 64, n4 = (te & 31) * 4, mg = te >> 5;
    const int nb = row0 + n4;
    for (int m0 = m_lo + mg; m0 < m_hi; m0 += 8) {          // two rows x all parts in flight at a time
      float4 v[2][kMaxSplits];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int m = min(m0 + 4 * j, m_hi - 1);
#pragma unroll
        for (int q = 0; q < kMaxSplits; ++q)
          if (q < a.n_splits) v[j][q] = ld_cluster_f32x4(smem + (uint32_t)((m * kTileN + n4) * 4), (unsigned)q);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int m = m0 + 4 * j;
        if (m >= m_hi) break;
        float4 acc = v[j][0];
#pragma unroll
        for (int q = 1; q < kMaxSplits; ++q)
          if (q < a.n_splits) { acc.x += v[j][q].x; acc.y += v[j][q].y; acc.z += v[j][q].z; acc.w += v[j][q].w; }
        const float o[4] = {acc.x, acc.y, acc.z, acc.w};
        if (a.out_f32) {
          float* dst = reinterpret_cast<float*>(a.out) + (size_t)m * a.ldo + nb;
          if (nb + 3 < a.N && (a.ldo & 3) == 0 && ((uintptr_t)a.out & 15) == 0) *reinterpret_cast<float4*>(dst) = acc;
          else
            for (int e = 0; e < 4; ++e) if (nb + e < a.N) dst[e] = o[e];
        } else {
          bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)m * a.ldo + nb;
          if (nb + 3 < a.N && (a.ldo & 3) == 0 && ((uintptr_t)a.out & 7) == 0) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
            uint2 u;
            u.x = *reinterpret_cast<const uint32_t*>(&lo);
            u.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst) = u;
          } else {
            for (int e = 0; e < 4; ++e) if (nb + e < a.N) dst[e] = __float2bfloat16_rn(o[e]);
          }
        }
      }
    }
  }
  // no block of the cluster may leave while another still reads its shared memory
  if (a.n_splits > 1) cluster_sync_all();
  else __syncthreads();
  if (*failed && tid == 0 && a.error_flag) atomicExch(a.error_flag, 4);
  tc_fence_after();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols));
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

// x: [M, K] bfloat16 (17 <= M <= 128 is what it is meant for; 1 <= M <= 128 is accepted), w: [N, K] bfloat16,
// out: [M, N] bfloat16 or float32.  K % 8 == 0, rows 16-byte aligned.  n_sms: the SMs of the device; the number of
// blocks that share a tile depends on N, K and n_sms only, so a row's result does not depend on M.
LMSF_API int lmsf_gemm_stream(void* out, const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw,
                              long long ldo, int out_f32, int n_sms, int* error_flag, void* stream) {
  using namespace lmsf;
  using namespace lmsf::stream;
  if (M <= 0 || N <= 0) return 0;
  if (M > kMaxRows) LMSF_REFUSE("gemm_stream: M=%d, this kernel takes at most %d rows", M, kMaxRows);
  if (K <= 0 || K % 8) LMSF_REFUSE("gemm_stream: K=%d must be a positive multiple of 8", K);
  if (ldx < K || ldw < K || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    LMSF_REFUSE("gemm_stream: the rows of x and w must be 16-byte aligned");
  if (ldo < N) LMSF_REFUSE("gemm_stream: ldo is smaller than the output row");
  if (n_sms <= 0 || n_sms > 1024) LMSF_REFUSE("gemm_stream: n_sms=%d", n_sms);
  Args a;
  a.out = out; a.ldo = ldo;
  a.M = M; a.N = N; a.K = K;
  a.rows_pad = (M + 15) / 16 * 16;
  a.tmem_cols = a.rows_pad <= 32 ? 32u : a.rows_pad <= 64 ? 64u : 128u;
  const int n_tiles = (N + kTileN - 1) / kTileN;
  if (n_tiles > 65535) LMSF_REFUSE("gemm_stream: N=%d has more than 65535 tiles of %d", N, kTileN);
  a.n_kblocks = (K + kBlockK - 1) / kBlockK;
  a.out_f32 = out_f32; a.error_flag = error_flag;
  // blocks per tile: the fewest that give every SM four blocks, while a block keeps at least 4 k blocks (64 KB of W)
  a.n_splits = 1;
  while (a.n_splits < kMaxSplits && (long long)n_tiles * a.n_splits < 4ll * n_sms && a.n_kblocks / (2 * a.n_splits) >= 4)
    a.n_splits *= 2;
  const int stage_bytes = kWBytes + a.rows_pad * 128;
  a.stages = a.rows_pad <= 16 ? 4 : 3;
  CUtensorMap w_map, x_map;
  if (!make_map_2d(w_map, w, K, N, ldw, kTileN) || !make_map_2d(x_map, x, K, M, ldx, a.rows_pad))
    LMSF_REFUSE("gemm_stream: cuTensorMapEncodeTiled is missing or refused the operands");
  int smem = a.stages * stage_bytes + 1024;
  if (smem < kMinSmem) smem = kMinSmem;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * (kWBytes + kMaxRows * 128) + 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)a.n_splits, (unsigned)n_tiles, 1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = (unsigned)a.n_splits;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, stream_kernel, a, w_map, x_map);
}
