// out[M, N] = x[M, K] * W[N, K]^T for a handful of rows (M <= 16, bfloat16): the matrix product of a
// decode step, where every weight is read once and the time is the time to stream W from memory.
// Optionally fused with the gated activation of the feed-forward: W = [gate; up] stacked along N and
// out[m, n] = act(x . gate_n) * (x . up_n).
//
// A third form serves the merged q, k, v projection of single tokens: the rows of q and k are rotated in the
// epilogue (rotary position encoding), q goes to its buffer and k and v straight into their cache pages, so that
// no kernel has to run between the projection and the attention.
//
// Two more forms take the RMSNorm between two products of a decode step into the products themselves.  The product
// before the norm adds its result to the float32 residual stream, stores residual x norm weight (bfloat16) and leaves,
// per block, the sum of the squares of its 16 residual values of every token ("residual form").  The product after
// the norm reads that as its x and multiplies its sums by 1 / sqrt(mean of squares + eps) of the token before
// anything else is done with them ("prenormed input"): the factor is common to a row of x, so it can wait until
// after the product.  The partial sums of squares are added in a fixed order.
//
// Counterpart in the reference: cublasLtMatmul for every M (tops/csrc/tops/tensorrt_llm/common/
// cublasMMWrapper.cpp:122-209) followed by silu_and_mul_kernel (vllm/kernels/activation_kernels.cu:26-41).
//
// Shape of the kernel: the weight rows are the M side of mma.sync m16n8k16 (16 output features per
// block), the tokens are its N side (8 per tile).  The 4 warps of a block split K among themselves; each
// warp streams its 16 x K/4 slice of W through a private ring of cp.async stages (16 rows x 64 k, each row
// 128 contiguous bytes of memory, swizzled in 16-byte chunks, read back with ldmatrix) and needs no block-wide barrier until the end,
// where the four partial sums are added in a fixed order.  The matching 64 k of x travel in the same
// stages (8 or 16 rows), so no load of the inner loop waits on anything but its stage.
#include "attention_mma.cuh"   // cp.async, ldmatrix and mma helpers

LMSF_DEFINE_LAST_ERROR(lmsf_gemm_skinny)

namespace lmsf {
namespace skinny {

using namespace lmsf::fa;

constexpr int kWarps = 4;
#ifndef LMSF_SKINNY_CH
#define LMSF_SKINNY_CH 1
#endif
constexpr int CH = LMSF_SKINNY_CH;          // a stage holds 64 * CH values of k per row
constexpr int kChunkK = 64 * CH;            // k per stage
constexpr int kRowBytes = kChunkK * 2;      // bytes of one row in a stage (contiguous in memory)
constexpr int kCPR = 8 * CH;                // 16-byte chunks per row
constexpr int kStageBytes = 16 * kRowBytes; // one group of 16 rows

struct Args {
  const bf16* x; long long ldx;
  const bf16* w; long long ldw;
  void* out; long long ldo;
  int M, N, K;
  int up_offset;      // FUSE: row of W where the "up" half starts (= N of the output)
  int act;            // FUSE: 0 silu, 1 gelu_tanh
  int out_f32;
  // the fused q/k/v form (ROPE): out is q [M, n_q_heads * head_dim]
  const int* positions; const int* token_seq;   // [M]
  const int* block_table; int max_blocks, block_size;
  bf16* cache; long long page_stride;           // one layer's pages [page][2][kv_head][slot][head_dim]
  const float* inv_freq; int rot_dim, is_neox;
  int n_q_heads, n_kv_heads, head_dim;
  int* error_flag;
  // prenormed input: x is residual x norm weight; token m's sums are multiplied by
  // 1 / sqrt(sum_p in_sumsq[m * in_ld + p] / in_width + in_eps), p < in_parts
  const float* in_sumsq; int in_parts; long long in_ld; float in_eps; int in_width;
  // residual form: res[m, n] += bfloat16(sum); out[m, n] = bfloat16(res[m, n] * norm_w[n]);
  // out_sumsq[m * out_ld + block] = sum of res[m, n]^2 over the block's n
  float* res; long long ldres; const void* norm_w; int norm_w_f32; float* out_sumsq; long long out_ld;
};

__device__ __forceinline__ float act_apply(float g, int act) {
  if (act == 0) return g / (1.0f + expf(-g));
  const float k = 0.7978845608028654f;
  return 0.5f * g * (1.0f + tanhf(k * (g + 0.044715f * g * g * g)));
}

// Copies `n_rows_stage` rows x k [k0, k0 + kChunkK) into a stage: row r of the stage comes from `base + r * ld`
// when `r < n_valid`, else it is zero-filled.  One warp instruction copies whole rows or half rows, so that
// memory sees contiguous requests of kRowBytes.  16-byte chunk c of row r lands at chunk c ^ (r & 7).
// `hi_off`: rows 8.. of the stage come from `hi_off` rows further down (the fused q/k/v form pairs a head's
// features i and i + rot/2 in one block).
template <int N_ROWS>
__device__ __forceinline__ void issue_rows(uint32_t stage, const bf16* __restrict__ base, long long ld, int n_valid,
                                           int k0, int K, int lane, int hi_off = 0, bool paired = false) {
  constexpr int kLanesPerRow = kCPR < 32 ? kCPR : 32;
  constexpr int kRowsPerInstr = 32 / kLanesPerRow;
  constexpr int kChunkPasses = kCPR / kLanesPerRow;
#pragma unroll
  for (int i = 0; i < N_ROWS / kRowsPerInstr; ++i) {
    const int r = lane / kLanesPerRow + kRowsPerInstr * i;
    const bool ok = (paired ? (r & 7) : r) < n_valid;   // paired: rows r and r + 8 belong together, n_valid counts pairs
#pragma unroll
    for (int j = 0; j < kChunkPasses; ++j) {
      const int c = lane % kLanesPerRow + j * kLanesPerRow;
      const bool okc = ok && k0 + c * 8 < K;          // K is a multiple of 8: a chunk is inside or outside
      const bf16* src = okc ? base + (size_t)(r + (r >= 8 ? hi_off : 0)) * ld + k0 + c * 8 : base;
      cp_async_16(stage + r * kRowBytes + ((c ^ (r & 7)) << 4), src, okc ? 16 : 0);
    }
  }
}

// PAIR: the gated form with 8 gate rows and the 8 matching up rows in one group of 16 (rows r and r + 8 belong together):
// twice the blocks of half the size of a group of gate rows beside a group of up rows, which leaves a shorter tail when
// the blocks do not fill their last wave.
template <int NT, int GROUPS, int STAGES, bool ROPE = false, bool PAIR = false>
__global__ void __launch_bounds__(kWarps * 32) skinny_kernel(Args a) {
  constexpr int kStage = GROUPS * kStageBytes + NT * 8 * kRowBytes;      // W group(s), then x
  extern __shared__ __align__(128) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g4 = lane >> 2, t4 = lane & 3;
  const int n0 = blockIdx.x * (PAIR ? 8 : 16);
  const int n_chunks_total = (a.K + kChunkK - 1) / kChunkK;
  // chunk c of warp w is chunk w + 4 c of the row: the four warps walk the same kilobyte of every row together
  const int c_begin = warp, c_stride = kWarps;
  const int n_chunks = (n_chunks_total - warp + kWarps - 1) / kWarps;
  const uint32_t ring = smem_u32(smem) + warp * (STAGES * kStage);
  const int rows_total = (GROUPS == 2 || PAIR) ? a.up_offset : a.N;       // rows of one group
  // ROPE: rows 0..7 of the block are features f0.., rows 8..15 features f1..: a rotated pair sits 8 rows apart
  int f0 = n0, f1 = n0 + 8;
  bool pair8 = false;                                            // the block holds NeoX pairs (i, i + rot/2)
  if (ROPE && a.inv_freq && a.is_neox) {
    const int head = n0 / a.head_dim, j = (n0 % a.head_dim) / 16;
    if (head < a.n_q_heads + a.n_kv_heads && j * 16 < a.rot_dim) {
      f0 = head * a.head_dim + 8 * j;
      f1 = f0 + a.rot_dim / 2;
      pair8 = true;
    }
  }
  const int hi_off = f1 - f0 - 8;

  auto issue_w = [&](int c) {
    const uint32_t st = ring + (c % STAGES) * kStage;
    const int k0 = (c_begin + c * c_stride) * kChunkK;
    if (ROPE) issue_rows<16>(st, a.w + (size_t)f0 * a.ldw, a.ldw, 16, k0, a.K, lane, hi_off);
    else if (PAIR) issue_rows<16>(st, a.w + (size_t)n0 * a.ldw, a.ldw, min(8, rows_total - n0), k0, a.K, lane, a.up_offset - 8, true);
    else issue_rows<16>(st, a.w + (size_t)n0 * a.ldw, a.ldw, rows_total - n0, k0, a.K, lane);
    if (GROUPS == 2)
      issue_rows<16>(st + kStageBytes, a.w + (size_t)(a.up_offset + n0) * a.ldw, a.ldw, rows_total - n0, k0, a.K, lane);
  };
  auto issue_x = [&](int c) {
    const uint32_t st = ring + (c % STAGES) * kStage;
    issue_rows<8 * NT>(st + GROUPS * kStageBytes, a.x, a.ldx, a.M, (c_begin + c * c_stride) * kChunkK, a.K, lane);
  };
  auto issue = [&](int c) { issue_w(c); issue_x(c); };
  // The weights do not depend on the kernel before this one: their first stages are requested while that
  // kernel may still be running; x is read only after it has finished.
  pdl_launch_dependents();
  for (int s = 0; s < STAGES - 1; ++s)
    if (s < n_chunks) issue_w(s);
  pdl_wait();
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_chunks) issue_x(s);
    cp_async_commit();
  }

  // prenormed input: 128 / (8 NT) threads share a token's partial sums of squares.  The first 16 of a thread are asked
  // for here (16-byte loads) and added after the loop, so that nothing waits for them; more parts than those 256 / NT (a
  // width above 4,096 / NT) are read then.  The order of the sum depends on the number of parts only.
  constexpr int kTPR = kWarps * 32 / (8 * NT);
  float4 ss_v[4];
  auto load_ss = [&](int q0) {
    const int m = threadIdx.x / kTPR, j = threadIdx.x % kTPR;
    const float* src = a.in_sumsq + (size_t)m * a.in_ld;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int q = q0 + u * kTPR + j;
      ss_v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m >= a.M) continue;
      if (q * 4 + 3 < a.in_parts) ss_v[u] = *reinterpret_cast<const float4*>(src + q * 4);
      else if (q * 4 < a.in_parts) {
        ss_v[u].x = src[q * 4];
        if (q * 4 + 1 < a.in_parts) ss_v[u].y = src[q * 4 + 1];
        if (q * 4 + 2 < a.in_parts) ss_v[u].z = src[q * 4 + 2];
      }
    }
  };
  if (a.in_sumsq) load_ss(0);
  // residual form: the residual values and norm weights of this thread's results, asked for before the loop
  float e_res[NT], e_nw[NT];
  if (!ROPE && !PAIR && GROUPS == 1 && a.res) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int idx = threadIdx.x + t * kWarps * 32;
      const int m = idx / 16, n = n0 + idx % 16;
      const bool ok = m < a.M && n < a.N;
      e_res[t] = ok ? a.res[(size_t)m * a.ldres + n] : 0.f;
      e_nw[t] = !ok ? 0.f : (a.norm_w_f32 ? reinterpret_cast<const float*>(a.norm_w)[n]
                                           : __bfloat162float(reinterpret_cast<const bf16*>(a.norm_w)[n]));
    }
  }

  // ROPE: where this thread's results go (one token per pass of the epilogue), asked for before the loop
  int e_pos[NT], e_page[NT];
  if (ROPE) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int m = (threadIdx.x + t * kWarps * 32) / 16;
      e_pos[t] = m < a.M ? a.positions[m] : 0;
      e_page[t] = -1;
      if (m < a.M && f0 >= a.n_q_heads * a.head_dim) {            // a block of k or v features
        const int blk = e_pos[t] / a.block_size;
        e_page[t] = blk < a.max_blocks ? a.block_table[(size_t)a.token_seq[m] * a.max_blocks + blk] : -1;
      }
    }
  }

  float acc[GROUPS][NT][4];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g)
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[g][t][0] = acc[g][t][1] = acc[g][t][2] = acc[g][t][3] = 0.f;

  for (int c = 0; c < n_chunks; ++c) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    if (c + STAGES - 1 < n_chunks) issue(c + STAGES - 1);
    cp_async_commit();
    const uint32_t st = ring + (c % STAGES) * kStage;
    const uint32_t xs = st + GROUPS * kStageBytes;
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kp = 0; kp < 2 * CH; ++kp) {          // pairs of k-steps (32 values of k)
      uint32_t xf[2][NT][2];
      if (NT == 1) {
        uint32_t b[4];
        ldmatrix_x4(b, xs + r * kRowBytes + (((kp * 4 + mi) ^ (r & 7)) << 4));
        xf[0][0][0] = b[0]; xf[0][0][1] = b[1];
        xf[1][0][0] = b[2]; xf[1][0][1] = b[3];
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t b[4];
          const int row = (mi >> 1) * 8 + r;
          ldmatrix_x4(b, xs + row * kRowBytes + ((((kp * 2 + h) * 2 + (mi & 1)) ^ (row & 7)) << 4));
          xf[h][0][0] = b[0]; xf[h][0][1] = b[1];
          xf[h][NT - 1][0] = b[2]; xf[h][NT - 1][1] = b[3];
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = (mi & 1) * 8 + r, chunk = (kp * 2 + h) * 2 + (mi >> 1);
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
          uint32_t af[4];
          ldmatrix_x4(af, st + g * kStageBytes + row * kRowBytes + ((chunk ^ (row & 7)) << 4));
#pragma unroll
          for (int t = 0; t < NT; ++t) mma_16816(acc[g][t], af, xf[h][t][0], xf[h][t][1]);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncwarp();

  // partial sums of the four warps: [warp][group][row 16][token 8 NT], added in warp order
  float* part = reinterpret_cast<float*>(smem + warp * (STAGES * kStage));
#pragma unroll
  for (int g = 0; g < GROUPS; ++g)
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      float* base = part + g * (16 * 8 * NT);
      base[g4 * (8 * NT) + t * 8 + t4 * 2] = acc[g][t][0];
      base[g4 * (8 * NT) + t * 8 + t4 * 2 + 1] = acc[g][t][1];
      base[(g4 + 8) * (8 * NT) + t * 8 + t4 * 2] = acc[g][t][2];
      base[(g4 + 8) * (8 * NT) + t * 8 + t4 * 2 + 1] = acc[g][t][3];
    }
  // prenormed input: token m's factor, kept in the region of the warp that summed it
  constexpr int kFactorOff = 2048;                                 // behind the largest set of partial sums
  if (a.in_sumsq) {
    float row_ss = 0.f;
    for (int q0 = 0;;) {
#pragma unroll
      for (int u = 0; u < 4; ++u) row_ss += (ss_v[u].x + ss_v[u].y) + (ss_v[u].z + ss_v[u].w);
      q0 += 4 * kTPR;
      if (q0 * 4 >= a.in_parts) break;
      load_ss(q0);
    }
#pragma unroll
    for (int o = kTPR / 2; o > 0; o >>= 1) row_ss += __shfl_xor_sync(0xffffffffu, row_ss, o);
    if (threadIdx.x % kTPR == 0 && threadIdx.x / kTPR < a.M)
      reinterpret_cast<float*>(smem + warp * (STAGES * kStage) + kFactorOff)[threadIdx.x / kTPR] =
          1.0f / sqrtf(row_ss / (float)a.in_width + a.in_eps);
  }
  __syncthreads();
  auto factor = [&](int m) -> float {
    if (!a.in_sumsq || m >= a.M) return 1.0f;
    return reinterpret_cast<const float*>(smem + ((m * kTPR) >> 5) * (STAGES * kStage) + kFactorOff)[m];
  };
  if constexpr (ROPE) {
    // one (token, feature) per thread and pass; the partner of a rotated pair is 8 lanes away (NeoX) or the neighbour
    const int q_size = a.n_q_heads * a.head_dim, kv_size = a.n_kv_heads * a.head_dim;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int idx = threadIdx.x + t * kWarps * 32;
      const int m = idx / 16, row = idx % 16;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w)
        sum += reinterpret_cast<const float*>(smem + w * (STAGES * kStage))[row * (8 * NT) + m];
      sum *= factor(m);
      const float val = __bfloat162float(__float2bfloat16_rn(sum));      // what the plain product would have stored
      const float other = __shfl_xor_sync(0xffffffffu, val, pair8 ? 8 : 1);
      if (m >= a.M) continue;
      const int n = row < 8 ? f0 + row : f1 + row - 8;                  // feature among q, k, v
      const int d = n % a.head_dim;
      const bool is_v = n >= q_size + kv_size;
      float r = val;
      if (a.inv_freq && !is_v && d < a.rot_dim) {
        const bool first = a.is_neox ? d < a.rot_dim / 2 : (d & 1) == 0;
        const int i = a.is_neox ? d % (a.rot_dim / 2) : d / 2;
        float sn, cs;
        sincosf((float)e_pos[t] * a.inv_freq[i], &sn, &cs);
        const float x = first ? val : other, y = first ? other : val;
        r = first ? rot_first(x, y, cs, sn) : rot_second(x, y, cs, sn);
      }
      if (n < q_size) {
        reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + n] = __float2bfloat16_rn(r);
      } else if (e_page[t] < 0) {
        if (a.error_flag) atomicExch(a.error_flag, 2);                   // the token has no page
      } else {
        const int g = (n - q_size - (is_v ? kv_size : 0)) / a.head_dim;
        bf16* page = a.cache + (size_t)e_page[t] * a.page_stride + (is_v ? (size_t)a.n_kv_heads * a.block_size * a.head_dim : 0);
        page[((size_t)g * a.block_size + e_pos[t] % a.block_size) * a.head_dim + d] = __float2bfloat16_rn(r);
      }
    }
  } else if constexpr (PAIR) {
    // one (token, row) per thread and pass; the up value of a gate row is 8 lanes away
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int idx = threadIdx.x + t * kWarps * 32;
      const int m = idx / 16, row = idx % 16;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w)
        sum += reinterpret_cast<const float*>(smem + w * (STAGES * kStage))[row * (8 * NT) + m];
      sum *= factor(m);
      const float up = __shfl_down_sync(0xffffffffu, sum, 8);
      if (row >= 8 || m >= a.M || n0 + row >= rows_total) continue;
      const float r = act_apply(sum, a.act) * up;
      if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + n0 + row] = r;
      else reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + n0 + row] = __float2bfloat16_rn(r);
    }
  } else {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int idx = threadIdx.x + t * kWarps * 32;
      const int m = idx / 16, row = idx % 16;          // consecutive threads write consecutive n
      const bool ok = m < a.M && n0 + row < rows_total;
      const float f = factor(m);
      float v[GROUPS];
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w)
          s += reinterpret_cast<const float*>(smem + w * (STAGES * kStage))[g * (16 * 8 * NT) + row * (8 * NT) + m];
        v[g] = s * f;
      }
      const float r = GROUPS == 2 ? act_apply(v[0], a.act) * v[GROUPS - 1] : v[0];
      if (GROUPS == 1 && a.res) {
        float nr = 0.f;
        if (ok) {
          nr = e_res[t] + __bfloat162float(__float2bfloat16_rn(r));   // the plain product's bfloat16 result, added in float32
          a.res[(size_t)m * a.ldres + n0 + row] = nr;
          reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + n0 + row] = __float2bfloat16_rn(nr * e_nw[t]);
        }
        float sq = nr * nr;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (row == 0 && m < a.M) a.out_sumsq[(size_t)m * a.out_ld + blockIdx.x] = sq;
      } else if (ok) {
        if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)m * a.ldo + n0 + row] = r;
        else reinterpret_cast<bf16*>(a.out)[(size_t)m * a.ldo + n0 + row] = __float2bfloat16_rn(r);
      }
    }
  }
}

template <int NT, int GROUPS, int STAGES, bool ROPE = false, bool PAIR = false>
static int launch(const Args& a, int rows, cudaStream_t s) {
  const int smem = kWarps * STAGES * (GROUPS * kStageBytes + NT * 8 * kRowBytes);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(skinny_kernel<NT, GROUPS, STAGES, ROPE, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_pdl(skinny_kernel<NT, GROUPS, STAGES, ROPE, PAIR>, dim3(ceil_div(rows, PAIR ? 8 : 16)), dim3(kWarps * 32), smem, s, a);
}

#ifndef LMSF_SKINNY_STAGES
#define LMSF_SKINNY_STAGES (CH == 1 ? 6 : (CH == 2 ? 4 : 3))
#endif
constexpr int kStagesPlain = LMSF_SKINNY_STAGES;
#ifndef LMSF_SKINNY_STAGES_M16
#define LMSF_SKINNY_STAGES_M16 (CH == 1 ? 4 : LMSF_SKINNY_STAGES)
#endif
// 9 to 16 rows: a stage holds twice as much of x; with four stages three blocks still fit an SM (six stages: two
// blocks, and the 128256 x 4096 head at 16 rows takes 207 us instead of 180)
constexpr int kStagesPlain16 = LMSF_SKINNY_STAGES_M16;
#ifndef LMSF_SKINNY_STAGES_FUSED
#define LMSF_SKINNY_STAGES_FUSED (CH == 1 ? 3 : 2)
#endif
constexpr int kStagesFused = LMSF_SKINNY_STAGES_FUSED;
// A launch of so few blocks that at most two of them fall to an SM, or one, leaves shared memory unused and has few
// bytes in flight per SM: such launches get deeper rings (the 4,096-row output and down products of Llama-3-8B, 256
// blocks: a decode step of 8 requests 3.37 -> 3.21 ms with eight stages instead of six, 3.24 with seven or nine; ten,
// with which one block fits an SM and the 256 run in two waves: 3.70 ms; 9 to 16 rows: six stages instead of four,
// a step of 16 requests 4.07 -> 3.95 ms).  Launches of at most one block an SM (2,048-row products, 128 blocks) are
// no faster with 12 or 16 stages than with eight.
#ifndef LMSF_SKINNY_STAGES_FEW
#define LMSF_SKINNY_STAGES_FEW 8
#endif
#ifndef LMSF_SKINNY_STAGES_ONE
#define LMSF_SKINNY_STAGES_ONE LMSF_SKINNY_STAGES_FEW
#endif
#ifndef LMSF_SKINNY_STAGES_FEW_M16
#define LMSF_SKINNY_STAGES_FEW_M16 (CH == 1 ? 6 : LMSF_SKINNY_STAGES_M16)
#endif
#ifndef LMSF_SKINNY_STAGES_ONE_M16
#define LMSF_SKINNY_STAGES_ONE_M16 LMSF_SKINNY_STAGES_FEW_M16
#endif
constexpr int kStagesFew = LMSF_SKINNY_STAGES_FEW, kStagesOne = LMSF_SKINNY_STAGES_ONE;
constexpr int kStagesFew16 = LMSF_SKINNY_STAGES_FEW_M16, kStagesOne16 = LMSF_SKINNY_STAGES_ONE_M16;

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
  }
  return n;
}

// The plain, residual, prenormed and q/k/v forms (one group of 16 rows a block): the ring's depth by the number of blocks.
template <bool ROPE>
static int launch_by_blocks(const Args& a, int rows, cudaStream_t s) {
  const int blocks = ceil_div(rows, 16), sms = sm_count();
  if (a.M <= 8) {
    if (kStagesOne != kStagesFew && blocks <= sms) return launch<1, 1, kStagesOne, ROPE>(a, rows, s);
    if (kStagesFew != kStagesPlain && blocks <= 2 * sms) return launch<1, 1, kStagesFew, ROPE>(a, rows, s);
    return launch<1, 1, kStagesPlain, ROPE>(a, rows, s);
  }
  if (kStagesOne16 != kStagesFew16 && blocks <= sms) return launch<2, 1, kStagesOne16, ROPE>(a, rows, s);
  if (kStagesFew16 != kStagesPlain16 && blocks <= 2 * sms) return launch<2, 1, kStagesFew16, ROPE>(a, rows, s);
  return launch<2, 1, kStagesPlain16, ROPE>(a, rows, s);
}

}  // namespace skinny
}  // namespace lmsf

namespace lmsf {
namespace skinny {

// What the product forms have in common: checks, then the kernel for the number of rows and the form.
static int run_product(Args& a, int fuse_act, cudaStream_t s) {
  const int M = a.M, N = a.N, K = a.K;
  if (M <= 0 || N <= 0) return 0;
  if (M > 16) LMSF_REFUSE("gemm_skinny: M=%d, this kernel takes at most 16 rows", M);
  if (K <= 0 || K % 8) LMSF_REFUSE("gemm_skinny: K=%d must be a positive multiple of 8", K);
  if (fuse_act > 1) LMSF_REFUSE("gemm_skinny: unknown activation code %d", fuse_act);
  if (fuse_act >= 0 && N % 2) LMSF_REFUSE("gemm_skinny: a gated product needs an even N, got %d", N);
  if (a.ldx < K || a.ldw < K || a.ldx % 8 || a.ldw % 8 || ((uintptr_t)a.x % 16) || ((uintptr_t)a.w % 16))
    LMSF_REFUSE("gemm_skinny: the rows of x and w must be 16-byte aligned");
  if (a.in_sumsq && (a.in_parts <= 0 || a.in_ld < a.in_parts || a.in_ld % 4 || ((uintptr_t)a.in_sumsq % 16) ||
                     a.in_width <= 0 || !(a.in_eps > 0.f)))
    LMSF_REFUSE("gemm_skinny: the sums of squares of a prenormed input need rows of a multiple of 4 floats, 16-byte "
                "aligned, a width and a positive eps");
  a.up_offset = fuse_act >= 0 ? N / 2 : 0; a.act = fuse_act;
  if (fuse_act >= 0) {
    if (a.ldo < N / 2) LMSF_REFUSE("gemm_skinny: ldo is smaller than the output row");
    // Up to 8 rows: gate and up rows paired in one group, blocks of half the size (Llama-3-8B sizes: a decode step of
    // 8 requests 3.45 -> 3.40 ms, of one 3.23 -> 3.16: 896 blocks were 2.02 waves of 444, and the last 8 cost a whole
    // block's time).  9 to 16 rows: a group of gate rows beside a group of up rows (a step of 16 requests 4.09 ms
    // against 4.15 paired).
    return M <= 8 ? launch<1, 1, kStagesPlain, false, true>(a, N / 2, s) : launch<2, 2, kStagesFused>(a, N / 2, s);
  }
  if (a.ldo < N) LMSF_REFUSE("gemm_skinny: ldo is smaller than the output row");
  return launch_by_blocks<false>(a, N, s);
}

}  // namespace skinny
}  // namespace lmsf

// x: [M, K] bfloat16 (M <= 16), w: [N, K] bfloat16, out: [M, N] bfloat16 or float32.  K % 8 == 0.
// fuse_act < 0: plain product.  fuse_act = 0 (silu) or 1 (gelu_tanh): w is [2 * N_out, K] (gate rows first),
// out is [M, N_out] = act(x gate^T) * (x up^T), N = 2 * N_out.
// in_sumsq (may be null): x is a prenormed input, a residual stream times a norm weight; the sums of token m are
// multiplied by 1 / sqrt(sum of in_sumsq[m * in_ld + 0 .. in_parts) / in_width + in_eps) first.
LMSF_API int lmsf_gemm_skinny(void* out, const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw,
                              long long ldo, int fuse_act, int out_f32, const float* in_sumsq, int in_parts,
                              long long in_ld, float in_eps, int in_width, void* stream) {
  using namespace lmsf;
  using namespace lmsf::skinny;
  Args a{};
  a.x = (const bf16*)x; a.ldx = ldx; a.w = (const bf16*)w; a.ldw = ldw; a.out = out; a.ldo = ldo; a.M = M; a.N = N; a.K = K;
  a.out_f32 = out_f32;
  a.in_sumsq = in_sumsq; a.in_parts = in_parts; a.in_ld = in_ld; a.in_eps = in_eps; a.in_width = in_width;
  return run_product(a, fuse_act, (cudaStream_t)stream);
}

// How many partial sums of squares per token the residual form leaves for N output features.
LMSF_API int lmsf_gemm_skinny_residual_parts(int N) { return (N + 15) / 16; }

// The residual form: res[M, N] (float32) += bfloat16(x w^T); out[M, N] (bfloat16) = res * norm_w (norm_w: [N], float32
// or bfloat16); out_sumsq[m * out_ld + b], b < lmsf_gemm_skinny_residual_parts(N): the sums of squares of token m's
// new residual values, 16 features each.  What a product, a residual add and the first half of an RMSNorm would do.
LMSF_API int lmsf_gemm_skinny_residual(void* out, long long ldo, const void* x, long long ldx, const void* w, long long ldw,
                                       int M, int N, int K, float* res, long long ldres, const void* norm_w,
                                       int norm_w_f32, float* out_sumsq, long long out_ld, void* stream) {
  using namespace lmsf;
  using namespace lmsf::skinny;
  if (!res || !norm_w || !out_sumsq || !out) LMSF_REFUSE("gemm_skinny_residual: a buffer is missing");
  if (ldres < N || out_ld < (N + 15) / 16) LMSF_REFUSE("gemm_skinny_residual: a row of the residual or of the sums is too short");
  Args a{};
  a.x = (const bf16*)x; a.ldx = ldx; a.w = (const bf16*)w; a.ldw = ldw; a.out = out; a.ldo = ldo; a.M = M; a.N = N; a.K = K;
  a.res = res; a.ldres = ldres; a.norm_w = norm_w; a.norm_w_f32 = norm_w_f32; a.out_sumsq = out_sumsq; a.out_ld = out_ld;
  return run_product(a, -1, (cudaStream_t)stream);
}

// The merged q, k, v projection of M <= 16 single tokens with the rotary encoding and the cache write in its
// epilogue.  w: [(n_q_heads + 2 n_kv_heads) * head_dim, K]; q_out: [M, n_q_heads * head_dim] bfloat16, rotated;
// k (rotated) and v go to the pages of `cache` ([page][2][kv_head][slot][head_dim]) that block_table names for
// positions[m] of request token_seq[m].  inv_freq: [rot_dim / 2] float32 or null (no rotation).  Results are those
// of lmsf_gemm_skinny (bfloat16 out) followed by the rotary / cache-write kernel, bit for bit.  in_sumsq: as there.
LMSF_API int lmsf_gemm_skinny_qkv_rope(void* q_out, long long ldq, const void* x, long long ldx, const void* w, long long ldw,
                                       int M, int K, const int* positions, const int* token_seq, const int* block_table,
                                       int max_blocks, int block_size, void* cache, long long page_stride,
                                       const float* inv_freq, int rot_dim, int is_neox, int n_q_heads, int n_kv_heads,
                                       int head_dim, int* error_flag, const float* in_sumsq, int in_parts,
                                       long long in_ld, float in_eps, int in_width, void* stream) {
  using namespace lmsf;
  using namespace lmsf::skinny;
  if (M <= 0) return 0;
  if (M > 16) LMSF_REFUSE("gemm_skinny_qkv_rope: M=%d, this kernel takes at most 16 rows", M);
  if (K <= 0 || K % 8) LMSF_REFUSE("gemm_skinny_qkv_rope: K=%d must be a positive multiple of 8", K);
  if (ldx < K || ldw < K || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    LMSF_REFUSE("gemm_skinny_qkv_rope: the rows of x and w must be 16-byte aligned");
  if (head_dim <= 0 || head_dim % 16 || n_q_heads <= 0 || n_kv_heads <= 0)
    LMSF_REFUSE("gemm_skinny_qkv_rope: head_dim=%d must be a multiple of 16", head_dim);
  if (inv_freq && (rot_dim <= 0 || rot_dim > head_dim || rot_dim % (is_neox ? 16 : 2)))
    LMSF_REFUSE("gemm_skinny_qkv_rope: rot_dim=%d is not taken (NeoX pairs need a multiple of 16)", rot_dim);
  if (ldq < (long long)n_q_heads * head_dim || block_size <= 0 || max_blocks <= 0 || !cache)
    LMSF_REFUSE("gemm_skinny_qkv_rope: bad q or cache geometry");
  Args a{};
  a.x = (const bf16*)x; a.ldx = ldx; a.w = (const bf16*)w; a.ldw = ldw; a.out = q_out; a.ldo = ldq;
  a.M = M; a.N = (n_q_heads + 2 * n_kv_heads) * head_dim; a.K = K; a.act = -1;
  a.positions = positions; a.token_seq = token_seq; a.block_table = block_table; a.max_blocks = max_blocks;
  a.block_size = block_size; a.cache = (bf16*)cache; a.page_stride = page_stride; a.inv_freq = inv_freq;
  a.rot_dim = inv_freq ? rot_dim : 0; a.is_neox = is_neox; a.n_q_heads = n_q_heads; a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim; a.error_flag = error_flag;
  if (in_sumsq && (in_parts <= 0 || in_ld < in_parts || in_ld % 4 || ((uintptr_t)in_sumsq % 16) || in_width <= 0 || !(in_eps > 0.f)))
    LMSF_REFUSE("gemm_skinny_qkv_rope: the sums of squares of a prenormed input need rows of a multiple of 4 floats, "
                "16-byte aligned, a width and a positive eps");
  a.in_sumsq = in_sumsq; a.in_parts = in_parts; a.in_ld = in_ld; a.in_eps = in_eps; a.in_width = in_width;
  cudaStream_t s = (cudaStream_t)stream;
  return launch_by_blocks<true>(a, a.N, s);
}
