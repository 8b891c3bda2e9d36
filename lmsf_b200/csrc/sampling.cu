// Token sampling from float32 logits: greedy (argmax, lowest index wins ties) and temperature
// sampling as an exponential race, argmax_v(softmax(logits / T)_v / q_v) with q_v ~ Exp(1),
// which is argmax_v(logits_v / T - log q_v).
// Counterparts in the reference: greedy_sample and multinomial in
// core/src/model_executor/layers/sampler.rs:326-384 with the exponential noise of
// tops/csrc/tops/oneflow/kernel/distribution/exponential_distribution.cu:80-155.  Difference: the
// noise is a pure function of (request seed, index of the output token, vocabulary id) through
// Philox-4x32-10, so a draw does not depend on which requests share the batch, on how prompts
// were cut or on a recomputation after preemption.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_sampling)

namespace lmsf {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// -log(q), q = -log(u), u = (r + 1) / 2^32 in (0, 1]
__device__ __forceinline__ double neg_log_exponential(uint32_t seed_lo, uint32_t seed_hi, uint32_t step, uint32_t v) {
  uint32_t r[4];
  philox4x32_10(v, step, 0u, 0u, seed_lo, seed_hi, r);
  const double u = ((double)r[0] + 1.0) * (1.0 / 4294967296.0);
  return -log(-log(u));
}

struct Best { double score; int index; };
__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.score > a.score || (b.score == a.score && b.index < a.index)) return b;
  return a;
}

__device__ __forceinline__ Best block_best(Best b, Best* sh) {
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, b.score, o), __shfl_xor_sync(0xffffffffu, b.index, o)};
    b = better(b, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = b;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  b = lane < nw ? sh[lane] : Best{-INFINITY, 0x7fffffff};
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, b.score, o), __shfl_xor_sync(0xffffffffu, b.index, o)};
    b = better(b, other);
  }
  return b;      // valid in warp 0
}

// gridDim = (rows, parts): block (r, p) scans its share of row r and leaves its best in partial[r][p];
// with parts == 1 it writes out[r] itself.  temperature < 1e-5 selects greedy
// (core/src/common/sampling_params.rs:156-164), which compares the float32 logits as they are.
__global__ void sample_kernel(int* __restrict__ out, Best* __restrict__ partial, const float* __restrict__ logits,
                              long long row_stride, int vocab, const float* __restrict__ temperature,
                              const unsigned long long* __restrict__ seed, const int* __restrict__ step) {
  __shared__ Best sh[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const float T = temperature ? temperature[r] : 0.f;
  const bool greedy = T < 1e-5f;
  const int per = (vocab + gridDim.y - 1) / gridDim.y;
  const int v0 = blockIdx.y * per, v1 = min(vocab, v0 + per);
  Best b{-INFINITY, 0x7fffffff};
  if (greedy) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      const float x = row[v];
      if (x > best) { best = x; arg = v; }      // ascending v per thread: the first of equal values stays
    }
    b = Best{(double)best, arg};
  } else {
    const uint32_t slo = (uint32_t)(seed[r] & 0xffffffffull), shi = (uint32_t)(seed[r] >> 32);
    const uint32_t st = step ? (uint32_t)step[r] : 0u;
    for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      const float x = row[v];
      if (x != x) continue;  // a NaN never wins
      b = better(b, Best{(double)x / (double)T + neg_log_exponential(slo, shi, st, (uint32_t)v), v});
    }
  }
  b = block_best(b, sh);
  if (threadIdx.x == 0) {
    if (gridDim.y == 1) out[r] = b.index == 0x7fffffff ? 0 : b.index;
    else partial[(size_t)r * gridDim.y + blockIdx.y] = b;
  }
}

__global__ void sample_final_kernel(int* __restrict__ out, const Best* __restrict__ partial, int parts) {
  const int r = blockIdx.x;
  Best b{-INFINITY, 0x7fffffff};
  if ((int)threadIdx.x < parts) b = partial[(size_t)r * parts + threadIdx.x];
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, b.score, o), __shfl_xor_sync(0xffffffffu, b.index, o)};
    b = better(b, other);
  }
  if (threadIdx.x == 0) out[r] = b.index == 0x7fffffff ? 0 : b.index;
}

// ---------------------------------------------------------------------------------------------- penalties
// One thread per (row, token) pair that occurs in the row's prompt or output.  Order as in the reference
// (core/src/model_executor/layers/sampler.rs:48-137): repetition first (x > 0 ? x / r : x * r, for tokens of the
// prompt or the output), then x -= frequency * count_in_output, then x -= presence * (count_in_output > 0).
__global__ void penalties_kernel(float* __restrict__ logits, long long row_stride, const int* __restrict__ rows,
                                 const int* __restrict__ tokens, const int* __restrict__ out_counts, int n,
                                 const float* __restrict__ presence, const float* __restrict__ frequency,
                                 const float* __restrict__ repetition) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = rows[i];
  float* p = logits + (size_t)r * row_stride + tokens[i];
  float x = *p;
  const float rep = repetition[r];
  x = x > 0.f ? x / rep : x * rep;
  const int c = out_counts[i];
  x -= frequency[r] * (float)c;
  if (c > 0) x -= presence[r];
  *p = x;
}

// ---------------------------------------------------------------------------------------------- filters
// Order-preserving map of a float to an unsigned key (larger float, larger key).
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float block_sum_f(float v, float* scratch) { return block_sum(v, scratch); }
__device__ __forceinline__ float block_max_f(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Calls f(base + index, value) for every value of the row, the block's threads sharing the work; 16 bytes per load when the
// row is aligned (a thread with one 4-byte load in flight at a time would wait for L2 most of the time).
template <typename F>
__device__ __forceinline__ void for_each_value(const float* __restrict__ row, int vocab, F f, int base = 0) {
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int n4 = vocab >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row);
#pragma unroll 2
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 x = r4[i];
      f(base + 4 * i, x.x);
      f(base + 4 * i + 1, x.y);
      f(base + 4 * i + 2, x.z);
      f(base + 4 * i + 3, x.w);
    }
    for (int v = (n4 << 2) + threadIdx.x; v < vocab; v += blockDim.x) f(base + v, row[v]);
  } else {
    for (int v = threadIdx.x; v < vocab; v += blockDim.x) f(base + v, row[v]);
  }
}

// Block-wide sum of 64-bit integers (any order gives the same sum); the result is valid in every thread.
__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  unsigned long long t = 0ull;
  for (int w = 0; w < nwarps; ++w) t += scratch[w];
  return t;
}

// A row may be shared by the blocks of a thread-block cluster (gridDim.x of them, each with its share of the
// vocabulary); what they count is exchanged through their shared memory.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_addr(const void* local, unsigned rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  return remote;
}
__device__ __forceinline__ unsigned ld_cluster_u32(const unsigned* local, unsigned rank) {
  unsigned v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr(local, rank)) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_cluster_u64(const unsigned long long* local, unsigned rank) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(cluster_addr(local, rank)) : "memory");
  return v;
}

constexpr int kSelBits = 6;                  // key bits settled per pass over the row
constexpr int kSelBins = 1 << kSelBits;
constexpr float kMassOne = 1099511627776.0f; // 2^40: probabilities relative to the largest are summed as integers
constexpr int kCompact = 2048;                // what top-k keeps moves to shared memory when it is at most this many values

// One pass of the selection: among the values that `scan` visits whose key is at least `key_floor` and whose bits above
// (shift + width) equal `prefix`, how many fall into each value of the next `width` bits and (MASS) how much
// probability, as integers, so that the sums do not depend on the order.  Each warp counts into bins of its
// own (lanes of one warp may meet in a bin, warps never), then the warps' bins are added.
template <bool MASS, typename Scan>
__device__ __forceinline__ void select_pass(Scan scan, float invT, float m, uint32_t key_floor,
                                            uint32_t prefix, int shift, int width, unsigned (*w_cnt)[kSelBins],
                                            unsigned long long (*w_mass)[kSelBins], unsigned* cnt, unsigned long long* mass,
                                            unsigned (*x_cnt)[kSelBins], unsigned long long (*x_mass)[kSelBins], int& phase) {
  const int warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  for (int i = threadIdx.x; i < nwarps * kSelBins; i += blockDim.x) {
    w_cnt[0][i] = 0u;
    if (MASS) w_mass[0][i] = 0ull;
  }
  __syncthreads();
  const int top = shift + width;
  const uint32_t dmask = (1u << width) - 1u;
  // a thread sums runs of values that fall into the same bin in registers (in the first passes most values share a
  // few bins) and adds a run to its warp's bins when the bin changes
  uint32_t run_d = 0xffffffffu;
  unsigned run_c = 0u;
  unsigned long long run_m = 0ull;
  auto flush = [&]() {
    if (run_c == 0u) return;
    atomicAdd(&w_cnt[warp][run_d], run_c);
    if (MASS) atomicAdd(&w_mass[warp][run_d], run_m);
  };
  scan([&](int, float x) {
    const float z = x * invT;
    if (z != z) return;
    const uint32_t key = float_key(z);
    if (key < key_floor) return;
    if (top < 32 && (key >> top) != prefix) return;
    const uint32_t d = (key >> shift) & dmask;
    if (d != run_d) {
      flush();
      run_d = d;
      run_c = 0u;
      run_m = 0ull;
    }
    ++run_c;
    if (MASS) run_m += (unsigned long long)(expf(z - m) * kMassOne);
  });
  flush();
  __syncthreads();
  const int R = gridDim.x, par = phase & 1;
  if (threadIdx.x < kSelBins) {
    unsigned c = 0u;
    unsigned long long ms = 0ull;
    for (int w = 0; w < nwarps; ++w) {
      c += w_cnt[w][threadIdx.x];
      if (MASS) ms += w_mass[w][threadIdx.x];
    }
    if (R == 1) {
      cnt[threadIdx.x] = c;
      if (MASS) mass[threadIdx.x] = ms;
    } else {
      x_cnt[par][threadIdx.x] = c;
      if (MASS) x_mass[par][threadIdx.x] = ms;
    }
  }
  if (R > 1) {
    // The blocks' bins are added by every block (integers: the same totals everywhere).  The exchange arrays
    // alternate from pass to pass, so a block that is ahead does not write what a block behind still reads.
    cluster_sync_all();
    if (threadIdx.x < kSelBins) {
      unsigned c = 0u;
      unsigned long long ms = 0ull;
      for (int q = 0; q < R; ++q) {
        c += ld_cluster_u32(&x_cnt[par][threadIdx.x], (unsigned)q);
        if (MASS) ms += ld_cluster_u64(&x_mass[par][threadIdx.x], (unsigned)q);
      }
      cnt[threadIdx.x] = c;
      if (MASS) mass[threadIdx.x] = ms;
    }
    ++phase;
  }
  __syncthreads();
}

// Temperature sampling with top-k, top-p and min-p; a row is served by the blocks of one thread-block cluster
// (gridDim.x of them, one when there are many rows).  With z = logits / T:
//   top-k keeps the k largest z (ties at the k-th value are all kept);
//   top-p keeps a token iff the probability mass of the strictly larger kept tokens is < p
//         (the reference removes the ascending prefix whose cumulative mass is <= 1 - p,
//         core/src/model_executor/layers/sampler.rs:139-210: the same set when values are distinct);
//   min-p keeps z >= max z + log(min_p) (sampler.rs:305-312);
// and the token is drawn among the kept ones by the exponential race of sample_kernel.
// A value's order-preserving 32-bit key is settled six bits per pass over the row (six passes for a threshold
// instead of the 32 of a bisection): the pass counts, for every value of the next six bits, the values (and their
// probability) under the prefix found so far.  Counts and probabilities are integers, so the kept set, and with
// it the draw, is reproducible.  When top-k leaves at most kCompact values they move to shared memory, and the top-p
// passes and the draw visit only those.
__global__ void __launch_bounds__(1024) sample_filtered_kernel(int* __restrict__ out, const float* __restrict__ logits, long long row_stride,
                                       int vocab, const float* __restrict__ temperature,
                                       const unsigned long long* __restrict__ seed, const int* __restrict__ step,
                                       const int* __restrict__ top_k, const float* __restrict__ top_p,
                                       const float* __restrict__ min_p, const int* __restrict__ row_ids) {
  __shared__ float scratch[33];
  __shared__ unsigned long long scratch64[32];
  __shared__ Best sh[32];
  __shared__ unsigned w_cnt[32][kSelBins];
  __shared__ unsigned long long w_mass[32][kSelBins];
  __shared__ unsigned cnt[kSelBins];
  __shared__ unsigned long long mass[kSelBins];
  __shared__ float c_val[kCompact];          // the values that top-k keeps, when they are few, and their places
  __shared__ int c_idx[kCompact];
  __shared__ int c_n;
  __shared__ unsigned x_cnt[2][kSelBins];    // what the blocks of a cluster exchange, alternating from one exchange to the next
  __shared__ unsigned long long x_mass[2][kSelBins];
  __shared__ unsigned long long x_scalar[2][2];
  const int r = row_ids ? row_ids[blockIdx.y] : blockIdx.y;
  const int R = gridDim.x, rank = blockIdx.x;                    // the blocks that share the row, and this one among them
  int phase = 0;                             // exchanges so far (the same in every block of the cluster)
  const int per = (((vocab + R - 1) / R) + 3) & ~3;             // a share starts at a multiple of 4 values
  const int v0 = min(vocab, rank * per), n_mine = min(vocab, v0 + per) - v0;
  const float* row_all = logits + (size_t)r * row_stride;
  const float* row = row_all + v0;           // this block's share of the row
  const float T = temperature[r];
  const float invT = 1.0f / T;
  const int k = top_k ? top_k[r] : -1;
  const float p = top_p ? top_p[r] : 1.0f;
  const float mp = min_p ? min_p[r] : 0.0f;

  float m = -INFINITY;
  for_each_value(row, n_mine, [&](int, float x) {
    const float z = x * invT;
    if (z == z) m = fmaxf(m, z);
  });
  m = block_max_f(m, scratch);
  if (R > 1) {
    if (threadIdx.x == 0) x_scalar[phase & 1][0] = (unsigned long long)__float_as_uint(m);
    cluster_sync_all();
    for (int q = 0; q < R; ++q) m = fmaxf(m, __uint_as_float((unsigned)ld_cluster_u64(&x_scalar[phase & 1][0], (unsigned)q)));
    ++phase;
  }

  // what the later passes visit: the whole row, or (after top-k has left few values) those values in shared memory
  bool compact = false;
  auto scan = [&](auto f) {
    if (compact) {
      for (int i = threadIdx.x; i < c_n; i += blockDim.x) f(c_idx[i], c_val[i]);
    } else {
      for_each_value(row, n_mine, f, v0);
    }
  };
  uint32_t key_min = 0u;                     // tokens with key >= key_min are kept
  if (k > 0 && k < vocab) {                  // the key of the k-th largest value
    uint32_t prefix = 0u;
    unsigned above = 0u;                     // values whose settled bits are larger than the prefix's
    unsigned kept = 0u;                      // values with key >= the prefix (at the end: what top-k keeps)
    bool enough = true;
    for (int shift = 32 - kSelBits; enough; shift = shift >= kSelBits ? shift - kSelBits : 0) {
      const int width = shift == 0 && (32 % kSelBits) ? 32 % kSelBits : kSelBits;
      select_pass<false>(scan, invT, m, 0u, prefix, shift, width, w_cnt, w_mass, cnt, mass, x_cnt, x_mass, phase);
      unsigned c = above;
      int d = (1 << width) - 1;
      for (; d >= 0; --d) {
        if (c + cnt[d] >= (unsigned)k) break;
        c += cnt[d];
      }
      if (d < 0) { enough = false; break; }  // fewer than k values in all: everything is kept
      above = c;
      kept = c + cnt[d];
      prefix = (prefix << width) | (uint32_t)d;
      if (shift == 0) break;
    }
    key_min = enough ? prefix : 0u;
    if (enough && kept <= (unsigned)kCompact) {
      // the kept values move to shared memory (in any order: what follows sums integers and breaks ties by place)
      if (threadIdx.x == 0) c_n = 0;
      __syncthreads();
      for_each_value(row, n_mine, [&](int v, float x) {
        const float z = x * invT;
        if (z == z && float_key(z) >= key_min) {
          const int i = atomicAdd(&c_n, 1);
          if (i < kCompact) {
            c_val[i] = x;
            c_idx[i] = v;
          }
        }
      }, v0);
      __syncthreads();
      compact = true;
    }
  }
  if (p < 1.0f) {
    unsigned long long Z = 0ull;
    scan([&](int, float x) {
      const float z = x * invT;
      if (z == z && float_key(z) >= key_min) Z += (unsigned long long)(expf(z - m) * kMassOne);
    });
    Z = block_sum_u64(Z, scratch64);
    if (R > 1) {
      if (threadIdx.x == 0) x_scalar[phase & 1][0] = Z;
      cluster_sync_all();
      Z = 0ull;
      for (int q = 0; q < R; ++q) Z += ld_cluster_u64(&x_scalar[phase & 1][0], (unsigned)q);
      ++phase;
    }
    const unsigned long long target = (unsigned long long)((double)p * (double)Z);   // kept iff mass of strictly larger keys < p * Z
    // the smallest key of a kept token: the lowest value that still has less than the target above it
    uint32_t prefix = 0u;
    unsigned long long above = 0ull;         // probability of the values whose settled bits are larger than the prefix's
    for (int shift = 32 - kSelBits;; shift = shift >= kSelBits ? shift - kSelBits : 0) {
      const int width = shift == 0 && (32 % kSelBits) ? 32 % kSelBits : kSelBits;
      select_pass<true>(scan, invT, m, key_min, prefix, shift, width, w_cnt, w_mass, cnt, mass, x_cnt, x_mass, phase);
      unsigned long long a_run = above, a_best = above;
      int best = -1;
      for (int d = (1 << width) - 1; d >= 0; --d) {
        if (cnt[d] > 0u) {
          if (a_run < target || best < 0) { best = d; a_best = a_run; }   // (the largest value is always kept)
          else break;
        }
        a_run += mass[d];
      }
      if (best < 0) break;                   // no value at all (every logit NaN)
      above = a_best;
      prefix = (prefix << width) | (uint32_t)best;
      if (shift == 0) { key_min = prefix; break; }
    }
  }
  if (mp > 0.0f) {
    const uint32_t kmp = float_key(m + logf(mp));
    if (kmp > key_min) key_min = kmp;
  }

  const uint32_t slo = (uint32_t)(seed[r] & 0xffffffffull), shi = (uint32_t)(seed[r] >> 32);
  const uint32_t st = (uint32_t)step[r];
  Best b{-INFINITY, 0x7fffffff};
  scan([&](int v, float x) {
    const float z = x * invT;
    if (z != z || float_key(z) < key_min) return;
    b = better(b, Best{(double)x / (double)T + neg_log_exponential(slo, shi, st, (uint32_t)v), v});
  });
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, b.score, o), __shfl_xor_sync(0xffffffffu, b.index, o)};
    b = better(b, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = b;
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    b = lane < nw ? sh[lane] : Best{-INFINITY, 0x7fffffff};
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, b.score, o), __shfl_xor_sync(0xffffffffu, b.index, o)};
      b = better(b, other);
    }
    if (lane == 0) {
      if (R == 1) {
        out[r] = b.index == 0x7fffffff ? 0 : b.index;
      } else {
        x_scalar[phase & 1][0] = (unsigned long long)__double_as_longlong(b.score);
        x_scalar[phase & 1][1] = (unsigned long long)(unsigned)b.index;
      }
    }
  }
  if (R > 1) {
    cluster_sync_all();
    if (rank == 0 && threadIdx.x == 0) {     // the blocks' winners meet in the first block
      Best w{-INFINITY, 0x7fffffff};
      for (int q = 0; q < R; ++q) {
        const Best o{__longlong_as_double((long long)ld_cluster_u64(&x_scalar[phase & 1][0], (unsigned)q)),
                     (int)(unsigned)ld_cluster_u64(&x_scalar[phase & 1][1], (unsigned)q)};
        w = better(w, o);
      }
      out[r] = w.index == 0x7fffffff ? 0 : w.index;
    }
    cluster_sync_all();                      // no block leaves while the first one still reads its shared memory
  }
}

}  // namespace lmsf

// logits: [rows, vocab] float32; temperature [rows] float32, seed [rows] uint64, step [rows] int32
// (all three may be null: greedy).  out: [rows] int32.  A row is scanned by `parts` blocks (1..32); with
// parts > 1, scratch must hold rows * parts * 16 bytes.
LMSF_API int lmsf_sample(int* out, const float* logits, long long row_stride, int rows, int vocab,
                         const float* temperature, const unsigned long long* seed, const int* step, int parts,
                         void* scratch, void* stream) {
  using namespace lmsf;
  if (rows <= 0) return 0;
  if (vocab <= 0 || row_stride < vocab) LMSF_REFUSE("sample: vocab=%d, row_stride=%lld", vocab, row_stride);
  if (parts < 1 || parts > 32) LMSF_REFUSE("sample: parts=%d must be between 1 and 32", parts);
  if (parts > 1 && !scratch) LMSF_REFUSE("sample: %d parts need scratch memory", parts);
  if (temperature && !seed) LMSF_REFUSE("sample: temperature sampling needs seeds");
  const int threads = vocab / parts >= 4096 ? 512 : 256;
  cudaStream_t s = (cudaStream_t)stream;
  sample_kernel<<<dim3(rows, parts), threads, 0, s>>>(out, (Best*)scratch, logits, row_stride, vocab, temperature, seed, step);
  int rc = LMSF_LAUNCH_STATUS();
  if (rc || parts == 1) return rc;
  sample_final_kernel<<<rows, 32, 0, s>>>(out, (const Best*)scratch, parts);
  return LMSF_LAUNCH_STATUS();
}

// logits are changed in place.  rows/tokens/out_counts: [n] int32; presence/frequency/repetition: [n_rows] float32.
LMSF_API int lmsf_apply_penalties(float* logits, long long row_stride, const int* rows, const int* tokens,
                                  const int* out_counts, int n, const float* presence, const float* frequency,
                                  const float* repetition, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  penalties_kernel<<<ceil_div(n, 256), 256, 0, (cudaStream_t)stream>>>(logits, row_stride, rows, tokens, out_counts, n,
                                                                       presence, frequency, repetition);
  return LMSF_LAUNCH_STATUS();
}

// The rows listed in row_ids (null: rows 0 .. n_rows-1) are sampled at their temperature (> 0) among the
// tokens that their top_k (<= 0: off), top_p (1: off) and min_p (0: off) keep; out[row] receives the token.
// All per-row arrays are indexed by row.  top_k, top_p, min_p may be null (off for all rows).
LMSF_API int lmsf_sample_filtered(int* out, const float* logits, long long row_stride, int rows, int vocab,
                                  const float* temperature, const unsigned long long* seed, const int* step,
                                  const int* top_k, const float* top_p, const float* min_p, const int* row_ids,
                                  void* stream) {
  using namespace lmsf;
  if (rows <= 0) return 0;
  if (vocab <= 0 || row_stride < vocab) LMSF_REFUSE("sample_filtered: vocab=%d, row_stride=%lld", vocab, row_stride);
  if (!temperature || !seed || !step) LMSF_REFUSE("sample_filtered: temperature, seed and step are needed");
  if (rows > 65535) LMSF_REFUSE("sample_filtered: %d rows are more than one launch takes (65535)", rows);
  // A row is shared by as many blocks (a thread-block cluster, at most 8) as leaves every row its blocks at once.
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      n_sms = 1;
  }
  int share = n_sms / rows;
  share = share < 1 ? 1 : share > 8 ? 8 : share;
  if (vocab < 4096 * share) share = vocab < 8192 ? 1 : vocab / 4096;      // a share is at least 4096 values
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)share, (unsigned)rows, 1);
  cfg.blockDim = dim3(1024);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)share;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, sample_filtered_kernel, out, logits, row_stride, vocab, temperature, seed, step, top_k,
                                 top_p, min_p, row_ids);
}
