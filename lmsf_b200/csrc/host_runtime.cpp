// Host side of the cache, native: page pools, block tables, state slots, and the layout of a step's batch.
//
// Role of the reference's BlockAllocator / BlockSpaceManager (core/src/sched/block_manager.rs:14-58, :69-347)
// and of the batch preparation in its worker (core/src/worker/model_worker.rs:266-353, :427-505), which are
// native (Rust) there.  Semantics are those documented in lmsf_b200/cache/manager.py, whose classes are thin
// faces of this library:
//   * one pool per group of layers, LIFO reuse (the page given back last is handed out next);
//   * reserve(n) claims pages for the next n positions in every group or in none;
//   * commit(n) counts n positions as cached and, for window groups, gives back the pages that no later
//     query can reach (their table entries become -1);
//   * state slots are claimed at add, released at free; slots claimed since the last take_fresh are "fresh".
// Return codes: 0 ok, -1 out of pages / slots, -2 unknown request, -3 request exists, -4 bad argument,
// -5 page bookkeeping violated (double free, foreign page).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <vector>

#define LMSF_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

struct Pool {
  int n = 0;
  std::vector<int> free_list;    // taken from the back, returned to the back
  std::vector<char> is_free;
  int allocate() {
    if (free_list.empty()) return -1;
    const int b = free_list.back();
    free_list.pop_back();
    is_free[b] = 0;
    return b;
  }
  int release(int b) {
    if (b < 0 || b >= n) return -5;
    if (is_free[b]) return -5;
    is_free[b] = 1;
    free_list.push_back(b);
    return 0;
  }
};

struct Request {
  std::vector<std::vector<int>> tables;   // per group; -1 where a window has passed
  int num_tokens = 0;                     // positions whose keys are cached
  int num_reserved = 0;                   // positions that have pages
  int slot = -1;
};

struct Manager {
  std::vector<int> windows;               // per group, <= 0: all keys
  std::vector<Pool> pools;
  int block_size = 16;
  int n_slots = 0;
  std::vector<int> free_slots, fresh_slots;
  std::unordered_map<int64_t, Request> reqs;

  int entries_for(int tokens) const { return (tokens + block_size - 1) / block_size; }
  int first_needed_entry(int g, int start) const {
    const int w = windows[g];
    if (w <= 0) return 0;
    return std::max(0, start - w + 1) / block_size;
  }
};

Manager* M(void* h) { return static_cast<Manager*>(h); }

int pages_needed(const Manager& m, const Request& r, int n, int g) {
  return std::max(0, m.entries_for(r.num_reserved + n) - (int)r.tables[g].size());
}

}  // namespace

LMSF_HOST_API void* lmsf_cm_create(int n_groups, const int* windows, const int* num_blocks, int block_size, int n_slots) {
  if (n_groups < 0 || block_size <= 0 || n_slots < 0) return nullptr;
  for (int g = 0; g < n_groups; ++g)
    if (num_blocks[g] <= 0) return nullptr;
  Manager* m = new Manager();
  m->block_size = block_size;
  m->n_slots = n_slots;
  m->windows.assign(windows, windows + n_groups);
  m->pools.resize(n_groups);
  for (int g = 0; g < n_groups; ++g) {
    Pool& p = m->pools[g];
    p.n = num_blocks[g];
    p.is_free.assign(p.n, 1);
    p.free_list.resize(p.n);
    for (int i = 0; i < p.n; ++i) p.free_list[i] = p.n - 1 - i;   // page 0 is handed out first
  }
  for (int s = n_slots - 1; s >= 0; --s) m->free_slots.push_back(s);
  return m;
}

LMSF_HOST_API void lmsf_cm_destroy(void* h) { delete M(h); }

LMSF_HOST_API int lmsf_cm_has(void* h, int64_t rid) { return M(h)->reqs.count(rid) ? 1 : 0; }
LMSF_HOST_API int lmsf_cm_can_add(void* h) { return M(h)->free_slots.empty() ? 0 : 1; }

// Returns the state slot (>= 0) or an error code.
LMSF_HOST_API int lmsf_cm_add(void* h, int64_t rid) {
  Manager& m = *M(h);
  if (m.reqs.count(rid)) return -3;
  if (m.free_slots.empty()) return -1;
  const int slot = m.free_slots.back();
  m.free_slots.pop_back();
  m.fresh_slots.push_back(slot);
  Request r;
  r.tables.resize(m.pools.size());
  r.slot = slot;
  m.reqs.emplace(rid, std::move(r));
  return slot;
}

LMSF_HOST_API int lmsf_cm_free(void* h, int64_t rid) {
  Manager& m = *M(h);
  auto it = m.reqs.find(rid);
  if (it == m.reqs.end()) return -2;
  Request& r = it->second;
  int rc = 0;
  for (size_t g = 0; g < r.tables.size(); ++g)
    for (auto b = r.tables[g].rbegin(); b != r.tables[g].rend(); ++b)
      if (*b >= 0 && m.pools[g].release(*b) != 0) rc = -5;
  auto f = std::find(m.fresh_slots.begin(), m.fresh_slots.end(), r.slot);
  if (f != m.fresh_slots.end()) m.fresh_slots.erase(f);
  m.free_slots.push_back(r.slot);
  m.reqs.erase(it);
  return rc;
}

LMSF_HOST_API int lmsf_cm_take_fresh_slots(void* h, int* out, int cap) {
  Manager& m = *M(h);
  const int n = std::min<int>(cap, (int)m.fresh_slots.size());
  std::copy(m.fresh_slots.begin(), m.fresh_slots.begin() + n, out);
  m.fresh_slots.erase(m.fresh_slots.begin(), m.fresh_slots.begin() + n);
  return n;
}

// out[g] = pages that reserve(rid, n) would claim in group g.
LMSF_HOST_API int lmsf_cm_pages_needed(void* h, int64_t rid, int n, int* out) {
  Manager& m = *M(h);
  auto it = m.reqs.find(rid);
  if (it == m.reqs.end()) return -2;
  for (size_t g = 0; g < m.pools.size(); ++g) out[g] = pages_needed(m, it->second, n, (int)g);
  return 0;
}

// 1 if every pool keeps at least `headroom` free pages after reserve(rid, n).
LMSF_HOST_API int lmsf_cm_can_reserve(void* h, int64_t rid, int n, int headroom) {
  Manager& m = *M(h);
  auto it = m.reqs.find(rid);
  if (it == m.reqs.end()) return -2;
  for (size_t g = 0; g < m.pools.size(); ++g)
    if ((int)m.pools[g].free_list.size() - pages_needed(m, it->second, n, (int)g) < headroom) return 0;
  return 1;
}

LMSF_HOST_API int lmsf_cm_reserve(void* h, int64_t rid, int n) {
  Manager& m = *M(h);
  auto it = m.reqs.find(rid);
  if (it == m.reqs.end()) return -2;
  if (n < 0) return -4;
  Request& r = it->second;
  for (size_t g = 0; g < m.pools.size(); ++g)
    if ((int)m.pools[g].free_list.size() < pages_needed(m, r, n, (int)g)) return -1;
  for (size_t g = 0; g < m.pools.size(); ++g) {
    const int k = pages_needed(m, r, n, (int)g);
    for (int i = 0; i < k; ++i) r.tables[g].push_back(m.pools[g].allocate());
  }
  r.num_reserved += n;
  return 0;
}

LMSF_HOST_API int lmsf_cm_commit(void* h, int64_t rid, int n) {
  Manager& m = *M(h);
  auto it = m.reqs.find(rid);
  if (it == m.reqs.end()) return -2;
  Request& r = it->second;
  if (n < 0 || r.num_tokens + n > r.num_reserved) return -4;
  r.num_tokens += n;
  int rc = 0;
  for (size_t g = 0; g < m.pools.size(); ++g) {
    if (m.windows[g] <= 0) continue;
    const int first = std::min<int>(m.first_needed_entry((int)g, r.num_tokens), (int)r.tables[g].size());
    for (int i = 0; i < first; ++i)
      if (r.tables[g][i] >= 0) {
        if (m.pools[g].release(r.tables[g][i]) != 0) rc = -5;
        r.tables[g][i] = -1;
      }
  }
  return rc;
}

LMSF_HOST_API int lmsf_cm_rollback(void* h, int64_t rid) {
  Manager& m = *M(h);
  auto it = m.reqs.find(rid);
  if (it == m.reqs.end()) return -2;
  Request& r = it->second;
  const int entries = m.entries_for(r.num_tokens);
  int rc = 0;
  for (size_t g = 0; g < m.pools.size(); ++g)
    while ((int)r.tables[g].size() > entries) {
      const int b = r.tables[g].back();
      r.tables[g].pop_back();
      if (b >= 0 && m.pools[g].release(b) != 0) rc = -5;
    }
  r.num_reserved = r.num_tokens;
  return rc;
}

// what = 0: num_tokens, 1: num_reserved, 2: state slot, 3: length of the table of group `g`
LMSF_HOST_API int lmsf_cm_query(void* h, int64_t rid, int what, int g) {
  Manager& m = *M(h);
  auto it = m.reqs.find(rid);
  if (it == m.reqs.end()) return -2;
  const Request& r = it->second;
  switch (what) {
    case 0: return r.num_tokens;
    case 1: return r.num_reserved;
    case 2: return r.slot;
    case 3: return (g >= 0 && g < (int)r.tables.size()) ? (int)r.tables[g].size() : -4;
    default: return -4;
  }
}

LMSF_HOST_API int lmsf_cm_table(void* h, int64_t rid, int g, int* out, int cap) {
  Manager& m = *M(h);
  auto it = m.reqs.find(rid);
  if (it == m.reqs.end()) return -2;
  if (g < 0 || g >= (int)it->second.tables.size()) return -4;
  const auto& t = it->second.tables[g];
  const int n = std::min<int>(cap, (int)t.size());
  std::copy(t.begin(), t.begin() + n, out);
  return (int)t.size();
}

LMSF_HOST_API int lmsf_cm_num_free(void* h, int g) { return (int)M(h)->pools[g].free_list.size(); }
LMSF_HOST_API int lmsf_cm_num_total(void* h, int g) { return M(h)->pools[g].n; }
LMSF_HOST_API int lmsf_cm_num_live(void* h) { return (int)M(h)->reqs.size(); }
LMSF_HOST_API int lmsf_cm_live(void* h, int64_t* out, int cap) {
  int i = 0;
  for (auto& kv : M(h)->reqs) {
    if (i >= cap) break;
    out[i++] = kv.first;
  }
  return i;
}

// 0 when no page or slot is lost, held twice, or both free and held; else 1..4 names the fault.
LMSF_HOST_API int lmsf_cm_check(void* h) {
  Manager& m = *M(h);
  for (size_t g = 0; g < m.pools.size(); ++g) {
    const Pool& p = m.pools[g];
    std::vector<int> seen(p.n, 0);
    int held = 0;
    for (auto& kv : m.reqs)
      for (int b : kv.second.tables[g])
        if (b >= 0) {
          if (b >= p.n || seen[b]++) return 1;       // a page is held twice
          ++held;
        }
    std::vector<int> fr(p.n, 0);
    for (int b : p.free_list) {
      if (fr[b]++) return 2;                          // twice in the free list
      if (seen[b]) return 3;                          // both free and held
    }
    if (held + (int)p.free_list.size() != p.n) return 4;   // pages are lost
  }
  std::vector<int> slots(m.n_slots, 0);
  for (auto& kv : m.reqs)
    if (kv.second.slot < 0 || kv.second.slot >= m.n_slots || slots[kv.second.slot]++) return 5;
  for (int s : m.free_slots)
    if (slots[s]++) return 5;
  if ((int)m.reqs.size() + (int)m.free_slots.size() != m.n_slots) return 5;
  return 0;
}

// ------------------------------------------------------------------------------------------------ a step's batch
// Lays the batch out in one int32 buffer; every segment starts on a 16-byte boundary.  Segment order (the
// offsets and lengths are returned in seg[2 * i], seg[2 * i + 1]):
//   0 token_ids[N]  1 positions[N]  2 token_seq[N]  3 cu_q[S+1]  4 ctx_len[S]  5 state_slot[S]  6 patch_dst[S]
//   7 patch_src[S]  8 rows[R]  9 dec_ids[n_dec]  10 tile_seq[T64]  11 tile_q0[T64]  12 tile128_seq[T128]
//   13 tile128_q0[T128]  14.. block table of group g [S * max_blocks[g]]
// info: 0 N, 1 R, 2 n_dec, 3 T64, 4 T128, 5 has_patches, 6 total ints, 7.. max_blocks per group.
// With pad_to > S the batch is filled up to pad_to requests with stand-ins that bring one token (id 0 at
// position 0), whose block tables name null_pages[g], a page outside the pools, and whose state slot is n_slots,
// one past the slots of real requests (the state tensors have that row to spare): a decode batch can then be
// replayed from a graph captured for a rounder size.  Their logits rows come after the real ones.
// With out == nullptr only the sizes are computed.  Returns 0, -2 for an unknown request, -4 when cap is too small.
LMSF_HOST_API int lmsf_cm_build_batch(void* h, int S, const int64_t* rids, const int* q_lens, const int* tokens_flat,
                                      const int* want_counts, const int* want_flat, const int* last_from,
                                      int static_blocks, int q_tile, int pad_to, const int* null_pages, int* out,
                                      long long cap, int* seg, int* info, int* ctx_lens_out) {
  Manager& m = *M(h);
  const int G = (int)m.pools.size();
  const int n_real = S;
  const int n_pad = pad_to > S ? pad_to - S : 0;
  std::vector<const Request*> rq(S);
  long long N = n_pad, R = n_pad;
  int n_dec = n_pad, t64 = 0, t128 = 0, has_patches = 0;
  std::vector<int> max_blocks(G, std::max(static_blocks, 1));
  for (int s = 0; s < S; ++s) {
    auto it = m.reqs.find(rids[s]);
    if (it == m.reqs.end()) return -2;
    rq[s] = &it->second;
    N += q_lens[s];
    R += want_counts[s];
    if (q_lens[s] == 1) ++n_dec;
    else { t64 += (q_lens[s] + q_tile - 1) / q_tile; t128 += (q_lens[s] + 2 * q_tile - 1) / (2 * q_tile); }
    if (last_from[s] >= 0) has_patches = 1;
    for (int g = 0; g < G; ++g) max_blocks[g] = std::max<int>(max_blocks[g], (int)rq[s]->tables[g].size());
  }
  auto align4 = [](long long n) { return (std::max<long long>(n, 1) + 3) / 4 * 4; };
  S += n_pad;                                   // from here on S counts the stand-ins too
  const long long lens[14] = {N, N, N, S + 1, S, S, S, S, R, n_dec, t64, t64, t128, t128};
  long long total = 0;
  for (int i = 0; i < 14; ++i) { seg[2 * i] = (int)total; seg[2 * i + 1] = (int)lens[i]; total += align4(lens[i]); }
  for (int g = 0; g < G; ++g) {
    seg[2 * (14 + g)] = (int)total;
    seg[2 * (14 + g) + 1] = S * max_blocks[g];
    total += align4((long long)S * max_blocks[g]);
  }
  info[0] = (int)N; info[1] = (int)R; info[2] = n_dec; info[3] = t64; info[4] = t128; info[5] = has_patches;
  info[6] = (int)total;
  for (int g = 0; g < G; ++g) info[7 + g] = max_blocks[g];
  if (out == nullptr) return 0;
  if (total > cap) return -4;
  std::fill(out, out + total, -1);
  int* token_ids = out + seg[0]; int* positions = out + seg[2]; int* token_seq = out + seg[4];
  int* cu_q = out + seg[6]; int* ctx_len = out + seg[8]; int* state_slot = out + seg[10];
  int* patch_dst = out + seg[12]; int* patch_src = out + seg[14]; int* rows = out + seg[16]; int* dec_ids = out + seg[18];
  int* tile_seq = out + seg[20]; int* tile_q0 = out + seg[22]; int* tile128_seq = out + seg[24]; int* tile128_q0 = out + seg[26];
  std::memcpy(token_ids, tokens_flat, sizeof(int) * (N - n_pad));
  int off = 0, r = 0, w = 0, d = 0, a = 0, b = 0;
  cu_q[0] = 0;
  for (int s = 0; s < n_real; ++s) {
    const int n = q_lens[s], start = rq[s]->num_tokens;
    for (int i = 0; i < n; ++i) { positions[off + i] = start + i; token_seq[off + i] = s; }
    cu_q[s + 1] = off + n;
    ctx_len[s] = start + n;
    ctx_lens_out[s] = start + n;
    state_slot[s] = rq[s]->slot;
    patch_dst[s] = last_from[s] >= 0 ? off + n - 1 : -1;
    patch_src[s] = last_from[s] >= 0 ? last_from[s] : 0;
    for (int i = 0; i < want_counts[s]; ++i) rows[r++] = off + want_flat[w++];
    if (n == 1) dec_ids[d++] = s;
    else {
      for (int q0 = 0; q0 < n; q0 += q_tile) { tile_seq[a] = s; tile_q0[a++] = q0; }
      for (int q0 = 0; q0 < n; q0 += 2 * q_tile) { tile128_seq[b] = s; tile128_q0[b++] = q0; }
    }
    for (int g = 0; g < G; ++g) {
      int* bt = out + seg[2 * (14 + g)] + (long long)s * max_blocks[g];
      const auto& t = rq[s]->tables[g];
      std::copy(t.begin(), t.end(), bt);
    }
    off += n;
  }
  // Query tiles in the order of the keys they see, most first: the kernels start blocks in list order, and a
  // prompt's last tiles are its longest.
  auto sort_tiles = [&](int* tseq, int* tq0, int count, int tile) {
    std::vector<int> idx(count), key(count);
    for (int i = 0; i < count; ++i) {
      idx[i] = i;
      const int sq = tseq[i];
      key[i] = rq[sq]->num_tokens + std::min(tq0[i] + tile, q_lens[sq]);
    }
    std::stable_sort(idx.begin(), idx.end(), [&](int x, int y) { return key[x] > key[y]; });
    std::vector<int> a2(count), b2(count);
    for (int i = 0; i < count; ++i) { a2[i] = tseq[idx[i]]; b2[i] = tq0[idx[i]]; }
    std::copy(a2.begin(), a2.end(), tseq);
    std::copy(b2.begin(), b2.end(), tq0);
  };
  sort_tiles(tile_seq, tile_q0, a, q_tile);
  sort_tiles(tile128_seq, tile128_q0, b, 2 * q_tile);
  for (int s = n_real; s < S; ++s) {            // stand-ins
    token_ids[off] = 0; positions[off] = 0; token_seq[off] = s;
    cu_q[s + 1] = off + 1;
    ctx_len[s] = 1;
    ctx_lens_out[s] = 1;
    state_slot[s] = m.n_slots;                  // the spare slot behind the real ones: no request's state
    patch_dst[s] = -1; patch_src[s] = 0;
    rows[r++] = off;
    dec_ids[d++] = s;
    for (int g = 0; g < G; ++g) out[seg[2 * (14 + g)] + (long long)s * max_blocks[g]] = null_pages[g];
    off += 1;
  }
  return 0;
}

// ------------------------------------------------------------------------------------------------ the scheduler
// Role of the reference's Scheduler (core/src/sched/scheduler.rs:336-543, native there): it owns the waiting and
// running queues and decides every step what runs.  The policy is documented in lmsf_b200/engine/scheduler.py, whose
// class is a face of this code:
//   * running requests first, oldest first: one token for a request that decodes, the next portion of its prompt
//     otherwise, under the token budget; then admissions from the waiting queue, first come first served;
//   * a running request that cannot get its pages preempts the youngest running request (pages given back, it
//     returns to the FRONT of the waiting queue and is recomputed later); alone and still too large, it ends;
//   * admission keeps a watermark of 1 % of the pages free, except into an idle engine; nothing is admitted in a step
//     that preempted; a prompt beyond max_model_len or the cache's size is ignored;
//   * a portion that a windowed group could never hold at once is halved until it fits.
// What the scheduler knows of a request is told before every step (lmsf_sched_update): its length (tokens known or
// on their way), how many are cached, how many sampled tokens the host has not read yet, whether it is on hold.
#include <deque>

namespace {

struct SeqState {
  double arrival = 0.0;
  int len = 0, num_computed = 0, num_pending = 0, hold = 0;
};

struct Sched {
  Manager* cm = nullptr;
  int max_tokens = 0, max_seqs = 0, max_model_len = 0;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;
  std::unordered_map<int64_t, SeqState> seqs;
  std::vector<int> watermark;
  long long num_preemptions = 0;
};

Sched* S(void* h) { return static_cast<Sched*>(h); }

void release_request(Sched& s, int64_t rid) {
  if (s.cm->reqs.count(rid)) lmsf_cm_free(s.cm, rid);
}

bool fits_alone(const Sched& s, int num_tokens) {
  const Manager& m = *s.cm;
  for (size_t g = 0; g < m.pools.size(); ++g) {
    const int toks = m.windows[g] <= 0 ? num_tokens : std::min(num_tokens, m.windows[g] + 2 * m.block_size);
    if (m.entries_for(toks) > m.pools[g].n) return false;
  }
  return true;
}

// The portion of n tokens that request rid may run now (see the policy's last point).
int portion_that_fits(const Sched& s, int64_t rid, int n) {
  const Manager& m = *s.cm;
  bool any_window = false;
  for (int w : m.windows) any_window |= w > 0;
  if (!any_window) return n;
  const Request& r = m.reqs.at(rid);
  bool fits_now = true;
  for (size_t g = 0; g < m.pools.size(); ++g)
    if (m.windows[g] > 0 && pages_needed(m, r, n, (int)g) > (int)m.pools[g].free_list.size()) fits_now = false;
  if (fits_now) return n;
  std::vector<int> held(m.pools.size(), 0);
  for (size_t g = 0; g < m.pools.size(); ++g)
    for (int p : r.tables[g]) held[g] += p >= 0;
  auto ok = [&](int k) {
    for (size_t g = 0; g < m.pools.size(); ++g)
      if (m.windows[g] > 0 && pages_needed(m, r, k, (int)g) + held[g] > m.pools[g].n) return false;
    return true;
  };
  while (n > 1 && !ok(n)) n = std::max(1, n / 2);
  return n;
}

}  // namespace

LMSF_HOST_API void* lmsf_sched_create(void* cache_manager, int max_num_batched_tokens, int max_num_seqs, int max_model_len) {
  if (!cache_manager || max_num_batched_tokens <= 0 || max_num_seqs <= 0) return nullptr;
  Sched* s = new Sched();
  s->cm = M(cache_manager);
  s->max_tokens = max_num_batched_tokens;
  s->max_seqs = max_num_seqs;
  s->max_model_len = max_model_len;
  for (const Pool& p : s->cm->pools) s->watermark.push_back((int)std::nearbyint(0.01 * p.n));   // half to even
  return s;
}
LMSF_HOST_API void lmsf_sched_destroy(void* h) { delete S(h); }

// A new request joins the back of the waiting queue.  Returns -3 if the id is already known.
LMSF_HOST_API int lmsf_sched_add(void* h, int64_t rid, double arrival, int len) {
  Sched& s = *S(h);
  if (s.seqs.count(rid)) return -3;
  SeqState st;
  st.arrival = arrival;
  st.len = len;
  s.seqs.emplace(rid, st);
  s.waiting.push_back(rid);
  return 0;
}

// What changed about requests since the last step, for n of them.
LMSF_HOST_API int lmsf_sched_update(void* h, int n, const int64_t* rids, const int* len, const int* num_computed,
                                    const int* num_pending, const int* hold) {
  Sched& s = *S(h);
  for (int i = 0; i < n; ++i) {
    auto it = s.seqs.find(rids[i]);
    if (it == s.seqs.end()) return -2;
    it->second.len = len[i];
    it->second.num_computed = num_computed[i];
    it->second.num_pending = num_pending[i];
    it->second.hold = hold[i];
  }
  return 0;
}

// The request leaves whichever queue holds it (finished or aborted) and gives back what it holds.
// Returns 1 if it was running, 2 if it was waiting, 0 if it was in neither queue.
LMSF_HOST_API int lmsf_sched_remove(void* h, int64_t rid) {
  Sched& s = *S(h);
  int where = 0;
  auto r = std::find(s.running.begin(), s.running.end(), rid);
  if (r != s.running.end()) { s.running.erase(r); where = 1; }
  else {
    auto w = std::find(s.waiting.begin(), s.waiting.end(), rid);
    if (w != s.waiting.end()) { s.waiting.erase(w); where = 2; }
  }
  release_request(s, rid);
  s.seqs.erase(rid);
  return where;
}

// which = 0: the waiting queue, 1: the running queue, in their order.  Returns the queue's length.
LMSF_HOST_API int lmsf_sched_queue(void* h, int which, int64_t* out, int cap) {
  Sched& s = *S(h);
  int i = 0;
  if (which == 0) { for (int64_t r : s.waiting) { if (i < cap) out[i] = r; ++i; } }
  else { for (int64_t r : s.running) { if (i < cap) out[i] = r; ++i; } }
  return i;
}
LMSF_HOST_API long long lmsf_sched_num_preemptions(void* h) { return S(h)->num_preemptions; }
LMSF_HOST_API int lmsf_sched_watermark(void* h, int g) { return S(h)->watermark[g]; }

// One step's decisions.  Entries (request, first position, tokens, whether the portion ends the known tokens so that
// its last place is sampled) go to e_*; requests preempted in this step to pre; requests that end without running
// (kind 0: the prompt can never fit, "ignored") or because they outgrew the cache (kind 1: "length") to ign_*.
// counts: entries, preempted, ignored.  cap: room in every output array (the number of requests known is enough).
// Pages for every entry are reserved in the cache manager.  Returns 0, or -4 when cap is too small.
LMSF_HOST_API int lmsf_sched_schedule(void* h, int cap, int64_t* e_rid, int* e_start, int* e_n, int* e_wants,
                                      int64_t* pre, int64_t* ign_rid, int* ign_kind, int* counts) {
  Sched& s = *S(h);
  Manager& m = *s.cm;
  int ne = 0, np = 0, ni = 0;
  if (cap < (int)s.seqs.size()) return -4;
  int budget = s.max_tokens;
  std::stable_sort(s.running.begin(), s.running.end(),
                   [&](int64_t a, int64_t b) { return s.seqs[a].arrival < s.seqs[b].arrival; });   // age order
  auto preempt = [&](int64_t victim) {
    s.running.erase(std::find(s.running.begin(), s.running.end(), victim));
    release_request(s, victim);
    s.seqs[victim].num_computed = 0;
    s.waiting.push_front(victim);
    pre[np++] = victim;
    ++s.num_preemptions;
  };
  // 1. running requests, oldest first
  size_t i = 0;
  while (i < s.running.size() && budget > 0) {
    const int64_t rid = s.running[i];
    const SeqState st = s.seqs[rid];
    const int uncomputed = st.len - st.num_computed;
    if (st.hold || uncomputed <= 0) { ++i; continue; }        // waits for a token that is still on the device
    const int n = portion_that_fits(s, rid, std::min(uncomputed, budget));
    // only the newest pending token can be taken from the device, and only as a portion's last token
    if (st.num_pending > 1 || (st.num_pending && n < uncomputed)) { ++i; continue; }
    const int lack = st.num_computed + n - m.reqs.at(rid).num_reserved;
    bool gone = false;
    while (lack > 0 && lmsf_cm_can_reserve(&m, rid, lack, 0) != 1) {
      const int64_t victim = s.running.back();
      if (victim == rid && s.running.size() == 1 && !fits_alone(s, st.num_computed + n)) {
        s.running.clear();                                     // alone and still too large for the cache: it ends here
        release_request(s, rid);
        s.seqs.erase(rid);
        ign_rid[ni] = rid;
        ign_kind[ni++] = 1;
        gone = true;
        break;
      }
      preempt(victim);
      if (victim == rid) { gone = true; break; }
    }
    if (gone) continue;
    if (lack > 0 && lmsf_cm_reserve(&m, rid, lack) != 0) return -1;
    e_rid[ne] = rid; e_start[ne] = st.num_computed; e_n[ne] = n; e_wants[ne++] = n == uncomputed;
    budget -= n;
    ++i;
  }
  // 2. admissions, first come first served; nothing is admitted in a step that preempted
  std::vector<int> need(m.pools.size());
  while (!s.waiting.empty() && budget > 0 && np == 0) {
    const int64_t rid = s.waiting.front();
    const SeqState st = s.seqs[rid];
    if (st.num_pending) break;                                 // preempted with a token still on the device: next step
    if (st.len > s.max_model_len || !fits_alone(s, st.len)) {
      s.waiting.pop_front();
      s.seqs.erase(rid);
      ign_rid[ni] = rid;
      ign_kind[ni++] = 0;
      continue;
    }
    if ((int)s.running.size() >= s.max_seqs || m.free_slots.empty()) break;
    if (lmsf_cm_add(&m, rid) < 0) return -1;
    const int uncomputed = st.len - st.num_computed;
    const int n = portion_that_fits(s, rid, std::min(uncomputed, budget));
    lmsf_cm_pages_needed(&m, rid, n, need.data());
    const bool idle = s.running.empty();                       // an empty engine admits its first request without a watermark
    bool room = true;
    for (size_t g = 0; g < m.pools.size(); ++g)
      if ((int)m.pools[g].free_list.size() - need[g] < (idle ? 0 : s.watermark[g])) room = false;
    if (!room) {
      lmsf_cm_free(&m, rid);
      break;
    }
    if (lmsf_cm_reserve(&m, rid, n) != 0) return -1;
    s.waiting.pop_front();
    s.running.push_back(rid);
    e_rid[ne] = rid; e_start[ne] = st.num_computed; e_n[ne] = n; e_wants[ne++] = n == uncomputed;
    budget -= n;
  }
  counts[0] = ne; counts[1] = np; counts[2] = ni;
  return 0;
}
