// The engine's host-side bookkeeping in C++: the page pools, the cache manager, the scheduler's per-step
// decisions and the packed plan of a decode step.  No CUDA here: plain C++17 behind a C ABI, loaded with ctypes
// like the kernel libraries.  The Python classes of the same names (cache/block_pool.py, cache/manager.py,
// engine/scheduler.py, engine/batch.py) define the behaviour; the CPU tests run against both.
//
// In the reference the same pieces are Rust: crates/core/src/kv/block_pool.rs (reference counts, a free list
// in order of use, the hash index), kv/manager.rs (tables per request and group, all-or-nothing allocation),
// sched/mod.rs (the scheduler) and runner.rs:745-876 (the flat batch plan), gated at under 200 us for scheduling
// and updating 1024 decoding requests (crates/core/benches/scheduler.rs:1-5).
//
// Requests are named by 64-bit handles that the caller chooses (the Python side maps its request ids to them).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#define DH_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;
int fail(const char* fmt, long long a = 0, long long b = 0, long long c = 0) {
  char buf[256];
  std::snprintf(buf, sizeof buf, fmt, a, b, c);
  g_error = buf;
  return -1;
}

// ---- content hashes of the prefix cache: 128 bits chained over a page's tokens and the page before it.
// Two multiply-xorshift lanes with different constants; the lanes see each other's state every token.
struct Hash128 {
  uint64_t a = 0, b = 0;
  bool operator==(const Hash128& o) const { return a == o.a && b == o.b; }
};
struct HashOf {
  size_t operator()(const Hash128& h) const { return (size_t)(h.a ^ (h.b * 0x9E3779B97F4A7C15ull)); }
};
inline uint64_t stir(uint64_t z, uint64_t m1, uint64_t m2) {
  z ^= z >> 31; z *= m1; z ^= z >> 29; z *= m2; z ^= z >> 32;
  return z;
}
Hash128 chain_hash(const Hash128& parent, const int32_t* tokens, int n) {
  Hash128 h{parent.a ^ 0x6A09E667F3BCC908ull, parent.b ^ 0xBB67AE8584CAA73Bull};
  for (int i = 0; i < n; ++i) {
    const uint64_t t = (uint64_t)(uint32_t)tokens[i] + ((uint64_t)(i + 1) << 40);
    h.a = stir(h.a + t + (h.b << 7), 0xD6E8FEB86659FD93ull, 0xA0761D6478BD642Full);
    h.b = stir(h.b ^ (t * 0x8EBC6AF09C88C6E3ull) ^ (h.a >> 9), 0xE7037ED1A0B428DBull, 0x589965CC75374CC3ull);
  }
  h.a = stir(h.a ^ (uint64_t)n, 0xD6E8FEB86659FD93ull, 0xA0761D6478BD642Full);
  return h;
}

// ---- a pool of pages
struct Pool {
  int num_blocks = 0;
  std::vector<int> refs, prev, next;
  std::vector<char> on_free, hashed;
  std::vector<Hash128> hash;
  std::unordered_map<Hash128, int, HashOf> cached;
  int head = -1, tail = -1, num_free = 0;
  long long evictions = 0;

  explicit Pool(int n) : num_blocks(n), refs(n, 0), prev(n, -1), next(n, -1), on_free(n, 0), hashed(n, 0), hash(n) {
    for (int b = 0; b < n; ++b) push_tail(b);
  }
  void unlink(int b) {
    if (prev[b] >= 0) next[prev[b]] = next[b]; else head = next[b];
    if (next[b] >= 0) prev[next[b]] = prev[b]; else tail = prev[b];
    prev[b] = next[b] = -1;
    on_free[b] = 0;
    --num_free;
  }
  void push_tail(int b) {
    prev[b] = tail; next[b] = -1;
    if (tail >= 0) next[tail] = b; else head = b;
    tail = b;
    on_free[b] = 1;
    ++num_free;
  }
  void push_head(int b) {
    next[b] = head; prev[b] = -1;
    if (head >= 0) prev[head] = b; else tail = b;
    head = b;
    on_free[b] = 1;
    ++num_free;
  }
  // the head of the free list; a page that carried a hash loses it (its old contents can no longer be found)
  int take() {
    const int b = head;
    unlink(b);
    if (hashed[b]) { cached.erase(hash[b]); hashed[b] = 0; ++evictions; }
    refs[b] = 1;
    return b;
  }
  // one holder lets go; a page without holders joins the free list: at its tail when it carries a hash (found
  // again for as long as possible), at its head otherwise (used again at once)
  int release(int b) {
    if (b < 0 || b >= num_blocks) return fail("block %lld is not of this pool", b);
    if (refs[b] <= 0) return fail("block %lld freed while not held", b);
    if (--refs[b] == 0) { if (hashed[b]) push_tail(b); else push_head(b); }
    return 0;
  }
  void touch(int b) {                     // one more holder of a page found through its hash (it may have been free)
    if (refs[b] == 0) unlink(b);
    ++refs[b];
  }
  bool set_hash(int b, const Hash128& h) {
    if (hashed[b] || cached.count(h)) return false;
    hashed[b] = 1; hash[b] = h; cached.emplace(h, b);
    return true;
  }
  int lookup(const Hash128& h) const {
    auto it = cached.find(h);
    return it == cached.end() ? -1 : it->second;
  }
  int check() const {
    int n = 0;
    for (int b = head, p = -1; b >= 0; p = b, b = next[b], ++n) {
      if (prev[b] != p || !on_free[b] || refs[b] != 0) return fail("page %lld: the free list is broken", b);
      if (n > num_blocks) return fail("the free list has a loop");
    }
    if (n != num_free) return fail("the free list holds %lld pages, the count says %lld", n, num_free);
    for (int b = 0; b < num_blocks; ++b) {
      if ((refs[b] == 0) != (bool)on_free[b]) return fail("page %lld: %lld holders but its free-list mark disagrees", b, refs[b]);
      if (hashed[b] && lookup(hash[b]) != b) return fail("page %lld has a hash the cache does not map to it", b);
    }
    for (auto& kv : cached)
      if (!hashed[kv.second] || !(hash[kv.second] == kv.first)) return fail("the cache maps a hash to page %lld, which does not carry it", kv.second);
    return 0;
  }
};

struct Held {
  std::vector<std::vector<int32_t>> tables;      // per group: page id per block index, -1 = given back
  int num_tokens = 0, num_computed = 0, capacity = 0;
  std::vector<int32_t> tokens;                   // prefix cache: ids of the computed tokens that are known
  std::vector<Hash128> hashes;                   // prefix cache: chained hash per full page so far
  int slot = -1;
  bool fresh = false;
};

struct Manager {
  std::vector<int> windows;                      // per group: 0 = every key is kept
  std::vector<int> block_sizes;                  // per group: tokens a page holds (one size for all with the prefix cache on)
  std::vector<Pool> pools;
  bool prefix = false;
  long long prefix_queries = 0, prefix_hits = 0;
  std::vector<int> free_slots;
  int max_slots = 0;
  std::unordered_map<int64_t, Held> reqs;
  std::vector<int64_t> order;                    // requests in the order they came (what requests() lists)

  Held* find(int64_t r) {
    auto it = reqs.find(r);
    return it == reqs.end() ? nullptr : &it->second;
  }
  int first_needed_block(int g, int num_computed) const {
    if (!windows[g]) return 0;
    return std::max(0, num_computed - windows[g] + 1) / block_sizes[g];
  }
  int need(const Held* h, int g, int total) const {
    const int want = (total + block_sizes[g] - 1) / block_sizes[g];
    const int have = h ? (int)h->tables[g].size() : 0;
    return std::max(0, want - have);
  }
  bool can_allocate(int64_t r, int total) {
    const Held* h = find(r);
    if (!h && free_slots.empty()) return false;
    for (size_t g = 0; g < pools.size(); ++g)
      if (need(h, (int)g, total) > pools[g].num_free) return false;
    return true;
  }
  bool allocate(int64_t r, int total) {
    Held* h = find(r);
    if (h && total <= h->capacity) {             // the usual decode step: room on the last page
      if (total > h->num_tokens) h->num_tokens = total;
      return true;
    }
    if (!can_allocate(r, total)) return false;
    if (!h) {
      Held fresh_one;
      fresh_one.tables.resize(pools.size());
      fresh_one.slot = free_slots.back();
      free_slots.pop_back();
      fresh_one.fresh = true;
      h = &reqs.emplace(r, std::move(fresh_one)).first->second;
      order.push_back(r);
    }
    int cap = 1 << 30;
    for (size_t g = 0; g < pools.size(); ++g) {
      for (int n = need(h, (int)g, total); n > 0; --n) h->tables[g].push_back(pools[g].take());
      cap = std::min(cap, (int)h->tables[g].size() * block_sizes[g]);
    }
    h->capacity = cap;
    h->num_tokens = std::max(h->num_tokens, total);
    return true;
  }
  void hash_full_pages(Held& h) {
    const int block_size = block_sizes[0];         // the same for all groups with the prefix cache on
    const int ready = std::min((int)h.tokens.size(), h.num_computed);
    while (((int)h.hashes.size() + 1) * block_size <= ready) {
      const int i = (int)h.hashes.size();
      const Hash128 parent = i ? h.hashes.back() : Hash128{};
      const Hash128 hh = chain_hash(parent, h.tokens.data() + (size_t)i * block_size, block_size);
      h.hashes.push_back(hh);
      for (size_t g = 0; g < pools.size(); ++g) pools[g].set_hash(h.tables[g][i], hh);
    }
  }
  int release(int64_t r) {
    auto it = reqs.find(r);
    if (it == reqs.end()) return fail("request %lld holds nothing", r);
    Held& h = it->second;
    for (size_t g = 0; g < pools.size(); ++g)
      for (auto p = h.tables[g].rbegin(); p != h.tables[g].rend(); ++p)
        if (*p >= 0 && pools[g].release(*p)) return -1;
    free_slots.push_back(h.slot);
    reqs.erase(it);
    order.erase(std::find(order.begin(), order.end(), r));
    return 0;
  }
};

}  // namespace

DH_API const char* dh_last_error() { return g_error.c_str(); }

// ---- cache manager
DH_API void* dh_manager_new(int n_groups, const int* windows, const int* block_sizes, const int* num_blocks, int max_num_seqs,
                            int prefix_caching) {
  if (n_groups <= 0 || max_num_seqs < 0) { fail("bad sizes"); return nullptr; }
  for (int g = 0; g < n_groups; ++g) {
    if (block_sizes[g] <= 0) { fail("a group's block size must be positive"); return nullptr; }
    if (prefix_caching && block_sizes[g] != block_sizes[0]) { fail("the prefix cache needs one page size for all groups"); return nullptr; }
  }
  auto* m = new Manager();
  m->windows.assign(windows, windows + n_groups);
  m->block_sizes.assign(block_sizes, block_sizes + n_groups);
  for (int g = 0; g < n_groups; ++g) {
    if (num_blocks[g] <= 0) { delete m; fail("a pool needs at least one block"); return nullptr; }
    m->pools.emplace_back(num_blocks[g]);
  }
  m->prefix = prefix_caching != 0;
  m->max_slots = max_num_seqs;
  for (int s = max_num_seqs - 1; s >= 0; --s) m->free_slots.push_back(s);
  return m;
}
DH_API void dh_manager_delete(void* m) { delete static_cast<Manager*>(m); }

DH_API int dh_contains(void* m, int64_t r) { return static_cast<Manager*>(m)->find(r) != nullptr; }
DH_API int dh_num_requests(void* m) { return (int)static_cast<Manager*>(m)->order.size(); }
DH_API int dh_requests(void* m, int64_t* out, int cap) {
  auto& o = static_cast<Manager*>(m)->order;
  const int n = std::min(cap, (int)o.size());
  std::copy(o.begin(), o.begin() + n, out);
  return (int)o.size();
}
DH_API int dh_num_tokens(void* m, int64_t r) { Held* h = static_cast<Manager*>(m)->find(r); return h ? h->num_tokens : fail("request %lld holds nothing", r); }
DH_API int dh_num_computed(void* m, int64_t r) { Held* h = static_cast<Manager*>(m)->find(r); return h ? h->num_computed : fail("request %lld holds nothing", r); }
DH_API int dh_table_len(void* m, int64_t r, int g) { Held* h = static_cast<Manager*>(m)->find(r); return h ? (int)h->tables[g].size() : fail("request %lld holds nothing", r); }
DH_API int dh_table(void* m, int64_t r, int g, int32_t* out, int cap) {
  Held* h = static_cast<Manager*>(m)->find(r);
  if (!h) return fail("request %lld holds nothing", r);
  const auto& t = h->tables[g];
  const int n = std::min(cap, (int)t.size());
  std::copy(t.begin(), t.begin() + n, out);
  return (int)t.size();
}
DH_API int dh_pool_free(void* m, int g) { return static_cast<Manager*>(m)->pools[g].num_free; }
DH_API int dh_pool_blocks(void* m, int g) { return static_cast<Manager*>(m)->pools[g].num_blocks; }
DH_API long long dh_pool_evictions(void* m, int g) { return static_cast<Manager*>(m)->pools[g].evictions; }
DH_API int dh_pool_refcount(void* m, int g, int b) { return static_cast<Manager*>(m)->pools[g].refs[b]; }
DH_API int dh_pool_check(void* m, int g) { return static_cast<Manager*>(m)->pools[g].check(); }
DH_API long long dh_prefix_queries(void* m) { return static_cast<Manager*>(m)->prefix_queries; }
DH_API long long dh_prefix_hits(void* m) { return static_cast<Manager*>(m)->prefix_hits; }
DH_API int dh_slots_free(void* m) { return (int)static_cast<Manager*>(m)->free_slots.size(); }
DH_API int dh_slot(void* m, int64_t r) { Held* h = static_cast<Manager*>(m)->find(r); return h ? h->slot : fail("request %lld holds no slot", r); }
DH_API int dh_take_fresh(void* m, int64_t r) {
  Held* h = static_cast<Manager*>(m)->find(r);
  if (!h) return 0;
  const bool f = h->fresh;
  h->fresh = false;
  return f;
}

DH_API int dh_can_allocate(void* m, int64_t r, int total) { return static_cast<Manager*>(m)->can_allocate(r, total); }
// every (request, total) of a step's batch together; nothing changes
DH_API int dh_can_allocate_all(void* mp, const int64_t* rs, const int* totals, int n) {
  auto* m = static_cast<Manager*>(mp);
  std::vector<int> need(m->pools.size(), 0);
  int fresh = 0;
  for (int i = 0; i < n; ++i) {
    const Held* h = m->find(rs[i]);
    fresh += h == nullptr;
    if (h && totals[i] <= h->capacity) continue;
    for (size_t g = 0; g < m->pools.size(); ++g) need[g] += m->need(h, (int)g, totals[i]);
  }
  if (fresh > (int)m->free_slots.size()) return 0;
  for (size_t g = 0; g < m->pools.size(); ++g)
    if (need[g] > m->pools[g].num_free) return 0;
  return 1;
}
DH_API int dh_allocate(void* m, int64_t r, int total) { return static_cast<Manager*>(m)->allocate(r, total); }

// A request enters with these tokens: take the pages of their longest cached beginning (whole pages, every group,
// never the last token); returns the tokens they cover (0 without the prefix cache, for a request that holds pages
// already, or when no state slot is free).
DH_API int dh_begin(void* mp, int64_t r, const int32_t* tokens, int n) {
  auto* m = static_cast<Manager*>(mp);
  if (!m->prefix || m->find(r)) return 0;
  const int bs = m->block_sizes[0];
  const int limit = (n - 1) / bs;
  m->prefix_queries += n;
  std::vector<Hash128> chain;
  std::vector<std::vector<int32_t>> found(m->pools.size());
  Hash128 parent{};
  for (int i = 0; i < limit; ++i) {
    parent = chain_hash(parent, tokens + (size_t)i * bs, bs);
    bool all = true;
    std::vector<int> pages(m->pools.size());
    for (size_t g = 0; g < m->pools.size(); ++g) { pages[g] = m->pools[g].lookup(parent); all = all && pages[g] >= 0; }
    if (!all) break;
    chain.push_back(parent);
    for (size_t g = 0; g < m->pools.size(); ++g) found[g].push_back(pages[g]);
  }
  const int k = (int)chain.size();
  if (k == 0 || m->free_slots.empty()) return 0;
  Held h;
  h.slot = m->free_slots.back();
  m->free_slots.pop_back();
  h.fresh = true;
  for (size_t g = 0; g < m->pools.size(); ++g)
    for (int b : found[g]) m->pools[g].touch(b);
  h.tables = std::move(found);
  h.num_tokens = h.num_computed = h.capacity = k * bs;
  h.tokens.assign(tokens, tokens + (size_t)k * bs);
  h.hashes = std::move(chain);
  m->reqs.emplace(r, std::move(h));
  m->order.push_back(r);
  m->prefix_hits += (long long)k * bs;
  return k * bs;
}

// The cache now holds the keys of the first `num_computed` tokens: pages every window has passed go back.  With the
// prefix cache, `new_tokens` (n_new of them; null = not told) are the ids of the tokens computed since the last call;
// ids not known yet (negative) may stand at their end.
DH_API int dh_advance(void* mp, int64_t r, int num_computed, const int32_t* new_tokens, int n_new) {
  auto* m = static_cast<Manager*>(mp);
  Held* h = m->find(r);
  if (!h) return fail("request %lld holds nothing", r);
  if (num_computed > h->num_tokens) return fail("request %lld: %lld tokens computed but pages cover %lld", r, num_computed, h->num_tokens);
  if (m->prefix && new_tokens) {
    int known = n_new;
    while (known > 0 && new_tokens[known - 1] < 0) --known;
    for (int i = 0; i < known; ++i)
      if (new_tokens[i] < 0) return fail("request %lld: an unknown token before a known one", r);
    const int behind = (int)h->tokens.size() + n_new - num_computed;
    if (behind > 0 || (behind < 0 && known > 0))
      return fail("request %lld: %lld known + new tokens do not make %lld", r, (long long)h->tokens.size() + n_new, num_computed);
    h->tokens.insert(h->tokens.end(), new_tokens, new_tokens + known);
    h->num_computed = num_computed;
    m->hash_full_pages(*h);
  }
  h->num_computed = num_computed;
  for (size_t g = 0; g < m->pools.size(); ++g) {
    if (!m->windows[g]) continue;
    auto& t = h->tables[g];
    const int stop = std::min(m->first_needed_block((int)g, num_computed), (int)t.size());
    for (int i = 0; i < stop; ++i)
      if (t[i] >= 0) { if (m->pools[g].release(t[i])) return -1; t[i] = -1; }
  }
  return 0;
}
DH_API int dh_resolve(void* mp, int64_t r, const int32_t* tokens, int n) {
  auto* m = static_cast<Manager*>(mp);
  Held* h = m->find(r);
  if (!h || !m->prefix) return 0;
  if ((int)h->tokens.size() + n > h->num_computed) return fail("request %lld: more tokens resolved than were computed", r);
  h->tokens.insert(h->tokens.end(), tokens, tokens + n);
  m->hash_full_pages(*h);
  return 0;
}
DH_API int dh_free(void* m, int64_t r) { return static_cast<Manager*>(m)->release(r); }

// No page lost or held twice: per group, held pages + free pages = the pool; shared pages carry a common hash.
DH_API int dh_check_invariants(void* mp) {
  auto* m = static_cast<Manager*>(mp);
  for (size_t g = 0; g < m->pools.size(); ++g) {
    Pool& pool = m->pools[g];
    std::vector<int> holders(pool.num_blocks, 0);
    for (auto& kv : m->reqs) {
      const auto& t = kv.second.tables[g];
      for (size_t i = 0; i < t.size(); ++i) {
        const int b = t[i];
        if (b < 0) continue;
        if (holders[b] && !m->prefix) return fail("group %lld: page %lld held twice", (long long)g, b);
        if (holders[b] && (i >= kv.second.hashes.size() || !pool.hashed[b] || !(pool.hash[b] == kv.second.hashes[i])))
          return fail("group %lld: page %lld shared without a common hash", (long long)g, b);
        if (pool.refs[b] <= 0) return fail("group %lld: page %lld of request %lld is marked free", (long long)g, b, kv.first);
        ++holders[b];
      }
    }
    int held = 0;
    for (int b = 0; b < pool.num_blocks; ++b) {
      if (holders[b] && pool.refs[b] != holders[b]) return fail("group %lld: page %lld has %lld references", (long long)g, b, pool.refs[b]);
      held += holders[b] > 0;
    }
    if (held + pool.num_free != pool.num_blocks) return fail("group %lld: %lld held + free pages do not make the pool", (long long)g, held);
    if (pool.check()) return -1;
  }
  std::vector<char> used(m->max_slots, 0);
  for (auto& kv : m->reqs) {
    const int s = kv.second.slot;
    if (s < 0 || s >= m->max_slots || used[s]) return fail("a state slot is held twice or out of range");
    used[s] = 1;
  }
  if ((int)m->reqs.size() + (int)m->free_slots.size() != m->max_slots) return fail("state slots and page holders differ");
  return 0;
}

// ---- the packed plan of a decode-only step (the layout of engine/batch.py: PlanBuilder.layout for T = B = R =
// bucket): ids, pos, rows, cu, seq, sslots, fresh, then per group slot and table, each aligned to 4 words.
// `words` points at the plan's int32 words (pinned host memory), written whole: the live rows from the requests'
// tables, the rest as dummy rows (token 0, position 0, no slot, no pages, the spare state slot).
DH_API int dh_decode_plan_fill(void* mp, int32_t* words, int bucket, int width, const int64_t* rs, const int32_t* tokens,
                               const int32_t* starts, int n, int spare_state_slot) {
  auto* m = static_cast<Manager*>(mp);
  if (n > bucket) return fail("more requests than the graph's bucket");
  auto align = [](int x) { return (x + 3) / 4 * 4; };
  const int ng = (int)m->pools.size();
  int off = 0;
  int32_t* ids = words + off; off = align(off + bucket);
  int32_t* pos = words + off; off = align(off + bucket);
  int32_t* rows = words + off; off = align(off + bucket);
  int32_t* cu = words + off; off = align(off + bucket + 1);
  int32_t* seq = words + off; off = align(off + bucket);
  int32_t* sslots = words + off; off = align(off + bucket);
  int32_t* fresh = words + off; off = align(off + bucket);
  std::vector<int32_t*> slot(ng), tab(ng);
  for (int g = 0; g < ng; ++g) {
    slot[g] = words + off; off = align(off + bucket);
    tab[g] = words + off; off = align(off + bucket * width);
  }
  for (int i = 0; i <= bucket; ++i) cu[i] = i;
  for (int i = 0; i < bucket; ++i) rows[i] = i;
  for (int i = 0; i < n; ++i) {
    Held* h = m->find(rs[i]);
    if (!h) return fail("request %lld holds nothing", rs[i]);
    const int p = starts[i];
    ids[i] = tokens[i]; pos[i] = p; seq[i] = p + 1;
    sslots[i] = h->slot; fresh[i] = h->fresh; h->fresh = false;
    for (int g = 0; g < ng; ++g) {
      const auto& t = h->tables[g];
      const int k = std::min((int)t.size(), width);
      int32_t* row = tab[g] + (size_t)i * width;
      std::copy(t.begin(), t.begin() + k, row);
      std::fill(row + k, row + width, -1);
      const int bs = m->block_sizes[g];
      const int blk = p / bs < k ? t[p / bs] : -1;
      slot[g][i] = blk >= 0 ? blk * bs + p % bs : -1;
    }
  }
  for (int i = n; i < bucket; ++i) {
    ids[i] = 0; pos[i] = 0; seq[i] = 1; sslots[i] = spare_state_slot; fresh[i] = 0;
    for (int g = 0; g < ng; ++g) {
      slot[g][i] = -1;
      std::fill(tab[g] + (size_t)i * width, tab[g] + (size_t)(i + 1) * width, -1);
    }
  }
  return off;
}

// ---- the scheduler: continuous batching above the step function (engine/scheduler.py defines the policy: running
// requests first, then waiting ones while the token budget, max_num_seqs and the pages last; prompts cut into
// portions; the LAST running request preempted when pages run out, never the one that asks while others run; a
// request that alone does not fit finished with `length`; nothing admitted in a step that preempted; with
// `lookahead` a request that samples counts as one token longer at once).  crates/core/src/sched/mod.rs:318-828.
namespace {

enum { ST_WAITING = 0, ST_RUNNING = 1, ST_FINISHED = 2 };
enum { FIN_NONE = 0, FIN_STOP = 1, FIN_LENGTH = 2, FIN_ABORT = 3 };

struct Rec {
  int prompt_len = 0;
  std::vector<int32_t> tokens;                   // prompt, then the output tokens the host knows
  int num_computed = 0, placeholders = 0;
  int max_tokens = 0, min_tokens = 0;
  bool ignore_eos = false, every_prompt_row = false;
  std::vector<int32_t> stop_ids;
  int status = ST_WAITING, reason = FIN_NONE, preemptions = 0;
  int n_out() const { return (int)tokens.size() - prompt_len; }
};

struct Sched {
  Manager* m = nullptr;
  int budget = 0, threshold = 0, max_model_len = 0, max_num_seqs = 0;
  bool exempt = true;
  std::vector<int32_t> eos;
  std::unordered_map<int64_t, Rec> recs;
  std::vector<int64_t> waiting, running;         // waiting[0] is the front of the queue
  long long preemptions = 0;

  void finish(int64_t id, Rec& r, int reason) {
    r.status = ST_FINISHED;
    r.reason = reason;
    if (m->find(id)) m->release(id);
  }
  void preempt(int64_t id) {
    Rec& r = recs[id];
    if (m->find(id)) m->release(id);
    r.num_computed = 0;
    r.placeholders = 0;                          // a token in flight is still appended when it arrives (update)
    r.status = ST_WAITING;
    ++r.preemptions;
    ++preemptions;
    waiting.insert(waiting.begin(), id);
  }
  int check_stop(const Rec& r, int tok) const {
    const int n_out = r.n_out();
    if (n_out >= r.min_tokens) {
      if (!r.ignore_eos && std::find(eos.begin(), eos.end(), tok) != eos.end()) return FIN_STOP;
      if (std::find(r.stop_ids.begin(), r.stop_ids.end(), tok) != r.stop_ids.end()) return FIN_STOP;
    }
    if (n_out >= r.max_tokens || (int)r.tokens.size() >= max_model_len) return FIN_LENGTH;
    return FIN_NONE;
  }
};

}  // namespace

DH_API void* dh_sched_new(void* manager, int max_num_batched_tokens, int long_prefill_token_threshold, int max_model_len,
                          int max_num_seqs, int decode_exempt, const int32_t* eos, int n_eos) {
  auto* s = new Sched();
  s->m = static_cast<Manager*>(manager);
  s->budget = max_num_batched_tokens; s->threshold = long_prefill_token_threshold; s->max_model_len = max_model_len;
  s->max_num_seqs = max_num_seqs; s->exempt = decode_exempt != 0;
  s->eos.assign(eos, eos + n_eos);
  return s;
}
DH_API void dh_sched_delete(void* s) { delete static_cast<Sched*>(s); }

DH_API int dh_sched_add(void* sp, int64_t id, const int32_t* prompt, int n, int max_tokens, int min_tokens, int ignore_eos,
                        const int32_t* stop_ids, int n_stop, int every_prompt_row) {
  auto* s = static_cast<Sched*>(sp);
  if (s->recs.count(id)) return fail("request %lld is known already", id);
  Rec r;
  r.prompt_len = n;
  r.tokens.assign(prompt, prompt + n);
  r.max_tokens = max_tokens; r.min_tokens = min_tokens; r.ignore_eos = ignore_eos != 0;
  r.every_prompt_row = every_prompt_row != 0;
  r.stop_ids.assign(stop_ids, stop_ids + n_stop);
  s->recs.emplace(id, std::move(r));
  s->waiting.push_back(id);
  return 0;
}
// a request that is over (finished or aborted) is forgotten
DH_API void dh_sched_forget(void* sp, int64_t id) { static_cast<Sched*>(sp)->recs.erase(id); }
DH_API int dh_sched_abort(void* sp, int64_t id) {
  auto* s = static_cast<Sched*>(sp);
  auto it = s->recs.find(id);
  if (it == s->recs.end() || it->second.status == ST_FINISHED) return 0;
  for (auto* q : {&s->running, &s->waiting}) {
    auto p = std::find(q->begin(), q->end(), id);
    if (p != q->end()) { q->erase(p); s->finish(id, it->second, FIN_ABORT); return 1; }
  }
  return 0;
}
DH_API int dh_sched_counts(void* sp, int* n_waiting, int* n_running) {
  auto* s = static_cast<Sched*>(sp);
  *n_waiting = (int)s->waiting.size(); *n_running = (int)s->running.size();
  return 0;
}
DH_API int dh_sched_queue(void* sp, int which, int64_t* out, int cap) {
  auto& q = which ? static_cast<Sched*>(sp)->running : static_cast<Sched*>(sp)->waiting;
  const int n = std::min(cap, (int)q.size());
  std::copy(q.begin(), q.begin() + n, out);
  return (int)q.size();
}
DH_API long long dh_sched_preemptions(void* sp) { return static_cast<Sched*>(sp)->preemptions; }

// One step's decisions.  Scheduled requests come back as columns (ids, start, num_tokens, samples, num_generated) of
// at most `cap` entries, the preempted and the finished (no fit) as id lists of at most `cap`; counts[0..2] = how
// many of each.  Returns 0, or -1 when `cap` is too small.
DH_API int dh_sched_schedule(void* sp, int lookahead, int cap, int64_t* ids, int32_t* start, int32_t* num,
                             int32_t* samples, int32_t* ngen, int64_t* preempted, int64_t* finished, int32_t* counts) {
  auto* s = static_cast<Sched*>(sp);
  Manager* m = s->m;
  int n_s = 0, n_p = 0, n_f = 0;
  int budget = s->budget;
  auto emit = [&](int64_t id, int st, int n, bool smp, int gen) {
    if (n_s >= cap) return false;
    ids[n_s] = id; start[n_s] = st; num[n_s] = n; samples[n_s] = smp; ngen[n_s] = gen;
    ++n_s;
    return true;
  };
  size_t i = 0;
  while (i < s->running.size()) {
    const int64_t id = s->running[i];
    Rec& r = s->recs[id];
    const int ahead = r.placeholders, n_out = r.n_out();
    const int known = (int)r.tokens.size() + ahead, computed = r.num_computed;
    if (ahead && (n_out + ahead >= r.max_tokens || known >= s->max_model_len)) { ++i; continue; }
    int num_new = known - computed;
    const bool is_decode = num_new == 1 && computed > 0;
    if (s->threshold > 0) num_new = std::min(num_new, s->threshold);
    if (!(is_decode && s->exempt)) num_new = std::min(num_new, budget);
    if (computed + num_new > s->max_model_len) num_new = s->max_model_len - computed;
    if (num_new <= 0) { ++i; continue; }
    bool placed = true, gone = false;
    while (!m->allocate(id, computed + num_new)) {
      const int64_t victim = s->running.back();
      if (victim == id) {
        if (s->running.size() > 1) {
          placed = false;                        // others run: sit this step out, keep the pages
        } else {
          s->running.pop_back();                 // alone and still no fit: it can never finish
          s->finish(id, r, FIN_LENGTH);
          if (n_f >= cap) return fail("the result columns are too short");
          finished[n_f++] = id;
          placed = false; gone = true;
        }
        break;
      }
      s->running.pop_back();
      s->preempt(victim);
      if (n_p >= cap) return fail("the result columns are too short");
      preempted[n_p++] = victim;
    }
    if (!placed) { if (!gone) ++i; continue; }
    if (!emit(id, computed, num_new, computed + num_new == known, n_out + ahead)) return fail("the result columns are too short");
    if (!(is_decode && s->exempt)) budget -= num_new;
    ++i;
  }
  if (n_p == 0) {
    while (!s->waiting.empty() && budget > 0 && (int)s->running.size() < s->max_num_seqs) {
      const int64_t id = s->waiting.front();
      Rec& r = s->recs[id];
      bool began = false;
      if (r.num_computed == 0 && m->prefix && !m->find(id) && !r.every_prompt_row) {
        // pages of an earlier request with the same beginning: those tokens are not run again
        r.num_computed = dh_begin(m, id, r.tokens.data(), (int)r.tokens.size());
        began = r.num_computed > 0;
      }
      int num_new = (int)r.tokens.size() - r.num_computed;
      if (s->threshold > 0) num_new = std::min(num_new, s->threshold);
      num_new = std::min({num_new, budget, s->max_model_len - r.num_computed});
      if (num_new <= 0 || !m->allocate(id, r.num_computed + num_new)) {
        if (began) { m->release(id); r.num_computed = 0; }
        break;
      }
      s->waiting.erase(s->waiting.begin());
      r.status = ST_RUNNING;
      s->running.push_back(id);
      if (!emit(id, r.num_computed, num_new, r.num_computed + num_new == (int)r.tokens.size(), r.n_out()))
        return fail("the result columns are too short");
      budget -= num_new;
    }
  }
  for (int k = 0; k < n_s; ++k) {                // the cache will hold these once the step has run
    Rec& r = s->recs[ids[k]];
    r.num_computed += num[k];
    if (lookahead && samples[k]) ++r.placeholders;
  }
  counts[0] = n_s; counts[1] = n_p; counts[2] = n_f;
  return 0;
}

// After the step: the sampled token of every scheduled request that samples (tokens[k] for entry k; ignored where
// samples[k] is 0) is appended, the stop conditions are checked, what has finished is freed.  done_ids / reasons get
// the requests that finished (at most n); returns how many.
DH_API int dh_sched_update(void* sp, int n, const int64_t* ids, const int32_t* samples, const int32_t* tokens,
                           int64_t* done_ids, int32_t* reasons) {
  auto* s = static_cast<Sched*>(sp);
  int n_done = 0;
  for (int k = 0; k < n; ++k) {
    if (!samples[k]) continue;
    auto it = s->recs.find(ids[k]);
    if (it == s->recs.end() || it->second.status == ST_FINISHED) continue;   // finished meanwhile: dropped
    Rec& r = it->second;
    r.tokens.push_back(tokens[k]);
    const int reason = s->check_stop(r, tokens[k]);
    if (r.status == ST_RUNNING) {
      if (r.placeholders > 0) --r.placeholders;
      if (reason) s->running.erase(std::find(s->running.begin(), s->running.end(), ids[k]));
    } else if (reason) {                         // preempted while this token was in flight, and it ends the request
      s->waiting.erase(std::find(s->waiting.begin(), s->waiting.end(), ids[k]));
    }
    if (reason) {
      s->finish(ids[k], r, reason);
      done_ids[n_done] = ids[k]; reasons[n_done] = reason; ++n_done;
    }
  }
  return n_done;
}

// The same as dh_advance for every request of a step at once (no token ids: not for the prefix cache).
DH_API int dh_advance_many(void* mp, const int64_t* rs, const int32_t* computed, int n) {
  for (int i = 0; i < n; ++i)
    if (dh_advance(mp, rs[i], computed[i], nullptr, 0)) return -1;
  return 0;
}
