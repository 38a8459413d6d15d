// Warm-prefix cache bookkeeping: SHA-256 block-hash chain, the LRU list of
// block-boundary snapshots, page pinning by reference count, and the byte
// budget. Follows BlockHash / BlockAwarePrefixCache (src/serve/cache.rs:11-219)
// and the budget loop of remember_prefix_block (src/serve/state.rs:613-639):
// the same operation trace yields the same hits and the same sequence of
// evicted (session, hash, tokens) keys as the reference's Vec-based LRU.
#include <algorithm>
#include <cstring>

#include "host.h"

namespace sgk {

// ---- SHA-256 (FIPS 180-4); the reference uses the sha2 crate for the same digest ----
static const uint32_t KC[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

namespace {
struct Sha256 {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  uint8_t buf[64];
  size_t fill = 0;
  uint64_t total = 0;
  static uint32_t ror(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void compress(const uint8_t* p) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = uint32_t(p[4 * i]) << 24 | uint32_t(p[4 * i + 1]) << 16 | uint32_t(p[4 * i + 2]) << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      uint32_t s0 = ror(w[i - 15], 7) ^ ror(w[i - 15], 18) ^ (w[i - 15] >> 3);
      uint32_t s1 = ror(w[i - 2], 17) ^ ror(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t v[8];
    std::memcpy(v, h, sizeof(v));
    for (int i = 0; i < 64; ++i) {
      uint32_t t1 = v[7] + (ror(v[4], 6) ^ ror(v[4], 11) ^ ror(v[4], 25)) + ((v[4] & v[5]) ^ (~v[4] & v[6])) + KC[i] + w[i];
      uint32_t t2 = (ror(v[0], 2) ^ ror(v[0], 13) ^ ror(v[0], 22)) + ((v[0] & v[1]) ^ (v[0] & v[2]) ^ (v[1] & v[2]));
      for (int j = 7; j > 0; --j) v[j] = v[j - 1];
      v[4] += t1;
      v[0] = t1 + t2;
    }
    for (int i = 0; i < 8; ++i) h[i] += v[i];
  }
  void update(const uint8_t* data, size_t n) {
    total += n;
    while (n > 0) {
      size_t take = std::min(n, 64 - fill);
      std::memcpy(buf + fill, data, take);
      fill += take;
      data += take;
      n -= take;
      if (fill == 64) {
        compress(buf);
        fill = 0;
      }
    }
  }
  void finish(uint8_t out[32]) {
    uint64_t bits = total * 8;
    uint8_t pad = 0x80;
    update(&pad, 1);
    uint8_t zero = 0;
    while (fill != 56) update(&zero, 1);
    uint8_t lenb[8];
    for (int i = 0; i < 8; ++i) lenb[i] = uint8_t(bits >> (56 - 8 * i));
    update(lenb, 8);
    for (int i = 0; i < 8; ++i) {
      out[4 * i] = uint8_t(h[i] >> 24);
      out[4 * i + 1] = uint8_t(h[i] >> 16);
      out[4 * i + 2] = uint8_t(h[i] >> 8);
      out[4 * i + 3] = uint8_t(h[i]);
    }
  }
};
}  // namespace

void sha256(const uint8_t* data, size_t n, uint8_t out[32]) {
  Sha256 s;
  s.update(data, n);
  s.finish(out);
}

Hash32 hash_chain(const Hash32& prev, const uint64_t* tokens, size_t n) {
  // SHA-256(prev || each token as u64 little-endian), src/serve/cache.rs:37-46
  Sha256 s;
  s.update(prev.data(), 32);
  for (size_t i = 0; i < n; ++i) {
    uint8_t le[8];
    for (int j = 0; j < 8; ++j) le[j] = uint8_t(tokens[i] >> (8 * j));
    s.update(le, 8);
  }
  Hash32 out;
  s.finish(out.data());
  return out;
}

// ---- Prefix ----------------------------------------------------------------------
int64_t Prefix::pinned_bytes() const {
  int64_t page_bytes = pool ? pool->page_b : 0;
  return pinned_pages * page_bytes + state_bytes;
}

int64_t Prefix::session_count(const Hash32& s) const {
  auto it = sessions.find(s);
  return it == sessions.end() ? 0 : static_cast<int64_t>(it->second.size());
}

// Moves an entry to the front of the cache and of its session's list (cache.rs:139-146).
void Prefix::touch(PrefixList::iterator it) {
  entries.splice(entries.begin(), entries, it);
  auto& list = sessions[it->key.session];
  list.splice(list.begin(), list, it->in_session);
}

// Gives up one reference to a run; a run nobody holds any more returns its pages to the pool and
// lets go of the block before it (a loop, not a recursion: a chain may be thousands of blocks deep).
void Prefix::release_run(std::shared_ptr<PageRun>& run) {
  std::shared_ptr<PageRun> cur = std::move(run);
  run.reset();
  while (cur && cur.use_count() == 1) {
    if (!cur->pages.empty()) {
      auto it = run_by_last_page.find(cur->pages.back());
      if (it != run_by_last_page.end()) {
        auto held = it->second.lock();
        if (!held || held.get() == cur.get()) run_by_last_page.erase(it);
      }
    }
    for (int32_t p : cur->pages)
      if (pool) pool->release(p);
    pinned_pages -= static_cast<int64_t>(cur->pages.size());
    std::shared_ptr<PageRun> parent = std::move(cur->parent);
    cur = std::move(parent);
  }
}

void Prefix::collect_pages(const PageRun* run, std::vector<int32_t>* out) const {
  std::vector<const PageRun*> chain;
  for (const PageRun* r = run; r != nullptr; r = r->parent.get()) chain.push_back(r);
  for (auto it = chain.rbegin(); it != chain.rend(); ++it) out->insert(out->end(), (*it)->pages.begin(), (*it)->pages.end());
}

std::shared_ptr<PageRun> Prefix::chain_for(const Seq* seq, int64_t tokens, bool create, int64_t* fresh_pages) {
  const int64_t per_block = block_tokens / PAGE_TOKENS;
  const int64_t n_blocks = tokens / block_tokens;
  const int64_t n_pages = tokens / PAGE_TOKENS;
  auto holds_block = [&](const PageRun* r, int64_t blk) {
    if (r->first_page != blk * per_block || static_cast<int64_t>(r->pages.size()) != per_block) return false;
    for (int64_t i = 0; i < per_block; ++i)
      if (r->pages[i] != seq->pages[r->first_page + i]) return false;
    return true;
  };
  std::shared_ptr<PageRun> base;
  int64_t base_blocks = 0;
  // Where the previous call for this sequence left off (the blocks of a prompt come in order) ...
  if (cursor.seq == seq && cursor.epoch == seq->epoch && cursor.blocks <= n_blocks) {
    base = cursor.run.lock();
    if (base) base_blocks = cursor.blocks;
  }
  // ... else the deepest live run that holds exactly the sequence's pages [0, its end): found through
  // the last page of a block, then compared page by page down to the root.
  for (int64_t b = n_blocks; b >= 1 && !base; --b) {
    auto it = run_by_last_page.find(seq->pages[b * per_block - 1]);
    if (it == run_by_last_page.end()) continue;
    std::shared_ptr<PageRun> cand = it->second.lock();
    if (!cand) continue;
    bool same = true;
    int64_t depth = 0;
    for (const PageRun* r = cand.get(); r != nullptr && same; r = r->parent.get()) {
      ++depth;
      same = b - depth >= 0 && holds_block(r, b - depth);
    }
    if (same && depth == b) {
      base = cand;
      base_blocks = b;
    }
  }
  // Live runs that continue the chain block by block (a re-inserted prompt finds its old runs).
  while (base_blocks < n_blocks) {
    auto it = run_by_last_page.find(seq->pages[(base_blocks + 1) * per_block - 1]);
    if (it == run_by_last_page.end()) break;
    std::shared_ptr<PageRun> cand = it->second.lock();
    if (!cand || cand->parent.get() != base.get() || !holds_block(cand.get(), base_blocks)) break;
    base = cand;
    base_blocks += 1;
  }
  if (fresh_pages) *fresh_pages = n_pages - base_blocks * per_block;
  if (create) {
    for (int64_t b = base_blocks; b < n_blocks; ++b) {
      auto run = std::make_shared<PageRun>();
      run->first_page = b * per_block;
      run->pages.assign(seq->pages.begin() + b * per_block, seq->pages.begin() + (b + 1) * per_block);
      run->parent = base;
      for (int32_t p : run->pages) pool->retain(p);
      pinned_pages += per_block;
      run_by_last_page[run->pages.back()] = run;
      base = run;
    }
    base_blocks = n_blocks;
  }
  if (base) {
    cursor.seq = seq;
    cursor.epoch = seq->epoch;
    cursor.blocks = base_blocks;
    cursor.run = base;
  }
  return base_blocks == n_blocks ? base : nullptr;
}

void Prefix::drop(PrefixList::iterator it, bool log) {
  if (log) {
    evicted_total += 1;
    if (evicted_log.size() < EVICTED_LOG_MAX) evicted_log.push_back(it->key);
  }
  index.erase(it->key);
  by_id.erase(it->id);
  auto sess = sessions.find(it->key.session);
  if (sess != sessions.end()) {
    sess->second.erase(it->in_session);
    if (sess->second.empty()) sessions.erase(sess);
  }
  if (it->ls) state_bytes -= it->ls->estimated_bytes();
  entry_bytes -= it->bytes;
  release_run(it->run);
  entries.erase(it);
}

bool Prefix::evict_lru(int64_t* bytes_out) {
  if (entries.empty()) return false;
  if (bytes_out) *bytes_out = entries.back().bytes;
  drop(std::prev(entries.end()), true);
  return true;
}

Prefix::~Prefix() {
  while (!entries.empty()) drop(std::prev(entries.end()), false);
}

void Prefix::match(const Hash32& session, const uint64_t* tokens, size_t n, int64_t* tokens_out, Hash32* hash_out,
                   uint64_t* entry_out) {
  *entry_out = 0;
  *tokens_out = 0;
  if (capacity == 0) return;   // cache.rs:127-129
  Hash32 previous = session;
  const size_t bt = static_cast<size_t>(block_tokens);
  for (size_t i = 0; i < n / bt; ++i) {
    const Hash32 hash = hash_chain(previous, tokens + i * bt, bt);
    auto it = index.find(PrefixKey{session, hash, static_cast<int64_t>((i + 1) * bt)});
    if (it == index.end()) break;   // stop at the first miss (cache.rs:134-138)
    touch(it->second);              // every touched block moves to the front (cache.rs:139-146)
    *tokens_out = it->second->key.tokens;
    *hash_out = hash;
    *entry_out = it->second->id;
    previous = hash;
  }
}

int Prefix::insert(const Hash32& session, const Hash32& hash, int64_t tokens, Seq* seq, LinState* ls, void* stream,
                   int32_t* inserted_out) {
  if (inserted_out) *inserted_out = 0;
  if (capacity == 0) return SGK_OK;  // cache.rs:162-164
  if (tokens <= 0) return fail(SGK_ERR_DIMENSION, "prefix block boundary must be positive");
  if (pool && !seq) return fail(SGK_ERR_BACKEND, "prefix insert needs the sequence to snapshot");
  if (seq) {
    if (seq->pool != pool) return fail(SGK_ERR_CONFIG, "sequence belongs to another pool");
    if (tokens % block_tokens != 0)
      return fail(SGK_ERR_DIMENSION, "snapshot boundary %lld is not on a block boundary", (long long)tokens);
    for (int64_t l : seq->len)
      if (l < tokens)
        return fail(SGK_ERR_DIMENSION, "snapshot of %lld rows from a sequence holding %lld", (long long)tokens, (long long)l);
    if (seq->released_pages > 0) return fail(SGK_ERR_DIMENSION, "snapshot of a sequence whose head was released");
  }
  const PrefixKey key{session, hash, tokens};
  const bool scrub = pool && !pool->host_only();
  // Budget loop of remember_prefix_block (src/serve/state.rs:627-635), run BEFORE the insert and
  // therefore with an older duplicate of this block still in the cache: what the new entry adds is
  // the pages no live run holds yet plus its state snapshot.
  auto additional = [&]() {
    int64_t fresh = 0;
    if (seq) chain_for(seq, tokens, false, &fresh);
    return fresh * (pool ? pool->page_b : 0) + (ls ? ls->estimated_bytes() : 0);
  };
  if (budget > 0) {
    while (pinned_bytes() + additional() > budget) {
      if (!evict_lru(nullptr)) {
        if (scrub) SGK_TRY(pool->flush_scrub(pool->st->stream));
        return SGK_OK;  // cache empty and still over budget: skip the insert
      }
    }
  }
  PrefixEntry e;
  e.key = key;
  e.bytes = additional();
  auto dup = index.find(key);
  // a refresh over the same pages takes over what its duplicate accounted for
  if (dup != index.end() && e.bytes < dup->second->bytes) e.bytes = dup->second->bytes;
  // The new entry's pages are pinned before the duplicate lets go of the same ones.
  if (seq) e.run = chain_for(seq, tokens, true, nullptr);
  // a refresh replaces the older duplicate without counting as an eviction (cache.rs:165-169)
  if (dup != index.end()) drop(dup->second, false);
  if (ls) {
    LinState* snap = nullptr;
    int rc = linstate_snapshot(ls, stream, &snap);
    if (rc != SGK_OK) {
      release_run(e.run);
      return rc;
    }
    e.ls.reset(snap);
    state_bytes += snap->estimated_bytes();
  }
  e.id = next_id++;
  entry_bytes += e.bytes;
  entries.push_front(std::move(e));  // cache.rs:173-183
  auto it = entries.begin();
  index[key] = it;
  by_id[it->id] = it;
  auto& list = sessions[session];
  list.push_front(it);
  it->in_session = list.begin();
  // per-session cap: that session's rear-most entries leave first (cache.rs:184-188)
  while (session_count(session) > blocks_per_session) {
    auto sess = sessions.find(session);
    if (sess == sessions.end() || sess->second.empty()) break;
    drop(sess->second.back(), true);
  }
  while (static_cast<int64_t>(entries.size()) > capacity) drop(std::prev(entries.end()), true);  // :189-191
  if (scrub) SGK_TRY(pool->flush_scrub(pool->st->stream));
  if (inserted_out) *inserted_out = 1;
  return SGK_OK;
}

// ---- DecoderPrefix ---------------------------------------------------------------
void DecoderPrefix::drop(size_t index) {
  for (int32_t p : entries[index].pages)
    if (pool) pool->release(p);
  entries.erase(entries.begin() + static_cast<long>(index));
}

DecoderPrefix::~DecoderPrefix() {
  while (!entries.empty()) drop(entries.size() - 1);
}

// ---- Budget (src/memory_guard.rs:168-185) -------------------------------------------
bool Budget::limit(uint64_t* out) const {
  bool any = false;
  uint64_t best = 0;
  auto consider = [&](uint64_t v) {
    if (v == 0) return;
    if (!any || v < best) best = v;
    any = true;
  };
  consider(static_cap);
  if (total_memory > 0) consider(total_memory > headroom ? total_memory - headroom : 0);
  consider(device_cap);
  if (any) *out = best;
  return any;
}

}  // namespace sgk
