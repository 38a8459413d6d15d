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
  return static_cast<int64_t>(pins.size()) * page_bytes + state_bytes;
}

int64_t Prefix::session_count(const Hash32& s) const {
  int64_t n = 0;
  for (const auto& e : entries) n += e.session == s ? 1 : 0;
  return n;
}

void Prefix::drop(size_t index, bool log) {
  PrefixEntry& e = entries[index];
  if (log) evicted_log.push_back(PrefixKey{e.session, e.hash, e.tokens});
  for (int32_t p : e.pages) {
    auto it = pins.find(p);
    if (it != pins.end() && --it->second == 0) pins.erase(it);
    if (pool) pool->release(p);
  }
  if (e.ls) state_bytes -= e.ls->estimated_bytes();
  entries.erase(entries.begin() + static_cast<long>(index));
}

bool Prefix::evict_lru(int64_t* bytes_out) {
  if (entries.empty()) return false;
  if (bytes_out) *bytes_out = entries.back().bytes;
  drop(entries.size() - 1, true);
  return true;
}

Prefix::~Prefix() {
  while (!entries.empty()) drop(entries.size() - 1, false);
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
