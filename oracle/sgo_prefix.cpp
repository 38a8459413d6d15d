// CPU oracle (test infrastructure only): bookkeeping half of the path —
// SHA-256 block-hash chain, the LRU prefix cache, longest-prefix selection,
// the memory budget and the linear-attention state container.
#include <algorithm>
#include <cstring>

#include "sgo.hpp"

namespace sgo {

bool Hash32::operator==(const Hash32& o) const { return std::memcmp(b, o.b, 32) == 0; }

// ---- SHA-256 (FIPS 180-4). The reference calls the sha2 crate 0.10.9
// (Cargo.lock:1739-1741) at src/serve/cache.rs:26-31,37-45; digest VALUES are
// not pinned by any reference test (parity unpinned), so this is checked
// against the FIPS vectors and Python hashlib instead.
static const uint32_t K256[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

static inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

static void sha256_block(uint32_t h[8], const uint8_t* p) {
  uint32_t w[64];
  for (int i = 0; i < 16; ++i)
    w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) |
           (uint32_t(p[4 * i + 2]) << 8) | uint32_t(p[4 * i + 3]);
  for (int i = 16; i < 64; ++i) {
    uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
  for (int i = 0; i < 64; ++i) {
    uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
    uint32_t ch = (e & f) ^ (~e & g);
    uint32_t t1 = hh + S1 + ch + K256[i] + w[i];
    uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
    uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
    uint32_t t2 = S0 + mj;
    hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
  }
  h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}

void sha256(const uint8_t* data, size_t n, uint8_t out[32]) {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                   0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  size_t full = n / 64;
  for (size_t i = 0; i < full; ++i) sha256_block(h, data + 64 * i);
  uint8_t tail[128] = {0};
  size_t rem = n - 64 * full;
  std::memcpy(tail, data + 64 * full, rem);
  tail[rem] = 0x80;
  size_t tail_len = (rem + 9 <= 64) ? 64 : 128;
  uint64_t bits = static_cast<uint64_t>(n) * 8;
  for (int i = 0; i < 8; ++i) tail[tail_len - 1 - i] = static_cast<uint8_t>(bits >> (8 * i));
  sha256_block(h, tail);
  if (tail_len == 128) sha256_block(h, tail + 64);
  for (int i = 0; i < 8; ++i) {
    out[4 * i] = static_cast<uint8_t>(h[i] >> 24);
    out[4 * i + 1] = static_cast<uint8_t>(h[i] >> 16);
    out[4 * i + 2] = static_cast<uint8_t>(h[i] >> 8);
    out[4 * i + 3] = static_cast<uint8_t>(h[i]);
  }
}

// ---- BlockHash (src/serve/cache.rs:11-47) ----------------------------------
Hash32 block_hash_root() {  // :16-18
  Hash32 h;
  std::memset(h.b, 0, 32);
  return h;
}

Hash32 block_hash_for_session(const char* key, size_t key_len, bool present) {  // :22-33
  if (!present || key_len == 0) return block_hash_root();  // None or "" => root
  Hash32 h;
  sha256(reinterpret_cast<const uint8_t*>(key), key_len, h.b);
  return h;
}

Hash32 block_hash_chain(const Hash32& prev, const uint64_t* tokens, size_t n) {  // :37-46
  // digest(prev32 || each token as u64 little-endian)
  std::vector<uint8_t> buf(32 + 8 * n);
  std::memcpy(buf.data(), prev.b, 32);
  for (size_t i = 0; i < n; ++i)
    for (int j = 0; j < 8; ++j) buf[32 + 8 * i + j] = static_cast<uint8_t>(tokens[i] >> (8 * j));
  Hash32 h;
  sha256(buf.data(), buf.size(), h.b);
  return h;
}

// ---- BlockAwarePrefixCache (src/serve/cache.rs:74-219) ---------------------
BlockAwarePrefixCache::BlockAwarePrefixCache(size_t bt, size_t cap, size_t per_session)
    : block_tokens(std::max<size_t>(bt, 1)),  // :111 block_tokens.max(1)
      capacity(cap),
      blocks_per_session(per_session) {}

PrefixHit BlockAwarePrefixCache::match_prefix(const Hash32& root, const uint64_t* tokens, size_t n) {
  PrefixHit best;
  if (capacity == 0) return best;  // :126-128
  Hash32 previous = root;
  size_t blocks = n / block_tokens;  // chunks_exact: full blocks only
  for (size_t index = 0; index < blocks; ++index) {
    Hash32 hash = block_hash_chain(previous, tokens + index * block_tokens, block_tokens);
    size_t expected_tokens = (index + 1) * block_tokens;
    // :134-138 — first entry with the same (session, hash, tokens); stop at the first miss.
    auto it = std::find_if(entries.begin(), entries.end(), [&](const PrefixEntry& e) {
      return e.session == root && e.hash == hash && e.tokens == expected_tokens;
    });
    if (it == entries.end()) break;
    PrefixEntry entry = *it;
    entries.erase(it);
    best.found = true;
    best.tokens = entry.tokens;
    best.hash = entry.hash;
    best.payload = entry.payload;
    entries.insert(entries.begin(), entry);  // :146 — every touched block moves to the front
    previous = hash;
  }
  return best;
}

size_t BlockAwarePrefixCache::session_block_count(const Hash32& session) const {  // :204-209
  size_t n = 0;
  for (const auto& e : entries) n += (e.session == session) ? 1 : 0;
  return n;
}

size_t BlockAwarePrefixCache::insert(const Hash32& session, const Hash32& hash, size_t tokens,
                                     uint64_t payload, size_t bytes) {
  if (capacity == 0) return 0;  // :162-164
  auto it = std::find_if(entries.begin(), entries.end(), [&](const PrefixEntry& e) {
    return e.session == session && e.hash == hash && e.tokens == tokens;
  });
  // :165-169 — a refresh silently replaces the older duplicate (not an eviction).
  if (it != entries.end()) entries.erase(it);
  entries.insert(entries.begin(), PrefixEntry{session, hash, tokens, payload, bytes});  // :173-183
  // :184-188 — per-session cap: drop that session's rear-most entries first.
  while (session_block_count(session) > blocks_per_session) {
    long idx = -1;
    for (long i = static_cast<long>(entries.size()) - 1; i >= 0; --i)
      if (entries[static_cast<size_t>(i)].session == session) {
        idx = i;
        break;
      }
    if (idx < 0) break;
    evicted_log.push_back(entries[static_cast<size_t>(idx)]);
    entries.erase(entries.begin() + idx);
  }
  // :189-191 — global cap: pop the rear.
  while (entries.size() > capacity) {
    evicted_log.push_back(entries.back());
    entries.pop_back();
  }
  return bytes;
}

bool BlockAwarePrefixCache::evict_lru_block(size_t* bytes_out) {  // :196-198
  if (entries.empty()) return false;
  if (bytes_out) *bytes_out = entries.back().bytes;
  evicted_log.push_back(entries.back());
  entries.pop_back();
  return true;
}

size_t BlockAwarePrefixCache::estimated_bytes() const {  // :200-203
  size_t total = 0;
  for (const auto& e : entries) total += e.bytes;
  return total;
}

// ---- longest-prefix selection (src/decoder/generation.rs:190-204) ----------
long longest_prefix_entry_index(const std::vector<std::vector<uint64_t>>& entries,
                                const uint64_t* prompt, size_t n) {
  long best = -1;
  size_t best_len = 0;
  for (size_t i = 0; i < entries.size(); ++i) {
    size_t len = entries[i].size();
    if (len > best_len && len <= n && std::equal(entries[i].begin(), entries[i].end(), prompt)) {
      best = static_cast<long>(i);
      best_len = len;
    }
  }
  return best;
}

// ---- memory budget (src/memory_guard.rs:155-185,331-370) -------------------
bool MemoryLimits::effective_limit(uint64_t* out) const {
  // min over the present, non-zero candidates: static cap, host - headroom, device cap.
  bool any = false;
  uint64_t best = 0;
  auto consider = [&](bool has, uint64_t v) {
    if (!has || v == 0) return;
    if (!any || v < best) best = v;
    any = true;
  };
  consider(has_static, static_cap);
  consider(has_host, host_memory > headroom_bytes ? host_memory - headroom_bytes : 0);
  consider(has_device, device_cap);
  if (any) *out = best;
  return any;
}

static uint64_t sat_add(uint64_t a, uint64_t b) { return a + b < a ? UINT64_MAX : a + b; }

bool MemoryGuard::projection(uint64_t requested, MemoryProjection* out) const {  // :336-352
  if (!enabled) return false;
  uint64_t limit;
  if (!limits.effective_limit(&limit)) return false;
  uint64_t before = sat_add(current, reserved);
  out->current = current;
  out->reserved = reserved;
  out->requested = requested;
  out->projected = sat_add(before, requested);
  out->limit = limit;
  out->available = limit > before ? limit - before : 0;
  return true;
}

bool MemoryGuard::projection_over_limit(uint64_t requested, MemoryProjection* out) const {  // :355-358
  MemoryProjection p;
  if (!projection(requested, &p)) return false;
  if (p.projected > p.limit) {
    if (out) *out = p;
    return true;
  }
  return false;
}

bool MemoryGuard::check_allocation(uint64_t requested, MemoryProjection* over) const {  // :365-370
  return !projection_over_limit(requested, over);
}

// ---- linear-attention state (snapshot = deep copy; restore validates shape) --
LinearState linear_state_snapshot(const LinearState& s) { return s; }

Status linear_state_restore(LinearState* state, const LinearState& snapshot) {
  // src/metal_backend/linear_attention.rs:3133-3149 — lengths and dtype must agree.
  if (state->conv.size() != snapshot.conv.size() || state->ssm.size() != snapshot.ssm.size() ||
      state->ssm_bf16 != snapshot.ssm_bf16)
    return ERR_SHAPE;
  state->conv = snapshot.conv;
  state->ssm = snapshot.ssm;
  return OK;
}

// ---- Gated DeltaNet step (src/linear_attention.rs:896-991) ---------------------
Status gated_delta_step(const float* q, const float* k, const float* v, const float* g, const float* beta,
                        const LinearShape& sh, std::vector<float>* ssm, float* out) {
  if (sh.num_key_heads == 0 || sh.num_value_heads % sh.num_key_heads != 0) return ERR_DIMENSION;
  const size_t head_len = sh.value_head_dim * sh.key_head_dim;
  if (ssm->size() != sh.num_value_heads * head_len) return ERR_DIMENSION;  // ensure_ssm_cache, :994-1024
  const size_t repeat = sh.num_value_heads / sh.num_key_heads;
  for (size_t vh = 0; vh < sh.num_value_heads; ++vh) {
    const size_t kh = vh / repeat;  // GQA: q/k of key head floor(h / repeat)
    const float* q_head = q + kh * sh.key_head_dim;
    const float* k_head = k + kh * sh.key_head_dim;
    const float* v_head = v + vh * sh.value_head_dim;
    const float decay = g[vh], beta_value = beta[vh];
    float* state_head = ssm->data() + vh * head_len;
    for (size_t col = 0; col < sh.value_head_dim; ++col) {
      float* row = state_head + col * sh.key_head_dim;
      float kv_mem = 0.0f;
      for (size_t i = 0; i < sh.key_head_dim; ++i) {  // :964-967 decay in place, read before write
        row[i] *= decay;
        kv_mem += row[i] * k_head[i];
      }
      const float delta = (v_head[col] - kv_mem) * beta_value;  // :970
      float y = 0.0f;
      for (size_t i = 0; i < sh.key_head_dim; ++i) {  // :974-980 outer product and read-out fused
        row[i] += delta * k_head[i];
        y += row[i] * q_head[i];
      }
      out[vh * sh.value_head_dim + col] = y;
    }
  }
  return OK;
}

// ---- depthwise causal conv, one token (src/linear_attention.rs:802-852) --------
Status depthwise_conv_step(const float* qkv, const float* weight, size_t conv_dim, size_t kernel,
                           std::vector<float>* history, float* out) {
  if (kernel == 0) return ERR_DIMENSION;
  const size_t keep = kernel - 1;
  if (history->size() != keep * conv_dim) return ERR_DIMENSION;  // :816-823
  for (size_t c = 0; c < conv_dim; ++c) {
    float acc = 0.0f;
    for (size_t kk = 0; kk < kernel; ++kk) {
      const float input = kk < keep ? (*history)[kk * conv_dim + c] : qkv[c];
      acc += input * weight[c * kernel + kk];  // conv_weight_value: [conv_dim][K]
    }
    out[c] = acc;
  }
  // the history advances to the last K-1 tokens (:841-848)
  if (keep > 0) {
    std::vector<float> next(keep * conv_dim);
    for (size_t r = 0; r + 1 < keep; ++r)
      std::memcpy(next.data() + r * conv_dim, history->data() + (r + 1) * conv_dim, conv_dim * sizeof(float));
    std::memcpy(next.data() + (keep - 1) * conv_dim, qkv, conv_dim * sizeof(float));
    *history = next;
  }
  return OK;
}

// ---- greedy epilogue (src/sampling.rs:49-62 over a biasless Linear) -------------
Status lm_head_argmax(const float* weight, size_t vocab, size_t hidden, const float* x, size_t* index, float* value) {
  if (vocab == 0) return ERR_DIMENSION;
  size_t best = 0;
  float best_value = 0.0f;
  for (size_t r = 0; r < vocab; ++r) {
    float acc = 0.0f;
    for (size_t c = 0; c < hidden; ++c) acc += weight[r * hidden + c] * x[c];
    if (r == 0 || acc > best_value) {  // strictly greater: the first maximum stays
      best = r;
      best_value = acc;
    }
  }
  *index = best;
  *value = best_value;
  return OK;
}

// ---- token feed (src/kernels.metal:308-325) ------------------------------------
bool embed_gather(const float* table, size_t vocab, size_t dim, size_t token, float scale, bool recast_bf16, float* out) {
  if (token >= vocab) return false;
  for (size_t i = 0; i < dim; ++i) {
    const float value = table[token * dim + i] * scale;
    out[i] = recast_bf16 ? bf16_round_f32(value) : value;
  }
  return true;
}

}  // namespace sgo
