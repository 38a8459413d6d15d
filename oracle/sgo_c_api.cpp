// CPU oracle (test infrastructure only): flat C entry points so that the tests
// (ctypes) and bench.py's cpu_baseline leg can drive the C++ restatement.
#include <cstring>
#include <map>
#include <memory>

#include "sgo.hpp"

using namespace sgo;

extern "C" {

uint16_t sgo_f32_to_bf16_bits(float v) { return f32_to_bf16_bits(v); }
float sgo_bf16_round_f32(float v) { return bf16_round_f32(v); }
void sgo_bf16_round_array(const float* in, size_t n, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = bf16_round_f32(in[i]);
}
void sgo_f32_to_bf16_array(const float* in, size_t n, uint16_t* out) {
  for (size_t i = 0; i < n; ++i) out[i] = f32_to_bf16_bits(in[i]);
}

// ---- LayerKvCache -----------------------------------------------------------
void* sgo_cache_new() { return new LayerKvCache(); }
void sgo_cache_free(void* c) { delete static_cast<LayerKvCache*>(c); }
int32_t sgo_cache_append(void* c, const float* k, size_t kr, size_t kd, const float* v, size_t vr,
                         size_t vd, size_t expected) {
  return static_cast<LayerKvCache*>(c)->append(k, kr, kd, v, vr, vd, expected);
}
int32_t sgo_cache_append_batch(void* c, const float* k, size_t kr, size_t kd, const float* v,
                               size_t vr, size_t vd, size_t expected) {
  return static_cast<LayerKvCache*>(c)->append_batch(k, kr, kd, v, vr, vd, expected);
}
size_t sgo_cache_len(void* c) { return static_cast<LayerKvCache*>(c)->len(); }
int32_t sgo_cache_truncate(void* c, size_t len) { return static_cast<LayerKvCache*>(c)->truncate(len); }
const float* sgo_cache_keys(void* c) { return static_cast<LayerKvCache*>(c)->keys.data(); }
const float* sgo_cache_values(void* c) { return static_cast<LayerKvCache*>(c)->values.data(); }

// ---- ResidentKv -------------------------------------------------------------
int32_t sgo_rkv_new(size_t capacity, size_t q_heads, size_t kv_heads, size_t head_dim,
                    int32_t dtype, void** out) {
  auto kv = std::make_unique<ResidentKv>();
  Status s = ResidentKv::create(capacity, q_heads, kv_heads, head_dim, static_cast<KvDtype>(dtype),
                                kv.get());
  if (s != OK) return s;
  *out = kv.release();
  return OK;
}
void sgo_rkv_free(void* p) { delete static_cast<ResidentKv*>(p); }
int32_t sgo_rkv_seed(void* p, const float* k, size_t kl, const float* v, size_t vl, size_t n) {
  return static_cast<ResidentKv*>(p)->seed(k, kl, v, vl, n);
}
int32_t sgo_rkv_append_row(void* p, const float* k, size_t kl, const float* v, size_t vl) {
  return static_cast<ResidentKv*>(p)->append_row(k, kl, v, vl);
}
int32_t sgo_rkv_truncate(void* p, size_t len) { return static_cast<ResidentKv*>(p)->truncate(len); }
size_t sgo_rkv_len(void* p) { return static_cast<ResidentKv*>(p)->len; }
const float* sgo_rkv_keys(void* p) { return static_cast<ResidentKv*>(p)->keys.data(); }
const float* sgo_rkv_values(void* p) { return static_cast<ResidentKv*>(p)->values.data(); }
int32_t sgo_rkv_attention(void* p, const float* q, size_t window_start, float attn_scalar,
                          int threads, float* out) {
  auto* kv = static_cast<ResidentKv*>(p);
  return attention_windowed(q, kv->keys.data(), kv->values.data(), kv->len, window_start,
                            kv->q_heads, kv->kv_heads, kv->head_dim, attn_scalar, threads, out);
}

// ---- attention ----------------------------------------------------------------
int32_t sgo_cached_attention_one(const float* q, size_t q_dim, const float* keys,
                                 const float* values, size_t cache_len, size_t q_heads,
                                 size_t kv_heads, size_t head_dim, float attn_scalar,
                                 int32_t has_window, size_t window, int threads, float* out) {
  return cached_attention_one(q, q_dim, keys, values, cache_len, q_heads, kv_heads, head_dim,
                              attn_scalar, has_window != 0, window, threads, out);
}
int32_t sgo_attention_windowed(const float* q, const float* keys, const float* values, size_t len,
                               size_t window_start, size_t q_heads, size_t kv_heads,
                               size_t head_dim, float attn_scalar, int threads, float* out) {
  return attention_windowed(q, keys, values, len, window_start, q_heads, kv_heads, head_dim,
                            attn_scalar, threads, out);
}
void sgo_softmax_in_place(float* v, size_t n, float t) { softmax_in_place(v, n, t); }

// ---- RMSNorm / RoPE -------------------------------------------------------------
void sgo_rope_rotations(size_t position, size_t rope_dims, float theta, size_t frequency_dim,
                        float position_scale, float* cos_out, float* sin_out) {
  rope_rotations(position, rope_dims, RopeParams{theta, frequency_dim, position_scale}, cos_out,
                 sin_out);
}
int32_t sgo_rms_norm_heads(const float* x, size_t seq, size_t heads, size_t head_dim,
                           const float* w, float eps, float* out) {
  return rms_norm_heads(x, seq, heads, head_dim, w, eps, out);
}
int32_t sgo_apply_rope_heads_at(const float* x, size_t seq, size_t heads, size_t head_dim,
                                size_t rope_dims, float theta, size_t frequency_dim,
                                float position_scale, size_t position_offset, int32_t style,
                                float* out) {
  return apply_rope_heads_at(x, seq, heads, head_dim, rope_dims,
                             RopeParams{theta, frequency_dim, position_scale}, position_offset,
                             static_cast<RopeStyle>(style), out);
}
int32_t sgo_rms_norm_rope_heads_at(const float* x, size_t seq, size_t heads, size_t head_dim,
                                   size_t rope_dims, const float* w, float eps, float theta,
                                   size_t frequency_dim, float position_scale,
                                   size_t position_offset, int32_t style, float* out) {
  return rms_norm_rope_heads_at(x, seq, heads, head_dim, rope_dims, w, eps,
                                RopeParams{theta, frequency_dim, position_scale}, position_offset,
                                static_cast<RopeStyle>(style), out);
}

// ---- u8 group-32 ------------------------------------------------------------------
void sgo_quantize_row_u8(const float* x, size_t n, uint8_t* codes, uint16_t* scale, uint16_t* bias) {
  quantize_row_u8(x, n, codes, scale, bias);
}
void sgo_dequantize_row_u8(const uint8_t* codes, const uint16_t* scale, const uint16_t* bias,
                           size_t n, float* out) {
  dequantize_row_u8(codes, scale, bias, n, out);
}

// ---- hashes -------------------------------------------------------------------------
void sgo_sha256(const uint8_t* data, size_t n, uint8_t* out) { sha256(data, n, out); }
void sgo_hash_root(uint8_t* out) { std::memcpy(out, block_hash_root().b, 32); }
void sgo_hash_for_session(const char* key, size_t n, int32_t present, uint8_t* out) {
  std::memcpy(out, block_hash_for_session(key, n, present != 0).b, 32);
}
void sgo_hash_chain(const uint8_t* prev, const uint64_t* tokens, size_t n, uint8_t* out) {
  Hash32 p;
  std::memcpy(p.b, prev, 32);
  std::memcpy(out, block_hash_chain(p, tokens, n).b, 32);
}

// ---- prefix cache ----------------------------------------------------------------------
void* sgo_prefix_new(size_t block_tokens, size_t capacity, size_t per_session) {
  return new BlockAwarePrefixCache(block_tokens, capacity, per_session);
}
void sgo_prefix_free(void* p) { delete static_cast<BlockAwarePrefixCache*>(p); }
size_t sgo_prefix_block_tokens(void* p) { return static_cast<BlockAwarePrefixCache*>(p)->block_tokens; }
int32_t sgo_prefix_match(void* p, const uint8_t* root, const uint64_t* tokens, size_t n,
                         size_t* tokens_out, uint8_t* hash_out, uint64_t* payload_out) {
  Hash32 r;
  std::memcpy(r.b, root, 32);
  PrefixHit hit = static_cast<BlockAwarePrefixCache*>(p)->match_prefix(r, tokens, n);
  if (!hit.found) return 0;
  *tokens_out = hit.tokens;
  std::memcpy(hash_out, hit.hash.b, 32);
  *payload_out = hit.payload;
  return 1;
}
size_t sgo_prefix_insert(void* p, const uint8_t* session, const uint8_t* hash, size_t tokens,
                         uint64_t payload, size_t bytes) {
  Hash32 s, h;
  std::memcpy(s.b, session, 32);
  std::memcpy(h.b, hash, 32);
  return static_cast<BlockAwarePrefixCache*>(p)->insert(s, h, tokens, payload, bytes);
}
int32_t sgo_prefix_evict_lru(void* p, size_t* bytes_out) {
  return static_cast<BlockAwarePrefixCache*>(p)->evict_lru_block(bytes_out) ? 1 : 0;
}
size_t sgo_prefix_bytes(void* p) { return static_cast<BlockAwarePrefixCache*>(p)->estimated_bytes(); }
size_t sgo_prefix_len(void* p) { return static_cast<BlockAwarePrefixCache*>(p)->entries.size(); }
size_t sgo_prefix_session_count(void* p, const uint8_t* session) {
  Hash32 s;
  std::memcpy(s.b, session, 32);
  return static_cast<BlockAwarePrefixCache*>(p)->session_block_count(s);
}
// which: 0 = live entries front-to-rear, 1 = the eviction log in order.
size_t sgo_prefix_dump(void* p, int32_t which, size_t cap, uint8_t* sessions, uint8_t* hashes,
                       size_t* tokens, uint64_t* payloads) {
  auto* c = static_cast<BlockAwarePrefixCache*>(p);
  const auto& v = which == 0 ? c->entries : c->evicted_log;
  size_t n = std::min(cap, v.size());
  for (size_t i = 0; i < n; ++i) {
    std::memcpy(sessions + 32 * i, v[i].session.b, 32);
    std::memcpy(hashes + 32 * i, v[i].hash.b, 32);
    tokens[i] = v[i].tokens;
    payloads[i] = v[i].payload;
  }
  return v.size();
}
long sgo_longest_prefix_entry_index(const uint64_t* flat, const size_t* lens, size_t n_entries,
                                    const uint64_t* prompt, size_t n) {
  std::vector<std::vector<uint64_t>> entries;
  size_t off = 0;
  for (size_t i = 0; i < n_entries; ++i) {
    entries.emplace_back(flat + off, flat + off + lens[i]);
    off += lens[i];
  }
  return longest_prefix_entry_index(entries, prompt, n);
}

// ---- memory budget -------------------------------------------------------------------
void* sgo_guard_new(int32_t has_static, uint64_t static_cap, int32_t has_host, uint64_t host_memory,
                    uint64_t headroom, int32_t has_device, uint64_t device_cap) {
  auto* g = new MemoryGuard();
  g->limits.has_static = has_static != 0;
  g->limits.static_cap = static_cap;
  g->limits.has_host = has_host != 0;
  g->limits.host_memory = host_memory;
  g->limits.headroom_bytes = headroom;
  g->limits.has_device = has_device != 0;
  g->limits.device_cap = device_cap;
  return g;
}
void sgo_guard_free(void* g) { delete static_cast<MemoryGuard*>(g); }
void sgo_guard_set(void* g, uint64_t current, uint64_t reserved) {
  static_cast<MemoryGuard*>(g)->current = current;
  static_cast<MemoryGuard*>(g)->reserved = reserved;
}
int32_t sgo_guard_limit(void* g, uint64_t* out) {
  return static_cast<MemoryGuard*>(g)->limits.effective_limit(out) ? 1 : 0;
}
// returns 1 when the request is accepted; fills projected/available either way.
int32_t sgo_guard_check(void* g, uint64_t requested, uint64_t* projected, uint64_t* available) {
  MemoryProjection p{};
  auto* guard = static_cast<MemoryGuard*>(g);
  if (!guard->projection(requested, &p)) return 1;
  *projected = p.projected;
  *available = p.available;
  return p.projected > p.limit ? 0 : 1;
}

// ---- linear state ----------------------------------------------------------------------
int32_t sgo_linear_restore_check(size_t conv_a, size_t ssm_a, int32_t bf16_a, size_t conv_b,
                                 size_t ssm_b, int32_t bf16_b) {
  LinearState a, b;
  a.conv.resize(conv_a);
  a.ssm.resize(ssm_a);
  a.ssm_bf16 = bf16_a != 0;
  b.conv.resize(conv_b);
  b.ssm.resize(ssm_b);
  b.ssm_bf16 = bf16_b != 0;
  return linear_state_restore(&a, b);
}

int32_t sgo_gated_delta_step(const float* q, const float* k, const float* v, const float* g, const float* beta,
                             size_t num_key_heads, size_t num_value_heads, size_t key_head_dim,
                             size_t value_head_dim, float* ssm, size_t ssm_len, float* out) {
  LinearShape sh{num_key_heads, num_value_heads, key_head_dim, value_head_dim, 0};
  std::vector<float> state(ssm, ssm + ssm_len);
  Status st = gated_delta_step(q, k, v, g, beta, sh, &state, out);
  if (st == OK) std::memcpy(ssm, state.data(), state.size() * sizeof(float));
  return st;
}
int32_t sgo_depthwise_conv_step(const float* qkv, const float* weight, size_t conv_dim, size_t kernel,
                                float* history, size_t history_len, float* out) {
  std::vector<float> h(history, history + history_len);
  Status st = depthwise_conv_step(qkv, weight, conv_dim, kernel, &h, out);
  if (st == OK && !h.empty()) std::memcpy(history, h.data(), h.size() * sizeof(float));
  return st;
}

int32_t sgo_lm_head_argmax(const float* weight, size_t vocab, size_t hidden, const float* x, size_t* index,
                           float* value) {
  return lm_head_argmax(weight, vocab, hidden, x, index, value);
}

int32_t sgo_embed_gather(const float* table, size_t vocab, size_t dim, size_t token, float scale, int32_t recast_bf16,
                         float* out) {
  return embed_gather(table, vocab, dim, token, scale, recast_bf16 != 0, out) ? 1 : 0;
}

// ---- generators ---------------------------------------------------------------------------
float sgo_pseudo(uint64_t seed) { return pseudo(seed); }
void sgo_pseudo_array(uint64_t seed0, size_t n, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = pseudo(seed0 + i);
}
uint64_t sgo_splitmix64(uint64_t x) { return splitmix64(x); }
float sgo_normal8(uint64_t seed, uint64_t stream, uint64_t index) { return normal8(seed, stream, index); }
void sgo_fill_normal8(float* out, size_t n, uint64_t seed, uint64_t stream, uint64_t index0) {
  fill_normal8(out, n, seed, stream, index0);
}

}  // extern "C"
