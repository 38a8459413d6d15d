// CPU oracle for the saragossa KV-cache hot path.
//
// TEST INFRASTRUCTURE ONLY. This is a plain C++17 restatement of the reference's
// own CPU algorithms for the path (KV append, single-query GQA attention,
// RMSNorm+RoPE, block-hash prefix cache, linear-attention state container,
// memory budget). Nothing in the product library links, imports or calls it; it
// is the checker the parity tests and the reported CPU baseline use.
//
// Pinning: the reference is Rust and cannot be built where this oracle is built,
// so each function is pinned against the known-answer vectors, closed forms and
// ordering assertions of the reference's own unit tests (cited per function and
// replayed in tests/test_oracle_*.py). Two items have NO reference pin and are
// marked "parity unpinned" where they are defined: SHA-256 digest values (the
// reference only tests equality/inequality; pinned here against the published
// FIPS 180-4 vectors and Python hashlib) and the u8 group-32 KV quantiser (the
// reference has no KV quantiser; only its dequant formula q*scale+bias is pinned).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace sgo {

// Status codes mirror the reference's InferError variants (src/error.rs:12-75).
enum Status : int32_t {
  OK = 0,
  ERR_DIMENSION = 1,  // InferError::Dimension
  ERR_CONFIG = 2,     // InferError::Config
  ERR_BACKEND = 3,    // InferError::Metal
  ERR_MEMORY_GUARD = 4,
  ERR_SHAPE = 5,      // InferError::Shape
};

// ---- bf16 ---------------------------------------------------------------
// src/decode_resident/utils.rs:55-60 (same code src/decoder.rs:1629-1633).
uint16_t f32_to_bf16_bits(float value);
float bf16_bits_to_f32(uint16_t bits);
float bf16_round_f32(float value);  // utils.rs:236-238

// ---- CPU KV cache (src/decoder/attention_cache.rs:7-100) -----------------
struct LayerKvCache {
  std::vector<float> keys;
  std::vector<float> values;
  bool has_dim = false;
  size_t kv_dim = 0;
  // key/value are [rows, dim] matrices.
  Status append(const float* key, size_t key_rows, size_t key_dim, const float* value,
                size_t value_rows, size_t value_dim, size_t expected_dim);
  Status append_batch(const float* key, size_t key_rows, size_t key_dim, const float* value,
                      size_t value_rows, size_t value_dim, size_t expected_dim);
  size_t len() const;
  Status truncate(size_t len);
};

// ---- resident KV semantics (src/decode_resident/attention.rs:56-108,501-644) ----
enum KvDtype : int32_t { KV_F32 = 0, KV_BF16 = 1, KV_U8G32 = 2 };
struct ResidentKv {
  size_t capacity = 0, len = 0, q_heads = 0, kv_heads = 0, head_dim = 0;
  KvDtype dtype = KV_F32;
  // Stored values as f32 after the storage rounding (bf16 RNE or u8 dequant),
  // which is what the reference's bf16 test oracle feeds its attention
  // (src/decode_resident/tests.rs:1462-1472).
  std::vector<float> keys, values;
  static Status create(size_t capacity, size_t q_heads, size_t kv_heads, size_t head_dim,
                       KvDtype dtype, ResidentKv* out);
  size_t kv_dim() const { return kv_heads * head_dim; }
  Status seed(const float* k, size_t k_len, const float* v, size_t v_len, size_t n_rows);
  Status append_row(const float* k, size_t k_len, const float* v, size_t v_len);
  Status truncate(size_t new_len);
  void store_row(size_t row, const float* k, const float* v);
};

// ---- decode attention (src/decoder/attention_ops.rs:889-974,1019-1046) ----
// Single-query GQA attention over rows [window_start, len) of a contiguous
// [len, kv_dim] f32 cache. threads<=1: the serial branch; threads>1: the
// per-q-head parallel branch (the reference switches at len >= 128, rayon over
// heads, which does not change any per-head float order).
Status cached_attention_one(const float* q, size_t q_dim, const float* keys, const float* values,
                            size_t cache_len, size_t q_heads, size_t kv_heads, size_t head_dim,
                            float attn_scalar, bool has_window, size_t sliding_window,
                            int threads, float* out);
// Same with an explicit window start (src/decode_resident/tests.rs:1035-1082).
Status attention_windowed(const float* q, const float* keys, const float* values, size_t len,
                          size_t window_start, size_t q_heads, size_t kv_heads, size_t head_dim,
                          float attn_scalar, int threads, float* out);
void softmax_in_place(float* values, size_t n, float temperature);  // attention_ops.rs:1019-1038
float dot_product(const float* a, const float* b, size_t n);        // attention_ops.rs:1040-1046

// ---- RMSNorm + RoPE (src/decoder/attention_ops.rs:598-887) ----------------
struct RopeParams {
  float theta;
  size_t frequency_dim;
  float position_scale;
};
enum RopeStyle : int32_t { ROPE_INTERLEAVED = 0, ROPE_HALVES = 1 };
void rope_rotations(size_t position, size_t rope_dims, RopeParams rope, float* cos_out,
                    float* sin_out);  // :848-887, pairs = rope_dims/2 entries
Status rms_norm_heads(const float* x, size_t seq, size_t heads, size_t head_dim, const float* weight,
                      float eps, float* out);  // :598-636
Status apply_rope_heads_at(const float* x, size_t seq, size_t heads, size_t head_dim,
                           size_t rope_dims, RopeParams rope, size_t position_offset,
                           RopeStyle style, float* out);  // :779-836
Status rms_norm_rope_heads_at(const float* x, size_t seq, size_t heads, size_t head_dim,
                              size_t rope_dims, const float* weight, float eps, RopeParams rope,
                              size_t position_offset, RopeStyle style, float* out);  // :682-777

// ---- u8 group-32 affine KV (PARITY UNPINNED on the encode side) ----------
// Dequant is the reference's affine formula q*scale+bias (src/quantization.rs:173-179)
// with bf16 scale/bias (README.md:32). The encoder is defined HERE because the
// reference has none; per group of 32 contiguous elements of one head row:
//   bias  = bf16_rne(min(x))
//   scale = bf16_rne(max((max(x) - bias) / 255, 2^-40))
//   q     = clamp(rint((x - bias) / scale), 0, 255)   (IEEE divide, half-to-even)
constexpr size_t QGROUP = 32;
void quantize_group_u8(const float* x, uint8_t* codes, uint16_t* scale_bits, uint16_t* bias_bits);
void quantize_row_u8(const float* x, size_t n, uint8_t* codes, uint16_t* scale_bits,
                     uint16_t* bias_bits);
void dequantize_row_u8(const uint8_t* codes, const uint16_t* scale_bits, const uint16_t* bias_bits,
                       size_t n, float* out);

// ---- SHA-256 + block hash chain (src/serve/cache.rs:11-47) ----------------
struct Hash32 {
  uint8_t b[32];
  bool operator==(const Hash32& o) const;
};
void sha256(const uint8_t* data, size_t n, uint8_t out[32]);  // FIPS 180-4 (sha2 0.10.9 upstream)
Hash32 block_hash_root();
Hash32 block_hash_for_session(const char* key, size_t key_len, bool present);
Hash32 block_hash_chain(const Hash32& prev, const uint64_t* tokens, size_t n);

// ---- BlockAwarePrefixCache (src/serve/cache.rs:62-219) --------------------
struct PrefixEntry {
  Hash32 session, hash;
  size_t tokens;
  uint64_t payload;  // stands for (state, metal): an opaque snapshot id
  size_t bytes;
};
struct PrefixHit {
  bool found = false;
  size_t tokens = 0;
  Hash32 hash{};
  uint64_t payload = 0;
};
struct BlockAwarePrefixCache {
  size_t block_tokens, capacity, blocks_per_session;
  std::vector<PrefixEntry> entries;          // index 0 = most recent
  std::vector<PrefixEntry> evicted_log;      // every entry that left, in order
  BlockAwarePrefixCache(size_t block_tokens, size_t capacity, size_t blocks_per_session);
  PrefixHit match_prefix(const Hash32& root, const uint64_t* tokens, size_t n);
  size_t insert(const Hash32& session, const Hash32& hash, size_t tokens, uint64_t payload,
                size_t bytes);
  bool evict_lru_block(size_t* bytes_out);
  size_t estimated_bytes() const;
  size_t session_block_count(const Hash32& session) const;
};
// Decoder-internal longest-prefix selection (src/decoder/generation.rs:190-204).
long longest_prefix_entry_index(const std::vector<std::vector<uint64_t>>& entries,
                                const uint64_t* prompt, size_t n);

// ---- memory budget (src/memory_guard.rs:155-185,331-370) ------------------
struct MemoryLimits {
  bool has_static = false, has_host = false, has_device = false;
  uint64_t static_cap = 0, host_memory = 0, headroom_bytes = 0, device_cap = 0;
  bool effective_limit(uint64_t* out) const;
};
struct MemoryProjection {
  uint64_t current, reserved, requested, projected, limit, available;
};
struct MemoryGuard {
  MemoryLimits limits;
  uint64_t current = 0, reserved = 0;
  bool enabled = true;
  bool projection(uint64_t requested, MemoryProjection* out) const;
  bool projection_over_limit(uint64_t requested, MemoryProjection* out) const;
  bool check_allocation(uint64_t requested, MemoryProjection* over) const;  // true = accepted
};

// ---- linear-attention recurrent state (src/linear_attention.rs:194-231;
//      src/metal_backend/linear_attention.rs:3027-3198) --------------------
struct LinearState {
  std::vector<float> conv;   // [(K-1), conv_dim]
  std::vector<float> ssm;    // [H_v][d_v][d_k]; holds bf16-rounded values when ssm_bf16
  bool ssm_bf16 = false;
};
LinearState linear_state_snapshot(const LinearState& s);
Status linear_state_restore(LinearState* state, const LinearState& snapshot);
// One decode token of the Gated DeltaNet recurrence on the SSM state [H_v][d_v][d_k]
// (src/linear_attention.rs:896-991): per value head h (key head h / repeat), per state row:
//   S *= g; kv = S.k; delta = (v - kv) * beta; S += delta * k; y = S.q     (sequential f32 sums)
struct LinearShape {
  size_t num_key_heads, num_value_heads, key_head_dim, value_head_dim, conv_kernel_dim;
};
Status gated_delta_step(const float* q, const float* k, const float* v, const float* g, const float* beta,
                        const LinearShape& shape, std::vector<float>* ssm, float* out);
// Depthwise causal conv of one token with the sliding history [(K-1), conv_dim]
// (src/linear_attention.rs:802-852); weight is [conv_dim][K].
Status depthwise_conv_step(const float* qkv, const float* weight, size_t conv_dim, size_t kernel,
                           std::vector<float>* history, float* out);

// Greedy epilogue: logits = W . x for a biasless [vocab][hidden] weight (sequential f32 sums), then
// the FIRST maximum (src/sampling.rs:49-62: a later equal value does not replace the best; the Metal
// path breaks ties the same way, src/kernels.metal:8362-8440). ERR_DIMENSION when vocab is 0 (the
// reference returns None).
Status lm_head_argmax(const float* weight, size_t vocab, size_t hidden, const float* x, size_t* index, float* value);

// Token feed: out = table[token] * scale, rounded to bf16 (RNE) and widened again when recast_bf16
// (embed_gather_dense_from_u32_f32, src/kernels.metal:308-325). A token outside the table leaves out
// untouched and returns false.
bool embed_gather(const float* table, size_t vocab, size_t dim, size_t token, float scale, bool recast_bf16, float* out);

// ---- deterministic input generators ---------------------------------------
// pseudo(): the closed form of the reference's tests (src/decode_resident/tests.rs:544-547).
float pseudo(uint64_t seed);
// Counter-based approximate N(0,1): integer-only (exactly reproducible on host,
// in numpy and on the device): two splitmix64 draws, the sum of their eight
// 16-bit fields, centred and scaled to unit variance (Irwin-Hall, n = 8).
uint64_t splitmix64(uint64_t x);
float normal8(uint64_t seed, uint64_t stream, uint64_t index);
void fill_normal8(float* out, size_t n, uint64_t seed, uint64_t stream, uint64_t index0);

}  // namespace sgo
