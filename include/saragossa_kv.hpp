// saragossa_kv.hpp — C++ host face of libsgk, named after the reference's Rust surface.
//
// The reference's host language is Rust; where no Rust toolchain exists this header is the
// host layer above the C ABI (sgk.h): same type and method names, same argument meaning,
// same error behaviour as the crate's resident-cache API, so a test written against it reads
// like the reference's own tests. Every fallible method returns Result<T>, a value or an
// InferError whose kind is the reference's variant (src/error.rs:12-75); nothing throws.
// The types are move-only: a resident KV state belongs to one decode and is never cloned
// (src/decode_resident.rs:21-27).
#pragma once
#include <cctype>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <utility>
#include <array>
#include <vector>

#include "sgk.h"

namespace saragossa {

struct InferError {
  enum Kind { None = 0, Dimension = 1, Config = 2, Metal = 3, MemoryGuard = 4, Shape = 5, Timeout = 6 };
  Kind kind = None;
  std::string message;
};

template <class T>
struct Result {
  bool ok = false;
  T value{};
  InferError error;
  static Result Ok(T v) {
    Result r;
    r.ok = true;
    r.value = std::move(v);
    return r;
  }
  static Result Err(int32_t code) {
    Result r;
    r.error.kind = static_cast<InferError::Kind>(code);
    r.error.message = sgk_last_error();
    return r;
  }
  bool is_err() const { return !ok; }
};
struct Unit {};

enum class GpuElement : int32_t { F32 = SGK_KV_F32, Bf16 = SGK_KV_BF16, U8G32 = SGK_KV_U8G32 };

// KV dtype policy of the reference (src/decode_resident/utils.rs:202-228): an explicit
// RETI_RUST_KV_BF16 (1/true/on, 0/false/off) wins; otherwise bf16 when sampling, f32 greedy.
inline bool kv_bf16_for(bool sampled) {
  const char* e = std::getenv("RETI_RUST_KV_BF16");
  if (e != nullptr) {
    std::string v(e);
    size_t a = v.find_first_not_of(" \t"), b = v.find_last_not_of(" \t");
    v = a == std::string::npos ? "" : v.substr(a, b - a + 1);
    for (auto& c : v) c = static_cast<char>(std::tolower(c));
    if (v == "1" || v == "true" || v == "on") return true;
    if (v == "0" || v == "false" || v == "off") return false;
  }
  return sampled;
}

// FullAttentionMetalState (src/decode_resident/attention.rs:446-1038).
class FullAttentionState {
 public:
  FullAttentionState() = default;
  explicit FullAttentionState(sgk_kv* h) : h_(h) {}
  FullAttentionState(FullAttentionState&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
  FullAttentionState& operator=(FullAttentionState&& o) noexcept {
    if (this != &o) {
      reset();
      h_ = o.h_;
      o.h_ = nullptr;
    }
    return *this;
  }
  FullAttentionState(const FullAttentionState&) = delete;
  FullAttentionState& operator=(const FullAttentionState&) = delete;
  ~FullAttentionState() { reset(); }

  size_t kv_dim() const { return static_cast<size_t>(sgk_kv_kv_dim(h_)); }
  size_t len() const { return static_cast<size_t>(sgk_kv_len(h_)); }
  size_t capacity() const { return static_cast<size_t>(sgk_kv_capacity(h_)); }
  size_t q_heads() const { return static_cast<size_t>(sgk_kv_q_heads(h_)); }
  size_t kv_heads() const { return static_cast<size_t>(sgk_kv_kv_heads(h_)); }
  size_t head_dim() const { return static_cast<size_t>(sgk_kv_head_dim(h_)); }
  GpuElement element() const { return static_cast<GpuElement>(sgk_kv_dtype(h_)); }
  size_t byte_len() const { return static_cast<size_t>(sgk_kv_byte_len(h_)); }

  Result<Unit> truncate(size_t len) { return unit(sgk_kv_truncate(h_, static_cast<int64_t>(len))); }
  Result<Unit> seed(const std::vector<float>& keys_rows, const std::vector<float>& values_rows, size_t n_rows) {
    return unit(sgk_kv_seed_f32(h_, keys_rows.data(), keys_rows.size(), values_rows.data(), values_rows.size(),
                                static_cast<int64_t>(n_rows)));
  }
  Result<Unit> append_row(const std::vector<float>& key, const std::vector<float>& value) {
    return unit(sgk_kv_append_row_f32(h_, key.data(), key.size(), value.data(), value.size()));
  }
  Result<std::vector<float>> attention_decode(const std::vector<float>& q) { return attention_decode_windowed(q, 0); }
  Result<std::vector<float>> attention_decode_windowed(const std::vector<float>& q, size_t window_start) {
    std::vector<float> out(q_heads() * head_dim());
    int32_t rc = sgk_kv_attention_decode(h_, q.data(), q.size(), static_cast<int64_t>(window_start), 0.0f, out.data());
    if (rc != SGK_OK) return Result<std::vector<float>>::Err(rc);
    return Result<std::vector<float>>::Ok(std::move(out));
  }
  // encode_* only enqueue (stream = the "encoder"); d_* are device pointers.
  Result<Unit> encode_append_kv(void* stream, const float* d_k, const float* d_v) {
    return unit(sgk_kv_enqueue_append(h_, stream, d_k, d_v));
  }
  Result<Unit> encode_attention_decode_windowed(void* stream, const float* d_q, float* d_out, size_t window_start) {
    return unit(sgk_kv_enqueue_attention(h_, stream, d_q, d_out, static_cast<int64_t>(window_start), 0.0f));
  }
  // One launch for append + attention (the fused form of the two calls above).
  Result<Unit> encode_append_attention(void* stream, const float* d_k, const float* d_v, const float* d_q, float* d_out,
                                       size_t sliding_window = 0) {
    return unit(sgk_kv_enqueue_append_attention(h_, stream, d_k, d_v, d_q, d_out, static_cast<int64_t>(sliding_window), 0.0f));
  }
  // Speculative verify of n_rows draft rows (src/decode_resident/layers.rs:1295-1433); d_* are [n_rows][...].
  Result<Unit> encode_verify_rows(void* stream, const float* d_k, const float* d_v, const float* d_q, float* d_out,
                                  size_t n_rows, size_t sliding_window = 0) {
    return unit(sgk_kv_enqueue_verify_rows(h_, stream, d_k, d_v, d_q, d_out, static_cast<int32_t>(n_rows),
                                           static_cast<int64_t>(sliding_window), 0.0f));
  }
  // Prompt rows: RMSNorm + RoPE on K at positions len.., storage rounding, pages; one launch.
  Result<Unit> encode_rope_append_rows(void* stream, const float* d_k_raw, const float* d_v, size_t n_rows,
                                       const float* d_knorm_weight, size_t rope_dims, float theta, float eps) {
    sgk_rope rope{static_cast<int32_t>(rope_dims), static_cast<int32_t>(rope_dims), theta, 1.0f, eps, 0};
    return unit(sgk_kv_enqueue_rope_append_rows(h_, stream, d_k_raw, d_v, static_cast<int64_t>(n_rows), d_knorm_weight, &rope));
  }
  // kv.keys() / kv.values() read-back of the valid rows, decoded to f32.
  Result<std::vector<float>> keys() { return rows(true); }
  Result<std::vector<float>> values() { return rows(false); }
  // raw bf16 bit patterns of the valid rows (bf16 states only)
  Result<std::vector<uint16_t>> keys_bf16_bits() {
    std::vector<uint16_t> k(len() * kv_dim()), v(len() * kv_dim());
    int32_t rc = sgk_kv_gather_rows(h_, 0, static_cast<int64_t>(len()), k.data(), v.data());
    if (rc != SGK_OK) return Result<std::vector<uint16_t>>::Err(rc);
    return Result<std::vector<uint16_t>>::Ok(std::move(k));
  }
  sgk_kv* handle() const { return h_; }

 private:
  static Result<Unit> unit(int32_t rc) { return rc == SGK_OK ? Result<Unit>::Ok(Unit{}) : Result<Unit>::Err(rc); }
  Result<std::vector<float>> rows(bool want_keys) {
    std::vector<float> k(len() * kv_dim()), v(len() * kv_dim());
    int32_t rc = sgk_kv_gather_rows_f32(h_, 0, static_cast<int64_t>(len()), k.data(), v.data());
    if (rc != SGK_OK) return Result<std::vector<float>>::Err(rc);
    return Result<std::vector<float>>::Ok(std::move(want_keys ? k : v));
  }
  void reset() {
    if (h_) sgk_kv_destroy(h_);
    h_ = nullptr;
  }
  sgk_kv* h_ = nullptr;
};

// DecodeResidentState (src/decode_resident/arena.rs:247-349).
class DecodeResidentState {
 public:
  DecodeResidentState() = default;
  DecodeResidentState(DecodeResidentState&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
  DecodeResidentState& operator=(DecodeResidentState&& o) noexcept {
    if (this != &o) {
      if (h_) sgk_state_destroy(h_);
      h_ = o.h_;
      o.h_ = nullptr;
    }
    return *this;
  }
  DecodeResidentState(const DecodeResidentState&) = delete;
  DecodeResidentState& operator=(const DecodeResidentState&) = delete;
  ~DecodeResidentState() {
    if (h_) sgk_state_destroy(h_);
  }
  static Result<DecodeResidentState> create(int device = 0) {
    sgk_state* h = nullptr;
    int32_t rc = sgk_state_create(device, &h);
    if (rc != SGK_OK) return Result<DecodeResidentState>::Err(rc);
    DecodeResidentState s;
    s.h_ = h;
    return Result<DecodeResidentState>::Ok(std::move(s));
  }
  // state.full_attention(capacity, q_heads, kv_heads, head_dim, sampled)
  Result<FullAttentionState> full_attention(size_t capacity, size_t q_heads, size_t kv_heads, size_t head_dim,
                                            bool sampled) {
    return full_attention_with_element(capacity, q_heads, kv_heads, head_dim,
                                       kv_bf16_for(sampled) ? GpuElement::Bf16 : GpuElement::F32);
  }
  Result<FullAttentionState> full_attention_with_element(size_t capacity, size_t q_heads, size_t kv_heads,
                                                         size_t head_dim, GpuElement element) {
    sgk_kv* kv = nullptr;
    int32_t rc = sgk_kv_create(h_, static_cast<int64_t>(capacity), static_cast<int32_t>(q_heads),
                               static_cast<int32_t>(kv_heads), static_cast<int32_t>(head_dim),
                               static_cast<int32_t>(element), SGK_PAGE_TOKENS, &kv);
    if (rc != SGK_OK) return Result<FullAttentionState>::Err(rc);
    return Result<FullAttentionState>::Ok(FullAttentionState(kv));
  }
  Result<std::vector<float>> rms_norm_rope_decode(const std::vector<float>& x, const std::vector<float>& weight,
                                                  size_t heads, size_t head_dim, size_t rope_dims, size_t position,
                                                  float eps, float theta) {
    sgk_rope rope{static_cast<int32_t>(rope_dims), static_cast<int32_t>(rope_dims), theta, 1.0f, eps, 0};
    std::vector<float> out(heads * head_dim);
    int32_t rc = sgk_rms_norm_rope_decode(h_, x.data(), weight.data(), static_cast<int32_t>(heads),
                                          static_cast<int32_t>(head_dim), &rope, static_cast<int64_t>(position),
                                          out.data());
    if (rc != SGK_OK) return Result<std::vector<float>>::Err(rc);
    return Result<std::vector<float>>::Ok(std::move(out));
  }
  // encode_lm_head_argmax (src/metal_backend/lm_head.rs:288-337) for a dense biasless weight; n_rows > 1 is
  // the verify form (:766-820). Enqueue only: the indices land in d_index_out on the device.
  Result<Unit> encode_lm_head_argmax(void* stream, const void* d_weight, GpuElement weight_element, size_t vocab,
                                     size_t hidden, const float* d_x, size_t n_rows, int32_t* d_index_out,
                                     int32_t index_offset = 0, float* d_value_out = nullptr) {
    return unit(sgk_lm_head_enqueue_argmax(h_, stream, d_weight, static_cast<int32_t>(weight_element),
                                           static_cast<int64_t>(vocab), static_cast<int32_t>(hidden), d_x,
                                           static_cast<int32_t>(n_rows), index_offset, d_index_out, d_value_out));
  }
  // encode_affine_argmax_qmv_fast (src/metal_backend/lm_head.rs:934-990): the same epilogue over an
  // affine-quantised weight (u32 code words, bf16 scales and biases per group of 64 or 128 inputs).
  Result<Unit> encode_lm_head_argmax_affine(void* stream, const uint32_t* d_packed, const uint16_t* d_scales,
                                            const uint16_t* d_biases, size_t bits, size_t group_size, size_t vocab,
                                            size_t hidden, const float* d_x, size_t n_rows, int32_t* d_index_out,
                                            int32_t index_offset = 0, float* d_value_out = nullptr) {
    sgk_affine_weight w{d_packed, d_scales, d_biases, static_cast<int32_t>(bits), static_cast<int32_t>(group_size)};
    return unit(sgk_lm_head_enqueue_argmax_affine(h_, stream, &w, static_cast<int64_t>(vocab),
                                                  static_cast<int32_t>(hidden), d_x, static_cast<int32_t>(n_rows),
                                                  index_offset, d_index_out, d_value_out));
  }
  sgk_state* handle() const { return h_; }

 private:
  static Result<Unit> unit(int32_t rc) { return rc == SGK_OK ? Result<Unit>::Ok(Unit{}) : Result<Unit>::Err(rc); }
  sgk_state* h_ = nullptr;
};

// One rank's end of the output exchange between GPUs that share one sequence by KV-head group
// (sgk_exchange_*; the reference runs on one device and has no counterpart). handle() goes to the
// peers over the host's own channel, connect() takes theirs.
class OutputExchange {
 public:
  OutputExchange() = default;
  OutputExchange(OutputExchange&& o) noexcept : h_(o.h_), handle_(o.handle_) { o.h_ = nullptr; }
  OutputExchange& operator=(OutputExchange&& o) noexcept {
    if (this != &o) {
      if (h_) sgk_exchange_destroy(h_);
      h_ = o.h_;
      handle_ = o.handle_;
      o.h_ = nullptr;
    }
    return *this;
  }
  OutputExchange(const OutputExchange&) = delete;
  OutputExchange& operator=(const OutputExchange&) = delete;
  ~OutputExchange() {
    if (h_) sgk_exchange_destroy(h_);
  }
  static Result<OutputExchange> create(DecodeResidentState& state, int rank, int n_ranks) {
    OutputExchange ex;
    int32_t rc = sgk_exchange_create(state.handle(), rank, n_ranks, &ex.h_, ex.handle_.data());
    if (rc != SGK_OK) return Result<OutputExchange>::Err(rc);
    return Result<OutputExchange>::Ok(std::move(ex));
  }
  const std::array<uint8_t, 64>& handle() const { return handle_; }
  Result<Unit> connect(int peer_rank, const std::array<uint8_t, 64>& peer_handle) {
    return unit(sgk_exchange_connect(h_, peer_rank, peer_handle.data()));
  }
  // the exchange as a kernel of its own, after an attention launch that wrote the local slice
  Result<Unit> encode(void* stream, float* d_local_row, float* const* d_peer_rows, size_t slice_offset,
                      size_t slice_floats) {
    return unit(sgk_exchange_enqueue(h_, stream, d_local_row, d_peer_rows, static_cast<int64_t>(slice_offset),
                                     static_cast<int32_t>(slice_floats)));
  }
  sgk_exchange* raw() const { return h_; }

 private:
  static Result<Unit> unit(int32_t rc) { return rc == SGK_OK ? Result<Unit>::Ok(Unit{}) : Result<Unit>::Err(rc); }
  sgk_exchange* h_ = nullptr;
  std::array<uint8_t, 64> handle_{};
};

// LinearAttentionMetalState of all recurrent layers (src/metal_backend/mod.rs:507-531) with the
// decode step on it (src/linear_attention.rs:802-852,896-991) and the snapshot / restore /
// per-row capture copies (src/metal_backend/linear_attention.rs:44-127,3027-3198).
class LinearAttentionState {
 public:
  LinearAttentionState() = default;
  explicit LinearAttentionState(sgk_linstate* h) : h_(h) {}
  LinearAttentionState(LinearAttentionState&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
  LinearAttentionState& operator=(LinearAttentionState&& o) noexcept {
    if (this != &o) {
      if (h_) sgk_linstate_destroy(h_);
      h_ = o.h_;
      o.h_ = nullptr;
    }
    return *this;
  }
  LinearAttentionState(const LinearAttentionState&) = delete;
  LinearAttentionState& operator=(const LinearAttentionState&) = delete;
  ~LinearAttentionState() {
    if (h_) sgk_linstate_destroy(h_);
  }
  static Result<LinearAttentionState> create(DecodeResidentState& state, size_t layers, size_t conv_len, size_t ssm_len,
                                             bool ssm_bf16) {
    sgk_linstate* h = nullptr;
    int32_t rc = sgk_linstate_create(state.handle(), static_cast<int32_t>(layers), static_cast<int64_t>(conv_len),
                                     static_cast<int64_t>(ssm_len), ssm_bf16 ? 1 : 0, &h);
    if (rc != SGK_OK) return Result<LinearAttentionState>::Err(rc);
    return Result<LinearAttentionState>::Ok(LinearAttentionState(h));
  }
  size_t estimated_bytes() const { return static_cast<size_t>(sgk_linstate_bytes(h_)); }
  Result<Unit> write(size_t layer, const std::vector<float>& conv, const std::vector<float>& ssm) {
    return unit(sgk_linstate_write(h_, static_cast<int32_t>(layer), conv.empty() ? nullptr : conv.data(), ssm.data()));
  }
  Result<Unit> read(size_t layer, std::vector<float>& conv, std::vector<float>& ssm) {
    return unit(sgk_linstate_read(h_, static_cast<int32_t>(layer), conv.empty() ? nullptr : conv.data(), ssm.data()));
  }
  Result<LinearAttentionState> snapshot(void* stream = nullptr) {
    sgk_linstate* snap = nullptr;
    int32_t rc = sgk_linstate_snapshot(h_, stream, &snap);
    if (rc != SGK_OK) return Result<LinearAttentionState>::Err(rc);
    return Result<LinearAttentionState>::Ok(LinearAttentionState(snap));
  }
  Result<Unit> restore(const LinearAttentionState& snap, void* stream = nullptr) {
    return unit(sgk_linstate_restore(h_, stream, snap.h_));
  }
  Result<Unit> encode_capture(LinearAttentionState& capture, void* stream = nullptr) {
    return unit(sgk_linstate_enqueue_capture(h_, stream, capture.h_));
  }
  Result<Unit> encode_conv_step(void* stream, size_t layer, const float* d_qkv, const float* d_weight, size_t conv_dim,
                                size_t conv_kernel_dim, float* d_out) {
    return unit(sgk_linstate_enqueue_conv_step(h_, stream, static_cast<int32_t>(layer), d_qkv, d_weight,
                                               static_cast<int32_t>(conv_dim), static_cast<int32_t>(conv_kernel_dim), d_out));
  }
  Result<Unit> encode_gated_delta_step(void* stream, size_t layer, size_t num_key_heads, size_t num_value_heads,
                                       size_t key_head_dim, size_t value_head_dim, const float* d_q, const float* d_k,
                                       const float* d_v, const float* d_g, const float* d_beta, float* d_out) {
    sgk_linear_shape shape{static_cast<int32_t>(num_key_heads), static_cast<int32_t>(num_value_heads),
                           static_cast<int32_t>(key_head_dim), static_cast<int32_t>(value_head_dim)};
    return unit(sgk_linstate_enqueue_gated_delta_step(h_, stream, static_cast<int32_t>(layer), &shape, d_q, d_k, d_v, d_g,
                                                      d_beta, d_out));
  }
  // The resident decode of a recurrent layer between its projections in one launch
  // (src/linear_attention.rs:313-342; linear_attn_conv_norm_gates_k4_dk128_f32 + linear_attn_gated_delta_dk128_tg4_f32).
  Result<Unit> encode_decode_step(void* stream, size_t layer, size_t num_key_heads, size_t num_value_heads,
                                  const float* d_qkv, const float* d_conv_weight, size_t conv_kernel_dim,
                                  const float* d_beta_input, const float* d_gate_input, const float* d_a_log,
                                  const float* d_dt_bias, float* d_out) {
    sgk_linear_shape shape{static_cast<int32_t>(num_key_heads), static_cast<int32_t>(num_value_heads), 128, 128};
    return unit(sgk_linstate_enqueue_decode_step(h_, stream, static_cast<int32_t>(layer), &shape, d_qkv, d_conv_weight,
                                                 static_cast<int32_t>(conv_kernel_dim), d_beta_input, d_gate_input,
                                                 d_a_log, d_dt_bias, d_out));
  }
  sgk_linstate* handle() const { return h_; }

 private:
  static Result<Unit> unit(int32_t rc) { return rc == SGK_OK ? Result<Unit>::Ok(Unit{}) : Result<Unit>::Err(rc); }
  sgk_linstate* h_ = nullptr;
};

// BlockHash (src/serve/cache.rs:11-47).
struct BlockHash {
  uint8_t bytes[32];
  static BlockHash root() {
    BlockHash h;
    sgk_hash_root(h.bytes);
    return h;
  }
  static BlockHash for_session(const char* session_key) {  // nullptr = None
    BlockHash h;
    sgk_hash_for_session(session_key, session_key ? std::strlen(session_key) : 0, session_key != nullptr, h.bytes);
    return h;
  }
  BlockHash chain(const std::vector<uint64_t>& tokens) const {
    BlockHash h;
    sgk_hash_chain(bytes, tokens.data(), tokens.size(), h.bytes);
    return h;
  }
  bool operator==(const BlockHash& o) const { return std::memcmp(bytes, o.bytes, 32) == 0; }
  bool operator!=(const BlockHash& o) const { return !(*this == o); }
};

struct PrefixBlockHit {
  size_t tokens = 0;
  BlockHash hash{};
  uint64_t entry = 0;
};

// BlockAwarePrefixCache (src/serve/cache.rs:74-219), bookkeeping form (no pool).
class BlockAwarePrefixCache {
 public:
  BlockAwarePrefixCache(size_t block_tokens, size_t capacity) : BlockAwarePrefixCache(block_tokens, capacity, capacity) {}
  BlockAwarePrefixCache(size_t block_tokens, size_t capacity, size_t blocks_per_session) {
    sgk_prefix_create(nullptr, static_cast<int64_t>(block_tokens), static_cast<int64_t>(capacity),
                      static_cast<int64_t>(blocks_per_session), 0, &h_);
  }
  BlockAwarePrefixCache(const BlockAwarePrefixCache&) = delete;
  BlockAwarePrefixCache& operator=(const BlockAwarePrefixCache&) = delete;
  ~BlockAwarePrefixCache() { sgk_prefix_destroy(h_); }
  size_t block_tokens() const { return static_cast<size_t>(sgk_prefix_block_tokens(h_)); }
  // Some(hit) / None as {found, hit}
  std::pair<bool, PrefixBlockHit> match_prefix(const BlockHash& root, const std::vector<uint64_t>& tokens) {
    PrefixBlockHit hit;
    int64_t n = 0;
    sgk_prefix_match(h_, root.bytes, tokens.data(), tokens.size(), &n, hit.hash.bytes, &hit.entry);
    hit.tokens = static_cast<size_t>(n);
    return {hit.entry != 0, hit};
  }
  bool insert(const BlockHash& session, const BlockHash& hash, size_t tokens) {
    int32_t inserted = 0;
    sgk_prefix_insert(h_, session.bytes, hash.bytes, static_cast<int64_t>(tokens), nullptr, nullptr, nullptr, &inserted);
    return inserted != 0;
  }
  // prefill_prompt_state's loop over the full blocks of a prompt (src/serve/state.rs:596-604) in one call;
  // returns the number of blocks inserted.
  size_t insert_chain(const BlockHash& root, const std::vector<uint64_t>& tokens, size_t from_tokens = 0) {
    int32_t inserted = 0;
    sgk_prefix_insert_chain(h_, root.bytes, tokens.data(), tokens.size(), static_cast<int64_t>(from_tokens), nullptr,
                            nullptr, &inserted, nullptr);
    return static_cast<size_t>(inserted);
  }
  bool evict_lru_block() {
    int32_t ev = 0;
    sgk_prefix_evict_lru(h_, &ev, nullptr);
    return ev != 0;
  }
  size_t estimated_bytes() const { return static_cast<size_t>(sgk_prefix_bytes(h_)); }
  size_t session_block_count(const BlockHash& s) const { return static_cast<size_t>(sgk_prefix_session_count(h_, s.bytes)); }
  std::vector<BlockHash> entry_hashes() const {  // front (most recent) to rear
    int64_t n = sgk_prefix_len(h_);
    std::vector<uint8_t> raw(static_cast<size_t>(n) * 32);
    sgk_prefix_dump(h_, 0, n, nullptr, raw.data(), nullptr);
    std::vector<BlockHash> out(static_cast<size_t>(n));
    for (int64_t i = 0; i < n; ++i) std::memcpy(out[static_cast<size_t>(i)].bytes, raw.data() + 32 * i, 32);
    return out;
  }

 private:
  sgk_prefix* h_ = nullptr;
};

// The decoder's own prefix cache (prefix_cache_get / prefix_cache_put, src/decoder/generation.rs:2998-3139),
// bookkeeping form (no pool): at most `capacity` prompts, the most recent at the front; get moves the entry
// with the longest token prefix of the prompt to the front and returns its length (0: miss).
class PrefixCache {
 public:
  explicit PrefixCache(size_t capacity) { sgk_dprefix_create(nullptr, static_cast<int64_t>(capacity), &h_); }
  PrefixCache(const PrefixCache&) = delete;
  PrefixCache& operator=(const PrefixCache&) = delete;
  ~PrefixCache() { sgk_dprefix_destroy(h_); }
  size_t get(const std::vector<uint64_t>& prompt) {
    int64_t cached = 0;
    sgk_dprefix_get(h_, prompt.data(), prompt.size(), nullptr, nullptr, nullptr, &cached);
    return static_cast<size_t>(cached);
  }
  void put(const std::vector<uint64_t>& tokens) { sgk_dprefix_put(h_, tokens.data(), tokens.size(), nullptr, nullptr, nullptr); }
  size_t len() const { return static_cast<size_t>(sgk_dprefix_len(h_)); }
  std::vector<uint64_t> entry_tokens(size_t index) const {  // front = 0; empty past the end
    std::vector<uint64_t> out(4096);
    int64_t n = sgk_dprefix_entry_tokens(h_, static_cast<int64_t>(index), out.data(), static_cast<int64_t>(out.size()));
    out.resize(n > 0 ? static_cast<size_t>(n) : 0);
    return out;
  }

 private:
  sgk_dprefix* h_ = nullptr;
};

}  // namespace saragossa
