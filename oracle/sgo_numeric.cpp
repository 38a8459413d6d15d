// CPU oracle (test infrastructure only): numeric half of the path.
// Every function cites the reference lines it restates; see sgo.hpp for pinning.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <thread>

#include "sgo.hpp"

namespace sgo {

// ---- bf16 (src/decode_resident/utils.rs:55-60) ----------------------------
// bits + 0x7fff + lsb, then >> 16. No NaN special case, exactly like the reference.
uint16_t f32_to_bf16_bits(float value) {
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  uint32_t lsb = (bits >> 16) & 1u;
  uint32_t rounded = bits + (0x7fffu + lsb);  // wrapping add
  return static_cast<uint16_t>(rounded >> 16);
}

float bf16_bits_to_f32(uint16_t bits) {
  uint32_t wide = static_cast<uint32_t>(bits) << 16;
  float out;
  std::memcpy(&out, &wide, 4);
  return out;
}

float bf16_round_f32(float value) { return bf16_bits_to_f32(f32_to_bf16_bits(value)); }

// ---- LayerKvCache (src/decoder/attention_cache.rs:7-100) -------------------
Status LayerKvCache::append(const float* key, size_t key_rows, size_t key_dim, const float* value,
                            size_t value_rows, size_t value_dim, size_t expected_dim) {
  // :15-23 — both operands must be exactly [1, expected_dim].
  if (key_rows != 1 || value_rows != 1 || key_dim != expected_dim || value_dim != expected_dim)
    return ERR_DIMENSION;
  // :24-32 — the first append fixes kv_dim, later ones must agree.
  if (has_dim && kv_dim != expected_dim) return ERR_DIMENSION;
  if (!has_dim) {
    has_dim = true;
    kv_dim = expected_dim;
  }
  keys.insert(keys.end(), key, key + expected_dim);
  values.insert(values.end(), value, value + expected_dim);
  return OK;
}

Status LayerKvCache::append_batch(const float* key, size_t key_rows, size_t key_dim,
                                  const float* value, size_t value_rows, size_t value_dim,
                                  size_t expected_dim) {
  // :47-58 — seq > 0, same row count, both [seq, expected_dim].
  if (key_rows == 0 || key_rows != value_rows || key_dim != expected_dim ||
      value_dim != expected_dim)
    return ERR_DIMENSION;
  if (has_dim && kv_dim != expected_dim) return ERR_DIMENSION;
  if (!has_dim) {
    has_dim = true;
    kv_dim = expected_dim;
  }
  keys.insert(keys.end(), key, key + key_rows * expected_dim);
  values.insert(values.end(), value, value + value_rows * expected_dim);
  return OK;
}

size_t LayerKvCache::len() const {  // :72-77
  if (has_dim && kv_dim > 0) return keys.size() / kv_dim;
  return 0;
}

Status LayerKvCache::truncate(size_t new_rows) {  // :79-100
  if (!has_dim) return new_rows == 0 ? OK : ERR_DIMENSION;
  if (kv_dim != 0 && new_rows > std::numeric_limits<size_t>::max() / kv_dim) return ERR_DIMENSION;
  size_t cells = new_rows * kv_dim;
  if (cells > keys.size() || cells > values.size()) return ERR_DIMENSION;
  keys.resize(cells);
  values.resize(cells);
  return OK;
}

// ---- ResidentKv (src/decode_resident/attention.rs:56-108,501-644) ----------
Status ResidentKv::create(size_t capacity, size_t q_heads, size_t kv_heads, size_t head_dim,
                          KvDtype dtype, ResidentKv* out) {
  // :64-68 zero dimension => Config; :69-74 q_heads % kv_heads != 0 => Config.
  if (capacity == 0 || q_heads == 0 || kv_heads == 0 || head_dim == 0) return ERR_CONFIG;
  if (q_heads % kv_heads != 0) return ERR_CONFIG;
  // A u8 row is quantised per 32 elements of one head row (format defined in sgo.hpp).
  if (dtype == KV_U8G32 && head_dim % QGROUP != 0) return ERR_CONFIG;
  out->capacity = capacity;
  out->len = 0;
  out->q_heads = q_heads;
  out->kv_heads = kv_heads;
  out->head_dim = head_dim;
  out->dtype = dtype;
  out->keys.assign(capacity * kv_heads * head_dim, 0.0f);
  out->values.assign(capacity * kv_heads * head_dim, 0.0f);
  return OK;
}

static void store_values(KvDtype dtype, const float* in, size_t n, float* out) {
  switch (dtype) {
    case KV_F32:
      std::memcpy(out, in, n * sizeof(float));
      break;
    case KV_BF16:  // write_f32_as_bf16_at, utils.rs:76-110
      for (size_t i = 0; i < n; ++i) out[i] = bf16_round_f32(in[i]);
      break;
    case KV_U8G32: {
      std::vector<uint8_t> codes(n);
      std::vector<uint16_t> scale(n / QGROUP), bias(n / QGROUP);
      quantize_row_u8(in, n, codes.data(), scale.data(), bias.data());
      dequantize_row_u8(codes.data(), scale.data(), bias.data(), n, out);
      break;
    }
  }
}

void ResidentKv::store_row(size_t row, const float* k, const float* v) {
  size_t d = kv_dim();
  store_values(dtype, k, d, keys.data() + row * d);
  store_values(dtype, v, d, values.data() + row * d);
}

Status ResidentKv::seed(const float* k, size_t k_len, const float* v, size_t v_len, size_t n_rows) {
  // :555-572 — n_rows <= capacity and both inputs exactly n_rows*kv_dim long.
  if (n_rows > capacity) return ERR_DIMENSION;
  size_t expected = n_rows * kv_dim();
  if (k_len != expected || v_len != expected) return ERR_DIMENSION;
  for (size_t r = 0; r < n_rows; ++r) store_row(r, k + r * kv_dim(), v + r * kv_dim());
  len = n_rows;  // :600
  return OK;
}

Status ResidentKv::append_row(const float* k, size_t k_len, const float* v, size_t v_len) {
  // :612-625 — wrong row length, then overflow at capacity; nothing is written on error.
  if (k_len != kv_dim() || v_len != kv_dim()) return ERR_DIMENSION;
  if (len >= capacity) return ERR_DIMENSION;
  store_row(len, k, v);
  len += 1;
  return OK;
}

Status ResidentKv::truncate(size_t new_len) {  // :501-510 — only the cursor moves.
  if (new_len > capacity) return ERR_DIMENSION;
  len = new_len;
  return OK;
}

// ---- attention (src/decoder/attention_ops.rs:889-1046) ---------------------
float dot_product(const float* a, const float* b, size_t n) {  // :1040-1046, sequential
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) sum += a[i] * b[i];
  return sum;
}

void softmax_in_place(float* values, size_t n, float temperature) {  // :1019-1038
  temperature = std::max(temperature, 0.0001f);
  float max = -std::numeric_limits<float>::infinity();
  for (size_t i = 0; i < n; ++i) max = std::max(max, values[i]);
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) {
    values[i] = std::exp((values[i] - max) / temperature);
    sum += values[i];
  }
  if (sum <= std::numeric_limits<float>::epsilon()) {  // uniform fallback
    float uniform = 1.0f / static_cast<float>(n);
    for (size_t i = 0; i < n; ++i) values[i] = uniform;
    return;
  }
  for (size_t i = 0; i < n; ++i) values[i] /= sum;
}

// One query head: the loop body shared by both branches of cached_attention_one
// (:930-950 parallel closure, :956-972 serial loop; identical arithmetic).
static void attend_head(const float* q_row, const float* keys, const float* values,
                        size_t window_start, size_t window_len, size_t kv_dim, size_t head_dim,
                        size_t kv_group, float inv_scale, size_t q_head, float* scores,
                        float* out_head) {
  size_t kv_head = q_head / kv_group;
  const float* q_slice = q_row + q_head * head_dim;
  size_t k_start = kv_head * head_dim;
  for (size_t off = 0; off < window_len; ++off) {
    const float* k_slice = keys + (window_start + off) * kv_dim + k_start;
    scores[off] = dot_product(q_slice, k_slice, head_dim) * inv_scale;
  }
  softmax_in_place(scores, window_len, 1.0f);
  for (size_t off = 0; off < window_len; ++off) {
    float prob = scores[off];
    const float* v_slice = values + (window_start + off) * kv_dim + k_start;
    for (size_t col = 0; col < head_dim; ++col) out_head[col] += prob * v_slice[col];
  }
}

Status attention_windowed(const float* q, const float* keys, const float* values, size_t len,
                          size_t window_start, size_t q_heads, size_t kv_heads, size_t head_dim,
                          float attn_scalar, int threads, float* out) {
  if (len == 0 || window_start >= len) return ERR_DIMENSION;
  if (kv_heads == 0 || q_heads % kv_heads != 0) return ERR_CONFIG;
  size_t kv_dim = kv_heads * head_dim;
  size_t kv_group = q_heads / kv_heads;
  size_t window_len = len - window_start;
  float inv_scale = 1.0f / std::sqrt(attn_scalar);  // :912
  std::fill(out, out + q_heads * head_dim, 0.0f);
  if (threads <= 1) {
    std::vector<float> scores(window_len);
    for (size_t h = 0; h < q_heads; ++h)
      attend_head(q, keys, values, window_start, window_len, kv_dim, head_dim, kv_group, inv_scale,
                  h, scores.data(), out + h * head_dim);
    return OK;
  }
  size_t workers = std::min<size_t>(static_cast<size_t>(threads), q_heads);
  std::vector<std::thread> pool;
  pool.reserve(workers);
  for (size_t w = 0; w < workers; ++w) {
    pool.emplace_back([=]() {
      std::vector<float> scores(window_len);
      for (size_t h = w; h < q_heads; h += workers)
        attend_head(q, keys, values, window_start, window_len, kv_dim, head_dim, kv_group,
                    inv_scale, h, scores.data(), out + h * head_dim);
    });
  }
  for (auto& t : pool) t.join();
  return OK;
}

Status cached_attention_one(const float* q, size_t q_dim, const float* keys, const float* values,
                            size_t cache_len, size_t q_heads, size_t kv_heads, size_t head_dim,
                            float attn_scalar, bool has_window, size_t sliding_window, int threads,
                            float* out) {
  // :895-911 — shape checks, empty cache is a Dimension error.
  if (q_dim != q_heads * head_dim) return ERR_DIMENSION;
  if (cache_len == 0) return ERR_DIMENSION;
  // :915-918 — window_start = len.saturating_sub(window); None => 0.
  size_t window_start = 0;
  if (has_window) window_start = cache_len > sliding_window ? cache_len - sliding_window : 0;
  return attention_windowed(q, keys, values, cache_len, window_start, q_heads, kv_heads, head_dim,
                            attn_scalar, threads, out);
}

// ---- RMSNorm + RoPE (src/decoder/attention_ops.rs:598-887) -----------------
void rope_rotations(size_t position, size_t rope_dims, RopeParams rope, float* cos_out,
                    float* sin_out) {
  // :872-878 — position scaled BEFORE the frequency; exponent 2*pair/frequency_dim;
  // angle = scaled_position / theta^exponent, all in f32.
  size_t pairs = rope_dims / 2;
  float scaled_position = static_cast<float>(position) * rope.position_scale;
  for (size_t pair = 0; pair < pairs; ++pair) {
    float exponent = static_cast<float>(2 * pair) / static_cast<float>(rope.frequency_dim);
    float angle = scaled_position / std::pow(rope.theta, exponent);
    cos_out[pair] = std::cos(angle);
    sin_out[pair] = std::sin(angle);
  }
}

Status rms_norm_heads(const float* x, size_t seq, size_t heads, size_t head_dim,
                      const float* weight, float eps, float* out) {
  if (heads == 0 || head_dim == 0) return ERR_DIMENSION;
  size_t dim = heads * head_dim;
  for (size_t pos = 0; pos < seq; ++pos) {
    for (size_t head = 0; head < heads; ++head) {
      const float* xs = x + pos * dim + head * head_dim;
      float sum = 0.0f;  // :627 — sequential f32 sum of squares
      for (size_t c = 0; c < head_dim; ++c) sum += xs[c] * xs[c];
      float mean_square = sum / static_cast<float>(head_dim);
      float inv_rms = 1.0f / std::sqrt(mean_square + eps);
      for (size_t c = 0; c < head_dim; ++c)
        out[pos * dim + head * head_dim + c] = xs[c] * inv_rms * weight[c];
    }
  }
  return OK;
}

static void rotate_head(float* head, size_t pairs, const float* cos_t, const float* sin_t,
                        RopeStyle style) {
  if (style == ROPE_INTERLEAVED) {  // :747-755
    for (size_t pair = 0; pair < pairs; ++pair) {
      float even = head[2 * pair], odd = head[2 * pair + 1];
      head[2 * pair] = even * cos_t[pair] - odd * sin_t[pair];
      head[2 * pair + 1] = even * sin_t[pair] + odd * cos_t[pair];
    }
  } else {  // Halves, :757-767 — pair (i, i + pairs)
    for (size_t pair = 0; pair < pairs; ++pair) {
      float first = head[pair], second = head[pairs + pair];
      head[pair] = first * cos_t[pair] - second * sin_t[pair];
      head[pairs + pair] = first * sin_t[pair] + second * cos_t[pair];
    }
  }
}

Status apply_rope_heads_at(const float* x, size_t seq, size_t heads, size_t head_dim,
                           size_t rope_dims, RopeParams rope, size_t position_offset,
                           RopeStyle style, float* out) {
  if (rope.theta <= 0.0f) return ERR_DIMENSION;
  size_t dim = heads * head_dim;
  size_t pairs = rope_dims / 2;
  std::vector<float> cos_t(pairs), sin_t(pairs);
  std::memcpy(out, x, seq * dim * sizeof(float));
  for (size_t pos = 0; pos < seq; ++pos) {
    rope_rotations(position_offset + pos, rope_dims, rope, cos_t.data(), sin_t.data());
    for (size_t head = 0; head < heads; ++head)
      rotate_head(out + pos * dim + head * head_dim, pairs, cos_t.data(), sin_t.data(), style);
  }
  return OK;
}

Status rms_norm_rope_heads_at(const float* x, size_t seq, size_t heads, size_t head_dim,
                              size_t rope_dims, const float* weight, float eps, RopeParams rope,
                              size_t position_offset, RopeStyle style, float* out) {
  if (heads == 0 || head_dim == 0) return ERR_DIMENSION;                          // :710-718
  if (rope_dims == 0 || rope_dims > head_dim || rope_dims % 2 != 0) return ERR_DIMENSION;  // :719-724
  size_t dim = heads * head_dim;
  size_t pairs = rope_dims / 2;
  std::vector<float> cos_t(pairs), sin_t(pairs);
  for (size_t pos = 0; pos < seq; ++pos) {
    rope_rotations(position_offset + pos, rope_dims, rope, cos_t.data(), sin_t.data());
    for (size_t head = 0; head < heads; ++head) {
      const float* xs = x + pos * dim + head * head_dim;
      float* o = out + pos * dim + head * head_dim;
      float sum = 0.0f;
      for (size_t c = 0; c < head_dim; ++c) sum += xs[c] * xs[c];
      float inv_rms = 1.0f / std::sqrt(sum / static_cast<float>(head_dim) + eps);  // :741-743
      for (size_t c = 0; c < head_dim; ++c) o[c] = xs[c] * inv_rms * weight[c];
      rotate_head(o, pairs, cos_t.data(), sin_t.data(), style);
    }
  }
  return OK;
}

// ---- u8 group-32 affine KV (encoder defined here; see sgo.hpp) -------------
void quantize_group_u8(const float* x, uint8_t* codes, uint16_t* scale_bits, uint16_t* bias_bits) {
  float lo = x[0], hi = x[0];
  for (size_t i = 1; i < QGROUP; ++i) {
    lo = std::min(lo, x[i]);
    hi = std::max(hi, x[i]);
  }
  uint16_t bb = f32_to_bf16_bits(lo);
  float bias = bf16_bits_to_f32(bb);
  float raw = (hi - bias) / 255.0f;
  const float floor_scale = 9.094947017729282e-13f;  // 2^-40
  uint16_t sb = f32_to_bf16_bits(std::max(raw, floor_scale));
  float scale = bf16_bits_to_f32(sb);
  for (size_t i = 0; i < QGROUP; ++i) {
    float t = std::nearbyint((x[i] - bias) / scale);  // half-to-even in the default mode
    t = std::min(std::max(t, 0.0f), 255.0f);
    codes[i] = static_cast<uint8_t>(t);
  }
  *scale_bits = sb;
  *bias_bits = bb;
}

void quantize_row_u8(const float* x, size_t n, uint8_t* codes, uint16_t* scale_bits,
                     uint16_t* bias_bits) {
  for (size_t g = 0; g < n / QGROUP; ++g)
    quantize_group_u8(x + g * QGROUP, codes + g * QGROUP, scale_bits + g, bias_bits + g);
}

void dequantize_row_u8(const uint8_t* codes, const uint16_t* scale_bits, const uint16_t* bias_bits,
                       size_t n, float* out) {
  // src/quantization.rs:173-179 — value = q * scale + bias in f32 (two roundings, no fma).
  for (size_t i = 0; i < n; ++i) {
    float scale = bf16_bits_to_f32(scale_bits[i / QGROUP]);
    float bias = bf16_bits_to_f32(bias_bits[i / QGROUP]);
    float prod = static_cast<float>(codes[i]) * scale;
    out[i] = prod + bias;
  }
}

// ---- generators -------------------------------------------------------------
float pseudo(uint64_t seed) {  // src/decode_resident/tests.rs:544-547 (usize = u64)
  uint64_t x = ((seed * 2654435761ull) ^ 0x9E3779B9ull) % 1000ull;
  return (static_cast<float>(x) / 1000.0f - 0.5f) * 0.2f;
}

uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

float normal8(uint64_t seed, uint64_t stream, uint64_t index) {
  uint64_t key = splitmix64(seed * 0xD1342543DE82EF95ull + stream);
  uint64_t a = splitmix64(key + 2 * index);
  uint64_t b = splitmix64(key + 2 * index + 1);
  int64_t sum = 0;
  for (int i = 0; i < 4; ++i) {
    sum += static_cast<int64_t>((a >> (16 * i)) & 0xFFFF);
    sum += static_cast<int64_t>((b >> (16 * i)) & 0xFFFF);
  }
  // mean 8 * 32767.5 = 262140; variance 8 * (65536^2 - 1) / 12; 1/sigma below.
  return static_cast<float>(static_cast<int32_t>(sum - 262140)) * 0x1.3988e2p-16f;  // 1/sigma = 1.8688124e-05
}

void fill_normal8(float* out, size_t n, uint64_t seed, uint64_t stream, uint64_t index0) {
  for (size_t i = 0; i < n; ++i) out[i] = normal8(seed, stream, index0 + i);
}

}  // namespace sgo
