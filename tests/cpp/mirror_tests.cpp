// Ports of the reference's own unit tests, written against the C++ host face
// (include/saragossa_kv.hpp) so they read like the originals. `cpu` runs the
// prefix-cache cases (no device); `gpu` also runs the resident-KV cases and checks
// attention against the CPU oracle (test infrastructure, linked in directly).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/saragossa_kv.hpp"
#include "../../oracle/sgo.hpp"

using namespace saragossa;

static int g_failed = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #cond);          \
      ++g_failed;                                                          \
    }                                                                      \
  } while (0)

static float pseudo(size_t seed) { return sgo::pseudo(seed); }

// src/serve/cache.rs:341-375
static void prefix_cache_evicts_lru_block() {
  BlockAwarePrefixCache cache(1, 2);
  BlockHash root = BlockHash::root();
  BlockHash first = root.chain({1}), second = first.chain({2}), third = second.chain({3});
  cache.insert(root, first, 1);
  cache.insert(root, second, 2);
  cache.insert(root, third, 3);
  CHECK(!cache.match_prefix(root, {1}).first);
  CHECK(!cache.match_prefix(root, {1, 2, 3}).first);
}

// src/serve/cache.rs:421-466
static void reduced_session_cap_evicts_only_that_session_first() {
  BlockAwarePrefixCache cache(1, 2, 1);
  BlockHash alpha = BlockHash::for_session("agent-a"), beta = BlockHash::for_session("agent-b");
  BlockHash beta_first = beta.chain({9}), alpha_first = alpha.chain({1}), alpha_second = alpha_first.chain({2});
  cache.insert(beta, beta_first, 1);
  cache.insert(alpha, alpha_first, 1);
  cache.insert(alpha, alpha_second, 2);
  auto hashes = cache.entry_hashes();
  CHECK(hashes.size() == 2 && hashes[0] == alpha_second && hashes[1] == beta_first);
  auto hit = cache.match_prefix(beta, {9});
  CHECK(hit.first && hit.second.hash == beta_first);
  CHECK(cache.session_block_count(alpha) == 1);
}

// src/serve/cache.rs:281-339,468-493
static void hashes_and_longest_chain() {
  BlockHash first = BlockHash::root().chain({1, 2});
  CHECK(first.chain({3, 4}) != BlockHash::root().chain({3, 4}));
  CHECK(BlockHash::for_session("alpha") == BlockHash::for_session("alpha"));
  CHECK(BlockHash::for_session("alpha") != BlockHash::for_session("beta"));
  CHECK(BlockHash::for_session(nullptr) == BlockHash::root());
  BlockAwarePrefixCache cache(2, 8);
  BlockHash root = BlockHash::root(), second = first.chain({3, 4});
  cache.insert(root, first, 2);
  cache.insert(root, second, 4);
  auto hit = cache.match_prefix(root, {1, 2, 3, 4, 5});
  CHECK(hit.first && hit.second.tokens == 4 && hit.second.hash == second);
  CHECK(!cache.match_prefix(BlockHash::for_session("agent-b"), {1, 2, 3, 4}).first);
}

// prefill_prompt_state's block loop (src/serve/state.rs:596-604): all full blocks of a prompt in one call
// leave the cache as the block-by-block inserts do, and blocks before the matched prefix are not inserted again.
static void chain_insert_equals_block_by_block() {
  const std::vector<uint64_t> prompt = {5, 6, 7, 8, 9, 10, 11};     // three full blocks of 2 and a tail
  BlockHash root = BlockHash::for_session("s");
  BlockAwarePrefixCache one(2, 8), all(2, 8);
  BlockHash prev = root;
  for (size_t b = 0; b < 3; ++b) {
    prev = prev.chain({prompt[2 * b], prompt[2 * b + 1]});
    CHECK(one.insert(root, prev, 2 * (b + 1)));
  }
  CHECK(all.insert_chain(root, prompt) == 3);
  auto h1 = one.entry_hashes(), h2 = all.entry_hashes();
  CHECK(h1.size() == 3 && h2.size() == 3);
  for (size_t i = 0; i < h1.size() && i < h2.size(); ++i) CHECK(h1[i] == h2[i]);
  auto hit = all.match_prefix(root, prompt);
  CHECK(hit.first && hit.second.tokens == 6 && hit.second.hash == prev);
  // a longer prompt of the same conversation: only the new blocks
  std::vector<uint64_t> longer = prompt;
  longer.insert(longer.end(), {12, 13, 14});
  CHECK(all.insert_chain(root, longer, 6) == 2);
  CHECK(all.match_prefix(root, longer).second.tokens == 10);
}

// prefix_cache_selects_longest_append_prefix (src/decoder/tests.rs:428-465) through the cache itself, and
// the bookkeeping of prefix_cache_get / prefix_cache_put (src/decoder/generation.rs:2998-3024,3105-3139).
static void decoder_prefix_cache_keeps_the_reference_order() {
  PrefixCache cache(4);
  cache.put({1, 2});
  cache.put({1, 2, 3});
  cache.put({1});
  CHECK(cache.len() == 3);
  CHECK(cache.get({1, 2, 3, 4}) == 3);                       // entry [1,2,3] wins and moves to the front
  CHECK(cache.entry_tokens(0) == std::vector<uint64_t>({1, 2, 3}));
  CHECK(cache.get({1, 9}) == 1);
  CHECK(cache.entry_tokens(0) == std::vector<uint64_t>({1}));
  CHECK(cache.get({9}) == 0);
  cache.put({1, 2, 3});                                      // same tokens: replaced, not doubled
  CHECK(cache.len() == 3 && cache.entry_tokens(0) == std::vector<uint64_t>({1, 2, 3}));
  cache.put({4});
  cache.put({5});                                            // beyond the capacity the rear entry goes
  CHECK(cache.len() == 4);
  CHECK(cache.get({1, 2, 7}) == 1);                          // [1,2] fell off the rear; [1] is the longest left
  PrefixCache none(0);
  none.put({1});
  CHECK(none.len() == 0 && none.get({1}) == 0);
}

// src/decode_resident/tests.rs:380-430
static void kv_seed_then_append_matches_cpu(DecodeResidentState& state) {
  const size_t q_heads = 16, kv_heads = 2, head_dim = 256, kv_dim = kv_heads * head_dim, capacity = 6;
  auto made = state.full_attention(capacity, q_heads, kv_heads, head_dim, false);
  CHECK(made.ok);
  FullAttentionState kv = std::move(made.value);
  CHECK(kv.kv_dim() == kv_dim);
  std::vector<float> cpu_keys, cpu_values, seed_k, seed_v;
  const size_t seed_rows = 3;
  for (size_t r = 0; r < seed_rows; ++r)
    for (size_t c = 0; c < kv_dim; ++c) {
      seed_k.push_back(static_cast<float>(r * kv_dim + c) * 0.001f);
      seed_v.push_back(static_cast<float>(r * kv_dim + c) * -0.002f + 1.0f);
    }
  CHECK(kv.seed(seed_k, seed_v, seed_rows).ok);
  cpu_keys = seed_k;
  cpu_values = seed_v;
  CHECK(kv.len() == seed_rows);
  for (size_t r = seed_rows; r < seed_rows + 2; ++r) {
    std::vector<float> k(kv_dim), v(kv_dim);
    for (size_t c = 0; c < kv_dim; ++c) {
      k[c] = static_cast<float>(r * kv_dim + c) * 0.003f;
      v[c] = static_cast<float>(r * kv_dim + c) * 0.004f - 0.5f;
    }
    CHECK(kv.append_row(k, v).ok);
    cpu_keys.insert(cpu_keys.end(), k.begin(), k.end());
    cpu_values.insert(cpu_values.end(), v.begin(), v.end());
  }
  CHECK(kv.len() == seed_rows + 2);
  auto gpu_keys = kv.keys(), gpu_values = kv.values();
  CHECK(gpu_keys.ok && gpu_keys.value == cpu_keys);          // bit-identical
  CHECK(gpu_values.ok && gpu_values.value == cpu_values);
}

// src/decode_resident/tests.rs:435-478
static void kv_bf16_seed_then_append_rounds_to_bf16(DecodeResidentState& state) {
  const size_t kv_dim = 512, capacity = 4;
  auto made = state.full_attention_with_element(capacity, 16, 2, 256, GpuElement::Bf16);
  CHECK(made.ok);
  FullAttentionState kv = std::move(made.value);
  CHECK(kv.element() == GpuElement::Bf16 && kv.byte_len() == capacity * kv_dim * 2);
  std::vector<float> seed_k(2 * kv_dim), seed_v(2 * kv_dim), row_k(kv_dim), row_v(kv_dim);
  for (size_t i = 0; i < 2 * kv_dim; ++i) {
    seed_k[i] = (static_cast<float>(i) - 333.0f) * 0.0017f;
    seed_v[i] = (static_cast<float>(i) + 17.0f) * -0.0023f;
  }
  for (size_t i = 0; i < kv_dim; ++i) {
    row_k[i] = 1.0f + static_cast<float>(i) * 0.0009f;
    row_v[i] = -1.0f + static_cast<float>(i) * 0.0011f;
  }
  CHECK(kv.seed(seed_k, seed_v, 2).ok);
  CHECK(kv.append_row(row_k, row_v).ok);
  CHECK(kv.len() == 3);
  std::vector<float> cpu_k = seed_k;
  cpu_k.insert(cpu_k.end(), row_k.begin(), row_k.end());
  auto bits = kv.keys_bf16_bits();
  CHECK(bits.ok);
  for (size_t i = 0; i < cpu_k.size() && bits.ok; ++i) CHECK(bits.value[i] == sgo::f32_to_bf16_bits(cpu_k[i]));
}

// src/decode_resident/tests.rs:507-538
static void overflow_and_invalid_gqa(DecodeResidentState& state) {
  const size_t prefill_len = 3, kv_dim = 4;
  auto made = state.full_attention(prefill_len, 4, 2, 2, false);
  CHECK(made.ok);
  FullAttentionState kv = std::move(made.value);
  std::vector<float> seed(prefill_len * kv_dim);
  for (size_t i = 0; i < seed.size(); ++i) seed[i] = static_cast<float>(i);
  CHECK(kv.seed(seed, seed, prefill_len).ok);
  CHECK(kv.len() == kv.capacity());
  std::vector<float> row(kv_dim, 0.0f);
  auto r = kv.append_row(row, row);
  CHECK(r.is_err() && r.error.kind == InferError::Dimension);
  auto bad = state.full_attention(4, 3, 2, 8, false);
  CHECK(bad.is_err() && bad.error.kind == InferError::Config);
}

// run_attention_case / run_attention_case_bf16, src/decode_resident/tests.rs:1390-1492
static void run_attention_case(DecodeResidentState& state, size_t len, bool bf16) {
  const size_t q_heads = 16, kv_heads = 2, head_dim = 256, kv_dim = kv_heads * head_dim;
  auto made = state.full_attention_with_element(len, q_heads, kv_heads, head_dim, bf16 ? GpuElement::Bf16 : GpuElement::F32);
  CHECK(made.ok);
  FullAttentionState kv = std::move(made.value);
  std::vector<float> keys(len * kv_dim), values(len * kv_dim), q(q_heads * head_dim);
  for (size_t i = 0; i < keys.size(); ++i) {
    keys[i] = pseudo(i);
    values[i] = pseudo(i + 7);
  }
  for (size_t i = 0; i < q.size(); ++i) q[i] = pseudo(i + 99);
  CHECK(kv.seed(keys, values, len).ok);
  auto gpu = kv.attention_decode(q);
  CHECK(gpu.ok);
  std::vector<float> ok = keys, ov = values;
  if (bf16)
    for (size_t i = 0; i < ok.size(); ++i) {
      ok[i] = sgo::bf16_round_f32(ok[i]);
      ov[i] = sgo::bf16_round_f32(ov[i]);
    }
  std::vector<float> cpu(q.size());
  CHECK(sgo::cached_attention_one(q.data(), q.size(), ok.data(), ov.data(), len, q_heads, kv_heads, head_dim,
                                  static_cast<float>(head_dim), false, 0, 4, cpu.data()) == sgo::OK);
  float max_abs = 0.0f, sum_abs = 0.0f;
  for (size_t i = 0; i < cpu.size() && gpu.ok; ++i) {
    float d = std::fabs(gpu.value[i] - cpu[i]);
    max_abs = std::fmax(max_abs, d);
    sum_abs += d;
  }
  float mean_abs = sum_abs / static_cast<float>(cpu.size());
  CHECK(max_abs <= (bf16 ? 2.0e-3f : 1.0e-4f));      // the reference's bounds
  CHECK(mean_abs <= (bf16 ? 2.0e-4f : 1.0e-5f));
}

// Device copy of a host vector, freed with the test.
struct DeviceVec {
  sgk_state* st;
  float* d = nullptr;
  size_t n;
  DeviceVec(sgk_state* s, const std::vector<float>& h) : st(s), n(h.size()) {
    void* p = nullptr;
    CHECK(sgk_util_malloc(st, std::max<size_t>(n, 4) * sizeof(float), &p) == SGK_OK);
    d = static_cast<float*>(p);
    if (n) CHECK(sgk_util_h2d(st, d, h.data(), n * sizeof(float)) == SGK_OK);
  }
  std::vector<float> read() const {
    std::vector<float> h(n);
    CHECK(sgk_util_d2h(st, h.data(), d, n * sizeof(float)) == SGK_OK);
    return h;
  }
  ~DeviceVec() { sgk_util_free(st, d); }
};

// gated_delta_matches_naive_oracle_across_lengths_and_gqa_heads (src/linear_attention/tests.rs:304-372)
// on the device: the two shapes of that test, several tokens, state and outputs against the CPU
// recurrence within the reference's Metal-vs-CPU bound (1e-5), then the per-row capture / restore
// of the speculative path brings the state back bit for bit.
static void gated_delta_steps_match_cpu(DecodeResidentState& state) {
  const size_t shapes[2][4] = {{2, 4, 8, 6}, {1, 4, 128, 128}};
  for (const auto& sh : shapes) {
    const size_t hk = sh[0], hv = sh[1], dk = sh[2], dv = sh[3];
    const size_t ssm_len = hv * dv * dk;
    auto made = LinearAttentionState::create(state, 1, 0, ssm_len, false);
    auto cap = LinearAttentionState::create(state, 1, 0, ssm_len, false);
    CHECK(made.ok && cap.ok);
    if (!made.ok || !cap.ok) return;
    LinearAttentionState ls = std::move(made.value), capture = std::move(cap.value);
    std::vector<float> ssm(ssm_len, 0.0f), none;
    CHECK(ls.write(0, none, ssm).ok);
    std::vector<float> after_first;
    for (int t = 0; t < 5; ++t) {
      std::vector<float> q(hk * dk), k(hk * dk), v(hv * dv), g(hv), beta(hv);
      sgo::fill_normal8(q.data(), q.size(), 70 + t, 0, 0);
      sgo::fill_normal8(k.data(), k.size(), 70 + t, 1, 0);
      sgo::fill_normal8(v.data(), v.size(), 70 + t, 2, 0);
      for (auto& x : q) x /= static_cast<float>(dk);
      for (auto& x : k) x /= std::sqrt(static_cast<float>(dk));
      for (size_t h = 0; h < hv; ++h) g[h] = 0.9f + 0.02f * h, beta[h] = 0.2f + 0.1f * h;
      DeviceVec dq(state.handle(), q), dkk(state.handle(), k), dvv(state.handle(), v), dg(state.handle(), g),
          db(state.handle(), beta), dout(state.handle(), std::vector<float>(hv * dv));
      CHECK(ls.encode_gated_delta_step(nullptr, 0, hk, hv, dk, dv, dq.d, dkk.d, dvv.d, dg.d, db.d, dout.d).ok);
      if (t == 0) CHECK(ls.encode_capture(capture).ok);
      std::vector<float> want(hv * dv);
      sgo::LinearShape shape{hk, hv, dk, dv, 0};
      CHECK(sgo::gated_delta_step(q.data(), k.data(), v.data(), g.data(), beta.data(), shape, &ssm, want.data()) == sgo::OK);
      CHECK(sgk_state_sync(state.handle()) == SGK_OK);
      std::vector<float> got = dout.read(), got_ssm(ssm_len);
      CHECK(ls.read(0, none, got_ssm).ok);
      for (size_t i = 0; i < want.size(); ++i) CHECK(std::fabs(got[i] - want[i]) <= 1e-5f);
      for (size_t i = 0; i < ssm_len; ++i) CHECK(std::fabs(got_ssm[i] - ssm[i]) <= 1e-5f);
      if (t == 0) after_first = got_ssm;
    }
    CHECK(ls.restore(capture).ok);            // roll back to the state after the first token
    std::vector<float> back(ssm_len);
    CHECK(ls.read(0, none, back).ok);
    CHECK(back == after_first);
    auto other = LinearAttentionState::create(state, 1, 0, ssm_len, true);
    if (other.ok) {
      auto r = ls.encode_capture(other.value);   // storage type differs: a shape error, nothing copied
      CHECK(r.is_err() && r.error.kind == InferError::Shape);
    }
  }
}

// The greedy epilogue on the device against the CPU rule (first maximum, src/sampling.rs:49-62):
// a planted winner per verify row, an exact tie that must go to the lower index, and the
// dimension error of an empty vocabulary.
static void lm_head_argmax_matches_cpu(DecodeResidentState& state) {
  const size_t vocab = 1201, hidden = 96, rows = 3;
  std::vector<float> w(vocab * hidden), x(rows * hidden);
  sgo::fill_normal8(w.data(), w.size(), 91, 0, 0);
  sgo::fill_normal8(x.data(), x.size(), 91, 1, 0);
  for (auto& v : w) v *= 0.05f;
  const size_t winners[rows] = {1200, 17, 640};
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < hidden; ++c) w[winners[r] * hidden + c] = x[r * hidden + c];  // logit = |x|^2 ~ 96
  // row 1's winner gets an exact twin at a higher index: the lower one must stay
  for (size_t c = 0; c < hidden; ++c) w[900 * hidden + c] = w[17 * hidden + c];
  DeviceVec dw(state.handle(), w), dx(state.handle(), x), didx(state.handle(), std::vector<float>(8)),
      dval(state.handle(), std::vector<float>(8));
  CHECK(state.encode_lm_head_argmax(nullptr, dw.d, GpuElement::F32, vocab, hidden, dx.d, rows,
                                    reinterpret_cast<int32_t*>(didx.d), 0, dval.d).ok);
  CHECK(sgk_state_sync(state.handle()) == SGK_OK);
  std::vector<float> raw = didx.read(), val = dval.read();
  for (size_t r = 0; r < rows; ++r) {
    size_t want = 0;
    float want_value = 0.0f;
    CHECK(sgo::lm_head_argmax(w.data(), vocab, hidden, x.data() + r * hidden, &want, &want_value) == sgo::OK);
    int32_t got;
    std::memcpy(&got, &raw[r], sizeof(got));
    CHECK(want == winners[r]);
    CHECK(static_cast<size_t>(got) == want);
    CHECK(std::fabs(val[r] - want_value) <= 1e-4f * std::fabs(want_value));
  }
  auto bad = state.encode_lm_head_argmax(nullptr, dw.d, GpuElement::F32, 0, hidden, dx.d, 1,
                                         reinterpret_cast<int32_t*>(didx.d));
  CHECK(bad.is_err() && bad.error.kind == InferError::Dimension);
}

int main(int argc, char** argv) {
  const bool gpu = argc > 1 && std::string(argv[1]) == "gpu";
  prefix_cache_evicts_lru_block();
  reduced_session_cap_evicts_only_that_session_first();
  hashes_and_longest_chain();
  chain_insert_equals_block_by_block();
  decoder_prefix_cache_keeps_the_reference_order();
  if (gpu) {
    auto made = DecodeResidentState::create(0);
    CHECK(made.ok);
    if (made.ok) {
      DecodeResidentState state = std::move(made.value);
      kv_seed_then_append_matches_cpu(state);
      kv_bf16_seed_then_append_rounds_to_bf16(state);
      overflow_and_invalid_gqa(state);
      for (size_t len : {size_t(1), size_t(64), size_t(257), size_t(4096)}) {
        run_attention_case(state, len, false);
        run_attention_case(state, len, true);
      }
      gated_delta_steps_match_cpu(state);
      lm_head_argmax_matches_cpu(state);
    }
  } else {
    auto made = DecodeResidentState::create(0);
    // without a device the state cannot exist: a Metal/backend error, never a fallback
    if (made.is_err()) CHECK(made.error.kind == InferError::Metal);
  }
  std::printf("%s: %d failure(s)\n", gpu ? "gpu" : "cpu", g_failed);
  return g_failed == 0 ? 0 : 1;
}
