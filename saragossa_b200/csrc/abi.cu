// extern "C" surface of libsgk: argument validation in the reference's error
// vocabulary, then the host objects of host.h. Declared in include/sgk.h.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <random>

#include "host.h"

using namespace sgk;

struct sgk_state : State {};
struct sgk_pool : Pool {};
struct sgk_seq : Seq {};
struct sgk_kv : Kv {};
struct sgk_batch : Batch {};
struct sgk_step : Step {};
struct sgk_linstate : LinState {};
struct sgk_token_window : TokenWindow {};
struct sgk_exchange : Exchange {};
struct sgk_prefix : Prefix {};
struct sgk_budget : Budget {};
struct sgk_dprefix : DecoderPrefix {};

namespace sgk {
int create_batch(State* st, Kv** kvs, int n, Batch** out);
}

extern "C" {

const char* sgk_last_error(void) { return last_error_cstr(); }
const char* sgk_version(void) { return "sgk 0.1 (sm_100a)"; }

// ------------------------------------------------------------------ state
int32_t sgk_state_create(int32_t device, sgk_state** out) {
  if (!out) return fail(SGK_ERR_BACKEND, "state_create: null out pointer");
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(SGK_ERR_BACKEND, "no CUDA device: %s (this library has no CPU path)",
                e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
  if (device < 0 || device >= count) return fail(SGK_ERR_CONFIG, "device %d out of range [0,%d)", device, count);
  SGK_CUDA(cudaSetDevice(device));
  auto st = std::make_unique<sgk_state>();
  st->device = device;
  cudaDeviceProp prop;
  SGK_CUDA(cudaGetDeviceProperties(&prop, device));
  st->sm_count = prop.multiProcessorCount;
  if (prop.major < 10)
    return fail(SGK_ERR_BACKEND, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                prop.minor);
  SGK_CUDA(cudaStreamCreateWithFlags(&st->stream, cudaStreamNonBlocking));
  SGK_CUDA(cudaMalloc(&st->d_status, sizeof(int32_t)));
  SGK_CUDA(cudaMemset(st->d_status, 0, sizeof(int32_t)));
  SGK_CUDA(cudaMalloc(&st->d_lm_ws, 9 * sizeof(unsigned long long)));
  SGK_CUDA(cudaMemset(st->d_lm_ws, 0, 9 * sizeof(unsigned long long)));
  SGK_CUDA(attention_mma_configure());
  SGK_CUDA(attention_u8_configure());
  *out = st.release();
  return SGK_OK;
}

void sgk_state_destroy(sgk_state* st) {
  if (!st) return;
  cudaSetDevice(st->device);
  cudaStreamSynchronize(st->stream);
  if (st->d_status) cudaFree(st->d_status);
  if (st->d_lm_ws) cudaFree(st->d_lm_ws);
  if (st->d_rope_table) cudaFree(st->d_rope_table);
  if (st->order_event) cudaEventDestroy(st->order_event);
  if (st->stream) cudaStreamDestroy(st->stream);
  delete st;
}

void* sgk_state_stream(sgk_state* st) { return st ? st->stream : nullptr; }

int32_t sgk_state_sync(sgk_state* st) {
  if (!st) return fail(SGK_ERR_BACKEND, "null state");
  SGK_CUDA(cudaStreamSynchronize(st->stream));
  return SGK_OK;
}

int32_t sgk_state_device_status(sgk_state* st, int32_t* status_out) {
  if (!st || !status_out) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_CUDA(cudaStreamSynchronize(st->stream));
  SGK_CUDA(cudaMemcpy(status_out, st->d_status, sizeof(int32_t), cudaMemcpyDeviceToHost));
  if (*status_out != 0) SGK_CUDA(cudaMemset(st->d_status, 0, sizeof(int32_t)));
  return SGK_OK;
}

static int check_device_status(State* st) {
  int32_t status = 0;
  SGK_CUDA(cudaMemcpy(&status, st->d_status, sizeof(int32_t), cudaMemcpyDeviceToHost));
  if (status == 0) return SGK_OK;
  cudaMemset(st->d_status, 0, sizeof(int32_t));
  if (status == DEV_ERR_WAIT_TIMEOUT) return fail(SGK_ERR_TIMEOUT, "a bounded device-side wait expired");
  return fail(SGK_ERR_BACKEND, "kernel reported status %d (block-table entry out of range)", status);
}

int32_t sgk_state_set_concurrent_streams(sgk_state* st, int32_t enabled) {
  if (!st) return fail(SGK_ERR_BACKEND, "null state");
  st->concurrent_streams = enabled != 0;
  return SGK_OK;
}

int64_t sgk_state_launches(const sgk_state* st) { return st ? st->launches : 0; }

int32_t sgk_state_chain_begin(sgk_state* st, void* stream) {
  if (!st) return fail(SGK_ERR_BACKEND, "null state");
  if (st->chain_active) return fail(SGK_ERR_CONFIG, "a token chain is open already");
  st->chain_active = true;
  st->chain_stream = st->pick(stream);
  st->chain_mark = -1;
  return SGK_OK;
}

int32_t sgk_state_chain_end(sgk_state* st) {
  if (!st) return fail(SGK_ERR_BACKEND, "null state");
  st->chain_active = false;
  st->chain_mark = -1;
  return SGK_OK;
}

int32_t sgk_state_selftest_wait_timeout(sgk_state* st) {
  if (!st) return fail(SGK_ERR_BACKEND, "null state");
  SGK_CUDA(launch_wait_timeout_selftest(st->d_status, st->stream));
  st->launches += 1;
  SGK_CUDA(cudaStreamSynchronize(st->stream));
  return check_device_status(st);
}

// ------------------------------------------------------------------ pool
int32_t sgk_pool_create(sgk_state* st, int32_t layers, int32_t kv_heads, int32_t head_dim, int32_t dtype,
                        int32_t page_tokens, int64_t num_pages, int32_t max_seqs, int64_t max_seq_tokens,
                        sgk_pool** out) {
  if (!out) return fail(SGK_ERR_BACKEND, "pool_create: null out pointer");
  if (layers <= 0 || kv_heads <= 0 || head_dim <= 0 || num_pages <= 0 || max_seqs <= 0 || max_seq_tokens <= 0)
    return fail(SGK_ERR_CONFIG, "pool: zero dimension");
  if (page_tokens != SGK_PAGE_TOKENS) return fail(SGK_ERR_CONFIG, "pool: page_tokens must be %d", SGK_PAGE_TOKENS);
  if (dtype < SGK_KV_F32 || dtype > SGK_KV_U8G32) return fail(SGK_ERR_BACKEND, "pool: unknown KV element type %d", dtype);
  if (dtype == SGK_KV_U8G32 && head_dim % QGROUP != 0)
    return fail(SGK_ERR_CONFIG, "u8 KV needs head_dim to be a multiple of %d", QGROUP);
  if (head_dim > 512) return fail(SGK_ERR_CONFIG, "head_dim %d > 512 is not supported", head_dim);
  if (dtype != SGK_KV_U8G32 && (int64_t(head_dim) * (dtype == SGK_KV_F32 ? 4 : 2) * PAGE_TOKENS) % 16 != 0)
    return fail(SGK_ERR_CONFIG, "head_dim %d gives tiles that are not 16-byte multiples", head_dim);
  auto p = std::make_unique<sgk_pool>();
  p->st = st;
  p->layers = layers;
  p->kv_heads = kv_heads;
  p->head_dim = head_dim;
  p->dtype = dtype;
  p->num_pages = num_pages;
  p->max_seqs = max_seqs;
  p->max_seq_tokens = max_seq_tokens;
  p->table_stride = static_cast<int>((max_seq_tokens + PAGE_TOKENS - 1) / PAGE_TOKENS);
  p->tile_b = tile_bytes(dtype, head_dim);
  p->layer_b = int64_t(kv_heads) * 2 * p->tile_b;
  p->page_b = int64_t(layers) * p->layer_b;
  p->layer_stride = num_pages * p->layer_b;
  p->refcount.assign(static_cast<size_t>(num_pages), 0);
  p->free_list.resize(static_cast<size_t>(num_pages));
  for (int64_t i = 0; i < num_pages; ++i) p->free_list[static_cast<size_t>(i)] = static_cast<int32_t>(num_pages - 1 - i);
  for (int s = max_seqs - 1; s >= 0; --s) p->free_slots.push_back(s);
  if (st) {
    SGK_CUDA(cudaSetDevice(st->device));
    size_t bytes = static_cast<size_t>(p->page_b) * static_cast<size_t>(num_pages);
    cudaError_t e = cudaMalloc(&p->d_base, bytes);
    if (e != cudaSuccess)
      return fail(SGK_ERR_MEMORY_GUARD, "pool of %zu bytes does not fit the device: %s", bytes, cudaGetErrorString(e));
    SGK_CUDA(cudaMemset(p->d_base, 0, bytes));
    size_t tbytes = size_t(max_seqs) * p->table_stride * sizeof(int32_t);
    SGK_CUDA(cudaMalloc(&p->d_tables, tbytes));
    SGK_CUDA(cudaMemset(p->d_tables, 0xff, tbytes));
    SGK_CUDA(cudaMalloc(&p->d_lens, size_t(max_seqs) * layers * sizeof(int32_t)));
    SGK_CUDA(cudaMemset(p->d_lens, 0, size_t(max_seqs) * layers * sizeof(int32_t)));
    if (dtype == SGK_KV_U8G32) {
      SGK_CUDA(cudaMalloc(&p->d_scale_max, sizeof(uint32_t)));
      SGK_CUDA(cudaMemset(p->d_scale_max, 0, sizeof(uint32_t)));
    }
  }
  *out = p.release();
  return SGK_OK;
}

void sgk_pool_destroy(sgk_pool* p) {
  if (!p) return;
  if (p->st) {
    cudaSetDevice(p->st->device);
    cudaStreamSynchronize(p->st->stream);
  }
  if (p->d_base) cudaFree(p->d_base);
  if (p->d_tables) cudaFree(p->d_tables);
  if (p->d_lens) cudaFree(p->d_lens);
  if (p->d_scale_max) cudaFree(p->d_scale_max);
  p->stage_free();
  delete p;
}

int64_t sgk_pool_num_pages(const sgk_pool* p) { return p ? p->num_pages : 0; }
int64_t sgk_pool_free_pages(const sgk_pool* p) { return p ? static_cast<int64_t>(p->free_list.size()) : 0; }
int64_t sgk_pool_page_bytes(const sgk_pool* p) { return p ? p->page_b : 0; }
int64_t sgk_pool_used_bytes(const sgk_pool* p) { return p ? p->used_pages() * p->page_b : 0; }

int32_t sgk_pool_shuffle_free_list(sgk_pool* p, uint64_t seed) {
  if (!p) return fail(SGK_ERR_BACKEND, "null pool");
  // Fisher-Yates with splitmix64 draws
  uint64_t x = seed;
  auto next = [&]() {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  };
  for (size_t i = p->free_list.size(); i > 1; --i) std::swap(p->free_list[i - 1], p->free_list[next() % i]);
  return SGK_OK;
}

int32_t sgk_pool_page_refcount(const sgk_pool* p, int64_t page, int32_t* out) {
  if (!p || !out) return fail(SGK_ERR_BACKEND, "null argument");
  if (page < 0 || page >= p->num_pages) return fail(SGK_ERR_DIMENSION, "page %lld out of range", (long long)page);
  *out = p->refcount[static_cast<size_t>(page)];
  return SGK_OK;
}

int32_t sgk_pool_set_scrub_on_free(sgk_pool* p, int32_t enabled) {
  if (!p) return fail(SGK_ERR_BACKEND, "null pool");
  p->scrub_on_free = enabled != 0;
  return SGK_OK;
}

// ------------------------------------------------------------------ seq
int32_t sgk_seq_create(sgk_pool* p, int64_t capacity_tokens, sgk_seq** out) {
  if (!p || !out) return fail(SGK_ERR_BACKEND, "seq_create: null argument");
  if (capacity_tokens <= 0) return fail(SGK_ERR_CONFIG, "sequence capacity must be positive");
  if (capacity_tokens > p->max_seq_tokens)
    return fail(SGK_ERR_CONFIG, "sequence capacity %lld > pool max_seq_tokens %lld", (long long)capacity_tokens,
                (long long)p->max_seq_tokens);
  if (p->free_slots.empty()) return fail(SGK_ERR_MEMORY_GUARD, "pool holds its maximum of %d sequences", p->max_seqs);
  auto s = std::make_unique<sgk_seq>();
  s->pool = p;
  s->slot = p->free_slots.back();
  p->free_slots.pop_back();
  s->capacity = capacity_tokens;
  s->len.assign(static_cast<size_t>(p->layers), 0);
  if (!p->host_only()) {
    cudaStream_t stream = p->st->stream;
    int rc = s->set_len_all(0, stream);
    if (rc != SGK_OK) return rc;
    SGK_CUDA(cudaStreamSynchronize(stream));
  }
  p->live_seqs += 1;
  *out = s.release();
  return SGK_OK;
}

void sgk_seq_destroy(sgk_seq* s) {
  if (!s) return;
  Pool* p = s->pool;
  if (!p->host_only()) {
    // the pages go back to the pool: wait for whatever was enqueued on the state's stream and on
    // the caller stream used last
    cudaSetDevice(p->st->device);
    p->st->order_after_last_caller(p->st->stream);
    cudaStreamSynchronize(p->st->stream);
  }
  s->views.clear();
  s->release_all();
  if (!p->host_only()) p->flush_scrub(p->st->stream);
  p->free_slots.push_back(s->slot);
  p->live_seqs -= 1;
  delete s;
}

int32_t sgk_seq_reset(sgk_seq* s, void* stream) {
  if (!s) return fail(SGK_ERR_BACKEND, "null sequence");
  s->release_all();
  cudaStream_t cs = s->pool->host_only() ? nullptr : s->pool->st->pick(stream);
  SGK_TRY(s->set_len_all(0, cs));
  if (!s->pool->host_only()) SGK_TRY(s->pool->flush_scrub(cs));
  return SGK_OK;
}

int32_t sgk_seq_reserve(sgk_seq* s, int64_t tokens) {
  if (!s) return fail(SGK_ERR_BACKEND, "null sequence");
  return s->reserve(tokens);
}

int32_t sgk_seq_block_table(const sgk_seq* s, int32_t* pages_out, int64_t cap, int64_t* n_out) {
  if (!s || !n_out) return fail(SGK_ERR_BACKEND, "null argument");
  *n_out = static_cast<int64_t>(s->pages.size());
  if (pages_out)
    for (int64_t i = 0; i < std::min<int64_t>(cap, *n_out); ++i) pages_out[i] = s->pages[static_cast<size_t>(i)];
  return SGK_OK;
}

int32_t sgk_seq_release_before(sgk_seq* s, int64_t row) {
  if (!s) return fail(SGK_ERR_BACKEND, "null sequence");
  if (row < 0) return fail(SGK_ERR_DIMENSION, "negative row");
  if (!s->pool->host_only()) {
    SGK_CUDA(s->pool->st->order_after_last_caller(s->pool->st->stream));
    SGK_CUDA(cudaStreamSynchronize(s->pool->st->stream));
  }
  return s->release_before(row);
}

int32_t sgk_seq_layer(sgk_seq* s, int32_t layer, int32_t q_heads, sgk_kv** out) {
  if (!s || !out) return fail(SGK_ERR_BACKEND, "null argument");
  if (layer < 0 || layer >= s->pool->layers) return fail(SGK_ERR_DIMENSION, "layer %d out of range", layer);
  if (q_heads <= 0) return fail(SGK_ERR_CONFIG, "FullAttentionState: zero dimension");
  if (q_heads % s->pool->kv_heads != 0)
    return fail(SGK_ERR_CONFIG, "invalid GQA: q_heads=%d is not a multiple of kv_heads=%d", q_heads, s->pool->kv_heads);
  auto kv = std::make_unique<sgk_kv>();
  kv->st = s->pool->st;
  kv->seq = s;
  kv->layer = layer;
  kv->q_heads = q_heads;
  *out = kv.get();
  s->views.emplace_back(kv.release());
  return SGK_OK;
}

// ------------------------------------------------------------------ kv
static int32_t kv_create_impl(sgk_state* st, int64_t capacity, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                              int32_t dtype, int32_t page_tokens, bool shuffle, uint64_t seed, sgk_kv** out) {
  if (!st || !out) return fail(SGK_ERR_BACKEND, "kv_create: null argument");
  // src/decode_resident/attention.rs:64-74
  if (capacity <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0)
    return fail(SGK_ERR_CONFIG, "FullAttentionState: zero dimension");
  if (q_heads % kv_heads != 0)
    return fail(SGK_ERR_CONFIG, "invalid GQA: q_heads=%d is not a multiple of kv_heads=%d", q_heads, kv_heads);
  int64_t pages = (capacity + PAGE_TOKENS - 1) / PAGE_TOKENS;
  sgk_pool* pool = nullptr;
  SGK_TRY(sgk_pool_create(st, 1, kv_heads, head_dim, dtype, page_tokens, pages, 1, pages * PAGE_TOKENS, &pool));
  std::unique_ptr<Pool> pool_owner(pool);
  if (shuffle) sgk_pool_shuffle_free_list(pool, seed);
  sgk_seq* seq = nullptr;
  SGK_TRY(sgk_seq_create(pool, capacity, &seq));
  std::unique_ptr<Seq> seq_owner(seq);
  SGK_TRY(seq->reserve(capacity));  // the reference allocates the whole capacity up front
  auto kv = std::make_unique<sgk_kv>();
  kv->st = st;
  kv->seq = seq;
  kv->layer = 0;
  kv->q_heads = q_heads;
  kv->owned_pool = std::move(pool_owner);
  kv->owned_seq = std::move(seq_owner);
  *out = kv.release();
  return SGK_OK;
}

int32_t sgk_kv_create(sgk_state* st, int64_t capacity, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                      int32_t dtype, int32_t page_tokens, sgk_kv** out) {
  return kv_create_impl(st, capacity, q_heads, kv_heads, head_dim, dtype, page_tokens, false, 0, out);
}

int32_t sgk_kv_create_shuffled(sgk_state* st, int64_t capacity, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                               int32_t dtype, uint64_t seed, sgk_kv** out) {
  return kv_create_impl(st, capacity, q_heads, kv_heads, head_dim, dtype, SGK_PAGE_TOKENS, true, seed, out);
}

void sgk_kv_destroy(sgk_kv* kv) {
  if (!kv) return;
  if (!kv->owned_seq) return;  // views belong to their sequence
  cudaSetDevice(kv->st->device);
  cudaStreamSynchronize(kv->st->stream);
  kv->self_batch.reset();
  Pool* pool = kv->owned_pool.release();
  Seq* seq = kv->owned_seq.release();
  seq->release_all();
  delete static_cast<sgk_seq*>(seq);
  sgk_pool_destroy(static_cast<sgk_pool*>(pool));
  delete kv;
}

int64_t sgk_kv_len(const sgk_kv* kv) { return kv ? kv->len() : 0; }
int64_t sgk_kv_capacity(const sgk_kv* kv) { return kv ? kv->seq->capacity : 0; }
int32_t sgk_kv_kv_dim(const sgk_kv* kv) { return kv ? kv->kv_dim() : 0; }
int32_t sgk_kv_q_heads(const sgk_kv* kv) { return kv ? kv->q_heads : 0; }
int32_t sgk_kv_kv_heads(const sgk_kv* kv) { return kv ? kv->pool()->kv_heads : 0; }
int32_t sgk_kv_head_dim(const sgk_kv* kv) { return kv ? kv->pool()->head_dim : 0; }
int32_t sgk_kv_dtype(const sgk_kv* kv) { return kv ? kv->pool()->dtype : 0; }
int64_t sgk_kv_byte_len(const sgk_kv* kv) {
  if (!kv) return 0;
  return kv->seq->capacity * kv->pool()->kv_heads * row_head_bytes(kv->pool()->dtype, kv->pool()->head_dim);
}

int32_t sgk_kv_truncate(sgk_kv* kv, int64_t len) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  // src/decode_resident/attention.rs:501-510: only len > capacity is an error
  if (len < 0 || len > kv->seq->capacity)
    return fail(SGK_ERR_DIMENSION, "truncate KV %lld > capacity %lld", (long long)len, (long long)kv->seq->capacity);
  SGK_TRY(kv->seq->reserve(len));
  if (kv->pool()->host_only()) {
    kv->seq->len[kv->layer] = len;
    return SGK_OK;
  }
  SGK_TRY(kv->seq->set_len(kv->layer, len, kv->st->stream));
  SGK_CUDA(cudaStreamSynchronize(kv->st->stream));
  return SGK_OK;
}

static int32_t append_rows_host(sgk_kv* kv, const float* k, size_t k_len, const float* v, size_t v_len, int64_t n_rows,
                                bool reset) {
  const size_t kv_dim = static_cast<size_t>(kv->kv_dim());
  const size_t cells = static_cast<size_t>(n_rows) * kv_dim;
  if (!k || !v) return fail(SGK_ERR_BACKEND, "null host pointer");
  if (k_len != cells || v_len != cells)
    return fail(SGK_ERR_DIMENSION, "KV rows: expected %zu (=%lld x %zu), got keys=%zu values=%zu", cells,
                (long long)n_rows, kv_dim, k_len, v_len);
  cudaStream_t stream = kv->st->stream;
  if (reset) SGK_TRY(kv->seq->set_len(kv->layer, 0, stream));
  if (n_rows == 0) {
    SGK_CUDA(cudaStreamSynchronize(stream));
    return SGK_OK;
  }
  SGK_TRY(kv->ensure_self_batch());
  // stage in pieces so a long prefill needs no matching device buffer
  const int64_t piece_rows = std::max<int64_t>(1, std::min<int64_t>(n_rows, (64 << 20) / (kv_dim * 4)));
  SGK_TRY(kv->ensure_io(2 * static_cast<size_t>(piece_rows) * kv_dim * sizeof(float)));
  float* d_k = kv->d_io;
  float* d_v = kv->d_io + static_cast<size_t>(piece_rows) * kv_dim;
  for (int64_t done = 0; done < n_rows; done += piece_rows) {
    int64_t rows = std::min(piece_rows, n_rows - done);
    size_t bytes = static_cast<size_t>(rows) * kv_dim * sizeof(float);
    SGK_CUDA(cudaMemcpyAsync(d_k, k + done * kv_dim, bytes, cudaMemcpyHostToDevice, stream));
    SGK_CUDA(cudaMemcpyAsync(d_v, v + done * kv_dim, bytes, cudaMemcpyHostToDevice, stream));
    SGK_TRY(kv->self_batch->enqueue_append(stream, d_k, d_v, static_cast<int>(rows), nullptr, nullptr));
    SGK_CUDA(cudaStreamSynchronize(stream));
  }
  return check_device_status(kv->st);
}

int32_t sgk_kv_seed_f32(sgk_kv* kv, const float* k, size_t k_len, const float* v, size_t v_len, int64_t n_rows) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  // src/decode_resident/attention.rs:555-572
  if (n_rows < 0 || n_rows > kv->seq->capacity)
    return fail(SGK_ERR_DIMENSION, "seed KV %lld > capacity %lld", (long long)n_rows, (long long)kv->seq->capacity);
  const size_t cells = static_cast<size_t>(n_rows) * kv->kv_dim();
  if (k_len != cells || v_len != cells)
    return fail(SGK_ERR_DIMENSION, "seed KV: expected %zu (=%lld x %d), got keys=%zu values=%zu", cells,
                (long long)n_rows, kv->kv_dim(), k_len, v_len);
  int64_t saved = kv->len();
  kv->seq->len[kv->layer] = 0;
  int rc = append_rows_host(kv, k, k_len, v, v_len, n_rows, true);
  if (rc != SGK_OK && kv->len() == 0) kv->seq->len[kv->layer] = saved;
  return rc;
}

int32_t sgk_kv_append_row_f32(sgk_kv* kv, const float* k, size_t k_len, const float* v, size_t v_len) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  // src/decode_resident/attention.rs:612-625: wrong length, then overflow
  if (k_len != static_cast<size_t>(kv->kv_dim()) || v_len != static_cast<size_t>(kv->kv_dim()))
    return fail(SGK_ERR_DIMENSION, "append KV: expected %d, got key=%zu value=%zu", kv->kv_dim(), k_len, v_len);
  if (kv->len() >= kv->seq->capacity)
    return fail(SGK_ERR_DIMENSION, "append KV: capacity %lld reached (overflow)", (long long)kv->seq->capacity);
  return append_rows_host(kv, k, k_len, v, v_len, 1, false);
}

int32_t sgk_kv_append_rows_f32(sgk_kv* kv, const float* k, size_t k_len, const float* v, size_t v_len, int64_t n_rows) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  // LayerKvCache::append_batch (src/decoder/attention_cache.rs:47-58): seq > 0
  if (n_rows <= 0) return fail(SGK_ERR_DIMENSION, "append_batch needs at least one row");
  if (kv->len() + n_rows > kv->seq->capacity)
    return fail(SGK_ERR_DIMENSION, "append KV: capacity %lld reached (overflow)", (long long)kv->seq->capacity);
  return append_rows_host(kv, k, k_len, v, v_len, n_rows, false);
}

int32_t sgk_kv_enqueue_append(sgk_kv* kv, void* stream, const float* d_k, const float* d_v) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  SGK_TRY(kv->ensure_self_batch());
  return kv->self_batch->enqueue_append(kv->st->pick(stream), d_k, d_v, 1, nullptr, nullptr);
}

int32_t sgk_kv_enqueue_append_rows(sgk_kv* kv, void* stream, const float* d_k, const float* d_v, int64_t n_rows) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  if (n_rows <= 0) return fail(SGK_ERR_DIMENSION, "append_batch needs at least one row");
  SGK_TRY(kv->ensure_self_batch());
  return kv->self_batch->enqueue_append(kv->st->pick(stream), d_k, d_v, static_cast<int>(n_rows), nullptr, nullptr);
}

static int32_t check_rope(const sgk_rope* rope, int head_dim, RopeArgs* out) {
  if (!rope) return fail(SGK_ERR_BACKEND, "null rope parameters");
  // src/decoder/attention_ops.rs:719-724
  if (rope->rope_dims <= 0 || rope->rope_dims > head_dim || rope->rope_dims % 2 != 0)
    return fail(SGK_ERR_DIMENSION, "RMSNorm/RoPE rope_dims %d invalid for head_dim %d", rope->rope_dims, head_dim);
  if (rope->theta <= 0.0f) return fail(SGK_ERR_DIMENSION, "RoPE base_theta invalid: %f", rope->theta);
  if (rope->frequency_dim <= 0) return fail(SGK_ERR_DIMENSION, "RoPE frequency_dim invalid");
  out->rope_dims = rope->rope_dims;
  out->frequency_dim = rope->frequency_dim;
  out->theta = rope->theta;
  out->position_scale = rope->position_scale;
  out->eps = rope->eps;
  out->interleaved = rope->interleaved;
  return SGK_OK;
}

int32_t sgk_kv_enqueue_rope_append(sgk_kv* kv, void* stream, const float* d_k_raw, const float* d_v,
                                   const float* d_knorm_weight, const sgk_rope* rope) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  if (!d_knorm_weight) return fail(SGK_ERR_BACKEND, "null norm weight");
  RopeArgs r;
  SGK_TRY(check_rope(rope, kv->pool()->head_dim, &r));
  SGK_TRY(kv->ensure_self_batch());
  return kv->self_batch->enqueue_append(kv->st->pick(stream), d_k_raw, d_v, 1, &r, d_knorm_weight);
}

int32_t sgk_kv_enqueue_rope_append_rows(sgk_kv* kv, void* stream, const float* d_k_raw, const float* d_v,
                                        int64_t n_rows, const float* d_knorm_weight, const sgk_rope* rope) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  if (!d_knorm_weight) return fail(SGK_ERR_BACKEND, "null norm weight");
  if (n_rows < 0 || n_rows > INT32_MAX) return fail(SGK_ERR_DIMENSION, "append rows: n_rows %lld invalid", (long long)n_rows);
  if (n_rows == 0) return SGK_OK;
  RopeArgs r;
  SGK_TRY(check_rope(rope, kv->pool()->head_dim, &r));
  SGK_TRY(kv->ensure_self_batch());
  return kv->self_batch->enqueue_append(kv->st->pick(stream), d_k_raw, d_v, int(n_rows), &r, d_knorm_weight);
}

int32_t sgk_rms_norm_rope_decode(sgk_state* st, const float* x, const float* weight, int32_t heads, int32_t head_dim,
                                 const sgk_rope* rope, int64_t position, float* out) {
  if (!st || !x || !weight || !out) return fail(SGK_ERR_BACKEND, "null argument");
  if (heads <= 0 || head_dim <= 0 || head_dim > 512)
    return fail(SGK_ERR_DIMENSION, "RMSNorm/RoPE heads invalid: heads=%d, head_dim=%d", heads, head_dim);
  RopeArgs r;
  SGK_TRY(check_rope(rope, head_dim, &r));
  size_t n = size_t(heads) * head_dim;
  float* d = nullptr;
  SGK_CUDA(cudaMalloc(&d, (2 * n + head_dim) * sizeof(float)));
  float *d_x = d, *d_out = d + n, *d_w = d + 2 * n;
  cudaStream_t stream = st->stream;
  AppendArgs a{};
  a.pool.kv_heads = heads;
  a.pool.head_dim = head_dim;
  a.pool.layers = 1;
  a.k = d_x;
  a.v = d_x;
  a.n_rows = 1;
  a.row0 = position;
  a.use_device_len = 0;
  a.bump_len = 0;
  a.has_rope = 1;
  a.knorm_w = d_w;
  a.rope = r;
  a.out_k = d_out;
  a.status = st->d_status;
  // lens is dereferenced only when use_device_len is set; give it a valid word anyway
  a.pool.lens = st->d_status;
  cudaError_t e = cudaMemcpyAsync(d_x, x, n * sizeof(float), cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(d_w, weight, head_dim * sizeof(float), cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = launch_append_rows(a, 1, stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(out, d_out, n * sizeof(float), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  cudaFree(d);
  st->launches += 1;
  if (e != cudaSuccess) return fail(SGK_ERR_BACKEND, "rms_norm_rope_decode failed: %s", cudaGetErrorString(e));
  return SGK_OK;
}

int32_t sgk_kv_attention_decode(sgk_kv* kv, const float* q, size_t q_len, int64_t window_start, float attn_scalar,
                                float* out) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  if (!q || !out) return fail(SGK_ERR_BACKEND, "null host pointer");
  // src/decode_resident/attention.rs:683-698
  if (kv->len() == 0) return fail(SGK_ERR_DIMENSION, "attention_decode on an empty KV");
  const size_t q_dim = static_cast<size_t>(kv->q_dim());
  if (q_len != q_dim) return fail(SGK_ERR_DIMENSION, "attention_decode: q expected [%zu], got %zu", q_dim, q_len);
  SGK_TRY(kv->ensure_self_batch());
  SGK_TRY(kv->ensure_io(2 * q_dim * sizeof(float)));
  cudaStream_t stream = kv->st->stream;
  float* d_q = kv->d_io;
  float* d_out = kv->d_io + q_dim;
  SGK_CUDA(cudaMemcpyAsync(d_q, q, q_dim * sizeof(float), cudaMemcpyHostToDevice, stream));
  SGK_TRY(kv->self_batch->enqueue_attention(stream, d_q, d_out, window_start, 0, attn_scalar, nullptr, nullptr));
  SGK_CUDA(cudaMemcpyAsync(out, d_out, q_dim * sizeof(float), cudaMemcpyDeviceToHost, stream));
  SGK_CUDA(cudaStreamSynchronize(stream));
  return check_device_status(kv->st);
}

int32_t sgk_kv_enqueue_attention(sgk_kv* kv, void* stream, const float* d_q, float* d_out, int64_t window_start,
                                 float attn_scalar) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  SGK_TRY(kv->ensure_self_batch());
  return kv->self_batch->enqueue_attention(kv->st->pick(stream), d_q, d_out, window_start, 0, attn_scalar, nullptr,
                                           nullptr);
}

int32_t sgk_kv_enqueue_append_attention(sgk_kv* kv, void* stream, const float* d_k, const float* d_v,
                                        const float* d_q, float* d_out, int64_t sliding_window, float attn_scalar) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  if (!d_k || !d_v) return fail(SGK_ERR_BACKEND, "append: null device pointer");
  if (sliding_window < 0) return fail(SGK_ERR_DIMENSION, "negative sliding window");
  SGK_TRY(kv->ensure_self_batch());
  return kv->self_batch->enqueue_attention(kv->st->pick(stream), d_q, d_out, 0, sliding_window, attn_scalar, d_k, d_v);
}

int32_t sgk_kv_enqueue_verify_rows(sgk_kv* kv, void* stream, const float* d_k, const float* d_v, const float* d_q,
                                   float* d_out, int32_t n_rows, int64_t sliding_window, float attn_scalar) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  SGK_TRY(kv->ensure_self_batch());
  return sgk_batch_enqueue_verify_rows(static_cast<sgk_batch*>(kv->self_batch.get()), stream, d_k, d_v, d_q, d_out, n_rows,
                                       sliding_window, attn_scalar);
}

static int32_t gather_impl(sgk_kv* kv, int64_t row0, int64_t n, int mode, void* k_out, void* v_out, uint16_t* ks,
                           uint16_t* kb, uint16_t* vs, uint16_t* vb) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  if (!k_out || !v_out) return fail(SGK_ERR_BACKEND, "null host pointer");
  if (row0 < 0 || n < 0 || row0 + n > kv->len())
    return fail(SGK_ERR_DIMENSION, "gather rows [%lld,%lld) outside len %lld", (long long)row0, (long long)(row0 + n),
                (long long)kv->len());
  if (n == 0) return SGK_OK;
  if (row0 / PAGE_TOKENS < kv->seq->released_pages)
    return fail(SGK_ERR_DIMENSION, "gather reaches rows released by the sliding window");
  Pool* pool = kv->pool();
  const size_t cells = static_cast<size_t>(n) * kv->kv_dim();
  size_t esz = mode == 1 ? 4 : (pool->dtype == KV_F32 ? 4 : pool->dtype == KV_BF16 ? 2 : 1);
  const size_t groups = pool->dtype == KV_U8G32 && mode == 2 ? cells / QGROUP : 0;
  size_t bytes = 2 * cells * esz + 4 * groups * sizeof(uint16_t);
  uint8_t* d = nullptr;
  SGK_CUDA(cudaMalloc(&d, bytes));
  GatherArgs a{};
  a.pool = pool->view();
  a.layer = kv->layer;
  a.slot = kv->seq->slot;
  a.row0 = row0;
  a.n = n;
  a.mode = mode;
  a.k_out = d;
  a.v_out = d + cells * esz;
  uint16_t* meta = reinterpret_cast<uint16_t*>(d + 2 * cells * esz);
  a.k_scale = meta;
  a.k_bias = meta + groups;
  a.v_scale = meta + 2 * groups;
  a.v_bias = meta + 3 * groups;
  a.num_pages = pool->num_pages;
  a.status = kv->st->d_status;
  cudaStream_t stream = kv->st->stream;
  cudaError_t e = launch_gather(a, stream);
  kv->st->launches += 1;
  if (e == cudaSuccess) e = cudaMemcpyAsync(k_out, a.k_out, cells * esz, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(v_out, a.v_out, cells * esz, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess && groups) {
    e = cudaMemcpyAsync(ks, a.k_scale, groups * 2, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(kb, a.k_bias, groups * 2, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(vs, a.v_scale, groups * 2, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(vb, a.v_bias, groups * 2, cudaMemcpyDeviceToHost, stream);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  cudaFree(d);
  if (e != cudaSuccess) return fail(SGK_ERR_BACKEND, "gather failed: %s", cudaGetErrorString(e));
  return check_device_status(kv->st);
}

int32_t sgk_kv_gather_rows(sgk_kv* kv, int64_t row0, int64_t n, void* k_out, void* v_out) {
  if (kv && kv->pool()->dtype == KV_U8G32)
    return fail(SGK_ERR_BACKEND, "gather_rows on a u8 KV: use gather_rows_u8 or gather_rows_f32");
  return gather_impl(kv, row0, n, 0, k_out, v_out, nullptr, nullptr, nullptr, nullptr);
}

int32_t sgk_kv_gather_rows_u8(sgk_kv* kv, int64_t row0, int64_t n, uint8_t* k_codes, uint16_t* k_scale,
                              uint16_t* k_bias, uint8_t* v_codes, uint16_t* v_scale, uint16_t* v_bias) {
  if (kv && kv->pool()->dtype != KV_U8G32) return fail(SGK_ERR_BACKEND, "gather_rows_u8 on a KV that is not u8");
  if (!k_scale || !k_bias || !v_scale || !v_bias) return fail(SGK_ERR_BACKEND, "null host pointer");
  return gather_impl(kv, row0, n, 2, k_codes, v_codes, k_scale, k_bias, v_scale, v_bias);
}

int32_t sgk_kv_gather_rows_f32(sgk_kv* kv, int64_t row0, int64_t n, float* k_out, float* v_out) {
  return gather_impl(kv, row0, n, 1, k_out, v_out, nullptr, nullptr, nullptr, nullptr);
}

int32_t sgk_kv_block_table(const sgk_kv* kv, int32_t* pages_out, int64_t cap, int64_t* n_out) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  return sgk_seq_block_table(static_cast<const sgk_seq*>(kv->seq), pages_out, cap, n_out);
}

int32_t sgk_kv_set_attention_kernel(sgk_kv* kv, int32_t which) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  if (which < 0 || which > 2) return fail(SGK_ERR_CONFIG, "kernel selector %d", which);
  SGK_TRY(kv->ensure_self_batch());
  kv->self_batch->kernel_override = which;
  if (kv->self_batch->choose_kernel() < 0) {
    kv->self_batch->kernel_override = 0;
    return fail(SGK_ERR_BACKEND, "tensor-core attention kernel does not take this shape");
  }
  return SGK_OK;
}

// ------------------------------------------------------------------ batch
int32_t sgk_batch_create(sgk_state* st, sgk_kv** kvs, int32_t n, sgk_batch** out) {
  if (!st || !kvs || !out) return fail(SGK_ERR_BACKEND, "batch_create: null argument");
  std::vector<Kv*> list(kvs, kvs + std::max(n, 0));
  Batch* b = nullptr;
  SGK_TRY(create_batch(st, list.data(), n, &b));
  *out = static_cast<sgk_batch*>(b);
  return SGK_OK;
}

void sgk_batch_destroy(sgk_batch* b) {
  if (!b) return;
  cudaSetDevice(b->st->device);
  cudaStreamSynchronize(b->st->stream);
  delete static_cast<Batch*>(b);
}

int32_t sgk_batch_enqueue_append(sgk_batch* b, void* stream, const float* d_k, const float* d_v) {
  if (!b) return fail(SGK_ERR_BACKEND, "null batch");
  return b->enqueue_append(b->st->pick(stream), d_k, d_v, 1, nullptr, nullptr);
}

int32_t sgk_batch_enqueue_attention(sgk_batch* b, void* stream, const float* d_q, float* d_out,
                                    int64_t sliding_window, float attn_scalar) {
  if (!b) return fail(SGK_ERR_BACKEND, "null batch");
  if (sliding_window < 0) return fail(SGK_ERR_DIMENSION, "negative sliding window");
  return b->enqueue_attention(b->st->pick(stream), d_q, d_out, 0, sliding_window, attn_scalar, nullptr, nullptr);
}

int32_t sgk_batch_enqueue_step(sgk_batch* b, void* stream, const float* d_k, const float* d_v, const float* d_q,
                               float* d_out, int64_t sliding_window, float attn_scalar) {
  if (!b) return fail(SGK_ERR_BACKEND, "null batch");
  if (!d_k || !d_v) return fail(SGK_ERR_BACKEND, "append: null device pointer");
  if (sliding_window < 0) return fail(SGK_ERR_DIMENSION, "negative sliding window");
  return b->enqueue_attention(b->st->pick(stream), d_q, d_out, 0, sliding_window, attn_scalar, d_k, d_v);
}

int32_t sgk_batch_enqueue_verify_rows(sgk_batch* b, void* stream, const float* d_k, const float* d_v,
                                      const float* d_q, float* d_out, int32_t n_rows, int64_t sliding_window,
                                      float attn_scalar) {
  if (!b) return fail(SGK_ERR_BACKEND, "null batch");
  if (!d_k || !d_v || !d_q || !d_out) return fail(SGK_ERR_BACKEND, "verify rows: null device pointer");
  if (sliding_window < 0) return fail(SGK_ERR_DIMENSION, "negative sliding window");
  if (n_rows < 0) return fail(SGK_ERR_DIMENSION, "verify rows: n_rows %d invalid", n_rows);
  for (Kv* kv : b->kvs)
    if (kv->len() + n_rows > kv->seq->capacity)
      return fail(SGK_ERR_DIMENSION, "append KV: capacity %lld reached (overflow)", (long long)kv->seq->capacity);
  const size_t kv_step = size_t(b->n()) * b->kvs[0]->kv_dim();
  const size_t q_step = size_t(b->n()) * b->q_heads * b->pool->head_dim;
  cudaStream_t s = b->st->pick(stream);
  for (int32_t r = 0; r < n_rows; ++r)
    SGK_TRY(b->enqueue_attention(s, d_q + r * q_step, d_out + r * q_step, 0, sliding_window, attn_scalar,
                                 d_k + r * kv_step, d_v + r * kv_step));
  return SGK_OK;
}

int32_t sgk_batch_set_splits(sgk_batch* b, int32_t splits) {
  if (!b) return fail(SGK_ERR_BACKEND, "null batch");
  if (splits < 0 || splits > b->max_splits)
    return fail(SGK_ERR_CONFIG, "splits %d outside [0,%d]", splits, b->max_splits);
  b->splits_override = splits;
  return SGK_OK;
}

int32_t sgk_batch_get_splits(const sgk_batch* b, int32_t* splits_out) {
  if (!b || !splits_out) return fail(SGK_ERR_BACKEND, "null argument");
  *splits_out = b->last_splits;
  return SGK_OK;
}

int32_t sgk_batch_set_kernel(sgk_batch* b, int32_t which) {
  if (!b) return fail(SGK_ERR_BACKEND, "null batch");
  if (which < 0 || which > 2) return fail(SGK_ERR_CONFIG, "kernel selector %d", which);
  int saved = b->kernel_override;
  b->kernel_override = which;
  if (b->choose_kernel() < 0) {
    b->kernel_override = saved;
    return fail(SGK_ERR_BACKEND, "tensor-core attention kernel does not take this shape");
  }
  return SGK_OK;
}

int32_t sgk_batch_last_kernel(const sgk_batch* b, int32_t* which_out) {
  if (!b || !which_out) return fail(SGK_ERR_BACKEND, "null argument");
  *which_out = b->last_kernel;
  return SGK_OK;
}

// ------------------------------------------------------------------ step
int32_t sgk_step_create(sgk_state* st, sgk_batch** layers, int32_t n_layers, sgk_step** out) {
  if (!st || !layers || !out) return fail(SGK_ERR_BACKEND, "step_create: null argument");
  if (n_layers <= 0) return fail(SGK_ERR_CONFIG, "step needs at least one layer");
  auto s = std::make_unique<sgk_step>();
  s->st = st;
  for (int i = 0; i < n_layers; ++i) {
    if (!layers[i]) return fail(SGK_ERR_BACKEND, "null batch in step");
    if (layers[i]->n() != layers[0]->n() || layers[i]->q_heads != layers[0]->q_heads ||
        layers[i]->pool->kv_heads != layers[0]->pool->kv_heads || layers[i]->pool->head_dim != layers[0]->pool->head_dim)
      return fail(SGK_ERR_CONFIG, "the layers of a step must share batch size and head shape");
    s->layers.push_back(layers[i]);
  }
  *out = s.release();
  return SGK_OK;
}

void sgk_step_destroy(sgk_step* s) {
  if (!s) return;
  cudaSetDevice(s->st->device);
  cudaStreamSynchronize(s->st->stream);
  delete static_cast<Step*>(s);
}

int32_t sgk_step_enqueue(sgk_step* s, void* stream, const float* d_k, const float* d_v, const float* d_q,
                         float* d_out, const int64_t* sliding_windows, float attn_scalar) {
  if (!s) return fail(SGK_ERR_BACKEND, "null step");
  if (!d_k || !d_v || !d_q || !d_out) return fail(SGK_ERR_BACKEND, "step: null device pointer");
  return s->enqueue(s->st->pick(stream), d_k, d_v, d_q, d_out, sliding_windows, attn_scalar);
}

int32_t sgk_step_capture(sgk_step* s, const float* d_k, const float* d_v, const float* d_q, float* d_out,
                         const int64_t* sliding_windows, float attn_scalar) {
  if (!s) return fail(SGK_ERR_BACKEND, "null step");
  if (!d_k || !d_v || !d_q || !d_out) return fail(SGK_ERR_BACKEND, "step: null device pointer");
  if (s->graph_exec) {
    cudaGraphExecDestroy(s->graph_exec);
    s->graph_exec = nullptr;
  }
  if (s->graph) {
    cudaGraphDestroy(s->graph);
    s->graph = nullptr;
  }
  // No host-side table update may fall inside the capture: make every row of the
  // sequences addressable first, and take private copies of shared tail pages.
  cudaStream_t stream = s->st->stream;
  for (Batch* b : s->layers)
    for (Kv* kv : b->kvs) {
      SGK_TRY(kv->seq->reserve(kv->seq->capacity));
      if (kv->len() < kv->seq->capacity) SGK_TRY(kv->seq->ensure_writable(kv->len(), stream));
    }
  SGK_CUDA(cudaStreamSynchronize(stream));
  // The capture moves the host cursors once; put them back, the first replay moves them again.
  std::vector<std::vector<int64_t>> saved;
  for (Batch* b : s->layers) {
    saved.emplace_back();
    for (Kv* kv : b->kvs) saved.back().push_back(kv->len());
  }
  int64_t launches_before = s->launches;
  SGK_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
  int rc = s->enqueue(stream, d_k, d_v, d_q, d_out, sliding_windows, attn_scalar);
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(stream, &graph);
  for (size_t l = 0; l < s->layers.size(); ++l)
    for (size_t i = 0; i < s->layers[l]->kvs.size(); ++i)
      s->layers[l]->kvs[i]->seq->len[s->layers[l]->layer] = saved[l][i];
  s->launches_per_replay = s->launches - launches_before;
  s->launches = launches_before;
  if (rc != SGK_OK) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (e != cudaSuccess) return fail(SGK_ERR_BACKEND, "graph capture failed: %s", cudaGetErrorString(e));
  s->graph = graph;
  SGK_CUDA(cudaGraphInstantiate(&s->graph_exec, graph, 0));
  return SGK_OK;
}

int32_t sgk_step_replay(sgk_step* s, void* stream) {
  if (!s) return fail(SGK_ERR_BACKEND, "null step");
  if (!s->graph_exec) return fail(SGK_ERR_CONFIG, "step_replay before step_capture");
  for (Batch* b : s->layers)
    for (Kv* kv : b->kvs)
      if (kv->len() >= kv->seq->capacity)
        return fail(SGK_ERR_DIMENSION, "append KV: capacity %lld reached (overflow)", (long long)kv->seq->capacity);
  SGK_CUDA(cudaGraphLaunch(s->graph_exec, s->st->pick(stream)));
  for (Batch* b : s->layers)
    for (Kv* kv : b->kvs) kv->seq->len[b->layer] += 1;
  s->launches += s->launches_per_replay;
  s->st->launches += s->launches_per_replay;
  return SGK_OK;
}

int32_t sgk_step_run_host(sgk_step* s, const float* k, const float* v, const float* q, float* out,
                          const int64_t* sliding_windows, float attn_scalar) {
  if (!s) return fail(SGK_ERR_BACKEND, "null step");
  if (!k || !v || !q || !out) return fail(SGK_ERR_BACKEND, "step: null host pointer");
  size_t n = size_t(s->layers[0]->n());
  size_t kv_cells = s->layers.size() * n * s->layers[0]->kvs[0]->kv_dim();
  size_t q_cells = s->layers.size() * n * s->layers[0]->kvs[0]->q_dim();
  if (!s->d_k) {
    SGK_CUDA(cudaMalloc(&s->d_k, kv_cells * sizeof(float)));
    SGK_CUDA(cudaMalloc(&s->d_v, kv_cells * sizeof(float)));
    SGK_CUDA(cudaMalloc(&s->d_q, q_cells * sizeof(float)));
    SGK_CUDA(cudaMalloc(&s->d_out, q_cells * sizeof(float)));
  }
  // The layers go in a few groups: the inputs of every group are sent on a copy stream as soon
  // as the call starts, a group's kernels wait only for its own inputs, and its outputs leave on
  // a second copy stream while the next group computes. What stays exposed is the first group's
  // inputs and the last group's outputs.
  cudaStream_t stream = s->st->stream;
  const size_t L = s->layers.size();
  const size_t groups = std::min<size_t>(L, 6);
  if (!s->copy_in) {
    SGK_CUDA(cudaStreamCreateWithFlags(&s->copy_in, cudaStreamNonBlocking));
    SGK_CUDA(cudaStreamCreateWithFlags(&s->copy_out, cudaStreamNonBlocking));
  }
  while (s->events.size() < 2 * groups + 1) {
    cudaEvent_t e = nullptr;
    SGK_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    s->events.push_back(e);
  }
  const size_t kv_layer = n * s->layers[0]->kvs[0]->kv_dim(), q_layer = n * s->layers[0]->kvs[0]->q_dim();
  // the copy streams start after whatever the state's stream was given before this call
  SGK_CUDA(cudaEventRecord(s->events[2 * groups], stream));
  SGK_CUDA(cudaStreamWaitEvent(s->copy_in, s->events[2 * groups], 0));
  SGK_CUDA(cudaStreamWaitEvent(s->copy_out, s->events[2 * groups], 0));
  for (size_t g = 0; g < groups; ++g) {
    const size_t l0 = L * g / groups, l1 = L * (g + 1) / groups;
    SGK_CUDA(cudaMemcpyAsync(s->d_k + l0 * kv_layer, k + l0 * kv_layer, (l1 - l0) * kv_layer * sizeof(float),
                             cudaMemcpyHostToDevice, s->copy_in));
    SGK_CUDA(cudaMemcpyAsync(s->d_v + l0 * kv_layer, v + l0 * kv_layer, (l1 - l0) * kv_layer * sizeof(float),
                             cudaMemcpyHostToDevice, s->copy_in));
    SGK_CUDA(cudaMemcpyAsync(s->d_q + l0 * q_layer, q + l0 * q_layer, (l1 - l0) * q_layer * sizeof(float),
                             cudaMemcpyHostToDevice, s->copy_in));
    SGK_CUDA(cudaEventRecord(s->events[2 * g], s->copy_in));
  }
  int rc = SGK_OK;
  for (size_t g = 0; g < groups && rc == SGK_OK; ++g) {
    const size_t l0 = L * g / groups, l1 = L * (g + 1) / groups;
    SGK_CUDA(cudaStreamWaitEvent(stream, s->events[2 * g], 0));
    rc = s->enqueue_range(stream, l0, l1, s->d_k, s->d_v, s->d_q, s->d_out, sliding_windows, attn_scalar);
    if (rc != SGK_OK) break;
    SGK_CUDA(cudaEventRecord(s->events[2 * g + 1], stream));
    SGK_CUDA(cudaStreamWaitEvent(s->copy_out, s->events[2 * g + 1], 0));
    SGK_CUDA(cudaMemcpyAsync(out + l0 * q_layer, s->d_out + l0 * q_layer, (l1 - l0) * q_layer * sizeof(float),
                             cudaMemcpyDeviceToHost, s->copy_out));
  }
  SGK_CUDA(cudaStreamSynchronize(s->copy_in));
  SGK_CUDA(cudaStreamSynchronize(stream));
  SGK_CUDA(cudaStreamSynchronize(s->copy_out));
  return rc;
}

int64_t sgk_step_launches(const sgk_step* s) { return s ? s->launches : 0; }

// ------------------------------------------------------------------ linear state
int32_t sgk_linstate_create(sgk_state* st, int32_t layers, int64_t conv_len, int64_t ssm_len, int32_t ssm_bf16,
                            sgk_linstate** out) {
  if (!st || !out) return fail(SGK_ERR_BACKEND, "linstate_create: null argument");
  if (layers <= 0 || conv_len < 0 || ssm_len <= 0) return fail(SGK_ERR_CONFIG, "linear state: zero dimension");
  auto ls = std::make_unique<sgk_linstate>();
  ls->st = st;
  ls->layers = layers;
  ls->conv_len = conv_len;
  ls->ssm_len = ssm_len;
  ls->ssm_bf16 = ssm_bf16 != 0;
  auto up = [](int64_t b) { return (b + 255) / 256 * 256; };
  ls->conv_stride = up(conv_len * 4);
  ls->layer_stride = ls->conv_stride + up(ssm_len * ls->ssm_elem());
  ls->total_bytes = ls->layer_stride * layers;
  SGK_CUDA(cudaSetDevice(st->device));
  cudaError_t e = cudaMalloc(&ls->d_base, static_cast<size_t>(ls->total_bytes));
  if (e != cudaSuccess)
    return fail(SGK_ERR_MEMORY_GUARD, "linear state of %lld bytes does not fit: %s", (long long)ls->total_bytes,
                cudaGetErrorString(e));
  SGK_CUDA(cudaMemset(ls->d_base, 0, static_cast<size_t>(ls->total_bytes)));
  SGK_CUDA(cudaMalloc(&ls->d_head_counters, 64 * sizeof(int32_t)));
  SGK_CUDA(cudaMemset(ls->d_head_counters, 0, 64 * sizeof(int32_t)));
  *out = ls.release();
  return SGK_OK;
}

void sgk_linstate_destroy(sgk_linstate* ls) {
  if (!ls) return;
  cudaSetDevice(ls->st->device);
  cudaStreamSynchronize(ls->st->stream);
  delete static_cast<LinState*>(ls);
}

int64_t sgk_linstate_bytes(const sgk_linstate* ls) { return ls ? ls->estimated_bytes() : 0; }

void* sgk_linstate_conv_ptr(sgk_linstate* ls, int32_t layer) {
  if (!ls || layer < 0 || layer >= ls->layers) return nullptr;
  return ls->d_base + ls->layer_stride * layer;
}
void* sgk_linstate_ssm_ptr(sgk_linstate* ls, int32_t layer) {
  if (!ls || layer < 0 || layer >= ls->layers) return nullptr;
  return ls->d_base + ls->layer_stride * layer + ls->conv_stride;
}

int32_t sgk_linstate_write(sgk_linstate* ls, int32_t layer, const float* conv, const float* ssm) {
  if (!ls || !ssm || (ls && ls->conv_len > 0 && !conv)) return fail(SGK_ERR_BACKEND, "null argument");
  if (layer < 0 || layer >= ls->layers) return fail(SGK_ERR_DIMENSION, "layer %d out of range", layer);
  if (ls->conv_len > 0)
    SGK_CUDA(cudaMemcpy(sgk_linstate_conv_ptr(ls, layer), conv, size_t(ls->conv_len) * 4, cudaMemcpyHostToDevice));
  if (ls->ssm_bf16) {
    // same rounding as buffer_from_linear_ssm_seed: f32 -> bf16 RNE on the host
    std::vector<uint16_t> tmp(static_cast<size_t>(ls->ssm_len));
    for (size_t i = 0; i < tmp.size(); ++i) {
      uint32_t bits;
      std::memcpy(&bits, ssm + i, 4);
      tmp[i] = static_cast<uint16_t>((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
    }
    SGK_CUDA(cudaMemcpy(sgk_linstate_ssm_ptr(ls, layer), tmp.data(), tmp.size() * 2, cudaMemcpyHostToDevice));
  } else {
    SGK_CUDA(cudaMemcpy(sgk_linstate_ssm_ptr(ls, layer), ssm, size_t(ls->ssm_len) * 4, cudaMemcpyHostToDevice));
  }
  return SGK_OK;
}

int32_t sgk_linstate_read(sgk_linstate* ls, int32_t layer, float* conv, float* ssm) {
  if (!ls || !ssm || (ls && ls->conv_len > 0 && !conv)) return fail(SGK_ERR_BACKEND, "null argument");
  if (layer < 0 || layer >= ls->layers) return fail(SGK_ERR_DIMENSION, "layer %d out of range", layer);
  SGK_CUDA(cudaStreamSynchronize(ls->st->stream));
  if (ls->conv_len > 0)
    SGK_CUDA(cudaMemcpy(conv, sgk_linstate_conv_ptr(ls, layer), size_t(ls->conv_len) * 4, cudaMemcpyDeviceToHost));
  if (ls->ssm_bf16) {
    std::vector<uint16_t> tmp(static_cast<size_t>(ls->ssm_len));
    SGK_CUDA(cudaMemcpy(tmp.data(), sgk_linstate_ssm_ptr(ls, layer), tmp.size() * 2, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < tmp.size(); ++i) {
      uint32_t bits = static_cast<uint32_t>(tmp[i]) << 16;
      std::memcpy(ssm + i, &bits, 4);
    }
  } else {
    SGK_CUDA(cudaMemcpy(ssm, sgk_linstate_ssm_ptr(ls, layer), size_t(ls->ssm_len) * 4, cudaMemcpyDeviceToHost));
  }
  return SGK_OK;
}

int32_t sgk_linstate_snapshot(sgk_linstate* ls, void* stream, sgk_linstate** snapshot_out) {
  if (!ls || !snapshot_out) return fail(SGK_ERR_BACKEND, "null argument");
  sgk_linstate* snap = nullptr;
  SGK_TRY(sgk_linstate_create(static_cast<sgk_state*>(ls->st), ls->layers, ls->conv_len, ls->ssm_len, ls->ssm_bf16, &snap));
  // all layers in one launch (the reference: one blit encoder, one submission)
  cudaError_t e = launch_copy_bytes(snap->d_base, ls->d_base, ls->total_bytes, ls->st->pick(stream));
  ls->st->launches += 1;
  if (e != cudaSuccess) {
    sgk_linstate_destroy(snap);
    return fail(SGK_ERR_BACKEND, "linear-state snapshot failed: %s", cudaGetErrorString(e));
  }
  *snapshot_out = snap;
  return SGK_OK;
}

int32_t sgk_linstate_restore(sgk_linstate* ls, void* stream, const sgk_linstate* snap) {
  if (!ls || !snap) return fail(SGK_ERR_BACKEND, "null argument");
  // src/metal_backend/linear_attention.rs:3133-3149,3172-3187
  if (ls->conv_len != snap->conv_len || ls->ssm_len != snap->ssm_len || ls->ssm_bf16 != snap->ssm_bf16 ||
      ls->layers != snap->layers)
    return fail(SGK_ERR_SHAPE, "restore linear-attn: snapshot conv=%lld/ssm=%lld/bf16=%d != state conv=%lld/ssm=%lld/bf16=%d",
                (long long)snap->conv_len, (long long)snap->ssm_len, int(snap->ssm_bf16), (long long)ls->conv_len,
                (long long)ls->ssm_len, int(ls->ssm_bf16));
  SGK_CUDA(launch_copy_bytes(ls->d_base, snap->d_base, ls->total_bytes, ls->st->pick(stream)));
  ls->st->launches += 1;
  return SGK_OK;
}

int32_t sgk_lm_head_enqueue_argmax(sgk_state* st, void* stream, const void* d_weight, int32_t weight_dtype,
                                   int64_t vocab, int32_t hidden, const float* d_x, int32_t n_rows,
                                   int32_t index_offset, int32_t* d_index_out, float* d_value_out) {
  if (!st || !d_weight || !d_x || !d_index_out) return fail(SGK_ERR_BACKEND, "null argument");
  if (weight_dtype != SGK_KV_F32 && weight_dtype != SGK_KV_BF16)
    return fail(SGK_ERR_CONFIG, "lm_head weight dtype %d: only dense f32 and bf16 weights are supported", weight_dtype);
  // argmax of an empty slice is None (src/sampling.rs:49-62); the device form has no None to write
  if (vocab <= 0 || hidden <= 0) return fail(SGK_ERR_DIMENSION, "lm_head argmax: vocab %lld, hidden %d must be positive",
                                              (long long)vocab, hidden);
  if (vocab > 0x7fffffffLL) return fail(SGK_ERR_DIMENSION, "lm_head argmax: vocab %lld exceeds the 32-bit index", (long long)vocab);
  if (n_rows < 1 || n_rows > 8) return fail(SGK_ERR_DIMENSION, "lm_head argmax: %d rows, 1 to 8 per call", n_rows);
  if (hidden % 8 != 0) return fail(SGK_ERR_CONFIG, "lm_head argmax: hidden %d must be a multiple of 8", hidden);
  if (lm_head_smem_bytes(weight_dtype == SGK_KV_BF16, n_rows, hidden) > size_t(200) * 1024)
    return fail(SGK_ERR_CONFIG, "lm_head argmax: %d rows of %d values do not fit 200 KiB of shared memory", n_rows, hidden);
  if ((reinterpret_cast<uintptr_t>(d_weight) & 15) || (reinterpret_cast<uintptr_t>(d_x) & 15))
    return fail(SGK_ERR_CONFIG, "lm_head argmax: weight and x must be 16-byte aligned");
  LmHeadArgs a{};
  a.w = d_weight;
  a.w_bf16 = weight_dtype == SGK_KV_BF16;
  a.vocab = vocab;
  a.hidden = hidden;
  a.n_rows = n_rows;
  a.x = d_x;
  a.keys = st->d_lm_ws;
  a.counter = reinterpret_cast<unsigned int*>(st->d_lm_ws + 8);
  a.index_offset = index_offset;
  a.index_out = d_index_out;
  a.value_out = d_value_out;
  a.index_mirror = st->lm_index_mirror;
  st->lm_index_mirror = nullptr;
  cudaStream_t cs = st->pick(stream);
  const bool member = st->chain_member(cs);
  a.pdl_trigger = member ? 1 : 0;
  a.pdl_wait = st->chain_follows(cs) ? 1 : 0;
  SGK_CUDA(launch_lm_head_argmax(a, st->sm_count, cs));
  st->launches += 1;
  if (member) st->chain_note();
  return SGK_OK;
}

int32_t sgk_embed_enqueue_from_index(sgk_state* st, void* stream, const void* d_table, int32_t table_dtype,
                                     int64_t vocab, int32_t hidden, const int32_t* d_index, float embedding_scale,
                                     int32_t recast_bf16, float* d_out) {
  if (!st || !d_table || !d_index || !d_out) return fail(SGK_ERR_BACKEND, "null argument");
  if (table_dtype != SGK_KV_F32 && table_dtype != SGK_KV_BF16)
    return fail(SGK_ERR_CONFIG, "embedding table dtype %d: only dense f32 and bf16 tables are supported", table_dtype);
  if (vocab <= 0 || hidden <= 0 || vocab > 0x7fffffffLL)
    return fail(SGK_ERR_DIMENSION, "embedding: vocab %lld, hidden %d invalid", (long long)vocab, hidden);
  cudaStream_t cs = st->pick(stream);
  const bool member = st->chain_member(cs);
  SGK_CUDA(launch_embed_gather(d_table, table_dtype == SGK_KV_BF16, d_index, vocab, hidden, embedding_scale,
                               recast_bf16 != 0, d_out, member ? 1 : 0, st->chain_follows(cs) ? 1 : 0, cs));
  st->launches += 1;
  if (member) st->chain_note();
  return SGK_OK;
}

static int32_t check_affine(const sgk_affine_weight* w, int32_t hidden, const char* what) {
  if (!w || !w->d_packed || !w->d_scales || !w->d_biases) return fail(SGK_ERR_BACKEND, "%s: null pointer in the quantised weight", what);
  if (w->bits != 4 && w->bits != 8) return fail(SGK_ERR_CONFIG, "%s: %d-bit codes (4 and 8 are supported)", what, w->bits);
  if (w->group_size != 64 && w->group_size != 128)
    return fail(SGK_ERR_CONFIG, "%s: group size %d (64 and 128 are supported)", what, w->group_size);
  if (hidden <= 0 || hidden % w->group_size != 0)
    return fail(SGK_ERR_DIMENSION, "%s: hidden %d is not a multiple of the group size %d", what, hidden, w->group_size);
  if (reinterpret_cast<uintptr_t>(w->d_packed) & 15) return fail(SGK_ERR_CONFIG, "%s: codes must be 16-byte aligned", what);
  return SGK_OK;
}

int32_t sgk_lm_head_enqueue_argmax_affine(sgk_state* st, void* stream, const sgk_affine_weight* weight, int64_t vocab,
                                          int32_t hidden, const float* d_x, int32_t n_rows, int32_t index_offset,
                                          int32_t* d_index_out, float* d_value_out) {
  if (!st || !d_x || !d_index_out) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_TRY(check_affine(weight, hidden, "lm_head argmax"));
  if (vocab <= 0 || vocab > 0x7fffffffLL) return fail(SGK_ERR_DIMENSION, "lm_head argmax: vocab %lld invalid", (long long)vocab);
  if (n_rows < 1 || n_rows > 8) return fail(SGK_ERR_DIMENSION, "lm_head argmax: %d rows, 1 to 8 per call", n_rows);
  if (lm_head_affine_smem_bytes(n_rows, hidden, weight->group_size) > size_t(200) * 1024)
    return fail(SGK_ERR_CONFIG, "lm_head argmax: %d rows of %d values do not fit 200 KiB of shared memory", n_rows, hidden);
  LmHeadAffineArgs a{};
  a.w = AffineWeight{weight->d_packed, weight->d_scales, weight->d_biases, weight->bits, weight->group_size};
  a.vocab = vocab;
  a.hidden = hidden;
  a.n_rows = n_rows;
  a.x = d_x;
  a.keys = st->d_lm_ws;
  a.counter = reinterpret_cast<unsigned int*>(st->d_lm_ws + 8);
  a.index_offset = index_offset;
  a.index_out = d_index_out;
  a.value_out = d_value_out;
  a.index_mirror = st->lm_index_mirror;
  st->lm_index_mirror = nullptr;
  cudaStream_t cs = st->pick(stream);
  const bool member = st->chain_member(cs);
  a.pdl_trigger = member ? 1 : 0;
  a.pdl_wait = st->chain_follows(cs) ? 1 : 0;
  SGK_CUDA(launch_lm_head_argmax_affine(a, st->sm_count, cs));
  st->launches += 1;
  if (member) st->chain_note();
  return SGK_OK;
}

int32_t sgk_embed_enqueue_from_index_affine(sgk_state* st, void* stream, const sgk_affine_weight* table, int64_t vocab,
                                            int32_t hidden, const int32_t* d_index, float embedding_scale,
                                            int32_t recast_bf16, float* d_out) {
  if (!st || !d_index || !d_out) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_TRY(check_affine(table, hidden, "embedding"));
  if (vocab <= 0 || vocab > 0x7fffffffLL) return fail(SGK_ERR_DIMENSION, "embedding: vocab %lld invalid", (long long)vocab);
  cudaStream_t cs = st->pick(stream);
  const bool member = st->chain_member(cs);
  SGK_CUDA(launch_embed_gather_affine(AffineWeight{table->d_packed, table->d_scales, table->d_biases, table->bits, table->group_size},
                                      d_index, vocab, hidden, embedding_scale, recast_bf16 != 0, d_out, member ? 1 : 0,
                                      st->chain_follows(cs) ? 1 : 0, cs));
  st->launches += 1;
  if (member) st->chain_note();
  return SGK_OK;
}

// ------------------------------------------------------------------ peer memory and the exchange
int32_t sgk_peer_export(sgk_state* st, void* d_ptr, uint8_t handle_out[64]) {
  if (!st || !d_ptr || !handle_out) return fail(SGK_ERR_BACKEND, "null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  SGK_CUDA(cudaSetDevice(st->device));
  cudaIpcMemHandle_t h;
  SGK_CUDA(cudaIpcGetMemHandle(&h, d_ptr));
  std::memcpy(handle_out, &h, 64);
  return SGK_OK;
}

int32_t sgk_peer_open(sgk_state* st, const uint8_t handle[64], void** d_ptr_out) {
  if (!st || !handle || !d_ptr_out) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_CUDA(cudaSetDevice(st->device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  SGK_CUDA(cudaIpcOpenMemHandle(d_ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  return SGK_OK;
}

int32_t sgk_peer_close(sgk_state* st, void* d_ptr) {
  if (!st || !d_ptr) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_CUDA(cudaSetDevice(st->device));
  SGK_CUDA(cudaIpcCloseMemHandle(d_ptr));
  return SGK_OK;
}

int32_t sgk_exchange_create(sgk_state* st, int32_t rank, int32_t n_ranks, sgk_exchange** out, uint8_t flags_handle_out[64]) {
  if (!st || !out || !flags_handle_out) return fail(SGK_ERR_BACKEND, "null argument");
  if (n_ranks < 2 || n_ranks > EXCHANGE_MAX_RANKS || rank < 0 || rank >= n_ranks)
    return fail(SGK_ERR_CONFIG, "exchange: rank %d of %d (2 to %d ranks)", rank, n_ranks, EXCHANGE_MAX_RANKS);
  SGK_CUDA(cudaSetDevice(st->device));
  auto ex = std::make_unique<sgk_exchange>();
  ex->st = st;
  ex->rank = rank;
  ex->n_ranks = n_ranks;
  SGK_CUDA(cudaMalloc(&ex->d_flags, sizeof(int32_t) * (n_ranks + 2)));
  SGK_CUDA(cudaMemset(ex->d_flags, 0, sizeof(int32_t) * (n_ranks + 2)));
  cudaIpcMemHandle_t h;
  SGK_CUDA(cudaIpcGetMemHandle(&h, ex->d_flags));
  std::memcpy(flags_handle_out, &h, 64);
  *out = ex.release();
  return SGK_OK;
}

void sgk_exchange_destroy(sgk_exchange* ex) {
  if (!ex) return;
  cudaSetDevice(ex->st->device);
  delete ex;
}

int32_t sgk_exchange_connect(sgk_exchange* ex, int32_t peer_rank, const uint8_t peer_flags_handle[64]) {
  if (!ex || !peer_flags_handle) return fail(SGK_ERR_BACKEND, "null argument");
  if (peer_rank < 0 || peer_rank >= ex->n_ranks || peer_rank == ex->rank)
    return fail(SGK_ERR_CONFIG, "exchange: peer %d of %d (own rank %d)", peer_rank, ex->n_ranks, ex->rank);
  if (ex->peer_flags[peer_rank]) return fail(SGK_ERR_CONFIG, "exchange: peer %d is connected already", peer_rank);
  SGK_CUDA(cudaSetDevice(ex->st->device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, peer_flags_handle, 64);
  void* p = nullptr;
  SGK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  ex->peer_flags[peer_rank] = static_cast<int32_t*>(p);
  return SGK_OK;
}

int32_t sgk_exchange_enqueue(sgk_exchange* ex, void* stream, float* d_local_row, float* const* d_peer_rows,
                             int64_t slice_offset, int32_t slice_floats) {
  if (!ex || !d_local_row || !d_peer_rows) return fail(SGK_ERR_BACKEND, "null argument");
  if (slice_offset < 0 || slice_floats <= 0 || slice_offset % 4 != 0 || slice_floats % 4 != 0)
    return fail(SGK_ERR_DIMENSION, "exchange: slice of %d floats at %lld (multiples of 4)", slice_floats,
                (long long)slice_offset);
  ExchangeArgs a{};
  a.local_row = d_local_row;
  for (int p = 0; p < ex->n_ranks; ++p) {
    if (p == ex->rank) continue;
    if (!ex->peer_flags[p]) return fail(SGK_ERR_CONFIG, "exchange: peer %d is not connected", p);
    if (!d_peer_rows[p]) return fail(SGK_ERR_BACKEND, "exchange: no row for peer %d", p);
    if (reinterpret_cast<uintptr_t>(d_peer_rows[p]) & 15) return fail(SGK_ERR_CONFIG, "exchange: rows must be 16-byte aligned");
    a.peer_row[p] = d_peer_rows[p];
    a.peer_flags[p] = ex->peer_flags[p];
  }
  if (reinterpret_cast<uintptr_t>(d_local_row) & 15) return fail(SGK_ERR_CONFIG, "exchange: rows must be 16-byte aligned");
  a.local_flags = ex->d_flags;
  a.step = ex->d_flags + ex->n_ranks;
  a.slice_offset = slice_offset;
  a.slice_floats = slice_floats;
  a.rank = ex->rank;
  a.n_ranks = ex->n_ranks;
  a.status = ex->st->d_status;
  SGK_CUDA(launch_exchange_slices(a, ex->st->pick(stream)));
  ex->st->launches += 1;
  return SGK_OK;
}

int32_t sgk_batch_enqueue_step_exchange(sgk_batch* b, void* stream, const float* d_k, const float* d_v, const float* d_q,
                                        sgk_exchange* ex, float* d_local_row, float* const* d_peer_rows,
                                        int64_t slice_offset, int64_t sliding_window, float attn_scalar) {
  if (!b || !ex || !d_local_row || !d_peer_rows) return fail(SGK_ERR_BACKEND, "null argument");
  if (!d_k || !d_v || !d_q) return fail(SGK_ERR_BACKEND, "append: null device pointer");
  if (sliding_window < 0) return fail(SGK_ERR_DIMENSION, "negative sliding window");
  if (slice_offset < 0 || slice_offset % 4 != 0) return fail(SGK_ERR_DIMENSION, "exchange: slice offset %lld", (long long)slice_offset);
  const int64_t slice = int64_t(b->n()) * b->q_heads * b->pool->head_dim;
  PeerTarget target;
  target.ex = ex;
  for (int p = 0; p < ex->n_ranks; ++p) {
    if (p == ex->rank) continue;
    if (!ex->peer_flags[p]) return fail(SGK_ERR_CONFIG, "exchange: peer %d is not connected", p);
    if (!d_peer_rows[p]) return fail(SGK_ERR_BACKEND, "exchange: no row for peer %d", p);
    if (reinterpret_cast<uintptr_t>(d_peer_rows[p]) & 15) return fail(SGK_ERR_CONFIG, "exchange: rows must be 16-byte aligned");
    target.peer_out[p] = d_peer_rows[p] + slice_offset;
  }
  if (reinterpret_cast<uintptr_t>(d_local_row) & 15) return fail(SGK_ERR_CONFIG, "exchange: rows must be 16-byte aligned");
  b->peer_target = &target;
  b->peer_target_fused = false;
  int32_t rc = b->enqueue_attention(b->st->pick(stream), d_q, d_local_row + slice_offset, 0, sliding_window, attn_scalar,
                                    d_k, d_v);
  b->peer_target = nullptr;
  if (rc != SGK_OK) return rc;
  if (b->peer_target_fused) return SGK_OK;
  // the launch could not take the peers (generic kernel, uneven batch, cluster merge): the small kernel does it
  return sgk_exchange_enqueue(ex, stream, d_local_row, d_peer_rows, slice_offset, static_cast<int32_t>(slice));
}

// ------------------------------------------------------------------ token window
int32_t sgk_token_window_create(sgk_state* st, int32_t depth, sgk_token_window** out) {
  if (!st || !out) return fail(SGK_ERR_BACKEND, "null argument");
  if (depth < 1 || depth > 64) return fail(SGK_ERR_CONFIG, "token window depth %d: 1 to 64", depth);
  SGK_CUDA(cudaSetDevice(st->device));
  auto w = std::make_unique<sgk_token_window>();
  w->st = st;
  w->depth = depth;
  SGK_CUDA(cudaMalloc(&w->d_ring, sizeof(int32_t) * depth));
  SGK_CUDA(cudaMemset(w->d_ring, 0xff, sizeof(int32_t) * depth));
  SGK_CUDA(cudaHostAlloc(&w->h_ring, sizeof(int32_t) * depth, cudaHostAllocMapped));
  SGK_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&w->h_ring_dev), w->h_ring, 0));
  for (int i = 0; i < depth; ++i) {
    w->h_ring[i] = -1;
    cudaEvent_t e;
    SGK_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    w->done.push_back(e);
  }
  *out = w.release();
  return SGK_OK;
}

void sgk_token_window_destroy(sgk_token_window* w) { delete w; }

int32_t* sgk_token_window_output_slot(sgk_token_window* w) {
  if (!w || w->inflight >= w->depth) return nullptr;
  return w->d_ring + (w->enqueued % w->depth);
}

const int32_t* sgk_token_window_previous_slot(sgk_token_window* w) {
  if (!w || w->enqueued == 0) return nullptr;
  return w->d_ring + ((w->enqueued - 1) % w->depth);
}

int32_t sgk_token_window_submit(sgk_token_window* w, void* stream) {
  if (!w) return fail(SGK_ERR_BACKEND, "null argument");
  if (w->inflight >= w->depth)
    return fail(SGK_ERR_DIMENSION, "token window: %d tokens in flight, the window holds %d", w->inflight, w->depth);
  const int slot = static_cast<int>(w->enqueued % w->depth);
  cudaStream_t s = w->st->pick(stream);
  SGK_CUDA(cudaMemcpyAsync(w->h_ring + slot, w->d_ring + slot, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  SGK_CUDA(cudaEventRecord(w->done[slot], s));
  w->enqueued += 1;
  w->inflight += 1;
  return SGK_OK;
}

int32_t sgk_token_window_pop(sgk_token_window* w, int32_t* token_out) {
  if (!w || !token_out) return fail(SGK_ERR_BACKEND, "null argument");
  if (w->inflight == 0) return fail(SGK_ERR_DIMENSION, "token window: nothing in flight");
  const int slot = static_cast<int>((w->enqueued - w->inflight) % w->depth);
  SGK_CUDA(cudaEventSynchronize(w->done[slot]));
  *token_out = w->h_ring[slot];
  w->inflight -= 1;
  return SGK_OK;
}

int32_t sgk_token_window_inflight(const sgk_token_window* w) { return w ? w->inflight : 0; }
int64_t sgk_token_window_enqueued(const sgk_token_window* w) { return w ? w->enqueued : 0; }
int32_t sgk_token_window_depth(const sgk_token_window* w) { return w ? w->depth : 0; }

int32_t sgk_token_window_drain(sgk_token_window* w) {
  if (!w) return fail(SGK_ERR_BACKEND, "null argument");
  while (w->inflight > 0) {
    const int slot = static_cast<int>((w->enqueued - w->inflight) % w->depth);
    SGK_CUDA(cudaEventSynchronize(w->done[slot]));
    w->inflight -= 1;
  }
  return SGK_OK;
}

// ------------------------------------------------------------------ the whole token as one graph
int32_t sgk_token_capture(sgk_step* s, sgk_token_window* w, const sgk_token_io* io, const float* d_k, const float* d_v,
                          const float* d_q, float* d_out, const int64_t* sliding_windows, float attn_scalar) {
  if (!s || !w || !io) return fail(SGK_ERR_BACKEND, "token_capture: null argument");
  if (!d_k || !d_v || !d_q || !d_out) return fail(SGK_ERR_BACKEND, "token_capture: null device pointer");
  if ((!io->d_table && !io->table_affine) || !io->d_x || (!io->d_lm_weight && !io->lm_affine) || !io->d_final)
    return fail(SGK_ERR_BACKEND, "token_capture: null pointer in the token's inputs");
  if (w->st != s->st) return fail(SGK_ERR_CONFIG, "token_capture: window and step belong to different states");
  if (w->inflight != 0) return fail(SGK_ERR_DIMENSION, "token_capture with %d tokens in flight", w->inflight);
  State* st = s->st;
  for (cudaGraphExec_t e : s->token_execs)
    if (e) cudaGraphExecDestroy(e);
  s->token_execs.clear();
  s->token_window = nullptr;
  cudaStream_t stream = st->stream;
  // as in sgk_step_capture: no host-side table update may fall inside the capture
  for (Batch* b : s->layers)
    for (Kv* kv : b->kvs) {
      SGK_TRY(kv->seq->reserve(kv->seq->capacity));
      if (kv->len() < kv->seq->capacity) SGK_TRY(kv->seq->ensure_writable(kv->len(), stream));
    }
  SGK_CUDA(cudaStreamSynchronize(stream));
  std::vector<std::vector<int64_t>> saved;
  for (Batch* b : s->layers) {
    saved.emplace_back();
    for (Kv* kv : b->kvs) saved.back().push_back(kv->len());
  }
  const int64_t launches_before = s->launches, state_before = st->launches;
  int rc = SGK_OK;
  // One graph per slot of the ring: token n runs graph n % depth, which reads the index token n-1
  // left in slot (n-1) % depth and leaves its own in slot n % depth (and in the pinned mirror).
  for (int slot = 0; slot < w->depth && rc == SGK_OK; ++slot) {
    const int32_t* d_prev = w->d_ring + (slot + w->depth - 1) % w->depth;
    SGK_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    st->chain_active = true;   // the token is one chain: embedding, layers, epilogue
    st->chain_stream = stream;
    st->chain_mark = -1;
    rc = io->table_affine
             ? sgk_embed_enqueue_from_index_affine(static_cast<sgk_state*>(st), stream, io->table_affine, io->vocab, io->hidden,
                                                   d_prev, io->embedding_scale, io->recast_bf16, io->d_x)
             : sgk_embed_enqueue_from_index(static_cast<sgk_state*>(st), stream, io->d_table, io->table_dtype, io->vocab,
                                            io->hidden, d_prev, io->embedding_scale, io->recast_bf16, io->d_x);
    if (rc == SGK_OK) rc = s->enqueue(stream, d_k, d_v, d_q, d_out, sliding_windows, attn_scalar);
    // the epilogue writes the token's index into the ring slot and into the slot's pinned mirror
    // itself: no copy node sits between this token's last kernel and the next token's first one
    if (rc == SGK_OK) st->lm_index_mirror = w->h_ring_dev + slot;
    if (rc == SGK_OK)
      rc = io->lm_affine
               ? sgk_lm_head_enqueue_argmax_affine(static_cast<sgk_state*>(st), stream, io->lm_affine, io->vocab, io->hidden,
                                                   io->d_final, 1, 0, w->d_ring + slot, nullptr)
               : sgk_lm_head_enqueue_argmax(static_cast<sgk_state*>(st), stream, io->d_lm_weight, io->lm_weight_dtype,
                                            io->vocab, io->hidden, io->d_final, 1, 0, w->d_ring + slot, nullptr);
    st->chain_active = false;
    st->lm_index_mirror = nullptr;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(stream, &graph);
    for (size_t l = 0; l < s->layers.size(); ++l)
      for (size_t i = 0; i < s->layers[l]->kvs.size(); ++i)
        s->layers[l]->kvs[i]->seq->len[s->layers[l]->layer] = saved[l][i];
    if (slot == 0) s->launches_per_replay = st->launches - state_before;
    if (rc == SGK_OK && e != cudaSuccess) rc = fail(SGK_ERR_BACKEND, "graph capture failed: %s", cudaGetErrorString(e));
    if (rc == SGK_OK) {
      cudaGraphExec_t exec = nullptr;
      cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
      if (ie != cudaSuccess) rc = fail(SGK_ERR_BACKEND, "graph instantiation failed: %s", cudaGetErrorString(ie));
      else s->token_execs.push_back(exec);
    }
    if (graph) cudaGraphDestroy(graph);
  }
  s->launches = launches_before;
  st->launches = state_before;
  if (rc != SGK_OK) {
    for (cudaGraphExec_t e : s->token_execs)
      if (e) cudaGraphExecDestroy(e);
    s->token_execs.clear();
    return rc;
  }
  s->token_window = w;
  return SGK_OK;
}

int32_t sgk_token_seed(sgk_step* s, int32_t first_token, void* stream) {
  if (!s || !s->token_window) return fail(SGK_ERR_CONFIG, "token_seed before token_capture");
  TokenWindow* w = s->token_window;
  if (w->inflight != 0) return fail(SGK_ERR_DIMENSION, "token_seed with %d tokens in flight", w->inflight);
  // the slot the NEXT token's graph reads its input index from
  const int prev = static_cast<int>((w->enqueued + w->depth - 1) % w->depth);
  SGK_CUDA(launch_set_len(w->d_ring + prev, first_token, s->st->pick(stream)));
  s->st->launches += 1;
  return SGK_OK;
}

int32_t sgk_token_submit(sgk_step* s, void* stream) {
  if (!s || !s->token_window || s->token_execs.empty()) return fail(SGK_ERR_CONFIG, "token_submit before token_capture");
  TokenWindow* w = s->token_window;
  if (w->inflight >= w->depth)
    return fail(SGK_ERR_DIMENSION, "token window: %d tokens in flight, the window holds %d", w->inflight, w->depth);
  for (Batch* b : s->layers)
    for (Kv* kv : b->kvs)
      if (kv->len() >= kv->seq->capacity)
        return fail(SGK_ERR_DIMENSION, "append KV: capacity %lld reached (overflow)", (long long)kv->seq->capacity);
  const int slot = static_cast<int>(w->enqueued % w->depth);
  cudaStream_t cs = s->st->pick(stream);
  SGK_CUDA(cudaGraphLaunch(s->token_execs[slot], cs));   // the token's ONE submission
  SGK_CUDA(cudaEventRecord(w->done[slot], cs));
  for (Batch* b : s->layers)
    for (Kv* kv : b->kvs) kv->seq->len[b->layer] += 1;
  s->launches += s->launches_per_replay;
  s->st->launches += s->launches_per_replay;
  w->enqueued += 1;
  w->inflight += 1;
  return SGK_OK;
}

int32_t sgk_linstate_enqueue_capture(sgk_linstate* ls, void* stream, sgk_linstate* capture) {
  if (!ls || !capture) return fail(SGK_ERR_BACKEND, "null argument");
  if (ls == capture) return fail(SGK_ERR_SHAPE, "capture linear-attn: the capture is the state itself");
  // src/metal_backend/linear_attention.rs:105-124
  if (ls->conv_len != capture->conv_len || ls->ssm_len != capture->ssm_len || ls->ssm_bf16 != capture->ssm_bf16 ||
      ls->layers != capture->layers)
    return fail(SGK_ERR_SHAPE, "capture linear-attn: capture conv=%lld/ssm=%lld/bf16=%d != state conv=%lld/ssm=%lld/bf16=%d",
                (long long)capture->conv_len, (long long)capture->ssm_len, int(capture->ssm_bf16),
                (long long)ls->conv_len, (long long)ls->ssm_len, int(ls->ssm_bf16));
  SGK_CUDA(launch_copy_bytes(capture->d_base, ls->d_base, ls->total_bytes, ls->st->pick(stream)));
  ls->st->launches += 1;
  return SGK_OK;
}

static int32_t conv_impl(sgk_linstate* ls, void* stream, int32_t layer, const float* d_qkv, const float* d_weight,
                         int32_t conv_dim, int32_t conv_kernel_dim, int32_t n_tokens, float* d_out) {
  if (!ls || !d_qkv || !d_weight || !d_out) return fail(SGK_ERR_BACKEND, "null argument");
  if (layer < 0 || layer >= ls->layers) return fail(SGK_ERR_DIMENSION, "layer %d out of range", layer);
  if (conv_dim <= 0 || conv_kernel_dim <= 0) return fail(SGK_ERR_DIMENSION, "conv shape must be positive");
  if (conv_kernel_dim > 16) return fail(SGK_ERR_CONFIG, "conv kernel %d > 16 is not supported", conv_kernel_dim);
  if (n_tokens < 0) return fail(SGK_ERR_DIMENSION, "n_tokens %d invalid", n_tokens);
  // ensure_conv_cache (src/linear_attention.rs:856-886): the history is [(K-1), conv_dim]
  if (ls->conv_len != int64_t(conv_kernel_dim - 1) * conv_dim)
    return fail(SGK_ERR_DIMENSION, "conv history holds %lld values, expected %lld", (long long)ls->conv_len,
                (long long)(int64_t(conv_kernel_dim - 1) * conv_dim));
  if (n_tokens == 0) return SGK_OK;
  State* st = ls->st;
  cudaStream_t s = st->pick(stream);
  const bool member = st->chain_member(s);
  SGK_CUDA(launch_conv_step(d_qkv, d_weight, static_cast<float*>(sgk_linstate_conv_ptr(ls, layer)), d_out, conv_dim,
                            conv_kernel_dim, n_tokens, member ? 1 : 0, st->chain_follows(s) ? 1 : 0, s));
  st->launches += 1;
  if (member) st->chain_note();
  return SGK_OK;
}

int32_t sgk_linstate_enqueue_decode_step(sgk_linstate* ls, void* stream, int32_t layer, const sgk_linear_shape* shape,
                                         const float* d_qkv, const float* d_conv_weight, int32_t conv_kernel_dim,
                                         const float* d_beta_input, const float* d_gate_input, const float* d_a_log,
                                         const float* d_dt_bias, float* d_out) {
  if (!ls || !shape || !d_qkv || !d_conv_weight || !d_beta_input || !d_gate_input || !d_a_log || !d_dt_bias || !d_out)
    return fail(SGK_ERR_BACKEND, "null argument");
  if (layer < 0 || layer >= ls->layers) return fail(SGK_ERR_DIMENSION, "layer %d out of range", layer);
  const int hk = shape->num_key_heads, hv = shape->num_value_heads;
  // the validation of LinearAttentionConfig (src/linear_attention.rs:113-150)
  if (hk <= 0 || hv <= 0 || shape->key_head_dim <= 0 || shape->value_head_dim <= 0)
    return fail(SGK_ERR_CONFIG, "linear attention: zero dimension");
  if (hv % hk != 0) return fail(SGK_ERR_CONFIG, "value heads %d are not a multiple of key heads %d", hv, hk);
  if (shape->key_head_dim != 128 || shape->value_head_dim != 128)
    return fail(SGK_ERR_CONFIG, "the one-launch decode step takes head dims of 128 (got %d / %d): use the conv and "
                "gated-delta steps", shape->key_head_dim, shape->value_head_dim);
  if (hk > 64) return fail(SGK_ERR_CONFIG, "more than 64 key heads");
  if (conv_kernel_dim < 1 || conv_kernel_dim > 8)
    return fail(SGK_ERR_CONFIG, "conv kernel %d: 1 to 8 taps in the one-launch decode step", conv_kernel_dim);
  const int64_t conv_dim = int64_t(2) * hk * 128 + int64_t(hv) * 128;
  if (ls->conv_len != int64_t(conv_kernel_dim - 1) * conv_dim)
    return fail(SGK_ERR_DIMENSION, "conv history holds %lld values, expected %lld", (long long)ls->conv_len,
                (long long)(int64_t(conv_kernel_dim - 1) * conv_dim));
  if (ls->ssm_len != int64_t(hv) * 128 * 128)
    return fail(SGK_ERR_DIMENSION, "recurrent state holds %lld values, expected %lld", (long long)ls->ssm_len,
                (long long)(int64_t(hv) * 128 * 128));
  State* st = ls->st;
  cudaStream_t s = st->pick(stream);
  const bool member = st->chain_member(s);
  LinearDecodeArgs a{};
  a.ssm = sgk_linstate_ssm_ptr(ls, layer);
  a.history = static_cast<float*>(sgk_linstate_conv_ptr(ls, layer));
  a.qkv = d_qkv;
  a.conv_weight = d_conv_weight;
  a.beta_input = d_beta_input;
  a.gate_input = d_gate_input;
  a.a_log = d_a_log;
  a.dt_bias = d_dt_bias;
  a.out = d_out;
  a.head_counters = ls->d_head_counters;
  a.conv_dim = static_cast<int32_t>(conv_dim);
  a.kernel = conv_kernel_dim;
  a.num_key_heads = hk;
  a.num_value_heads = hv;
  // key_scale (src/linear_attention.rs:1203-1210): d^-1/2 for k, its square for q
  const float inv = std::pow(128.0f, -0.5f);
  a.q_scale = inv * inv;
  a.k_scale = inv;
  a.eps = 1.0e-6f;
  a.ssm_bf16 = ls->ssm_bf16 ? 1 : 0;
  a.pdl_trigger = member ? 1 : 0;
  a.pdl_wait = st->chain_follows(s) ? 1 : 0;
  SGK_CUDA(launch_linear_decode_step(a, s));
  st->launches += 1;
  if (member) st->chain_note();
  return SGK_OK;
}

int32_t sgk_linstate_enqueue_conv_step(sgk_linstate* ls, void* stream, int32_t layer, const float* d_qkv,
                                       const float* d_weight, int32_t conv_dim, int32_t conv_kernel_dim,
                                       float* d_out) {
  return conv_impl(ls, stream, layer, d_qkv, d_weight, conv_dim, conv_kernel_dim, 1, d_out);
}

int32_t sgk_linstate_enqueue_conv_seq(sgk_linstate* ls, void* stream, int32_t layer, const float* d_qkv,
                                      const float* d_weight, int32_t conv_dim, int32_t conv_kernel_dim,
                                      int32_t n_tokens, float* d_out) {
  return conv_impl(ls, stream, layer, d_qkv, d_weight, conv_dim, conv_kernel_dim, n_tokens, d_out);
}

static int32_t gated_delta_impl(sgk_linstate* const* states, int32_t n_states, void* stream, int32_t layer,
                                const sgk_linear_shape* shape, const float* d_q, const float* d_k, const float* d_v,
                                const float* d_g, const float* d_beta, int32_t n_tokens, float* d_out) {
  if (!states || !shape || !d_q || !d_k || !d_v || !d_g || !d_beta || !d_out) return fail(SGK_ERR_BACKEND, "null argument");
  if (n_states <= 0 || n_states > GATED_DELTA_MAX_STATES)
    return fail(SGK_ERR_CONFIG, "n_states %d outside 1..%d", n_states, GATED_DELTA_MAX_STATES);
  if (shape->num_key_heads <= 0 || shape->num_value_heads <= 0 || shape->key_head_dim <= 0 ||
      shape->value_head_dim <= 0 || shape->num_value_heads % shape->num_key_heads != 0)
    return fail(SGK_ERR_DIMENSION, "gated-delta shape invalid");
  if (shape->key_head_dim > 256) return fail(SGK_ERR_CONFIG, "key_head_dim %d > 256 is not supported", shape->key_head_dim);
  // ensure_ssm_cache (src/linear_attention.rs:994-1024): the state is [H_v][d_v][d_k]
  int64_t expect = int64_t(shape->num_value_heads) * shape->value_head_dim * shape->key_head_dim;
  GatedDeltaArgs a{};
  for (int32_t i = 0; i < n_states; ++i) {
    sgk_linstate* ls = states[i];
    if (!ls) return fail(SGK_ERR_BACKEND, "null state %d", i);
    if (layer < 0 || layer >= ls->layers) return fail(SGK_ERR_DIMENSION, "layer %d out of range", layer);
    if (ls->ssm_len != expect)
      return fail(SGK_ERR_DIMENSION, "ssm state holds %lld values, shape wants %lld", (long long)ls->ssm_len,
                  (long long)expect);
    if (ls->st != states[0]->st || ls->ssm_bf16 != states[0]->ssm_bf16)
      return fail(SGK_ERR_CONFIG, "states of one batch must share device and storage type");
    a.ssm[i] = sgk_linstate_ssm_ptr(ls, layer);
  }
  a.n_states = n_states;
  a.n_tokens = n_tokens;
  a.ssm_bf16 = states[0]->ssm_bf16 ? 1 : 0;
  a.num_key_heads = shape->num_key_heads;
  a.num_value_heads = shape->num_value_heads;
  a.key_head_dim = shape->key_head_dim;
  a.value_head_dim = shape->value_head_dim;
  a.q = d_q;
  a.k = d_k;
  a.v = d_v;
  a.g = d_g;
  a.beta = d_beta;
  a.out = d_out;
  State* st = states[0]->st;
  cudaStream_t s = st->pick(stream);
  const bool member = st->chain_member(s);
  a.pdl_trigger = member ? 1 : 0;
  a.pdl_wait = st->chain_follows(s) ? 1 : 0;
  SGK_CUDA(launch_gated_delta_step(a, st->sm_count, s));
  st->launches += 1;
  if (member) st->chain_note();
  return SGK_OK;
}

int32_t sgk_linstate_enqueue_gated_delta_step_batch(sgk_linstate* const* states, int32_t n_states, void* stream,
                                                    int32_t layer, const sgk_linear_shape* shape,
                                                    const float* d_q, const float* d_k, const float* d_v,
                                                    const float* d_g, const float* d_beta, float* d_out) {
  return gated_delta_impl(states, n_states, stream, layer, shape, d_q, d_k, d_v, d_g, d_beta, 1, d_out);
}

int32_t sgk_linstate_enqueue_gated_delta_step(sgk_linstate* ls, void* stream, int32_t layer,
                                              const sgk_linear_shape* shape, const float* d_q, const float* d_k,
                                              const float* d_v, const float* d_g, const float* d_beta,
                                              float* d_out) {
  if (!ls) return fail(SGK_ERR_BACKEND, "null argument");
  return gated_delta_impl(&ls, 1, stream, layer, shape, d_q, d_k, d_v, d_g, d_beta, 1, d_out);
}

int32_t sgk_linstate_enqueue_gated_delta_seq(sgk_linstate* ls, void* stream, int32_t layer,
                                             const sgk_linear_shape* shape, const float* d_q, const float* d_k,
                                             const float* d_v, const float* d_g, const float* d_beta,
                                             int32_t n_tokens, float* d_out) {
  if (!ls) return fail(SGK_ERR_BACKEND, "null argument");
  if (n_tokens < 0) return fail(SGK_ERR_DIMENSION, "n_tokens %d invalid", n_tokens);
  if (n_tokens == 0) return SGK_OK;
  return gated_delta_impl(&ls, 1, stream, layer, shape, d_q, d_k, d_v, d_g, d_beta, n_tokens, d_out);
}

// ------------------------------------------------------------------ hashes
void sgk_hash_root(uint8_t out[32]) { std::memset(out, 0, 32); }

void sgk_hash_for_session(const char* key, size_t key_len, int32_t present, uint8_t out[32]) {
  // src/serve/cache.rs:22-33: None or "" keeps the global root
  if (!present || !key || key_len == 0) {
    std::memset(out, 0, 32);
    return;
  }
  sha256(reinterpret_cast<const uint8_t*>(key), key_len, out);
}

void sgk_hash_chain(const uint8_t prev[32], const uint64_t* tokens, size_t n, uint8_t out[32]) {
  Hash32 p;
  std::memcpy(p.data(), prev, 32);
  Hash32 h = hash_chain(p, tokens, n);
  std::memcpy(out, h.data(), 32);
}

// ------------------------------------------------------------------ prefix cache
int32_t sgk_prefix_create(sgk_pool* pool, int64_t block_tokens, int64_t capacity_blocks, int64_t blocks_per_session,
                          int64_t budget_bytes, sgk_prefix** out) {
  if (!out) return fail(SGK_ERR_BACKEND, "prefix_create: null out pointer");
  if (capacity_blocks < 0 || blocks_per_session < 0 || budget_bytes < 0)
    return fail(SGK_ERR_CONFIG, "prefix cache: negative size");
  auto pc = std::make_unique<sgk_prefix>();
  pc->pool = pool;
  pc->block_tokens = std::max<int64_t>(block_tokens, 1);  // src/serve/cache.rs:111
  if (pool && pc->block_tokens % PAGE_TOKENS != 0)
    return fail(SGK_ERR_CONFIG, "block_tokens %lld must be a multiple of the %d-token page", (long long)pc->block_tokens,
                PAGE_TOKENS);
  pc->capacity = capacity_blocks;
  pc->blocks_per_session = blocks_per_session;
  pc->budget = budget_bytes;
  *out = pc.release();
  return SGK_OK;
}

void sgk_prefix_destroy(sgk_prefix* pc) {
  if (!pc) return;
  Pool* pool = pc->pool;
  if (pool && !pool->host_only()) {
    cudaSetDevice(pool->st->device);
    cudaStreamSynchronize(pool->st->stream);
  }
  delete static_cast<Prefix*>(pc);
  if (pool && !pool->host_only()) pool->flush_scrub(pool->st->stream);
}

int64_t sgk_prefix_block_tokens(const sgk_prefix* pc) { return pc ? pc->block_tokens : 0; }

int32_t sgk_prefix_match(sgk_prefix* pc, const uint8_t root[32], const uint64_t* tokens, size_t n,
                         int64_t* tokens_out, uint8_t hash_out[32], uint64_t* entry_out) {
  if (!pc || !root || !tokens_out || !hash_out || !entry_out) return fail(SGK_ERR_BACKEND, "null argument");
  *entry_out = 0;
  *tokens_out = 0;
  if (n > 0 && !tokens) return SGK_OK;
  Hash32 session, hash{};
  std::memcpy(session.data(), root, 32);
  pc->match(session, tokens, n, tokens_out, &hash, entry_out);
  if (*entry_out) std::memcpy(hash_out, hash.data(), 32);
  return SGK_OK;
}

int32_t sgk_prefix_insert(sgk_prefix* pc, const uint8_t session[32], const uint8_t hash[32], int64_t tokens,
                          sgk_seq* seq, sgk_linstate* ls, void* stream, int32_t* inserted_out) {
  if (!pc || !session || !hash) return fail(SGK_ERR_BACKEND, "null argument");
  Hash32 s, h;
  std::memcpy(s.data(), session, 32);
  std::memcpy(h.data(), hash, 32);
  return pc->insert(s, h, tokens, seq, ls, stream, inserted_out);
}

int32_t sgk_prefix_insert_chain(sgk_prefix* pc, const uint8_t root[32], const uint64_t* tokens, size_t n,
                                int64_t from_tokens, sgk_seq* seq, void* stream, int32_t* inserted_out,
                                uint8_t last_hash_out[32]) {
  if (!pc || !root || (n > 0 && !tokens)) return fail(SGK_ERR_BACKEND, "null argument");
  if (inserted_out) *inserted_out = 0;
  if (from_tokens < 0 || from_tokens % pc->block_tokens != 0)
    return fail(SGK_ERR_DIMENSION, "from_tokens %lld is not on a block boundary", (long long)from_tokens);
  Hash32 session;
  std::memcpy(session.data(), root, 32);
  Hash32 previous = session;
  const size_t bt = static_cast<size_t>(pc->block_tokens);
  // prefill_prompt_state's loop (src/serve/state.rs:596-604): every full block of the prompt is
  // remembered in order, each with its own budget loop; blocks before from_tokens (the matched
  // prefix) only advance the hash chain.
  for (size_t i = 0; i < n / bt; ++i) {
    const Hash32 hash = hash_chain(previous, tokens + i * bt, bt);
    previous = hash;
    const int64_t boundary = static_cast<int64_t>((i + 1) * bt);
    if (boundary <= from_tokens) continue;
    int32_t inserted = 0;
    SGK_TRY(pc->insert(session, hash, boundary, seq, nullptr, stream, &inserted));
    if (inserted_out) *inserted_out += inserted;
  }
  if (last_hash_out) std::memcpy(last_hash_out, previous.data(), 32);
  return SGK_OK;
}

int32_t sgk_prefix_restore(sgk_prefix* pc, uint64_t entry, sgk_seq* seq, sgk_linstate* ls, void* stream, int32_t mode,
                           int64_t* bytes_copied_out) {
  if (!pc || !seq) return fail(SGK_ERR_BACKEND, "null argument");
  if (bytes_copied_out) *bytes_copied_out = 0;
  if (mode != 0 && mode != 1) return fail(SGK_ERR_CONFIG, "restore mode %d", mode);
  auto found = pc->by_id.find(entry);
  if (found == pc->by_id.end()) return fail(SGK_ERR_DIMENSION, "prefix entry %llu is no longer cached", (unsigned long long)entry);
  const PrefixEntry& e = *found->second;
  if (seq->pool != pc->pool) return fail(SGK_ERR_CONFIG, "sequence belongs to another pool");
  if (e.key.tokens > seq->capacity)
    return fail(SGK_ERR_DIMENSION, "restore of %lld rows > capacity %lld", (long long)e.key.tokens, (long long)seq->capacity);
  if (e.ls && !ls) return fail(SGK_ERR_SHAPE, "entry holds a linear-attention state but none was given to restore into");
  Pool* pool = pc->pool;
  std::vector<int32_t> src;
  pc->collect_pages(e.run.get(), &src);
  if (mode == 0) {
    // Nothing is touched unless the copy can be made: the pages the sequence itself gives back
    // (those nobody else holds) count as free.
    size_t own = 0;
    for (int32_t p : seq->pages)
      if (p >= 0 && pool->refcount[p] == 1) own += 1;
    if (src.size() > pool->free_list.size() + own)
      return fail(SGK_ERR_MEMORY_GUARD, "page pool exhausted: need %zu pages, %zu free", src.size(),
                  pool->free_list.size() + own);
  }
  // Everything below is enqueued on the call's stream in order: earlier launches on it still read
  // the old table and pages, later ones the restored ones. When the caller stream used last is
  // another one, the call's stream first waits for what was enqueued there (no host wait).
  // (Launches on further streams that use this sequence must have finished: the stream rule.)
  cudaStream_t cs = nullptr;
  if (!pool->host_only()) {
    State* st = pool->st;
    cs = stream ? static_cast<cudaStream_t>(stream) : st->stream;
    SGK_CUDA(st->order_after_last_caller(cs));
    cs = st->pick(stream);
  }
  seq->release_all();
  if (mode == 1) {
    for (int32_t p : src) pool->retain(p);
    seq->pages = src;
  } else {
    std::vector<int32_t> dst;
    dst.reserve(src.size());
    for (size_t i = 0; i < src.size(); ++i) {
      int32_t p;
      SGK_TRY(pool->alloc_page(&p));
      dst.push_back(p);
    }
    seq->pages = dst;
    if (pool->host_only() || src.empty()) {
      SGK_TRY(seq->set_len_all(e.key.tokens, cs));
    } else {
      // one staging copy and one launch: the copy kernel also installs the block table and the cursors
      CopyInstall install;
      install.table = pool->d_tables + int64_t(seq->slot) * pool->table_stride;
      install.lens = pool->d_lens + int64_t(seq->slot) * pool->layers;
      install.n_lens = pool->layers;
      install.len_value = static_cast<int32_t>(e.key.tokens);
      SGK_TRY(pool->copy_pages(dst, src, cs, &install));
      for (int l = 0; l < pool->layers; ++l) seq->len[l] = e.key.tokens;
    }
    if (bytes_copied_out) *bytes_copied_out = static_cast<int64_t>(src.size()) * pool->page_b;
  }
  if (mode == 1) {
    SGK_TRY(seq->publish(0, static_cast<int64_t>(seq->pages.size()), cs, true));
    SGK_TRY(seq->set_len_all(e.key.tokens, cs));
  }
  if (e.ls) {
    SGK_TRY(sgk_linstate_restore(ls, stream, static_cast<sgk_linstate*>(e.ls.get())));
    if (bytes_copied_out) *bytes_copied_out += e.ls->total_bytes;
  }
  return SGK_OK;
}

int32_t sgk_prefix_evict_lru(sgk_prefix* pc, int32_t* evicted_out, int64_t* bytes_out) {
  if (!pc || !evicted_out) return fail(SGK_ERR_BACKEND, "null argument");
  int64_t bytes = 0;
  *evicted_out = pc->evict_lru(&bytes) ? 1 : 0;
  if (bytes_out) *bytes_out = bytes;
  if (pc->pool && !pc->pool->host_only()) SGK_TRY(pc->pool->flush_scrub(pc->pool->st->stream));
  return SGK_OK;
}

int64_t sgk_prefix_bytes(const sgk_prefix* pc) { return pc ? pc->entry_bytes : 0; }
int64_t sgk_prefix_pinned_bytes(const sgk_prefix* pc) { return pc ? pc->pinned_bytes() : 0; }
int64_t sgk_prefix_len(const sgk_prefix* pc) { return pc ? static_cast<int64_t>(pc->entries.size()) : 0; }
int64_t sgk_prefix_evicted_count(const sgk_prefix* pc) { return pc ? pc->evicted_total : 0; }
int64_t sgk_prefix_session_count(const sgk_prefix* pc, const uint8_t session[32]) {
  if (!pc || !session) return 0;
  Hash32 s;
  std::memcpy(s.data(), session, 32);
  return pc->session_count(s);
}

int64_t sgk_prefix_dump(const sgk_prefix* pc, int32_t which, int64_t cap, uint8_t* sessions, uint8_t* hashes,
                        int64_t* tokens) {
  if (!pc) return 0;
  int64_t total = which == 0 ? static_cast<int64_t>(pc->entries.size()) : static_cast<int64_t>(pc->evicted_log.size());
  auto put = [&](int64_t i, const PrefixKey& k) {
    if (sessions) std::memcpy(sessions + 32 * i, k.session.data(), 32);
    if (hashes) std::memcpy(hashes + 32 * i, k.hash.data(), 32);
    if (tokens) tokens[i] = k.tokens;
  };
  if (which == 0) {
    int64_t i = 0;
    for (auto it = pc->entries.begin(); it != pc->entries.end() && i < cap; ++it, ++i) put(i, it->key);
  } else {
    for (int64_t i = 0; i < std::min(cap, total); ++i) put(i, pc->evicted_log[i]);
  }
  return total;
}

int64_t sgk_longest_prefix_entry_index(const uint64_t* flat, const size_t* lens, size_t n_entries,
                                       const uint64_t* prompt, size_t n) {
  // src/decoder/generation.rs:190-204: strictly longer wins, first among equals
  int64_t best = -1;
  size_t best_len = 0, off = 0;
  for (size_t i = 0; i < n_entries; ++i) {
    size_t len = lens[i];
    if (len > best_len && len <= n && std::equal(flat + off, flat + off + len, prompt)) {
      best = static_cast<int64_t>(i);
      best_len = len;
    }
    off += len;
  }
  return best;
}

// ------------------------------------------------------------------ decoder-internal prefix cache
int32_t sgk_dprefix_create(sgk_pool* pool, int64_t capacity, sgk_dprefix** out) {
  if (!out) return fail(SGK_ERR_BACKEND, "dprefix_create: null out pointer");
  if (capacity < 0) return fail(SGK_ERR_CONFIG, "prefix cache: negative capacity");
  auto dp = std::make_unique<sgk_dprefix>();
  dp->pool = pool;
  dp->capacity = capacity;
  *out = dp.release();
  return SGK_OK;
}

void sgk_dprefix_destroy(sgk_dprefix* dp) {
  if (!dp) return;
  Pool* pool = dp->pool;
  if (pool && !pool->host_only()) {
    cudaSetDevice(pool->st->device);
    cudaStreamSynchronize(pool->st->stream);
  }
  delete static_cast<DecoderPrefix*>(dp);
  if (pool && !pool->host_only()) pool->flush_scrub(pool->st->stream);
}

int64_t sgk_dprefix_len(const sgk_dprefix* dp) { return dp ? static_cast<int64_t>(dp->entries.size()) : 0; }

int64_t sgk_dprefix_entry_tokens(const sgk_dprefix* dp, int64_t index, uint64_t* tokens_out, int64_t cap) {
  if (!dp || index < 0 || index >= static_cast<int64_t>(dp->entries.size())) return -1;
  const auto& t = dp->entries[static_cast<size_t>(index)].tokens;
  if (tokens_out)
    for (int64_t i = 0; i < std::min<int64_t>(cap, static_cast<int64_t>(t.size())); ++i) tokens_out[i] = t[static_cast<size_t>(i)];
  return static_cast<int64_t>(t.size());
}

// prefix_cache_put (src/decoder/generation.rs:3105-3139)
int32_t sgk_dprefix_put(sgk_dprefix* dp, const uint64_t* tokens, size_t n, sgk_seq* seq, sgk_linstate* ls, void* stream) {
  if (!dp || (n > 0 && !tokens)) return fail(SGK_ERR_BACKEND, "null argument");
  if (dp->capacity == 0) return SGK_OK;   // :3110-3113
  if (dp->pool && !seq) return fail(SGK_ERR_BACKEND, "prefix cache put needs the sequence to snapshot");
  DecoderPrefixEntry e;
  e.tokens.assign(tokens, tokens + n);
  if (seq) {
    if (seq->pool != dp->pool) return fail(SGK_ERR_CONFIG, "sequence belongs to another pool");
    for (int64_t l : seq->len)
      if (l < static_cast<int64_t>(n))
        return fail(SGK_ERR_DIMENSION, "snapshot of %zu rows from a sequence holding %lld", n, (long long)l);
    if (seq->released_pages > 0) return fail(SGK_ERR_DIMENSION, "snapshot of a sequence whose head was released");
    const size_t n_pages = (n + PAGE_TOKENS - 1) / PAGE_TOKENS;
    e.pages.assign(seq->pages.begin(), seq->pages.begin() + static_cast<long>(n_pages));
  }
  if (ls) {
    LinState* snap = nullptr;
    SGK_TRY(linstate_snapshot(ls, stream, &snap));
    e.ls.reset(snap);
  }
  for (int32_t p : e.pages) dp->pool->retain(p);
  // an entry with the same tokens is replaced (:3118-3125), the new one goes to the front, the rear is cut (:3137)
  for (size_t i = 0; i < dp->entries.size(); ++i)
    if (dp->entries[i].tokens == e.tokens) {
      dp->drop(i);
      break;
    }
  dp->entries.insert(dp->entries.begin(), std::move(e));
  while (static_cast<int64_t>(dp->entries.size()) > dp->capacity) dp->drop(dp->entries.size() - 1);
  if (dp->pool && !dp->pool->host_only()) SGK_TRY(dp->pool->flush_scrub(dp->pool->st->stream));
  return SGK_OK;
}

// prefix_cache_get (:2998-3024) up to the point where the caller extends the suffix: the longest
// entry that is a prefix of the prompt moves to the front and its rows become the sequence's
// (shared by reference; the entry is never aliased for writing: a shared page is copied before
// it is written). *cached_len_out = 0 on a miss (the sequence is left alone). The caller appends
// the rows of prompt[cached_len..] and, when there were any, calls sgk_dprefix_put with the whole
// prompt, as the reference does (:3019-3022).
int32_t sgk_dprefix_get(sgk_dprefix* dp, const uint64_t* prompt, size_t n, sgk_seq* seq, sgk_linstate* ls, void* stream,
                        int64_t* cached_len_out) {
  if (!dp || !cached_len_out || (n > 0 && !prompt)) return fail(SGK_ERR_BACKEND, "null argument");
  *cached_len_out = 0;
  long best = -1;
  size_t best_len = 0;
  for (size_t i = 0; i < dp->entries.size(); ++i) {   // longest_prefix_entry_index (:190-204)
    const auto& t = dp->entries[i].tokens;
    if (t.size() > best_len && t.size() <= n && std::equal(t.begin(), t.end(), prompt)) {
      best = static_cast<long>(i);
      best_len = t.size();
    }
  }
  if (best < 0) return SGK_OK;
  std::rotate(dp->entries.begin(), dp->entries.begin() + best, dp->entries.begin() + best + 1);
  const DecoderPrefixEntry& e = dp->entries.front();
  if (dp->pool) {
    if (!seq) return fail(SGK_ERR_BACKEND, "prefix cache get needs a sequence to restore into");
    if (seq->pool != dp->pool) return fail(SGK_ERR_CONFIG, "sequence belongs to another pool");
    if (static_cast<int64_t>(best_len) > seq->capacity)
      return fail(SGK_ERR_DIMENSION, "restore of %zu rows > capacity %lld", best_len, (long long)seq->capacity);
    if (e.ls && !ls) return fail(SGK_ERR_SHAPE, "entry holds a linear-attention state but none was given to restore into");
    Pool* pool = dp->pool;
    cudaStream_t cs = pool->host_only() ? nullptr : pool->st->pick(stream);
    std::vector<int32_t> pages = e.pages;          // the entry may not be referenced across release_all
    for (int32_t p : pages) pool->retain(p);
    seq->release_all();
    seq->pages = pages;
    SGK_TRY(seq->publish(0, static_cast<int64_t>(seq->pages.size()), cs, true));
    SGK_TRY(seq->set_len_all(static_cast<int64_t>(best_len), cs));
    if (e.ls) SGK_TRY(sgk_linstate_restore(ls, stream, static_cast<sgk_linstate*>(e.ls.get())));
  }
  *cached_len_out = static_cast<int64_t>(best_len);
  return SGK_OK;
}

// ------------------------------------------------------------------ budget
int32_t sgk_budget_create(uint64_t static_cap, uint64_t total_memory, uint64_t headroom_bytes, uint64_t device_cap,
                          sgk_budget** out) {
  if (!out) return fail(SGK_ERR_BACKEND, "budget_create: null out pointer");
  auto b = std::make_unique<sgk_budget>();
  b->static_cap = static_cap;
  b->total_memory = total_memory;
  b->headroom = headroom_bytes;
  b->device_cap = device_cap;
  *out = b.release();
  return SGK_OK;
}
void sgk_budget_destroy(sgk_budget* b) { delete b; }
void sgk_budget_set_usage(sgk_budget* b, uint64_t current, uint64_t reserved) {
  if (!b) return;
  b->current = current;
  b->reserved = reserved;
}
int32_t sgk_budget_limit(const sgk_budget* b, uint64_t* limit_out) {
  if (!b || !limit_out) return 0;
  return b->limit(limit_out) ? 1 : 0;
}
int32_t sgk_budget_check_allocation(const sgk_budget* b, uint64_t requested, uint64_t* projected_out,
                                    uint64_t* available_out) {
  if (!b) return fail(SGK_ERR_BACKEND, "null budget");
  uint64_t limit = 0;
  if (!b->limit(&limit)) return SGK_OK;  // no limit: everything is accepted
  auto sat = [](uint64_t x, uint64_t y) { return x + y < x ? UINT64_MAX : x + y; };
  uint64_t before = sat(b->current, b->reserved);
  uint64_t projected = sat(before, requested);
  if (projected_out) *projected_out = projected;
  if (available_out) *available_out = limit > before ? limit - before : 0;
  if (projected > limit)
    return fail(SGK_ERR_MEMORY_GUARD, "memory budget: projected %llu > limit %llu", (unsigned long long)projected,
                (unsigned long long)limit);
  return SGK_OK;
}

// ------------------------------------------------------------------ utilities
int32_t sgk_util_fill_normal(sgk_state* st, void* stream, float* d_out, int64_t n, uint64_t seed, uint64_t stream_id,
                             uint64_t index0) {
  if (!st || !d_out) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_CUDA(launch_fill_normal(d_out, n, seed, stream_id, index0, st->pick(stream)));
  st->launches += 1;
  return SGK_OK;
}
int32_t sgk_util_malloc(sgk_state* st, size_t bytes, void** d_out) {
  if (!st || !d_out) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_CUDA(cudaSetDevice(st->device));
  SGK_CUDA(cudaMalloc(d_out, bytes));
  return SGK_OK;
}
int32_t sgk_util_free(sgk_state* st, void* d_ptr) {
  if (!st) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_CUDA(cudaStreamSynchronize(st->stream));
  SGK_CUDA(cudaFree(d_ptr));
  return SGK_OK;
}
int32_t sgk_util_h2d(sgk_state* st, void* d_dst, const void* src, size_t bytes) {
  if (!st || !d_dst || !src) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_CUDA(cudaMemcpyAsync(d_dst, src, bytes, cudaMemcpyHostToDevice, st->stream));
  SGK_CUDA(cudaStreamSynchronize(st->stream));
  return SGK_OK;
}
int32_t sgk_util_d2h(sgk_state* st, void* dst, const void* d_src, size_t bytes) {
  if (!st || !dst || !d_src) return fail(SGK_ERR_BACKEND, "null argument");
  SGK_CUDA(cudaMemcpyAsync(dst, d_src, bytes, cudaMemcpyDeviceToHost, st->stream));
  SGK_CUDA(cudaStreamSynchronize(st->stream));
  return SGK_OK;
}
int32_t sgk_util_copy_blocks(sgk_state* st, void* stream, void* d_dst, const void* d_src, const int32_t* dst_pages,
                             const int32_t* src_pages, int32_t n_pages, int64_t page_bytes) {
  if (!st || !d_dst || !d_src) return fail(SGK_ERR_BACKEND, "null argument");
  if (page_bytes <= 0 || page_bytes % 16 != 0) return fail(SGK_ERR_DIMENSION, "page_bytes must be a positive multiple of 16");
  SGK_CUDA(launch_copy_pages(static_cast<uint8_t*>(d_dst), static_cast<const uint8_t*>(d_src), dst_pages, src_pages,
                             n_pages, page_bytes, 1, 0, st->sm_count, st->pick(stream)));
  st->launches += 1;
  return SGK_OK;
}

}  // extern "C"

namespace sgk {
int linstate_snapshot(LinState* ls, void* stream, LinState** out) {
  sgk_linstate* snap = nullptr;
  int rc = sgk_linstate_snapshot(static_cast<sgk_linstate*>(ls), stream, &snap);
  *out = snap;
  return rc;
}
}  // namespace sgk
