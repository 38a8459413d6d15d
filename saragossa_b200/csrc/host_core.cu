// Host side of the resident KV path: page pool, block tables, per-layer cursors,
// kernel selection and split sizing. The residency rule of the reference's
// scratch pool (two live tensors never share memory; a slot is reused only after
// release, src/decode_resident/arena.rs:130-234) becomes: every batch owns its
// split-K workspace, sized once at creation, and reuse is ordered by the stream.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "host.h"

namespace sgk {

#ifdef SGK_TRACE
unsigned long long* g_trace = nullptr;
int g_trace_timeline = 0;   // > 0: every attention launch gets its own 4096 blocks of the buffer, global-timer stamps
int g_trace_launch = 0;
extern "C" void sgk_debug_set_trace(unsigned long long* p) { g_trace = p; g_trace_launch = 0; }
extern "C" void sgk_debug_set_trace_timeline(int on) { g_trace_timeline = on; g_trace_launch = 0; }
#endif

static thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}
const char* last_error_cstr() { return g_last_error.c_str(); }

// ---------------------------------------------------------------- Pool
PoolView Pool::view() const {
  PoolView v;
  v.base = d_base;
  v.page_bytes = layer_b;
  v.layer_bytes = layer_stride;
  v.tile_bytes = tile_b;
  v.tables = d_tables;
  v.lens = d_lens;
  v.scale_max = d_scale_max;
  v.table_stride = table_stride;
  v.layers = layers;
  v.kv_heads = kv_heads;
  v.head_dim = head_dim;
  v.dtype = dtype;
  return v;
}

int Pool::alloc_page(int32_t* out) {
  if (free_list.empty())
    return fail(SGK_ERR_MEMORY_GUARD, "page pool exhausted: %lld pages all in use", (long long)num_pages);
  int32_t p = free_list.back();
  free_list.pop_back();
  refcount[p] = 1;
  *out = p;
  return SGK_OK;
}

void Pool::release(int32_t page) {
  if (page < 0 || page >= num_pages || refcount[page] <= 0) return;
  refcount[page] -= 1;
  if (refcount[page] == 0) {
    free_list.push_back(page);
    if (scrub_on_free && !host_only()) pending_scrub.push_back(page);
  }
}

int Pool::stage_words(const int32_t* a, size_t na, const int32_t* b, size_t nb, cudaStream_t stream, int* slot_out) {
  const int need = static_cast<int>(na + nb);
  const int idx = stage_next;
  stage_next = (stage_next + 1) % STAGE_SLOTS;
  StageSlot& s = stage[idx];
  if (s.pending) {
    // the slot's previous user: by now long finished unless the host is a whole ring ahead
    SGK_CUDA(cudaEventSynchronize(s.done));
    s.pending = false;
  }
  if (need > s.cap) {
    if (s.h) cudaFreeHost(s.h);
    if (s.d) cudaFree(s.d);
    s.h = nullptr, s.d = nullptr, s.cap = 0;
    const int cap = std::max(need, 4096);
    SGK_CUDA(cudaMallocHost(&s.h, size_t(cap) * sizeof(int32_t)));
    SGK_CUDA(cudaMalloc(&s.d, size_t(cap) * sizeof(int32_t)));
    s.cap = cap;
  }
  if (!s.done) SGK_CUDA(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
  if (na) std::memcpy(s.h, a, na * sizeof(int32_t));
  if (nb) std::memcpy(s.h + na, b, nb * sizeof(int32_t));
  SGK_CUDA(cudaMemcpyAsync(s.d, s.h, size_t(need) * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
  *slot_out = idx;
  return SGK_OK;
}

int Pool::stage_done(int slot, cudaStream_t stream) {
  SGK_CUDA(cudaEventRecord(stage[slot].done, stream));
  stage[slot].pending = true;
  return SGK_OK;
}

void Pool::stage_free() {
  for (StageSlot& s : stage) {
    if (s.pending) cudaEventSynchronize(s.done);
    if (s.done) cudaEventDestroy(s.done);
    if (s.h) cudaFreeHost(s.h);
    if (s.d) cudaFree(s.d);
    s = StageSlot{};
  }
}

int Pool::flush_scrub(cudaStream_t stream) {
  if (pending_scrub.empty() || host_only()) {
    pending_scrub.clear();
    return SGK_OK;
  }
  // A page freed and taken again before the flush must not be wiped.
  std::vector<int32_t> list;
  for (int32_t p : pending_scrub)
    if (refcount[p] == 0) list.push_back(p);
  pending_scrub.clear();
  if (list.empty()) return SGK_OK;
  int slot;
  SGK_TRY(stage_words(list.data(), list.size(), nullptr, 0, stream, &slot));
  SGK_CUDA(launch_scrub_pages(d_base, stage[slot].d, static_cast<int>(list.size()), layer_b, layers, layer_stride,
                              st->sm_count, stream));
  st->launches += 1;
  SGK_TRY(stage_done(slot, stream));
  // a scrubbed page may be handed out and written through another stream right after this call
  SGK_CUDA(cudaStreamSynchronize(stream));
  return SGK_OK;
}

int Pool::copy_pages(const std::vector<int32_t>& dst, const std::vector<int32_t>& src, cudaStream_t stream,
                     const CopyInstall* install) {
  if (dst.size() != src.size()) return fail(SGK_ERR_DIMENSION, "copy_pages: list sizes differ");
  if (dst.empty() || host_only()) return SGK_OK;
  int slot;
  SGK_TRY(stage_words(dst.data(), dst.size(), src.data(), src.size(), stream, &slot));
  SGK_CUDA(launch_copy_pages(d_base, d_base, stage[slot].d, stage[slot].d + dst.size(), static_cast<int>(dst.size()),
                             layer_b, layers, layer_stride, st->sm_count, stream, install));
  st->launches += 1;
  return stage_done(slot, stream);
}

// ---------------------------------------------------------------- Seq
int Seq::publish(int64_t first_page, int64_t n, cudaStream_t stream, bool ordered) {
  if (pool->host_only() || n <= 0) return SGK_OK;
  int32_t* dst = pool->d_tables + int64_t(slot) * pool->table_stride + first_page;
  if (!ordered) {
    SGK_CUDA(cudaMemcpy(dst, pages.data() + first_page, size_t(n) * sizeof(int32_t), cudaMemcpyHostToDevice));
    return SGK_OK;
  }
  int s;
  SGK_TRY(pool->stage_words(pages.data() + first_page, static_cast<size_t>(n), nullptr, 0, stream, &s));
  SGK_CUDA(cudaMemcpyAsync(dst, pool->stage[s].d, size_t(n) * sizeof(int32_t), cudaMemcpyDeviceToDevice, stream));
  return pool->stage_done(s, stream);
}

int Seq::reserve(int64_t tokens) {
  if (tokens > capacity)
    return fail(SGK_ERR_DIMENSION, "reserve %lld > capacity %lld", (long long)tokens, (long long)capacity);
  int64_t need = (tokens + PAGE_TOKENS - 1) / PAGE_TOKENS;
  int64_t have = static_cast<int64_t>(pages.size());
  if (need <= have) return SGK_OK;
  if (need - have > static_cast<int64_t>(pool->free_list.size()))
    return fail(SGK_ERR_MEMORY_GUARD, "page pool exhausted: need %lld pages, %lld free", (long long)(need - have),
                (long long)pool->free_list.size());
  for (int64_t i = have; i < need; ++i) {
    int32_t p;
    SGK_TRY(pool->alloc_page(&p));
    pages.push_back(p);
  }
  return publish(have, need - have);
}

void Seq::new_epoch() {
  static uint64_t counter = 0;
  epoch = ++counter;
}

int Seq::release_before(int64_t row) {
  int64_t upto = std::min<int64_t>(row / PAGE_TOKENS, static_cast<int64_t>(pages.size()));
  for (int64_t i = released_pages; i < upto; ++i) {
    if (pages[i] >= 0) pool->release(pages[i]);
    pages[i] = -1;
  }
  if (upto > released_pages) {
    new_epoch();
    int64_t first = released_pages;
    released_pages = upto;
    SGK_TRY(publish(first, upto - first));
  }
  if (!pool->host_only()) SGK_TRY(pool->flush_scrub(pool->st->stream));
  return SGK_OK;
}

int Seq::release_all() {
  new_epoch();
  for (auto& p : pages)
    if (p >= 0) pool->release(p);
  pages.clear();
  released_pages = 0;
  return SGK_OK;
}

int Seq::ensure_writable(int64_t row, cudaStream_t stream) {
  int64_t idx = row / PAGE_TOKENS;
  if (idx >= static_cast<int64_t>(pages.size())) return SGK_OK;
  int32_t page = pages[idx];
  if (page < 0)
    return fail(SGK_ERR_DIMENSION, "row %lld lies in a page released by the sliding window", (long long)row);
  if (pool->refcount[page] <= 1) return SGK_OK;
  int32_t fresh;
  SGK_TRY(pool->alloc_page(&fresh));
  SGK_TRY(pool->copy_pages({fresh}, {page}, stream));
  pool->release(page);
  pages[idx] = fresh;
  new_epoch();
  if (!pool->host_only()) {
    // in-stream table update: earlier kernels still see the shared page
    SGK_CUDA(launch_set_len(pool->d_tables + int64_t(slot) * pool->table_stride + idx, fresh, stream));
    pool->st->launches += 1;
  }
  return SGK_OK;
}

int Seq::set_len(int layer, int64_t value, cudaStream_t stream) {
  len[layer] = value;
  if (pool->host_only()) return SGK_OK;
  SGK_CUDA(launch_set_len(pool->d_lens + int64_t(slot) * pool->layers + layer, static_cast<int32_t>(value), stream));
  pool->st->launches += 1;
  return SGK_OK;
}

int Seq::set_len_all(int64_t value, cudaStream_t stream) {
  for (int l = 0; l < pool->layers; ++l) len[l] = value;
  if (pool->host_only()) return SGK_OK;
  SGK_CUDA(launch_set_len(pool->d_lens + int64_t(slot) * pool->layers, static_cast<int32_t>(value), stream,
                          pool->layers));
  pool->st->launches += 1;
  return SGK_OK;
}

// ---------------------------------------------------------------- Kv
Kv::~Kv() {
  self_batch.reset();
  if (d_io) cudaFree(d_io);
}

int Kv::ensure_io(size_t bytes) {
  if (bytes <= d_io_bytes) return SGK_OK;
  if (d_io) cudaFree(d_io);
  d_io = nullptr;
  d_io_bytes = 0;
  SGK_CUDA(cudaMalloc(&d_io, bytes));
  d_io_bytes = bytes;
  return SGK_OK;
}

int create_batch(State* st, Kv** kvs, int n, Batch** out);

int Kv::ensure_self_batch() {
  if (self_batch) return SGK_OK;
  Batch* b = nullptr;
  Kv* self = this;
  SGK_TRY(create_batch(st, &self, 1, &b));
  self_batch.reset(b);
  return SGK_OK;
}

// ---------------------------------------------------------------- Batch
Batch::~Batch() {
  if (d_slots) cudaFree(d_slots);
  if (d_counters) cudaFree(d_counters);
  if (d_part_o) cudaFree(d_part_o);
  if (d_part_ml) cudaFree(d_part_ml);
  if (d_part2_o) cudaFree(d_part2_o);
  if (d_part2_ml) cudaFree(d_part2_ml);
  if (d_group_counters) cudaFree(d_group_counters);
}

int create_batch(State* st, Kv** kvs, int n, Batch** out) {
  if (n <= 0 || kvs == nullptr) return fail(SGK_ERR_CONFIG, "batch needs at least one KV state");
  auto b = std::make_unique<Batch>();
  b->st = st;
  b->pool = kvs[0]->pool();
  b->layer = kvs[0]->layer;
  b->q_heads = kvs[0]->q_heads;
  if (b->pool->host_only()) return fail(SGK_ERR_BACKEND, "batch over a bookkeeping-only pool");
  std::vector<int32_t> slots;
  for (int i = 0; i < n; ++i) {
    if (kvs[i]->pool() != b->pool || kvs[i]->layer != b->layer || kvs[i]->q_heads != b->q_heads)
      return fail(SGK_ERR_CONFIG, "batch members must share pool, layer and q_heads");
    b->kvs.push_back(kvs[i]);
    slots.push_back(kvs[i]->seq->slot);
  }
  const int heads = std::max(b->q_heads, b->pool->kv_heads);
  // Splits never need to exceed about two blocks per SM for the whole launch.
  int by_sm = (2 * st->sm_count) / (n * b->pool->kv_heads);
  b->uniform_splits = std::min(144, std::max(1, by_sm));  // two merge levels of at most 12 partials each
  // an uneven batch cuts its long sequences finer than that (the workspace is sized for it)
  b->max_splits = n > 1 ? std::max(b->uniform_splits, 16) : b->uniform_splits;
  SGK_CUDA(cudaMalloc(&b->d_slots, size_t(n) * sizeof(int32_t)));
  SGK_CUDA(cudaMemcpy(b->d_slots, slots.data(), size_t(n) * sizeof(int32_t), cudaMemcpyHostToDevice));
  size_t counters = size_t(n) * heads + 2 * size_t(n);
  SGK_CUDA(cudaMalloc(&b->d_counters, counters * sizeof(int32_t)));
  SGK_CUDA(cudaMemset(b->d_counters, 0, counters * sizeof(int32_t)));
  size_t rows = size_t(n) * b->q_heads * b->max_splits;
  SGK_CUDA(cudaMalloc(&b->d_part_o, rows * b->pool->head_dim * sizeof(float)));
  SGK_CUDA(cudaMalloc(&b->d_part_ml, rows * 2 * sizeof(float)));
  b->max_groups = 12;
  size_t rows2 = size_t(n) * b->q_heads * b->max_groups;
  SGK_CUDA(cudaMalloc(&b->d_part2_o, rows2 * b->pool->head_dim * sizeof(float)));
  SGK_CUDA(cudaMalloc(&b->d_part2_ml, rows2 * 2 * sizeof(float)));
  size_t gc = size_t(n) * b->pool->kv_heads * b->max_groups;
  SGK_CUDA(cudaMalloc(&b->d_group_counters, gc * sizeof(int32_t)));
  SGK_CUDA(cudaMemset(b->d_group_counters, 0, gc * sizeof(int32_t)));
  *out = b.release();
  return SGK_OK;
}

int Batch::choose_kernel() const {
  int gqa = q_heads / pool->kv_heads;
  // 1 = generic CUDA-core kernel, 2 = tensor-core kernel over bf16 pages, 3 = over u8 pages
  int tensor = attention_mma_supported(pool->dtype, pool->head_dim, gqa)  ? 2
               : attention_u8_supported(pool->dtype, pool->head_dim, gqa) ? 3
                                                                          : 0;
  if (kernel_override == 2 && tensor == 0) return -1;
  if (kernel_override == 1) return 1;
  return tensor ? tensor : 1;
}

int Batch::choose_splits(int kernel, int64_t max_rows) const {
  int s = splits_override;
  // tuning flag: a split count for every launch of the process
  static const int env_splits = [] {
    const char* e = std::getenv("SGK_SPLITS");
    return e ? std::atoi(e) : 0;
  }();
  if (s <= 0 && env_splits > 0) s = env_splits;
  if (s <= 0) {
    // Blocks per launch = heads * n * s over `slots` resident blocks (two per SM
    // for the tensor-core kernel, eight for the generic one). Take the split count
    // with the best whole-wave fill (first one above 98.5%), while every split
    // keeps a few pages of work.
    const int heads = kernel >= 2 ? pool->kv_heads : q_heads;
    const int64_t slots = int64_t(st->sm_count) * (kernel >= 2 ? 2 : 8);
    const int64_t units = int64_t(heads) * n();
    const int64_t pages = (max_rows + PAGE_TOKENS - 1) / PAGE_TOKENS;
    const int min_pages = kernel >= 2 ? 8 : 2;
    int64_t cap = std::max<int64_t>(1, pages / min_pages);
    cap = std::min<int64_t>(cap, uniform_splits);
    int best = 1;
    double best_eff = 0.0;
    for (int c = 1; c <= cap; ++c) {
      int64_t blocks = units * c;
      int64_t waves = (blocks + slots - 1) / slots;
      double eff = double(blocks) / double(waves * slots);
      if (eff > best_eff + 1e-9) {
        best_eff = eff;
        best = c;
      }
      if (eff >= 0.985) break;
    }
    s = best;
  }
  return std::max(1, std::min(s, max_splits));
}

int Batch::enqueue_append(cudaStream_t stream, const float* d_k, const float* d_v, int n_rows, const RopeArgs* rope,
                          const float* knorm_w) {
  if (d_k == nullptr || d_v == nullptr) return fail(SGK_ERR_BACKEND, "append: null device pointer");
  for (Kv* kv : kvs) {
    // overflow is an error and nothing is written (src/decode_resident/attention.rs:967-972)
    if (kv->len() + n_rows > kv->seq->capacity)
      return fail(SGK_ERR_DIMENSION, "append KV: capacity %lld reached (overflow)", (long long)kv->seq->capacity);
  }
  for (Kv* kv : kvs) {
    SGK_TRY(kv->seq->reserve(std::min(kv->seq->capacity, kv->len() + n_rows)));
    for (int64_t r = kv->len(); r < kv->len() + n_rows; r += PAGE_TOKENS) SGK_TRY(kv->seq->ensure_writable(r, stream));
    SGK_TRY(kv->seq->ensure_writable(kv->len() + n_rows - 1, stream));
  }
  AppendArgs a{};
  a.pool = pool->view();
  a.layer = layer;
  a.slots = n() == 1 ? nullptr : d_slots;
  a.slot0 = kvs[0]->seq->slot;
  a.k = d_k;
  a.v = d_v;
  a.row0 = 0;
  a.use_device_len = 1;
  a.bump_len = 1;
  a.done_counters = d_counters + size_t(n()) * std::max(q_heads, pool->kv_heads) + n();
  a.status = st->d_status;
  a.num_pages = pool->num_pages;
  a.has_rope = rope != nullptr;
  if (rope) {
    a.rope = *rope;
    a.knorm_w = knorm_w;
  }
  a.out_k = nullptr;
  // gridDim.y is limited: feed long appends in pieces
  int done = 0;
  while (done < n_rows) {
    int piece = std::min(n_rows - done, 32768);
    if (n() > 1 && piece != n_rows) return fail(SGK_ERR_DIMENSION, "batched append of more than 32768 rows");
    a.n_rows = piece;
    a.k = d_k + size_t(done) * kvs[0]->kv_dim();
    a.v = d_v + size_t(done) * kvs[0]->kv_dim();
    a.rope_table = nullptr;
    if (rope != nullptr && piece >= 16) {
      // cos and sin of (row, pair) depend neither on the head nor on the sequence: one small launch
      // makes them for the rows of this piece, every page tile of every head reads them
      int64_t lo = INT64_MAX, hi = 0;
      for (Kv* kv : kvs) lo = std::min(lo, kv->len() + done), hi = std::max(hi, kv->len() + done + piece);
      const size_t pairs = size_t(rope->rope_dims / 2);
      const size_t need = size_t(hi - lo) * pairs;
      if (pairs > 0 && hi - lo <= 65536) {
        if (need > st->rope_table_cap) {
          if (st->d_rope_table) cudaFree(st->d_rope_table);
          st->d_rope_table = nullptr, st->rope_table_cap = 0, st->rope_table_rows = 0;
          const size_t cap = std::max(need, size_t(4096) * 64);
          SGK_CUDA(cudaMalloc(&st->d_rope_table, cap * sizeof(float2)));
          st->rope_table_cap = cap;
        }
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        SGK_CUDA(cudaStreamIsCapturing(stream, &capturing));
        const RopeArgs& have = st->rope_table_args;
        const bool held = capturing == cudaStreamCaptureStatusNone && !st->rope_table_in_graph && st->rope_table_rows > 0 &&
                          st->rope_table_stream == stream && lo >= st->rope_table_lo &&
                          hi <= st->rope_table_lo + st->rope_table_rows && have.rope_dims == rope->rope_dims &&
                          have.frequency_dim == rope->frequency_dim && have.theta == rope->theta &&
                          have.position_scale == rope->position_scale;
        if (!held) {
          SGK_CUDA(launch_rope_table(st->d_rope_table, lo, static_cast<int>(hi - lo), *rope, stream));
          st->launches += 1;
          // a captured launch fills the table when the graph runs, not now: nothing is held then
          st->rope_table_rows = capturing == cudaStreamCaptureStatusNone ? hi - lo : 0;
          st->rope_table_lo = lo;
          st->rope_table_stream = stream;
          st->rope_table_args = *rope;
          if (capturing != cudaStreamCaptureStatusNone) st->rope_table_in_graph = true;
        }
        a.rope_table = st->d_rope_table;
        a.rope_row0 = st->rope_table_lo;
      }
    }
    SGK_CUDA(launch_append_rows(a, n(), stream));
    st->launches += 1;
    done += piece;
  }
  for (Kv* kv : kvs) kv->seq->len[layer] += n_rows;
  return SGK_OK;
}

int Batch::enqueue_attention(cudaStream_t stream, const float* d_q, float* d_out, int64_t window_start,
                             int64_t sliding_window, float attn_scalar, const float* d_k_new,
                             const float* d_v_new) {
  if (d_q == nullptr || d_out == nullptr) return fail(SGK_ERR_BACKEND, "attention: null device pointer");
  const bool fused = d_k_new != nullptr;
  int kernel = choose_kernel();
  if (kernel < 0) return fail(SGK_ERR_BACKEND, "tensor-core attention kernel does not take this shape");
  int64_t max_rows = 0;
  for (Kv* kv : kvs) {
    int64_t len_after = kv->len() + (fused ? 1 : 0);
    if (fused && kv->len() >= kv->seq->capacity)
      return fail(SGK_ERR_DIMENSION, "append KV: capacity %lld reached (overflow)", (long long)kv->seq->capacity);
    if (len_after == 0) return fail(SGK_ERR_DIMENSION, "attention_decode on an empty KV");
    int64_t ws = sliding_window > 0 ? std::max<int64_t>(len_after - sliding_window, 0) : window_start;
    if (ws < 0 || ws >= len_after)
      return fail(SGK_ERR_DIMENSION, "attention_decode empty window: start=%lld, len=%lld", (long long)ws,
                  (long long)len_after);
    if (ws / PAGE_TOKENS < kv->seq->released_pages)
      return fail(SGK_ERR_DIMENSION, "attention window reaches rows released by the sliding window");
    max_rows = std::max(max_rows, len_after - ws);
  }
  if (fused && kernel < 2) {
    SGK_TRY(enqueue_append(stream, d_k_new, d_v_new, 1, nullptr, nullptr));
  } else if (fused) {
    for (Kv* kv : kvs) {
      SGK_TRY(kv->seq->reserve(kv->len() + 1));
      SGK_TRY(kv->seq->ensure_writable(kv->len(), stream));
    }
  }
  AttnArgs a{};
  a.pool = pool->view();
  a.layer = layer;
  a.slots = n() == 1 ? nullptr : d_slots;
  a.slot0 = kvs[0]->seq->slot;
  a.q_heads = q_heads;
  a.q = d_q;
  a.out = d_out;
  a.window_start = window_start;
  a.sliding_window = sliding_window;
  float scalar = attn_scalar > 0.0f ? attn_scalar : static_cast<float>(pool->head_dim);
  a.scale_log2e = 1.4426950408889634f / std::sqrt(scalar);
  const bool chained = st->chain_member(stream) && kernel >= 2;
  a.splits = choose_splits(kernel, max_rows);
  a.pages_per_split = 0;
  if (kernel >= 2 && splits_override <= 0 && n() > 1) {
    // Uneven batch (longest sequence more than a quarter above the shortest): equal split counts
    // would make the launch as long as its longest block. Cut every sequence into pieces of the
    // same size instead, about three waves of blocks in all, and let the scheduler balance them.
    int64_t lo = INT64_MAX, hi = 0, total = 0;
    for (Kv* kv : kvs) {
      int64_t rows = kv->len() + (fused ? 1 : 0);
      if (sliding_window > 0) rows = std::min<int64_t>(rows, sliding_window + PAGE_TOKENS);
      else rows -= std::min<int64_t>(rows, window_start);
      const int64_t pages = (rows + PAGE_TOKENS - 1) / PAGE_TOKENS;
      lo = std::min(lo, pages), hi = std::max(hi, pages), total += pages;
    }
    if (hi * 4 > lo * 5 && hi >= 32) {
      const int64_t slots = int64_t(st->sm_count) * 2;
      int64_t pps = (total * pool->kv_heads + slots * 3 - 1) / (slots * 3);
      pps = std::max<int64_t>(pps, 8);
      const int64_t need = (hi + pps - 1) / pps + 1;   // one spare: lengths grow while a graph is replayed
      a.splits = static_cast<int>(std::min<int64_t>(need, max_splits));
      a.pages_per_split = static_cast<int32_t>(pps);
    }
  }
  a.part.o = d_part_o;
  a.part.ml = d_part_ml;
  a.part2.o = d_part2_o;
  a.part2.ml = d_part2_ml;
  a.group_counters = d_group_counters;
  a.max_groups = max_groups;
  // up to 12 partials are merged in one go; beyond that in groups of about sqrt(splits)
  a.group_size = a.splits;
  if (a.splits > 12) {
    int g = static_cast<int>(std::ceil(std::sqrt(double(a.splits))));
    a.group_size = std::min(g, 12);
  }
  a.n_groups = (a.splits + a.group_size - 1) / a.group_size;
  a.head_counters = d_counters;
  a.seq_counters = d_counters + size_t(n()) * std::max(q_heads, pool->kv_heads);
  a.status = st->d_status;
  a.num_pages = pool->num_pages;
  if (kernel >= 2) {
    a.k_new = d_k_new;
    a.v_new = d_v_new;
    a.n_stages = attention_mma_max_stages(pool->head_dim);
    // tuning flag (stages of the shared-memory ring), in the spirit of the reference's RETI_RUST_* switches
    static const int env_stages = [] {
      const char* e = std::getenv("SGK_ATTN_STAGES");
      return e ? std::atoi(e) : 0;
    }();
    if (kernel == 3) a.n_stages = attention_u8_max_stages(pool->head_dim);
    if (env_stages >= 4 && env_stages <= a.n_stages) a.n_stages = env_stages / 4 * 4;
#ifdef SGK_TRACE
    a.trace = g_trace;
    if (g_trace && g_trace_timeline) {
      a.trace = g_trace + size_t(g_trace_launch++) * 4096 * 16;
      a.trace_gt = 1;
    }
#endif
    // When every block of the launch is resident at once, all blocks of a (sequence, KV head)
    // can merge a slice each after waiting for one another; otherwise (several waves, uneven
    // batches) the last arriver of a group merges, which needs nobody to wait. Blocks that wait
    // for each other make the launch a cooperative one. Used where the other scheme needs two
    // merge levels (more than 12 splits); below that, measured, the last arriver alone is faster.
    static const bool shared_merge_off = std::getenv("SGK_NO_SHARED_MERGE") != nullptr;
    if (!shared_merge_off && a.pages_per_split == 0 && a.splits > 12 && a.splits <= 160) {
      if (resident_per_sm < 0 || resident_stages != a.n_stages)   // asked once per batch
        resident_per_sm = kernel == 3 ? attention_u8_resident_blocks(pool->head_dim, a.n_stages)
                                      : attention_mma_resident_blocks(pool->head_dim, a.n_stages),
        resident_stages = a.n_stages;
      const int per_sm = resident_per_sm;
      const int64_t blocks = int64_t(a.splits) * pool->kv_heads * n();
      // Blocks that wait for each other must all be resident. A cooperative launch guarantees it
      // next to launches of other streams too, and costs about 2 us per launch inside a graph; when
      // the state's streams never run two launches at once (the default: one decode stream, as in
      // the reference), the launches of one stream are placed in order and the check above suffices.
      if (per_sm > 0 && blocks <= int64_t(per_sm) * st->sm_count) a.shared_merge = st->concurrent_streams ? 1 : 2;
    }
    // The launches of one decode token: each lets the next one start while it still runs, and a
    // launch that follows another layer's launch directly starts its block-table walk and its first
    // page copies before that launch has finished (programmatic dependent launch); q, k_new and v_new
    // are read after the wait. C2 at batch 1, 48 layers in one graph: 18.6 -> 15.8 us per layer.
    if (chained) {
      a.pdl_trigger = 1;
      a.pdl_wait = st->chain_follows(stream) ? 1 : 0;
    }
    // Up to 16 splits run as one thread-block cluster and merge through distributed shared memory:
    // no partial goes through L2 and no device-wide atomic sits between the last page and the output.
    // Only when every cluster of the launch is resident at once: a launch that would fit one wave of
    // blocks must not get a second one from the placement of clusters.
    static const bool cluster_merge_off = std::getenv("SGK_NO_CLUSTER_MERGE") != nullptr;
    if (!cluster_merge_off && a.pages_per_split == 0 && a.splits >= 2 && a.splits <= 16) {
      if (cluster_stages != a.n_stages) {
        for (int& c : max_clusters) c = -1;
        cluster_stages = a.n_stages;
      }
      if (max_clusters[a.splits] < 0)
        max_clusters[a.splits] = kernel == 3 ? attention_u8_max_clusters(pool->head_dim, a.n_stages, a.splits)
                                             : attention_mma_max_clusters(pool->head_dim, a.n_stages, a.splits);
      a.cluster_merge = int64_t(pool->kv_heads) * n() <= max_clusters[a.splits];
    }
    // Several GPUs share the sequence: the launch sends its outputs to the peers itself and its last
    // block exchanges flags with them, when every block of the launch reaches its end (even splits)
    // and the merge is not the cluster one (that instance has no peer stores).
    if (peer_target != nullptr && a.pages_per_split == 0) {
      const Exchange* ex = peer_target->ex;
      a.cluster_merge = 0;
      a.n_peers = 0;
      a.rank = ex->rank;
      for (int p = 0; p < ex->n_ranks; ++p) {
        if (p == ex->rank) continue;
        a.peer_out[a.n_peers] = peer_target->peer_out[p];
        a.peer_flags[a.n_peers] = ex->peer_flags[p];
        a.peer_rank[a.n_peers] = p;
        a.n_peers += 1;
      }
      a.local_flags = ex->d_flags;
      a.ex_step = ex->d_flags + ex->n_ranks;
      a.exit_counter = ex->d_flags + ex->n_ranks + 1;
      peer_target_fused = true;
    }
    if (kernel == 3) {
      SGK_CUDA(launch_attention_u8(a, n(), stream));
    } else {
      SGK_CUDA(launch_attention_mma(a, n(), stream));
    }
    if (fused)
      for (Kv* kv : kvs) kv->seq->len[layer] += 1;
  } else {
    SGK_CUDA(launch_attention_generic(a, n(), stream));
  }
  st->launches += 1;
  if (chained) st->chain_note();
  last_kernel = kernel;
  last_splits = a.splits;
  return SGK_OK;
}

// ---------------------------------------------------------------- Step
Step::~Step() {
  for (cudaGraphExec_t e : token_execs)
    if (e) cudaGraphExecDestroy(e);
  if (graph_exec) cudaGraphExecDestroy(graph_exec);
  if (graph) cudaGraphDestroy(graph);
  if (copy_in) cudaStreamDestroy(copy_in);
  if (copy_out) cudaStreamDestroy(copy_out);
  for (cudaEvent_t e : events)
    if (e) cudaEventDestroy(e);
  for (float* p : {d_k, d_v, d_q, d_out})
    if (p) cudaFree(p);
}

int Step::enqueue(cudaStream_t stream, const float* k, const float* v, const float* q, float* out,
                  const int64_t* sliding_windows, float attn_scalar) {
  return enqueue_range(stream, 0, layers.size(), k, v, q, out, sliding_windows, attn_scalar);
}

int Step::enqueue_range(cudaStream_t stream, size_t l0, size_t l1, const float* k, const float* v, const float* q,
                        float* out, const int64_t* sliding_windows, float attn_scalar) {
  // The layers of a step are a token chain of their own (unless the caller has opened one around
  // the step): each launch lets the next one start early. Two launches over the SAME layer in a
  // row (not a decode token) break it: the second reads the cursor the first one moves.
  const bool own_chain = !st->chain_active && layers.size() > 1;
  if (own_chain) {
    st->chain_active = true;
    st->chain_stream = stream;
    st->chain_mark = -1;
  }
  int rc = SGK_OK;
  for (size_t l = l0; l < l1 && rc == SGK_OK; ++l) {
    Batch* b = layers[l];
    size_t kv_stride = size_t(b->n()) * b->kvs[0]->kv_dim();
    size_t q_stride = size_t(b->n()) * b->kvs[0]->q_dim();
    int64_t before = st->launches;
    const Batch* prev = l > l0 ? layers[l - 1] : nullptr;
    if (prev != nullptr && prev->pool == b->pool && prev->layer == b->layer) st->chain_break();
    rc = b->enqueue_attention(stream, q + l * q_stride, out + l * q_stride, 0,
                              sliding_windows ? sliding_windows[l] : 0, attn_scalar, k + l * kv_stride,
                              v + l * kv_stride);
    launches += st->launches - before;
  }
  if (own_chain) st->chain_active = false;
  return rc;
}

// ---------------------------------------------------------------- LinState
cudaError_t State::order_after_last_caller(cudaStream_t cs) {
  cudaStream_t prev = last_caller;
  if (prev == nullptr || prev == cs) return cudaSuccess;
  cudaStreamCaptureStatus a = cudaStreamCaptureStatusNone, b = cudaStreamCaptureStatusNone;
  cudaError_t e = cudaStreamIsCapturing(prev, &a);
  if (e != cudaSuccess) {
    // the caller has destroyed that stream since: its work is done, nothing to order after
    cudaGetLastError();
    last_caller = nullptr;
    return cudaSuccess;
  }
  e = cudaStreamIsCapturing(cs, &b);
  if (e != cudaSuccess) return e;
  if (a != cudaStreamCaptureStatusNone || b != cudaStreamCaptureStatusNone) return cudaSuccess;
  if (order_event == nullptr) {
    e = cudaEventCreateWithFlags(&order_event, cudaEventDisableTiming);
    if (e != cudaSuccess) return e;
  }
  e = cudaEventRecord(order_event, prev);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(cs, order_event, 0);
  return e;
}

LinState::~LinState() {
  if (d_base) cudaFree(d_base);
  if (d_head_counters) cudaFree(d_head_counters);
}

Exchange::~Exchange() {
  for (int p = 0; p < n_ranks; ++p)
    if (p != rank && peer_flags[p]) cudaIpcCloseMemHandle(peer_flags[p]);
  if (d_flags) cudaFree(d_flags);
}

TokenWindow::~TokenWindow() {
  // copies still in flight write into h_ring: wait for them before the memory goes
  for (cudaEvent_t e : done) {
    cudaEventSynchronize(e);
    cudaEventDestroy(e);
  }
  if (d_ring) cudaFree(d_ring);
  if (h_ring) cudaFreeHost(h_ring);
}

}  // namespace sgk
