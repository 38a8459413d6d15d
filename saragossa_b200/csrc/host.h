// Host-side objects behind the C ABI: the resident state, the page pool with its
// free list and reference counts, sequences (block tables), per-layer KV views,
// batches, steps, the linear-attention state container, the prefix cache and the
// memory budget.
#pragma once
#include <cuda_runtime.h>

#include <array>
#include <cstdarg>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <list>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/sgk.h"
#include "kernels.h"

namespace sgk {

int fail(int code, const char* fmt, ...);
const char* last_error_cstr();

#define SGK_CUDA(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess)                                                               \
      return ::sgk::fail(SGK_ERR_BACKEND, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)
#define SGK_TRY(expr)              \
  do {                             \
    int rc_ = (expr);              \
    if (rc_ != SGK_OK) return rc_; \
  } while (0)

struct Exchange;
// Where the next attention launch of a batch also sends its outputs (set by the exchange entry point
// for one enqueue): the peers' counterparts of d_out.
struct PeerTarget {
  Exchange* ex = nullptr;
  float* peer_out[8] = {};   // indexed by rank; the own entry is unused
};

struct Batch;
struct Seq;
struct Pool;

struct State {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  int32_t* d_status = nullptr;
  // {cos, sin} table of a bulk append with rope (grown on demand; reuse is ordered by the stream)
  float2* d_rope_table = nullptr;
  size_t rope_table_cap = 0;
  // what the table holds now: the layers of a prompt append the same rows one after the other on
  // one stream, so the table is made for the first layer and read by the others
  int64_t rope_table_lo = 0, rope_table_rows = 0;
  cudaStream_t rope_table_stream = nullptr;
  RopeArgs rope_table_args{};
  bool rope_table_in_graph = false;   // a captured graph rewrites the table whenever it runs: never held again
  // where the NEXT lm_head launch also writes its indices (mapped host memory); taken and cleared by that launch
  int32_t* lm_index_mirror = nullptr;
  unsigned long long* d_lm_ws = nullptr;  // lm_head argmax: [0..8) best key per row, [8] blocks-done counter; zero between launches
  int64_t launches = 0;  // kernels launched through this state
  // false (default): the caller never has two launches of this state in flight on different
  // streams at once, so launches whose blocks wait for each other go as ordinary launches;
  // true: they go as cooperative launches (sgk_state_set_concurrent_streams)
  bool concurrent_streams = false;
  // Token chain (sgk_state_chain_begin / _end, and every step): the launches of one decode token on
  // one stream. A member launch lets its successor start early; it carries the programmatic
  // stream-serialisation attribute itself when the launch enqueued just before it through this
  // state was a member too (chain_mark == launches: nothing of ours in between, e.g. no
  // copy-on-write). What a member reads before its wait is persistent state of its own layer only.
  bool chain_active = false;
  cudaStream_t chain_stream = nullptr;
  int64_t chain_mark = -1;
  // kill-switch, in the spirit of the reference's RETI_RUST_* flags
  static bool chain_disabled() {
    static const bool off = std::getenv("SGK_NO_CHAIN") != nullptr;
    return off;
  }
  bool chain_member(cudaStream_t s) const { return chain_active && s == chain_stream && !chain_disabled(); }
  bool chain_follows(cudaStream_t s) const { return chain_member(s) && chain_mark == launches; }
  void chain_note() { chain_mark = launches; }   // call right after counting a member's launch
  void chain_break() { chain_mark = -1; }
  // The caller's stream used last (the library's own stream when none was given). A call that frees,
  // shares or replaces pages first orders itself after what was enqueued there.
  mutable cudaStream_t last_caller = nullptr;
  cudaEvent_t order_event = nullptr;
  cudaStream_t pick(void* s) const {
    if (s) last_caller = static_cast<cudaStream_t>(s);
    return s ? static_cast<cudaStream_t>(s) : stream;
  }
  // Makes `cs` wait for everything enqueued so far on the caller stream used last (no host wait).
  // Nothing to do when that is `cs` itself; skipped while either stream is being captured (a capture
  // cannot wait for work outside it, and frees no pages).
  cudaError_t order_after_last_caller(cudaStream_t cs);
};

struct Pool {
  State* st = nullptr;  // NULL: bookkeeping only, no device memory
  int layers = 0, kv_heads = 0, head_dim = 0, dtype = 0;
  int64_t num_pages = 0;
  int max_seqs = 0;
  int64_t max_seq_tokens = 0;
  int table_stride = 0;
  // tile_b: one K or V tile; layer_b: one page of one layer (all heads, K and V); page_b: one page
  // over all layers (what a page costs); layer_stride: distance between layers in the pool
  int64_t tile_b = 0, layer_b = 0, page_b = 0, layer_stride = 0;
  uint8_t* d_base = nullptr;
  int32_t* d_tables = nullptr;
  int32_t* d_lens = nullptr;
  uint32_t* d_scale_max = nullptr;  // u8 pools only
  // Staging of small host arrays (page lists of a copy or scrub, block-table entries of a restore)
  // on their way to the device: a ring of pinned host slots with a device twin each. A slot is
  // filled, copied and consumed in stream order, and its event says when the host may fill it
  // again, so none of these calls waits for the device unless it is a whole ring ahead.
  struct StageSlot {
    int32_t* h = nullptr;
    int32_t* d = nullptr;
    int cap = 0;
    cudaEvent_t done = nullptr;
    bool pending = false;
  };
  static constexpr int STAGE_SLOTS = 8;
  StageSlot stage[STAGE_SLOTS];
  int stage_next = 0;
  // Puts a ++ b into a slot and enqueues its copy to the slot's device twin on `stream`.
  int stage_words(const int32_t* a, size_t na, const int32_t* b, size_t nb, cudaStream_t stream, int* slot_out);
  // To be called once the work that reads the slot (or the copy out of it) is enqueued on `stream`.
  int stage_done(int slot, cudaStream_t stream);
  void stage_free();
  std::vector<int32_t> free_list;  // taken from the back
  std::vector<int32_t> refcount;
  std::vector<int> free_slots;
  std::vector<int32_t> pending_scrub;
  bool scrub_on_free = false;
  int live_seqs = 0;

  PoolView view() const;
  bool host_only() const { return st == nullptr; }
  int alloc_page(int32_t* out);
  void retain(int32_t page) { refcount[page] += 1; }
  void release(int32_t page);
  int flush_scrub(cudaStream_t stream);
  int64_t used_pages() const { return num_pages - static_cast<int64_t>(free_list.size()); }
  // Copies pages src[i] -> dst[i] inside the pool (page lists are host arrays).
  int copy_pages(const std::vector<int32_t>& dst, const std::vector<int32_t>& src, cudaStream_t stream,
                 const CopyInstall* install = nullptr);
};

struct Kv;

struct Seq {
  Pool* pool = nullptr;
  int slot = -1;
  int64_t capacity = 0;
  std::vector<int32_t> pages;  // page id per page index, -1 once released
  int64_t released_pages = 0;  // leading page indices already returned to the pool
  std::vector<int64_t> len;    // per layer, host mirror of the device cursor
  std::vector<std::unique_ptr<Kv>> views;
  // Changes whenever pages of the sequence are released or replaced (never when pages are only
  // added behind them): what the prefix cache remembers of the sequence is valid for one epoch.
  uint64_t epoch = 0;
  void new_epoch();

  int reserve(int64_t tokens);
  int release_before(int64_t row);
  int release_all();
  // Makes the page holding `row` exclusively owned (copy-on-write of a shared page).
  int ensure_writable(int64_t row, cudaStream_t stream);
  int set_len(int layer, int64_t value, cudaStream_t stream);
  int set_len_all(int64_t value, cudaStream_t stream);
  // Block-table entries [first_page, first_page + n) to the device: at once (stream == NULL: entries no
  // enqueued launch reads yet) or in stream order (entries of a live sequence being replaced).
  int publish(int64_t first_page, int64_t n, cudaStream_t stream = nullptr, bool ordered = false);
};

struct Kv {
  State* st = nullptr;
  Seq* seq = nullptr;
  int layer = 0;
  int q_heads = 0;
  // standalone KV owns its pool and sequence
  std::unique_ptr<Pool> owned_pool;
  std::unique_ptr<Seq> owned_seq;
  std::unique_ptr<Batch> self_batch;
  float* d_io = nullptr;  // staging for the host-pointer calls
  size_t d_io_bytes = 0;

  Pool* pool() const { return seq->pool; }
  int64_t len() const { return seq->len[layer]; }
  int kv_dim() const { return pool()->kv_heads * pool()->head_dim; }
  int q_dim() const { return q_heads * pool()->head_dim; }
  int ensure_io(size_t bytes);
  int ensure_self_batch();
  ~Kv();
};

struct Batch {
  State* st = nullptr;
  Pool* pool = nullptr;
  std::vector<Kv*> kvs;
  int layer = 0, q_heads = 0;
  int32_t* d_slots = nullptr;
  int32_t* d_counters = nullptr;  // [n*max(q_heads,kv_heads)] head, [n] seq, [n] append-done
  float* d_part_o = nullptr;
  float* d_part_ml = nullptr;
  float* d_part2_o = nullptr;   // second merge level
  float* d_part2_ml = nullptr;
  int32_t* d_group_counters = nullptr;
  int uniform_splits = 1;
  int resident_per_sm = -1, resident_stages = 0;   // blocks of the attention kernel an SM holds at once
  const PeerTarget* peer_target = nullptr;   // not null: the launch being enqueued sends its outputs to the peers too
  bool peer_target_fused = false;            // set by enqueue_attention when the launch did take the peers
  int max_clusters[17] = {-1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1};   // per split count: clusters of
                                                     // that many blocks the device holds at once (asked once)
  int cluster_stages = 0;
  int max_splits = 1;
  int max_groups = 1;
  int splits_override = 0;
  int kernel_override = 0;
  int last_kernel = 0;
  int last_splits = 0;

  int n() const { return static_cast<int>(kvs.size()); }
  int choose_kernel() const;
  int choose_splits(int kernel, int64_t max_rows) const;
  int enqueue_append(cudaStream_t stream, const float* d_k, const float* d_v, int n_rows, const RopeArgs* rope,
                     const float* knorm_w);
  int enqueue_attention(cudaStream_t stream, const float* d_q, float* d_out, int64_t window_start,
                        int64_t sliding_window, float attn_scalar, const float* d_k_new, const float* d_v_new);
  ~Batch();
};

struct Step {
  State* st = nullptr;
  std::vector<Batch*> layers;
  cudaGraphExec_t graph_exec = nullptr;
  cudaGraph_t graph = nullptr;
  int64_t launches = 0;
  int64_t launches_per_replay = 0;
  // staging of run_host
  float *d_k = nullptr, *d_v = nullptr, *d_q = nullptr, *d_out = nullptr;
  // run_host overlaps the copies of one group of layers with the kernels of another
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  std::vector<cudaEvent_t> events;
  // whole-token graphs (sgk_token_capture): one per slot of the submission window's ring
  std::vector<cudaGraphExec_t> token_execs;
  struct TokenWindow* token_window = nullptr;
  int enqueue(cudaStream_t stream, const float* d_k, const float* d_v, const float* d_q, float* d_out,
              const int64_t* sliding_windows, float attn_scalar);
  int enqueue_range(cudaStream_t stream, size_t l0, size_t l1, const float* d_k, const float* d_v, const float* d_q,
                    float* d_out, const int64_t* sliding_windows, float attn_scalar);
  ~Step();
};

struct LinState {
  State* st = nullptr;
  int layers = 0;
  int64_t conv_len = 0, ssm_len = 0;
  bool ssm_bf16 = false;
  int64_t conv_stride = 0, layer_stride = 0, total_bytes = 0;
  uint8_t* d_base = nullptr;
  int32_t* d_head_counters = nullptr;   // [64] arrivals per key head of the one-launch decode step; zero between launches
  int64_t ssm_elem() const { return ssm_bf16 ? 2 : 4; }
  int64_t estimated_bytes() const { return layers * (conv_len * 4 + ssm_len * ssm_elem()); }
  ~LinState();
};

// The submission window of the resident decode loop (src/decoder/resident/decode.rs:114-173,
// RESIDENT_PIPELINE_WINDOW = 4, src/decoder/resident/types.rs:23): a ring of token indices on the
// device, written by the argmax of token n into slot n % depth and read by the embedding lookup of
// token n+1, so the host can enqueue up to `depth` tokens before it reads the oldest back.
struct TokenWindow {
  State* st = nullptr;
  int depth = 0;
  int64_t enqueued = 0;  // tokens submitted so far
  int inflight = 0;      // submitted and not yet popped
  int32_t* d_ring = nullptr;
  int32_t* h_ring = nullptr;  // pinned mirror, one word per slot (mapped: kernels may write it)
  int32_t* h_ring_dev = nullptr;   // the device's address of h_ring
  std::vector<cudaEvent_t> done;
  ~TokenWindow();
};

// One rank's end of the exchange between the GPUs that share a sequence by KV-head group: its
// flag array and step counter (device memory that the peers map), and the peers' mapped arrays.
struct Exchange {
  State* st = nullptr;
  int rank = 0, n_ranks = 1;
  int32_t* d_flags = nullptr;   // [n_ranks] flags, then the step counter, then the exit counter of fused launches
  int32_t* peer_flags[8] = {};  // mapped from the peers' handles
  ~Exchange();
};

// A fresh state holding a copy of `ls` (snapshot_linear_attn_states); defined beside the ABI.
int linstate_snapshot(LinState* ls, void* stream, LinState** out);

using Hash32 = std::array<uint8_t, 32>;
void sha256(const uint8_t* data, size_t n, uint8_t out[32]);
Hash32 hash_chain(const Hash32& prev, const uint64_t* tokens, size_t n);

// The pages of ONE block of a cached prefix, linked to the run of the block before it. An entry
// of the cache holds the run of its own block; the run keeps its ancestors alive, so an entry pins
// its whole prefix (what the reference's entry does by cloning the whole state,
// src/serve/cache.rs:170-183) while the cache stores every page id once: memory is linear in the
// number of blocks, not quadratic in the prompt length.
struct PageRun {
  std::vector<int32_t> pages;        // this block's pages only
  std::shared_ptr<PageRun> parent;   // the block before it (NULL for the first block)
  int64_t first_page = 0;            // index of pages[0] in the sequence's block table
};

struct PrefixKey {
  Hash32 session, hash;
  int64_t tokens;
  bool operator==(const PrefixKey& o) const { return tokens == o.tokens && hash == o.hash && session == o.session; }
};
struct PrefixKeyHash {
  size_t operator()(const PrefixKey& k) const {
    uint64_t a, b;   // the digests are uniformly distributed already
    std::memcpy(&a, k.hash.data(), 8);
    std::memcpy(&b, k.session.data() + 8, 8);
    return static_cast<size_t>(a ^ (b * 0x9e3779b97f4a7c15ull) ^ (static_cast<uint64_t>(k.tokens) << 1));
  }
};
struct Hash32Hash {
  size_t operator()(const Hash32& h) const {
    uint64_t a;
    std::memcpy(&a, h.data(), 8);
    return static_cast<size_t>(a);
  }
};

struct PrefixEntry;
using PrefixList = std::list<PrefixEntry>;
struct PrefixEntry {
  PrefixKey key;
  uint64_t id = 0;
  std::shared_ptr<PageRun> run;
  std::unique_ptr<LinState> ls;
  int64_t bytes = 0;
  std::list<PrefixList::iterator>::iterator in_session;   // its place in its session's list
};

// BlockAwarePrefixCache (src/serve/cache.rs:74-219) over the page pool. Order and every observable
// effect are the reference's (front = most recently used; a matched chain is touched root to leaf;
// a refresh replaces its duplicate silently; per-session cap, then global cap); the structure is
// not: the reference scans a Vec per block, here a block is found through a hash index and moved
// by relinking a list node, so a match costs O(1) per block whatever the cache holds.
struct Prefix {
  Pool* pool = nullptr;
  int64_t block_tokens = 1, capacity = 0, blocks_per_session = 0, budget = 0;
  PrefixList entries;  // front = most recently used
  std::unordered_map<PrefixKey, PrefixList::iterator, PrefixKeyHash> index;
  std::unordered_map<uint64_t, PrefixList::iterator> by_id;
  // per session: its entries in the same relative order as `entries`
  std::unordered_map<Hash32, std::list<PrefixList::iterator>, Hash32Hash> sessions;
  std::unordered_map<int32_t, std::weak_ptr<PageRun>> run_by_last_page;   // finds the run a new block continues
  std::vector<PrefixKey> evicted_log;   // trace hook: the first EVICTED_LOG_MAX keys that left
  static constexpr size_t EVICTED_LOG_MAX = size_t(1) << 20;
  int64_t evicted_total = 0;
  // The run chain found or made for a sequence last time: the next block of the same sequence
  // continues it instead of searching again.
  struct {
    const Seq* seq = nullptr;
    uint64_t epoch = 0;
    int64_t blocks = 0;
    std::weak_ptr<PageRun> run;
  } cursor;
  int64_t pinned_pages = 0;   // pages of all live runs
  int64_t state_bytes = 0;    // linear-state snapshots held
  int64_t entry_bytes = 0;    // sum of the entries' own byte counts
  uint64_t next_id = 1;

  int64_t pinned_bytes() const;
  int64_t session_count(const Hash32& s) const;
  void touch(PrefixList::iterator it);
  void drop(PrefixList::iterator it, bool log);
  bool evict_lru(int64_t* bytes_out);
  // The run chain of rows [0, tokens) of `seq`: reuses the live runs that hold the same pages and
  // makes the missing ones; *fresh_pages = pages of the runs it would have to make.
  std::shared_ptr<PageRun> chain_for(const Seq* seq, int64_t tokens, bool create, int64_t* fresh_pages);
  void release_run(std::shared_ptr<PageRun>& run);
  void collect_pages(const PageRun* run, std::vector<int32_t>* out) const;
  // match_prefix / insert with the budget loop of remember_prefix_block (src/serve/state.rs:613-639)
  void match(const Hash32& session, const uint64_t* tokens, size_t n, int64_t* tokens_out, Hash32* hash_out,
             uint64_t* entry_out);
  int insert(const Hash32& session, const Hash32& hash, int64_t tokens, Seq* seq, LinState* ls, void* stream,
             int32_t* inserted_out);
  ~Prefix();
};

// The decoder-internal prefix cache (src/decoder/generation.rs:2998-3139): whole prompts, most
// recent first, capacity RETI_RUST_PREFIX_CACHE_CAP (4 by default). An entry holds the pages of
// its prompt by reference (a partly filled last page is shared too: whoever appends to it next
// copies it first) and, when the model has recurrent layers, a snapshot of their state.
struct DecoderPrefixEntry {
  std::vector<uint64_t> tokens;
  std::vector<int32_t> pages;
  std::unique_ptr<LinState> ls;
};
struct DecoderPrefix {
  Pool* pool = nullptr;
  int64_t capacity = 4;
  std::vector<DecoderPrefixEntry> entries;   // front = most recently used
  void drop(size_t index);
  ~DecoderPrefix();
};

struct Budget {
  uint64_t static_cap = 0, total_memory = 0, headroom = 0, device_cap = 0;
  uint64_t current = 0, reserved = 0;
  bool limit(uint64_t* out) const;
};

}  // namespace sgk
