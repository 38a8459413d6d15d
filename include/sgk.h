/*
 * sgk.h — C ABI of the B200-native KV-cache hot path (libsgk.so).
 *
 * This is the drop-in boundary for the reference engine's resident KV cache,
 * decode attention and warm-prefix cache. Every entry point names the
 * reference interface (file:line inside the reference crate) it replaces.
 *
 * Conventions (mirroring the reference's Result<_, InferError> surface,
 * src/error.rs:12-75):
 *   - every fallible call returns an int32 status, 0 = SGK_OK; results come
 *     back through out-pointers; nothing throws or aborts across the boundary;
 *   - sgk_last_error() returns the thread-local message of the last failure;
 *   - `stream` arguments are a cudaStream_t passed as void* (NULL = the
 *     state's own stream); "enqueue" calls only enqueue work and move the
 *     host-side length cursor at enqueue time, like the reference's encode_*
 *     methods (src/decode_resident/attention.rs:950-1038); host-pointer calls
 *     are synchronous;
 *   - one stream per pool: the calls that use a pool's sequences (append, attention, restore,
 *     release, destroy) are ordered by the stream they are enqueued on. The library remembers the
 *     caller stream used last: sgk_prefix_restore makes its own stream wait for what was enqueued
 *     there, sgk_seq_release_before and sgk_seq_destroy wait for it on the host before pages go
 *     back to the pool. A caller that spreads the calls over MORE streams orders them itself
 *     (events) before a call that frees, shares or replaces pages of a sequence (the three above,
 *     sgk_kv_truncate followed by appends): the library does not track further streams. A stream
 *     given to the library stays alive until another one has been given or the state is destroyed;
 *   - pointers named d_* are device pointers, everything else is host memory;
 *   - there is no CPU fallback: without a CUDA device sgk_state_create fails.
 */
#ifndef SGK_H_
#define SGK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: the reference's InferError variants (src/error.rs:12-75). */
enum {
  SGK_OK = 0,
  SGK_ERR_DIMENSION = 1,    /* InferError::Dimension: shape mismatch, overflow at capacity, empty KV/window */
  SGK_ERR_CONFIG = 2,       /* InferError::Config: zero dimension, invalid GQA */
  SGK_ERR_BACKEND = 3,      /* InferError::Metal: wrong element type, null pointer, CUDA failure */
  SGK_ERR_MEMORY_GUARD = 4, /* InferError::MemoryGuard: budget exceeded / pool out of pages */
  SGK_ERR_SHAPE = 5,        /* InferError::Shape: linear-state restore mismatch */
  SGK_ERR_TIMEOUT = 6       /* a bounded device-side wait expired (status word set by a kernel) */
};

/* KV storage types: GpuElement::{F32,Bf16} (src/decode_resident/arena.rs:26-41)
 * plus the u8 group-32 affine format (32 codes + bf16 scale + bf16 bias). */
enum { SGK_KV_F32 = 0, SGK_KV_BF16 = 1, SGK_KV_U8G32 = 2 };

/* Tokens per page. The page is the unit of allocation, sharing and copy. */
#define SGK_PAGE_TOKENS 16

typedef struct sgk_state sgk_state;       /* DecodeResidentState (src/decode_resident/arena.rs:247-349) */
typedef struct sgk_pool sgk_pool;         /* block allocator: pages of all layers of one model shape */
typedef struct sgk_seq sgk_seq;           /* one sequence: block table shared by its layers */
typedef struct sgk_kv sgk_kv;             /* FullAttentionMetalState: one layer of one sequence */
typedef struct sgk_batch sgk_batch;       /* sequences decoded together in one launch (one layer) */
typedef struct sgk_step sgk_step;         /* all layers of a batch: one decode token = one submission */
typedef struct sgk_linstate sgk_linstate; /* LinearAttentionMetalState of all recurrent layers */
typedef struct sgk_prefix sgk_prefix;     /* BlockAwarePrefixCache (src/serve/cache.rs:74-219) */
typedef struct sgk_budget sgk_budget;     /* MemoryGuard (src/memory_guard.rs:155-185,331-370) */

const char* sgk_last_error(void);
const char* sgk_version(void);

/* ---- state: DecodeResidentState::new (src/decode_resident/arena.rs:247-349) ---- */
int32_t sgk_state_create(int32_t device, sgk_state** out);
void sgk_state_destroy(sgk_state* state);
void* sgk_state_stream(sgk_state* state);
int32_t sgk_state_sync(sgk_state* state);
/* Reads and clears the device status word kernels set when a bounded wait expires. */
int32_t sgk_state_device_status(sgk_state* state, int32_t* status_out);

/* Streams. By default the caller promises what the reference does anyway (one decode thread, one
 * command queue per device, src/decode_resident/arena.rs:247-349): launches enqueued through one
 * state never run on two streams at the same time. Launches whose blocks wait for one another (the
 * shared merge of a long single sequence) then go as ordinary launches, placed in stream order,
 * and the launches of one decode token may overlap their neighbours (sgk_step_*). A caller that
 * does run two streams of one state at once says so here (enabled = 1): such launches then become
 * cooperative launches, which the driver places all at once or not at all, at about 2 us more per
 * launch. Set before the first enqueue; a captured step keeps the mode it was captured in. */
int32_t sgk_state_set_concurrent_streams(sgk_state* state, int32_t enabled);
/* Kernels launched so far through this state (a graph replay counts the launches it holds). */
int64_t sgk_state_launches(const sgk_state* state);

/* Token chain: the launches of ONE decode token, enqueued one after the other on one stream
 * (the reference encodes them into one command buffer, src/decoder/resident/decode.rs:243-253).
 * Between _begin and _end every enqueue of this state on `stream` lets the launch after it start
 * early, and a launch that directly follows another member (nothing else of this library in
 * between) starts before its predecessor has finished: it reads the persistent state of its own
 * layer (cursor, block table, pages, recurrent state, conv history and taps) at once and waits for
 * the predecessor before it reads its per-token inputs (q, k, v, g, beta, qkv) or writes anything.
 * The caller's part of the contract: inside a chain, no launch on the stream (the caller's own
 * kernels between two members included) writes persistent state that the NEXT member reads, i.e.
 * consecutive members work on different layers, and truncate / restore / reserve calls stay
 * outside the chain. sgk_step_* open a chain of their own around their layers. A chain may be
 * captured into a CUDA graph; the dependencies are kept as programmatic edges. */
int32_t sgk_state_chain_begin(sgk_state* state, void* stream);
int32_t sgk_state_chain_end(sgk_state* state);

/* Failure-detection self test: launches a kernel whose only wait (on an mbarrier nobody
 * completes) must expire. Returns SGK_ERR_TIMEOUT when the bounded wait reported through the
 * status word as designed; the device and the state stay usable. */
int32_t sgk_state_selftest_wait_timeout(sgk_state* state);

/* ---- page pool (new design: the reference KV is contiguous, not paged) ---- */
int32_t sgk_pool_create(sgk_state* state, int32_t layers, int32_t kv_heads, int32_t head_dim,
                        int32_t dtype, int32_t page_tokens, int64_t num_pages, int32_t max_seqs,
                        int64_t max_seq_tokens, sgk_pool** out);
void sgk_pool_destroy(sgk_pool* pool);
int64_t sgk_pool_num_pages(const sgk_pool* pool);
int64_t sgk_pool_free_pages(const sgk_pool* pool);
int64_t sgk_pool_page_bytes(const sgk_pool* pool); /* one page, all layers, K and V */
int64_t sgk_pool_used_bytes(const sgk_pool* pool);
/* Fisher-Yates shuffle of the free list (seeded): later reservations get a
 * non-contiguous block table. */
int32_t sgk_pool_shuffle_free_list(sgk_pool* pool, uint64_t seed);
int32_t sgk_pool_page_refcount(const sgk_pool* pool, int64_t page, int32_t* out);
/* Zero-fills pages when they return to the free list (eviction scrub kernel). */
int32_t sgk_pool_set_scrub_on_free(sgk_pool* pool, int32_t enabled);

/* ---- sequence: a block table over the pool, shared by the layers ---- */
int32_t sgk_seq_create(sgk_pool* pool, int64_t capacity_tokens, sgk_seq** out);
void sgk_seq_destroy(sgk_seq* seq);
/* Makes rows [0, tokens) addressable: takes pages from the pool and publishes
 * the block-table entries to the device (synchronous). */
int32_t sgk_seq_reserve(sgk_seq* seq, int64_t tokens);
int32_t sgk_seq_block_table(const sgk_seq* seq, int32_t* pages_out, int64_t cap, int64_t* n_out);
/* Empties the sequence for its next use (a decode lane that serves one conversation turn after
 * another keeps its slot, its KV views, its batches and its captured step): every page goes back
 * to the pool and the cursors of all layers return to 0, in stream order. */
int32_t sgk_seq_reset(sgk_seq* seq, void* stream);
/* Sliding-window layers: returns pages that lie wholly before `row` to the pool. */
int32_t sgk_seq_release_before(sgk_seq* seq, int64_t row);
/* FullAttentionMetalState view of (sequence, layer). Owned by the sequence. */
int32_t sgk_seq_layer(sgk_seq* seq, int32_t layer, int32_t q_heads, sgk_kv** out);

/* ---- KV state: state.full_attention(capacity,q,kv,hd,sampled)
 *      (src/decode_resident/attention.rs:26-108). Standalone: owns a private
 *      one-layer pool of ceil(capacity/16) pages. ---- */
int32_t sgk_kv_create(sgk_state* state, int64_t capacity, int32_t q_heads, int32_t kv_heads,
                      int32_t head_dim, int32_t dtype, int32_t page_tokens, sgk_kv** out);
/* Same, with the pool's free list shuffled first (non-contiguous block table). */
int32_t sgk_kv_create_shuffled(sgk_state* state, int64_t capacity, int32_t q_heads, int32_t kv_heads,
                               int32_t head_dim, int32_t dtype, uint64_t seed, sgk_kv** out);
void sgk_kv_destroy(sgk_kv* kv);
/* kv.{len,capacity,kv_dim,q_heads,kv_heads,head_dim} (attention.rs:486-548) */
int64_t sgk_kv_len(const sgk_kv* kv);
int64_t sgk_kv_capacity(const sgk_kv* kv);
int32_t sgk_kv_kv_dim(const sgk_kv* kv);
int32_t sgk_kv_q_heads(const sgk_kv* kv);
int32_t sgk_kv_kv_heads(const sgk_kv* kv);
int32_t sgk_kv_head_dim(const sgk_kv* kv);
int32_t sgk_kv_dtype(const sgk_kv* kv);
int64_t sgk_kv_byte_len(const sgk_kv* kv); /* capacity * kv_dim * storage bytes, K or V */
/* kv.truncate(len) (attention.rs:501-510): moves the cursor only. */
int32_t sgk_kv_truncate(sgk_kv* kv, int64_t len);
/* kv.seed(keys_rows, values_rows, n_rows) (attention.rs:550-602) */
int32_t sgk_kv_seed_f32(sgk_kv* kv, const float* k, size_t k_len, const float* v, size_t v_len,
                        int64_t n_rows);
/* kv.append_row(key, value) (attention.rs:611-644) */
int32_t sgk_kv_append_row_f32(sgk_kv* kv, const float* k, size_t k_len, const float* v, size_t v_len);
/* LayerKvCache::append_batch (src/decoder/attention_cache.rs:38-70): n rows at the cursor. */
int32_t sgk_kv_append_rows_f32(sgk_kv* kv, const float* k, size_t k_len, const float* v, size_t v_len,
                               int64_t n_rows);
/* kv.encode_append_kv_with_offsets(enc,k,koff,v,voff) (attention.rs:950-1001):
 * device-side append of one f32 row; len += 1 at enqueue time. */
int32_t sgk_kv_enqueue_append(sgk_kv* kv, void* stream, const float* d_k, const float* d_v);
/* Device-side append of n rows (the prefill-side producer that replaces
 * append_batch + seed, src/decoder/generation.rs:3338-3361). */
int32_t sgk_kv_enqueue_append_rows(sgk_kv* kv, void* stream, const float* d_k, const float* d_v,
                                   int64_t n_rows);
/* Fused encode_rms_norm_rope_decode on K (attention.rs:297-385) + append:
 * d_k_raw is the un-normalised K projection; V is appended as is. The rotation
 * position is the row being written times position_scale. */
typedef struct {
  int32_t rope_dims;     /* rotated leading dims of each head (even, <= head_dim) */
  int32_t frequency_dim; /* exponent denominator (RopeParams::frequency_dim) */
  float theta;
  float position_scale;
  float eps;
  int32_t interleaved;   /* 0 = rotate-half pairs (i, i+rope_dims/2), 1 = pairs (2i, 2i+1) */
} sgk_rope;
int32_t sgk_kv_enqueue_rope_append(sgk_kv* kv, void* stream, const float* d_k_raw, const float* d_v,
                                   const float* d_knorm_weight, const sgk_rope* rope);
/* The prefill-side producer: n_rows raw K rows [n_rows][kv_dim] are normalised, rotated at
 * positions len .. len+n_rows-1, rounded to the storage type and written straight into the pages,
 * V beside them, in ONE launch. Replaces rms_norm_rope_heads_at over the prompt
 * (src/decoder/attention_ops.rs:682-777) + append_batch + the read-back and re-upload of seed
 * (src/decoder/generation.rs:3338-3361, src/decode_resident/attention.rs:550-602). */
int32_t sgk_kv_enqueue_rope_append_rows(sgk_kv* kv, void* stream, const float* d_k_raw, const float* d_v,
                                        int64_t n_rows, const float* d_knorm_weight, const sgk_rope* rope);
/* The single-sequence form of sgk_batch_enqueue_verify_rows (n_seq = 1). */
int32_t sgk_kv_enqueue_verify_rows(sgk_kv* kv, void* stream, const float* d_k, const float* d_v, const float* d_q,
                                   float* d_out, int32_t n_rows, int64_t sliding_window, float attn_scalar);
/* DecodeResidentState::rms_norm_rope_decode (attention.rs:386-444): host in/out. */
int32_t sgk_rms_norm_rope_decode(sgk_state* state, const float* x, const float* weight,
                                 int32_t heads, int32_t head_dim, const sgk_rope* rope,
                                 int64_t position, float* out);
/* kv.attention_decode_windowed(q, window_start) (attention.rs:661-720): host q/out.
 * attn_scalar <= 0 means head_dim (scale = 1/sqrt(attn_scalar),
 * src/decoder/attention_ops.rs:912). */
int32_t sgk_kv_attention_decode(sgk_kv* kv, const float* q, size_t q_len, int64_t window_start,
                                float attn_scalar, float* out);
/* kv.encode_attention_decode_windowed(enc,q,scores,out,ws) (attention.rs:736-835) */
int32_t sgk_kv_enqueue_attention(sgk_kv* kv, void* stream, const float* d_q, float* d_out,
                                 int64_t window_start, float attn_scalar);
/* NO COUNTERPART IN THE REFERENCE. Same computation and same errors as
 * sgk_kv_enqueue_attention, for callers that cannot allocate device memory (a host
 * that owns the whole device through its own arena, a latency-critical loop that
 * must not take cudaMalloc's implicit synchronisation, code running under stream
 * capture). It never calls cudaMalloc/cudaFree: the split-K workspace is one static
 * device array of SGK_NOALLOC_SCRATCH_BYTES that every GPU loading the library
 * holds until exit. Limits: q_heads*head_dim <= SGK_NOALLOC_MAX_Q_DIM (larger shapes
 * get SGK_ERR_CONFIG); the split count is reduced to fit the array. The first call
 * on a device resolves the array's device address (cudaGetSymbolAddress): make it
 * before any stream capture. All calls share the array: calls whose kernels may
 * overlap on the GPU race and must be ordered by the caller. */
#define SGK_NOALLOC_SCRATCH_BYTES (4u << 20)
#define SGK_NOALLOC_MAX_Q_DIM 16384
int32_t sgk_kv_enqueue_attention_noalloc(sgk_kv* kv, void* stream, const float* d_q, float* d_out,
                                         int64_t window_start, float attn_scalar);
/* encode_append_kv + encode_attention_decode_windowed in ONE launch
 * (the per-layer pair at src/decode_resident/layers.rs:259-288). */
int32_t sgk_kv_enqueue_append_attention(sgk_kv* kv, void* stream, const float* d_k, const float* d_v,
                                        const float* d_q, float* d_out, int64_t sliding_window,
                                        float attn_scalar);
/* kv.keys()/values() read-back used by the reference's tests (tests.rs:380-478):
 * the paged GATHER. Rows [row0,row0+n) as contiguous [n, kv_dim] in the storage
 * type (f32: float, bf16: uint16 bit patterns). For u8 use the _u8 form. */
int32_t sgk_kv_gather_rows(sgk_kv* kv, int64_t row0, int64_t n, void* k_out, void* v_out);
int32_t sgk_kv_gather_rows_u8(sgk_kv* kv, int64_t row0, int64_t n, uint8_t* k_codes, uint16_t* k_scale,
                              uint16_t* k_bias, uint8_t* v_codes, uint16_t* v_scale, uint16_t* v_bias);
/* Same rows decoded to f32 (bf16 upcast, u8 q*scale+bias, src/quantization.rs:173-179). */
int32_t sgk_kv_gather_rows_f32(sgk_kv* kv, int64_t row0, int64_t n, float* k_out, float* v_out);
int32_t sgk_kv_block_table(const sgk_kv* kv, int32_t* pages_out, int64_t cap, int64_t* n_out);
/* Forces one attention kernel: 0 = automatic, 1 = generic CUDA-core kernel,
 * 2 = tensor-core paged kernel (errors if the shape does not qualify). */
int32_t sgk_kv_set_attention_kernel(sgk_kv* kv, int32_t which);

/* ---- batch: n sequences of ONE layer decoded in one launch. The reference's
 *      multi-stream mode loops the solo path per stream
 *      (src/decode_resident/duo.rs:97-199); results are per sequence identical
 *      to decoding each alone. ---- */
int32_t sgk_batch_create(sgk_state* state, sgk_kv** kvs, int32_t n, sgk_batch** out);
void sgk_batch_destroy(sgk_batch* batch);
/* d_k/d_v: [n, kv_dim] f32; d_q/d_out: [n, q_heads*head_dim] f32.
 * sliding_window 0 = none, else window_start = len.saturating_sub(window)
 * (src/decoder/attention_ops.rs:915-918), evaluated after the append. */
int32_t sgk_batch_enqueue_append(sgk_batch* batch, void* stream, const float* d_k, const float* d_v);
int32_t sgk_batch_enqueue_attention(sgk_batch* batch, void* stream, const float* d_q, float* d_out,
                                    int64_t sliding_window, float attn_scalar);
int32_t sgk_batch_enqueue_step(sgk_batch* batch, void* stream, const float* d_k, const float* d_v,
                               const float* d_q, float* d_out, int64_t sliding_window,
                               float attn_scalar);
/* Tuning hooks read by the benchmark: 0 = automatic. */
/* Speculative-decoding verify (src/decode_resident/layers.rs:1295-1433; CPU twin
 * cached_attention_prefill_rows, src/decoder/attention_ops.rs:976-1017): n_rows draft rows
 * go through append + attention one after the other, so the attention of row r sees exactly the
 * rows 0 .. len+r, like n_rows single decode steps. Inputs are row-major over the rows:
 * d_k, d_v [n_rows][n_seq][kv_dim], d_q and d_out [n_rows][n_seq][q_dim]. Capacity is checked for
 * all rows first: an overflow is an error and writes nothing. The rejected tail is dropped with
 * sgk_kv_truncate (src/decoder/generation.rs:1019-1022). */
int32_t sgk_batch_enqueue_verify_rows(sgk_batch* batch, void* stream, const float* d_k, const float* d_v,
                                      const float* d_q, float* d_out, int32_t n_rows, int64_t sliding_window,
                                      float attn_scalar);
int32_t sgk_batch_set_splits(sgk_batch* batch, int32_t splits);
int32_t sgk_batch_get_splits(const sgk_batch* batch, int32_t* splits_out);
int32_t sgk_batch_set_kernel(sgk_batch* batch, int32_t which);
int32_t sgk_batch_last_kernel(const sgk_batch* batch, int32_t* which_out);

/* ---- step: every layer of a batch; one decode token = one stream submission
 *      (src/decoder/resident/decode.rs:183-458: one command buffer per token). ---- */
int32_t sgk_step_create(sgk_state* state, sgk_batch** layers, int32_t n_layers, sgk_step** out);
void sgk_step_destroy(sgk_step* step);
/* d_k/d_v: [layers, n, kv_dim]; d_q/d_out: [layers, n, q_dim]; sliding_windows:
 * one entry per layer (NULL = none). */
int32_t sgk_step_enqueue(sgk_step* step, void* stream, const float* d_k, const float* d_v,
                         const float* d_q, float* d_out, const int64_t* sliding_windows,
                         float attn_scalar);
/* Captures one sgk_step_enqueue into a CUDA graph; each replay is one submission
 * and advances every layer's cursor by one on the device and on the host. */
int32_t sgk_step_capture(sgk_step* step, const float* d_k, const float* d_v, const float* d_q,
                         float* d_out, const int64_t* sliding_windows, float attn_scalar);
int32_t sgk_step_replay(sgk_step* step, void* stream);
/* Same step with HOST buffers: copies inputs in, runs, copies outputs back, waits. */
int32_t sgk_step_run_host(sgk_step* step, const float* k, const float* v, const float* q, float* out,
                          const int64_t* sliding_windows, float attn_scalar);
int64_t sgk_step_launches(const sgk_step* step); /* kernels launched so far by this step */

/* ---- linear-attention recurrent state: LinearAttentionMetalState
 *      (src/metal_backend/mod.rs:507-531) for all recurrent layers of a sequence;
 *      snapshot_linear_attn_states / restore_linear_attn_states
 *      (src/metal_backend/linear_attention.rs:3027-3067,3163-3198). ---- */
int32_t sgk_linstate_create(sgk_state* state, int32_t layers, int64_t conv_len, int64_t ssm_len,
                            int32_t ssm_bf16, sgk_linstate** out);
void sgk_linstate_destroy(sgk_linstate* ls);
int64_t sgk_linstate_bytes(const sgk_linstate* ls); /* estimated_bytes, mod.rs:521-530 */
int32_t sgk_linstate_write(sgk_linstate* ls, int32_t layer, const float* conv, const float* ssm);
int32_t sgk_linstate_read(sgk_linstate* ls, int32_t layer, float* conv, float* ssm);
int32_t sgk_linstate_snapshot(sgk_linstate* ls, void* stream, sgk_linstate** snapshot_out);
int32_t sgk_linstate_restore(sgk_linstate* ls, void* stream, const sgk_linstate* snapshot);
/* Greedy token epilogue, resident on the device: for each of n_rows (1..8) activation rows x
 * [n_rows][hidden] (f32), the index of the largest of W . x over a dense biasless [vocab][hidden]
 * weight (weight_dtype SGK_KV_F32 or SGK_KV_BF16), without writing the logits; the rows of a
 * speculative verify share ONE pass over the weight (argmax_linear_biasless_rows_buffers,
 * src/metal_backend/lm_head.rs:766-820, re-reads it per row). Replaces encode_lm_head_argmax / argmax_linear_biasless for dense weights
 * (src/metal_backend/lm_head.rs:150-195,288-337; kernels argmax_blocks_f32 / argmax_finalize_f32,
 * src/kernels.metal:8362-8440). Ties go to the LOWEST index (src/sampling.rs:49-62). Products are
 * accumulated in f32; against bf16 weights x enters the tensor cores as the sum of two bf16 values
 * (16 mantissa bits), and a row's logit is the same bit for bit whichever rows share the call.
 * d_index_out [n_rows] receives index + index_offset (a vocabulary shard adds its first row);
 * d_value_out [n_rows] (may be NULL) the winning logits. hidden: a multiple of 8; the rows must fit
 * 200 KiB of shared memory (4 bytes per value; f32 weights pad the rows to 1, 2, 4 or 8); weight
 * and x 16-byte aligned. Enqueue only; calls on one state must be stream-ordered (they share a
 * 16-byte workspace). Quantised weights are not handled here. */
int32_t sgk_lm_head_enqueue_argmax(sgk_state* state, void* stream, const void* d_weight, int32_t weight_dtype,
                                   int64_t vocab, int32_t hidden, const float* d_x, int32_t n_rows,
                                   int32_t index_offset, int32_t* d_index_out, float* d_value_out);
/* Affine-quantised weight in the layout the reference loads (src/quantization.rs:173-238; MLX's):
 * codes of `bits` (4 or 8) packed LSB-first into 32-bit words, row-major [rows][cols * bits / 32];
 * one bf16 scale and one bf16 bias per (row, group of `group_size` columns), [rows][cols /
 * group_size] each; value = code * scale + bias. */
typedef struct {
  const uint32_t* d_packed;
  const uint16_t* d_scales;
  const uint16_t* d_biases;
  int32_t bits;
  int32_t group_size;
} sgk_affine_weight;
/* sgk_lm_head_enqueue_argmax over an affine-quantised weight (encode_affine_argmax_qmv_fast,
 * src/metal_backend/lm_head.rs:934-990; kernel affine_argmax_qmv_fast_u4_gs64_f32): bits 4 or 8,
 * group_size 64 or 128, hidden a multiple of the group size, 1-8 activation rows. The codes go
 * through the tensor cores as exact fp16 values, scale and bias are applied per group in f32. */
int32_t sgk_lm_head_enqueue_argmax_affine(sgk_state* state, void* stream, const sgk_affine_weight* weight,
                                          int64_t vocab, int32_t hidden, const float* d_x, int32_t n_rows,
                                          int32_t index_offset, int32_t* d_index_out, float* d_value_out);
/* sgk_embed_enqueue_from_index over an affine-quantised table: the row is dequantised
 * (code * scale + bias, rounded like the CPU path: one multiply, one add) and scaled. */
int32_t sgk_embed_enqueue_from_index_affine(sgk_state* state, void* stream, const sgk_affine_weight* table,
                                            int64_t vocab, int32_t hidden, const int32_t* d_index,
                                            float embedding_scale, int32_t recast_bf16, float* d_out);
/* Token feed: the input row of the next token, looked up by an index that lives on the device
 * (encode_embedding_from_index_buffers_scaled, src/metal_backend/matmul_encode.rs:424-557; kernel
 * embed_gather_dense_from_u32_f32, src/kernels.metal:308-325): d_out[hidden] = table[*d_index] *
 * embedding_scale, then rounded to bf16 and widened again when recast_bf16 is set. Dense table
 * [vocab][hidden], SGK_KV_F32 or SGK_KV_BF16. Like the reference kernel, an index outside the table
 * writes nothing. Enqueue only. */
int32_t sgk_embed_enqueue_from_index(sgk_state* state, void* stream, const void* d_table, int32_t table_dtype,
                                     int64_t vocab, int32_t hidden, const int32_t* d_index, float embedding_scale,
                                     int32_t recast_bf16, float* d_out);

/* Several GPUs sharing ONE long sequence by KV-head group (one process per GPU): every rank computes
 * the attention output of its own heads and needs the whole row [q_heads * head_dim]. The reference
 * runs on one device and has no counterpart; on one GPU this is `out` of sgk_kv_enqueue_attention.
 * Device memory is made visible between the processes with the runtime's IPC handles (64 bytes,
 * carried by whatever channel the host already has):
 *   sgk_peer_export   handle of a device allocation of this process (its base address)
 *   sgk_peer_open     maps a peer's allocation; the pointer is valid in kernels of this process
 *   sgk_peer_close    unmaps it
 * sgk_exchange_*: rank r of n (2..8). create returns the handle of this rank's flag array; connect
 * takes every peer's. enqueue (ONE small kernel, enqueue only): stores this rank's slice
 * [slice_offset, slice_offset + slice_floats) of d_local_row into the same place of every peer's
 * row d_peer_rows[p] (entry `rank` ignored), raises this rank's flag at every peer and waits, with
 * a bound, for every peer's flag: when the kernel has run, d_local_row is complete. A wait that runs
 * out sets the device status (SGK_ERR_TIMEOUT through sgk_state_check_device) and the kernel
 * returns. Every rank enqueues the same sequence of exchanges. A peer can be one exchange ahead:
 * alternate between two rows, or keep a row per layer. Graph capture is allowed (the step number
 * lives on the device). */
typedef struct sgk_exchange sgk_exchange;
/* sgk_batch_enqueue_step_exchange: sgk_batch_enqueue_step whose output goes to d_local_row +
 * slice_offset AND, from the same launch, to the same place of every peer's row: the fused
 * append + attention kernel stores every final output cell to the peers as well, and the block
 * that leaves the launch last raises the flags and waits (bounded) for the peers': compute and
 * exchange are ONE kernel. Where the launch cannot do it (generic kernel, uneven batch) the call
 * enqueues the attention launch and then sgk_exchange_enqueue: same result, two launches. */
int32_t sgk_batch_enqueue_step_exchange(sgk_batch* batch, void* stream, const float* d_k, const float* d_v,
                                        const float* d_q, sgk_exchange* ex, float* d_local_row,
                                        float* const* d_peer_rows, int64_t slice_offset, int64_t sliding_window,
                                        float attn_scalar);
int32_t sgk_peer_export(sgk_state* state, void* d_ptr, uint8_t handle_out[64]);
int32_t sgk_peer_open(sgk_state* state, const uint8_t handle[64], void** d_ptr_out);
int32_t sgk_peer_close(sgk_state* state, void* d_ptr);
int32_t sgk_exchange_create(sgk_state* state, int32_t rank, int32_t n_ranks, sgk_exchange** out,
                            uint8_t flags_handle_out[64]);
void sgk_exchange_destroy(sgk_exchange* ex);
int32_t sgk_exchange_connect(sgk_exchange* ex, int32_t peer_rank, const uint8_t peer_flags_handle[64]);
int32_t sgk_exchange_enqueue(sgk_exchange* ex, void* stream, float* d_local_row, float* const* d_peer_rows,
                             int64_t slice_offset, int32_t slice_floats);

/* The submission window of the resident decode loop (src/decoder/resident/decode.rs:114-173;
 * RESIDENT_PIPELINE_WINDOW = 4, src/decoder/resident/types.rs:23): a ring of `depth` token indices
 * on the device. Token n's epilogue writes its index into output_slot() (slot n % depth), token
 * n+1's embedding lookup reads previous_slot(); the host enqueues up to `depth` tokens before it
 * reads the oldest back.
 *   output_slot    device word the next token's argmax must write; NULL while the window is full
 *   submit         call after the token's work has been enqueued on `stream`: copies the slot to
 *                  pinned host memory behind that work and marks it; Dimension error when full
 *   previous_slot  device word the last submitted token wrote; NULL before the first submit
 *   pop            waits for the OLDEST token in flight and returns its index; Dimension error
 *                  when nothing is in flight
 *   drain          waits for everything in flight and forgets it (the stop-token exit, :167-169)
 * All tokens of one window go to one stream. */
typedef struct sgk_token_window sgk_token_window;
int32_t sgk_token_window_create(sgk_state* state, int32_t depth, sgk_token_window** out);
void sgk_token_window_destroy(sgk_token_window* w);
int32_t* sgk_token_window_output_slot(sgk_token_window* w);
const int32_t* sgk_token_window_previous_slot(sgk_token_window* w);
int32_t sgk_token_window_submit(sgk_token_window* w, void* stream);
int32_t sgk_token_window_pop(sgk_token_window* w, int32_t* token_out);
int32_t sgk_token_window_inflight(const sgk_token_window* w);
int64_t sgk_token_window_enqueued(const sgk_token_window* w);
int32_t sgk_token_window_depth(const sgk_token_window* w);
int32_t sgk_token_window_drain(sgk_token_window* w);

/* The WHOLE token as one submission (one command buffer per token in the reference,
 * src/decoder/resident/decode.rs:183-458: embedding lookup by the previous token's index ->
 * every layer's fused append + attention -> greedy epilogue -> `commit_nonblocking`, :417).
 * sgk_token_capture records, for every slot of the window's ring, ONE CUDA graph:
 *   sgk_embed_enqueue_from_index (index of the previous slot -> io.d_x)
 *   the step's layers (as sgk_step_capture: d_k, d_v, d_q in, d_out out, cursors on the device)
 *   sgk_lm_head_enqueue_argmax (io.d_final -> this slot; the kernel writes the index into the slot's
 *   pinned host mirror as well, so no copy node follows the token's last launch)
 * as one token chain (every launch lets the next one start early). What lies between these
 * pieces in a model (projections, MLP) is the caller's and belongs in the same capture when it
 * exists; here the pointers are fixed device buffers. sgk_token_seed puts the first input token
 * into the ring; sgk_token_submit launches the next token's graph (Dimension error when the
 * window is full) and sgk_token_window_pop returns the oldest token's index. */
typedef struct {
  const void* d_table;      /* embedding table [vocab][hidden], dense (NULL when table_affine is given) */
  int32_t table_dtype;      /* SGK_KV_F32 or SGK_KV_BF16 */
  int64_t vocab;
  int32_t hidden;
  float embedding_scale;
  int32_t recast_bf16;
  float* d_x;               /* the looked-up row */
  const void* d_lm_weight;  /* lm_head weight [vocab][hidden] (may be the table: tied) */
  int32_t lm_weight_dtype;
  const float* d_final;     /* the final hidden row the epilogue reads */
  const sgk_affine_weight* table_affine;  /* not NULL: the table is affine-quantised (d_table ignored) */
  const sgk_affine_weight* lm_affine;     /* not NULL: the lm_head weight is (d_lm_weight ignored) */
} sgk_token_io;
int32_t sgk_token_capture(sgk_step* step, sgk_token_window* window, const sgk_token_io* io, const float* d_k,
                          const float* d_v, const float* d_q, float* d_out, const int64_t* sliding_windows,
                          float attn_scalar);
int32_t sgk_token_seed(sgk_step* step, int32_t first_token, void* stream);
int32_t sgk_token_submit(sgk_step* step, void* stream);

/* encode_capture_linear_attn_state (src/metal_backend/linear_attention.rs:93-127): copies the
 * state into an EXISTING state of the same shape (one made ahead with sgk_linstate_create, like the
 * reference's leased per-row captures, :44-91): enqueue only, no allocation. Shape error if the
 * lengths or the SSM storage type differ. sgk_linstate_restore copies a capture back. */
int32_t sgk_linstate_enqueue_capture(sgk_linstate* ls, void* stream, sgk_linstate* capture);
void* sgk_linstate_conv_ptr(sgk_linstate* ls, int32_t layer);
/* One decode token on a layer's state, in stream order (the "next" step of the path:
 * the state this library snapshots is also advanced here).
 * depthwise_causal_conv for one token (src/linear_attention.rs:802-852): d_qkv, d_out
 * [conv_dim]; d_weight [conv_dim][conv_kernel_dim]; the history [(K-1), conv_dim] slides. */
int32_t sgk_linstate_enqueue_conv_step(sgk_linstate* ls, void* stream, int32_t layer, const float* d_qkv,
                                       const float* d_weight, int32_t conv_dim, int32_t conv_kernel_dim,
                                       float* d_out);
/* gated_delta for one token (src/linear_attention.rs:896-991): S <- g*S; kv = S.k;
 * delta = (v - kv)*beta; S <- S + delta*k^T; y = S.q, value head h reading the q/k of key
 * head h / (H_v / H_k). d_q, d_k [H_k*d_k]; d_v, d_out [H_v*d_v]; d_g, d_beta [H_v]. */
typedef struct {
  int32_t num_key_heads, num_value_heads, key_head_dim, value_head_dim;
} sgk_linear_shape;
int32_t sgk_linstate_enqueue_gated_delta_step(sgk_linstate* ls, void* stream, int32_t layer,
                                              const sgk_linear_shape* shape, const float* d_q, const float* d_k,
                                              const float* d_v, const float* d_g, const float* d_beta,
                                              float* d_out);
/* The prompt-side forms: n_tokens tokens of ONE sequence run one after the other with the state
 * (or the conv window) kept in registers and written back once, like the reference's sequence
 * kernels (linear_attn_gated_delta_seq_dk128_*_tg4_f32, src/kernels.metal:2644-2840). Inputs and
 * outputs gain a leading [n_tokens] dimension. With bf16 SSM storage the state is rounded once, at
 * the end (the step form rounds after every token). */
int32_t sgk_linstate_enqueue_conv_seq(sgk_linstate* ls, void* stream, int32_t layer, const float* d_qkv,
                                      const float* d_weight, int32_t conv_dim, int32_t conv_kernel_dim,
                                      int32_t n_tokens, float* d_out);
int32_t sgk_linstate_enqueue_gated_delta_seq(sgk_linstate* ls, void* stream, int32_t layer,
                                             const sgk_linear_shape* shape, const float* d_q, const float* d_k,
                                             const float* d_v, const float* d_g, const float* d_beta,
                                             int32_t n_tokens, float* d_out);
/* The same step for n_states sequences (at most 64) in one launch, as the reference's batch
 * decode does for its sequences (src/metal_backend/lightbatch_duo.rs): states[i] is sequence
 * i's state and every input and the output gain a leading [n_states] dimension. All states
 * must have the same length and storage type. */
int32_t sgk_linstate_enqueue_gated_delta_step_batch(sgk_linstate* const* states, int32_t n_states, void* stream,
                                                    int32_t layer, const sgk_linear_shape* shape,
                                                    const float* d_q, const float* d_k, const float* d_v,
                                                    const float* d_g, const float* d_beta, float* d_out);
/* The whole decode step of a recurrent layer between its projections, ONE launch: the reference's
 * resident decode issues conv + SiLU + unit RMS norm of q and k + gates as one dispatch and the
 * gated-delta update as the next (linear_attn_conv_norm_gates_k4_dk128_f32 and
 * linear_attn_gated_delta_dk128_tg4_f32, src/kernels.metal:2295-2416,2569-2643); CPU order of
 * operations src/linear_attention.rs:313-342:
 *   c = silu(depthwise_causal_conv(qkv))                     (the history slides by one token)
 *   q = rms_norm_heads_unit(c[0 : key_dim], eps 1e-6) * d_k^-1;  k = ...(c[key_dim : 2 key_dim]) * d_k^-1/2
 *   v = c[2 key_dim :];  beta = sigmoid(beta_input);  g = exp(-exp(a_log) * softplus(gate_input + dt_bias))
 *   out = gated_delta(q, k, v, g, beta) on the layer's state
 * d_qkv [2 H_k d_k + H_v d_v]; d_conv_weight [conv_dim][conv_kernel_dim]; d_beta_input, d_gate_input,
 * d_a_log, d_dt_bias [H_v]; d_out [H_v d_v]. Head dims of 128 and 1 to 8 taps (Config error otherwise:
 * the two steps below take every shape). Within 1e-5 of the CPU order (f32 state), the reference's own
 * bound for its fused dispatches; the conv part is bit-exact. */
int32_t sgk_linstate_enqueue_decode_step(sgk_linstate* ls, void* stream, int32_t layer, const sgk_linear_shape* shape,
                                         const float* d_qkv, const float* d_conv_weight, int32_t conv_kernel_dim,
                                         const float* d_beta_input, const float* d_gate_input, const float* d_a_log,
                                         const float* d_dt_bias, float* d_out);
void* sgk_linstate_ssm_ptr(sgk_linstate* ls, int32_t layer);

/* ---- block hashes: BlockHash::{root,for_session,chain} (src/serve/cache.rs:11-47) ---- */
void sgk_hash_root(uint8_t out[32]);
void sgk_hash_for_session(const char* key, size_t key_len, int32_t present, uint8_t out[32]);
void sgk_hash_chain(const uint8_t prev[32], const uint64_t* tokens, size_t n, uint8_t out[32]);

/* ---- warm-prefix cache: BlockAwarePrefixCache (src/serve/cache.rs:74-219) with
 *      the budget loop of remember_prefix_block (src/serve/state.rs:613-639).
 *      Entries sit at block boundaries and pin the pages of their prefix; pages
 *      are shared between entries by reference count, so an entry costs one
 *      block. pool may be NULL: pure bookkeeping (no device), used to check
 *      match / insert / eviction order. ---- */
int32_t sgk_prefix_create(sgk_pool* pool, int64_t block_tokens, int64_t capacity_blocks,
                          int64_t blocks_per_session, int64_t budget_bytes, sgk_prefix** out);
void sgk_prefix_destroy(sgk_prefix* pc);
int64_t sgk_prefix_block_tokens(const sgk_prefix* pc);
/* match_prefix (cache.rs:121-151): walks full blocks from the root, moves each hit
 * to the front, returns the deepest. *entry_out = 0 when nothing matched. */
int32_t sgk_prefix_match(sgk_prefix* pc, const uint8_t root[32], const uint64_t* tokens, size_t n,
                         int64_t* tokens_out, uint8_t hash_out[32], uint64_t* entry_out);
/* remember_prefix_block + insert (state.rs:613-639, cache.rs:154-193): snapshots
 * the first `tokens` rows of `seq` (and `ls` when not NULL) at a block boundary.
 * Evicts LRU blocks while the budget would be exceeded; if the cache runs empty
 * first the insert is skipped (*inserted_out = 0). seq may be NULL only when the
 * cache was created without a pool. */
int32_t sgk_prefix_insert(sgk_prefix* pc, const uint8_t session[32], const uint8_t hash[32],
                          int64_t tokens, sgk_seq* seq, sgk_linstate* ls, void* stream,
                          int32_t* inserted_out);
/* prefill_prompt_state's loop over the full blocks of a prompt (src/serve/state.rs:596-604) in
 * one call: for every full block of tokens[0..n) that ends after from_tokens (the matched prefix;
 * a block boundary, 0 for none) the hash chain is advanced and the block is remembered as
 * sgk_prefix_insert does, each with its own budget loop; `seq` must hold the prompt's rows.
 * *inserted_out = blocks inserted; last_hash_out (may be NULL) = hash of the last full block.
 * A turn of a conversation costs one call instead of one per 16-token block. */
int32_t sgk_prefix_insert_chain(sgk_prefix* pc, const uint8_t root[32], const uint64_t* tokens, size_t n,
                                int64_t from_tokens, sgk_seq* seq, void* stream, int32_t* inserted_out,
                                uint8_t last_hash_out[32]);
/* copy_prompt_state_metal_snapshot + restore_prompt_state_metal
 * (src/decoder/generation.rs:2851-2892): makes `seq` hold the entry's rows.
 * mode 0 = physical copy into pages owned by the sequence (the reference's
 * never-aliased rule), 1 = share the pages by reference (copy-on-write).
 * Enqueue-only: the page copy, the new block table and the new cursors follow each other on
 * `stream`; launches enqueued on it before the call still see the old sequence. When the pool
 * cannot hold the copy (mode 0) the call fails with SGK_ERR_MEMORY_GUARD and the sequence is
 * left exactly as it was. */
int32_t sgk_prefix_restore(sgk_prefix* pc, uint64_t entry, sgk_seq* seq, sgk_linstate* ls,
                           void* stream, int32_t mode, int64_t* bytes_copied_out);
/* evict_lru_block (cache.rs:196-198): *evicted_out = 0 when the cache is empty. */
int32_t sgk_prefix_evict_lru(sgk_prefix* pc, int32_t* evicted_out, int64_t* bytes_out);
int64_t sgk_prefix_bytes(const sgk_prefix* pc); /* estimated_bytes (cache.rs:200-203) */
/* What the budget is compared with: distinct pages pinned by the cache x page bytes + state snapshots. */
int64_t sgk_prefix_pinned_bytes(const sgk_prefix* pc);
int64_t sgk_prefix_len(const sgk_prefix* pc);
/* Entries that left the cache so far (the dump below keeps the first 2^20 keys of them). */
int64_t sgk_prefix_evicted_count(const sgk_prefix* pc);
int64_t sgk_prefix_session_count(const sgk_prefix* pc, const uint8_t session[32]);
/* Trace hook: which = 0 live entries front-to-rear, 1 = every entry that left, in order. */
int64_t sgk_prefix_dump(const sgk_prefix* pc, int32_t which, int64_t cap, uint8_t* sessions,
                        uint8_t* hashes, int64_t* tokens);
/* The decoder-internal prefix cache (src/decoder/generation.rs:2998-3139; capacity
 * RETI_RUST_PREFIX_CACHE_CAP, 4 by default, src/runtime_flags.rs:670-678): whole prompts, most
 * recent first.
 *   get  prefix_cache_get (:2998-3024) up to the suffix: the longest entry that is a prefix of the
 *        prompt moves to the front, its rows become `seq`'s (pages shared by reference, copied
 *        before anybody writes to them; the recurrent state, if the entry has one, is copied into
 *        `ls`) and *cached_len_out = its length; 0 on a miss, the sequence untouched. The caller
 *        appends the rows of prompt[cached_len..] and then puts the whole prompt (:3019-3022).
 *   put  prefix_cache_put (:3105-3139): an entry with the same tokens is replaced, the new one
 *        goes to the front, entries beyond the capacity fall off the rear; capacity 0 stores nothing.
 * pool may be NULL (bookkeeping only; seq and ls NULL then). */
typedef struct sgk_dprefix sgk_dprefix;
int32_t sgk_dprefix_create(sgk_pool* pool, int64_t capacity, sgk_dprefix** out);
void sgk_dprefix_destroy(sgk_dprefix* dp);
int32_t sgk_dprefix_get(sgk_dprefix* dp, const uint64_t* prompt, size_t n, sgk_seq* seq, sgk_linstate* ls,
                        void* stream, int64_t* cached_len_out);
int32_t sgk_dprefix_put(sgk_dprefix* dp, const uint64_t* tokens, size_t n, sgk_seq* seq, sgk_linstate* ls,
                        void* stream);
int64_t sgk_dprefix_len(const sgk_dprefix* dp);
/* Trace hook: the tokens of entry `index` (front = 0); returns their number, -1 past the end. */
int64_t sgk_dprefix_entry_tokens(const sgk_dprefix* dp, int64_t index, uint64_t* tokens_out, int64_t cap);
/* Decoder-internal longest-prefix selection (src/decoder/generation.rs:190-204). */
int64_t sgk_longest_prefix_entry_index(const uint64_t* flat_tokens, const size_t* lens,
                                       size_t n_entries, const uint64_t* prompt, size_t n);

/* ---- memory budget: MemoryGuard::{check_allocation,projection_over_limit}
 *      (src/memory_guard.rs:331-370) over device bytes. A cap of 0 is "absent". ---- */
int32_t sgk_budget_create(uint64_t static_cap, uint64_t total_memory, uint64_t headroom_bytes,
                          uint64_t device_cap, sgk_budget** out);
void sgk_budget_destroy(sgk_budget* b);
void sgk_budget_set_usage(sgk_budget* b, uint64_t current, uint64_t reserved);
int32_t sgk_budget_limit(const sgk_budget* b, uint64_t* limit_out); /* 1 when a limit exists */
/* SGK_OK when accepted, SGK_ERR_MEMORY_GUARD when projected > limit. */
int32_t sgk_budget_check_allocation(const sgk_budget* b, uint64_t requested, uint64_t* projected_out,
                                    uint64_t* available_out);

/* ---- TEST AND BENCHMARK SUPPORT: not part of the drop-in boundary --------------------------
 * No interface of the reference stands behind the functions below: they feed the parity tests
 * and the benchmark (seeded inputs made on the device, raw device buffers for callers without a
 * CUDA runtime of their own, the block copier on raw ranges). A binding of the crate leaves them
 * out by defining SGK_NO_TEST_SUPPORT before including this header. ---- */
#ifndef SGK_NO_TEST_SUPPORT
/* Device fill with the counter-based approximate-normal generator (integer only,
 * bit-identical to the host restatement used for parity inputs). */
int32_t sgk_util_fill_normal(sgk_state* state, void* stream, float* d_out, int64_t n, uint64_t seed,
                             uint64_t stream_id, uint64_t index0);
int32_t sgk_util_malloc(sgk_state* state, size_t bytes, void** d_out);
int32_t sgk_util_free(sgk_state* state, void* d_ptr);
int32_t sgk_util_h2d(sgk_state* state, void* d_dst, const void* src, size_t bytes);
int32_t sgk_util_d2h(sgk_state* state, void* dst, const void* d_src, size_t bytes);
/* Block copy kernel on raw device ranges (the prefix-restore data mover). */
int32_t sgk_util_copy_blocks(sgk_state* state, void* stream, void* d_dst, const void* d_src,
                             const int32_t* dst_pages, const int32_t* src_pages, int32_t n_pages,
                             int64_t page_bytes);
#endif /* SGK_NO_TEST_SUPPORT */

#ifdef __cplusplus
}
#endif
#endif /* SGK_H_ */
