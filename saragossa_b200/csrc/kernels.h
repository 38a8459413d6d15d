// Kernel argument blocks and launchers (device side of libsgk).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_common.cuh"
#include "layout.h"

namespace sgk {

struct RopeArgs {
  int32_t rope_dims;
  int32_t frequency_dim;
  float theta;
  float position_scale;
  float eps;
  int32_t interleaved;
};

struct AppendArgs {
  PoolView pool;
  int32_t layer;
  const int32_t* slots;  // [n_seq] sequence slots; NULL => slot0 for the only sequence
  int32_t slot0;
  const float* k;        // [n_seq][n_rows][kv_dim]
  const float* v;
  int32_t n_rows;
  int64_t row0;             // first row when use_device_len == 0
  int32_t use_device_len;   // first row = the device cursor lens[slot][layer]
  int32_t bump_len;         // cursor += n_rows once every block has finished
  int32_t* done_counters;   // [n_seq], zero between launches
  int32_t* status;          // device status word
  int64_t num_pages;
  int32_t has_rope;
  const float* knorm_w;     // [head_dim]
  RopeArgs rope;
  float* out_k;             // not NULL: write normalised+rotated K rows here, touch no page
  // not NULL (bulk appends with rope): {cos, sin} of (row - rope_row0, pair), [n][rope_dims / 2], made by
  // launch_rope_table for this launch's rows: the angle does not depend on the head or on the sequence
  const float2* rope_table;
  int64_t rope_row0;
};
// {cos, sin}(position * position_scale / theta^(2 pair / frequency_dim)) for positions row0 .. row0 + n_rows - 1,
// evaluated in double precision and rounded once to f32, like the CPU path (src/decoder/attention_ops.rs:848-887).
cudaError_t launch_rope_table(float2* table, int64_t row0, int n_rows, const RopeArgs& rope, cudaStream_t stream);

struct AttnArgs {
  PoolView pool;
  int32_t layer;
  const int32_t* slots;  // [n_seq]; NULL => slot0
  int32_t slot0;
  int32_t q_heads;
  const float* q;        // [n_seq][q_heads*head_dim]
  float* out;            // [n_seq][q_heads*head_dim]
  int64_t window_start;     // explicit start row when sliding_window == 0
  int64_t sliding_window;   // > 0: start = max(len - window, 0)
  int32_t shared_merge;     // 1: every block of a (sequence, KV head) merges a slice once all have arrived
                            //    (a cooperative launch); 2: the same as an ordinary launch
  int32_t cluster_merge;    // 1: the splits of a (sequence, KV head) are one thread-block cluster and merge through
                            //    distributed shared memory (2..16 splits)
  // Several GPUs share the sequence by KV-head group (n_peers > 0): final output cells also go to
  // the same place of every peer's row, and the block that leaves last exchanges flags with the peers.
  int32_t n_peers;          // peers = the other ranks
  int32_t rank;             // this rank's index in the flag arrays
  float* peer_out[7];       // a.out's counterpart in every peer's memory
  int32_t* peer_flags[7];   // every peer's flag array
  int32_t peer_rank[7];     // every peer's index in this rank's flag array
  int32_t* local_flags;     // this rank's flag array, written by the peers
  int32_t* ex_step;         // this rank's step counter
  int32_t* exit_counter;    // blocks of the launch that have finished; zero between launches
  int32_t pages_per_split;  // > 0: a sequence is cut into ceil(pages / this) splits (<= splits), blocks beyond exit
  float scale_log2e;        // log2(e) / sqrt(attn_scalar)
  int32_t splits;
  Partials part;
  // two-level merge of the tensor-core kernel: splits are merged in groups of
  // group_size by the block that completes a group, the n_groups group results by
  // the block that completes the head
  int32_t group_size;
  int32_t n_groups;
  int32_t max_groups;
  Partials part2;           // [n_seq * q_heads][max_groups][head_dim] and {max, sum}
  int32_t* group_counters;  // [n_seq][kv_heads][max_groups]
  int32_t* head_counters;   // [n_seq][kv_heads] (tensor-core kernel) or [n_seq][q_heads] (generic)
  int32_t* seq_counters;    // [n_seq]
  int32_t* status;
  int64_t num_pages;
  // fused append (tensor-core kernel only): one new f32 row per sequence
  const float* k_new;  // [n_seq][kv_dim] or NULL
  const float* v_new;
  int32_t n_stages;
  // Launches of one decode token that follow each other on a stream (layer after layer):
  int32_t pdl_trigger;      // 1: lets the next launch of the stream start before this one has finished
  int32_t pdl_wait;         // 1: launched with programmatic stream serialisation: the block reads its cursor and
                            //    block table and starts its first copies at once, and waits for the previous
                            //    launch before it touches q, k_new, v_new or writes anything
#ifdef SGK_TRACE
  unsigned long long* trace;  // [blocks][16] timestamps, debugging builds only
  int32_t trace_gt;           // 1: the points record the global timer (ns) instead of the SM's cycle counter
#endif
};

cudaError_t launch_append_rows(const AppendArgs& a, int n_seq, cudaStream_t stream);
// Writes `value` into n consecutive int32 words (cursors, block-table entries), in stream order.
cudaError_t launch_set_len(int32_t* ptr, int32_t value, cudaStream_t stream, int n = 1);

cudaError_t launch_attention_generic(const AttnArgs& a, int n_seq, cudaStream_t stream);
// Tensor-core paged kernel: bf16 pages, head_dim 128 or 256, q_heads/kv_heads <= 8.
bool attention_mma_supported(int dtype, int head_dim, int gqa);
cudaError_t launch_attention_mma(const AttnArgs& a, int n_seq, cudaStream_t stream);
cudaError_t attention_mma_configure();
// A kernel whose only wait can never complete: it must time out, set the status word and return.
cudaError_t launch_wait_timeout_selftest(int32_t* status, cudaStream_t stream);
int attention_mma_max_stages(int head_dim);
// Blocks of the kernel one SM holds at once with `n_stages` stages (0 when the query fails).
int attention_mma_resident_blocks(int head_dim, int n_stages);
int attention_mma_max_clusters(int head_dim, int n_stages, int splits);
// Tensor-core paged kernel for u8 group-32 pages: head_dim 128 or 256, q_heads/kv_heads <= 8.
bool attention_u8_supported(int dtype, int head_dim, int gqa);
cudaError_t launch_attention_u8(const AttnArgs& a, int n_seq, cudaStream_t stream);
cudaError_t attention_u8_configure();
int attention_u8_max_stages(int head_dim);
int attention_u8_resident_blocks(int head_dim, int n_stages);
int attention_u8_max_clusters(int head_dim, int n_stages, int splits);

// Gather rows [row0, row0+n) of one layer into contiguous [n, kv_dim] arrays.
// mode 0: storage type (f32 / bf16 bits), 1: decoded f32, 2: u8 codes + scale + bias.
struct GatherArgs {
  PoolView pool;
  int32_t layer;
  int32_t slot;
  int64_t row0;
  int64_t n;
  int32_t mode;
  void* k_out;
  void* v_out;
  uint16_t* k_scale;
  uint16_t* k_bias;
  uint16_t* v_scale;
  uint16_t* v_bias;
  int64_t num_pages;
  int32_t* status;
};
cudaError_t launch_gather(const GatherArgs& a, cudaStream_t stream);

// What a restore installs with its copy: table[i] = dst_pages[i] for every copied page, and
// lens[0 .. n_lens) = len_value (the cursors of the sequence's layers).
struct CopyInstall {
  int32_t* table = nullptr;
  int32_t* lens = nullptr;
  int32_t n_lens = 0;
  int32_t len_value = 0;
};
// Page copy: dst_pages[i] <- src_pages[i]; a page is n_layers pieces of page_bytes, layer_stride
// apart (16-byte vectors).
cudaError_t launch_copy_pages(uint8_t* dst_base, const uint8_t* src_base, const int32_t* d_dst_pages,
                              const int32_t* d_src_pages, int n_pages, int64_t page_bytes, int n_layers,
                              int64_t layer_stride, int sm_count,
                              cudaStream_t stream, const CopyInstall* install = nullptr);
// Contiguous device copy (linear-state snapshot / restore).
cudaError_t launch_copy_bytes(void* dst, const void* src, int64_t bytes, cudaStream_t stream);
// Zero-fill of freed pages (eviction scrub).
cudaError_t launch_scrub_pages(uint8_t* base, const int32_t* d_pages, int n_pages, int64_t page_bytes, int n_layers,
                               int64_t layer_stride, int sm_count,
                               cudaStream_t stream);
// Gated DeltaNet step on one layer's state [H_v][d_v][d_k] (f32 or bf16).
constexpr int GATED_DELTA_MAX_STATES = 64;
struct GatedDeltaArgs {
  void* ssm[GATED_DELTA_MAX_STATES];  // one state per sequence, passed by value: no device table
  int32_t n_states;
  int32_t n_tokens;   // tokens run one after the other on the state kept in registers; inputs gain a [n_tokens] dim
  int32_t ssm_bf16;
  int32_t num_key_heads, num_value_heads, key_head_dim, value_head_dim;
  const float* q;     // [n_states][n_tokens][H_k * d_k]
  const float* k;     // [n_states][n_tokens][H_k * d_k]
  const float* v;     // [n_states][n_tokens][H_v * d_v]
  const float* g;     // [n_states][n_tokens][H_v] decay
  const float* beta;  // [n_states][n_tokens][H_v] write gate
  float* out;         // [n_states][n_tokens][H_v * d_v]
  // member of a token chain: lets the next launch start early / was itself launched with programmatic
  // stream serialisation and reads the state before, its inputs after, the wait for the previous launch
  int32_t pdl_trigger, pdl_wait;
};
cudaError_t launch_gated_delta_step(const GatedDeltaArgs& a, int sm_count, cudaStream_t stream);
// One decode token of a whole recurrent layer between its projections, one launch:
// conv + SiLU + unit RMS norm of q and k + gates + gated-delta update (key and value head dim 128).
struct LinearDecodeArgs {
  void* ssm;                  // [H_v][128][128] state of this layer
  float* history;             // [(K-1)][conv_dim] conv history of this layer
  const float* qkv;           // [conv_dim] the token's projected q | k | v
  const float* conv_weight;   // [conv_dim][K]
  const float* beta_input;    // [H_v]
  const float* gate_input;    // [H_v]
  const float* a_log;         // [H_v]
  const float* dt_bias;       // [H_v]
  float* out;                 // [H_v * 128]
  int32_t* head_counters;     // [H_k] arrivals of a key head's blocks; zero between launches
  int32_t conv_dim, kernel;
  int32_t num_key_heads, num_value_heads;
  float q_scale, k_scale, eps;
  int32_t ssm_bf16, pdl_trigger, pdl_wait;
};
cudaError_t launch_linear_decode_step(const LinearDecodeArgs& a, cudaStream_t stream);
cudaError_t launch_conv_step(const float* qkv, const float* weight, float* history, float* out, int conv_dim,
                             int kernel, int n_tokens, int pdl_trigger, int pdl_wait, cudaStream_t stream);
// Launch configuration shared by the small kernels of a token chain.
struct ChainLaunch {
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  ChainLaunch(dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl_wait) {
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_wait ? 1 : 0;
  }
};
// Greedy epilogue: argmax over W . x without materialising the logits.
struct LmHeadArgs {
  const void* w;   // [vocab][hidden], f32 or bf16
  int32_t w_bf16;
  int64_t vocab;
  int32_t hidden;  // multiple of 8; the activation rows are held in shared memory (lm_head_smem_bytes)
  int32_t n_rows;  // 1..8 activation rows sharing the pass over the weight
  const float* x;  // [n_rows][hidden]
  unsigned long long* keys;  // workspace [8]: packed (value, index) of the best row so far; zero between launches
  unsigned int* counter;    // workspace: blocks done; zero between launches
  int32_t index_offset;
  int32_t* index_out;  // [n_rows]
  float* value_out;    // [n_rows], may be NULL
  int32_t pdl_trigger, pdl_wait;   // member of a token chain (see GatedDeltaArgs)
  int32_t* index_mirror;   // mapped host memory that gets the indices too (may be NULL)
  // 16-row tiles handed out in whole rounds (a multiple of every grid's warp count, set by the launcher
  // from the SM count alone so that it does not depend on the number of activation rows); the rest
  // are split across the warps of a block
  int64_t whole_tiles;
};
cudaError_t launch_lm_head_argmax(const LmHeadArgs& a, int sm_count, cudaStream_t stream);
// The same over an affine-quantised weight (MLX layout, src/quantization.rs:173-238): codes of
// `bits` (4 or 8) packed LSB-first into u32 words, row-major [vocab][hidden * bits / 32]; one bf16
// scale and one bf16 bias per (row, group of group_size columns); value = code * scale + bias.
struct AffineWeight {
  const uint32_t* packed;
  const uint16_t* scales;
  const uint16_t* biases;
  int32_t bits, group_size;
};
struct LmHeadAffineArgs {
  AffineWeight w;
  int64_t vocab;
  int32_t hidden;   // multiple of the group size (64 or 128)
  int32_t n_rows;   // 1..8
  const float* x;
  unsigned long long* keys;
  unsigned int* counter;
  int32_t index_offset;
  int32_t* index_out;
  float* value_out;
  int32_t pdl_trigger, pdl_wait;
  int32_t* index_mirror;   // mapped host memory that gets the indices too (may be NULL)
  // 16-row tiles handed out in whole rounds (a multiple of every grid's warp count, set by the launcher
  // from the SM count alone so that it does not depend on the number of activation rows); the rest
  // are split across the warps of a block
  int64_t whole_tiles;
};
cudaError_t launch_lm_head_argmax_affine(const LmHeadAffineArgs& a, int sm_count, cudaStream_t stream);
size_t lm_head_affine_smem_bytes(int n_rows, int hidden, int group_size);
cudaError_t launch_embed_gather_affine(const AffineWeight& table, const int32_t* index, int64_t vocab, int hidden,
                                       float scale, int recast_bf16, float* out, int pdl_trigger, int pdl_wait,
                                       cudaStream_t stream);
size_t lm_head_smem_bytes(int w_bf16, int n_rows, int hidden);  // shared memory a launch needs
// out[hidden] = table[*index] * scale (dense f32 or bf16 table); an index outside the table writes nothing.
cudaError_t launch_embed_gather(const void* table, int table_bf16, const int32_t* index, int64_t vocab, int hidden,
                                float scale, int recast_bf16, float* out, int pdl_trigger, int pdl_wait,
                                cudaStream_t stream);
// Exchange of output slices between ranks over peer memory (kernels_exchange.cu).
constexpr int EXCHANGE_MAX_RANKS = 8;
struct ExchangeArgs {
  const float* local_row;   // this rank's full row; its own slice has been written
  float* peer_row[EXCHANGE_MAX_RANKS];      // the same row in every peer's memory (entry `rank` unused)
  int32_t* peer_flags[EXCHANGE_MAX_RANKS];  // every peer's flag array [n_ranks] (entry `rank` unused)
  int32_t* local_flags;     // this rank's flag array [n_ranks], written by the peers
  int32_t* step;            // this rank's step counter
  int64_t slice_offset;     // floats, multiple of 4
  int32_t slice_floats;     // multiple of 4
  int32_t rank, n_ranks;
  int32_t* status;
};
cudaError_t launch_exchange_slices(const ExchangeArgs& a, cudaStream_t stream);
cudaError_t launch_fill_normal(float* out, int64_t n, uint64_t seed, uint64_t stream_id,
                               uint64_t index0, cudaStream_t stream);

}  // namespace sgk
