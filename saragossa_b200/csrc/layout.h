// Page layout of the KV pool in HBM, shared by host and device code.
//
// pool  = [page][layer][kv_head][K tile | V tile]
// tile  = the 16 rows of one (page, layer, kv_head) for K or for V, contiguous,
//         so a K tile and its V tile are one contiguous range that a single
//         bulk (TMA) copy brings into shared memory, and one page (all layers)
//         is one contiguous range for the prefix-cache block copy.
//
// In-tile layouts (chosen so that the tile, copied verbatim into shared memory,
// is read conflict-free by the tensor-core kernels):
//   f32  : [row][dim] linear.
//   bf16 : [row][dim]; when head_dim % 64 == 0 the 16-byte chunks of a row are
//          XOR-swizzled inside each 128-byte segment: chunk c -> c ^ (row & 7).
//   u8   : K codes [row][dim] (one byte each) with 16-byte chunks swizzled by
//          c ^ (row & 7) inside each 128-byte segment (head_dim % 128 == 0), so the
//          eight rows a warp reads together fall into different banks; V codes are stored
//          TRANSPOSED, [dim][16 row slots], row r in slot vslot(r); after the
//          codes come the per-(row, group-of-32) pairs {scale bf16, bias bf16},
//          [row][group], 4 bytes each.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SGK_HD __host__ __device__ __forceinline__
#else
#define SGK_HD inline
#endif

namespace sgk {

constexpr int PAGE_TOKENS = 16;
constexpr int QGROUP = 32;
enum : int32_t { KV_F32 = 0, KV_BF16 = 1, KV_U8G32 = 2 };

SGK_HD int64_t tile_code_bytes(int dtype, int hd) {
  return dtype == KV_F32 ? int64_t(PAGE_TOKENS) * hd * 4
         : dtype == KV_BF16 ? int64_t(PAGE_TOKENS) * hd * 2
                            : int64_t(PAGE_TOKENS) * hd;
}
SGK_HD int64_t tile_bytes(int dtype, int hd) {
  int64_t meta = dtype == KV_U8G32 ? int64_t(PAGE_TOKENS) * (hd / QGROUP) * 4 : 0;
  return tile_code_bytes(dtype, hd) + meta;
}
// Bytes one stored row of one head occupies (reported as the storage size).
SGK_HD int64_t row_head_bytes(int dtype, int hd) { return tile_bytes(dtype, hd) / PAGE_TOKENS; }

// What every kernel needs to address the pool. Passed by value.
struct PoolView {
  uint8_t* base;
  int64_t page_bytes;   // all layers of one page
  int64_t layer_bytes;  // kv_heads * 2 * tile
  int64_t tile_bytes;
  const int32_t* tables;  // [max_seqs][table_stride] page ids
  int32_t* lens;          // [max_seqs][layers] rows held, per layer
  uint32_t* scale_max;    // u8 pools: f32 bits of the largest group scale ever stored (else NULL)
  int32_t table_stride;
  int32_t layers;
  int32_t kv_heads;
  int32_t head_dim;
  int32_t dtype;
};

// Byte offset of the (page, layer, head, K|V) tile.
SGK_HD int64_t tile_offset(const PoolView& p, int64_t page, int layer, int head, int is_v) {
  return page * p.page_bytes + int64_t(layer) * p.layer_bytes + (int64_t(head) * 2 + is_v) * p.tile_bytes;
}

SGK_HD bool bf16_swizzled(int hd) { return hd % 64 == 0; }

// Element index (in 2-byte units) of (row, dim) inside a bf16 tile.
SGK_HD int bf16_elem_index(int row, int dim, int hd) {
  int chunk = dim >> 3;
  if (bf16_swizzled(hd)) chunk = (chunk & ~7) | ((chunk ^ row) & 7);
  return row * hd + chunk * 8 + (dim & 7);
}

// Byte index of K code (row, dim) inside a u8 tile.
SGK_HD int u8_k_code_index(int row, int dim, int hd) {
  int chunk = dim >> 4;
  if (hd % 128 == 0) chunk = (chunk & ~7) | ((chunk ^ row) & 7);
  return row * hd + chunk * 16 + (dim & 15);
}
// Slot of row r inside the 16 bytes a V dim holds: threads of a quad read the
// four bytes {2t, 2t+1, 2t+8, 2t+9} they need for one mma A fragment as one word.
SGK_HD int u8_v_slot(int row) {
  return row < 8 ? 4 * (row >> 1) + (row & 1) : 4 * ((row - 8) >> 1) + 2 + (row & 1);
}
SGK_HD int u8_v_code_index(int row, int dim) { return dim * PAGE_TOKENS + u8_v_slot(row); }
// Byte offset of the {scale, bias} pair of (row, group) inside a u8 tile.
SGK_HD int u8_meta_offset(int row, int group, int hd) {
  return PAGE_TOKENS * hd + (row * (hd / QGROUP) + group) * 4;
}

}  // namespace sgk
