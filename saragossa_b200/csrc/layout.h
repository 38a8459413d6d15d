// Page layout of the KV pool in HBM, shared by host and device code.
//
// pool  = [layer][page][kv_head][K tile | V tile]
// tile  = the 16 rows of one (layer, page, kv_head) for K or for V, contiguous,
//         so a K tile and its V tile are one contiguous range that a single
//         bulk (TMA) copy brings into shared memory. Layer-major: the pages a
//         decode kernel streams (one layer of every sequence) sit in one dense
//         region instead of being a whole-page stride apart, which keeps the
//         number of address translations a launch needs small; the prefix-cache
//         block copy moves a page as one contiguous piece per layer.
//
// In-tile layouts (chosen so that the tile, copied verbatim into shared memory,
// is read conflict-free by the tensor-core kernels):
//   f32  : [row][dim] linear.
//   bf16 : [row][dim]; when head_dim % 64 == 0 the 16-byte chunks of a row are
//          XOR-swizzled inside each 128-byte segment: chunk c -> c ^ (row & 7).
//   u8   : K codes [row][dim] (one byte each); when head_dim % 128 == 0 the 32-byte
//          granules (= quantisation groups) of a row are XOR-swizzled inside each 128-byte
//          segment, granule c -> c ^ (row & 3), so the four rows a half-warp reads
//          together with 8-byte loads fall into different banks. V codes are stored
//          TRANSPOSED, row r in byte slot vslot(r) of a 4-byte word per (dim, quad), and
//          (head_dim % 64 == 0) the words are ordered so that a lane's words of four
//          consecutive 16-dim steps are two 16-byte loads, see u8_v_code_index. After the
//          codes: the bf16 scales [row][group], then the bf16 biases, [row][group] for K
//          and [group][row] for V (the order the tensor-core bias products read them in).
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
  int64_t page_bytes;   // stride between pages inside a layer: kv_heads * 2 * tile
  int64_t layer_bytes;  // stride between layers: num_pages * page_bytes
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
  int gran = dim >> 5;
  if (hd % 128 == 0) gran = (gran & ~3) | ((gran ^ row) & 3);
  return row * hd + gran * 32 + (dim & 31);
}
// Slot of row r inside the 16 bytes a V dim holds: threads of a quad read the
// four bytes {2t, 2t+1, 2t+8, 2t+9} they need for one mma A fragment as one word.
SGK_HD int u8_v_slot(int row) {
  return row < 8 ? 4 * (row >> 1) + (row & 1) : 4 * ((row - 8) >> 1) + 2 + (row & 1);
}
// Byte index of V code (row, dim). With j = dim / 16 the 16-dim step, lane = (dim % 8) * 4 +
// slot / 4 the lane that owns the word in the mma A fragment and half = (dim / 8) % 2 its
// upper or lower eight dims, the words of steps 4q .. 4q+3 lie as [q][j / 2 % 2][lane][(j % 2) * 2 + half]:
// a lane reads them with two 16-byte loads at consecutive-lane addresses.
SGK_HD int u8_v_code_index(int row, int dim, int hd) {
  const int slot = u8_v_slot(row);
  if (hd % 64 != 0) return dim * PAGE_TOKENS + slot;
  const int j = dim >> 4, half = (dim >> 3) & 1, g = dim & 7;
  const int word = ((((j >> 2) * 2 + ((j >> 1) & 1)) * 32 + g * 4 + (slot >> 2)) * 4) + (j & 1) * 2 + half;
  return word * 4 + (slot & 3);
}
// Byte offsets of the bf16 scale and bias of (row, group) inside a u8 tile.
SGK_HD int u8_scale_offset(int row, int group, int hd) {
  return PAGE_TOKENS * hd + (row * (hd / QGROUP) + group) * 2;
}
SGK_HD int u8_bias_offset(int is_v, int row, int group, int hd) {
  const int groups = hd / QGROUP;
  return PAGE_TOKENS * hd + PAGE_TOKENS * groups * 2 +
         (is_v ? group * PAGE_TOKENS + row : row * groups + group) * 2;
}

}  // namespace sgk
