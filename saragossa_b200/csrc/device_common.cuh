// Device helpers shared by the kernels: storage conversions (bit-exact with the
// reference's host code), element access through the page layout, and the
// split-K partial merge.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "layout.h"

namespace sgk {

// Device status word values (read back by sgk_state_device_status).
constexpr int DEV_OK = 0;
constexpr int DEV_ERR_WAIT_TIMEOUT = 6;  // a bounded mbarrier wait expired
constexpr int DEV_ERR_BAD_PAGE = 7;      // a block-table entry was out of range

// f32 -> bf16 bits, round to nearest even: bits + 0x7fff + lsb, >> 16, the integer
// form of the reference (src/decode_resident/utils.rs:55-60), NaN not special-cased.
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
  uint32_t bits = __float_as_uint(v);
  uint32_t lsb = (bits >> 16) & 1u;
  return static_cast<uint16_t>((bits + 0x7fffu + lsb) >> 16);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}

// One stored element (row, dim) of a tile decoded to f32: f32 as is, bf16 upcast,
// u8 q*scale+bias with separate roundings (src/quantization.rs:173-179).
__device__ __forceinline__ float load_tile_elem(const uint8_t* tile, int dtype, int hd, int is_v,
                                                int row, int dim) {
  if (dtype == KV_F32) return reinterpret_cast<const float*>(tile)[row * hd + dim];
  if (dtype == KV_BF16)
    return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(tile)[bf16_elem_index(row, dim, hd)]);
  int idx = is_v ? u8_v_code_index(row, dim, hd) : u8_k_code_index(row, dim, hd);
  float scale = bf16_bits_to_f32(*reinterpret_cast<const uint16_t*>(tile + u8_scale_offset(row, dim / QGROUP, hd)));
  float bias = bf16_bits_to_f32(*reinterpret_cast<const uint16_t*>(tile + u8_bias_offset(is_v, row, dim / QGROUP, hd)));
  return __fadd_rn(__fmul_rn(static_cast<float>(tile[idx]), scale), bias);
}

// Split-K partials: for every (sequence, q head, split) an un-normalised output
// row, its running maximum (log2 domain) and its sum of weights.
struct Partials {
  float* o;   // [n_seq * q_heads][splits][head_dim]
  float* ml;  // [n_seq * q_heads][splits][2] = {max, sum}
};

// Merges the `splits` partials of q head `qh_global` and writes the normalised
// output. Called by every thread of the block that arrived last.
__device__ __forceinline__ void merge_partials(const Partials& part, int64_t qh_global, int splits,
                                               int hd, float* out_row, int tid, int nthreads) {
  const float* ml = part.ml + qh_global * splits * 2;
  float m = -1.0e30f;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) m = fmaxf(m, __ldcg(ml + 2 * s));
  float denom = 0.0f;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) denom += __ldcg(ml + 2 * s + 1) * exp2f(__ldcg(ml + 2 * s) - m);
  float inv = 1.0f / denom;
  const float* o = part.o + qh_global * splits * hd;
  for (int d = tid; d < hd; d += nthreads) {
    float acc = 0.0f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s)
      acc += __ldcg(o + int64_t(s) * hd + d) * exp2f(__ldcg(ml + 2 * s) - m);
    out_row[d] = acc * inv;
  }
}

}  // namespace sgk
