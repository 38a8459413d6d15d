// KV append: f32 K/V rows -> (optional RMSNorm + RoPE on K) -> storage type
// (f32 / bf16 RNE / u8 group-32) -> scattered into the page the block table
// names. One block per (kv head, row, sequence). Replaces the reference's
// copy_at_f32 / copy_at_f32_to_bf16 dispatches (src/decode_resident/kernels.rs:1026-1044),
// the host f32->bf16 loop of seed/append_row (src/decode_resident/utils.rs:76-110)
// and, when fused, rms_norm_rope_heads_decode_f32 (kernels.rs:975-1024).
#include "kernels.h"

namespace sgk {

// RMSNorm x weight then RoPE of one head held in shared memory, in the float
// order of the CPU path (src/decoder/attention_ops.rs:737-768): sequential sum
// of squares, 1/sqrt, x*inv_rms*w, then first*cos - second*sin with separate
// roundings. cos/sin are evaluated in double and rounded once to f32.
__device__ void norm_rope_head(float* xs, int hd, const float* weight, const RopeArgs& rope,
                               int64_t position, float* scratch) {
  int tid = threadIdx.x;
  if (tid == 0) {
    float sum = 0.0f;
    for (int c = 0; c < hd; ++c) sum = __fadd_rn(sum, __fmul_rn(xs[c], xs[c]));
    float mean_square = __fdiv_rn(sum, static_cast<float>(hd));
    scratch[0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_square, rope.eps)));
  }
  __syncthreads();
  float inv_rms = scratch[0];
  for (int c = tid; c < hd; c += blockDim.x) xs[c] = __fmul_rn(__fmul_rn(xs[c], inv_rms), weight[c]);
  __syncthreads();
  int pairs = rope.rope_dims / 2;
  float scaled_position = __fmul_rn(static_cast<float>(position), rope.position_scale);
  for (int pair = tid; pair < pairs; pair += blockDim.x) {
    float exponent = __fdiv_rn(static_cast<float>(2 * pair), static_cast<float>(rope.frequency_dim));
    float denom = static_cast<float>(pow(static_cast<double>(rope.theta), static_cast<double>(exponent)));
    float angle = __fdiv_rn(scaled_position, denom);
    float c = static_cast<float>(cos(static_cast<double>(angle)));
    float s = static_cast<float>(sin(static_cast<double>(angle)));
    int i0 = rope.interleaved ? 2 * pair : pair;
    int i1 = rope.interleaved ? 2 * pair + 1 : pair + pairs;
    float first = xs[i0], second = xs[i1];
    xs[i0] = __fsub_rn(__fmul_rn(first, c), __fmul_rn(second, s));
    xs[i1] = __fadd_rn(__fmul_rn(first, s), __fmul_rn(second, c));
  }
  __syncthreads();
}

// Quantises the 32 values one warp holds (one per lane) to u8 codes with a bf16
// scale and bias; returns the code, lane 0 also gets the packed {scale, bias}.
__device__ __forceinline__ uint32_t quantize_group_warp(float x, uint32_t* meta_out) {
  float lo = x, hi = x;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
  }
  uint16_t bias_bits = f32_to_bf16_bits(lo);
  float bias = bf16_bits_to_f32(bias_bits);
  float raw = __fdiv_rn(__fsub_rn(hi, bias), 255.0f);
  uint16_t scale_bits = f32_to_bf16_bits(fmaxf(raw, 0x1p-40f));
  float scale = bf16_bits_to_f32(scale_bits);
  float t = rintf(__fdiv_rn(__fsub_rn(x, bias), scale));
  t = fminf(fmaxf(t, 0.0f), 255.0f);
  *meta_out = static_cast<uint32_t>(scale_bits) | (static_cast<uint32_t>(bias_bits) << 16);
  return static_cast<uint32_t>(t);
}

// Writes one head row (hd f32 values in shared memory) into its tile.
__device__ void store_head_row(uint8_t* tile, int dtype, int hd, int is_v, int row, const float* xs,
                               uint32_t* scale_max) {
  int tid = threadIdx.x;
  if (dtype == KV_F32) {
    float* dst = reinterpret_cast<float*>(tile) + row * hd;
    for (int c = tid; c < hd; c += blockDim.x) dst[c] = xs[c];
  } else if (dtype == KV_BF16) {
    uint16_t* dst = reinterpret_cast<uint16_t*>(tile);
    if (hd % 8 == 0) {
      for (int chunk = tid; chunk < hd / 8; chunk += blockDim.x) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          w[i] = static_cast<uint32_t>(f32_to_bf16_bits(xs[chunk * 8 + 2 * i])) |
                 (static_cast<uint32_t>(f32_to_bf16_bits(xs[chunk * 8 + 2 * i + 1])) << 16);
        *reinterpret_cast<uint4*>(dst + bf16_elem_index(row, chunk * 8, hd)) =
            make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
      for (int c = tid; c < hd; c += blockDim.x) dst[bf16_elem_index(row, c, hd)] = f32_to_bf16_bits(xs[c]);
    }
  } else {
    int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    for (int g = warp; g < hd / QGROUP; g += warps) {
      int dim = g * QGROUP + lane;
      uint32_t meta;
      uint32_t code = quantize_group_warp(xs[dim], &meta);
      int idx = is_v ? u8_v_code_index(row, dim, hd) : u8_k_code_index(row, dim, hd);
      tile[idx] = static_cast<uint8_t>(code);
      if (lane == 0) {
        *reinterpret_cast<uint16_t*>(tile + u8_scale_offset(row, g, hd)) = static_cast<uint16_t>(meta & 0xffffu);
        *reinterpret_cast<uint16_t*>(tile + u8_bias_offset(is_v, row, g, hd)) = static_cast<uint16_t>(meta >> 16);
        // largest scale of the pool (positive floats order like their bit patterns)
        const uint32_t scale_f32_bits = (meta & 0xffffu) << 16;
        if (scale_max != nullptr && scale_f32_bits > *reinterpret_cast<volatile uint32_t*>(scale_max))
          atomicMax(scale_max, scale_f32_bits);
      }
    }
  }
}

__global__ void __launch_bounds__(128) append_rows_kernel(AppendArgs a) {
  extern __shared__ float smem[];
  const int hd = a.pool.head_dim;
  float* ks = smem;
  float* vs = smem + hd;
  float* scratch = smem + 2 * hd;
  const int head = blockIdx.x, r = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x;
  const int kv_dim = a.pool.kv_heads * hd;
  const int slot = a.slots ? a.slots[seq] : a.slot0;
  int32_t* len_ptr = a.pool.lens + int64_t(slot) * a.pool.layers + a.layer;
  const int64_t len0 = a.use_device_len ? static_cast<int64_t>(*len_ptr) : a.row0;
  const int64_t row = len0 + r;

  const float* ksrc = a.k + (int64_t(seq) * a.n_rows + r) * kv_dim + head * hd;
  const float* vsrc = a.v + (int64_t(seq) * a.n_rows + r) * kv_dim + head * hd;
  for (int c = tid; c < hd; c += blockDim.x) {
    ks[c] = ksrc[c];
    vs[c] = vsrc[c];
  }
  __syncthreads();
  if (a.has_rope) norm_rope_head(ks, hd, a.knorm_w, a.rope, row, scratch);

  if (a.out_k != nullptr) {
    // Standalone RMSNorm+RoPE: write the f32 result, touch no page.
    for (int c = tid; c < hd; c += blockDim.x)
      a.out_k[(int64_t(seq) * a.n_rows + r) * kv_dim + head * hd + c] = ks[c];
    return;
  }

  const int64_t page_index = row / PAGE_TOKENS;
  int32_t page = -1;
  if (page_index < a.pool.table_stride) page = a.pool.tables[int64_t(slot) * a.pool.table_stride + page_index];
  if (page >= 0 && page < a.num_pages) {
    const int rin = static_cast<int>(row % PAGE_TOKENS);
    uint8_t* ktile = a.pool.base + tile_offset(a.pool, page, a.layer, head, 0);
    uint8_t* vtile = a.pool.base + tile_offset(a.pool, page, a.layer, head, 1);
    store_head_row(ktile, a.pool.dtype, hd, 0, rin, ks, a.pool.scale_max);
    store_head_row(vtile, a.pool.dtype, hd, 1, rin, vs, a.pool.scale_max);
  } else if (tid == 0) {
    atomicExch(a.status, DEV_ERR_BAD_PAGE);
  }

  if (a.bump_len) {
    // The block that arrives last moves the cursor: every block has read it by then.
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      int total = gridDim.x * gridDim.y;
      int old = atomicAdd(a.done_counters + seq, 1);
      if (old == total - 1) {
        *len_ptr = static_cast<int32_t>(len0 + a.n_rows);
        a.done_counters[seq] = 0;
        __threadfence();
      }
    }
  }
}

__global__ void set_len_kernel(int32_t* ptr, int n, int32_t value) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ptr[i] = value;
}

cudaError_t launch_append_rows(const AppendArgs& a, int n_seq, cudaStream_t stream) {
  dim3 grid(a.pool.kv_heads, a.n_rows, n_seq);
  size_t smem = (2 * size_t(a.pool.head_dim) + 4) * sizeof(float);
  append_rows_kernel<<<grid, 128, smem, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_set_len(int32_t* ptr, int32_t value, cudaStream_t stream, int n) {
  set_len_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ptr, n, value);
  return cudaGetLastError();
}

}  // namespace sgk
