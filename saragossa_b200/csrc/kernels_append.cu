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


// ---- bulk append: one block per (kv head, page, sequence) -------------------------------------
// The rows of a multi-row append that fall into one page are one tile: the block reads them with
// 16-byte loads, does what the single-row kernel does per row (same arithmetic, so the bits are
// the same whichever kernel wrote a row), and writes the tile region with 16-byte stores. One
// cursor arrival per block instead of one per row: a seeding launch of 8192 rows made 32768
// atomic arrivals on one counter and ran at 0.9 TB/s.
template <int N>
__device__ __forceinline__ void quantize_groups_warp(const float (&x)[N], uint32_t (&code)[N], uint32_t (&meta)[N]) {
  float lo[N], hi[N];
  // warp-wide float min / max in one instruction each (sm_100a), instead of a five-step butterfly
#pragma unroll
  for (int i = 0; i < N; ++i) {
    asm("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(lo[i]) : "f"(x[i]));
    asm("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(hi[i]) : "f"(x[i]));
  }
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const uint16_t bias_bits = f32_to_bf16_bits(lo[i]);
    const float bias = bf16_bits_to_f32(bias_bits);
    const float raw = __fdiv_rn(__fsub_rn(hi[i], bias), 255.0f);
    const uint16_t scale_bits = f32_to_bf16_bits(fmaxf(raw, 0x1p-40f));
    const float scale = bf16_bits_to_f32(scale_bits);
    float t = rintf(__fdiv_rn(__fsub_rn(x[i], bias), scale));
    t = fminf(fmaxf(t, 0.0f), 255.0f);
    meta[i] = static_cast<uint32_t>(scale_bits) | (static_cast<uint32_t>(bias_bits) << 16);
    code[i] = static_cast<uint32_t>(t);
  }
}

// One (row, K or V) of a u8 tile: all groups of the head row at once, one warp.
template <int G>
__device__ __forceinline__ uint32_t store_u8_row(uint8_t* tile, int hd, int is_v, int rin, const float* xs, int lane) {
  float x[G];
  uint32_t code[G], meta[G];
#pragma unroll
  for (int g = 0; g < G; ++g) x[g] = xs[g * QGROUP + lane];
  quantize_groups_warp<G>(x, code, meta);
  uint32_t biggest = 0;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int dim = g * QGROUP + lane;
    tile[is_v ? u8_v_code_index(rin, dim, hd) : u8_k_code_index(rin, dim, hd)] = static_cast<uint8_t>(code[g]);
    biggest = max(biggest, (meta[g] & 0xffffu) << 16);
    if (lane == g) {
      *reinterpret_cast<uint16_t*>(tile + u8_scale_offset(rin, g, hd)) = static_cast<uint16_t>(meta[g] & 0xffffu);
      *reinterpret_cast<uint16_t*>(tile + u8_bias_offset(is_v, rin, g, hd)) = static_cast<uint16_t>(meta[g] >> 16);
    }
  }
  return biggest;
}

// DIRECT: rows that need no arithmetic across a row (no rope, f32 or bf16 storage) go from registers
// to the page; that instance is held to 32 registers so that sixteen blocks fit an SM and a launch
// of a few thousand tiles is ONE wave (with 64 registers it was 1.74 waves: 15.3 us for 50 MB).
template <bool DIRECT>
__global__ void __launch_bounds__(128, DIRECT ? 16 : 8) append_tiles_kernel(AppendArgs a) {
  extern __shared__ float smem[];
  const int hd = a.pool.head_dim;
  // staged path only: K rows [16][hd + 4], 1/rms per row [16], rope denominators [128], and for
  // u8 pools the V rows [16][hd] and a tile pair being put together
  const int kstride = hd + 4;
  float* ks = smem;
  float* inv_s = ks + PAGE_TOKENS * kstride;
  float* denom_s = inv_s + PAGE_TOKENS;
  float* vs = denom_s + 128;
  uint8_t* stage = reinterpret_cast<uint8_t*>(vs + PAGE_TOKENS * hd);
  __shared__ uint32_t big_s;
  const int head = blockIdx.x, tile_i = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kv_dim = a.pool.kv_heads * hd;
  const int slot = a.slots ? a.slots[seq] : a.slot0;
  int32_t* len_ptr = a.pool.lens + int64_t(slot) * a.pool.layers + a.layer;
  const int64_t len0 = a.use_device_len ? static_cast<int64_t>(*len_ptr) : a.row0;
  const int64_t page_index = len0 / PAGE_TOKENS + tile_i;
  const int64_t row_lo = max(len0, page_index * PAGE_TOKENS);
  const int64_t row_hi = min(len0 + a.n_rows, (page_index + 1) * PAGE_TOKENS);
  const int rows = static_cast<int>(row_hi - row_lo);
  if (tid == 0) big_s = 0;

  if (rows > 0 && DIRECT) {
    // nothing to compute across a row: registers only, no staging. The block-table entry is asked
    // for first and looked at only before the stores: the rows' loads do not wait for it.
    const int rin0 = static_cast<int>(row_lo % PAGE_TOKENS);
    const float* kbase = a.k + (int64_t(seq) * a.n_rows + (row_lo - len0)) * kv_dim + head * hd;
    const float* vbase = a.v + (int64_t(seq) * a.n_rows + (row_lo - len0)) * kv_dim + head * hd;
    int32_t page = -1;
    if (page_index < a.pool.table_stride) page = a.pool.tables[int64_t(slot) * a.pool.table_stride + page_index];
    // head_dim is 64, 128 or 256 here: the chunk arithmetic is shifts and masks, not divisions
    const int chunk_shift = hd == 64 ? 3 : hd == 128 ? 4 : 5;
    const int chunks = 1 << chunk_shift, half = rows << chunk_shift;
    const int total = 2 * half;
    // two chunks of eight values per thread and pass, every load issued before the first store
    // (sixteen blocks per SM keep 128 KB of loads in flight; four chunks would spill at 32 registers)
    constexpr int U = 2;
    for (int base = 0; base < total; base += U * blockDim.x) {
      float4 x0[U], x1[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * blockDim.x + tid;
        if (i < total) {
          const int is_v = i >= half, rest = is_v ? i - half : i;
          const int r = rest >> chunk_shift, chunk = rest & (chunks - 1);
          const float4* src = reinterpret_cast<const float4*>((is_v ? vbase : kbase) + int64_t(r) * kv_dim + chunk * 8);
          x0[u] = __ldg(src);
          x1[u] = __ldg(src + 1);
        }
      }
      if (page < 0 || page >= a.num_pages) break;   // uniform over the block; reported below
      uint8_t* ktile = a.pool.base + tile_offset(a.pool, page, a.layer, head, 0);
      uint8_t* vtile = a.pool.base + tile_offset(a.pool, page, a.layer, head, 1);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * blockDim.x + tid;
        if (i >= total) continue;
        const int is_v = i >= half, rest = is_v ? i - half : i;
        const int r = rest >> chunk_shift, chunk = rest & (chunks - 1);
        uint8_t* tile = is_v ? vtile : ktile;
        if (a.pool.dtype == KV_F32) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(tile) + (rin0 + r) * hd + chunk * 8);
          dst[0] = x0[u];
          dst[1] = x1[u];
        } else {
          const uint4 w = make_uint4(uint32_t(f32_to_bf16_bits(x0[u].x)) | (uint32_t(f32_to_bf16_bits(x0[u].y)) << 16),
                                     uint32_t(f32_to_bf16_bits(x0[u].z)) | (uint32_t(f32_to_bf16_bits(x0[u].w)) << 16),
                                     uint32_t(f32_to_bf16_bits(x1[u].x)) | (uint32_t(f32_to_bf16_bits(x1[u].y)) << 16),
                                     uint32_t(f32_to_bf16_bits(x1[u].z)) | (uint32_t(f32_to_bf16_bits(x1[u].w)) << 16));
          *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(tile) + bf16_elem_index(rin0 + r, chunk * 8, hd)) = w;
        }
      }
    }
    if ((page < 0 || page >= a.num_pages) && tid == 0) atomicExch(a.status, DEV_ERR_BAD_PAGE);
  } else if (rows > 0 && !DIRECT) {
    // K is worked on in shared memory; V only when it is quantised. K rows sit kstride floats
    // apart: with the rows a whole number of 128-byte lines apart, the sixteen threads that
    // walk one row each for the sequential sums hit one bank sixteen times per step, which made
    // a launch of 2056 tiles shared-memory bound (47.9 us against 15.3 us without rope).
    const int rin0 = static_cast<int>(row_lo % PAGE_TOKENS);
    const bool stage_v = a.pool.dtype == KV_U8G32;
    // head_dim is 64, 128 or 256 here: the chunk arithmetic is shifts and masks, not divisions
    const int chunk_shift = hd == 64 ? 3 : hd == 128 ? 4 : 5;
    const int chunks = 1 << chunk_shift, total = rows << chunk_shift;
    const float* kbase = a.k + (int64_t(seq) * a.n_rows + (row_lo - len0)) * kv_dim + head * hd;
    const float* vbase = a.v + (int64_t(seq) * a.n_rows + (row_lo - len0)) * kv_dim + head * hd;
    int32_t page = -1;
    if (page_index < a.pool.table_stride) page = a.pool.tables[int64_t(slot) * a.pool.table_stride + page_index];
    const bool page_ok = page >= 0 && page < a.num_pages;
    uint8_t* ktile = page_ok ? a.pool.base + tile_offset(a.pool, page, a.layer, head, 0) : nullptr;
    uint8_t* vtile = page_ok ? a.pool.base + tile_offset(a.pool, page, a.layer, head, 1) : nullptr;
    // two chunks of eight values of K and of V per thread and pass: all loads of a pass are
    // issued before anything waits for one
    constexpr int U = 2;
    for (int base = 0; base < total; base += U * blockDim.x) {
      float4 k0[U], k1[U], v0[U], v1[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * blockDim.x + tid;
        if (i < total) {
          const int r = i >> chunk_shift, chunk = i & (chunks - 1);
          const float4* ksrc = reinterpret_cast<const float4*>(kbase + int64_t(r) * kv_dim + chunk * 8);
          const float4* vsrc = reinterpret_cast<const float4*>(vbase + int64_t(r) * kv_dim + chunk * 8);
          k0[u] = __ldg(ksrc);
          k1[u] = __ldg(ksrc + 1);
          v0[u] = __ldg(vsrc);
          v1[u] = __ldg(vsrc + 1);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * blockDim.x + tid;
        if (i >= total) continue;
        const int r = i >> chunk_shift, chunk = i & (chunks - 1);
        float4* kd = reinterpret_cast<float4*>(ks + r * kstride + chunk * 8);
        kd[0] = k0[u];
        kd[1] = k1[u];
        if (stage_v) {
          float4* vd = reinterpret_cast<float4*>(vs + r * hd + chunk * 8);
          vd[0] = v0[u];
          vd[1] = v1[u];
        } else if (page_ok) {
          if (a.pool.dtype == KV_F32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(vtile) + (rin0 + r) * hd + chunk * 8);
            dst[0] = v0[u];
            dst[1] = v1[u];
          } else {
            const uint4 w = make_uint4(uint32_t(f32_to_bf16_bits(v0[u].x)) | (uint32_t(f32_to_bf16_bits(v0[u].y)) << 16),
                                       uint32_t(f32_to_bf16_bits(v0[u].z)) | (uint32_t(f32_to_bf16_bits(v0[u].w)) << 16),
                                       uint32_t(f32_to_bf16_bits(v1[u].x)) | (uint32_t(f32_to_bf16_bits(v1[u].y)) << 16),
                                       uint32_t(f32_to_bf16_bits(v1[u].z)) | (uint32_t(f32_to_bf16_bits(v1[u].w)) << 16));
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(vtile) + bf16_elem_index(rin0 + r, chunk * 8, hd)) = w;
          }
        }
      }
    }
    __syncthreads();
    if (a.has_rope) {
      // same float order as norm_rope_head, one thread per row for the sequential sums
      if (tid < rows) {
        const float4* xs = reinterpret_cast<const float4*>(ks + tid * kstride);
        float sum = 0.0f;
#pragma unroll 4
        for (int c = 0; c < hd / 4; ++c) {
          const float4 x = xs[c];
          sum = __fadd_rn(sum, __fmul_rn(x.x, x.x));
          sum = __fadd_rn(sum, __fmul_rn(x.y, x.y));
          sum = __fadd_rn(sum, __fmul_rn(x.z, x.z));
          sum = __fadd_rn(sum, __fmul_rn(x.w, x.w));
        }
        const float mean_square = __fdiv_rn(sum, static_cast<float>(hd));
        inv_s[tid] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_square, a.rope.eps)));
      }
      const int pairs = a.rope.rope_dims / 2;
      if (a.rope_table == nullptr) {
        // theta^(2i/d) depends on the pair only: once per pair, not once per (row, pair)
        for (int pair = tid; pair < pairs; pair += blockDim.x) {
          const float exponent = __fdiv_rn(static_cast<float>(2 * pair), static_cast<float>(a.rope.frequency_dim));
          denom_s[pair] = static_cast<float>(pow(static_cast<double>(a.rope.theta), static_cast<double>(exponent)));
        }
      }
      __syncthreads();
      // x * inv_rms * w and the rotation of a pair in one pass: a pair's two values are
      // read, scaled and rotated by the same thread
      // (row, pair) items over the block; the usual power-of-two pair count splits with a shift
      const int pair_shift = (pairs & (pairs - 1)) == 0 ? 31 - __clz(pairs) : -1;
      for (int i = tid; i < rows * pairs; i += blockDim.x) {
        const int r = pair_shift >= 0 ? i >> pair_shift : i / pairs;
        const int pair = i - r * pairs;
        float* xs = ks + r * kstride;
        float c, s;
        if (a.rope_table != nullptr) {
          // made once per launch: cos and sin of (row, pair) depend neither on the head nor on the sequence
          const float2 cs = __ldg(a.rope_table + (row_lo + r - a.rope_row0) * pairs + pair);
          c = cs.x, s = cs.y;
        } else {
          const float scaled_position = __fmul_rn(static_cast<float>(row_lo + r), a.rope.position_scale);
          const float angle = __fdiv_rn(scaled_position, denom_s[pair]);
          double sd, cd;
          sincos(static_cast<double>(angle), &sd, &cd);
          c = static_cast<float>(cd);
          s = static_cast<float>(sd);
        }
        const int i0 = a.rope.interleaved ? 2 * pair : pair;
        const int i1 = a.rope.interleaved ? 2 * pair + 1 : pair + pairs;
        const float inv = inv_s[r];
        const float first = __fmul_rn(__fmul_rn(xs[i0], inv), a.knorm_w[i0]);
        const float second = __fmul_rn(__fmul_rn(xs[i1], inv), a.knorm_w[i1]);
        xs[i0] = __fsub_rn(__fmul_rn(first, c), __fmul_rn(second, s));
        xs[i1] = __fadd_rn(__fmul_rn(first, s), __fmul_rn(second, c));
      }
      // dims the rotation leaves alone are still normalised
      for (int r = 0; r < rows; ++r)
        for (int c = 2 * pairs + tid; c < hd; c += blockDim.x)
          ks[r * kstride + c] = __fmul_rn(__fmul_rn(ks[r * kstride + c], inv_s[r]), a.knorm_w[c]);
      __syncthreads();
    }

    if (page_ok) {
      if (a.pool.dtype == KV_F32) {
        for (int i = tid; i < rows * (hd / 4); i += blockDim.x) {
          const int r = i >> (chunk_shift + 1), c = i & (hd / 4 - 1);
          reinterpret_cast<float4*>(reinterpret_cast<float*>(ktile) + (rin0 + r) * hd)[c] = reinterpret_cast<const float4*>(ks + r * kstride)[c];
        }
      } else if (a.pool.dtype == KV_BF16) {
        for (int i = tid; i < total; i += blockDim.x) {
          const int r = i >> chunk_shift, chunk = i & (chunks - 1);
          const float4 x0 = reinterpret_cast<const float4*>(ks + r * kstride + chunk * 8)[0];
          const float4 x1 = reinterpret_cast<const float4*>(ks + r * kstride + chunk * 8)[1];
          const uint4 w = make_uint4(uint32_t(f32_to_bf16_bits(x0.x)) | (uint32_t(f32_to_bf16_bits(x0.y)) << 16),
                                     uint32_t(f32_to_bf16_bits(x0.z)) | (uint32_t(f32_to_bf16_bits(x0.w)) << 16),
                                     uint32_t(f32_to_bf16_bits(x1.x)) | (uint32_t(f32_to_bf16_bits(x1.y)) << 16),
                                     uint32_t(f32_to_bf16_bits(x1.z)) | (uint32_t(f32_to_bf16_bits(x1.w)) << 16));
          *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(ktile) + bf16_elem_index(rin0 + r, chunk * 8, hd)) = w;
        }
      } else {
        uint32_t biggest = 0;
        // a full tile is put together in shared memory and leaves with 16-byte stores; a
        // partial one (first or last page of the append) is written in place, byte by byte
        const int tile_b = static_cast<int>(a.pool.tile_bytes);
        const bool full = rows == PAGE_TOKENS;
        for (int task = warp; task < 2 * rows; task += blockDim.x / 32) {
          const int is_v = task / rows, r = task % rows;
          const float* xs = is_v ? vs + r * hd : ks + r * kstride;
          uint8_t* tile = full ? stage + is_v * tile_b : (is_v ? vtile : ktile);
          if (hd == 256) biggest = max(biggest, store_u8_row<8>(tile, hd, is_v, rin0 + r, xs, lane));
          else if (hd == 128) biggest = max(biggest, store_u8_row<4>(tile, hd, is_v, rin0 + r, xs, lane));
          else biggest = max(biggest, store_u8_row<2>(tile, hd, is_v, rin0 + r, xs, lane));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) biggest = max(biggest, __shfl_xor_sync(0xffffffffu, biggest, off));
        if (lane == 0) atomicMax(&big_s, biggest);
        __syncthreads();
        if (full) {
          // the K tile and the V tile are neighbours in the page: one contiguous range
          const uint4* src = reinterpret_cast<const uint4*>(stage);
          uint4* dst = reinterpret_cast<uint4*>(ktile);
          for (int i = tid; i < 2 * tile_b / 16; i += blockDim.x) dst[i] = src[i];
        }
        // largest scale of the pool (positive floats order like their bit patterns)
        if (tid == 0 && a.pool.scale_max != nullptr && big_s > *reinterpret_cast<volatile uint32_t*>(a.pool.scale_max))
          atomicMax(a.pool.scale_max, big_s);
      }
    } else if (tid == 0) {
      atomicExch(a.status, DEV_ERR_BAD_PAGE);
    }
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

__global__ void __launch_bounds__(128) rope_table_kernel(float2* table, int64_t row0, int n_rows, RopeArgs rope) {
  const int pairs = rope.rope_dims / 2;
  const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i >= int64_t(n_rows) * pairs) return;
  const int64_t r = i / pairs;
  const int pair = static_cast<int>(i % pairs);
  // the float order of norm_rope_head
  const float exponent = __fdiv_rn(static_cast<float>(2 * pair), static_cast<float>(rope.frequency_dim));
  const float denom = static_cast<float>(pow(static_cast<double>(rope.theta), static_cast<double>(exponent)));
  const float scaled_position = __fmul_rn(static_cast<float>(row0 + r), rope.position_scale);
  const float angle = __fdiv_rn(scaled_position, denom);
  double sd, cd;
  sincos(static_cast<double>(angle), &sd, &cd);
  table[i] = make_float2(static_cast<float>(cd), static_cast<float>(sd));
}

cudaError_t launch_rope_table(float2* table, int64_t row0, int n_rows, const RopeArgs& rope, cudaStream_t stream) {
  const int64_t n = int64_t(n_rows) * (rope.rope_dims / 2);
  if (n <= 0) return cudaSuccess;
  rope_table_kernel<<<static_cast<unsigned>((n + 127) / 128), 128, 0, stream>>>(table, row0, n_rows, rope);
  return cudaGetLastError();
}

cudaError_t launch_append_rows(const AppendArgs& a, int n_seq, cudaStream_t stream) {
  const int hd = a.pool.head_dim;
  if (a.n_rows >= 4 && a.out_k == nullptr && (hd == 64 || hd == 128 || hd == 256)) {
    // bulk: one block per page tile; the first row may sit anywhere in its page, so one tile more
    dim3 grid(a.pool.kv_heads, (a.n_rows + PAGE_TOKENS - 1) / PAGE_TOKENS + 1, n_seq);
    // the kernel's carve-up: K rows, 1/rms per row, rope denominators (<= 128 pairs); V rows and a
    // tile pair being put together only where V is quantised
    size_t smem = (size_t(PAGE_TOKENS) * (hd + 4) + PAGE_TOKENS + 128) * sizeof(float);
    if (a.pool.dtype == KV_U8G32) smem += size_t(PAGE_TOKENS) * hd * sizeof(float) + 2 * size_t(a.pool.tile_bytes);
    if (!a.has_rope && a.pool.dtype != KV_U8G32) append_tiles_kernel<true><<<grid, 128, 0, stream>>>(a);
    else append_tiles_kernel<false><<<grid, 128, smem, stream>>>(a);
    return cudaGetLastError();
  }
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
