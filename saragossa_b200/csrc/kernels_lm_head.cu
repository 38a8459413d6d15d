// Greedy epilogue of a decode token: logits = W . x over a dense [vocab][hidden] weight (f32 or
// bf16) and their argmax, in one launch, without writing the logits. It closes the token on
// the device: the index lands in device memory where the next step reads it
// (encode_lm_head_argmax, src/metal_backend/lm_head.rs:288-337; argmax_blocks_f32 /
// argmax_finalize_f32, src/kernels.metal:8362-8440; CPU: src/sampling.rs:49-62). HBM-bound: the
// weight is read once (622 MB for 151 936 x 2048 bf16).
//
// Up to eight activation rows (the rows of a speculative verify,
// argmax_linear_biasless_rows_buffers, lm_head.rs:766-820) sit in shared memory and share the one
// pass over the weight.
//
// bf16 weights: a warp takes 16 vocabulary rows at a time and multiplies them with the (up to) 8
// activation rows on the tensor cores (mma.sync m16n8k16, f32 accumulators): with plain FMAs every
// 16 bytes of weight need 32 bytes of x per activation row from shared memory, which bounds four
// rows at a third of HBM speed. Each lane loads 16 contiguous bytes of a weight row straight from
// global memory; since a dot product does not care about the order of k, those 8 values serve as
// the k-slots of the lane in two products and the activation is read from shared memory in the same
// order (16 bytes per lane, row stride = 64 mod 128 bytes: no bank conflict). The f32 activation
// enters as hi + lo, two bf16 values (16 mantissa bits), accumulated separately. A row's logit
// does not depend on which other rows ride along: the verify form reproduces the one-row form bit
// for bit.
//
// f32 weights: a warp takes rows two at a time with 16-byte loads and FMAs. The best (value, index) of a block goes into one 64-bit atomicMax: the value as
// an order-preserving integer in the high word, the complemented index in the low word, so that
// equal values resolve to the LOWEST index like the reference. The block that finishes last
// decodes the winner and clears the two words for the next launch.
#include "mma_common.cuh"

namespace sgk {

constexpr int LM_THREADS = 256;
constexpr int LM_WARPS = LM_THREADS / 32;

__device__ __forceinline__ uint32_t ordered_bits(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float unordered_bits(uint32_t u) {
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// ---- f32 weights -------------------------------------------------------------------------
// Partial products of one weight row against R activation rows held in shared memory.
template <int R>
__device__ __forceinline__ void dot_row(const float* w, int64_t row, int hidden, const float* xs, int lane, float (&acc)[R]) {
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.0f;
  const float4* p = reinterpret_cast<const float4*>(w + row * hidden);
  for (int c = lane; c < hidden / 4; c += 32) {
    const float4 v = __ldcs(p + c);  // read once: streamed past L2's resident data
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float4 x = reinterpret_cast<const float4*>(xs + size_t(r) * hidden)[c];
      float t = acc[r];
      t = fmaf(v.x, x.x, t);
      t = fmaf(v.y, x.y, t);
      t = fmaf(v.z, x.z, t);
      t = fmaf(v.w, x.w, t);
      acc[r] = t;
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
}

__device__ __forceinline__ unsigned long long pack_key(float v, int64_t row) {
  return (static_cast<unsigned long long>(ordered_bits(v)) << 32) | (0xffffffffu - uint32_t(row));
}

// Programmatic dependent launch (see mma_common.cuh): no-ops in a launch without such a neighbour.
__device__ __forceinline__ void lm_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void lm_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <int R>
__global__ void __launch_bounds__(LM_THREADS) lm_head_argmax_f32_kernel(LmHeadArgs a) {
  extern __shared__ __align__(16) float xs[];
  __shared__ unsigned long long best_s[LM_WARPS][R];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (a.pdl_trigger) lm_pdl_trigger();
  if (a.pdl_wait) lm_pdl_wait();
  for (int i = tid; i < a.n_rows * a.hidden / 4; i += LM_THREADS)
    reinterpret_cast<float4*>(xs)[i] = reinterpret_cast<const float4*>(a.x)[i];
  for (int i = a.n_rows * a.hidden + tid; i < R * a.hidden; i += LM_THREADS) xs[i] = 0.0f;
  __syncthreads();
  unsigned long long best[R];  // 0 is below every real key (the low word of a key is never zero)
#pragma unroll
  for (int r = 0; r < R; ++r) best[r] = 0;
  const int64_t stride = int64_t(gridDim.x) * LM_WARPS * 2;
  for (int64_t row = (int64_t(blockIdx.x) * LM_WARPS + warp) * 2; row < a.vocab; row += stride) {
    float v0[R], v1[R];
    const bool two = row + 1 < a.vocab;
    dot_row<R>(reinterpret_cast<const float*>(a.w), row, a.hidden, xs, lane, v0);
    dot_row<R>(reinterpret_cast<const float*>(a.w), two ? row + 1 : row, a.hidden, xs, lane, v1);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const unsigned long long k0 = pack_key(v0[r], row), k1 = pack_key(v1[r], two ? row + 1 : row);
      best[r] = k0 > best[r] ? k0 : best[r];
      best[r] = k1 > best[r] ? k1 : best[r];
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) best_s[warp][r] = best[r];
  }
  __syncthreads();
  if (tid < a.n_rows) {
    unsigned long long b = best_s[0][tid];
    for (int w = 1; w < LM_WARPS; ++w) b = best_s[w][tid] > b ? best_s[w][tid] : b;
    atomicMax(a.keys + tid, b);
    __threadfence();
  }
  __syncthreads();
  __shared__ unsigned int last_s;
  if (tid == 0) last_s = atomicAdd(a.counter, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last_s && tid < a.n_rows) {
    __threadfence();
    const unsigned long long win = atomicExch(a.keys + tid, 0ull);
    const int32_t winner = static_cast<int32_t>(0xffffffffu - uint32_t(win & 0xffffffffu)) + a.index_offset;
    a.index_out[tid] = winner;
    if (a.index_mirror) {   // the host's copy, written from here: no copy node behind the launch
      a.index_mirror[tid] = winner;
      __threadfence_system();
    }
    if (a.value_out) a.value_out[tid] = unordered_bits(uint32_t(win >> 32));
    if (tid == 0) *a.counter = 0;
  }
}

// ---- bf16 weights on the tensor cores ---------------------------------------------------
#ifndef SGK_LM_UNROLL
#define SGK_LM_UNROLL 8
#endif
#ifndef SGK_LM_BLOCKS_PER_SM
#define SGK_LM_BLOCKS_PER_SM 2
#endif
constexpr int LM_UNROLL = SGK_LM_UNROLL;     // 32-wide k chunks in flight per lane (2 x 16-byte loads each)
constexpr int LM_BLOCKS_PER_SM = SGK_LM_BLOCKS_PER_SM;
constexpr int LM_KPAD = 32 * LM_UNROLL;      // the activation rows are zero-padded to this many values

__host__ __device__ inline int lm_x_stride_bytes(int hidden) {
  const int padded = (hidden + LM_KPAD - 1) / LM_KPAD * LM_KPAD * 2;  // a multiple of 256 bytes
  return padded + 64;                                                 // = 64 mod 128: rows g and g+1 hit different banks
}

__global__ void __launch_bounds__(LM_THREADS, LM_BLOCKS_PER_SM) lm_head_argmax_bf16_kernel(LmHeadArgs a) {
  extern __shared__ __align__(16) unsigned char lm_smem[];
  __shared__ unsigned long long best_s[LM_WARPS][8];
  __shared__ unsigned int last_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if (a.pdl_trigger) lm_pdl_trigger();
  if (a.pdl_wait) lm_pdl_wait();   // x comes from the launch before
  const int stride = lm_x_stride_bytes(a.hidden);
  unsigned char* xhi = lm_smem;
  unsigned char* xlo = lm_smem + size_t(a.n_rows) * stride;
  // x -> hi + lo (bf16 each), zero padding behind every row
  const int per_row = stride / 2;
  for (int i = tid; i < a.n_rows * per_row; i += LM_THREADS) {
    const int r = i / per_row, c = i - r * per_row;
    const float v = c < a.hidden ? a.x[size_t(r) * a.hidden + c] : 0.0f;
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    const __nv_bfloat16 l = __float2bfloat16_rn(v - __bfloat162float(h));
    reinterpret_cast<__nv_bfloat16*>(xhi)[i] = h;
    reinterpret_cast<__nv_bfloat16*>(xlo)[i] = l;
  }
  __syncthreads();
  const bool has_col = g < a.n_rows;  // column g of the product is activation row g
  const unsigned char* bh = xhi + (has_col ? g : 0) * stride + t * 16;
  const unsigned char* bl = xlo + (has_col ? g : 0) * stride + t * 16;
  const int chunks = (a.hidden + 31) / 32;
  unsigned long long best0 = 0, best1 = 0;  // activation rows 2t and 2t+1; 0 is below every real key
  const int64_t tiles = (a.vocab + 15) / 16;
  // Every warp takes the same number of whole 16-row tiles; the tiles left over (151 936 rows are
  // 4.01 tiles per warp: a fifth tile for a few warps would run, pass after pass of DRAM round
  // trips, while the rest of the GPU is done) are shared out among the blocks afterwards, the
  // eight warps of a block splitting the columns of one tile.
  const int64_t n_warps = int64_t(gridDim.x) * LM_WARPS;
  const int64_t whole = a.whole_tiles;
  for (int64_t tile = int64_t(blockIdx.x) * LM_WARPS + warp; tile < whole; tile += n_warps) {
    const int64_t r0 = tile * 16 + g, r1 = r0 + 8;
    const uint16_t* w0 = reinterpret_cast<const uint16_t*>(a.w) + (r0 < a.vocab ? r0 : a.vocab - 1) * a.hidden + t * 8;
    const uint16_t* w1 = reinterpret_cast<const uint16_t*>(a.w) + (r1 < a.vocab ? r1 : a.vocab - 1) * a.hidden + t * 8;
    float h1[4] = {0, 0, 0, 0}, h2[4] = {0, 0, 0, 0}, l1[4] = {0, 0, 0, 0}, l2[4] = {0, 0, 0, 0};
    for (int c0 = 0; c0 < chunks; c0 += LM_UNROLL) {
      uint4 A0[LM_UNROLL], A1[LM_UNROLL];
#pragma unroll
      for (int u = 0; u < LM_UNROLL; ++u) {
        const int k = (c0 + u) * 32;
        const bool valid = k + t * 8 < a.hidden;
        A0[u] = valid ? __ldcs(reinterpret_cast<const uint4*>(w0 + k)) : make_uint4(0, 0, 0, 0);
        A1[u] = valid ? __ldcs(reinterpret_cast<const uint4*>(w1 + k)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < LM_UNROLL; ++u) {
        const int kb = (c0 + u) * 64;
        uint4 xh = make_uint4(0, 0, 0, 0), xl = make_uint4(0, 0, 0, 0);
        if (has_col) {
          xh = *reinterpret_cast<const uint4*>(bh + kb);
          xl = *reinterpret_cast<const uint4*>(bl + kb);
        }
        mma_bf16(h1, A0[u].x, A1[u].x, A0[u].y, A1[u].y, xh.x, xh.y);
        mma_bf16(l1, A0[u].x, A1[u].x, A0[u].y, A1[u].y, xl.x, xl.y);
        mma_bf16(h2, A0[u].z, A1[u].z, A0[u].w, A1[u].w, xh.z, xh.w);
        mma_bf16(l2, A0[u].z, A1[u].z, A0[u].w, A1[u].w, xl.z, xl.w);
      }
    }
    // c0,c1: vocabulary row r0 against activation rows 2t, 2t+1; c2,c3: row r1
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (h1[i] + h2[i]) + (l1[i] + l2[i]);
    if (r0 < a.vocab) {
      const unsigned long long k0 = pack_key(v[0], r0), k1 = pack_key(v[1], r0);
      best0 = k0 > best0 ? k0 : best0;
      best1 = k1 > best1 ? k1 : best1;
    }
    if (r1 < a.vocab) {
      const unsigned long long k0 = pack_key(v[2], r1), k1 = pack_key(v[3], r1);
      best0 = k0 > best0 ? k0 : best0;
      best1 = k1 > best1 ? k1 : best1;
    }
  }
  // the tiles left over: one per block and turn, warp w takes the 32-column chunks w, w + 8, ...
  __shared__ float left_s[LM_WARPS][16][8];
  unsigned long long left_best = 0;   // threads 0..127: (row tid / 8 of the tile, activation row tid % 8)
  for (int64_t tile = whole + blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t r0 = tile * 16 + g, r1 = r0 + 8;
    const uint16_t* w0 = reinterpret_cast<const uint16_t*>(a.w) + (r0 < a.vocab ? r0 : a.vocab - 1) * a.hidden + t * 8;
    const uint16_t* w1 = reinterpret_cast<const uint16_t*>(a.w) + (r1 < a.vocab ? r1 : a.vocab - 1) * a.hidden + t * 8;
    float h1[4] = {0, 0, 0, 0}, h2[4] = {0, 0, 0, 0}, l1[4] = {0, 0, 0, 0}, l2[4] = {0, 0, 0, 0};
#pragma unroll 4
    for (int c = warp; c < chunks; c += LM_WARPS) {
      const int k = c * 32;
      const bool valid = k + t * 8 < a.hidden;
      const uint4 A0 = valid ? __ldcs(reinterpret_cast<const uint4*>(w0 + k)) : make_uint4(0, 0, 0, 0);
      const uint4 A1 = valid ? __ldcs(reinterpret_cast<const uint4*>(w1 + k)) : make_uint4(0, 0, 0, 0);
      uint4 xh = make_uint4(0, 0, 0, 0), xl = make_uint4(0, 0, 0, 0);
      if (has_col) {
        xh = *reinterpret_cast<const uint4*>(bh + c * 64);
        xl = *reinterpret_cast<const uint4*>(bl + c * 64);
      }
      mma_bf16(h1, A0.x, A1.x, A0.y, A1.y, xh.x, xh.y);
      mma_bf16(l1, A0.x, A1.x, A0.y, A1.y, xl.x, xl.y);
      mma_bf16(h2, A0.z, A1.z, A0.w, A1.w, xh.z, xh.w);
      mma_bf16(l2, A0.z, A1.z, A0.w, A1.w, xl.z, xl.w);
    }
    __syncthreads();   // the turn before this one has been added up
    left_s[warp][g][2 * t] = (h1[0] + h2[0]) + (l1[0] + l2[0]);
    left_s[warp][g][2 * t + 1] = (h1[1] + h2[1]) + (l1[1] + l2[1]);
    left_s[warp][g + 8][2 * t] = (h1[2] + h2[2]) + (l1[2] + l2[2]);
    left_s[warp][g + 8][2 * t + 1] = (h1[3] + h2[3]) + (l1[3] + l2[3]);
    __syncthreads();
    if (tid < 128) {
      const int row = tid >> 3, arow = tid & 7;
      float sum = left_s[0][row][arow];
#pragma unroll
      for (int w = 1; w < LM_WARPS; ++w) sum += left_s[w][row][arow];
      const int64_t r = tile * 16 + row;
      if (r < a.vocab && arow < a.n_rows) {
        const unsigned long long key = pack_key(sum, r);
        left_best = key > left_best ? key : left_best;
      }
    }
  }
  // threads 0..127 hold the left-over tiles' best per (row, activation row): best per activation row
  __shared__ unsigned long long left_best_s[4][8];
#pragma unroll
  for (int off = 8; off < 32; off <<= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, left_best, off);
    left_best = o > left_best ? o : left_best;
  }
  if (tid < 128 && lane < 8) left_best_s[warp][lane] = left_best;
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    const unsigned long long o0 = __shfl_xor_sync(0xffffffffu, best0, off), o1 = __shfl_xor_sync(0xffffffffu, best1, off);
    best0 = o0 > best0 ? o0 : best0;
    best1 = o1 > best1 ? o1 : best1;
  }
  if (lane < 4) {
    best_s[warp][2 * lane] = best0;
    best_s[warp][2 * lane + 1] = best1;
  }
  __syncthreads();
  if (tid < a.n_rows) {
    unsigned long long b = best_s[0][tid];
    for (int w = 1; w < LM_WARPS; ++w) b = best_s[w][tid] > b ? best_s[w][tid] : b;
    for (int w = 0; w < 4; ++w) b = left_best_s[w][tid] > b ? left_best_s[w][tid] : b;
    atomicMax(a.keys + tid, b);
    __threadfence();
  }
  __syncthreads();
  if (tid == 0) last_s = atomicAdd(a.counter, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last_s && tid < a.n_rows) {
    __threadfence();
    const unsigned long long win = atomicExch(a.keys + tid, 0ull);
    const int32_t winner = static_cast<int32_t>(0xffffffffu - uint32_t(win & 0xffffffffu)) + a.index_offset;
    a.index_out[tid] = winner;
    if (a.index_mirror) {   // the host's copy, written from here: no copy node behind the launch
      a.index_mirror[tid] = winner;
      __threadfence_system();
    }
    if (a.value_out) a.value_out[tid] = unordered_bits(uint32_t(win >> 32));
    if (tid == 0) *a.counter = 0;
  }
}

template <int R>
static cudaError_t launch_r(const LmHeadArgs& a, int blocks, size_t smem, cudaStream_t stream) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(lm_head_argmax_f32_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
  }
  ChainLaunch l(dim3(blocks), dim3(LM_THREADS), smem, stream, a.pdl_wait != 0);
  return cudaLaunchKernelEx(&l.cfg, lm_head_argmax_f32_kernel<R>, a);
}

// ---- token feed: the next token's input row, looked up by an index that lives on the device --
// embed_gather_dense_from_u32_f32 (src/kernels.metal:308-325): out = table[token] * scale, optionally
// rounded to bf16 (RNE) and widened again; a token outside the table writes nothing.
template <bool BF16>
__global__ void embed_gather_kernel(const void* table, const int32_t* index, int64_t vocab, int hidden, float scale,
                                    int recast_bf16, float* out, int pdl_trigger, int pdl_wait) {
  if (pdl_trigger) lm_pdl_trigger();
  if (pdl_wait) lm_pdl_wait();   // the index is what the previous token's epilogue wrote
  const int64_t token = *index;
  if (token < 0 || token >= vocab) return;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) {
    const float w = BF16 ? __uint_as_float(uint32_t(reinterpret_cast<const uint16_t*>(table)[token * hidden + i]) << 16)
                         : reinterpret_cast<const float*>(table)[token * hidden + i];
    const float v = __fmul_rn(w, scale);
    out[i] = recast_bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : v;
  }
}

cudaError_t launch_embed_gather(const void* table, int table_bf16, const int32_t* index, int64_t vocab, int hidden,
                                float scale, int recast_bf16, float* out, int pdl_trigger, int pdl_wait,
                                cudaStream_t stream) {
  const int blocks = (hidden + 255) / 256 < 64 ? (hidden + 255) / 256 : 64;
  ChainLaunch l(dim3(blocks), dim3(256), 0, stream, pdl_wait != 0);
  return table_bf16 ? cudaLaunchKernelEx(&l.cfg, embed_gather_kernel<true>, table, index, vocab, hidden, scale,
                                         recast_bf16, out, pdl_trigger, pdl_wait)
                    : cudaLaunchKernelEx(&l.cfg, embed_gather_kernel<false>, table, index, vocab, hidden, scale,
                                         recast_bf16, out, pdl_trigger, pdl_wait);
}


// ---- affine-quantised weights (u4 / u8 codes, bf16 scale and bias per group) -----------------
// encode_affine_argmax_qmv_fast (src/metal_backend/lm_head.rs:934-990, kernel
// affine_argmax_qmv_fast_u4_gs64_f32) and the dequantisation rule code * scale + bias
// (src/quantization.rs:173-179). HBM-bound on a quarter (u4) or half (u8) of the dense bytes, so
// the products must cost next to nothing: a code becomes the fp16 SUBNORMAL code * 2^-24 by
// dropping it into the low bits of a zero half (one byte permute or one shift-and-mask for two
// codes, exact, nothing to subtract), a warp multiplies 16 vocabulary rows x 64 columns (one
// quantisation group, so one scale per row) with the activation rows on the tensor cores
// (m16n8k16, fp16 x fp16 -> f32, x as hi + lo halves), and the group's scale and bias are applied
// to the group sums in f32:  logit = sum_g scale_g * (codes_g . x_g) + bias_g * sum(x_g).
// A lane holds 16 consecutive columns of a group for rows g and g+8; as a dot product does not care
// about the order of k, the lane's codes serve as its k-slots in the order the unpacking yields
// them and the activation is laid out in shared memory in that same order.
__device__ __forceinline__ void mma_f16_lm(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 64-column blocks in flight per lane (independent accumulators): 16 bytes of codes per row and block at 8 bits, 8 at 4
template <int BITS> struct LmqGroups { static constexpr int N = BITS == 8 ? 6 : 8; };
constexpr float LMQ_UNIT_INV = 16777216.0f;   // 2^24: a code enters as code * 2^-24

// column that sits at position p of a lane's 16 slots (u4: the unpacking yields (c0,c4),(c1,c5),(c2,c6),(c3,c7)
// per 8-column word; u8: (c0,c1),(c2,c3) per 4-column word = natural order)
template <int BITS>
__device__ __forceinline__ int lmq_slot_column(int p) {
  if (BITS == 8) return p;
  const int word = p >> 3, q = p & 7;
  return word * 8 + (q >> 1) + (q & 1) * 4;
}

__host__ __device__ inline int lmq_x_stride_bytes(int hidden) { return hidden * 2 + 64; }

template <int BITS>
__global__ void __launch_bounds__(LM_THREADS, 2) lm_head_argmax_affine_kernel(LmHeadAffineArgs a) {
  extern __shared__ __align__(16) unsigned char lm_smem[];
  __shared__ unsigned long long best_s[LM_WARPS][8];
  __shared__ unsigned int last_s;
  __shared__ float red_s[LM_WARPS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if (a.pdl_trigger) lm_pdl_trigger();
  if (a.pdl_wait) lm_pdl_wait();
  const int stride = lmq_x_stride_bytes(a.hidden);
  const int blocks64 = a.hidden / 64;               // 64-column blocks of a row
  const int groups = a.hidden / a.w.group_size;     // quantisation groups of a row
  const int per_group = a.w.group_size / 64;        // blocks per group (1 or 2)
  unsigned char* xhi = lm_smem;
  unsigned char* xlo = lm_smem + size_t(a.n_rows) * stride;
  float* xsum = reinterpret_cast<float*>(lm_smem + size_t(2) * a.n_rows * stride);   // [n_rows][blocks64]
  // The activation is scaled by a power of two that puts its largest value in the middle of the
  // fp16 range (the same in every block: it depends on x only).
  float big = 0.0f;
  for (int i = tid; i < a.n_rows * a.hidden; i += LM_THREADS) big = fmaxf(big, fabsf(a.x[i]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
  if (lane == 0) red_s[warp] = big;
  __syncthreads();
  big = red_s[0];
  for (int w = 1; w < LM_WARPS; ++w) big = fmaxf(big, red_s[w]);
  int e = static_cast<int>((__float_as_uint(big) >> 23) & 0xffu) - 127;
  e = max(-100, min(100, e));
  const float xscale = exp2f(static_cast<float>(8 - e)), inv_xscale = exp2f(static_cast<float>(e - 8)) * LMQ_UNIT_INV;
  // x -> fp16 hi + lo in the slot order of the lanes; per 64-column block the sum of what the tensor core sees
  for (int i = tid; i < a.n_rows * a.hidden; i += LM_THREADS) {
    const int r = i / a.hidden, p = i - r * a.hidden;
    const int col = (p & ~15) + lmq_slot_column<BITS>(p & 15);
    const float v = a.x[size_t(r) * a.hidden + col] * xscale;
    const __half h = __float2half_rn(v);
    const __half l = __float2half_rn(v - __half2float(h));
    reinterpret_cast<__half*>(xhi + size_t(r) * stride)[p] = h;
    reinterpret_cast<__half*>(xlo + size_t(r) * stride)[p] = l;
  }
  __syncthreads();
  for (int i = tid; i < a.n_rows * blocks64; i += LM_THREADS) {
    const int r = i / blocks64, b = i - r * blocks64;
    const __half* ph = reinterpret_cast<const __half*>(xhi + size_t(r) * stride) + b * 64;
    const __half* pl = reinterpret_cast<const __half*>(xlo + size_t(r) * stride) + b * 64;
    float sum = 0.0f;
    for (int c = 0; c < 64; ++c) sum += __half2float(ph[c]) + __half2float(pl[c]);
    xsum[i] = sum * (1.0f / LMQ_UNIT_INV);   // in the unit of the code products (a code enters as code * 2^-24)
  }
  __syncthreads();
  // Up to four activation rows: column 2r of the product is the hi half of row r, column 2r+1 its lo
  // half, so ONE product per k-step serves both (lane t's two C columns then belong to row t). Five
  // to eight rows: column g is row g and hi and lo take a product each.
  const bool paired = a.n_rows <= 4;
  const int act = paired ? g >> 1 : g;                 // activation row this lane's B column belongs to
  const bool has_col = act < a.n_rows;
  const unsigned char* bh = (paired && (g & 1) ? xlo : xhi) + (has_col ? act : 0) * stride + t * 32;
  const unsigned char* bl = xlo + (has_col ? act : 0) * stride + t * 32;
  // activation rows of this lane's two C columns
  const int c_row0 = paired ? t : 2 * t, c_row1 = paired ? t : 2 * t + 1;
  const float* xs0 = xsum + (c_row0 < a.n_rows ? c_row0 : 0) * blocks64;
  const float* xs1 = xsum + (c_row1 < a.n_rows ? c_row1 : 0) * blocks64;
  constexpr int ROW_WORDS_PER_BLOCK = 64 * BITS / 32;   // u32 words of a row per 64-column block
  constexpr int LANE_WORDS = 16 * BITS / 32;            // words a lane holds per row per block (2 or 4)
  const int64_t row_words = int64_t(a.hidden) * BITS / 32;
  constexpr int LMQ_GROUPS = LmqGroups<BITS>::N;
  unsigned long long best0 = 0, best1 = 0;
  const int64_t tiles = (a.vocab + 15) / 16;
  for (int64_t tile = int64_t(blockIdx.x) * LM_WARPS + warp; tile < tiles; tile += int64_t(gridDim.x) * LM_WARPS) {
    const int64_t r0 = tile * 16 + g, r1 = r0 + 8;
    const int64_t rr0 = r0 < a.vocab ? r0 : a.vocab - 1, rr1 = r1 < a.vocab ? r1 : a.vocab - 1;
    const uint32_t* w0 = a.w.packed + rr0 * row_words + t * LANE_WORDS;
    const uint32_t* w1 = a.w.packed + rr1 * row_words + t * LANE_WORDS;
    const uint16_t* s0 = a.w.scales + rr0 * groups;
    const uint16_t* s1 = a.w.scales + rr1 * groups;
    const uint16_t* z0 = a.w.biases + rr0 * groups;
    const uint16_t* z1 = a.w.biases + rr1 * groups;
    float v[4] = {0.f, 0.f, 0.f, 0.f};   // (r0, act 2t), (r0, act 2t+1), (r1, act 2t), (r1, act 2t+1)
    for (int b0 = 0; b0 < blocks64; b0 += LMQ_GROUPS) {
      uint32_t A0[LMQ_GROUPS][LANE_WORDS], A1[LMQ_GROUPS][LANE_WORDS];
#pragma unroll
      for (int u = 0; u < LMQ_GROUPS; ++u) {
        const bool valid = b0 + u < blocks64;
        if (LANE_WORDS == 4) {
          const uint4 p0 = valid ? __ldcs(reinterpret_cast<const uint4*>(w0 + (b0 + u) * ROW_WORDS_PER_BLOCK)) : make_uint4(0, 0, 0, 0);
          const uint4 p1 = valid ? __ldcs(reinterpret_cast<const uint4*>(w1 + (b0 + u) * ROW_WORDS_PER_BLOCK)) : make_uint4(0, 0, 0, 0);
          A0[u][0] = p0.x, A0[u][1] = p0.y, A0[u][2 % LANE_WORDS] = p0.z, A0[u][3 % LANE_WORDS] = p0.w;
          A1[u][0] = p1.x, A1[u][1] = p1.y, A1[u][2 % LANE_WORDS] = p1.z, A1[u][3 % LANE_WORDS] = p1.w;
        } else {
          const uint2 p0 = valid ? __ldcs(reinterpret_cast<const uint2*>(w0 + (b0 + u) * ROW_WORDS_PER_BLOCK)) : make_uint2(0, 0);
          const uint2 p1 = valid ? __ldcs(reinterpret_cast<const uint2*>(w1 + (b0 + u) * ROW_WORDS_PER_BLOCK)) : make_uint2(0, 0);
          A0[u][0] = p0.x, A0[u][1] = p0.y;
          A1[u][0] = p1.x, A1[u][1] = p1.y;
        }
      }
      // the blocks' scales and biases, asked for with the codes (each is read once: a DRAM round trip)
      uint16_t sr0[LMQ_GROUPS], sr1[LMQ_GROUPS], zr0[LMQ_GROUPS], zr1[LMQ_GROUPS];
#pragma unroll
      for (int u = 0; u < LMQ_GROUPS; ++u) {
        const int grp = min(b0 + u, blocks64 - 1) / per_group;
        sr0[u] = s0[grp], sr1[u] = s1[grp], zr0[u] = z0[grp], zr1[u] = z1[grp];
      }
#pragma unroll
      for (int u = 0; u < LMQ_GROUPS; ++u) {
        if (b0 + u >= blocks64) break;   // uniform over the warp
        const int blk = b0 + u;
        uint4 xh[2], xl[2];
        xh[0] = xh[1] = xl[0] = xl[1] = make_uint4(0, 0, 0, 0);
        if (has_col) {
          xh[0] = *reinterpret_cast<const uint4*>(bh + blk * 128);
          xh[1] = *reinterpret_cast<const uint4*>(bh + blk * 128 + 16);
          if (!paired) {
            xl[0] = *reinterpret_cast<const uint4*>(bl + blk * 128);
            xl[1] = *reinterpret_cast<const uint4*>(bl + blk * 128 + 16);
          }
        }
        const uint32_t bhr[8] = {xh[0].x, xh[0].y, xh[0].z, xh[0].w, xh[1].x, xh[1].y, xh[1].z, xh[1].w};
        const uint32_t blr[8] = {xl[0].x, xl[0].y, xl[0].z, xl[0].w, xl[1].x, xl[1].y, xl[1].z, xl[1].w};
        float ch[4] = {0.f, 0.f, 0.f, 0.f}, cl[4] = {0.f, 0.f, 0.f, 0.f};
        // four k-steps: slots [4j, 4j+4) of the lane, i.e. B registers 2j and 2j+1
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a0, a1, a2, a3;
          if (BITS == 8) {
            a0 = __byte_perm(A0[u][j % LANE_WORDS], 0, 0x4140), a2 = __byte_perm(A0[u][j % LANE_WORDS], 0, 0x4342);
            a1 = __byte_perm(A1[u][j % LANE_WORDS], 0, 0x4140), a3 = __byte_perm(A1[u][j % LANE_WORDS], 0, 0x4342);
          } else {
            const uint32_t p0 = A0[u][(j >> 1) % LANE_WORDS] >> ((j & 1) * 8), p1 = A1[u][(j >> 1) % LANE_WORDS] >> ((j & 1) * 8);
            a0 = p0 & 0x000f000fu, a2 = (p0 >> 4) & 0x000f000fu;
            a1 = p1 & 0x000f000fu, a3 = (p1 >> 4) & 0x000f000fu;
          }
          mma_f16_lm(ch, a0, a1, a2, a3, bhr[2 * j], bhr[2 * j + 1]);
          if (!paired) mma_f16_lm(cl, a0, a1, a2, a3, blr[2 * j], blr[2 * j + 1]);
        }
        const float sc0 = __uint_as_float(uint32_t(sr0[u]) << 16), sc1 = __uint_as_float(uint32_t(sr1[u]) << 16);
        const float bi0 = __uint_as_float(uint32_t(zr0[u]) << 16), bi1 = __uint_as_float(uint32_t(zr1[u]) << 16);
        const float x0 = xs0[blk], x1 = xs1[blk];
        if (paired) {   // the two columns are hi and lo of one activation row
          v[0] += sc0 * (ch[0] + ch[1]) + bi0 * x0;
          v[2] += sc1 * (ch[2] + ch[3]) + bi1 * x0;
        } else {
          v[0] += sc0 * (ch[0] + cl[0]) + bi0 * x0;
          v[1] += sc0 * (ch[1] + cl[1]) + bi0 * x1;
          v[2] += sc1 * (ch[2] + cl[2]) + bi1 * x0;
          v[3] += sc1 * (ch[3] + cl[3]) + bi1 * x1;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= inv_xscale;   // out of the code unit and the activation's power of two
    if (r0 < a.vocab) {
      const unsigned long long k0 = pack_key(v[0], r0), k1 = pack_key(v[1], r0);
      best0 = k0 > best0 ? k0 : best0;
      best1 = k1 > best1 ? k1 : best1;
    }
    if (r1 < a.vocab) {
      const unsigned long long k0 = pack_key(v[2], r1), k1 = pack_key(v[3], r1);
      best0 = k0 > best0 ? k0 : best0;
      best1 = k1 > best1 ? k1 : best1;
    }
  }
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    const unsigned long long o0 = __shfl_xor_sync(0xffffffffu, best0, off), o1 = __shfl_xor_sync(0xffffffffu, best1, off);
    best0 = o0 > best0 ? o0 : best0;
    best1 = o1 > best1 ? o1 : best1;
  }
  if (lane < 4) {
    // paired: lane t's best0 is activation row t; else best0 / best1 are rows 2t / 2t+1
    if (paired) {
      best_s[warp][lane] = best0;
    } else {
      best_s[warp][2 * lane] = best0;
      best_s[warp][2 * lane + 1] = best1;
    }
  }
  __syncthreads();
  if (tid < a.n_rows) {
    unsigned long long b = best_s[0][tid];
    for (int w = 1; w < LM_WARPS; ++w) b = best_s[w][tid] > b ? best_s[w][tid] : b;
    atomicMax(a.keys + tid, b);
    __threadfence();
  }
  __syncthreads();
  if (tid == 0) last_s = atomicAdd(a.counter, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last_s && tid < a.n_rows) {
    __threadfence();
    const unsigned long long win = atomicExch(a.keys + tid, 0ull);
    const int32_t winner = static_cast<int32_t>(0xffffffffu - uint32_t(win & 0xffffffffu)) + a.index_offset;
    a.index_out[tid] = winner;
    if (a.index_mirror) {   // the host's copy, written from here: no copy node behind the launch
      a.index_mirror[tid] = winner;
      __threadfence_system();
    }
    if (a.value_out) a.value_out[tid] = unordered_bits(uint32_t(win >> 32));
    if (tid == 0) *a.counter = 0;
  }
}

// ---- the same epilogue, software-pipelined (hidden a multiple of 64 * P columns) --------------
// The kernel above asks for six blocks of codes, works through them and only then asks again; a
// profile showed about 130 warp instructions per 16 x 64 block (u16 loads of every scale and bias,
// an integer division per block, 64-bit address arithmetic per load) and the issue slots half
// busy at 46 % of the DRAM rate: it could not have doubled its speed. Here a pass is P blocks;
// the codes, scales and biases of pass i+1 are asked for before pass i is multiplied (two register
// buffers, also across the end of a 16-row tile), a pass's scales and biases arrive as one 4 to
// 16-byte load per row, addresses advance by increments, and the group of a block is known at
// compile time. Same products, same order of the f32 additions: bit-identical logits.
// Measured on 151 936 x 2 560, one row: 8 bits 99.9 -> 78.6 us (0.80 of the copy peak), 4 bits
// 95 -> 73 us. Both widths take about the same time: the limit is the warps' instruction stream
// per 16 x 64 block (unpack, four chained products, scale and bias: ~66 instructions whose
// latencies four warps per scheduler do not cover), not DRAM. Built, measured and removed, none
// faster at 8 bits: the codes through shared memory by bulk copies, as whole rows into a ring
// shared by the block (98.7 us: a block-wide barrier per tile) or as 256 to 512-byte pieces into
// per-warp rings (84.4 us with eight warps per SM, 85.6 with sixteen; 68.5 at 4 bits); an L2
// prefetch cursor three passes ahead of the loads (95.5 us); tiles handed out by an atomic counter
// instead of whole rounds plus shared left-overs (no change).
template <int BITS, int P, int PG>
struct LmqPass {
  static constexpr int LW = 16 * BITS / 32;       // words of a row a lane holds per block
  static constexpr int NS = P / PG;               // scales (and biases) of a row per pass
  static constexpr int MW = NS >= 2 ? NS / 2 : 1; // 32-bit words they come in
  uint32_t a0[P][LW], a1[P][LW];
  uint32_t s0[MW], s1[MW], z0[MW], z1[MW];
};

template <int N>
__device__ __forceinline__ void lmq_load_words(const void* p, uint32_t (&out)[N]) {
  if (N == 4) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(p));
    out[0] = v.x, out[1 % N] = v.y, out[2 % N] = v.z, out[3 % N] = v.w;
  } else if (N == 2) {
    const uint2 v = __ldcs(reinterpret_cast<const uint2*>(p));
    out[0] = v.x, out[1 % N] = v.y;
  } else {
    out[0] = __ldcs(reinterpret_cast<const uint32_t*>(p));
  }
}

// bf16 number `i` of a packed array of 32-bit words, as f32
template <int N>
__device__ __forceinline__ float lmq_meta(const uint32_t (&w)[N], int i) {
  const uint32_t word = w[(i >> 1) % N];
  return __uint_as_float((i & 1) ? (word & 0xffff0000u) : (word << 16));
}

template <int BITS, int P, int PG, bool PAIRED>
__global__ void __launch_bounds__(LM_THREADS, 2) lm_head_argmax_affine_pipe_kernel(LmHeadAffineArgs a) {
  extern __shared__ __align__(16) unsigned char lm_smem[];
  __shared__ unsigned long long best_s[LM_WARPS][8];
  __shared__ unsigned int last_s;
  __shared__ float red_s[LM_WARPS];
  using Pass = LmqPass<BITS, P, PG>;
  constexpr int LW = Pass::LW, NS = Pass::NS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if (a.pdl_trigger) lm_pdl_trigger();
  const int stride = lmq_x_stride_bytes(a.hidden);
  const int blocks64 = a.hidden / 64;
  const int groups = a.hidden / (64 * PG);
  constexpr int RW = 64 * BITS / 32;                    // u32 words of a row per 64-column block
  const int64_t row_words = int64_t(a.hidden) * BITS / 32;
  const int passes = blocks64 / P;
  const int64_t tiles = (a.vocab + 15) / 16;
  const int64_t n_warps = int64_t(gridDim.x) * LM_WARPS;
  const int64_t bias_delta = a.w.biases - a.w.scales;   // in elements; the two arrays have one shape

  // Tiles of 16 rows. 151 936 rows are 4.01 tiles per warp: whichever way whole tiles are handed
  // out, a few warps work through a fifth one (ten passes, each a DRAM round trip) while the
  // rest of the GPU is done. So a warp takes the same number of whole tiles as every other warp
  // (tile = its number + round * warps), and the tiles left over are shared out among the blocks
  // afterwards, the eight warps of a block splitting the columns of one tile. The load cursor
  // is one pass ahead of the compute cursor, also from one tile to the next.
  const int64_t rounds = a.whole_tiles / n_warps;
  const int64_t first_tile = int64_t(blockIdx.x) * LM_WARPS + warp;
  const int64_t end_tile = first_tile + rounds * n_warps;   // first tile this warp does not take
  int64_t l_tile = rounds > 0 ? first_tile : end_tile;
  int l_pass = 0;
  const uint32_t* wp = nullptr;   // codes of row r0 at the cursor's pass (this lane's 16 columns)
  const uint16_t* sp = nullptr;   // scales of row r0 at the cursor's pass
  int32_t w_delta = 0, s_delta = 0;   // from row r0 to row r1 (0 where r1 is past the last row)
  int64_t c_tile = l_tile;
  auto load = [&](Pass& b) {
    if (l_pass == 0) {
      const int64_t r0 = l_tile * 16 + g;
      const int64_t rr0 = r0 < a.vocab ? r0 : a.vocab - 1, rr1 = r0 + 8 < a.vocab ? r0 + 8 : a.vocab - 1;
      wp = a.w.packed + rr0 * row_words + t * LW;
      sp = a.w.scales + rr0 * groups;
      w_delta = static_cast<int32_t>((rr1 - rr0) * row_words);
      s_delta = static_cast<int32_t>((rr1 - rr0) * groups);
    }
#pragma unroll
    for (int u = 0; u < P; ++u) {
      lmq_load_words<LW>(wp + u * RW, b.a0[u]);
      lmq_load_words<LW>(wp + w_delta + u * RW, b.a1[u]);
    }
    lmq_load_words<Pass::MW>(sp, b.s0);
    lmq_load_words<Pass::MW>(sp + s_delta, b.s1);
    lmq_load_words<Pass::MW>(sp + bias_delta, b.z0);
    lmq_load_words<Pass::MW>(sp + bias_delta + s_delta, b.z1);
    wp += P * RW;
    sp += NS;
    if (++l_pass == passes) l_pass = 0, l_tile += n_warps;
  };
  // the weight does not depend on the launch before this one: the first pass is on its way
  // while that launch finishes and while the activation is staged
  Pass A, B;
  if (l_tile < end_tile) load(A);
  if (a.pdl_wait) lm_pdl_wait();
  unsigned char* xhi = lm_smem;
  unsigned char* xlo = lm_smem + size_t(a.n_rows) * stride;
  float* xsum = reinterpret_cast<float*>(lm_smem + size_t(2) * a.n_rows * stride);   // [n_rows][blocks64]
  // the activation, staged exactly as in the kernel above
  float big = 0.0f;
  for (int i = tid; i < a.n_rows * a.hidden; i += LM_THREADS) big = fmaxf(big, fabsf(a.x[i]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
  if (lane == 0) red_s[warp] = big;
  __syncthreads();
  big = red_s[0];
  for (int w = 1; w < LM_WARPS; ++w) big = fmaxf(big, red_s[w]);
  int e = static_cast<int>((__float_as_uint(big) >> 23) & 0xffu) - 127;
  e = max(-100, min(100, e));
  const float xscale = exp2f(static_cast<float>(8 - e)), inv_xscale = exp2f(static_cast<float>(e - 8)) * LMQ_UNIT_INV;
  for (int i = tid; i < a.n_rows * a.hidden; i += LM_THREADS) {
    const int r = i / a.hidden, p = i - r * a.hidden;
    const int col = (p & ~15) + lmq_slot_column<BITS>(p & 15);
    const float v = a.x[size_t(r) * a.hidden + col] * xscale;
    const __half h = __float2half_rn(v);
    const __half l = __float2half_rn(v - __half2float(h));
    reinterpret_cast<__half*>(xhi + size_t(r) * stride)[p] = h;
    reinterpret_cast<__half*>(xlo + size_t(r) * stride)[p] = l;
  }
  __syncthreads();
  for (int i = tid; i < a.n_rows * blocks64; i += LM_THREADS) {
    const int r = i / blocks64, b = i - r * blocks64;
    const __half* ph = reinterpret_cast<const __half*>(xhi + size_t(r) * stride) + b * 64;
    const __half* pl = reinterpret_cast<const __half*>(xlo + size_t(r) * stride) + b * 64;
    float sum = 0.0f;
    for (int c = 0; c < 64; ++c) sum += __half2float(ph[c]) + __half2float(pl[c]);
    xsum[i] = sum * (1.0f / LMQ_UNIT_INV);
  }
  __syncthreads();
  constexpr bool paired = PAIRED;   // up to four activation rows: hi and lo halves share a product
  const int act = paired ? g >> 1 : g;
  const bool has_col = act < a.n_rows;
  const unsigned char* bh = (paired && (g & 1) ? xlo : xhi) + (has_col ? act : 0) * stride + t * 32;
  const unsigned char* bl = xlo + (has_col ? act : 0) * stride + t * 32;
  const int c_row0 = paired ? t : 2 * t, c_row1 = paired ? t : 2 * t + 1;
  const float* xs0 = xsum + (c_row0 < a.n_rows ? c_row0 : 0) * blocks64;
  const float* xs1 = xsum + (c_row1 < a.n_rows ? c_row1 : 0) * blocks64;
  // compute cursor
  int c_pass = 0;
  float v[4] = {0.f, 0.f, 0.f, 0.f};   // (r0, act 2t), (r0, act 2t+1), (r1, act 2t), (r1, act 2t+1)
  unsigned long long best0 = 0, best1 = 0;
  auto compute = [&](const Pass& b) {
    const int blk0 = c_pass * P;
#pragma unroll
    for (int u = 0; u < P; ++u) {
      const int blk = blk0 + u;
      uint4 xh[2], xl[2];
      xh[0] = xh[1] = xl[0] = xl[1] = make_uint4(0, 0, 0, 0);
      if (has_col) {
        xh[0] = *reinterpret_cast<const uint4*>(bh + blk * 128);
        xh[1] = *reinterpret_cast<const uint4*>(bh + blk * 128 + 16);
        if (!paired) {
          xl[0] = *reinterpret_cast<const uint4*>(bl + blk * 128);
          xl[1] = *reinterpret_cast<const uint4*>(bl + blk * 128 + 16);
        }
      }
      const uint32_t bhr[8] = {xh[0].x, xh[0].y, xh[0].z, xh[0].w, xh[1].x, xh[1].y, xh[1].z, xh[1].w};
      const uint32_t blr[8] = {xl[0].x, xl[0].y, xl[0].z, xl[0].w, xl[1].x, xl[1].y, xl[1].z, xl[1].w};
      float ch[4] = {0.f, 0.f, 0.f, 0.f}, cl[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a0, a1, a2, a3;
        if (BITS == 8) {
          a0 = __byte_perm(b.a0[u][j % LW], 0, 0x4140), a2 = __byte_perm(b.a0[u][j % LW], 0, 0x4342);
          a1 = __byte_perm(b.a1[u][j % LW], 0, 0x4140), a3 = __byte_perm(b.a1[u][j % LW], 0, 0x4342);
        } else {
          const uint32_t p0 = b.a0[u][(j >> 1) % LW] >> ((j & 1) * 8), p1 = b.a1[u][(j >> 1) % LW] >> ((j & 1) * 8);
          a0 = p0 & 0x000f000fu, a2 = (p0 >> 4) & 0x000f000fu;
          a1 = p1 & 0x000f000fu, a3 = (p1 >> 4) & 0x000f000fu;
        }
        mma_f16_lm(ch, a0, a1, a2, a3, bhr[2 * j], bhr[2 * j + 1]);
        if (!paired) mma_f16_lm(cl, a0, a1, a2, a3, blr[2 * j], blr[2 * j + 1]);
      }
      const float sc0 = lmq_meta(b.s0, u / PG), sc1 = lmq_meta(b.s1, u / PG);
      const float bi0 = lmq_meta(b.z0, u / PG), bi1 = lmq_meta(b.z1, u / PG);
      const float x0 = xs0[blk];
      if (paired) {
        v[0] += sc0 * (ch[0] + ch[1]) + bi0 * x0;
        v[2] += sc1 * (ch[2] + ch[3]) + bi1 * x0;
      } else {
        const float x1 = xs1[blk];
        v[0] += sc0 * (ch[0] + cl[0]) + bi0 * x0;
        v[1] += sc0 * (ch[1] + cl[1]) + bi0 * x1;
        v[2] += sc1 * (ch[2] + cl[2]) + bi1 * x0;
        v[3] += sc1 * (ch[3] + cl[3]) + bi1 * x1;
      }
    }
    if (++c_pass == passes) {
      const int64_t r0 = c_tile * 16 + g, r1 = r0 + 8;
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] *= inv_xscale;
      if (r0 < a.vocab) {
        const unsigned long long k0 = pack_key(v[0], r0), k1 = pack_key(v[1], r0);
        best0 = k0 > best0 ? k0 : best0;
        best1 = k1 > best1 ? k1 : best1;
      }
      if (r1 < a.vocab) {
        const unsigned long long k0 = pack_key(v[2], r1), k1 = pack_key(v[3], r1);
        best0 = k0 > best0 ? k0 : best0;
        best1 = k1 > best1 ? k1 : best1;
      }
      v[0] = v[1] = v[2] = v[3] = 0.f;
      c_pass = 0, c_tile += n_warps;
    }
  };

  while (c_tile < end_tile) {
    if (l_tile < end_tile) load(B);
    compute(A);
    if (c_tile >= end_tile) break;
    if (l_tile < end_tile) load(A);
    compute(B);
  }

  // the tiles left over: one per block and turn, warp w takes the 64-column blocks w, w + 8, ...;
  // the partial sums meet in shared memory and are added in warp order
  __shared__ float left_s[LM_WARPS][16][8];
  unsigned long long left_best = 0;   // threads 0..127: (row tid / 8 of the tile, activation row tid % 8)
  for (int64_t tile = rounds * n_warps + blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t r0 = tile * 16 + g;
    const int64_t rr0 = r0 < a.vocab ? r0 : a.vocab - 1, rr1 = r0 + 8 < a.vocab ? r0 + 8 : a.vocab - 1;
    const uint32_t* w0 = a.w.packed + rr0 * row_words + t * LW;
    const uint32_t* w1 = a.w.packed + rr1 * row_words + t * LW;
    float lv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
    for (int blk = warp; blk < blocks64; blk += LM_WARPS) {
      uint32_t A0[LW], A1[LW];
      lmq_load_words<LW>(w0 + blk * RW, A0);
      lmq_load_words<LW>(w1 + blk * RW, A1);
      const int grp = blk / PG;
      const uint16_t s0 = a.w.scales[rr0 * groups + grp], s1 = a.w.scales[rr1 * groups + grp];
      const uint16_t z0 = a.w.biases[rr0 * groups + grp], z1 = a.w.biases[rr1 * groups + grp];
      uint4 xh[2], xl[2];
      xh[0] = xh[1] = xl[0] = xl[1] = make_uint4(0, 0, 0, 0);
      if (has_col) {
        xh[0] = *reinterpret_cast<const uint4*>(bh + blk * 128);
        xh[1] = *reinterpret_cast<const uint4*>(bh + blk * 128 + 16);
        if (!paired) {
          xl[0] = *reinterpret_cast<const uint4*>(bl + blk * 128);
          xl[1] = *reinterpret_cast<const uint4*>(bl + blk * 128 + 16);
        }
      }
      const uint32_t bhr[8] = {xh[0].x, xh[0].y, xh[0].z, xh[0].w, xh[1].x, xh[1].y, xh[1].z, xh[1].w};
      const uint32_t blr[8] = {xl[0].x, xl[0].y, xl[0].z, xl[0].w, xl[1].x, xl[1].y, xl[1].z, xl[1].w};
      float ch[4] = {0.f, 0.f, 0.f, 0.f}, cl[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a0, a1, a2, a3;
        if (BITS == 8) {
          a0 = __byte_perm(A0[j % LW], 0, 0x4140), a2 = __byte_perm(A0[j % LW], 0, 0x4342);
          a1 = __byte_perm(A1[j % LW], 0, 0x4140), a3 = __byte_perm(A1[j % LW], 0, 0x4342);
        } else {
          const uint32_t p0 = A0[(j >> 1) % LW] >> ((j & 1) * 8), p1 = A1[(j >> 1) % LW] >> ((j & 1) * 8);
          a0 = p0 & 0x000f000fu, a2 = (p0 >> 4) & 0x000f000fu;
          a1 = p1 & 0x000f000fu, a3 = (p1 >> 4) & 0x000f000fu;
        }
        mma_f16_lm(ch, a0, a1, a2, a3, bhr[2 * j], bhr[2 * j + 1]);
        if (!paired) mma_f16_lm(cl, a0, a1, a2, a3, blr[2 * j], blr[2 * j + 1]);
      }
      const float sc0 = __uint_as_float(uint32_t(s0) << 16), sc1 = __uint_as_float(uint32_t(s1) << 16);
      const float bi0 = __uint_as_float(uint32_t(z0) << 16), bi1 = __uint_as_float(uint32_t(z1) << 16);
      const float x0 = xs0[blk];
      if (paired) {
        lv[0] += sc0 * (ch[0] + ch[1]) + bi0 * x0;
        lv[2] += sc1 * (ch[2] + ch[3]) + bi1 * x0;
      } else {
        const float x1 = xs1[blk];
        lv[0] += sc0 * (ch[0] + cl[0]) + bi0 * x0;
        lv[1] += sc0 * (ch[1] + cl[1]) + bi0 * x1;
        lv[2] += sc1 * (ch[2] + cl[2]) + bi1 * x0;
        lv[3] += sc1 * (ch[3] + cl[3]) + bi1 * x1;
      }
    }
    __syncthreads();   // the turn before this one has been added up
    left_s[warp][g][c_row0] = lv[0];
    left_s[warp][g + 8][c_row0] = lv[2];
    if (!paired) {
      left_s[warp][g][c_row1] = lv[1];
      left_s[warp][g + 8][c_row1] = lv[3];
    }
    __syncthreads();
    if (tid < 128) {
      const int row = tid >> 3, arow = tid & 7;
      float sum = left_s[0][row][arow];
#pragma unroll
      for (int w = 1; w < LM_WARPS; ++w) sum += left_s[w][row][arow];
      const int64_t r = tile * 16 + row;
      if (r < a.vocab && arow < a.n_rows) {
        const unsigned long long key = pack_key(sum * inv_xscale, r);
        left_best = key > left_best ? key : left_best;
      }
    }
  }
  // threads 0..127 hold the left-over tiles' best per (row, activation row): best per activation row
  __shared__ unsigned long long left_best_s[4][8];
#pragma unroll
  for (int off = 8; off < 32; off <<= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, left_best, off);
    left_best = o > left_best ? o : left_best;
  }
  if (tid < 128 && lane < 8) left_best_s[warp][lane] = left_best;

#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    const unsigned long long o0 = __shfl_xor_sync(0xffffffffu, best0, off), o1 = __shfl_xor_sync(0xffffffffu, best1, off);
    best0 = o0 > best0 ? o0 : best0;
    best1 = o1 > best1 ? o1 : best1;
  }
  if (lane < 4) {
    if (paired) {
      best_s[warp][lane] = best0;
    } else {
      best_s[warp][2 * lane] = best0;
      best_s[warp][2 * lane + 1] = best1;
    }
  }
  __syncthreads();
  if (tid < a.n_rows) {
    unsigned long long b = best_s[0][tid];
    for (int w = 1; w < LM_WARPS; ++w) b = best_s[w][tid] > b ? best_s[w][tid] : b;
    for (int w = 0; w < 4; ++w) b = left_best_s[w][tid] > b ? left_best_s[w][tid] : b;
    atomicMax(a.keys + tid, b);
    __threadfence();
  }
  __syncthreads();
  if (tid == 0) last_s = atomicAdd(a.counter, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last_s && tid < a.n_rows) {
    __threadfence();
    const unsigned long long win = atomicExch(a.keys + tid, 0ull);
    const int32_t winner = static_cast<int32_t>(0xffffffffu - uint32_t(win & 0xffffffffu)) + a.index_offset;
    a.index_out[tid] = winner;
    if (a.index_mirror) {   // the host's copy, written from here: no copy node behind the launch
      a.index_mirror[tid] = winner;
      __threadfence_system();
    }
    if (a.value_out) a.value_out[tid] = unordered_bits(uint32_t(win >> 32));
    if (tid == 0) *a.counter = 0;
  }
}

// Tiles handed out in whole rounds: a multiple of the warp count of the largest grid (two blocks per
// SM), hence of every grid a launch of this vocabulary can get whatever its number of activation
// rows, so a tile is worked on the same way (and gives the same bits) in all of them. A grid that was
// cut down to the vocabulary has no whole round.
static int64_t lm_whole_tiles(int64_t tiles, int sm_count, int blocks) {
  const int64_t widest = int64_t(sm_count) * LM_BLOCKS_PER_SM * LM_WARPS;
  if (blocks != sm_count && blocks != sm_count * LM_BLOCKS_PER_SM) return 0;
  return tiles / widest * widest;
}

size_t lm_head_affine_smem_bytes(int n_rows, int hidden, int group_size) {
  (void)group_size;
  return size_t(2) * n_rows * lmq_x_stride_bytes(hidden) + size_t(n_rows) * (hidden / 64) * sizeof(float);
}

cudaError_t launch_lm_head_argmax_affine(const LmHeadAffineArgs& a, int sm_count, cudaStream_t stream) {
  const int64_t tiles = (a.vocab + 15) / 16;
  const int per_group = a.w.group_size / 64;
  const size_t smem = lm_head_affine_smem_bytes(a.n_rows, a.hidden, a.w.group_size);
  int per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
  per_sm = per_sm > 2 ? 2 : per_sm < 1 ? 1 : per_sm;
  int blocks = sm_count * per_sm;
  if (int64_t(blocks) * LM_WARPS > tiles) blocks = static_cast<int>((tiles + LM_WARPS - 1) / LM_WARPS);
  void (*kernel)(LmHeadAffineArgs) = a.w.bits == 8 ? lm_head_argmax_affine_kernel<8> : lm_head_argmax_affine_kernel<4>;
  // the pipelined kernel wherever a row is a whole number of passes and the rows' scales can be
  // fetched with aligned vector loads
  static const bool pipe_off = std::getenv("SGK_LM_NO_PIPE") != nullptr;
  const int pass_blocks = a.w.bits == 8 ? 4 : 8;
  const bool aligned = (reinterpret_cast<uintptr_t>(a.w.scales) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.w.biases) & 15) == 0 &&
                       ((a.hidden / a.w.group_size) * 2) % (pass_blocks / per_group * 2) == 0;
  if (!pipe_off && aligned && a.hidden % (64 * pass_blocks) == 0 && a.hidden >= 2 * 64 * pass_blocks) {
    const bool paired = a.n_rows <= 4;
    if (a.w.bits == 8 && paired) kernel = per_group == 1 ? lm_head_argmax_affine_pipe_kernel<8, 4, 1, true> : lm_head_argmax_affine_pipe_kernel<8, 4, 2, true>;
    else if (a.w.bits == 8) kernel = per_group == 1 ? lm_head_argmax_affine_pipe_kernel<8, 4, 1, false> : lm_head_argmax_affine_pipe_kernel<8, 4, 2, false>;
    else if (paired) kernel = per_group == 1 ? lm_head_argmax_affine_pipe_kernel<4, 8, 1, true> : lm_head_argmax_affine_pipe_kernel<4, 8, 2, true>;
    else kernel = per_group == 1 ? lm_head_argmax_affine_pipe_kernel<4, 8, 1, false> : lm_head_argmax_affine_pipe_kernel<4, 8, 2, false>;
  }
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
  }
  LmHeadAffineArgs b = a;
  b.whole_tiles = lm_whole_tiles(tiles, sm_count, blocks);
  ChainLaunch l(dim3(blocks), dim3(LM_THREADS), smem, stream, a.pdl_wait != 0);
  return cudaLaunchKernelEx(&l.cfg, kernel, b);
}

// Row `*index` of an affine-quantised table, dequantised (code * scale + bias), times `scale`
// (the quantised form of encode_embedding_from_index_buffers_scaled,
// src/metal_backend/matmul_encode.rs:424-557).
__global__ void embed_gather_affine_kernel(AffineWeight w, const int32_t* index, int64_t vocab, int hidden, float scale,
                                           int recast_bf16, float* out, int pdl_trigger, int pdl_wait) {
  if (pdl_trigger) lm_pdl_trigger();
  if (pdl_wait) lm_pdl_wait();
  const int64_t token = *index;
  if (token < 0 || token >= vocab) return;
  const int64_t row_words = int64_t(hidden) * w.bits / 32;
  const int groups = hidden / w.group_size;
  const uint32_t mask = (1u << w.bits) - 1u;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) {
    const int bit = i * w.bits;
    const uint32_t code = (w.packed[token * row_words + bit / 32] >> (bit % 32)) & mask;   // 4 and 8 divide 32
    const int grp = i / w.group_size;
    const float sc = __uint_as_float(uint32_t(w.scales[token * groups + grp]) << 16);
    const float bi = __uint_as_float(uint32_t(w.biases[token * groups + grp]) << 16);
    const float v = __fmul_rn(__fadd_rn(__fmul_rn(static_cast<float>(code), sc), bi), scale);
    out[i] = recast_bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : v;
  }
}

cudaError_t launch_embed_gather_affine(const AffineWeight& table, const int32_t* index, int64_t vocab, int hidden,
                                       float scale, int recast_bf16, float* out, int pdl_trigger, int pdl_wait,
                                       cudaStream_t stream) {
  const int blocks = (hidden + 255) / 256 < 64 ? (hidden + 255) / 256 : 64;
  ChainLaunch l(dim3(blocks), dim3(256), 0, stream, pdl_wait != 0);
  return cudaLaunchKernelEx(&l.cfg, embed_gather_affine_kernel, table, index, vocab, hidden, scale, recast_bf16, out,
                            pdl_trigger, pdl_wait);
}

size_t lm_head_smem_bytes(int w_bf16, int n_rows, int hidden) {
  if (w_bf16) return size_t(2) * n_rows * lm_x_stride_bytes(hidden);
  const int R = n_rows <= 1 ? 1 : n_rows <= 2 ? 2 : n_rows <= 4 ? 4 : 8;
  return size_t(R) * hidden * sizeof(float);
}

cudaError_t launch_lm_head_argmax(const LmHeadArgs& a, int sm_count, cudaStream_t stream) {
  const size_t smem = lm_head_smem_bytes(a.w_bf16, a.n_rows, a.hidden);
  int per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
  if (a.w_bf16) {
    per_sm = per_sm > LM_BLOCKS_PER_SM ? LM_BLOCKS_PER_SM : per_sm < 1 ? 1 : per_sm;
    int blocks = sm_count * per_sm;
    const int64_t tiles = (a.vocab + 15) / 16;
    if (int64_t(blocks) * LM_WARPS > tiles) blocks = static_cast<int>((tiles + LM_WARPS - 1) / LM_WARPS);
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(lm_head_argmax_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return e;
    }
    LmHeadArgs b = a;
    b.whole_tiles = lm_whole_tiles(tiles, sm_count, blocks);
    ChainLaunch l(dim3(blocks), dim3(LM_THREADS), smem, stream, a.pdl_wait != 0);
    return cudaLaunchKernelEx(&l.cfg, lm_head_argmax_bf16_kernel, b);
  }
  const int R = a.n_rows <= 1 ? 1 : a.n_rows <= 2 ? 2 : a.n_rows <= 4 ? 4 : 8;
  per_sm = per_sm > 4 ? 4 : per_sm < 1 ? 1 : per_sm;
  int blocks = sm_count * per_sm;
  const int64_t pairs = (a.vocab + 1) / 2;
  if (int64_t(blocks) * LM_WARPS > pairs) blocks = static_cast<int>((pairs + LM_WARPS - 1) / LM_WARPS);
  if (blocks < 1) blocks = 1;
  if (R == 1) return launch_r<1>(a, blocks, smem, stream);
  if (R == 2) return launch_r<2>(a, blocks, smem, stream);
  if (R == 4) return launch_r<4>(a, blocks, smem, stream);
  return launch_r<8>(a, blocks, smem, stream);
}

}  // namespace sgk
