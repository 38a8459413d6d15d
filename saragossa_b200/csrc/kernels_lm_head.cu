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
    a.index_out[tid] = static_cast<int32_t>(0xffffffffu - uint32_t(win & 0xffffffffu)) + a.index_offset;
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
  if (a.pdl_wait) lm_pdl_wait();
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
  for (int64_t tile = int64_t(blockIdx.x) * LM_WARPS + warp; tile < tiles; tile += int64_t(gridDim.x) * LM_WARPS) {
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
    atomicMax(a.keys + tid, b);
    __threadfence();
  }
  __syncthreads();
  if (tid == 0) last_s = atomicAdd(a.counter, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last_s && tid < a.n_rows) {
    __threadfence();
    const unsigned long long win = atomicExch(a.keys + tid, 0ull);
    a.index_out[tid] = static_cast<int32_t>(0xffffffffu - uint32_t(win & 0xffffffffu)) + a.index_offset;
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
    ChainLaunch l(dim3(blocks), dim3(LM_THREADS), smem, stream, a.pdl_wait != 0);
    return cudaLaunchKernelEx(&l.cfg, lm_head_argmax_bf16_kernel, a);
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
