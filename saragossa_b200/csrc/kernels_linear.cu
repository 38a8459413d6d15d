// One decode token on the linear-attention recurrent state this path stores:
// the depthwise causal conv with its sliding history, and the Gated DeltaNet update
//   S <- g*S;  kv = S.k;  delta = (v - kv)*beta;  S <- S + delta*k^T;  y = S.q
// on the state [H_v][d_v][d_k] (src/linear_attention.rs:802-852,896-991; Metal twins
// linear_attn_gated_delta_* in src/metal_backend/mod.rs:155-171). Both are HBM-bound:
// the state is read once and written once per token (4 MiB per layer at 32 x 128 x 128 f32).
#include <cstdlib>

#include "kernels.h"

namespace sgk {

// Programmatic dependent launch (see mma_common.cuh): no-ops in a launch without such a neighbour.
__device__ __forceinline__ void lin_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void lin_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

constexpr int GD_THREADS = 256;
constexpr int GD_WARPS = GD_THREADS / 32;
constexpr int GD_MAXJ = 8;  // key_head_dim <= 256

template <bool BF16>
__device__ __forceinline__ float load_state(const void* base, int64_t i) {
  if (BF16) return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(base)[i]);
  return reinterpret_cast<const float*>(base)[i];
}
template <bool BF16>
__device__ __forceinline__ void store_state(void* base, int64_t i, float v) {
  if (BF16)
    reinterpret_cast<uint16_t*>(base)[i] = f32_to_bf16_bits(v);
  else
    reinterpret_cast<float*>(base)[i] = v;
}

// One warp per state row (d_k values), rows strided over the grid. With a bf16 state the
// read-out uses the f32 values before they are rounded for storage, like
// linear_attn_gated_delta_dk128_bf16_tg4_f32 (src/kernels.metal:2842-2915).
// The two dot products of
// a row are warp reductions; everything else is element-wise on the lane's own values.
template <bool BF16>
__global__ void __launch_bounds__(GD_THREADS) gated_delta_step_kernel(GatedDeltaArgs a) {
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * GD_WARPS + (threadIdx.x >> 5);
  const int total_warps = gridDim.x * GD_WARPS;
  const int rows = a.num_value_heads * a.value_head_dim;
  const int dk = a.key_head_dim;
  const int repeat = a.num_value_heads / a.num_key_heads;
  // blockIdx.y picks the sequence: its own state, and its slice of every input and of the output
  const int b = blockIdx.y;
  void* ssm = a.ssm[b];
  const int T = a.n_tokens;
  if (a.pdl_trigger) lin_pdl_trigger();
  if (a.pdl_wait) lin_pdl_wait();
  const float* q_b = a.q + int64_t(b) * T * a.num_key_heads * dk;
  const float* k_b = a.k + int64_t(b) * T * a.num_key_heads * dk;
  const float* v_b = a.v + int64_t(b) * T * rows;
  const float* g_b = a.g + int64_t(b) * T * a.num_value_heads;
  const float* beta_b = a.beta + int64_t(b) * T * a.num_value_heads;
  float* out_b = a.out + int64_t(b) * T * rows;
  for (int row = warp; row < rows; row += total_warps) {
    const int vh = row / a.value_head_dim;
    const int kh = vh / repeat;
    const int64_t base = int64_t(row) * dk;
    float s[GD_MAXJ], kk[GD_MAXJ];
#pragma unroll
    for (int j = 0; j < GD_MAXJ; ++j) {
      const int i = lane + 32 * j;
      if (i < dk) s[j] = load_state<BF16>(ssm, base + i);
    }
    // the tokens of a sequence run on the row kept in registers; it goes back to memory once
    for (int t = 0; t < T; ++t) {
      const float decay = g_b[int64_t(t) * a.num_value_heads + vh], beta = beta_b[int64_t(t) * a.num_value_heads + vh];
      const float* kp = k_b + (int64_t(t) * a.num_key_heads + kh) * dk;
      const float* qp = q_b + (int64_t(t) * a.num_key_heads + kh) * dk;
      float kv = 0.0f;
#pragma unroll
      for (int j = 0; j < GD_MAXJ; ++j) {
        const int i = lane + 32 * j;
        if (i < dk) {
          kk[j] = kp[i];
          s[j] *= decay;
          kv += s[j] * kk[j];
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) kv += __shfl_xor_sync(0xffffffffu, kv, off);
      const float delta = (v_b[int64_t(t) * rows + row] - kv) * beta;
      float y = 0.0f;
#pragma unroll
      for (int j = 0; j < GD_MAXJ; ++j) {
        const int i = lane + 32 * j;
        if (i < dk) {
          s[j] += delta * kk[j];
          y += s[j] * qp[i];
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) y += __shfl_xor_sync(0xffffffffu, y, off);
      if (lane == 0) out_b[int64_t(t) * rows + row] = y;
    }
#pragma unroll
    for (int j = 0; j < GD_MAXJ; ++j) {
      const int i = lane + 32 * j;
      if (i < dk) store_state<BF16>(ssm, base + i, s[j]);
    }
  }
}

// key_head_dim 128 (the shape the reference ships its own dk128 kernels for): a lane owns four
// consecutive state values, so a row is one 16-byte (f32) or 8-byte (bf16) access per lane, and a
// warp carries R rows of one head at once to keep R independent loads in flight per lane.
// Spelled with intrinsics so that every instantiation rounds in the same places.
__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
  return __fmaf_rn(a.w, b.w, __fmaf_rn(a.z, b.z, __fmaf_rn(a.y, b.y, __fmul_rn(a.x, b.x))));
}

template <bool BF16, int R>
__global__ void __launch_bounds__(GD_THREADS) gated_delta_step_dk128_kernel(GatedDeltaArgs a) {
  const int lane = threadIdx.x & 31;
  const int rows = a.num_value_heads * a.value_head_dim;
  const int repeat = a.num_value_heads / a.num_key_heads;
  const int b = blockIdx.y;
  const int row0 = (blockIdx.x * GD_WARPS + (threadIdx.x >> 5)) * R;  // value_head_dim % R == 0
  if (a.pdl_trigger) lin_pdl_trigger();
  if (row0 >= rows) return;
  const int vh = row0 / a.value_head_dim;
  const int kh = vh / repeat;
  const int T = a.n_tokens;
  const int64_t base = int64_t(row0) * 128 + lane * 4;
  float4 s[R];
  float vv[R];
  if (BF16) {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(a.ssm[b]) + base;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint2 raw = *reinterpret_cast<const uint2*>(p + r * 128);
      s[r] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                         __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
    }
  } else {
    const float* p = reinterpret_cast<const float*>(a.ssm[b]) + base;
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = *reinterpret_cast<const float4*>(p + r * 128);
  }
  // The state rows are on their way; q, k, v, g and beta are what the previous launch of a token
  // chain may still be writing.
  if (a.pdl_wait) lin_pdl_wait();
  // the tokens of a sequence run on the rows kept in registers; they go back to memory once
  for (int t = 0; t < T; ++t) {
    const int64_t tok = int64_t(b) * T + t;
    const int64_t in_k = (tok * a.num_key_heads + kh) * 128 + lane * 4;
    const float4 kk = *reinterpret_cast<const float4*>(a.k + in_k);
    const float4 qq = *reinterpret_cast<const float4*>(a.q + in_k);
    const float decay = a.g[tok * a.num_value_heads + vh];
    const float beta = a.beta[tok * a.num_value_heads + vh];
#pragma unroll
    for (int r = 0; r < R; ++r) vv[r] = a.v[tok * rows + row0 + r];
    float kv[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      s[r].x = __fmul_rn(s[r].x, decay), s[r].y = __fmul_rn(s[r].y, decay);
      s[r].z = __fmul_rn(s[r].z, decay), s[r].w = __fmul_rn(s[r].w, decay);
      kv[r] = dot4(s[r], kk);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
      for (int r = 0; r < R; ++r) kv[r] += __shfl_xor_sync(0xffffffffu, kv[r], off);
    float y[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float delta = __fmul_rn(__fsub_rn(vv[r], kv[r]), beta);
      s[r].x = __fmaf_rn(delta, kk.x, s[r].x), s[r].y = __fmaf_rn(delta, kk.y, s[r].y);
      s[r].z = __fmaf_rn(delta, kk.z, s[r].z), s[r].w = __fmaf_rn(delta, kk.w, s[r].w);
      y[r] = dot4(s[r], qq);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
      for (int r = 0; r < R; ++r) y[r] += __shfl_xor_sync(0xffffffffu, y[r], off);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) a.out[tok * rows + row0 + r] = y[r];
    }
  }
  if (BF16) {
    uint16_t* p = reinterpret_cast<uint16_t*>(a.ssm[b]) + base;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint2 raw;
      raw.x = uint32_t(f32_to_bf16_bits(s[r].x)) | (uint32_t(f32_to_bf16_bits(s[r].y)) << 16);
      raw.y = uint32_t(f32_to_bf16_bits(s[r].z)) | (uint32_t(f32_to_bf16_bits(s[r].w)) << 16);
      *reinterpret_cast<uint2*>(p + r * 128) = raw;
    }
  } else {
    float* p = reinterpret_cast<float*>(a.ssm[b]) + base;
#pragma unroll
    for (int r = 0; r < R; ++r) *reinterpret_cast<float4*>(p + r * 128) = s[r];
  }
}

template <bool BF16, int R>
static cudaError_t launch_dk128(const GatedDeltaArgs& a, int rows, cudaStream_t stream) {
  const int warps = rows / R;
  ChainLaunch l(dim3((warps + GD_WARPS - 1) / GD_WARPS, a.n_states), dim3(GD_THREADS), 0, stream, a.pdl_wait != 0);
  return cudaLaunchKernelEx(&l.cfg, gated_delta_step_dk128_kernel<BF16, R>, a);
}

cudaError_t launch_gated_delta_step(const GatedDeltaArgs& a, int sm_count, cudaStream_t stream) {
  const int rows = a.num_value_heads * a.value_head_dim;
  const bool aligned = ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k)) & 15) == 0;
  if (a.key_head_dim == 128 && aligned) {
    // four rows per warp once that still leaves every SM several blocks; else one row per warp
    static const int wide_rows = [] {
      const char* e = std::getenv("SGK_GD_WIDE_ROWS");
      return e ? std::atoi(e) : 0;
    }();
    const int64_t need = wide_rows > 0 ? wide_rows : int64_t(4) * GD_WARPS * sm_count * 4;
    const bool wide = a.value_head_dim % 4 == 0 && int64_t(rows) * a.n_states >= need;
    if (a.ssm_bf16) return wide ? launch_dk128<true, 4>(a, rows, stream) : launch_dk128<true, 1>(a, rows, stream);
    return wide ? launch_dk128<false, 4>(a, rows, stream) : launch_dk128<false, 1>(a, rows, stream);
  }
  int blocks = (rows + GD_WARPS - 1) / GD_WARPS;
  // 8 resident blocks per SM over the whole grid; one row per warp needs no more than that
  int cap = (sm_count * 8 + a.n_states - 1) / a.n_states;
  if (blocks > cap) blocks = cap;
  ChainLaunch l(dim3(blocks, a.n_states), dim3(GD_THREADS), 0, stream, a.pdl_wait != 0);
  return a.ssm_bf16 ? cudaLaunchKernelEx(&l.cfg, gated_delta_step_kernel<true>, a)
                    : cudaLaunchKernelEx(&l.cfg, gated_delta_step_kernel<false>, a);
}

// ---- the whole decode step of a recurrent layer in one launch ----------------------------------
// The reference's resident decode runs conv + SiLU + unit RMS norm + gates as one dispatch and the
// gated-delta update as the next (linear_attn_conv_norm_gates_k4_dk128_f32 and
// linear_attn_gated_delta_dk128_tg4_f32, src/kernels.metal:2295-2416,2569-2643; CPU order of
// operations src/linear_attention.rs:313-342). Two small launches that depend on each other cost
// about 2 us each however they overlap their neighbours, and config 3 has 30 such layers per
// token. Here a block of 8 warps owns 8 state rows of one value head and does everything they
// need: the 256 threads redo the conv of the key head's 128 q and 128 k channels (8 KiB from L2),
// eight of them the conv of the block's own v channels, two block reductions give the norms, and
// each warp updates its row. The conv history of q and k is read by all 32 blocks of a key head
// and must be shifted by one of them only after all have read it: a block arrives on the head's
// counter once its history values are in registers, and the block that arrives last writes the
// shifted rows (from its registers). Nobody waits. v channels belong to one block each.
// Measured beside it and dropped: every warp redoing the head's conv for itself (lane l the
// channels 4l..4l+3, norms by warp shuffles, no shared memory and no block barrier before the
// state update; two rows per warp to keep all blocks resident at 128 registers): 305 us per
// token of config 3 against 290 us with this kernel.
// All 512 blocks of config 3's shape (32 value heads) must be resident at once or the launch takes two
// waves: at most 64 registers per thread (four blocks of 256 threads per SM), which the usual conv
// kernel of four taps fits; up to eight taps take the instance with longer tap arrays.
template <bool BF16, int LD_MAX_KERNEL>
__global__ void __launch_bounds__(GD_THREADS, LD_MAX_KERNEL <= 4 ? 4 : 3) linear_decode_step_dk128_kernel(LinearDecodeArgs a) {
  __shared__ float qk_s[256];        // normalised q [128] | k [128] of the key head
  __shared__ float red_s[GD_WARPS];
  __shared__ float v_s[GD_WARPS];    // silu(conv) of the block's eight v channels
  __shared__ float gate_s[2];        // beta, decay of the value head
  __shared__ int last_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int blocks_per_vh = 128 / GD_WARPS;                 // 16 blocks of 8 rows per value head
  const int vh = blockIdx.x / blocks_per_vh, rb = blockIdx.x % blocks_per_vh;
  const int repeat = a.num_value_heads / a.num_key_heads;
  const int kh = vh / repeat;
  const int key_dim = a.num_key_heads * 128;
  const int K = a.kernel, keep = K - 1;
  if (a.pdl_trigger) lin_pdl_trigger();

  // this warp's state row, and the taps and history of this thread's channels: none of them is
  // written by the launch before this one
  const int row = vh * 128 + rb * GD_WARPS + warp;
  const int64_t base = int64_t(row) * 128 + lane * 4;
  float4 s;
  if (BF16) {
    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(a.ssm) + base);
    s = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                    __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
  } else {
    s = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.ssm) + base);
  }
  // channel of this thread: q (threads 0..127) or k (128..255) of the key head
  const int c = (tid < 128 ? 0 : key_dim) + kh * 128 + (tid & 127);
  // and, for the first eight threads, one v channel of the block
  const bool has_v = tid < GD_WARPS;
  const int cv = 2 * key_dim + vh * 128 + rb * GD_WARPS + (has_v ? tid : 0);
  float w[LD_MAX_KERNEL], h[LD_MAX_KERNEL], wv[LD_MAX_KERNEL], hv[LD_MAX_KERNEL];
#pragma unroll
  for (int kk = 0; kk < LD_MAX_KERNEL; ++kk) {
    w[kk] = kk < K ? a.conv_weight[int64_t(c) * K + kk] : 0.0f;
    h[kk] = kk < keep ? a.history[int64_t(kk) * a.conv_dim + c] : 0.0f;
    wv[kk] = has_v && kk < K ? a.conv_weight[int64_t(cv) * K + kk] : 0.0f;
    hv[kk] = has_v && kk < keep ? a.history[int64_t(kk) * a.conv_dim + cv] : 0.0f;
  }
  const float a_log = a.a_log[vh], dt_bias = a.dt_bias[vh];
  if (a.pdl_wait) lin_pdl_wait();   // the token's inputs come from the launch before

  // depthwise conv in tap order with separate roundings (the CPU loop), then SiLU
  const float x = a.qkv[c];
  float acc = 0.0f;
#pragma unroll
  for (int kk = 0; kk < LD_MAX_KERNEL; ++kk)
    if (kk < K) acc = __fadd_rn(acc, __fmul_rn(kk < keep ? h[kk] : x, w[kk]));
  const float act = __fdiv_rn(acc, __fadd_rn(1.0f, expf(-acc)));
  float xv = 0.0f;
  if (has_v) {
    xv = a.qkv[cv];
    float av = 0.0f;
#pragma unroll
    for (int kk = 0; kk < LD_MAX_KERNEL; ++kk)
      if (kk < K) av = __fadd_rn(av, __fmul_rn(kk < keep ? hv[kk] : xv, wv[kk]));
    v_s[tid] = __fdiv_rn(av, __fadd_rn(1.0f, expf(-av)));
    // this block is the only reader of its v channels: their history slides at once
#pragma unroll
    for (int kk = 0; kk < LD_MAX_KERNEL; ++kk)
      if (kk < keep) a.history[int64_t(kk) * a.conv_dim + cv] = kk + 1 < keep ? hv[kk + 1] : xv;
  }
  if (tid == 0) {
    const float b = a.beta_input[vh];
    gate_s[0] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-b)));
    const float dt_arg = __fadd_rn(a.gate_input[vh], dt_bias);
    const float dt = dt_arg > 20.0f ? dt_arg : logf(__fadd_rn(1.0f, expf(dt_arg)));
    gate_s[1] = expf(__fmul_rn(-expf(a_log), dt));
  }
  // unit RMS norm per head: sum of squares over the head's 128 channels (warps 0-3: q, 4-7: k)
  float ss = __fmul_rn(act, act);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if (lane == 0) red_s[warp] = ss;
  __syncthreads();   // every history value of this block has been read (it went into acc)
  // The arrival is asked for now and looked at after the row's arithmetic, by a thread that has
  // no store of its own in flight (its fence has nothing to wait for): the round trip to the
  // counter stays off the path from the token's inputs to the state update.
  int arrived = 0;
  if (tid == 32) {
    __threadfence();
    arrived = atomicAdd(a.head_counters + kh, 1);
  }
  const int half = tid < 128 ? 0 : 4;
  const float sum = (red_s[half] + red_s[half + 1]) + (red_s[half + 2] + red_s[half + 3]);
  const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, 128.0f), a.eps)));
  qk_s[tid] = __fmul_rn(__fmul_rn(act, inv_rms), tid < 128 ? a.q_scale : a.k_scale);
  __syncthreads();

  // gated delta on this warp's row (the arithmetic of gated_delta_step_dk128_kernel)
  const float4 qq = *reinterpret_cast<const float4*>(qk_s + lane * 4);
  const float4 kk4 = *reinterpret_cast<const float4*>(qk_s + 128 + lane * 4);
  const float beta = gate_s[0], decay = gate_s[1];
  s.x = __fmul_rn(s.x, decay), s.y = __fmul_rn(s.y, decay), s.z = __fmul_rn(s.z, decay), s.w = __fmul_rn(s.w, decay);
  float kv = dot4(s, kk4);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) kv += __shfl_xor_sync(0xffffffffu, kv, off);
  const float delta = __fmul_rn(__fsub_rn(v_s[warp], kv), beta);
  s.x = __fmaf_rn(delta, kk4.x, s.x), s.y = __fmaf_rn(delta, kk4.y, s.y);
  s.z = __fmaf_rn(delta, kk4.z, s.z), s.w = __fmaf_rn(delta, kk4.w, s.w);
  float y = dot4(s, qq);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) y += __shfl_xor_sync(0xffffffffu, y, off);
  if (lane == 0) a.out[row] = y;
  if (BF16) {
    uint2 raw;
    raw.x = uint32_t(f32_to_bf16_bits(s.x)) | (uint32_t(f32_to_bf16_bits(s.y)) << 16);
    raw.y = uint32_t(f32_to_bf16_bits(s.z)) | (uint32_t(f32_to_bf16_bits(s.w)) << 16);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.ssm) + base) = raw;
  } else {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.ssm) + base) = s;
  }
  if (tid == 32) {
    last_s = arrived == repeat * blocks_per_vh - 1;
    if (last_s) a.head_counters[kh] = 0;
  }
  __syncthreads();
  if (last_s) {
    // every block of the key head has its history in registers: slide the q and k rows
    __threadfence();
#pragma unroll
    for (int kk = 0; kk < LD_MAX_KERNEL; ++kk)
      if (kk < keep) a.history[int64_t(kk) * a.conv_dim + c] = kk + 1 < keep ? h[kk + 1] : x;
  }
}

cudaError_t launch_linear_decode_step(const LinearDecodeArgs& a, cudaStream_t stream) {
  ChainLaunch l(dim3(a.num_value_heads * (128 / GD_WARPS)), dim3(GD_THREADS), 0, stream, a.pdl_wait != 0);
  if (a.kernel <= 4)
    return a.ssm_bf16 ? cudaLaunchKernelEx(&l.cfg, linear_decode_step_dk128_kernel<true, 4>, a)
                      : cudaLaunchKernelEx(&l.cfg, linear_decode_step_dk128_kernel<false, 4>, a);
  return a.ssm_bf16 ? cudaLaunchKernelEx(&l.cfg, linear_decode_step_dk128_kernel<true, 8>, a)
                    : cudaLaunchKernelEx(&l.cfg, linear_decode_step_dk128_kernel<false, 8>, a);
}

// One thread per channel: the products are summed in kernel-tap order with separate
// roundings, exactly like the CPU loop, then the channel's history slides by one token.
constexpr int CONV_MAX_KERNEL = 16;

__global__ void __launch_bounds__(256) conv_step_kernel(const float* __restrict__ qkv,
                                                       const float* __restrict__ weight, float* history,
                                                       float* __restrict__ out, int conv_dim, int kernel,
                                                       int n_tokens, int pdl_trigger, int pdl_wait) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (pdl_trigger) lin_pdl_trigger();
  if (c >= conv_dim) return;
  const int keep = kernel - 1;
  // the channel's taps and its window of past inputs stay in registers over the tokens
  float w[CONV_MAX_KERNEL], h[CONV_MAX_KERNEL];
#pragma unroll
  for (int kk = 0; kk < CONV_MAX_KERNEL; ++kk) {
    w[kk] = kk < kernel ? weight[int64_t(c) * kernel + kk] : 0.0f;
    h[kk] = kk < keep ? history[int64_t(kk) * conv_dim + c] : 0.0f;
  }
  if (pdl_wait) lin_pdl_wait();   // the taps and the history are here; qkv comes from the previous launch
  for (int t = 0; t < n_tokens; ++t) {
    const float x = qkv[int64_t(t) * conv_dim + c];
    float acc = 0.0f;
#pragma unroll
    for (int kk = 0; kk < CONV_MAX_KERNEL; ++kk)
      if (kk < kernel) acc = __fadd_rn(acc, __fmul_rn(kk < keep ? h[kk] : x, w[kk]));
    out[int64_t(t) * conv_dim + c] = acc;
#pragma unroll
    for (int kk = 0; kk + 1 < CONV_MAX_KERNEL; ++kk)
      if (kk < keep) h[kk] = kk + 1 < keep ? h[kk + 1] : x;
  }
#pragma unroll
  for (int kk = 0; kk < CONV_MAX_KERNEL; ++kk)
    if (kk < keep) history[int64_t(kk) * conv_dim + c] = h[kk];
}

cudaError_t launch_conv_step(const float* qkv, const float* weight, float* history, float* out, int conv_dim,
                             int kernel, int n_tokens, int pdl_trigger, int pdl_wait, cudaStream_t stream) {
  ChainLaunch l(dim3((conv_dim + 255) / 256), dim3(256), 0, stream, pdl_wait != 0);
  return cudaLaunchKernelEx(&l.cfg, conv_step_kernel, qkv, weight, history, out, conv_dim, kernel, n_tokens,
                            pdl_trigger, pdl_wait);
}

}  // namespace sgk
