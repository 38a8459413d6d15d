// Generic paged decode attention on CUDA cores: any head_dim <= 512, any storage
// type, any GQA ratio, explicit or sliding window. One block per
// (q head, split, sequence); warps stride over rows, lanes over dims; online
// softmax in the log2 domain; the block that arrives last for a q head merges the
// split partials. It is the path for f32 pages and for shapes the tensor-core
// kernel does not take, and it cross-checks that kernel in the tests. Computes
// what attention_decode_naive/flash compute (src/decode_resident/kernels.rs:11-366).
#include "kernels.h"

namespace sgk {

constexpr int GEN_THREADS = 128;
constexpr int GEN_WARPS = GEN_THREADS / 32;
constexpr int GEN_MAXJ = 16;  // head_dim <= 32 * 16

__global__ void __launch_bounds__(GEN_THREADS) attention_generic_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  const int hd = a.pool.head_dim;
  float* q_s = smem;                       // [hd]
  float* o_s = smem + hd;                  // [GEN_WARPS][hd]
  float* ml_s = o_s + GEN_WARPS * hd;      // [GEN_WARPS][2]
  __shared__ int is_last_s;

  const int qh = blockIdx.x, split = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gqa = a.q_heads / a.pool.kv_heads;
  const int kvh = qh / gqa;
  const int slot = a.slots ? a.slots[seq] : a.slot0;
  const int64_t len = a.pool.lens[int64_t(slot) * a.pool.layers + a.layer];
  int64_t ws = a.sliding_window > 0 ? (len > a.sliding_window ? len - a.sliding_window : 0) : a.window_start;
  if (ws > len) ws = len;
  const int64_t n = len - ws;
  const int64_t r0 = ws + (n * split) / a.splits;
  const int64_t r1 = ws + (n * (split + 1)) / a.splits;
  const int32_t* table = a.pool.tables + int64_t(slot) * a.pool.table_stride;

  const float* q = a.q + (int64_t(seq) * a.q_heads + qh) * hd;
  for (int c = tid; c < hd; c += GEN_THREADS) q_s[c] = q[c] * a.scale_log2e;
  __syncthreads();

  float m = -1.0e30f, l = 0.0f;
  float acc[GEN_MAXJ];
#pragma unroll
  for (int j = 0; j < GEN_MAXJ; ++j) acc[j] = 0.0f;

  for (int64_t r = r0 + warp; r < r1; r += GEN_WARPS) {
    int32_t page = table[r / PAGE_TOKENS];
    if (page < 0 || page >= a.num_pages) {
      if (lane == 0) atomicExch(a.status, DEV_ERR_BAD_PAGE);
      continue;
    }
    const int rin = static_cast<int>(r % PAGE_TOKENS);
    const uint8_t* ktile = a.pool.base + tile_offset(a.pool, page, a.layer, kvh, 0);
    const uint8_t* vtile = ktile + a.pool.tile_bytes;
    float dot = 0.0f;
#pragma unroll
    for (int j = 0; j < GEN_MAXJ; ++j) {
      int d = lane + 32 * j;
      if (d < hd) dot += q_s[d] * load_tile_elem(ktile, a.pool.dtype, hd, 0, rin, d);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    float m_new = fmaxf(m, dot);
    float alpha = exp2f(m - m_new);
    float p = exp2f(dot - m_new);
    l = l * alpha + p;
#pragma unroll
    for (int j = 0; j < GEN_MAXJ; ++j) {
      int d = lane + 32 * j;
      if (d < hd) acc[j] = acc[j] * alpha + p * load_tile_elem(vtile, a.pool.dtype, hd, 1, rin, d);
    }
    m = m_new;
  }

  // merge the warps of this block
#pragma unroll
  for (int j = 0; j < GEN_MAXJ; ++j) {
    int d = lane + 32 * j;
    if (d < hd) o_s[warp * hd + d] = acc[j];
  }
  if (lane == 0) {
    ml_s[2 * warp] = m;
    ml_s[2 * warp + 1] = l;
  }
  __syncthreads();
  float mb = -1.0e30f;
#pragma unroll
  for (int w = 0; w < GEN_WARPS; ++w) mb = fmaxf(mb, ml_s[2 * w]);
  float lb = 0.0f;
  float wgt[GEN_WARPS];
#pragma unroll
  for (int w = 0; w < GEN_WARPS; ++w) {
    wgt[w] = exp2f(ml_s[2 * w] - mb);
    lb += ml_s[2 * w + 1] * wgt[w];
  }
  const int64_t qh_global = int64_t(seq) * a.q_heads + qh;
  float* out_row = a.out + qh_global * hd;
  if (a.splits == 1) {
    float inv = 1.0f / lb;
    for (int d = tid; d < hd; d += GEN_THREADS) {
      float o = 0.0f;
#pragma unroll
      for (int w = 0; w < GEN_WARPS; ++w) o += o_s[w * hd + d] * wgt[w];
      out_row[d] = o * inv;
    }
    return;
  }
  float* po = a.part.o + (qh_global * a.splits + split) * hd;
  for (int d = tid; d < hd; d += GEN_THREADS) {
    float o = 0.0f;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; ++w) o += o_s[w * hd + d] * wgt[w];
    po[d] = o;
  }
  if (tid == 0) {
    float* pml = a.part.ml + (qh_global * a.splits + split) * 2;
    pml[0] = mb;
    pml[1] = lb;
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    int old = atomicAdd(a.head_counters + qh_global, 1);
    is_last_s = (old == a.splits - 1);
  }
  __syncthreads();
  if (is_last_s) {
    __threadfence();
    merge_partials(a.part, qh_global, a.splits, hd, out_row, tid, GEN_THREADS);
    if (tid == 0) a.head_counters[qh_global] = 0;
  }
}

cudaError_t launch_attention_generic(const AttnArgs& a, int n_seq, cudaStream_t stream) {
  dim3 grid(a.q_heads, a.splits, n_seq);
  size_t smem = (size_t(a.pool.head_dim) * (1 + GEN_WARPS) + 2 * GEN_WARPS) * sizeof(float);
  attention_generic_kernel<<<grid, GEN_THREADS, smem, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace sgk
