// Paged split-K flash-decoding over u8 group-32 pages (head_dim 128 / 256, GQA group
// <= 8), with the per-token append (quantisation included) fused in.
//
// Same pipeline as the bf16 kernel (producer warp, one bulk async copy per page into a
// shared-memory ring, consumer warps, two-level split merge); what differs is the math
// of a page. The codes are never expanded element by element: a byte b becomes the fp16
// subnormal b * 2^-24 with ONE byte-permute (the byte dropped into the low mantissa bits of a
// zero half), two codes per instruction and exactly, and the affine metadata is applied
// around the tensor-core products:
//
//   scores   s[row][h] = 2^24 * sum_g scale_k[row][g] * (sum_{d in g} q[h][d] * code * 2^-24)
//                              + sum_g bias_k[row][g] * qsum[h][g]
//            one m16n8k16 fp16 product per 16 dims, one accumulator per group of 32, the
//            per-(row, group) scale applied to the accumulator in f32;
//   outputs  O[d][h]  += sum_row code[row][d] * (scale_v[row][g(d)] * p[row][h])   (tensor core,
//            the scale folded into the B operand of the group)
//            +  sum_row bias_v[row][g(d)] * p[row][h]  (f32, per thread, reduced over the warp
//            once at the end).
//
// The weights p * scale_v are multiplied by a power of two chosen from the largest scale
// the pool has ever stored (kept by the append kernels in PoolView::scale_max, and raised
// by the row a fused append is about to write), so they sit in the middle of the fp16
// range whatever the data; the accumulators are divided by it at the end.
// q is split into fp16 hi + lo parts (22 significant bits).
// Layouts: see layout.h (K codes row-major with the bank swizzle, V codes transposed
// [dim][row slot]).
//
// The reference has no u8 KV; this kernel computes cached_attention_one
// (src/decoder/attention_ops.rs:889-974) over the dequantised rows q*scale+bias
// (src/quantization.rs:173-179).
#include "mma_common.cuh"

namespace sgk {

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// two bytes of w -> the fp16 pair (byte_lo, byte_hi) * 2^-24: a byte in the low mantissa bits of
// an fp16 with a zero exponent field is the subnormal byte * 2^-24, exactly
__device__ __forceinline__ uint32_t codes_lo(uint32_t w) { return __byte_perm(w, 0u, 0x4140); }
__device__ __forceinline__ uint32_t codes_hi(uint32_t w) { return __byte_perm(w, 0u, 0x4342); }
constexpr float CODE_UNIT_INV = 16777216.0f;  // 2^24
// x -> fp16 hi (nearest) and fp16 lo = nearest(x - hi)
__device__ __forceinline__ void split_f16(float x, uint16_t& hi, uint16_t& lo) {
  __half h = __float2half_rn(x);
  __half l = __float2half_rn(x - __half2float(h));
  hi = __half_as_ushort(h);
  lo = __half_as_ushort(l);
}
__device__ __forceinline__ uint32_t pack_f16(float x0, float x1) {
  __half2 v = __floats2half2_rn(x0, x1);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void mma_bf16_k8(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t pack_bf16(float x0, float x1) {  // x0 in the low half
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(x1), "f"(x0));
  return r;
}
__device__ __forceinline__ float bf16_lo_f32(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi_f32(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

template <int HD>
struct U8Smem {
  static constexpr int G = HD / QGROUP;
  static constexpr int CODES = PAGE_TOKENS * HD;            // bytes of K or V codes
  static constexpr int SCALES = CODES;                      // bf16 [row][group]
  static constexpr int BIASES = CODES + PAGE_TOKENS * G * 2;  // bf16, K [row][group], V [group][row]
  static constexpr int TILE = CODES + PAGE_TOKENS * G * 4;
  static constexpr int STAGE = 2 * TILE;
  static constexpr int OPAD = HD + 4;
  static constexpr int QROW = HD * 2 + 64;                // fp16 row of Q, rows 64 bytes apart modulo 128
  static constexpr int Q_BYTES = 2 * 8 * QROW;            // hi and lo
  static constexpr int QSUM_BYTES = 8 * 8 * 4;            // [head][8 groups], absent groups zero
  static constexpr int O_BYTES = MMA_CONSUMERS * 8 * OPAD * 4;
  static constexpr int ML_BYTES = 512;  // per-warp {max, sum}, then the merge weights and the block's {max, sum}
  static constexpr int BAR_BYTES = 2 * MMA_MAX_STAGES * 8;
  static constexpr int NEW_BYTES = 2 * HD * 4;            // the K and V row of a fused append, f32
  static constexpr int RECV_BYTES = ClusterRecv<HD>::BYTES;  // what the other blocks of a cluster send for the merge
  static constexpr int FIXED = Q_BYTES + QSUM_BYTES + ML_BYTES + BAR_BYTES + 64 + NEW_BYTES + RECV_BYTES;
  __host__ __device__ static size_t ring_bytes(int stages) {
    size_t r = size_t(stages) * STAGE;
    return r > size_t(O_BYTES) ? r : size_t(O_BYTES);
  }
  static size_t total(int stages) { return ring_bytes(stages) + FIXED + 1024; }
};

// Quantises N groups of 32 values at once (lane l holds element l of every group), with the
// arithmetic of the append kernel.
template <int N>
__device__ __forceinline__ void quantize_groups(const float (&x)[N], uint32_t (&code)[N], uint32_t (&meta)[N]) {
  float lo[N], hi[N];
  // warp-wide float min / max in one instruction each (sm_100a)
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

// The G bf16 scales of one row as f32, from one 16-byte (G = 8) or 8-byte (G = 4) load.
template <int G>
__device__ __forceinline__ void load_row_scales(const uint8_t* p, float (&sc)[G]) {
  if (G == 8) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    sc[0] = bf16_lo_f32(w.x), sc[1] = bf16_hi_f32(w.x), sc[2] = bf16_lo_f32(w.y), sc[3] = bf16_hi_f32(w.y);
    sc[4 % G] = bf16_lo_f32(w.z), sc[5 % G] = bf16_hi_f32(w.z), sc[6 % G] = bf16_lo_f32(w.w),
           sc[7 % G] = bf16_hi_f32(w.w);
  } else {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    sc[0] = bf16_lo_f32(w.x), sc[1] = bf16_hi_f32(w.x), sc[2] = bf16_lo_f32(w.y), sc[3] = bf16_hi_f32(w.y);
  }
}

template <int HD, bool CLUSTER, bool PEERS>
__global__ void __launch_bounds__(MMA_THREADS, 2) attention_u8_kernel(AttnArgs a) {
  using S = U8Smem<HD>;
  constexpr int G = S::G;
  constexpr int KSTEPS = HD / 16;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int nst = a.n_stages;
  uint8_t* fixed = ring + S::ring_bytes(nst);
  uint8_t* q_hi = fixed;                          // [8] rows of QROW bytes (fp16)
  uint8_t* q_lo = fixed + 8 * S::QROW;
  float* qsum_s = reinterpret_cast<float*>(fixed + S::Q_BYTES);                 // [8][8]
  float* o_s = reinterpret_cast<float*>(ring);    // aliases the ring once it has drained
  float* ml_s = reinterpret_cast<float*>(fixed + S::Q_BYTES + S::QSUM_BYTES);   // [warps][8][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed + S::Q_BYTES + S::QSUM_BYTES + S::ML_BYTES);
  int* flags = reinterpret_cast<int*>(bars + 2 * MMA_MAX_STAGES);
  float* new_s = reinterpret_cast<float*>(flags + 16);   // [K row | V row] of the append, staged once
  float* new_big = reinterpret_cast<float*>(flags + 8);  // [consumer warp] max |x| of its part of that row
  float* recv_s = reinterpret_cast<float*>(fixed + S::FIXED - S::RECV_BYTES);
  volatile int* abort_flag = flags;

  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef SGK_TRACE
  if (tid == 0) {
    SGK_TP(0);
    if (a.trace) {
      unsigned long long gt;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
      a.trace[((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 15] = gt;
      unsigned smid;
      asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
      a.trace[((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 13] = smid;
    }
  }
#endif
  const int gqa = a.q_heads / a.pool.kv_heads;
  const int slot = a.slots ? a.slots[seq] : a.slot0;
  int32_t* len_ptr = a.pool.lens + int64_t(slot) * a.pool.layers + a.layer;
  const bool do_append = a.k_new != nullptr;
  if (a.pdl_trigger) pdl_launch_dependents();

  const int64_t len_old = *reinterpret_cast<const volatile int32_t*>(len_ptr);
  const int64_t len = len_old + (do_append ? 1 : 0);
  int64_t ws = a.sliding_window > 0 ? (len > a.sliding_window ? len - a.sliding_window : 0) : a.window_start;
  if (ws >= len) ws = len > 0 ? len - 1 : 0;
  const int64_t p_first = ws / PAGE_TOKENS;
  const int64_t p_last = (len - 1) / PAGE_TOKENS;
  const int64_t n_pages = p_last - p_first + 1;
  // Sequences of one launch may differ a lot in length: each is cut into its own number of
  // splits of about pages_per_split pages, and the blocks beyond that number have nothing to do.
  int splits = a.splits;
  if (a.pages_per_split > 0) {
    const int64_t want = (n_pages + a.pages_per_split - 1) / a.pages_per_split;
    splits = static_cast<int>(want < 1 ? 1 : (want > a.splits ? a.splits : want));
  }
  if (split >= splits) return;
  const int64_t pb = p_first + (n_pages * split) / splits;
  const int64_t pe = p_first + (n_pages * (split + 1)) / splits;
  const int my_pages = static_cast<int>(pe - pb);
  const int32_t* table = a.pool.tables + int64_t(slot) * a.pool.table_stride;
  const int64_t head_off = int64_t(a.layer) * a.pool.layer_bytes + int64_t(kvh) * 2 * a.pool.tile_bytes;
  const int64_t append_page_index = len_old / PAGE_TOKENS;
  const bool owns_append = do_append && append_page_index >= pb && append_page_index < pe;
  const float* kn = new_s;
  const float* vn = new_s + HD;

  int32_t first_entry = -1;
  float smax = 0.0f;
  uint32_t smax_pool = 0;   // the pool's largest scale (f32 bits) as this launch found it
  if (warp == MMA_CONSUMERS) {
    if (lane == 0) {
      flags[0] = 0;
      flags[1] = 0;
      flags[5] = 0;   // set once the quantised row of a fused append is parked in shared memory
      for (int s = 0; s < nst; ++s) {
        mbar_init(smem_u32(bars + s), 1);
        mbar_init(smem_u32(bars + MMA_MAX_STAGES + s), 1);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (lane < my_pages) first_entry = table[pb + lane];
  } else {
    // Q of the group: scaled, fp16 hi/lo, rows of absent heads zero. One fp16 alone (11 bits)
    // would put an error of |logit| * 2^-12 on every logit, too much for rows with a large range.
    constexpr int NV = HD / 64;
    const float* q = a.q + (int64_t(seq) * a.q_heads + int64_t(kvh) * gqa) * HD;
    // q, the row to append and the pool's largest scale come from the launch before this one; the
    // cursor, the block table and the pages the producer has started to copy do not
    if (a.pdl_wait) pdl_wait();
    if (tid == 0) SGK_TP(8);
    smax_pool = *reinterpret_cast<const volatile uint32_t*>(a.pool.scale_max);
    smax = __uint_as_float(smax_pool);
    float4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int f = (tid + k * MMA_CONSUMERS * 32) * 4;
      v[k] = (f / HD < gqa) ? __ldg(reinterpret_cast<const float4*>(q + f)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // The row of a fused append comes into shared memory with the same round trip as Q: read
    // where it is quantised, element by element, each read would pay the latency again.
    const bool loads_row = owns_append && tid * 4 < 2 * HD;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    int32_t append_page = -1;
    if (loads_row) {
      const int64_t row_off = int64_t(seq) * a.pool.kv_heads * HD + kvh * HD;
      const float* src = tid * 4 < HD ? a.k_new + row_off + tid * 4 : a.v_new + row_off + (tid * 4 - HD);
      x = __ldg(reinterpret_cast<const float4*>(src));
    }
    if (owns_append && tid == 0) append_page = table[append_page_index];
    if (loads_row) {
      *reinterpret_cast<float4*>(new_s + tid * 4) = x;
      // bound of the scales the row will get: (max - min) / 255 <= 2 max|x| / 255
      float big = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
      if (lane == 0) new_big[warp] = big;
    }
    if (owns_append && tid == 0) flags[2] = append_page;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int f = (tid + k * MMA_CONSUMERS * 32) * 4;
      const int h = f / HD, d = f % HD;
      uint16_t hi[4], lo[4];
      split_f16(v[k].x * a.scale_log2e, hi[0], lo[0]);
      split_f16(v[k].y * a.scale_log2e, hi[1], lo[1]);
      split_f16(v[k].z * a.scale_log2e, hi[2], lo[2]);
      split_f16(v[k].w * a.scale_log2e, hi[3], lo[3]);
      *reinterpret_cast<uint2*>(q_hi + h * S::QROW + d * 2) =
          make_uint2(uint32_t(hi[0]) | (uint32_t(hi[1]) << 16), uint32_t(hi[2]) | (uint32_t(hi[3]) << 16));
      *reinterpret_cast<uint2*>(q_lo + h * S::QROW + d * 2) =
          make_uint2(uint32_t(lo[0]) | (uint32_t(lo[1]) << 16), uint32_t(lo[2]) | (uint32_t(lo[3]) << 16));
    }
  }
  // The producer only announces that the barriers exist and starts copying; the consumers wait
  // here for that and for each other's part of Q and of the appended row.
  if (warp == MMA_CONSUMERS) {
    __syncwarp();
    asm volatile("bar.arrive 3, %0;" ::"r"(MMA_THREADS) : "memory");
  } else {
    asm volatile("bar.sync 3, %0;" ::"r"(MMA_THREADS) : "memory");
  }
  // The row a fused append is about to write may carry a larger scale than any stored one.
  if (owns_append && warp < MMA_CONSUMERS) {
    float big = new_big[0];
#pragma unroll
    for (int w = 1; w < MMA_CONSUMERS; ++w)
      if (w * 32 * 4 < 2 * HD) big = fmaxf(big, new_big[w]);
    smax = fmaxf(smax, big * (2.02f / 255.0f));   // 1 % above the bound covers the bf16 rounding of a scale
  }
  // qsum[h][g] = sum over the group of the fp16 value of q (hi + lo), as the tensor core sees it;
  // each consumer thread keeps the two it feeds to the bias product, as three bf16 parts.
  uint32_t qs_hi = 0, qs_mid = 0, qs_lo = 0;
  if (warp < MMA_CONSUMERS) {
    if (tid < 64) {
      const int h = tid >> 3, grp = tid & 7;
      float sum = 0.0f;
      if (grp < G) {
        const __half2* ph = reinterpret_cast<const __half2*>(q_hi + h * S::QROW) + grp * (QGROUP / 2);
        const __half2* pl = reinterpret_cast<const __half2*>(q_lo + h * S::QROW) + grp * (QGROUP / 2);
#pragma unroll
        for (int d = 0; d < QGROUP / 2; ++d) {
          const float2 x = __half22float2(ph[d]), y = __half22float2(pl[d]);
          sum += (x.x + y.x) + (x.y + y.y);
        }
      }
      qsum_s[h * 8 + grp] = sum;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(MMA_CONSUMERS * 32) : "memory");
    // B fragment of the bias product: (k = groups 2t, 2t+1; n = head g)
    const float2 qs = *reinterpret_cast<const float2*>(qsum_s + (lane >> 2) * 8 + 2 * (lane & 3));
    qs_hi = pack_bf16(qs.x, qs.y);
    const float r0 = qs.x - bf16_lo_f32(qs_hi), r1 = qs.y - bf16_hi_f32(qs_hi);
    qs_mid = pack_bf16(r0, r1);
    qs_lo = pack_bf16(r0 - bf16_lo_f32(qs_mid), r1 - bf16_hi_f32(qs_mid));
  }
  if (tid == 0) SGK_TP(1);

  // The row of a fused append is quantised now, by the consumer warp with the fewest pages, while the
  // first pages are still on their way: codes and metadata go to the row's page in global memory at
  // once and are parked in shared memory (over the f32 row, which nothing reads any more) for the
  // warp that will meet the page in the ring. Done where the page is consumed, at the very end of
  // the block every other block of the sequence waits for, the quantiser's divides and its stores
  // delayed the whole launch.
  uint8_t* park = reinterpret_cast<uint8_t*>(new_s);   // [K codes HD | V codes HD | meta 2G x u32]
  if (owns_append && warp == MMA_CONSUMERS - 1) {
    const int rin = static_cast<int>(len_old % PAGE_TOKENS);
    const int32_t page = flags[2];
    float x[2 * G];
    uint32_t code[2 * G], meta[2 * G];
#pragma unroll
    for (int grp = 0; grp < G; ++grp) {
      x[grp] = kn[grp * QGROUP + lane];
      x[G + grp] = vn[grp * QGROUP + lane];
    }
    __syncwarp();
    quantize_groups<2 * G>(x, code, meta);
    uint32_t biggest = 0;
    const bool page_ok = page >= 0 && page < a.num_pages;   // a bad entry is reported by the producer, which meets it too
    uint8_t* gk = a.pool.base + int64_t(page_ok ? page : 0) * a.pool.page_bytes + head_off;
    uint8_t* gv = gk + S::TILE;
#pragma unroll
    for (int grp = 0; grp < G; ++grp) {
      const int dim = grp * QGROUP + lane;
      park[dim] = static_cast<uint8_t>(code[grp]);
      park[HD + dim] = static_cast<uint8_t>(code[G + grp]);
      if (page_ok) {
        gk[u8_k_code_index(rin, dim, HD)] = static_cast<uint8_t>(code[grp]);
        gv[u8_v_code_index(rin, dim, HD)] = static_cast<uint8_t>(code[G + grp]);
      }
      biggest = max(biggest, max((meta[grp] & 0xffffu) << 16, (meta[G + grp] & 0xffffu) << 16));
    }
    // lane grp writes the metadata of group grp (every lane holds every group's)
#pragma unroll
    for (int grp = 0; grp < G; ++grp) {
      if (lane == grp) {
        const uint32_t mk = meta[grp], mv = meta[G + grp];
        reinterpret_cast<uint32_t*>(park + 2 * HD)[grp] = mk;
        reinterpret_cast<uint32_t*>(park + 2 * HD)[G + grp] = mv;
        if (page_ok) {
          *reinterpret_cast<uint16_t*>(gk + u8_scale_offset(rin, grp, HD)) = static_cast<uint16_t>(mk & 0xffffu);
          *reinterpret_cast<uint16_t*>(gk + u8_bias_offset(0, rin, grp, HD)) = static_cast<uint16_t>(mk >> 16);
          *reinterpret_cast<uint16_t*>(gv + u8_scale_offset(rin, grp, HD)) = static_cast<uint16_t>(mv & 0xffffu);
          *reinterpret_cast<uint16_t*>(gv + u8_bias_offset(1, rin, grp, HD)) = static_cast<uint16_t>(mv >> 16);
        }
      }
    }
    if (lane == 0 && page_ok && biggest > smax_pool) atomicMax(a.pool.scale_max, biggest);
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      *reinterpret_cast<volatile int*>(flags + 5) = 1;
    }
  }

  if (warp == MMA_CONSUMERS) {
    // ---------------- producer warp ----------------
    produce_pages<S::STAGE>(a, table, pb, my_pages, first_entry, ring, bars, nst, head_off, abort_flag, lane);
    if (a.pdl_wait) pdl_wait();   // the tail writes to memory the earlier launch may still be using
    SGK_TP(12);
  } else {
    // ---------------- consumer warps ----------------
    const int g = lane >> 2, t = lane & 3;
    // power of two that puts scale * p in the middle of the fp16 range
    int e = static_cast<int>((__float_as_uint(smax) >> 23) & 0xffu) - 127;
    e = max(-60, min(60, e));
    const float pscale = exp2f(static_cast<float>(10 - e));
    const float inv_pscale = exp2f(static_cast<float>(e - 10)) * CODE_UNIT_INV;

    float o_acc[KSTEPS][4];
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j) o_acc[j][0] = o_acc[j][1] = o_acc[j][2] = o_acc[j][3] = 0.0f;
    // sum_row bias_v[row][grp] * p[row][head]: (m = group g, n = heads 2t, 2t+1) in [0], [1]
    float cacc[4] = {0.f, 0.f, 0.f, 0.f};
    float m0 = -1.0e30f, m1 = -1.0e30f, l0 = 0.0f, l1 = 0.0f;
    // this thread's fixed offsets inside a stage
    const int k_off = g * HD + 8 * t;                        // + (granule ^ (g & 3)) * 32; row g+8: + 8 * HD
    const int q_off = g * S::QROW + 16 * t;                  // + 64 * group
    const int kb_off = S::BIASES + (g * G + 2 * t) * 2;      // K biases of (row g; groups 2t, 2t+1)
    const int vb_off = S::TILE + S::BIASES + (g * PAGE_TOKENS + 2 * t) * 2;  // V biases of (group g; rows 2t, 2t+1)
    const bool kb_on = 2 * t < G, vb_on = g < G;

#ifdef SGK_TRACE
    long long tp_wait = 0, tp_s = 0, tp_soft = 0, tp_pv = 0, tp_prev = clock64();
#define U8_PHASE(acc) do { long long now_ = clock64(); acc += now_ - tp_prev; tp_prev = now_; } while (0)
#else
#define U8_PHASE(acc) do {} while (0)
#endif
    int stage = warp;
    uint32_t parity = 0;
    bool ready = false;  // the page's barrier was already seen complete during the previous page
    for (int i = warp; i < my_pages; i += MMA_CONSUMERS) {
      const bool ok = ready || mbar_wait(smem_u32(bars + stage), parity, abort_flag, a.status);
      U8_PHASE(tp_wait);
      if (i == 0) SGK_TP(2);
      uint8_t* ktile = ring + size_t(stage) * S::STAGE;
      uint8_t* vtile = ktile + S::TILE;
      const int64_t page_index = pb + i;
      const int64_t row_base = page_index * PAGE_TOKENS;

      if (ok && owns_append && page_index == append_page_index) {
        // The new row (quantised in the prologue, already on its way to the page) joins the staged copy.
        const int rin = static_cast<int>(len_old % PAGE_TOKENS);
        uint32_t spins = 0;
        while (*reinterpret_cast<volatile int*>(flags + 5) == 0) {
          if (++spins > WAIT_SPINS) {
            *abort_flag = 1;
            atomicExch(a.status, DEV_ERR_WAIT_TIMEOUT);
            break;
          }
        }
        __syncwarp();
#pragma unroll
        for (int grp = 0; grp < G; ++grp) {
          const int dim = grp * QGROUP + lane;
          ktile[u8_k_code_index(rin, dim, HD)] = park[dim];
          vtile[u8_v_code_index(rin, dim, HD)] = park[HD + dim];
        }
        if (lane < G) {
          const uint32_t mk = reinterpret_cast<const uint32_t*>(park + 2 * HD)[lane];
          const uint32_t mv = reinterpret_cast<const uint32_t*>(park + 2 * HD)[G + lane];
          *reinterpret_cast<uint16_t*>(ktile + u8_scale_offset(rin, lane, HD)) = static_cast<uint16_t>(mk & 0xffffu);
          *reinterpret_cast<uint16_t*>(ktile + u8_bias_offset(0, rin, lane, HD)) = static_cast<uint16_t>(mk >> 16);
          *reinterpret_cast<uint16_t*>(vtile + u8_scale_offset(rin, lane, HD)) = static_cast<uint16_t>(mv & 0xffffu);
          *reinterpret_cast<uint16_t*>(vtile + u8_bias_offset(1, rin, lane, HD)) = static_cast<uint16_t>(mv >> 16);
        }
        __syncwarp();
      }

      if (ok) {
        // ---- scores. Bias part on the tensor cores: [16 rows x groups] . [groups x 8 heads]
        //      in bf16 with the group sums of q in three bf16 parts (24 bits). ----
        float sb[4] = {0.f, 0.f, 0.f, 0.f};
        {
          const uint32_t a0 = kb_on ? *reinterpret_cast<const uint32_t*>(ktile + kb_off) : 0u;
          const uint32_t a1 = kb_on ? *reinterpret_cast<const uint32_t*>(ktile + kb_off + 8 * G * 2) : 0u;
          mma_bf16_k8(sb, a0, a1, qs_hi);
          mma_bf16_k8(sb, a0, a1, qs_mid);
          mma_bf16_k8(sb, a0, a1, qs_lo);
        }
        // Code part: one accumulator per group of 32 dims (two k-steps, q hi and lo), the
        // per-(row, group) scale applied to it in f32. A lane's 8 bytes of a group are its
        // dims 8t .. 8t+7: the first word is k-step 0, the second k-step 1.
        float acc[G][4];
#pragma unroll
        for (int grp = 0; grp < G; ++grp) acc[grp][0] = acc[grp][1] = acc[grp][2] = acc[grp][3] = 0.0f;
        // Four groups at a time, and for them first every product of the first k-step with q hi,
        // then with q lo, then the second k-step: the tensor-core instructions of one accumulator
        // depend on each other, so products of different groups are issued between them.
#pragma unroll
        for (int set = 0; set < G / 4; ++set) {
          uint2 w0[4], w1[4];
          uint4 qh[4], ql[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int grp = 4 * set + u;
            const int phys = (grp & ~3) | ((grp ^ g) & 3);
            w0[u] = *reinterpret_cast<const uint2*>(ktile + k_off + phys * 32);
            w1[u] = *reinterpret_cast<const uint2*>(ktile + k_off + phys * 32 + 8 * HD);
            qh[u] = *reinterpret_cast<const uint4*>(q_hi + q_off + 64 * grp);
            ql[u] = *reinterpret_cast<const uint4*>(q_lo + q_off + 64 * grp);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mma_f16(acc[4 * set + u], codes_lo(w0[u].x), codes_lo(w1[u].x), codes_hi(w0[u].x), codes_hi(w1[u].x),
                    qh[u].x, qh[u].y);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mma_f16(acc[4 * set + u], codes_lo(w0[u].x), codes_lo(w1[u].x), codes_hi(w0[u].x), codes_hi(w1[u].x),
                    ql[u].x, ql[u].y);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mma_f16(acc[4 * set + u], codes_lo(w0[u].y), codes_lo(w1[u].y), codes_hi(w0[u].y), codes_hi(w1[u].y),
                    qh[u].z, qh[u].w);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mma_f16(acc[4 * set + u], codes_lo(w0[u].y), codes_lo(w1[u].y), codes_hi(w0[u].y), codes_hi(w1[u].y),
                    ql[u].z, ql[u].w);
        }
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
          float sc0[G], sc1[G];
          load_row_scales<G>(ktile + S::SCALES + g * G * 2, sc0);
          load_row_scales<G>(ktile + S::SCALES + (g + 8) * G * 2, sc1);
#pragma unroll
          for (int grp = 0; grp < G; ++grp) {
            s[0] = fmaf(sc0[grp], acc[grp][0], s[0]);
            s[1] = fmaf(sc0[grp], acc[grp][1], s[1]);
            s[2] = fmaf(sc1[grp], acc[grp][2], s[2]);
            s[3] = fmaf(sc1[grp], acc[grp][3], s[3]);
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) s[r] = fmaf(s[r], CODE_UNIT_INV, sb[r]);  // the codes were in units of 2^-24
        U8_PHASE(tp_s);
        if (row_base < ws || row_base + PAGE_TOKENS > len) {
          int64_t ra = row_base + g, rb = row_base + g + 8;
          if (ra < ws || ra >= len) s[0] = s[1] = -1.0e30f;
          if (rb < ws || rb >= len) s[2] = s[3] = -1.0e30f;
        }
        float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const bool grew = (mn0 > m0) || (mn1 > m1);
        if (__any_sync(0xffffffffu, grew)) {
          const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
          l0 *= al0;
          l1 *= al1;
#pragma unroll
          for (int j = 0; j < KSTEPS; ++j) {
            o_acc[j][0] *= al0;
            o_acc[j][2] *= al0;
            o_acc[j][1] *= al1;
            o_acc[j][3] *= al1;
          }
          cacc[0] *= al0;
          cacc[1] *= al1;
          m0 = mn0;
          m1 = mn1;
        }
        float p[4];
        p[0] = exp2f(s[0] - m0);
        p[2] = exp2f(s[2] - m0);
        p[1] = exp2f(s[1] - m1);
        p[3] = exp2f(s[3] - m1);
        l0 += p[0] + p[2];
        l1 += p[1] + p[3];
        U8_PHASE(tp_soft);
        {
          // look at the next page's barrier now: the answer arrives while the products below run
          int ns = stage + MMA_CONSUMERS;
          uint32_t np = parity;
          if (ns >= nst) {
            ns -= nst;
            np ^= 1;
          }
          ready = (i + MMA_CONSUMERS < my_pages) && mbar_test_wait(smem_u32(bars + ns), np);
        }
        // ---- outputs. Bias part: [groups x 16 rows] . [16 rows x 8 heads] in bf16 with p in two
        //      bf16 parts; the movmatrix turns (row; heads 2t, 2t+1) into (rows 2t, 2t+1; head). ----
        {
          const uint32_t ph0 = pack_bf16(p[0], p[1]), ph1 = pack_bf16(p[2], p[3]);
          const uint32_t pl0 = pack_bf16(p[0] - bf16_lo_f32(ph0), p[1] - bf16_hi_f32(ph0));
          const uint32_t pl1 = pack_bf16(p[2] - bf16_lo_f32(ph1), p[3] - bf16_hi_f32(ph1));
          const uint32_t a0 = vb_on ? *reinterpret_cast<const uint32_t*>(ktile + vb_off) : 0u;
          const uint32_t a2 = vb_on ? *reinterpret_cast<const uint32_t*>(ktile + vb_off + 16) : 0u;
          mma_bf16(cacc, a0, 0u, a2, 0u, movmatrix_trans(ph0), movmatrix_trans(ph1));
          mma_bf16(cacc, a0, 0u, a2, 0u, movmatrix_trans(pl0), movmatrix_trans(pl1));
        }
        // Code part: scale_v folded into the weights of each group (fp16, times the pool's
        // power of two), then V^T codes . weights on the tensor cores.
        uint32_t pb0[G], pb1[G];
        {
          float sv0[G], sv1[G];
          load_row_scales<G>(vtile + S::SCALES + g * G * 2, sv0);
          load_row_scales<G>(vtile + S::SCALES + (g + 8) * G * 2, sv1);
          const uint32_t pw0 = pack_f16(p[0], p[1]), pw1 = pack_f16(p[2], p[3]);
#pragma unroll
          for (int grp = 0; grp < G; ++grp) {
            const float x0 = sv0[grp] * pscale, x1 = sv1[grp] * pscale;
            pb0[grp] = movmatrix_trans(hmul2_u32(pw0, pack_f16(x0, x0)));   // rows 0-7
            pb1[grp] = movmatrix_trans(hmul2_u32(pw1, pack_f16(x1, x1)));   // rows 8-15
          }
        }
#pragma unroll
        for (int jq = 0; jq < KSTEPS / 4; ++jq) {
          const uint4 wa = *reinterpret_cast<const uint4*>(vtile + ((jq * 2) * 32 + lane) * 16);
          const uint4 wb = *reinterpret_cast<const uint4*>(vtile + ((jq * 2 + 1) * 32 + lane) * 16);
          mma_f16(o_acc[4 * jq], codes_lo(wa.x), codes_lo(wa.y), codes_hi(wa.x), codes_hi(wa.y), pb0[2 * jq],
                  pb1[2 * jq]);
          mma_f16(o_acc[4 * jq + 1], codes_lo(wa.z), codes_lo(wa.w), codes_hi(wa.z), codes_hi(wa.w), pb0[2 * jq],
                  pb1[2 * jq]);
          mma_f16(o_acc[4 * jq + 2], codes_lo(wb.x), codes_lo(wb.y), codes_hi(wb.x), codes_hi(wb.y), pb0[2 * jq + 1],
                  pb1[2 * jq + 1]);
          mma_f16(o_acc[4 * jq + 3], codes_lo(wb.z), codes_lo(wb.w), codes_hi(wb.z), codes_hi(wb.w), pb0[2 * jq + 1],
                  pb1[2 * jq + 1]);
        }
      }
      else ready = false;
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bars + MMA_MAX_STAGES + stage));
      U8_PHASE(tp_pv);
      stage += MMA_CONSUMERS;   // the stage count is a multiple of the consumer count
      if (stage >= nst) {
        stage -= nst;
        parity ^= 1;
      }
    }
    if (warp == 0) SGK_TP(3);
#ifdef SGK_TRACE
    if (a.trace && warp == 0 && lane == 0) {
      unsigned long long* tr = a.trace + ((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16;
      tr[8] = tp_wait, tr[9] = tp_s, tr[10] = tp_soft, tr[11] = tp_pv, tr[12] = (my_pages + MMA_CONSUMERS - 1) / MMA_CONSUMERS;
    }
#endif

    // ---- hand this warp's state to the merge buffer (it aliases the ring) ----
    asm volatile("bar.sync 1, %0;" ::"r"(MMA_CONSUMERS * 32) : "memory");
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, off);
      l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    float* ow = o_s + warp * 8 * S::OPAD;
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j) {
      // the bias sums of group j/2 sit in the lanes of quad j/2
      const float c0 = __shfl_sync(0xffffffffu, cacc[0], (j / 2) * 4 + t);
      const float c1 = __shfl_sync(0xffffffffu, cacc[1], (j / 2) * 4 + t);
      ow[(2 * t) * S::OPAD + 16 * j + g] = o_acc[j][0] * inv_pscale + c0;
      ow[(2 * t + 1) * S::OPAD + 16 * j + g] = o_acc[j][1] * inv_pscale + c1;
      ow[(2 * t) * S::OPAD + 16 * j + g + 8] = o_acc[j][2] * inv_pscale + c0;
      ow[(2 * t + 1) * S::OPAD + 16 * j + g + 8] = o_acc[j][3] * inv_pscale + c1;
    }
    if (g == 0) {
      ml_s[(warp * 8 + 2 * t) * 2] = m0;
      ml_s[(warp * 8 + 2 * t) * 2 + 1] = l0;
      ml_s[(warp * 8 + 2 * t + 1) * 2] = m1;
      ml_s[(warp * 8 + 2 * t + 1) * 2 + 1] = l1;
    }
  }
  __syncthreads();
  finish_block<HD, CLUSTER, PEERS>(a, o_s, ml_s, S::OPAD, flags, seq, kvh, split, gqa, do_append, len_ptr, len, tid,
                                   splits, recv_s);
  if (tid == 0) SGK_TP(10);
  if (PEERS) peers_finish(a, tid, flags);
}

bool attention_u8_supported(int dtype, int head_dim, int gqa) {
  return dtype == KV_U8G32 && (head_dim == 128 || head_dim == 256) && gqa >= 1 && gqa <= 8;
}

int attention_u8_max_stages(int head_dim) {
  size_t budget = 113 * 1024;  // two blocks per SM
  size_t fixed = head_dim == 128 ? U8Smem<128>::FIXED : U8Smem<256>::FIXED;
  size_t stage = head_dim == 128 ? U8Smem<128>::STAGE : U8Smem<256>::STAGE;
  int n = static_cast<int>((budget - fixed - 1024) / stage);
  if (n > MMA_MAX_STAGES) n = MMA_MAX_STAGES;
  return n / MMA_CONSUMERS * MMA_CONSUMERS;  // a stage always belongs to the same warp
}

int attention_u8_resident_blocks(int head_dim, int n_stages) {
  int blocks = 0;
  cudaError_t e = head_dim == 128
                      ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_u8_kernel<128, false, false>, MMA_THREADS,
                                                                      U8Smem<128>::total(n_stages))
                      : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_u8_kernel<256, false, false>, MMA_THREADS,
                                                                      U8Smem<256>::total(n_stages));
  return e == cudaSuccess ? blocks : 0;
}

// How many clusters of `splits` blocks the device can hold at once (0: such a launch would fail).
int attention_u8_max_clusters(int head_dim, int n_stages, int splits) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(splits, 1, 1);
  cfg.blockDim = dim3(MMA_THREADS);
  cfg.dynamicSmemBytes = head_dim == 128 ? U8Smem<128>::total(n_stages) : U8Smem<256>::total(n_stages);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e = head_dim == 128 ? cudaOccupancyMaxActiveClusters(&n, attention_u8_kernel<128, true, false>, &cfg)
                                  : cudaOccupancyMaxActiveClusters(&n, attention_u8_kernel<256, true, false>, &cfg);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

cudaError_t attention_u8_configure() {
  const void* kernels[6] = {reinterpret_cast<const void*>(attention_u8_kernel<128, false, false>), reinterpret_cast<const void*>(attention_u8_kernel<256, false, false>),
                            reinterpret_cast<const void*>(attention_u8_kernel<128, true, false>), reinterpret_cast<const void*>(attention_u8_kernel<256, true, false>),
                            reinterpret_cast<const void*>(attention_u8_kernel<128, false, true>), reinterpret_cast<const void*>(attention_u8_kernel<256, false, true>)};
  for (int i = 0; i < 6; ++i) {
    cudaError_t e = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    // clusters of more than 8 blocks (up to 16 splits merge as one cluster) are an opt-in
    if (i == 2 || i == 3) e = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// A launch whose blocks wait for one another (shared merge) is a cooperative launch: the driver
// then places all its blocks at once or not at all, also next to launches of other streams. A
// launch whose splits merge through distributed shared memory is a cluster launch.
static cudaError_t launch_one(void (*kernel)(AttnArgs), dim3 grid, size_t smem, const AttnArgs& a,
                              cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(MMA_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (a.cluster_merge) {
    // the splits of a (sequence, KV head) are the x extent of the grid and of the cluster
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = grid.x;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    n_attr += 1;
  } else if (a.shared_merge == 1) {
    attr[n_attr].id = cudaLaunchAttributeCooperative;
    attr[n_attr].val.cooperative = 1;
    n_attr += 1;
  }
  if (a.pdl_wait) {
    // may start while the launch before it in the stream still runs; the kernel waits for that
    // launch itself, after its first copies are on their way
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    n_attr += 1;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

cudaError_t launch_attention_u8(const AttnArgs& a, int n_seq, cudaStream_t stream) {
  dim3 grid(a.splits, a.pool.kv_heads, n_seq);
  if (a.pool.head_dim == 128) {
    if (a.n_peers > 0) return launch_one(attention_u8_kernel<128, false, true>, grid, U8Smem<128>::total(a.n_stages), a, stream);
    return a.cluster_merge ? launch_one(attention_u8_kernel<128, true, false>, grid, U8Smem<128>::total(a.n_stages), a, stream)
                           : launch_one(attention_u8_kernel<128, false, false>, grid, U8Smem<128>::total(a.n_stages), a, stream);
  } else {
    if (a.n_peers > 0) return launch_one(attention_u8_kernel<256, false, true>, grid, U8Smem<256>::total(a.n_stages), a, stream);
    return a.cluster_merge ? launch_one(attention_u8_kernel<256, true, false>, grid, U8Smem<256>::total(a.n_stages), a, stream)
                           : launch_one(attention_u8_kernel<256, false, false>, grid, U8Smem<256>::total(a.n_stages), a, stream);
  }
  return cudaGetLastError();
}

}  // namespace sgk
