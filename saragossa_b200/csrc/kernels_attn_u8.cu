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

template <int HD>
struct U8Smem {
  static constexpr int G = HD / QGROUP;
  static constexpr int CODES = PAGE_TOKENS * HD;          // bytes of K or V codes
  static constexpr int TILE = CODES + PAGE_TOKENS * G * 4;  // + {scale, bias} pairs
  static constexpr int STAGE = 2 * TILE;
  static constexpr int OPAD = HD + 4;
  static constexpr int QROW = HD * 2 + 32;                // padded fp16 row of Q (bank spread)
  static constexpr int Q_BYTES = 2 * 8 * QROW;            // hi and lo
  static constexpr int QSUM_BYTES = 8 * G * 4;
  static constexpr int O_BYTES = MMA_CONSUMERS * 8 * OPAD * 4;
  static constexpr int ML_BYTES = 512;  // per-warp {max, sum}, then the merge weights and the block's {max, sum}
  static constexpr int BAR_BYTES = 2 * MMA_MAX_STAGES * 8;
  static constexpr int FIXED = Q_BYTES + QSUM_BYTES + ML_BYTES + BAR_BYTES + 64;
  __host__ __device__ static size_t ring_bytes(int stages) {
    size_t r = size_t(stages) * STAGE;
    return r > size_t(O_BYTES) ? r : size_t(O_BYTES);
  }
  static size_t total(int stages) { return ring_bytes(stages) + FIXED + 1024; }
};

// Largest scale (f32) of the 2*G groups of a row about to be appended; every lane gets it.
template <int HD>
__device__ __forceinline__ float new_row_max_scale(const float* kn, const float* vn, int lane) {
  float best = 0.0f;
#pragma unroll
  for (int g = 0; g < 2 * (HD / QGROUP); ++g) {
    const float* src = g < HD / QGROUP ? kn + g * QGROUP : vn + (g - HD / QGROUP) * QGROUP;
    float x = src[lane], lo = x, hi = x;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
    }
    float bias = bf16_bits_to_f32(f32_to_bf16_bits(lo));
    float raw = __fdiv_rn(__fsub_rn(hi, bias), 255.0f);
    best = fmaxf(best, bf16_bits_to_f32(f32_to_bf16_bits(fmaxf(raw, 0x1p-40f))));
  }
  return best;
}

// Quantises 32 values (one per lane), same arithmetic as the append kernel.
__device__ __forceinline__ uint32_t quantize_lane(float x, uint32_t* meta_out) {
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

template <int HD>
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
  float* qsum_s = reinterpret_cast<float*>(fixed + S::Q_BYTES);                 // [8][G]
  float* o_s = reinterpret_cast<float*>(ring);    // aliases the ring once it has drained
  float* ml_s = reinterpret_cast<float*>(fixed + S::Q_BYTES + S::QSUM_BYTES);   // [warps][8][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed + S::Q_BYTES + S::QSUM_BYTES + S::ML_BYTES);
  int* flags = reinterpret_cast<int*>(bars + 2 * MMA_MAX_STAGES);
  volatile int* abort_flag = flags;

  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gqa = a.q_heads / a.pool.kv_heads;
  const int slot = a.slots ? a.slots[seq] : a.slot0;
  int32_t* len_ptr = a.pool.lens + int64_t(slot) * a.pool.layers + a.layer;
  const bool do_append = a.k_new != nullptr;

  const int64_t len_old = *reinterpret_cast<const volatile int32_t*>(len_ptr);
  const int64_t len = len_old + (do_append ? 1 : 0);
  int64_t ws = a.sliding_window > 0 ? (len > a.sliding_window ? len - a.sliding_window : 0) : a.window_start;
  if (ws >= len) ws = len > 0 ? len - 1 : 0;
  const int64_t p_first = ws / PAGE_TOKENS;
  const int64_t p_last = (len - 1) / PAGE_TOKENS;
  const int64_t n_pages = p_last - p_first + 1;
  const int64_t pb = p_first + (n_pages * split) / a.splits;
  const int64_t pe = p_first + (n_pages * (split + 1)) / a.splits;
  const int my_pages = static_cast<int>(pe - pb);
  const int32_t* table = a.pool.tables + int64_t(slot) * a.pool.table_stride;
  const int64_t head_off = int64_t(a.layer) * a.pool.layer_bytes + int64_t(kvh) * 2 * a.pool.tile_bytes;
  const int64_t append_page_index = len_old / PAGE_TOKENS;
  const bool owns_append = do_append && append_page_index >= pb && append_page_index < pe;
  const float* kn = do_append ? a.k_new + int64_t(seq) * a.pool.kv_heads * HD + kvh * HD : nullptr;
  const float* vn = do_append ? a.v_new + int64_t(seq) * a.pool.kv_heads * HD + kvh * HD : nullptr;

  int32_t first_entry = -1;
  float smax = __uint_as_float(*reinterpret_cast<const volatile uint32_t*>(a.pool.scale_max));
  if (warp == MMA_CONSUMERS) {
    if (lane == 0) {
      flags[0] = 0;
      flags[1] = 0;
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
    float4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int f = (tid + k * MMA_CONSUMERS * 32) * 4;
      v[k] = (f / HD < gqa) ? __ldg(reinterpret_cast<const float4*>(q + f)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
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
    // The row a fused append is about to write may carry a larger scale than any stored one.
    if (owns_append) smax = fmaxf(smax, new_row_max_scale<HD>(kn, vn, lane));
  }
  __syncthreads();
  if (warp < MMA_CONSUMERS) {
    // qsum[h][g] = sum over the group of the fp16 value of q (hi + lo), as the tensor core sees it
    if (tid < 8 * G) {
      const int h = tid / G, grp = tid % G;
      const __half* ph = reinterpret_cast<const __half*>(q_hi + h * S::QROW) + grp * QGROUP;
      const __half* pl = reinterpret_cast<const __half*>(q_lo + h * S::QROW) + grp * QGROUP;
      float sum = 0.0f;
      for (int d = 0; d < QGROUP; ++d) sum += __half2float(ph[d]) + __half2float(pl[d]);
      qsum_s[h * G + grp] = sum;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(MMA_CONSUMERS * 32) : "memory");
  }

  if (warp == MMA_CONSUMERS) {
    // ---------------- producer warp ----------------
    for (int base = 0; base < my_pages; base += 32) {
      int idx = base + lane;
      int32_t entry = base == 0 ? first_entry : (idx < my_pages ? table[pb + idx] : -1);
      int cnt = min(32, my_pages - base);
      for (int j = 0; j < cnt; ++j) {
        int i = base + j;
        int32_t page = __shfl_sync(0xffffffffu, entry, j);
        int stage = i % nst;
        uint32_t parity = ((i / nst) & 1) ^ 1;
        if (lane == 0) {
          bool ok = mbar_wait(smem_u32(bars + MMA_MAX_STAGES + stage), parity, abort_flag, a.status);
          if (ok && (page < 0 || page >= a.num_pages)) {
            atomicExch(a.status, DEV_ERR_BAD_PAGE);
            *abort_flag = 1;
            ok = false;
          }
          if (ok) {
            uint32_t full = smem_u32(bars + stage);
            mbar_expect_tx(full, S::STAGE);
            bulk_copy_g2s(smem_u32(ring + size_t(stage) * S::STAGE),
                          a.pool.base + int64_t(page) * a.pool.page_bytes + head_off, S::STAGE, full);
          }
        }
      }
    }
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
    float corr[G][2];  // sum_row bias_v * p for heads 2t, 2t+1: this thread's rows only
#pragma unroll
    for (int grp = 0; grp < G; ++grp) corr[grp][0] = corr[grp][1] = 0.0f;
    float m0 = -1.0e30f, m1 = -1.0e30f, l0 = 0.0f, l1 = 0.0f;
    const uint8_t* qh_row = q_hi + g * S::QROW + 8 * t;   // + 32*ks: the four fp16 of dims 16ks+4t..+3
    const uint8_t* ql_row = q_lo + g * S::QROW + 8 * t;

    for (int i = warp; i < my_pages; i += MMA_CONSUMERS) {
      const int stage = i % nst;
      const uint32_t parity = (i / nst) & 1;
      const bool ok = mbar_wait(smem_u32(bars + stage), parity, abort_flag, a.status);
      uint8_t* ktile = ring + size_t(stage) * S::STAGE;
      uint8_t* vtile = ktile + S::TILE;
      const int64_t page_index = pb + i;
      const int64_t row_base = page_index * PAGE_TOKENS;

      if (ok && owns_append && page_index == append_page_index) {
        // Quantise the new row; store codes and metadata to its page and to the staged copy.
        const int rin = static_cast<int>(len_old % PAGE_TOKENS);
        int32_t page = table[page_index];
        if (page >= 0 && page < a.num_pages) {
          uint8_t* gk = a.pool.base + int64_t(page) * a.pool.page_bytes + head_off;
          uint8_t* gv = gk + S::TILE;
#pragma unroll
          for (int grp = 0; grp < G; ++grp) {
            const int dim = grp * QGROUP + lane;
            uint32_t mk, mv;
            const uint32_t ck = quantize_lane(kn[dim], &mk);
            const uint32_t cv = quantize_lane(vn[dim], &mv);
            const int ik = u8_k_code_index(rin, dim, HD), iv = u8_v_code_index(rin, dim);
            gk[ik] = static_cast<uint8_t>(ck);
            ktile[ik] = static_cast<uint8_t>(ck);
            gv[iv] = static_cast<uint8_t>(cv);
            vtile[iv] = static_cast<uint8_t>(cv);
            if (lane == 0) {
              const int mo = u8_meta_offset(rin, grp, HD);
              *reinterpret_cast<uint32_t*>(gk + mo) = mk;
              *reinterpret_cast<uint32_t*>(ktile + mo) = mk;
              *reinterpret_cast<uint32_t*>(gv + mo) = mv;
              *reinterpret_cast<uint32_t*>(vtile + mo) = mv;
              atomicMax(a.pool.scale_max, max((mk & 0xffffu) << 16, (mv & 0xffffu) << 16));
            }
          }
        }
        __syncwarp();
      }

      if (ok) {
        // ---- scores: one accumulator per group of 32 dims, scale applied in f32. The
        //      tensor-core instructions have a long latency and issue in order, so products
        //      that do not depend on each other are issued back to back: all groups for one
        //      half of their dims and the hi part of Q, then the lo part, then the other half. ----
        float s[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
        const uint8_t* kmeta = ktile + S::CODES;
        float acc[G][4];
#pragma unroll
        for (int grp = 0; grp < G; ++grp) acc[grp][0] = acc[grp][1] = acc[grp][2] = acc[grp][3] = 0.0f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t af[G][4];
#pragma unroll
          for (int grp = 0; grp < G; ++grp) {
            const int ks = 2 * grp + half;                 // 16-byte chunk index = k-step
            const int phys = (ks & ~7) | ((ks ^ g) & 7);   // rows g and g+8 share the swizzle
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(ktile + g * HD + phys * 16 + 4 * t);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(ktile + (g + 8) * HD + phys * 16 + 4 * t);
            af[grp][0] = codes_lo(w0);
            af[grp][1] = codes_lo(w1);
            af[grp][2] = codes_hi(w0);
            af[grp][3] = codes_hi(w1);
          }
#pragma unroll
          for (int grp = 0; grp < G; ++grp) {
            const uint2 qh = *reinterpret_cast<const uint2*>(qh_row + 32 * (2 * grp + half));
            mma_f16(acc[grp], af[grp][0], af[grp][1], af[grp][2], af[grp][3], qh.x, qh.y);
          }
#pragma unroll
          for (int grp = 0; grp < G; ++grp) {
            const uint2 ql = *reinterpret_cast<const uint2*>(ql_row + 32 * (2 * grp + half));
            mma_f16(acc[grp], af[grp][0], af[grp][1], af[grp][2], af[grp][3], ql.x, ql.y);
          }
        }
#pragma unroll
        for (int grp = 0; grp < G; ++grp) {
          const uint32_t mk0 = *reinterpret_cast<const uint32_t*>(kmeta + (g * G + grp) * 4);
          const uint32_t mk1 = *reinterpret_cast<const uint32_t*>(kmeta + ((g + 8) * G + grp) * 4);
          const float sc0 = __uint_as_float(mk0 << 16), bi0 = __uint_as_float(mk0 & 0xffff0000u);
          const float sc1 = __uint_as_float(mk1 << 16), bi1 = __uint_as_float(mk1 & 0xffff0000u);
          const float qs0 = qsum_s[(2 * t) * G + grp], qs1 = qsum_s[(2 * t + 1) * G + grp];
          s[0] = fmaf(sc0, acc[grp][0], s[0]), sb[0] = fmaf(bi0, qs0, sb[0]);
          s[1] = fmaf(sc0, acc[grp][1], s[1]), sb[1] = fmaf(bi0, qs1, sb[1]);
          s[2] = fmaf(sc1, acc[grp][2], s[2]), sb[2] = fmaf(bi1, qs0, sb[2]);
          s[3] = fmaf(sc1, acc[grp][3], s[3]), sb[3] = fmaf(bi1, qs1, sb[3]);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) s[r] = fmaf(s[r], CODE_UNIT_INV, sb[r]);  // the codes were in units of 2^-24
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
#pragma unroll
          for (int grp = 0; grp < G; ++grp) {
            corr[grp][0] *= al0;
            corr[grp][1] *= al1;
          }
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
        // ---- outputs: per group, fold scale_v into the weights; bias_v term in f32 ----
        const uint8_t* vmeta = vtile + S::CODES;
        uint32_t pb0[G], pb1[G];
#pragma unroll
        for (int grp = 0; grp < G; ++grp) {
          const uint32_t mv0 = *reinterpret_cast<const uint32_t*>(vmeta + (g * G + grp) * 4);
          const uint32_t mv1 = *reinterpret_cast<const uint32_t*>(vmeta + ((g + 8) * G + grp) * 4);
          const float sc0 = __uint_as_float(mv0 << 16) * pscale, bi0 = __uint_as_float(mv0 & 0xffff0000u);
          const float sc1 = __uint_as_float(mv1 << 16) * pscale, bi1 = __uint_as_float(mv1 & 0xffff0000u);
          corr[grp][0] += bi0 * p[0] + bi1 * p[2];
          corr[grp][1] += bi0 * p[1] + bi1 * p[3];
          pb0[grp] = movmatrix_trans(pack_f16(p[0] * sc0, p[1] * sc0));   // rows 0-7
          pb1[grp] = movmatrix_trans(pack_f16(p[2] * sc1, p[3] * sc1));   // rows 8-15
        }
#pragma unroll
        for (int j = 0; j < KSTEPS; ++j) {
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(vtile + (16 * j + g) * PAGE_TOKENS + 4 * t);
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(vtile + (16 * j + g + 8) * PAGE_TOKENS + 4 * t);
          mma_f16(o_acc[j], codes_lo(w0), codes_lo(w1), codes_hi(w0), codes_hi(w1), pb0[j / 2], pb1[j / 2]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bars + MMA_MAX_STAGES + stage));
    }

    // ---- hand this warp's state to the merge buffer (it aliases the ring) ----
    asm volatile("bar.sync 1, %0;" ::"r"(MMA_CONSUMERS * 32) : "memory");
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, off);
      l1 += __shfl_xor_sync(0xffffffffu, l1, off);
#pragma unroll
      for (int grp = 0; grp < G; ++grp) {
        corr[grp][0] += __shfl_xor_sync(0xffffffffu, corr[grp][0], off);
        corr[grp][1] += __shfl_xor_sync(0xffffffffu, corr[grp][1], off);
      }
    }
    float* ow = o_s + warp * 8 * S::OPAD;
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j) {
      const float c0 = corr[j / 2][0], c1 = corr[j / 2][1];
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
  finish_block<HD>(a, o_s, ml_s, S::OPAD, flags, seq, kvh, split, gqa, do_append, len_ptr, len, tid);
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

cudaError_t attention_u8_configure() {
  cudaError_t e = cudaFuncSetAttribute(attention_u8_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       227 * 1024);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(attention_u8_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

cudaError_t launch_attention_u8(const AttnArgs& a, int n_seq, cudaStream_t stream) {
  dim3 grid(a.splits, a.pool.kv_heads, n_seq);
  if (a.pool.head_dim == 128) {
    attention_u8_kernel<128><<<grid, MMA_THREADS, U8Smem<128>::total(a.n_stages), stream>>>(a);
  } else {
    attention_u8_kernel<256><<<grid, MMA_THREADS, U8Smem<256>::total(a.n_stages), stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace sgk
