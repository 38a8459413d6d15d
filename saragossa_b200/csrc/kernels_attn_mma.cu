// Paged split-K flash-decoding for bf16 pages (head_dim 128 / 256, GQA group <= 8),
// with the per-token append fused in.
//
// One block per (split, kv head, sequence). A producer warp walks the block table
// and brings each page's K tile + V tile (one contiguous range of the pool, see
// layout.h) into a shared-memory ring with one bulk async copy (TMA,
// cp.async.bulk) per page, completion signalled on an mbarrier. Consumer warps
// take pages round-robin; per page:
//     S^T[16 rows x 8 heads] = K_tile . Q^T          (mma.sync m16n8k16, bf16)
//     online softmax over the rows (warp shuffles, log2 domain)
//     O^T[dims x 8 heads]   += V_tile^T . P^T        (ldmatrix.trans + mma)
// so the K/V bytes of a kv head are read from HBM once for its whole GQA group.
// Q and P are split into bf16 hi + lo parts, which keeps the products at ~f32
// accuracy while the tensor cores stay far from being the limit (the kernel is
// HBM-bound: ~8 flop/byte). Warps merge in shared memory, the block writes an
// un-normalised partial, and the block that arrives last for (sequence, kv head)
// merges the splits and writes the output: one launch, no second pass.
//
// The pages are stored XOR-swizzled (layout.h), so the verbatim copy in shared
// memory is read by ldmatrix without bank conflicts.
//
// Fused append (k_new != NULL): the block whose range ends at the row being
// written converts that row to bf16 (same integer rounding as the append kernel),
// stores it into its page and patches it into the shared-memory copy of the page,
// and the block that arrives last for the sequence moves the device cursor.
//
// Counterparts in the reference: attention_decode_2pass_1/_2 and
// attention_decode_flash (src/decode_resident/kernels.rs:166-917) plus copy_at
// (kernels.rs:1026-1044); selection logic src/decode_resident/attention.rs:755-769.
#include "mma_common.cuh"

namespace sgk {

// x -> bf16 hi (nearest) and bf16 lo = nearest(x - hi), packed for two values.
__device__ __forceinline__ void split_hi_lo(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
  __nv_bfloat16 l0 = __float2bfloat16_rn(x0 - __bfloat162float(h0));
  __nv_bfloat16 l1 = __float2bfloat16_rn(x1 - __bfloat162float(h1));
  hi = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h1)) << 16);
  lo = static_cast<uint32_t>(__bfloat16_as_ushort(l0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(l1)) << 16);
}

template <int HD>
struct MmaSmem {
  static constexpr int TILE = PAGE_TOKENS * HD * 2;  // bytes of a K or V tile
  static constexpr int STAGE = 2 * TILE;             // K tile + V tile
  static constexpr int OPAD = HD + 4;                // padded row of the merge buffer
  static constexpr int Q_BYTES = 2 * 8 * HD * 2;     // hi and lo, 8 heads
  static constexpr int O_BYTES = MMA_CONSUMERS * 8 * OPAD * 4;  // aliases the ring once it has drained
  static constexpr int ML_BYTES = 512;  // per-warp {max, sum}, then the merge weights and the block's {max, sum}
  static constexpr int BAR_BYTES = 2 * MMA_MAX_STAGES * 8;
  static constexpr int NEW_BYTES = 2 * HD * 2;       // the K and V row of a fused append, bf16
  static constexpr int RECV_BYTES = ClusterRecv<HD>::BYTES;  // what the other blocks of a cluster send for the merge
  static constexpr int FIXED = Q_BYTES + ML_BYTES + BAR_BYTES + 64 + NEW_BYTES + RECV_BYTES;
  __host__ __device__ static size_t ring_bytes(int stages) {
    size_t r = size_t(stages) * STAGE;
    return r > size_t(O_BYTES) ? r : size_t(O_BYTES);
  }
  static size_t total(int stages) { return ring_bytes(stages) + FIXED + 1024; }
};

template <int HD, bool CLUSTER, bool PEERS>
__global__ void __launch_bounds__(MMA_THREADS, 2) attention_mma_kernel(AttnArgs a) {
  using S = MmaSmem<HD>;
  constexpr int KSTEPS = HD / 16;
  constexpr int ROWB = HD * 2;  // bytes of a tile row
  extern __shared__ uint8_t smem_raw[];
  // stage ring first, 1024-byte aligned so the swizzle pattern lines up with the banks
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int nst = a.n_stages;
  uint8_t* fixed = ring + S::ring_bytes(nst);
  uint16_t* q_hi = reinterpret_cast<uint16_t*>(fixed);          // [8][HD]
  uint16_t* q_lo = q_hi + 8 * HD;                               // [8][HD]
  float* o_s = reinterpret_cast<float*>(ring);                  // [warps][8][OPAD], used after the ring drained
  float* ml_s = reinterpret_cast<float*>(fixed + S::Q_BYTES);   // [warps][8][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed + S::Q_BYTES + S::ML_BYTES);
  int* flags = reinterpret_cast<int*>(bars + 2 * MMA_MAX_STAGES);  // [0]=abort [1]=last arriver
  uint32_t* new_s = reinterpret_cast<uint32_t*>(flags + 16);       // bf16 pairs of the appended [K row | V row]
  float* recv_s = reinterpret_cast<float*>(fixed + S::FIXED - S::RECV_BYTES);
  volatile int* abort_flag = flags;

  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gqa = a.q_heads / a.pool.kv_heads;
  const int slot = a.slots ? a.slots[seq] : a.slot0;
  int32_t* len_ptr = a.pool.lens + int64_t(slot) * a.pool.layers + a.layer;
  const bool do_append = a.k_new != nullptr;
  if (a.pdl_trigger) pdl_launch_dependents();
#ifdef SGK_TRACE
  if (a.trace && tid == 0) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    a.trace[((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 15] = gt;
  }
  if (tid == 0) SGK_TP(0);
#endif

  // Every thread reads the cursor itself (one broadcast L2 hit), so nothing below waits
  // on a shared-memory hand-off. With a fused append the cursor is rewritten only by the
  // block that arrives last for the sequence, i.e. after every block has read it.
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
  const int64_t pb = p_first + (n_pages * split) / splits;        // this block's pages [pb, pe)
  const int64_t pe = p_first + (n_pages * (split + 1)) / splits;
  const int my_pages = static_cast<int>(pe - pb);
  const int32_t* table = a.pool.tables + int64_t(slot) * a.pool.table_stride;
  const int64_t head_off = int64_t(a.layer) * a.pool.layer_bytes + int64_t(kvh) * 2 * a.pool.tile_bytes;
  // Page that receives the appended row, and whether this block owns it.
  const int64_t append_page_index = len_old / PAGE_TOKENS;
  const bool owns_append = do_append && append_page_index >= pb && append_page_index < pe;

  int32_t first_entry = -1;
  if (warp == MMA_CONSUMERS) {
    // producer warp: barriers, and the first block-table entries, while the others stage Q
    if (lane == 0) {
      flags[0] = 0;
      flags[1] = 0;
      for (int s = 0; s < nst; ++s) {
        mbar_init(smem_u32(bars + s), 1);                   // full: producer's expect_tx arrival
        mbar_init(smem_u32(bars + MMA_MAX_STAGES + s), 1);  // empty: one consumer lane
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (lane < my_pages) first_entry = table[pb + lane];
  } else {
    // Q of the group: scale, split into bf16 hi/lo; rows of absent heads are zero.
    // All loads are issued before the first conversion.
    constexpr int NV = HD / 64;  // float4 per consumer thread
    const float* q = a.q + (int64_t(seq) * a.q_heads + int64_t(kvh) * gqa) * HD;
    // q and the row to append come from the launch before this one; the cursor, the block table and
    // the pages the producer has started to copy do not
    if (a.pdl_wait) pdl_wait();
    if (tid == 0) SGK_TP(8);
    float4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int f = (tid + k * MMA_CONSUMERS * 32) * 4;
      v[k] = (f / HD < gqa) ? __ldg(reinterpret_cast<const float4*>(q + f)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // The row of a fused append is converted here, with the same round trip as Q, and waits in
    // shared memory for its page: read where it is stored, it would pay that latency at the very
    // end of the block that every other block of the sequence waits for.
    const bool loads_row = owns_append && tid * 4 < 2 * HD;
    const bool is_k = tid * 4 < HD;
    const int dim = is_k ? tid * 4 : tid * 4 - HD;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    int32_t page = -1;
    if (loads_row) {
      const int64_t row_off = int64_t(seq) * a.pool.kv_heads * HD + kvh * HD;
      const float* src = is_k ? a.k_new + row_off + dim : a.v_new + row_off + dim;
      page = table[append_page_index];   // issued with the row's load: one round trip for both
      x = __ldg(reinterpret_cast<const float4*>(src));
    }
    if (loads_row) {
      const uint2 packed = make_uint2(uint32_t(f32_to_bf16_bits(x.x)) | (uint32_t(f32_to_bf16_bits(x.y)) << 16),
                                      uint32_t(f32_to_bf16_bits(x.z)) | (uint32_t(f32_to_bf16_bits(x.w)) << 16));
      *reinterpret_cast<uint2*>(new_s + tid * 2) = packed;
      // The row goes to its page in global memory now: whatever the bulk copy of that page sees of
      // it, the staged copy gets the row again from shared memory; and a store issued here has long
      // been performed when the block's tail asks for its writes to be visible. A page id outside the
      // pool is reported by the producer, which meets the same table entry.
      if (page >= 0 && page < a.num_pages) {
        const int rin = static_cast<int>(len_old % PAGE_TOKENS);
        uint8_t* tile = a.pool.base + int64_t(page) * a.pool.page_bytes + head_off + (is_k ? 0 : S::TILE);
        *reinterpret_cast<uint2*>(tile + bf16_elem_index(rin, dim, HD) * 2) = packed;
      }
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int f = (tid + k * MMA_CONSUMERS * 32) * 4;
      uint32_t hi0, lo0, hi1, lo1;
      split_hi_lo(v[k].x * a.scale_log2e, v[k].y * a.scale_log2e, hi0, lo0);
      split_hi_lo(v[k].z * a.scale_log2e, v[k].w * a.scale_log2e, hi1, lo1);
      *reinterpret_cast<uint2*>(q_hi + f) = make_uint2(hi0, hi1);
      *reinterpret_cast<uint2*>(q_lo + f) = make_uint2(lo0, lo1);
    }
  }
  // The producer only announces that the barriers exist and starts copying; the consumers wait
  // here for that and for each other's part of Q. The first pages are then on their way while
  // Q is still being converted.
  if (warp == MMA_CONSUMERS) {
    __syncwarp();
    asm volatile("bar.arrive 3, %0;" ::"r"(MMA_THREADS) : "memory");
  } else {
    asm volatile("bar.sync 3, %0;" ::"r"(MMA_THREADS) : "memory");
  }
  if (tid == 0) SGK_TP(1);

  if (warp == MMA_CONSUMERS) {
    // ---------------- producer warp ----------------
    produce_pages<S::STAGE>(a, table, pb, my_pages, first_entry, ring, bars, nst, head_off, abort_flag, lane);
    if (a.pdl_wait) pdl_wait();   // the tail writes to memory the earlier launch may still be using
    SGK_TP(12);
  } else {
    // ---------------- consumer warps ----------------
    const int g = lane >> 2, t = lane & 3;
    // B fragments of Q^T: b0 = Q[head g][k0+2t, +1], b1 = Q[head g][k0+2t+8, +9]
    uint32_t qh_f[KSTEPS][2], ql_f[KSTEPS][2];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      qh_f[ks][0] = *reinterpret_cast<const uint32_t*>(q_hi + g * HD + ks * 16 + 2 * t);
      qh_f[ks][1] = *reinterpret_cast<const uint32_t*>(q_hi + g * HD + ks * 16 + 2 * t + 8);
      ql_f[ks][0] = *reinterpret_cast<const uint32_t*>(q_lo + g * HD + ks * 16 + 2 * t);
      ql_f[ks][1] = *reinterpret_cast<const uint32_t*>(q_lo + g * HD + ks * 16 + 2 * t + 8);
    }
    float o_acc[KSTEPS][4];
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j) o_acc[j][0] = o_acc[j][1] = o_acc[j][2] = o_acc[j][3] = 0.0f;
    float m0 = -1.0e30f, m1 = -1.0e30f, l0 = 0.0f, l1 = 0.0f;  // heads 2t and 2t+1

    // ldmatrix lane roles
    const int lm = lane >> 3, lr = lane & 7;
    const int k_row = lr + (lm & 1) * 8, k_csel = lm >> 1;   // K: matrices (r0-7,c0) (r8-15,c0) (r0-7,c1) (r8-15,c1)
    const int v_row = lr + (lm >> 1) * 8, v_csel = lm & 1;   // V^T: (r0-7,c0) (r0-7,c1) (r8-15,c0) (r8-15,c1)

    int stage = warp, next_stage = warp;   // the stage count is a multiple of the consumer count
    uint32_t parity = 0, next_parity = 0;
    for (int i = warp; i < my_pages; i += MMA_CONSUMERS) {
      stage = next_stage;
      parity = next_parity;
      next_stage = stage + MMA_CONSUMERS;
      if (next_stage >= nst) {
        next_stage -= nst;
        next_parity ^= 1;
      }
      const bool ok = mbar_wait(smem_u32(bars + stage), parity, abort_flag, a.status);
      if (i == 0) SGK_TP(2);
      uint8_t* ktile = ring + size_t(stage) * S::STAGE;
      uint8_t* vtile = ktile + S::TILE;
      const int64_t page_index = pb + i;
      const int64_t row_base = page_index * PAGE_TOKENS;

      if (ok && owns_append && page_index == append_page_index) {
        // The new row (converted in the prologue, already on its way to the page) joins the staged copy.
        const int rin = static_cast<int>(len_old % PAGE_TOKENS);
        for (int chunk = lane; chunk < HD / 8; chunk += 32) {
          const int off = bf16_elem_index(rin, chunk * 8, HD) * 2;
          *reinterpret_cast<uint4*>(ktile + off) = *reinterpret_cast<const uint4*>(new_s + chunk * 4);
          *reinterpret_cast<uint4*>(vtile + off) = *reinterpret_cast<const uint4*>(new_s + HD / 2 + chunk * 4);
        }
        __syncwarp();
      }

      if (ok) {
        // The tensor-core instructions have a long latency, so the page is processed as
        // few, wide dependency levels: all K fragments are loaded, then the QK products go
        // to eight independent accumulators (four for the hi part of Q, four for the lo part);
        // the V fragments are loaded before the softmax so the stage can be handed back to the
        // producer early; the PV products issue all hi parts, then all lo parts.
        constexpr int CH = 8;                 // k-steps (QK) / dim tiles (PV) per chunk
        constexpr int NCH = KSTEPS / CH;      // 1 for head_dim 128, 2 for 256
        float acc[8][4];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.0f;
        const uint32_t kbase = smem_u32(ktile) + k_row * ROWB;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint32_t ka[CH][4];
#pragma unroll
          for (int u = 0; u < CH; ++u) {
            int chunk = 2 * (c * CH + u) + k_csel;
            int phys = (chunk & ~7) | ((chunk ^ k_row) & 7);
            ldmatrix_x4(kbase + phys * 16, ka[u][0], ka[u][1], ka[u][2], ka[u][3]);
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int ks = c * CH + half * 4 + u;
              mma_bf16(acc[u], ka[half * 4 + u][0], ka[half * 4 + u][1], ka[half * 4 + u][2], ka[half * 4 + u][3],
                       qh_f[ks][0], qh_f[ks][1]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int ks = c * CH + half * 4 + u;
              mma_bf16(acc[4 + u], ka[half * 4 + u][0], ka[half * 4 + u][1], ka[half * 4 + u][2],
                       ka[half * 4 + u][3], ql_f[ks][0], ql_f[ks][1]);
            }
          }
        }
        // V fragments of the first chunk (all of V for head_dim 128)
        const uint32_t vbase = smem_u32(vtile) + v_row * ROWB;
        uint32_t va[CH][4];
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          int chunk = 2 * u + v_csel;
          int phys = (chunk & ~7) | ((chunk ^ v_row) & 7);
          ldmatrix_x4_trans(vbase + phys * 16, va[u][0], va[u][1], va[u][2], va[u][3]);
        }
        if (NCH == 1) {
          // every byte of the stage is in registers: give it back before the math
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(bars + MMA_MAX_STAGES + stage));
        }
        float s[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          s[e] = ((acc[0][e] + acc[1][e]) + (acc[2][e] + acc[3][e])) + ((acc[4][e] + acc[5][e]) + (acc[6][e] + acc[7][e]));
        // rows g (s0,s1) and g+8 (s2,s3); heads 2t (s0,s2) and 2t+1 (s1,s3)
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
        // P^T as the B operand: transpose the two 8x8 halves across the warp.
        uint32_t ph_a, pl_a, ph_b, pl_b;
        split_hi_lo(p[0], p[1], ph_a, pl_a);  // rows 0-7
        split_hi_lo(p[2], p[3], ph_b, pl_b);  // rows 8-15
        const uint32_t bh0 = movmatrix_trans(ph_a), bh1 = movmatrix_trans(ph_b);
        const uint32_t bl0 = movmatrix_trans(pl_a), bl1 = movmatrix_trans(pl_b);
        // ---- O^T += V^T . P^T ----
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (c > 0) {
#pragma unroll
            for (int u = 0; u < CH; ++u) {
              int chunk = 2 * (c * CH + u) + v_csel;
              int phys = (chunk & ~7) | ((chunk ^ v_row) & 7);
              ldmatrix_x4_trans(vbase + phys * 16, va[u][0], va[u][1], va[u][2], va[u][3]);
            }
            if (c == NCH - 1) {
              __syncwarp();
              if (lane == 0) mbar_arrive(smem_u32(bars + MMA_MAX_STAGES + stage));
            }
          }
#pragma unroll
          for (int u = 0; u < CH; ++u) mma_bf16(o_acc[c * CH + u], va[u][0], va[u][1], va[u][2], va[u][3], bh0, bh1);
#pragma unroll
          for (int u = 0; u < CH; ++u) mma_bf16(o_acc[c * CH + u], va[u][0], va[u][1], va[u][2], va[u][3], bl0, bl1);
        }
      } else {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(bars + MMA_MAX_STAGES + stage));
      }
    }

    if (warp == 0) SGK_TP(3);
    // ---- hand this warp's state to the merge buffer (it aliases the ring: wait
    //      until every warp has consumed its last stage) ----
    asm volatile("bar.sync 1, %0;" ::"r"(MMA_CONSUMERS * 32) : "memory");
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, off);
      l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    float* ow = o_s + warp * 8 * S::OPAD;
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j) {
      ow[(2 * t) * S::OPAD + 16 * j + g] = o_acc[j][0];
      ow[(2 * t + 1) * S::OPAD + 16 * j + g] = o_acc[j][1];
      ow[(2 * t) * S::OPAD + 16 * j + g + 8] = o_acc[j][2];
      ow[(2 * t + 1) * S::OPAD + 16 * j + g + 8] = o_acc[j][3];
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

// Exercises the bounded wait on purpose: one warp waits on an mbarrier that nobody completes.
// The wait gives up after its spin limit, sets the device status word and the kernel returns;
// the context stays usable. Used by the failure-detection test.
__global__ void wait_timeout_selftest_kernel(int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 1;  // start with the short spin limit
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, &abort_flag, status);
}

cudaError_t launch_wait_timeout_selftest(int32_t* status, cudaStream_t stream) {
  wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(status);
  return cudaGetLastError();
}

bool attention_mma_supported(int dtype, int head_dim, int gqa) {
  return dtype == KV_BF16 && (head_dim == 128 || head_dim == 256) && gqa >= 1 && gqa <= 8;
}

int attention_mma_max_stages(int head_dim) {
  // Two blocks per SM: each gets half of the 227 KiB an SM offers.
  size_t budget = 113 * 1024;
  size_t fixed = head_dim == 128 ? MmaSmem<128>::FIXED : MmaSmem<256>::FIXED;
  size_t stage = head_dim == 128 ? MmaSmem<128>::STAGE : MmaSmem<256>::STAGE;
  int n = static_cast<int>((budget - fixed - 1024) / stage);
  if (n > MMA_MAX_STAGES) n = MMA_MAX_STAGES;
  // A stage must always be consumed by the same warp (stage = i % n, warp = i % MMA_CONSUMERS):
  // otherwise a warp could wait on a phase of a barrier two ahead of the current one.
  return n / MMA_CONSUMERS * MMA_CONSUMERS;
}

int attention_mma_resident_blocks(int head_dim, int n_stages) {
  int blocks = 0;
  cudaError_t e = head_dim == 128
                      ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_mma_kernel<128, false, false>, MMA_THREADS,
                                                                      MmaSmem<128>::total(n_stages))
                      : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_mma_kernel<256, false, false>, MMA_THREADS,
                                                                      MmaSmem<256>::total(n_stages));
  return e == cudaSuccess ? blocks : 0;
}

// How many clusters of `splits` blocks the device can hold at once (0: such a launch would fail).
int attention_mma_max_clusters(int head_dim, int n_stages, int splits) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(splits, 1, 1);
  cfg.blockDim = dim3(MMA_THREADS);
  cfg.dynamicSmemBytes = head_dim == 128 ? MmaSmem<128>::total(n_stages) : MmaSmem<256>::total(n_stages);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e = head_dim == 128 ? cudaOccupancyMaxActiveClusters(&n, attention_mma_kernel<128, true, false>, &cfg)
                                  : cudaOccupancyMaxActiveClusters(&n, attention_mma_kernel<256, true, false>, &cfg);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

cudaError_t attention_mma_configure() {
  const void* kernels[6] = {reinterpret_cast<const void*>(attention_mma_kernel<128, false, false>), reinterpret_cast<const void*>(attention_mma_kernel<256, false, false>),
                            reinterpret_cast<const void*>(attention_mma_kernel<128, true, false>), reinterpret_cast<const void*>(attention_mma_kernel<256, true, false>),
                            reinterpret_cast<const void*>(attention_mma_kernel<128, false, true>), reinterpret_cast<const void*>(attention_mma_kernel<256, false, true>)};
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

cudaError_t launch_attention_mma(const AttnArgs& a, int n_seq, cudaStream_t stream) {
  dim3 grid(a.splits, a.pool.kv_heads, n_seq);
  if (a.pool.head_dim == 128) {
    if (a.n_peers > 0) return launch_one(attention_mma_kernel<128, false, true>, grid, MmaSmem<128>::total(a.n_stages), a, stream);
    return a.cluster_merge ? launch_one(attention_mma_kernel<128, true, false>, grid, MmaSmem<128>::total(a.n_stages), a, stream)
                           : launch_one(attention_mma_kernel<128, false, false>, grid, MmaSmem<128>::total(a.n_stages), a, stream);
  } else {
    if (a.n_peers > 0) return launch_one(attention_mma_kernel<256, false, true>, grid, MmaSmem<256>::total(a.n_stages), a, stream);
    return a.cluster_merge ? launch_one(attention_mma_kernel<256, true, false>, grid, MmaSmem<256>::total(a.n_stages), a, stream)
                           : launch_one(attention_mma_kernel<256, false, false>, grid, MmaSmem<256>::total(a.n_stages), a, stream);
  }
  return cudaGetLastError();
}

}  // namespace sgk
