// Pieces shared by the paged tensor-core attention kernels (bf16 and u8 pages): the
// mbarrier / bulk-copy (TMA) primitives with bounded waits, the warp-level matrix
// instructions, and the block-cooperative merge of split-K partials.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"

namespace sgk {

constexpr int MMA_CONSUMERS = 4;                       // consumer warps
constexpr int MMA_THREADS = (MMA_CONSUMERS + 1) * 32;  // + one producer warp
constexpr int MMA_MAX_STAGES = 32;
constexpr int MERGE_MAX = 12;  // partials merged at once (bound of group size and of group count)
constexpr uint32_t WAIT_SPINS = 1u << 22;        // bound of every mbarrier wait
constexpr uint32_t WAIT_SPINS_ABORTED = 1u << 10;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking probe (try_wait may park the thread for a while when the phase is not complete).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. On expiry: sets the block's abort flag and the device status
// word and returns false; the caller skips the work of that stage but keeps
// walking its stages, so copies still in flight are waited for (with the short
// bound) before the block exits.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* status) {
  uint32_t limit = *abort_flag ? WAIT_SPINS_ABORTED : WAIT_SPINS;
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  *abort_flag = 1;
  atomicExch(status, DEV_ERR_WAIT_TIMEOUT);
  return false;
}
// Pages are read once per launch: their copies carry the L2 evict-first policy, so that they do
// not push the small data every block needs at once (cursors, block tables, q, split partials)
// out of L2. Measured on the u8 kernel at batch 8: 64.4 -> 60.5 us per layer.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
#ifdef SGK_TRACE
__device__ __forceinline__ unsigned long long sgk_trace_now(int gt) {
  unsigned long long t;
  if (gt) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  else t = clock64();
  return t;
}
#define SGK_TP(slot)                                                                               \
  do {                                                                                             \
    if (a.trace && (threadIdx.x & 31) == 0)                                                        \
      a.trace[((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (slot)] = sgk_trace_now(a.trace_gt); \
  } while (0)
#else
#define SGK_TP(slot) do {} while (0)
#endif

// Programmatic dependent launch: a launch that carries the stream-serialisation attribute may start
// while the launch before it is still running, once every block of that launch has executed
// launch_dependents (or exited); what the earlier launch wrote is visible after wait. Both are
// no-ops in a launch without such a neighbour.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The producer warp's walk over the block's pages [pb, pb + my_pages): one bulk copy of
// STAGE_BYTES per page into stage (page index % nst), completion on the stage's "full" barrier
// (bars[stage]); a stage is refilled once its "empty" barrier (bars[MMA_MAX_STAGES + stage]) has
// completed. The first min(my_pages, nst) copies find fresh stages and wait for nothing: lane j
// starts page j, so one pass of the warp puts them all in flight (issued one after the other by
// one lane, each costs that lane a round trip to its barrier first). first_entry: lane l holds
// table[pb + l] for l < my_pages.
template <int STAGE_BYTES>
__device__ __forceinline__ void produce_pages(const AttnArgs& a, const int32_t* table, int64_t pb, int my_pages,
                                              int32_t first_entry, uint8_t* ring, uint64_t* bars, int nst,
                                              int64_t head_off, volatile int* abort_flag, int lane) {
  const uint64_t policy = l2_policy_evict_first();
  const int first = my_pages < nst ? my_pages : nst;
  if (lane < first) {
    if (first_entry < 0 || first_entry >= a.num_pages) {
      atomicExch(a.status, DEV_ERR_BAD_PAGE);
      *abort_flag = 1;
    } else {
      const uint32_t full = smem_u32(bars + lane);
      mbar_expect_tx(full, STAGE_BYTES);
      bulk_copy_g2s(smem_u32(ring + size_t(lane) * STAGE_BYTES),
                    a.pool.base + int64_t(first_entry) * a.pool.page_bytes + head_off, STAGE_BYTES, full, policy);
    }
  }
  __syncwarp();
  SGK_TP(11);
  if (my_pages <= nst) return;
  int stage = 0;          // page i uses stage i % nst, in phase i / nst: kept as running counters
  uint32_t parity = 0;    // second use of a stage: wait for the consumers' first release
  for (int base = 0; base < my_pages; base += 32) {
    const int idx = base + lane;
    const int32_t entry = base == 0 ? first_entry : (idx < my_pages ? table[pb + idx] : -1);
    const int cnt = min(32, my_pages - base);
    for (int j = base == 0 ? nst : 0; j < cnt; ++j) {
      const int32_t page = __shfl_sync(0xffffffffu, entry, j);
      if (lane == 0) {
        bool ok = mbar_wait(smem_u32(bars + MMA_MAX_STAGES + stage), parity, abort_flag, a.status);
        if (ok && (page < 0 || page >= a.num_pages)) {
          atomicExch(a.status, DEV_ERR_BAD_PAGE);
          *abort_flag = 1;
          ok = false;
        }
        if (ok) {
          const uint32_t full = smem_u32(bars + stage);
          mbar_expect_tx(full, STAGE_BYTES);
          bulk_copy_g2s(smem_u32(ring + size_t(stage) * STAGE_BYTES),
                        a.pool.base + int64_t(page) * a.pool.page_bytes + head_off, STAGE_BYTES, full, policy);
        }
      }
      if (++stage == nst) {
        stage = 0;
        parity ^= 1;
      }
    }
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// Arrival on a device-wide counter that publishes the block's earlier global writes and, for
// the block that arrives last, makes the others' writes visible: one acquire-release atomic
// instead of a fence, a relaxed atomic and a second fence (the block barrier before it orders
// the other threads' writes before this thread's release).
__device__ __forceinline__ int arrive_acq_rel(int32_t* counter) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  return old;
}

__device__ __forceinline__ int ld_acquire_gpu(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---- outputs that go to the peers as well -------------------------------------------------
// PEERS: the kernel instance used when several GPUs share the sequence by KV-head group: every final
// output cell is stored into the same place of every peer's row too (plain 16-byte stores to peer
// memory over NVLink), and the block that leaves the launch last raises this rank's flag at every
// peer and waits, with a bound, for theirs: when the kernel has run, the local row is complete.
// The compute and the exchange are one launch.
template <bool PEERS>
__device__ __forceinline__ void store_out(const AttnArgs& a, int64_t index, float4 v) {
  *reinterpret_cast<float4*>(a.out + index) = v;
  if (PEERS) {
    for (int p = 0; p < a.n_peers; ++p) *reinterpret_cast<float4*>(a.peer_out[p] + index) = v;
  }
}
__device__ __forceinline__ void st_release_sys_s32(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys_s32(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Last statement of every block of a PEERS launch (all blocks must get here).
__device__ __forceinline__ void peers_finish(const AttnArgs& a, int tid, int* flags) {
  volatile int* last_s = flags + 4;   // a free word of the block's flag area
  // Ordering, from a store to a peer by any thread of any block to the peer's read after its wait:
  // block barrier -> this block's arrival (release, gpu scope) -> the last block's arrival (acquire)
  // -> block barrier -> the flag's store (release, system scope) -> the peer's acquire load. Every
  // link synchronises at a scope that holds both ends, so the chain is a causality order and the
  // peer sees the store; no block needs a system-scope fence of its own.
  __syncthreads();
  if (tid == 0) {
    const int total = gridDim.x * gridDim.y * gridDim.z;
    *last_s = arrive_acq_rel(a.exit_counter) == total - 1;
  }
  __syncthreads();
  if (!*last_s) return;
  // one thread per peer: flag up, then wait for the peer's
  int32_t step = *a.ex_step + 1;
  if (tid < a.n_peers) {
    st_release_sys_s32(a.peer_flags[tid] + a.rank, step);
    uint32_t spins = 0;
    while (ld_acquire_sys_s32(a.local_flags + a.peer_rank[tid]) - step < 0) {
      if (++spins > WAIT_SPINS) {
        atomicExch(a.status, DEV_ERR_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    *a.ex_step = step;
    *a.exit_counter = 0;
  }
}

// Merge shared by ALL blocks of a (sequence, KV head), for launches whose blocks are all resident
// at once (the host checks that the grid fits the device): every block publishes its partial,
// waits (bounded) until all `splits` partials are there, and then merges a slice of the output:
// one warp per cell of four dims, a lane per partial (strided), one round of loads, the sums
// reduced with shuffles. The tail of the launch is then one wait and one L2 round trip instead of
// two merge levels done by single blocks. Returns false when the wait ran out.
constexpr int SHARED_MERGE_MAX_SPLITS = 160;   // five partials per lane
template <int HD, int NT, bool PEERS = false>
__device__ __forceinline__ bool shared_merge(const AttnArgs& a, int splits, int split, int gqa, int64_t qh0,
                                             int32_t* arrive_counter, int32_t* depart_counter, int* flags, int tid) {
  volatile int* abort_flag = flags;
  if (tid == 0) {
    arrive_acq_rel(arrive_counter);   // releases this block's partial (the block has synchronised before)
    uint32_t spins = 0;
    while (ld_acquire_gpu(arrive_counter) < splits) {
      if (++spins > WAIT_SPINS) {
        *abort_flag = 1;
        atomicExch(a.status, DEV_ERR_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  const bool ok = *abort_flag == 0;
  if (ok) {
    const int lane = tid & 31;
    const int warps = NT / 32;
    const int cells = gqa * (HD / 4);
    if (splits <= 32) {
      // One partial per lane. With few splits a block owns many cells (29 at 18 splits, head_dim
      // 256): four cells per pass, all their loads issued before the first reduction, so the
      // block pays a quarter of the L2 round trips.
      constexpr int CELLS = 4;
      const int stride = splits * warps;
      for (int cell0 = split * warps + (tid >> 5); cell0 < cells; cell0 += CELLS * stride) {
        float2 ml[CELLS];
        float4 v[CELLS];
#pragma unroll
        for (int c = 0; c < CELLS; ++c) {
          const int cell = cell0 + c * stride;
          if (cell < cells && lane < splits) {
            const int h = cell / (HD / 4), d = (cell % (HD / 4)) * 4;
            ml[c] = __ldcg(reinterpret_cast<const float2*>(a.part.ml + ((qh0 + h) * a.splits + lane) * 2));
            v[c] = __ldcg(reinterpret_cast<const float4*>(a.part.o + ((qh0 + h) * a.splits + lane) * HD + d));
          }
        }
#pragma unroll
        for (int c = 0; c < CELLS; ++c) {
          const int cell = cell0 + c * stride;
          if (cell >= cells) break;   // uniform over the warp
          const int h = cell / (HD / 4), d = (cell % (HD / 4)) * 4;
          float m = lane < splits ? ml[c].x : -1.0e30f;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
          float l = 0.0f;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          if (lane < splits) {
            const float w = exp2f(ml[c].x - m);
            l += ml[c].y * w;
            acc.x += v[c].x * w;
            acc.y += v[c].y * w;
            acc.z += v[c].z * w;
            acc.w += v[c].w * w;
          }
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) {
            l += __shfl_xor_sync(0xffffffffu, l, off);
            acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
            acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
            acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
            acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
          }
          if (lane == 0) {
            const float inv = 1.0f / l;
            store_out<PEERS>(a, (qh0 + h) * HD + d, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
          }
        }
      }
    } else
    for (int cell = split * warps + (tid >> 5); cell < cells; cell += splits * warps) {
      const int h = cell / (HD / 4), d = (cell % (HD / 4)) * 4;
      const float* pm = a.part.ml + (qh0 + h) * a.splits * 2;
      const float* po = a.part.o + (qh0 + h) * a.splits * HD + d;
      float2 ml[5];
      float4 v[5];
#pragma unroll
      for (int i = 0; i < 5; ++i) {
        const int p = lane + 32 * i;
        if (p < splits) {
          ml[i] = __ldcg(reinterpret_cast<const float2*>(pm + 2 * p));
          v[i] = __ldcg(reinterpret_cast<const float4*>(po + int64_t(p) * HD));
        }
      }
      float m = -1.0e30f;
#pragma unroll
      for (int i = 0; i < 5; ++i)
        if (lane + 32 * i < splits) m = fmaxf(m, ml[i].x);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
      float l = 0.0f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 5; ++i)
        if (lane + 32 * i < splits) {
          const float w = exp2f(ml[i].x - m);
          l += ml[i].y * w;
          acc.x += v[i].x * w;
          acc.y += v[i].y * w;
          acc.z += v[i].z * w;
          acc.w += v[i].w * w;
        }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, off);
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
      }
      if (lane == 0) {
        const float inv = 1.0f / l;
        store_out<PEERS>(a, (qh0 + h) * HD + d, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
      }
    }
  }
  __syncthreads();
  // the block that leaves last puts both counters back (every other block is past its wait)
  if (tid == 0) {
    int old = atomicAdd(depart_counter, 1);
    if (old == splits - 1) {
      *arrive_counter = 0;
      *depart_counter = 0;
    }
  }
  return ok;
}

// ---- thread-block cluster: the splits of one (sequence, KV head) as one cluster ------------
constexpr int CLUSTER_MERGE_MAX_SPLITS = 16;  // the largest cluster the hardware takes (above 8: opt-in per kernel)
__device__ __forceinline__ uint32_t cluster_map_shared(const void* p, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(p)), "r"(cta_rank));
  return remote;
}
// Hardware barrier over all threads of the cluster (like bar.sync over a block: no spinning on
// memory; threads that have exited count as arrived).
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Merge of the splits of one (sequence, KV head) when they run as one thread-block cluster
// (grid x = cluster x = splits, so the rank in the cluster is the split). Cell c (four dims of
// one head) of the output belongs to block c % splits. Every block SENDS each cell of its
// un-normalised output, and its {max, sum} pairs, into the owner's shared memory (distributed
// shared memory stores into a buffer that nothing else uses, so a block that is still streaming
// is not disturbed); the cluster meets at one barrier; every block then merges the cells it owns
// from its own shared memory and writes them out. No partial travels through L2, no device-wide
// atomic is on the path, and after the barrier nobody touches anybody else's memory, so a block
// may leave as soon as it is done. Same arithmetic, in the same order, as merge_block.
//   recv layout: float4 o[splits][cells_per_block] then float2 ml[CLUSTER_MERGE_MAX_SPLITS][8]
template <int HD>
struct ClusterRecv {
  static constexpr int MAX_CELLS = 8 * (HD / 4);                         // gqa <= 8
  static constexpr int O_FLOATS = (MAX_CELLS + CLUSTER_MERGE_MAX_SPLITS) * 4;   // sum over sources of ceil(cells / splits)
  static constexpr int BYTES = O_FLOATS * 4 + CLUSTER_MERGE_MAX_SPLITS * 8 * 8;
};
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_cluster_f2(uint32_t addr, float2 v) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(v.x), "f"(v.y) : "memory");
}
// Sends cell `cell` of this block's output to its owner.
template <int HD>
__device__ __forceinline__ void cluster_send_cell(float* recv, int splits, int split, int gqa, int cell, float4 o) {
  const int cells_per_block = (gqa * (HD / 4) + splits - 1) / splits;
  const int owner = cell % splits, slot = cell / splits;
  st_cluster_f4(cluster_map_shared(recv + (split * cells_per_block + slot) * 4, owner), o);
}
// Sends this block's {max, sum} of every head to every block. Threads [0, gqa * splits).
template <int HD>
__device__ __forceinline__ void cluster_send_ml(float* recv, const float* hml_s, int splits, int split, int gqa,
                                                int tid) {
  if (tid < gqa * splits) {
    const int owner = tid / gqa, h = tid % gqa;
    float* dst = recv + ClusterRecv<HD>::O_FLOATS + (split * 8 + h) * 2;
    st_cluster_f2(cluster_map_shared(dst, owner), make_float2(hml_s[2 * h], hml_s[2 * h + 1]));
  }
}
// Every thread of the block must call this, after its sends.
template <int HD, int NT>
__device__ __forceinline__ void cluster_merge(const AttnArgs& a, const float* recv, int splits, int split, int gqa,
                                              int64_t qh0, int tid, int32_t* seq_counter, int seq_blocks,
                                              int32_t* len_ptr, int64_t len) {
  cluster_arrive_release();
  // After a fused append the block that arrives last for the sequence moves the cursor. The
  // arrival's round trip runs beside the barrier and the merge: issued here by a thread that
  // has little else to do, its result is looked at after the merge.
  int arrived = -1;
  if (seq_counter != nullptr && tid == NT - 1) arrived = arrive_acq_rel(seq_counter);
  cluster_wait_acquire();
  if (tid == 0) SGK_TP(5);
  const int total = gqa * (HD / 4);
  const int cells_per_block = (total + splits - 1) / splits;
  const float* recv_ml = recv + ClusterRecv<HD>::O_FLOATS;
  for (int i = tid; split + splits * i < total; i += NT) {
    const int cell = split + splits * i;
    const int h = cell / (HD / 4), d = (cell % (HD / 4)) * 4;
    // This code runs once per block, so what it costs is mostly the fetch of its instructions:
    // short loops, not sixteen unrolled copies.
    float m = -1.0e30f;
#pragma unroll 4
    for (int p = 0; p < splits; ++p) m = fmaxf(m, recv_ml[(p * 8 + h) * 2]);
    float l = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int p = 0; p < splits; ++p) {
      const float2 ml = *reinterpret_cast<const float2*>(recv_ml + (p * 8 + h) * 2);
      const float4 v = *reinterpret_cast<const float4*>(recv + (p * cells_per_block + i) * 4);
      const float w = exp2f(ml.x - m);
      l += ml.y * w;
      acc.x += v.x * w;
      acc.y += v.y * w;
      acc.z += v.z * w;
      acc.w += v.w * w;
    }
    const float inv = 1.0f / l;
    *reinterpret_cast<float4*>(a.out + (qh0 + h) * HD + d) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
  }
  if (arrived == seq_blocks - 1) {
    *len_ptr = static_cast<int32_t>(len);
    *seq_counter = 0;
  }
  if (tid == 0) SGK_TP(7);
}

// Block-cooperative merge of `count` (<= MERGE_MAX) partials (rows first..first+count
// of a [q head][stride][HD] array) for the gqa heads starting at qh0. A thread owns
// cells of four dims; per pass it handles two cells and issues every load it needs
// (the {max, sum} pairs of the cell's head and the partial values) before the first
// use, so a pass costs one L2 round trip and no block barrier. final != 0: writes the
// normalised output; else writes one un-normalised partial (row dst_row of dst).
template <int HD, int NT = MMA_THREADS, bool PEERS = false>
__device__ __forceinline__ void merge_block(const AttnArgs& a, const Partials& src, int stride, int first, int count, int gqa,
                                            int64_t qh0, bool final, const Partials& dst,
                                            int dst_stride, int dst_row, int tid) {
  constexpr int CELLS = NT >= 256 ? 1 : 2;   // the register budget of a 256-thread block is smaller
  const int total = gqa * (HD / 4);
  for (int base = 0; base < total; base += CELLS * NT) {
    float2 ml[CELLS][MERGE_MAX];
    float4 v[CELLS][MERGE_MAX];
    int cell[CELLS];
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      cell[c] = base + c * NT + tid;
      if (cell[c] < total) {
        const int h = cell[c] / (HD / 4), d = (cell[c] % (HD / 4)) * 4;
        const float* pm = src.ml + ((qh0 + h) * stride + first) * 2;
        const float* po = src.o + ((qh0 + h) * stride + first) * HD + d;
#pragma unroll
        for (int p = 0; p < MERGE_MAX; ++p)
          if (p < count) {
            ml[c][p] = __ldcg(reinterpret_cast<const float2*>(pm + 2 * p));
            v[c][p] = __ldcg(reinterpret_cast<const float4*>(po + int64_t(p) * HD));
          }
      }
    }
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      if (cell[c] >= total) continue;
      const int h = cell[c] / (HD / 4), d = (cell[c] % (HD / 4)) * 4;
      float m = -1.0e30f;
#pragma unroll
      for (int p = 0; p < MERGE_MAX; ++p)
        if (p < count) m = fmaxf(m, ml[c][p].x);
      float l = 0.0f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < MERGE_MAX; ++p)
        if (p < count) {
          const float w = exp2f(ml[c][p].x - m);
          l += ml[c][p].y * w;
          acc.x += v[c][p].x * w;
          acc.y += v[c][p].y * w;
          acc.z += v[c][p].z * w;
          acc.w += v[c][p].w * w;
        }
      if (final) {
        const float inv = 1.0f / l;
        store_out<PEERS>(a, (qh0 + h) * HD + d, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
      } else {
        *reinterpret_cast<float4*>(dst.o + ((qh0 + h) * dst_stride + dst_row) * HD + d) = acc;
        if (d == 0) *reinterpret_cast<float2*>(dst.ml + ((qh0 + h) * dst_stride + dst_row) * 2) = make_float2(m, l);
      }
    }
  }
}

// Tail shared by the paged attention kernels: merges the consumer warps' states
// (o_s: [warps][8][opad] un-normalised outputs, ml_s: [warps][8] {max, sum}), writes the
// block's partial (or the final output when there is one split), moves the device cursor
// after a fused append, and runs the two-level merge of the splits.
// CLUSTER: the kernel instance that is launched as clusters (its splits merge through distributed
// shared memory). A separate instance, so that the other one is compiled without a trace of that path:
// with both in one kernel the page loop of the long-stream case lost 1.3 % (register allocation).
template <int HD, bool CLUSTER, bool PEERS = false, int NT = MMA_THREADS>
__device__ __forceinline__ void finish_block(const AttnArgs& a, const float* o_s, const float* ml_s, int opad,
                                             int* flags, int seq, int kvh, int split, int gqa, bool do_append,
                                             int32_t* len_ptr, int64_t len, int tid, int splits, float* recv) {
  // recv: ClusterRecv<HD>::BYTES of shared memory used by nothing else, where the blocks of a
  // cluster leave their outputs for this block to merge
  // `splits` is this sequence's own split count (<= a.splits, the stride of the partial arrays)
  const int n_groups = (splits + a.group_size - 1) / a.group_size;
  if (tid == 0) SGK_TP(4);
  // ---- merge the consumer warps; write the partial or the final output ----
  // ml_s holds [warps][8]{max, sum}; behind it: the per-(head, warp) weights and the block's
  // {max, sum} per head (the shared-memory layouts reserve 512 bytes for this area).
  float* wgt_s = const_cast<float*>(ml_s) + MMA_CONSUMERS * 8 * 2;   // [8][warps]
  float* hml_s = wgt_s + 8 * MMA_CONSUMERS;                           // [8]{max, sum}
  const int64_t qh0 = int64_t(seq) * a.q_heads + int64_t(kvh) * gqa;
  if (tid < 8) {
    float mb = -1.0e30f;
#pragma unroll
    for (int w = 0; w < MMA_CONSUMERS; ++w) mb = fmaxf(mb, ml_s[(w * 8 + tid) * 2]);
    float lb = 0.0f;
#pragma unroll
    for (int w = 0; w < MMA_CONSUMERS; ++w) {
      const float wg = exp2f(ml_s[(w * 8 + tid) * 2] - mb);
      wgt_s[tid * MMA_CONSUMERS + w] = wg;
      lb += ml_s[(w * 8 + tid) * 2 + 1] * wg;
    }
    hml_s[2 * tid] = mb;
    hml_s[2 * tid + 1] = lb;
  }
  __syncthreads();
  for (int idx = tid; idx < gqa * (HD / 4); idx += NT) {
    const int h = idx / (HD / 4), d = (idx % (HD / 4)) * 4;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < MMA_CONSUMERS; ++w) {
      const float4 v = *reinterpret_cast<const float4*>(o_s + (w * 8 + h) * opad + d);
      const float wg = wgt_s[h * MMA_CONSUMERS + w];
      o.x += v.x * wg;
      o.y += v.y * wg;
      o.z += v.z * wg;
      o.w += v.w * wg;
    }
    if (splits == 1) {
      const float inv = 1.0f / hml_s[2 * h + 1];
      store_out<PEERS>(a, (qh0 + h) * HD + d, make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv));
    } else if (CLUSTER) {
      cluster_send_cell<HD>(recv, splits, split, gqa, idx, o);
    } else {
      *reinterpret_cast<float4*>(a.part.o + ((qh0 + h) * a.splits + split) * HD + d) = o;
      if (d == 0)
        *reinterpret_cast<float2*>(a.part.ml + ((qh0 + h) * a.splits + split) * 2) =
            make_float2(hml_s[2 * h], hml_s[2 * h + 1]);
    }
  }
  if (splits > 1 || do_append) {
    const int group = split / a.group_size;
    const int group_first = group * a.group_size;
    const int group_count = min(a.group_size, splits - group_first);
    int32_t* group_counter = a.group_counters + (int64_t(seq) * a.pool.kv_heads + kvh) * a.max_groups + group;
    int32_t* head_counter = a.head_counters + int64_t(seq) * a.pool.kv_heads + kvh;
    if (CLUSTER && splits > 1) {
      cluster_send_ml<HD>(recv, hml_s, splits, split, gqa, tid);
      cluster_merge<HD, NT>(a, recv, splits, split, gqa, qh0, tid, do_append ? a.seq_counters + seq : nullptr,
                            splits * a.pool.kv_heads, len_ptr, len);
      if (tid == 0) SGK_TP(6);
      return;
    }
    __syncthreads();
    if (a.shared_merge && splits > 1 && splits <= SHARED_MERGE_MAX_SPLITS) {
      if (tid == 32 && do_append) {
        // the block that arrives last for the sequence moves the cursor
        int total = splits * a.pool.kv_heads;
        int old = arrive_acq_rel(a.seq_counters + seq);
        if (old == total - 1) {
          *len_ptr = static_cast<int32_t>(len);
          a.seq_counters[seq] = 0;
        }
      }
      shared_merge<HD, NT, PEERS>(a, splits, split, gqa, qh0, head_counter, group_counter - group, flags, tid);
      if (tid == 0) SGK_TP(7);
      return;
    }
    // two arrivals, on two threads of different warps so that their round trips overlap
    if (tid == 0 && splits > 1) {
      int old = arrive_acq_rel(group_counter);
      flags[1] = (old == group_count - 1);
      if (flags[1]) *group_counter = 0;
    }
    if (tid == 32 && do_append) {
      // the block that arrives last for the sequence moves the cursor
      int total = splits * a.pool.kv_heads;
      int old = arrive_acq_rel(a.seq_counters + seq);
      if (old == total - 1) {
        *len_ptr = static_cast<int32_t>(len);
        a.seq_counters[seq] = 0;
      }
    }
    __syncthreads();
    if (tid == 0) SGK_TP(5);
    if (splits > 1 && flags[1]) {
      // this block completed its group: merge the group (or everything, if one group)
      const bool single = n_groups == 1;
      merge_block<HD, NT, PEERS>(a, a.part, a.splits, group_first, group_count, gqa, qh0, single, a.part2,
                      a.max_groups, group, tid);
      if (tid == 0) SGK_TP(6);
      if (!single) {
        __syncthreads();
        if (tid == 0) {
          int old = arrive_acq_rel(head_counter);
          flags[1] = (old == n_groups - 1);
          if (flags[1]) *head_counter = 0;
        }
        __syncthreads();
        if (flags[1]) {
          merge_block<HD, NT, PEERS>(a, a.part2, a.max_groups, 0, n_groups, gqa, qh0, true, a.part2,
                          a.max_groups, 0, tid);
          if (tid == 0) SGK_TP(7);
        }
      }
    }
  }
}

}  // namespace sgk
