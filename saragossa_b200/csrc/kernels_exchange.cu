// Exchange of attention outputs between the GPUs that share one long sequence by KV-head group:
// every rank holds the full output row [q_heads * head_dim] and has computed its own slice of it.
// One small kernel per rank and layer stores that slice straight into every peer's row (plain
// stores to peer memory over NVLink), then raises its flag in every peer's memory and waits, with
// a bound, until every peer has raised its own: when the kernel ends, the local row is complete.
// It replaces an all-gather call (one library launch and its protocol) by one launch of a few
// hundred threads. No multicast, no TMA: 16-byte stores, a release store and acquire loads at
// system scope.
//
// Flags carry a step number that the kernel itself keeps in device memory and advances, so a CUDA
// graph that contains the kernel can be replayed. A peer may be one exchange ahead (it has passed
// its wait and writes the next row while this rank still reads the current one): callers alternate
// between two output rows, or use a row per layer.
#include "device_common.cuh"
#include "kernels.h"

namespace sgk {

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

constexpr int EXCHANGE_THREADS = 512;
constexpr uint32_t EXCHANGE_SPINS = 1u << 22;   // bound of the wait for a peer (a second or so)

__global__ void __launch_bounds__(EXCHANGE_THREADS) exchange_slices_kernel(ExchangeArgs a) {
  const int tid = threadIdx.x;
  // 1. my slice into every peer's row
  const float4* src = reinterpret_cast<const float4*>(a.local_row + a.slice_offset);
  for (int i = tid; i < a.slice_floats / 4; i += EXCHANGE_THREADS) {
    const float4 v = src[i];
    for (int p = 0; p < a.n_ranks; ++p)
      if (p != a.rank) reinterpret_cast<float4*>(a.peer_row[p] + a.slice_offset)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  // 2. tell every peer (one thread per peer), 3. wait for every peer's slice
  __shared__ int32_t step_s;
  if (tid == 0) step_s = *a.step + 1;
  __syncthreads();
  const int32_t step = step_s;
  if (tid < a.n_ranks && tid != a.rank) {
    st_release_sys(a.peer_flags[tid] + a.rank, step);
    uint32_t spins = 0;
    // signed difference: the counter may wrap
    while (ld_acquire_sys(a.local_flags + tid) - step < 0) {
      if (++spins > EXCHANGE_SPINS) {
        atomicExch(a.status, DEV_ERR_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  if (tid == 0) *a.step = step;
}

cudaError_t launch_exchange_slices(const ExchangeArgs& a, cudaStream_t stream) {
  exchange_slices_kernel<<<1, EXCHANGE_THREADS, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace sgk
