// sgk_kv_enqueue_attention_noalloc: paged decode attention for callers that must
// not allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits or too slow to
// tolerate. Examples are a host that has handed the whole device to its own
// arena and forbids side allocations, a latency-critical serving loop that may
// not take the implicit device synchronisation and the driver lock that
// cudaMalloc/cudaFree bring, and code that runs while a stream is being captured
// into a CUDA graph (an allocation is illegal there). The regular entry point,
// sgk_kv_enqueue_attention, lazily allocates a split-K workspace the first time
// it is used on a KV state; this variant never does.
//
// How: the split-K workspace (un-normalised partial outputs, their {max, sum}
// pairs, the second-level partials and the arrival counters) lives in ONE
// file-scope __device__ array of SGK_NOALLOC_SCRATCH_BYTES (4 MiB). Every GPU
// that loads this library holds that array until the process exits. In host
// code the array's name is only a host-side stand-in for the symbol, not a
// device address, so the address the kernels get is obtained with
// cudaGetSymbolAddress, once per device, with that device current.
//
// Rules for the caller:
//   * The first call on a device performs that set-up (it may make the driver
//     load this module). Make the first call BEFORE any stream capture begins.
//   * All calls share the one array, and it keeps whatever the last call left
//     in it. The counters that must start at zero are cleared in stream order
//     at the start of every call. Two calls whose kernels can overlap on the GPU
//     (different streams without an ordering between them, or different KV
//     states on concurrent streams) race on the array: order them.
//   * Shapes whose workspace cannot fit are refused with a Config error; the
//     number of splits is reduced first so that it fits.
#include <algorithm>
#include <cmath>
#include <mutex>

#include "host.h"

namespace sgk {

constexpr size_t NOALLOC_SCRATCH_BYTES = 4u << 20;   // SGK_NOALLOC_SCRATCH_BYTES in sgk.h
constexpr int NOALLOC_MAX_Q_DIM = 16384;             // q_heads * head_dim
constexpr int NOALLOC_MAX_GROUPS = 12;
constexpr int NOALLOC_COUNTER_WORDS = 2048;          // head + sequence + group counters
constexpr int NOALLOC_MAX_DEVICES = 64;

// The workspace itself. Device code may name it directly; host code may not use
// the name as a pointer (see below).
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

static std::mutex g_noalloc_mutex;
static unsigned char* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};

// Device address of the workspace on `device`, resolved once per device with that
// device current. cudaGetSymbolAddress allocates nothing.
static int noalloc_scratch(int device, unsigned char** out) {
  if (device < 0 || device >= NOALLOC_MAX_DEVICES) return fail(SGK_ERR_CONFIG, "device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[device] == nullptr) {
    // the caller has made `device` current (DeviceGuard in the entry point)
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(SGK_ERR_BACKEND, "cudaGetSymbolAddress(no-alloc workspace) failed on device %d: %s", device,
                  cudaGetErrorString(e));
    g_noalloc_ptr[device] = static_cast<unsigned char*>(ptr);
  }
  *out = g_noalloc_ptr[device];
  return SGK_OK;
}

// Makes `device` current for the duration of a call and puts the caller's device back.
struct DeviceGuard {
  int previous = -1;
  bool switched = false;
  cudaError_t enter(int device) {
    cudaError_t e = cudaGetDevice(&previous);
    if (e != cudaSuccess) return e;
    if (previous == device) return cudaSuccess;
    e = cudaSetDevice(device);
    switched = e == cudaSuccess;
    return e;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(previous);
  }
};

// Bytes of workspace a launch with `splits` splits needs after the counters.
static size_t noalloc_need(int q_heads, int hd, int splits) {
  size_t level1 = size_t(q_heads) * splits * (size_t(hd) + 2) * sizeof(float);
  size_t level2 = size_t(q_heads) * NOALLOC_MAX_GROUPS * (size_t(hd) + 2) * sizeof(float);
  return level1 + level2 + 4 * 256;  // each of the four arrays starts on a 256-byte boundary
}

}  // namespace sgk

using namespace sgk;

struct sgk_kv : Kv {};

extern "C" int32_t sgk_kv_enqueue_attention_noalloc(sgk_kv* kv, void* stream, const float* d_q, float* d_out,
                                                    int64_t window_start, float attn_scalar) {
  if (!kv) return fail(SGK_ERR_BACKEND, "null KV state");
  if (!d_q || !d_out) return fail(SGK_ERR_BACKEND, "attention: null device pointer");
  Pool* pool = kv->pool();
  if (pool->host_only()) return fail(SGK_ERR_BACKEND, "attention over a bookkeeping-only pool");
  State* st = kv->st;
  const int hd = pool->head_dim, kvh = pool->kv_heads, qh = kv->q_heads;
  if (qh * hd > NOALLOC_MAX_Q_DIM)
    return fail(SGK_ERR_CONFIG,
                "no-alloc attention: q_heads*head_dim = %d exceeds the maximum %d the static workspace is sized for",
                qh * hd, NOALLOC_MAX_Q_DIM);
  const size_t counter_bytes = NOALLOC_COUNTER_WORDS * sizeof(int32_t);
  if (size_t(std::max(qh, kvh)) + 1 + size_t(kvh) * NOALLOC_MAX_GROUPS > NOALLOC_COUNTER_WORDS)
    return fail(SGK_ERR_CONFIG, "no-alloc attention: %d heads exceed the counters of the static workspace", qh);
  // same checks, same error kinds as the regular entry point
  const int64_t len = kv->len();
  if (len == 0) return fail(SGK_ERR_DIMENSION, "attention_decode on an empty KV");
  if (window_start < 0 || window_start >= len)
    return fail(SGK_ERR_DIMENSION, "attention_decode empty window: start=%lld, len=%lld", (long long)window_start,
                (long long)len);
  if (window_start / PAGE_TOKENS < kv->seq->released_pages)
    return fail(SGK_ERR_DIMENSION, "attention window reaches rows released by the sliding window");

  // The state's device is current for every call (not only for the first one, which resolves the
  // symbol), and the caller's own current device is put back on return.
  DeviceGuard guard;
  SGK_CUDA(guard.enter(st->device));
  unsigned char* scratch = nullptr;
  SGK_TRY(noalloc_scratch(st->device, &scratch));

  // the same kernel selection as the allocating entry point: tensor-core kernels over bf16 and over
  // u8 group-32 pages, the generic kernel for everything else
  const bool u8 = attention_u8_supported(pool->dtype, hd, qh / kvh);
  const bool mma = u8 || attention_mma_supported(pool->dtype, hd, qh / kvh);
  // split count: fill the SMs (two blocks each for the tensor-core kernel, eight for the
  // generic one), keep a few pages per split, and stay inside the static workspace
  const int64_t pages = (len - window_start + PAGE_TOKENS - 1) / PAGE_TOKENS;
  const int64_t units = mma ? kvh : qh;
  const int64_t slots = int64_t(st->sm_count) * (mma ? 2 : 8);
  int64_t splits = std::max<int64_t>(1, slots / units);
  splits = std::min<int64_t>(splits, std::max<int64_t>(1, pages / (mma ? 8 : 2)));
  splits = std::min<int64_t>(splits, 144);
  while (splits > 1 && noalloc_need(qh, hd, static_cast<int>(splits)) + counter_bytes > NOALLOC_SCRATCH_BYTES) --splits;
  if (noalloc_need(qh, hd, static_cast<int>(splits)) + counter_bytes > NOALLOC_SCRATCH_BYTES)
    return fail(SGK_ERR_CONFIG, "no-alloc attention: the workspace of this shape exceeds %zu bytes",
                NOALLOC_SCRATCH_BYTES);

  cudaStream_t cs = st->pick(stream);
  // The array keeps the previous call's contents; the arrival counters must start at zero.
  SGK_CUDA(cudaMemsetAsync(scratch, 0, counter_bytes, cs));

  int32_t* counters = reinterpret_cast<int32_t*>(scratch);
  unsigned char* cursor = scratch + counter_bytes;
  auto carve = [&cursor](size_t floats) {
    float* p = reinterpret_cast<float*>(cursor);
    cursor += (floats * sizeof(float) + 255) / 256 * 256;
    return p;
  };
  AttnArgs a{};
  a.pool = pool->view();
  a.layer = kv->layer;
  a.slots = nullptr;
  a.slot0 = kv->seq->slot;
  a.q_heads = qh;
  a.q = d_q;
  a.out = d_out;
  a.window_start = window_start;
  a.sliding_window = 0;
  const float scalar = attn_scalar > 0.0f ? attn_scalar : static_cast<float>(hd);
  a.scale_log2e = 1.4426950408889634f / std::sqrt(scalar);
  a.splits = static_cast<int>(splits);
  a.part.o = carve(size_t(qh) * a.splits * hd);
  a.part.ml = carve(size_t(qh) * a.splits * 2);
  a.part2.o = carve(size_t(qh) * NOALLOC_MAX_GROUPS * hd);
  a.part2.ml = carve(size_t(qh) * NOALLOC_MAX_GROUPS * 2);
  a.max_groups = NOALLOC_MAX_GROUPS;
  a.group_size = a.splits;
  if (a.splits > 12) a.group_size = std::min(static_cast<int>(std::ceil(std::sqrt(double(a.splits)))), 12);
  a.n_groups = (a.splits + a.group_size - 1) / a.group_size;
  a.head_counters = counters;
  a.seq_counters = counters + std::max(qh, kvh);
  a.group_counters = a.seq_counters + 1;
  a.status = st->d_status;
  a.num_pages = pool->num_pages;
  a.k_new = nullptr;
  a.v_new = nullptr;
  if (u8) {
    a.n_stages = attention_u8_max_stages(hd);
    SGK_CUDA(launch_attention_u8(a, 1, cs));
  } else if (mma) {
    a.n_stages = attention_mma_max_stages(hd);
    SGK_CUDA(launch_attention_mma(a, 1, cs));
  } else {
    SGK_CUDA(launch_attention_generic(a, 1, cs));
  }
  st->launches += 1;
  return SGK_OK;
}
