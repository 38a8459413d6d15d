// Data movers of the path: the paged gather (the read-back the reference does
// with kv.keys()/values()), the prefix-cache page copy (snapshot / restore), the
// linear-state copy (the reference's blit, src/metal_backend/linear_attention.rs:3027-3198),
// the eviction scrub and the deterministic input fill.
#include "kernels.h"

namespace sgk {

// SMs of the current device (asked once per device).
static int current_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 132;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 132;
    cached[dev] = n;
  }
  return cached[dev];
}


// ---- gather -------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_rows_kernel(GatherArgs a) {
  const int hd = a.pool.head_dim, kvh = a.pool.kv_heads;
  const int kv_dim = kvh * hd;
  const int64_t total = a.n * kv_dim;
  const int32_t* table = a.pool.tables + int64_t(a.slot) * a.pool.table_stride;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t r = i / kv_dim;
    const int col = static_cast<int>(i % kv_dim);
    const int head = col / hd, dim = col % hd;
    const int64_t row = a.row0 + r;
    const int32_t page = table[row / PAGE_TOKENS];
    if (page < 0 || page >= a.num_pages) {
      atomicExch(a.status, DEV_ERR_BAD_PAGE);
      continue;
    }
    const int rin = static_cast<int>(row % PAGE_TOKENS);
    const uint8_t* kt = a.pool.base + tile_offset(a.pool, page, a.layer, head, 0);
    const uint8_t* vt = kt + a.pool.tile_bytes;
    if (a.mode == 1) {
      reinterpret_cast<float*>(a.k_out)[i] = load_tile_elem(kt, a.pool.dtype, hd, 0, rin, dim);
      reinterpret_cast<float*>(a.v_out)[i] = load_tile_elem(vt, a.pool.dtype, hd, 1, rin, dim);
    } else if (a.pool.dtype == KV_F32) {
      reinterpret_cast<float*>(a.k_out)[i] = reinterpret_cast<const float*>(kt)[rin * hd + dim];
      reinterpret_cast<float*>(a.v_out)[i] = reinterpret_cast<const float*>(vt)[rin * hd + dim];
    } else if (a.pool.dtype == KV_BF16) {
      int e = bf16_elem_index(rin, dim, hd);
      reinterpret_cast<uint16_t*>(a.k_out)[i] = reinterpret_cast<const uint16_t*>(kt)[e];
      reinterpret_cast<uint16_t*>(a.v_out)[i] = reinterpret_cast<const uint16_t*>(vt)[e];
    } else {
      reinterpret_cast<uint8_t*>(a.k_out)[i] = kt[u8_k_code_index(rin, dim, hd)];
      reinterpret_cast<uint8_t*>(a.v_out)[i] = vt[u8_v_code_index(rin, dim, hd)];
      if (dim % QGROUP == 0) {
        const int groups = kv_dim / QGROUP;
        const int64_t gi = r * groups + col / QGROUP;
        const int grp = dim / QGROUP;
        a.k_scale[gi] = *reinterpret_cast<const uint16_t*>(kt + u8_scale_offset(rin, grp, hd));
        a.k_bias[gi] = *reinterpret_cast<const uint16_t*>(kt + u8_bias_offset(0, rin, grp, hd));
        a.v_scale[gi] = *reinterpret_cast<const uint16_t*>(vt + u8_scale_offset(rin, grp, hd));
        a.v_bias[gi] = *reinterpret_cast<const uint16_t*>(vt + u8_bias_offset(1, rin, grp, hd));
      }
    }
  }
}

cudaError_t launch_gather(const GatherArgs& a, cudaStream_t stream) {
  int64_t total = a.n * a.pool.kv_heads * a.pool.head_dim;
  int blocks = static_cast<int>(total / 256 + 1);
  if (blocks > current_sm_count() * 8) blocks = current_sm_count() * 8;
  gather_rows_kernel<<<blocks, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

// ---- page copy (prefix snapshot / restore) ---------------------------------------
// A page is one contiguous, 256-byte aligned range per layer (all heads, K and V). The grid
// is a multiple of the SM count; each block walks (page, layer, 16 KiB piece) work items,
// every thread moving four 16-byte vectors per item with all loads issued before
// the stores, so ~4 KiB per warp are in flight.
constexpr int COPY_THREADS = 256;
constexpr int COPY_VEC_PER_THREAD = 4;
constexpr int64_t COPY_PIECE = int64_t(COPY_THREADS) * COPY_VEC_PER_THREAD * 16;  // 16 KiB

__global__ void __launch_bounds__(COPY_THREADS) copy_pages_kernel(uint8_t* __restrict__ dst_base,
                                                                  const uint8_t* __restrict__ src_base,
                                                                  const int32_t* __restrict__ dst_pages,
                                                                  const int32_t* __restrict__ src_pages,
                                                                  int n_pages, int64_t page_bytes, int n_layers,
                                                                  int64_t layer_stride, CopyInstall install) {
  // A restore also makes the copied pages the sequence's block table and moves its cursors: done
  // here by the first block, so that the whole restore is one staging copy and one launch.
  if (blockIdx.x == 0 && install.table != nullptr) {
    for (int i = threadIdx.x; i < n_pages; i += COPY_THREADS) install.table[i] = dst_pages[i];
    for (int i = threadIdx.x; i < install.n_lens; i += COPY_THREADS) install.lens[i] = install.len_value;
  }
  const int64_t pieces_per_page = (page_bytes + COPY_PIECE - 1) / COPY_PIECE;
  const int64_t per_page = pieces_per_page * n_layers;
  const int64_t items = per_page * n_pages;
  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int64_t p = item / per_page, rest = item % per_page;
    const int64_t layer = rest / pieces_per_page, piece = rest % pieces_per_page;
    const int64_t dpage = dst_pages ? dst_pages[p] : p;
    const int64_t spage = src_pages ? src_pages[p] : p;
    const int64_t within = layer * layer_stride + piece * COPY_PIECE;
    const uint4* s = reinterpret_cast<const uint4*>(src_base + spage * page_bytes + within);
    uint4* d = reinterpret_cast<uint4*>(dst_base + dpage * page_bytes + within);
    const int64_t vecs = min(COPY_PIECE, page_bytes - piece * COPY_PIECE) / 16;
    uint4 r[COPY_VEC_PER_THREAD];
#pragma unroll
    for (int k = 0; k < COPY_VEC_PER_THREAD; ++k) {
      int64_t i = threadIdx.x + int64_t(k) * COPY_THREADS;
      if (i < vecs) r[k] = __ldcs(s + i);
    }
#pragma unroll
    for (int k = 0; k < COPY_VEC_PER_THREAD; ++k) {
      int64_t i = threadIdx.x + int64_t(k) * COPY_THREADS;
      if (i < vecs) __stcs(d + i, r[k]);
    }
  }
}

static int copy_grid(int64_t items, int sm_count = 0) {
  int64_t g = int64_t(sm_count > 0 ? sm_count : current_sm_count()) * 8;
  if (items < g) g = items;
  return static_cast<int>(g < 1 ? 1 : g);
}

cudaError_t launch_copy_pages(uint8_t* dst_base, const uint8_t* src_base, const int32_t* d_dst_pages,
                              const int32_t* d_src_pages, int n_pages, int64_t page_bytes, int n_layers,
                              int64_t layer_stride, int sm_count, cudaStream_t stream, const CopyInstall* install) {
  if (n_pages <= 0) return cudaSuccess;
  int64_t items = ((page_bytes + COPY_PIECE - 1) / COPY_PIECE) * n_layers * n_pages;
  copy_pages_kernel<<<copy_grid(items, sm_count), COPY_THREADS, 0, stream>>>(dst_base, src_base, d_dst_pages, d_src_pages,
                                                                   n_pages, page_bytes, n_layers, layer_stride,
                                                                   install ? *install : CopyInstall{});
  return cudaGetLastError();
}

// Contiguous copy: one "page" of `bytes` (16-byte multiple part) plus a byte tail.
__global__ void copy_tail_kernel(uint8_t* dst, const uint8_t* src, int64_t n) {
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i < n) dst[i] = src[i];
}

cudaError_t launch_copy_bytes(void* dst, const void* src, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return cudaSuccess;
  int64_t body = bytes & ~int64_t(15);
  bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0;
  if (!aligned) body = 0;
  if (body > 0) {
    int64_t items = (body + COPY_PIECE - 1) / COPY_PIECE;
    copy_pages_kernel<<<copy_grid(items), COPY_THREADS, 0, stream>>>(
        static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), nullptr, nullptr, 1, body, 1, 0, CopyInstall{});
  }
  int64_t tail = bytes - body;
  if (tail > 0) {
    copy_tail_kernel<<<static_cast<int>((tail + 255) / 256), 256, 0, stream>>>(
        static_cast<uint8_t*>(dst) + body, static_cast<const uint8_t*>(src) + body, tail);
  }
  return cudaGetLastError();
}

// ---- eviction scrub ------------------------------------------------------------------
__global__ void __launch_bounds__(COPY_THREADS) scrub_pages_kernel(uint8_t* base, const int32_t* pages,
                                                                   int n_pages, int64_t page_bytes, int n_layers,
                                                                   int64_t layer_stride) {
  const int64_t vecs_per_piece = page_bytes / 16;
  const int64_t vecs_per_page = vecs_per_piece * n_layers;
  const int64_t total = vecs_per_page * n_pages;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t p = i / vecs_per_page, rest = i % vecs_per_page;
    const int64_t layer = rest / vecs_per_piece, v = rest % vecs_per_piece;
    reinterpret_cast<uint4*>(base + int64_t(pages[p]) * page_bytes + layer * layer_stride)[v] = make_uint4(0, 0, 0, 0);
  }
}

cudaError_t launch_scrub_pages(uint8_t* base, const int32_t* d_pages, int n_pages, int64_t page_bytes, int n_layers,
                               int64_t layer_stride, int sm_count, cudaStream_t stream) {
  if (n_pages <= 0) return cudaSuccess;
  int64_t total = page_bytes / 16 * n_layers * n_pages;
  scrub_pages_kernel<<<copy_grid((total + COPY_THREADS - 1) / COPY_THREADS, sm_count), COPY_THREADS, 0, stream>>>(
      base, d_pages, n_pages, page_bytes, n_layers, layer_stride);
  return cudaGetLastError();
}

// ---- deterministic approximate-normal fill -----------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__global__ void fill_normal_kernel(float* out, int64_t n, uint64_t key, uint64_t index0) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n;
       i += int64_t(gridDim.x) * blockDim.x) {
    uint64_t idx = index0 + static_cast<uint64_t>(i);
    uint64_t a = splitmix64(key + 2 * idx), b = splitmix64(key + 2 * idx + 1);
    int32_t sum = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      sum += static_cast<int32_t>((a >> (16 * k)) & 0xFFFF);
      sum += static_cast<int32_t>((b >> (16 * k)) & 0xFFFF);
    }
    out[i] = __fmul_rn(static_cast<float>(sum - 262140), 0x1.3988e2p-16f);
  }
}

cudaError_t launch_fill_normal(float* out, int64_t n, uint64_t seed, uint64_t stream_id, uint64_t index0,
                               cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  uint64_t x = seed * 0xD1342543DE82EF95ull + stream_id;
  // host-side splitmix64 of the key, same function as on the device
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  uint64_t key = x ^ (x >> 31);
  int64_t blocks = (n + 255) / 256;
  if (blocks > int64_t(current_sm_count()) * 16) blocks = int64_t(current_sm_count()) * 16;
  fill_normal_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(out, n, key, index0);
  return cudaGetLastError();
}

}  // namespace sgk
