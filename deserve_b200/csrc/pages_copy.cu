// KV swap data movement: gather/scatter of scattered pages into the
// layer-major chunk layout (pack / unpack kernels), the pipelined
// pack -> DMA and DMA -> unpack drivers for per-task offload and reload, and
// the microbatch region swap (per-layer DMA, both link directions at once).
#include <algorithm>

#include "common.cuh"

namespace dsv {
namespace {

constexpr int kCopyThreads = 256;

// A "row" is one page of one layer (page_vecs 16-byte vectors). Rows of the
// layer window are dense, task after task: task t starts at row
// ids_indptr[t] * window and holds n_t * window rows, row = layer_local * n_t + p.
// A CTA copies whole rows: 16 bytes per thread per trip, 4 trips in flight.
template <bool kPack>
__global__ void __launch_bounds__(kCopyThreads)
pack_kernel(unsigned char* __restrict__ pages_base, int64_t layer_stride_bytes, int page_vecs, int64_t num_pages,
            const int32_t* __restrict__ page_ids, const int32_t* __restrict__ ids_indptr, int n_tasks,
            int64_t total_rows, int layer_begin, int window, unsigned char* __restrict__ packed,
            int* status) {
  for (int64_t r = blockIdx.x; r < total_rows; r += gridDim.x) {
    int lo = 0, hi = n_tasks;  // ids_indptr[lo]*window <= r < ids_indptr[hi]*window
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((int64_t)__ldg(ids_indptr + mid) * window <= r) lo = mid; else hi = mid;
    }
    const int i0 = __ldg(ids_indptr + lo);
    const int n_t = __ldg(ids_indptr + lo + 1) - i0;
    const int64_t local = r - (int64_t)i0 * window;
    if (n_t <= 0 || local < 0 || local >= (int64_t)n_t * window) {
      if (threadIdx.x == 0) record_status(status, ST_BAD_REQUEST);
      continue;
    }
    const int layer = layer_begin + (int)(local / n_t);
    const int page = __ldg(page_ids + i0 + (int)(local % n_t));
    if (page < 0 || page >= num_pages) {  // a stale id must never reach memory outside the slab
      if (threadIdx.x == 0) record_status(status, ST_BAD_PAGE_ID);
      continue;
    }
    uint4* pg = reinterpret_cast<uint4*>(pages_base + (int64_t)layer * layer_stride_bytes) +
                (int64_t)page * page_vecs;
    uint4* pk = reinterpret_cast<uint4*>(packed) + r * page_vecs;
    const uint4* src = kPack ? pg : pk;
    uint4* dst = kPack ? pk : pg;
    int v = threadIdx.x;
    for (; v + 3 * kCopyThreads < page_vecs; v += 4 * kCopyThreads) {
      const uint4 a = ld_stream16(src + v);
      const uint4 b = ld_stream16(src + v + kCopyThreads);
      const uint4 c = ld_stream16(src + v + 2 * kCopyThreads);
      const uint4 d = ld_stream16(src + v + 3 * kCopyThreads);
      st_stream16(dst + v, a);
      st_stream16(dst + v + kCopyThreads, b);
      st_stream16(dst + v + 2 * kCopyThreads, c);
      st_stream16(dst + v + 3 * kCopyThreads, d);
    }
    for (; v < page_vecs; v += kCopyThreads) st_stream16(dst + v, ld_stream16(src + v));
  }
}

// returns <0 error, 1 nothing to do, 0 go
int check_pack_args(const char* who, const void* pages_base, int64_t layer_stride_bytes, int64_t page_bytes,
                    int64_t num_pages, const int32_t* page_ids, const int32_t* ids_indptr, int n_tasks, int64_t total_ids,
                    int layer_begin, int layer_end, const void* packed) {
  DSV_REQUIRE(n_tasks >= 0 && total_ids >= 0, "%s: negative task or page count", who);
  if (n_tasks == 0 || total_ids == 0) return 1;
  DSV_REQUIRE(pages_base && page_ids && ids_indptr && packed, "%s: null pointer argument", who);
  DSV_REQUIRE(page_bytes > 0 && page_bytes % 16 == 0, "%s: page_bytes (%lld) must be a positive multiple of 16", who,
              (long long)page_bytes);
  DSV_REQUIRE(page_bytes / 16 < (1ll << 31), "%s: page too large", who);
  DSV_REQUIRE(num_pages > 0 && num_pages < (1ll << 31), "%s: num_pages (%lld) out of range", who,
              (long long)num_pages);
  DSV_REQUIRE(layer_stride_bytes % 16 == 0 && layer_stride_bytes >= num_pages * page_bytes,
              "%s: a layer slab of %lld bytes cannot hold %lld pages of %lld bytes", who,
              (long long)layer_stride_bytes, (long long)num_pages, (long long)page_bytes);
  DSV_REQUIRE(layer_begin >= 0 && layer_end > layer_begin, "%s: empty layer window [%d,%d)", who, layer_begin,
              layer_end);
  DSV_REQUIRE(aligned16(pages_base) && aligned16(packed), "%s: pointers must be 16-byte aligned", who);
  return 0;
}

template <bool kPack>
int launch_pack(unsigned char* pages_base, int64_t layer_stride_bytes, int64_t page_bytes, int64_t num_pages,
                const int32_t* page_ids,
                const int32_t* ids_indptr, int n_tasks, int64_t total_ids, int layer_begin, int layer_end,
                unsigned char* packed, cudaStream_t st) {
  const int window = layer_end - layer_begin;
  const int64_t total_rows = total_ids * window;
  // enough CTAs to cover the machine several times over; further rows are strided
  const unsigned grid = (unsigned)std::min<int64_t>(total_rows, 148 * 16);
  pack_kernel<kPack><<<grid, kCopyThreads, 0, st>>>(pages_base, layer_stride_bytes, (int)(page_bytes / 16), num_pages,
                                                    page_ids, ids_indptr, n_tasks, total_rows, layer_begin, window, packed,
                                                    device_status_ptr());
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

struct SwapArgs {
  unsigned char* pages_base;
  int64_t layer_stride_bytes, page_bytes, num_pages;
  int num_layers;
  const int32_t *page_ids, *ids_indptr, *ids_indptr_host;
  const int64_t* chunk_row_begin_host;
  int n_tasks;
  unsigned char* staging;
  int64_t staging_bytes;
  unsigned char* host_pool;
  cudaStream_t s_kernel, s_dma;
  cudaEvent_t* ev;  // [0..1] staging half filled, [2..3] staging half drained
};

int check_swap_args(const char* who, const SwapArgs& a, int64_t* total_ids, int* window) {
  DSV_REQUIRE(a.n_tasks >= 0 && a.num_layers >= 0, "%s: negative task or layer count", who);
  if (a.n_tasks == 0 || a.num_layers == 0) return 1;
  DSV_REQUIRE(a.ids_indptr_host && a.chunk_row_begin_host && a.staging && a.host_pool && a.ev,
              "%s: null pointer argument", who);
  DSV_REQUIRE(a.ids_indptr_host[0] == 0, "%s: ids_indptr must start at 0", who);
  for (int t = 0; t < a.n_tasks; ++t)
    DSV_REQUIRE(a.ids_indptr_host[t + 1] >= a.ids_indptr_host[t] && a.chunk_row_begin_host[t] >= 0,
                "%s: bad task descriptor %d", who, t);
  *total_ids = a.ids_indptr_host[a.n_tasks];
  if (*total_ids == 0) return 1;
  const int rc = check_pack_args(who, a.pages_base, a.layer_stride_bytes, a.page_bytes, a.num_pages, a.page_ids,
                                 a.ids_indptr,
                                 a.n_tasks, *total_ids, 0, a.num_layers, a.staging);
  if (rc != 0) return rc;
  for (int i = 0; i < 4; ++i) DSV_REQUIRE(a.ev[i] != nullptr, "%s: null event %d", who, i);
  const int64_t half = (a.staging_bytes / 2) & ~(int64_t)255;
  const int64_t per_layer = *total_ids * a.page_bytes;
  if (half < per_layer)
    return fail(DSV_E_WORKSPACE, "%s: half of the staging buffer (%lld B) cannot hold one layer of all tasks (%lld B)",
                who, (long long)half, (long long)per_layer);
  *window = (int)std::min<int64_t>(half / per_layer, a.num_layers);
  return 0;
}

}  // namespace
}  // namespace dsv

extern "C" {

int dsv_pack_pages(const void* pages_base, int64_t layer_stride_bytes, int64_t page_bytes, int64_t num_pages,
                   const int32_t* page_ids, const int32_t* ids_indptr, int n_tasks,
                   int64_t total_ids, int layer_begin, int layer_end, void* dst, void* stream) {
  using namespace dsv;
  const int rc = check_pack_args("pack_pages", pages_base, layer_stride_bytes, page_bytes, num_pages, page_ids, ids_indptr,
                                 n_tasks, total_ids, layer_begin, layer_end, dst);
  if (rc != 0) return rc < 0 ? rc : DSV_OK;
  return launch_pack<true>((unsigned char*)pages_base, layer_stride_bytes, page_bytes, num_pages, page_ids, ids_indptr, n_tasks,
                           total_ids, layer_begin, layer_end, (unsigned char*)dst, (cudaStream_t)stream);
}

int dsv_unpack_pages(const void* src, void* pages_base, int64_t layer_stride_bytes,
                     int64_t page_bytes, int64_t num_pages, const int32_t* page_ids, const int32_t* ids_indptr,
                     int n_tasks, int64_t total_ids, int layer_begin, int layer_end, void* stream) {
  using namespace dsv;
  const int rc = check_pack_args("unpack_pages", pages_base, layer_stride_bytes, page_bytes, num_pages, page_ids, ids_indptr,
                                 n_tasks, total_ids, layer_begin, layer_end, src);
  if (rc != 0) return rc < 0 ? rc : DSV_OK;
  return launch_pack<false>((unsigned char*)pages_base, layer_stride_bytes, page_bytes, num_pages, page_ids, ids_indptr, n_tasks,
                            total_ids, layer_begin, layer_end, (unsigned char*)src, (cudaStream_t)stream);
}

int dsv_swap_out_pages(const void* pages_base, int64_t layer_stride_bytes, int64_t page_bytes,
                       int64_t num_pages, int num_layers, const int32_t* page_ids, const int32_t* ids_indptr,
                       const int32_t* ids_indptr_host, const int64_t* chunk_row_begin_host,
                       int n_tasks, void* staging, int64_t staging_bytes, void* host_pool,
                       void* stream_kernel, void* stream_dma, void** events) {
  using namespace dsv;
  SwapArgs a{(unsigned char*)pages_base, layer_stride_bytes, page_bytes, num_pages, num_layers, page_ids, ids_indptr,
             ids_indptr_host, chunk_row_begin_host, n_tasks, (unsigned char*)staging, staging_bytes,
             (unsigned char*)host_pool, (cudaStream_t)stream_kernel, (cudaStream_t)stream_dma, (cudaEvent_t*)events};
  int64_t total_ids = 0;
  int window = 0;
  const int rc = check_swap_args("swap_out_pages", a, &total_ids, &window);
  if (rc != 0) return rc < 0 ? rc : DSV_OK;
  const int64_t half = (staging_bytes / 2) & ~(int64_t)255;
  int w = 0;
  for (int l0 = 0; l0 < num_layers; l0 += window, ++w) {
    const int l1 = std::min(num_layers, l0 + window), h = w & 1;
    unsigned char* buf = a.staging + h * half;
    // The DMA that last read this half must be done before it is refilled. That DMA may belong
    // to an EARLIER call that shares the staging buffer and the events (back-to-back offloads
    // with no host wait in between), so the edge is taken for every window, the first two
    // included; on a fresh event it is a no-op.
    DSV_CUDA(cudaStreamWaitEvent(a.s_kernel, a.ev[2 + h], 0));
    const int prc = launch_pack<true>(a.pages_base, layer_stride_bytes, page_bytes, num_pages, page_ids, ids_indptr, n_tasks,
                                      total_ids, l0, l1, buf, a.s_kernel);
    if (prc != DSV_OK) return prc;
    DSV_CUDA(cudaEventRecord(a.ev[h], a.s_kernel));
    DSV_CUDA(cudaStreamWaitEvent(a.s_dma, a.ev[h], 0));
    for (int t = 0; t < n_tasks; ++t) {
      const int64_t n_t = ids_indptr_host[t + 1] - ids_indptr_host[t];
      if (n_t == 0) continue;
      const int64_t bytes = n_t * (l1 - l0) * page_bytes;
      unsigned char* dst = a.host_pool + (chunk_row_begin_host[t] + (int64_t)l0 * n_t) * page_bytes;
      const unsigned char* src = buf + (int64_t)ids_indptr_host[t] * (l1 - l0) * page_bytes;
      DSV_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, a.s_dma));
    }
    DSV_CUDA(cudaEventRecord(a.ev[2 + h], a.s_dma));
  }
  return DSV_OK;
}

int dsv_swap_in_pages(const void* host_pool, void* pages_base, int64_t layer_stride_bytes,
                      int64_t page_bytes, int64_t num_pages, int num_layers, const int32_t* page_ids,
                      const int32_t* ids_indptr, const int32_t* ids_indptr_host,
                      const int64_t* chunk_row_begin_host, int n_tasks, void* staging,
                      int64_t staging_bytes, void* stream_kernel, void* stream_dma,
                      void** events) {
  using namespace dsv;
  SwapArgs a{(unsigned char*)pages_base, layer_stride_bytes, page_bytes, num_pages, num_layers, page_ids, ids_indptr,
             ids_indptr_host, chunk_row_begin_host, n_tasks, (unsigned char*)staging, staging_bytes,
             (unsigned char*)host_pool, (cudaStream_t)stream_kernel, (cudaStream_t)stream_dma, (cudaEvent_t*)events};
  int64_t total_ids = 0;
  int window = 0;
  const int rc = check_swap_args("swap_in_pages", a, &total_ids, &window);
  if (rc != 0) return rc < 0 ? rc : DSV_OK;
  const int64_t half = (staging_bytes / 2) & ~(int64_t)255;
  int w = 0;
  for (int l0 = 0; l0 < num_layers; l0 += window, ++w) {
    const int l1 = std::min(num_layers, l0 + window), h = w & 1;
    unsigned char* buf = a.staging + h * half;
    // The unpack that last read this half must be done before it is overwritten; as above, it may
    // be an earlier call's, so every window takes the edge.
    DSV_CUDA(cudaStreamWaitEvent(a.s_dma, a.ev[2 + h], 0));
    for (int t = 0; t < n_tasks; ++t) {
      const int64_t n_t = ids_indptr_host[t + 1] - ids_indptr_host[t];
      if (n_t == 0) continue;
      const int64_t bytes = n_t * (l1 - l0) * page_bytes;
      const unsigned char* src = a.host_pool + (chunk_row_begin_host[t] + (int64_t)l0 * n_t) * page_bytes;
      unsigned char* dst = buf + (int64_t)ids_indptr_host[t] * (l1 - l0) * page_bytes;
      DSV_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, a.s_dma));
    }
    DSV_CUDA(cudaEventRecord(a.ev[h], a.s_dma));
    DSV_CUDA(cudaStreamWaitEvent(a.s_kernel, a.ev[h], 0));
    const int prc = launch_pack<false>(a.pages_base, layer_stride_bytes, page_bytes, num_pages, page_ids, ids_indptr, n_tasks,
                                       total_ids, l0, l1, buf, a.s_kernel);
    if (prc != DSV_OK) return prc;
    DSV_CUDA(cudaEventRecord(a.ev[2 + h], a.s_kernel));
  }
  return DSV_OK;
}

int dsv_region_swap(void* pages_base, int num_layers, int64_t layer_stride_bytes,
                    int64_t region_offset_bytes, int64_t region_bytes, int64_t out_bytes, int64_t in_bytes,
                    void* host_out, const void* host_in, void* stream_out, void* stream_in, void* event,
                    int64_t page_bytes, int32_t page_size, int32_t out_rows, int32_t in_rows) {
  using namespace dsv;
  DSV_REQUIRE(num_layers >= 0 && region_bytes >= 0, "region_swap: negative size");
  DSV_REQUIRE(out_bytes >= 0 && out_bytes <= region_bytes && in_bytes >= 0 && in_bytes <= region_bytes,
              "region_swap: out_bytes (%lld) and in_bytes (%lld) must lie in [0, region_bytes = %lld]",
              (long long)out_bytes, (long long)in_bytes, (long long)region_bytes);
  if (host_out == nullptr) out_bytes = 0;
  if (host_in == nullptr) in_bytes = 0;
  if (num_layers == 0 || (out_bytes == 0 && in_bytes == 0)) return DSV_OK;
  DSV_REQUIRE(pages_base != nullptr, "region_swap: null pages_base");
  DSV_REQUIRE(region_offset_bytes >= 0 && region_offset_bytes + region_bytes <= layer_stride_bytes,
              "region_swap: region [%lld,+%lld) outside a layer of %lld bytes", (long long)region_offset_bytes,
              (long long)region_bytes, (long long)layer_stride_bytes);
  const bool both = out_bytes > 0 && in_bytes > 0;
  DSV_REQUIRE(!both || event != nullptr, "region_swap: an event is needed when both directions are given");
  unsigned char* dev = static_cast<unsigned char*>(pages_base) + region_offset_bytes;
  cudaStream_t s_out = (cudaStream_t)stream_out, s_in = (cudaStream_t)stream_in;
  // A page is [K: page_size token rows][V: page_size token rows]. When no page of the travelling head
  // holds more than `rows` tokens, only the first `rows` rows of every half travel: a 2-D copy whose
  // lines are the halves (pitch = half a page, the same on both sides, so the host image keeps the
  // region's layout). rows = page_size (or page_bytes = 0) is the plain contiguous copy.
  const bool by_rows = page_bytes > 0 && page_size > 0;
  DSV_REQUIRE(!by_rows || (page_bytes % (2 * (int64_t)page_size) == 0 && out_rows >= 0 && out_rows <= page_size &&
                           in_rows >= 0 && in_rows <= page_size && out_bytes % page_bytes == 0 && in_bytes % page_bytes == 0),
              "region_swap: rows (%d out, %d in) must lie in [0, page_size = %d] and the byte counts be whole pages",
              out_rows, in_rows, page_size);
  const int64_t half_bytes = by_rows ? page_bytes / 2 : 0, row_bytes = by_rows ? half_bytes / page_size : 0;
  const bool out_2d = by_rows && out_rows < page_size, in_2d = by_rows && in_rows < page_size;
  if (out_2d && out_rows == 0) out_bytes = 0;
  if (in_2d && in_rows == 0) in_bytes = 0;
  if (out_bytes == 0 && in_bytes == 0) return DSV_OK;
  const bool edge = out_bytes > 0 && in_bytes > 0;
  // groups of layers: one event edge per group keeps the number of API calls low
  const int group = std::max(1, (num_layers + 7) / 8);
  for (int l0 = 0; l0 < num_layers; l0 += group) {
    const int l1 = std::min(num_layers, l0 + group);
    if (out_bytes > 0) {
      for (int l = l0; l < l1; ++l) {
        unsigned char* h = static_cast<unsigned char*>(host_out) + (int64_t)l * region_bytes;
        const unsigned char* d = dev + (int64_t)l * layer_stride_bytes;
        if (out_2d)
          DSV_CUDA(cudaMemcpy2DAsync(h, (size_t)half_bytes, d, (size_t)half_bytes, (size_t)(out_rows * row_bytes),
                                     (size_t)(out_bytes / half_bytes), cudaMemcpyDeviceToHost, s_out));
        else
          DSV_CUDA(cudaMemcpyAsync(h, d, (size_t)out_bytes, cudaMemcpyDeviceToHost, s_out));
      }
      if (edge) {
        DSV_CUDA(cudaEventRecord((cudaEvent_t)event, s_out));
        DSV_CUDA(cudaStreamWaitEvent(s_in, (cudaEvent_t)event, 0));
      }
    }
    if (in_bytes > 0) {
      for (int l = l0; l < l1; ++l) {
        unsigned char* d = dev + (int64_t)l * layer_stride_bytes;
        const unsigned char* h = static_cast<const unsigned char*>(host_in) + (int64_t)l * region_bytes;
        if (in_2d)
          DSV_CUDA(cudaMemcpy2DAsync(d, (size_t)half_bytes, h, (size_t)half_bytes, (size_t)(in_rows * row_bytes),
                                     (size_t)(in_bytes / half_bytes), cudaMemcpyHostToDevice, s_in));
        else
          DSV_CUDA(cudaMemcpyAsync(d, h, (size_t)in_bytes, cudaMemcpyHostToDevice, s_in));
      }
    }
  }
  return DSV_OK;
}

}  // extern "C"
