// Device-resident allocator, page tables and descriptor build: the same step as
// host_step.cu, but the free bitmap, the prefetch buffer, the page tables and the
// per-row page counts live in device memory and are advanced by kernels, so that a
// step's page-id lists (the bulk of the descriptors: one int32 per page of every
// request) never cross the host link and a decode step needs no host-visible
// allocator state. What the host still sends per step is six int32 per request
// (table row, start position, new tokens, prompt length and the two prefix sums
// it can compute from the token counts alone).
//
// Replaces the same reference code as the host builder: FlashForwardCtx.
// init_paged_forward_ctx (deserve_worker/model/context/flash.py:29-64) with
// PagedKVCache.extend -> PagePool.alloc (kvcache/paged/kvcache.py:21-29,
// page_pool.py:38-55) and PagedKVCache.free (kvcache.py:31-33, page_pool.py:73-76).
// The allocation itself is one thread walking the requests in order through
// grow_request() — the function the host builder calls — because the order in
// which requests take pages IS the result (page ids must match the reference's).
#include "common.cuh"
#include "step_core.cuh"

namespace dsv {
namespace {

constexpr int kReqFields = 6;  // slot, start_pos, seqlen, initial_seqlen, qo_begin, kv_begin

// state[0] = free pages (int64); state[1] = {buffer_start, buffer_len} (2 x int32)
__global__ void device_grow_kernel(uint8_t* bitmap, int32_t num_pages, int32_t* buffer, int64_t* state,
                                   int32_t fetch_size, int32_t page_size, int32_t* tables, int64_t table_cols,
                                   int32_t* occupied, int32_t max_requests, const int32_t* req, int batch,
                                   int* status) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int32_t* win = reinterpret_cast<int32_t*>(state + 1);
  for (int i = 0; i < batch; ++i) {
    const int32_t* r = req + (int64_t)i * kReqFields;
    const int slot = r[0];
    if (slot < 0 || slot >= max_requests) {
      record_status(status, ST_BAD_REQUEST);
      return;
    }
    const int cur = r[1] + r[2];
    const int want_tokens = cur > r[3] ? cur : r[3];
    int32_t need = 0;
    // the host checked the page budget and the row length before the launch: any failure here means
    // that its mirror of the counts and the device state disagree
    if (grow_request(bitmap, num_pages, buffer, num_pages, win, win + 1, state, fetch_size, page_size, -1,
                     tables + (int64_t)slot * table_cols, nullptr, table_cols, want_tokens, occupied + slot,
                     &need) != GROW_OK) {
      record_status(status, ST_BAD_REQUEST);
      return;
    }
  }
}

// One CTA per request: its slice of every descriptor section, page ids straight from its table row.
__global__ void __launch_bounds__(128)
device_describe_kernel(const int32_t* __restrict__ tables, int64_t table_cols, int32_t page_size,
                       const int32_t* __restrict__ req, int batch, int32_t* __restrict__ indptr,
                       int32_t* __restrict__ kvp, int32_t* __restrict__ last, int32_t* __restrict__ offs,
                       int32_t* __restrict__ sl, int32_t* __restrict__ idx, const int32_t* __restrict__ occupied,
                       int* status) {
  const int i = blockIdx.x;
  const int32_t* r = req + (int64_t)i * kReqFields;
  const int slot = r[0], start = r[1], n_new = r[2], qo0 = r[4], kv0 = r[5];
  const int cur = start + n_new;
  const int n_pages = (cur + page_size - 1) / page_size;
  if (threadIdx.x == 0) {
    indptr[i] = qo0;
    kvp[i] = kv0;
    if (i == batch - 1) {
      indptr[batch] = qo0 + n_new;
      kvp[batch] = kv0 + n_pages;
    }
    last[i] = ((cur - 1) % page_size + page_size) % page_size + 1;  // (cur - 1) mod page_size + 1, floor semantics
    offs[i] = start;
    sl[i] = n_new;
    if (n_pages > occupied[slot]) record_status(status, ST_BAD_REQUEST);  // descriptors beyond what was grown
  }
  const int32_t* row = tables + (int64_t)slot * table_cols;
  for (int j = threadIdx.x; j < n_pages; j += blockDim.x) idx[kv0 + j] = row[j];
}

// Pages of the given table rows go back to the bitmap (not to the prefetch buffer), rows become empty.
__global__ void device_free_kernel(uint8_t* bitmap, int32_t num_pages, int64_t* state, const int32_t* tables,
                                   int64_t table_cols, int32_t* occupied, const int32_t* slots, int n, int* status) {
  const int s = slots[blockIdx.x];
  const int occ = occupied[s];
  const int32_t* row = tables + (int64_t)s * table_cols;
  for (int j = threadIdx.x; j < occ; j += blockDim.x) {
    const int pg = row[j];
    if (pg < 0 || pg >= num_pages) record_status(status, ST_BAD_PAGE_ID);
    else bitmap[pg] = 1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(reinterpret_cast<unsigned long long*>(state), (unsigned long long)occ);
    occupied[s] = 0;
  }
  (void)n;
}

}  // namespace
}  // namespace dsv

extern "C" {

int dsv_device_build_step(uint8_t* bitmap, int32_t num_pages, int32_t* buffer, int64_t* state, int32_t fetch_size,
                          int32_t page_size, int32_t* tables, int64_t table_cols, int32_t* occupied,
                          int32_t max_requests, const int32_t* req, int batch, int grow, int32_t* out,
                          const int64_t* section_offsets_host, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(batch >= 0, "device_build_step: negative batch");
  if (batch == 0) return DSV_OK;
  DSV_REQUIRE(bitmap && buffer && state && tables && occupied && req && out && section_offsets_host,
              "device_build_step: null pointer argument");
  DSV_REQUIRE(num_pages > 0 && page_size > 0 && fetch_size > 0 && table_cols > 0 && max_requests > 0,
              "device_build_step: bad shape");
  for (int k = 0; k < 6; ++k)
    DSV_REQUIRE(section_offsets_host[k] >= 0 && section_offsets_host[k] <= section_offsets_host[k + 1],
                "device_build_step: section offsets must ascend");
  cudaStream_t st = (cudaStream_t)stream;
  int* status = device_status_ptr();
  if (grow) {
    device_grow_kernel<<<1, 32, 0, st>>>(bitmap, num_pages, buffer, state, fetch_size, page_size, tables, table_cols,
                                         occupied, max_requests, req, batch, status);
    DSV_CUDA(cudaGetLastError());
  }
  const int64_t* o = section_offsets_host;
  device_describe_kernel<<<batch, 128, 0, st>>>(tables, table_cols, page_size, req, batch, out + o[0], out + o[1],
                                                out + o[2], out + o[3], out + o[4], out + o[5], occupied, status);
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

int dsv_device_free_rows(uint8_t* bitmap, int32_t num_pages, int64_t* state, const int32_t* tables,
                         int64_t table_cols, int32_t* occupied, const int32_t* slots, int n, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(n >= 0, "device_free_rows: negative count");
  if (n == 0) return DSV_OK;
  DSV_REQUIRE(bitmap && state && tables && occupied && slots, "device_free_rows: null pointer argument");
  DSV_REQUIRE(num_pages > 0 && table_cols > 0, "device_free_rows: bad shape");
  device_free_kernel<<<n, 128, 0, (cudaStream_t)stream>>>(bitmap, num_pages, state, tables, table_cols, occupied,
                                                         slots, n, device_status_ptr());
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

}  // extern "C"
