// Host-side half of a step in native code: grow every request's page list
// (free-page search in the reference's order: prefetch buffer first, then the
// lowest free indices, at least 64 at a time) and write the ragged-batch
// descriptors into one packed int32 buffer. Pure host arithmetic on caller-owned
// arrays; no CUDA call. It does for a whole batch in one call what the
// reference does per request in Python with device tensors
// (deserve_worker/model/context/flash.py:29-64, kvcache/paged/kvcache.py:21-29,
// kvcache/virtual.py:138-149, kvcache/paged/page_pool.py:38-55).
#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "step_core.cuh"

extern "C" {

int dsv_host_build_step(uint8_t* bitmap, int32_t num_pages, int32_t* buffer, int32_t buffer_cap,
                        int32_t* buffer_start, int32_t* buffer_len, int64_t* num_avails, int32_t fetch_size,
                        int32_t page_size, int32_t num_pages_main, int32_t* tables, uint8_t* isswap,
                        int64_t table_cols, int batch, const int32_t* slot, int32_t* occupied,
                        const int32_t* start_pos, const int32_t* seqlen, const int32_t* initial_seqlen,
                        int32_t* out, int64_t out_capacity, int64_t* section_offsets, int32_t* failed_request,
                        int32_t* failed_need) {
  using namespace dsv;
  DSV_REQUIRE(bitmap && buffer && buffer_start && buffer_len && num_avails && tables && slot && occupied && start_pos &&
                  seqlen && initial_seqlen && out && section_offsets && failed_request && failed_need,
              "host_build_step: null pointer argument");
  DSV_REQUIRE(batch >= 0 && page_size > 0 && num_pages > 0 && table_cols > 0 && fetch_size > 0 && buffer_cap >= num_pages,
              "host_build_step: bad shape");
  *failed_request = -1;
  // ---- 1. grow the caches, request by request (a failure leaves the earlier ones grown) -------
  int64_t total_pages = 0;
  for (int i = 0; i < batch; ++i) {
    const int cur = start_pos[i] + seqlen[i];
    const int want_tokens = std::max(cur, initial_seqlen[i]);
    int32_t need = 0;
    uint8_t* flags = isswap != nullptr ? isswap + (int64_t)slot[i] * table_cols : nullptr;
    const int rc = grow_request(bitmap, num_pages, buffer, buffer_cap, buffer_start, buffer_len, num_avails, fetch_size,
                                page_size, num_pages_main, tables + (int64_t)slot[i] * table_cols, flags, table_cols,
                                want_tokens, occupied + i, &need);
    DSV_REQUIRE(rc != GROW_ROW_FULL, "host_build_step: request %d needs %d pages, the table row holds %lld", i, need,
                (long long)table_cols);
    if (rc == GROW_NO_PAGES) {
      *failed_request = i;
      *failed_need = need;
      return DSV_E_WORKSPACE;
    }
    total_pages += (cur + page_size - 1) / page_size;
  }
  // ---- 2. descriptors: indptr | kv_page_indptr | kv_last_page_lens | offsets | seqlens | kv_page_indices
  auto ceil4 = [](int64_t n) { return (n + 3) & ~(int64_t)3; };
  const int64_t sizes[6] = {batch + 1, batch + 1, batch, batch, batch, total_pages};
  int64_t at = 0;
  for (int k = 0; k < 6; ++k) {
    section_offsets[k] = at;
    at += ceil4(sizes[k]);
  }
  section_offsets[6] = at;
  if (at > out_capacity) return fail(DSV_E_WORKSPACE, "host_build_step: descriptors need %lld int32, capacity %lld",
                                     (long long)at, (long long)out_capacity);
  int32_t *indptr = out + section_offsets[0], *kvp = out + section_offsets[1], *last = out + section_offsets[2],
          *offs = out + section_offsets[3], *sl = out + section_offsets[4], *idx = out + section_offsets[5];
  indptr[0] = 0;
  kvp[0] = 0;
  for (int i = 0; i < batch; ++i) {
    const int cur = start_pos[i] + seqlen[i];
    const int n_pages = (cur + page_size - 1) / page_size;
    indptr[i + 1] = indptr[i] + seqlen[i];
    kvp[i + 1] = kvp[i] + n_pages;
    // (cur - 1) mod page_size + 1 with Python's floor semantics for cur = 0
    last[i] = ((cur - 1) % page_size + page_size) % page_size + 1;
    offs[i] = start_pos[i];
    sl[i] = seqlen[i];
    std::memcpy(idx + kvp[i], tables + (int64_t)slot[i] * table_cols, sizeof(int32_t) * (size_t)n_pages);
  }
  return DSV_OK;
}

}  // extern "C"
